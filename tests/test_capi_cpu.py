"""The C-ABI library loads without a GPU and exports every symbol that
include/vdcores.h declares; tables agree with the header the host code parses."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    h = open(os.path.join(ROOT, "include", "vdcores.h")).read()
    h = re.sub(r"/\*.*?\*/", "", h, flags=re.S)
    return sorted(set(re.findall(r"\b(vdc_\w+)\s*\(", h)))


def test_library_exports_every_declared_symbol():
    from vdcores_b200 import runtime
    lib = ctypes.CDLL(runtime.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/vdcores.h but not exported"
    assert sorted(runtime.EXPORTED_SYMBOLS) == names


def test_opcode_table_matches_header():
    from vdcores_b200 import isa, runtime
    for name, value in isa.OPCODES.items():
        assert getattr(runtime.opcode, name) == value
    assert set(runtime.supported_compute_ops) == set(isa.COMPUTE_OPS)
    # wire-format facts schedules of the reference rely on
    assert isa.OP_ALLOC_TMA_LOAD_1D == (9 << 6) | 1 and isa.OP_ALLOC_WB_TMA_STORE_1D == (16 << 6) | 3
    assert isa.OP_ALLOC_WB_RAW_ADDRESS == (23 << 6) | 1 and isa.OP_REPEAT == 2 << 6 and isa.OP_LOOP == 3 << 6
    assert (isa.F_ALLOCATE, isa.F_WRITEBACK, isa.F_GROUP, isa.F_JUMP, isa.F_BARRIER, isa.F_PORT) == (1, 2, 4, 8, 16, 32)


def test_config_namespace():
    from vdcores_b200 import runtime
    c = runtime.config
    assert (c.slot_size, c.num_slots, c.max_insts, c.num_profile_events) == (8192, 24, 4096, 128)
    assert (c.max_tmas, c.max_bars, c.num_special_slots) == (1024, 1024, 9)
    assert c.dynamic_smem == 24 * 8192 + 1024 + 2048      # what the kernel is launched with: slots, alignment slack, guard


def test_argument_errors_without_a_gpu():
    """Calls that validate before touching the device report VDC_ERR_ARG."""
    from vdcores_b200 import isa, runtime
    lib = runtime._lib
    assert lib.vdc_set_smem_size(10 ** 9) == isa.ERR_ARG
    assert b"227 KB" in lib.vdc_last_error()
    buf = (ctypes.c_uint8 * 128)()
    shape = (ctypes.c_uint64 * 1)(64)
    box = (ctypes.c_uint32 * 1)(64)
    es = (ctypes.c_uint32 * 1)(1)
    rc = lib.vdc_build_tma_desc(buf, ctypes.c_void_p(8), 2, 1, shape, None, box, es, 0, 0)
    assert rc == isa.ERR_ARG and b"16-byte aligned" in lib.vdc_last_error()
    rc = lib.vdc_build_tma_desc(buf, ctypes.c_void_p(4096), 2, 7, shape, None, box, es, 0, 0)
    assert rc == isa.ERR_ARG
    assert lib.vdc_config(b"no_such_key") == -1


def _small_program():
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    P = Program(2)
    b = P.new_barrier()
    P.copy(1, Src(1 << 22, 1024), Dst(1 << 20, 1024, release=b), 1024)
    P.gemv(0, w_addr=1 << 30, n_rows=64, K=512, R=16, x=Src(1 << 20, 1024, wait=b),
           out=Dst(1 << 21, 128, "store"), fp8_scales=1 << 24, chunk_stride=2)
    P.insts_per_sm = 64
    return P, isa


def test_validate_streams_accepts_emitted_programs_and_names_what_is_wrong():
    """vdc_validate_streams walks host copies of both streams: what Program emits passes; an unknown opcode,
    a truncated multi-word instruction, a bad rows-per-chunk count, a forward loop and a missing terminator
    are each reported with the SM and the instruction index."""
    import numpy as np
    from vdcores_b200 import runtime
    from vdcores_b200.program import CINST, MINST
    P, isa = _small_program()
    c, m, _ = P.finalize()                      # runs the check itself
    runtime.validate_streams(2, 64, c, m)
    n_c0 = len(P.c[0])

    def broken(edit):
        cc, mm = c.copy().view(CINST).reshape(2, 64), m.copy().view(MINST).reshape(2, 64)
        edit(cc, mm)
        return cc.view(np.uint8).reshape(-1, 8), mm.view(np.uint8).reshape(-1, 16)

    def set_op(arr, sm, pc, op):
        if pc < 0:                                   # from the terminator to the end of the stream
            arr[sm, -pc:][arr.dtype.names[0]] = op
        else:
            arr[sm, pc][arr.dtype.names[0]] = op

    cases = [
        (lambda cc, mm: set_op(cc, 0, 0, 0x7999), r"compute stream of SM 0, instruction 0 .*unknown opcode"),
        (lambda cc, mm: set_op(cc, 0, 2, isa.OP_DUMMY), r"compute stream of SM 0, instruction 2 .*continuation word expected"),
        (lambda cc, mm: set_op(cc, 0, -(n_c0 - 1), isa.OP_DUMMY), r"compute stream of SM 0.*no TERMINATEC"),
        (lambda cc, mm: set_op(mm, 1, 0, 60 << 6), r"memory stream of SM 1, instruction 0 .*unknown opcode"),
        (lambda cc, mm: set_op(mm, 1, -(len(P.m[1]) - 1), isa.OP_ISSUE_BARRIER), r"memory stream of SM 1.*no TERMINATE"),
    ]
    for edit, pattern in cases:
        cc, mm = broken(edit)
        with pytest.raises(ValueError, match=pattern):
            runtime.validate_streams(2, 64, cc, mm)
    # rows per chunk: the low five bits of the flags word
    cc, mm = broken(lambda cc, mm: None)
    v = cc.view(CINST).reshape(2, 64)
    name1 = v.dtype.names[2]
    v[0, 0][name1] = (int(v[0, 0][name1]) & ~31) | 3
    with pytest.raises(ValueError, match="rows per chunk"):
        runtime.validate_streams(2, 64, v.view(np.uint8).reshape(-1, 8), mm)
    with pytest.raises(ValueError, match="num_sms \\* insts_per_sm"):
        runtime.validate_streams(3, 64, c, m)


def test_finalize_rejects_a_malformed_program_on_the_host():
    P, isa = _small_program()
    P.comp(0, 0x7999, 0, 0, 0)
    with pytest.raises(ValueError, match="unknown opcode"):
        P.finalize()
