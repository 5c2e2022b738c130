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
