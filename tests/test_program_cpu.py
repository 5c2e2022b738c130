"""Host-side logic of the instruction program builder (no GPU)."""
import numpy as np
import pytest

from vdcores_b200 import isa
from vdcores_b200.program import CINST, MINST, Dst, Program, Src, f32_bits, slots_for


def decode(P):
    c, m, bars = P.finalize()
    n = P.insts_per_sm
    return c.view(CINST).reshape(P.num_sms, n), m.view(MINST).reshape(P.num_sms, n), bars


def test_gemv_emission_matches_pop_order():
    P = Program(2, insts_per_sm=32)
    b_in, b_out = P.new_barrier(), P.new_barrier()
    P.gemv(1, w_addr=0x10000, n_rows=64, K=4096, R=4, x=Src(0x2000, 8192, wait=b_in),
           out=Dst(0x3000, 128, "add_bf16", release=b_out), norm_w=Src(0x4000, 8192), eps=1e-5)
    c, m, bars = decode(P)
    ops = [int(x) for x in m[1]["opcode"][:7]]
    # norm weight, x (slots + address handed to the task, which waits on b_in itself), out (raw address,
    # releases b_out), REPEAT header, chunk load, TERMINATE
    assert ops[0] == isa.OP_ALLOC_TMA_LOAD_1D | isa.F_PORT
    assert ops[1] == isa.OP_ALLOC_XVEC | isa.F_BARRIER
    assert int(m[1]["num_slots"][1]) == 1 | (b_in << 6) and int(m[1]["address"][1]) == 0x2000
    assert ops[2] == isa.OP_ALLOC_WB_RAW_ADDRESS | isa.F_BARRIER | isa.F_WRITEBACK
    assert int(m[1]["num_slots"][2]) >> 6 == b_out
    assert ops[3] == isa.OP_REPEAT and int(m[1]["size"][3]) == 16 and int(m[1]["address"][3]) == 4 * 4096 * 2
    assert ops[4] == isa.OP_ALLOC_TMA_LOAD_1D | isa.F_JUMP and int(m[1]["size"][4]) == 32768
    assert int(m[1]["num_slots"][4]) == 4
    assert ops[5] == isa.OP_TERMINATE
    assert int(bars[b_out]) == 1 and int(bars[b_in]) == 0
    # compute side: two words, then TERMINATEC; SM 0 only terminates
    assert int(c[1]["opcode"][0]) == isa.OP_GEMV_ROWS_BF16 and int(c[1]["opcode"][1]) == isa.OP_EXT
    a1 = int(c[1]["a1"][0])
    assert a1 & 31 == 4 and a1 & isa.GEMV_NORM_BIT and a1 & isa.GEMV_ACC_BIT and int(c[1]["a2"][0]) & 0xFF == 16
    e = f32_bits(1e-5)
    assert (int(c[1]["a0"][1]) << 16 | int(c[1]["a1"][1])) == e
    assert int(c[1]["opcode"][2]) == isa.OP_TERMINATEC and int(c[0]["opcode"][0]) == isa.OP_TERMINATEC


def test_repeat_headers_group_equal_deltas():
    P = Program(1, insts_per_sm=16)
    P.repeat(0, 0, [4, 0, 4, 0], dynamic=True)
    _, m, _ = decode(P)
    hdr = m[0][:4]
    assert [int(x) for x in hdr["opcode"]] == [isa.OP_REPEAT] * 4
    assert [int(x) for x in hdr["address"]] == [4, 0, 4, 0]
    assert [int(x) for x in hdr["num_slots"]] == [0 | 1 << 8, 1 | 2 << 8, 2 | 3 << 8, 3 | 4 << 8]
    assert [int(x) for x in hdr["size"]] == [0, 0, 0, 0xFFFF] and int(hdr["arg"][3]) == 4
    P2 = Program(1, insts_per_sm=16)
    P2.repeat(0, 7, [512, 512, 512])
    _, m2, _ = decode(P2)
    assert int(m2[0]["num_slots"][0]) == 0 | 3 << 8 and int(m2[0]["size"][0]) == 7


def test_barrier_counts_follow_releases():
    P = Program(3, insts_per_sm=32)
    b = P.new_barrier()
    for sm in range(3):
        P.copy(sm, Src(0x1000, 256), Dst(0x2000 + 256 * sm, 256, release=b), 256)
    P.raw_address(0, 0x9000, 25, release=b)
    _, _, bars = decode(P)
    assert int(bars[b]) == 4 and int(bars.sum()) == 4


def test_alignment_and_size_checks():
    P = Program(1)
    with pytest.raises(AssertionError):
        P.load(0, Src(0x1008, 256))            # bulk copies start on 16-byte boundaries
    with pytest.raises(AssertionError):
        P.load(0, Src(0x1000, 40000))          # at most 32 KB per instruction
    with pytest.raises(AssertionError):
        P.gemv(0, w_addr=0, n_rows=6, K=4096, R=4, x=Src(0, 8192), out=Dst(0, 12))   # rows not a multiple of R
    with pytest.raises(AssertionError):
        P.gemv(0, w_addr=0, n_rows=8, K=4096, R=8, x=Src(0, 8192), out=Dst(0, 16))   # chunk beyond 32 KB
    assert slots_for(1) == 1 and slots_for(8192) == 1 and slots_for(8193) == 2 and slots_for(28672) == 4


def test_ring_overflow_is_reported():
    P = Program(1, insts_per_sm=4)
    for _ in range(5):
        P.load(0, Src(0x1000, 256))
    with pytest.raises(ValueError):
        P.finalize()


def test_engine_quantisers_match_the_oracle_codecs():
    """The engine's own FP8 / NVFP4 encoders (product code) produce exactly the
    oracle's codes, block scales and tensor scales on the CPU."""
    import torch
    from oracle import decode_oracle as O
    from vdcores_b200.decode import quantize_fp8_rows, quantize_nvfp4_rows
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(48, 1024, generator=g) * 0.02).to(torch.bfloat16)
    w[5, 100:116] = 0                                  # an all-zero block
    q, s = quantize_fp8_rows(w)
    oq, os_ = O.fp8_quantize(w)
    assert torch.equal(q, oq.view(torch.uint8)) and torch.equal(s, os_)
    rows, ts = quantize_nvfp4_rows(w)
    op, obs, ots = O.nvfp4_quantize(w)
    assert torch.equal(rows[:, :512], op) and torch.equal(rows[:, 512:], obs.view(torch.uint8))
    assert float(ts) == float(ots)


def test_dynamic_expert_gemv_stream_order():
    """An expert task of the expert-parallel path: the count word is handed over behind the
    routing barrier, and the indirection sits directly in front of the dynamic loop, so that
    a skipped loop (expert of another rank) drops it with the loop."""
    P = Program(1)
    b_route = P.new_barrier()
    P.gemv(0, w_addr=1 << 30, n_rows=64, K=512, R=16, x=Src(1 << 20, 1024), out=Dst(1 << 21, 256, "store"),
           mode=isa.GEMV_MODE_MOE_DOWN, w_indirect=(1 << 22, 512 * 64 * 2), wait_issue=b_route,
           dyn_count_addr=(1 << 22) + 192, moe=dict(weight_addr=(1 << 22) + 64, acc_addr=0, cnt_addr=0, top_k=4))
    ids = [isa.op_id(m[0]) for m in P.m[0]]
    names = {isa.op_id(v): k for k, v in isa.OPCODES.items() if k in isa.MEMORY_OPS}
    seq = [names[i] for i in ids]
    assert seq == ["OP_ALLOC_XVEC", "OP_ALLOC_WB_RAW_ADDRESS", "OP_ISSUE_BARRIER", "OP_ALLOC_WB_RAW_ADDRESS",
                   "OP_DYN_COUNT", "OP_CC0_STRIDE32", "OP_REPEAT", "OP_ALLOC_TMA_LOAD_1D"], seq
    assert P.m[0][6][1] == 0xFFFF                       # the loop count comes from DYN_COUNT
    assert P.c[0][0][2] & isa.GEMV_DYN_BIT              # and the task clamps its chunk count the same way


def test_validate_catches_dead_barriers_and_oversized_loads():
    P = Program(2)
    b_in, b_out = P.new_barrier(), P.new_barrier()
    P.gemv(0, w_addr=1 << 30, n_rows=64, K=512, R=16, x=Src(1 << 20, 1024, wait=b_in),
           out=Dst(1 << 21, 128, "store", release=b_out))
    with pytest.raises(ValueError, match="never released"):
        P.validate()                                    # nobody counts b_in down
    P.copy(1, Src(1 << 22, 1024), Dst(1 << 20, 1024, release=b_in), 1024)
    assert P.validate()
    P.mem(1, isa.OP_ALLOC_TMA_LOAD_1D, size=20000, nslot=2, address=1 << 23)
    with pytest.raises(ValueError, match="into 2 slots"):
        P.validate()


def test_compute_word_counts_follow_the_table_in_the_header():
    """Every emitter writes exactly the number of words isa.h declares for its opcode (optional
    trailing words come on top): the kernel's dispatcher steps through the stream by that table."""
    P = Program(1)
    b = P.new_barrier()
    P.add_releases(b, 1)
    P.gemv(0, w_addr=1 << 30, n_rows=64, K=512, R=16, x=Src(1 << 20, 1024), out=Dst(1 << 21, 128, "store"))
    P.gemv(0, w_addr=1 << 30, n_rows=64, K=512, R=16, x=Src(1 << 20, 1024), out=Dst(1 << 21, 128, "store"),
           fp8_scales=1 << 22)
    P.attn_decode(0, G=4, state_addr=1 << 16, rope=Src(1 << 17, 512), norm_w=None, qkv=Src(1 << 18, 6 * 256, wait=b),
                  k_page_addr=1 << 24, v_page_addr=1 << 25, page_shift=15, base_page=0, max_pages=2,
                  records_addr=1 << 19, counter_addr=1 << 20, out_addr=1 << 21, split=0, n_splits=1, release=b)
    P.l2_prefetch(0, 1 << 30, 4096)
    P.argmax_final(0, records=Src(1 << 20, 64), n=4, state_addr=1 << 16, log_addr=1 << 17)
    # the in-kernel tensor-parallel exchange: tagged-entry reducers and the candidate collector
    P.xreduce(0, n=128, n_ranks=2, xbuf_addr=1 << 26, hidden_elems=4096, ex=3, n_ex=65, hidden_addr=1 << 21,
              state_addr=1 << 16, release=b)
    P.xwait(0, n_ranks=2, ex=64, n_ex=65, entries_addr=1 << 27, state_addr=1 << 16, records_addr=1 << 22, release=b)
    i, stream = 0, P.c[0]
    seen = []
    while i < len(stream):
        op = stream[i][0]
        assert op != isa.OP_EXT, f"word {i}: a continuation word where an instruction must start"
        n = isa.OP_WORDS[op]
        assert all(stream[i + k][0] == isa.OP_EXT for k in range(1, n)), (hex(op), n)
        seen.append(op)
        i += n
    assert seen == [isa.OP_GEMV_ROWS_BF16, isa.OP_GEMV_ROWS_FP8, isa.OP_ATTN_DECODE_PAGED_G4, isa.OP_L2_PREFETCH,
                    isa.OP_ARGMAX_FINAL, isa.OP_XREDUCE, isa.OP_XWAIT]
    # XREDUCE carries [entries per rank / 2, exchange number, exchanges per step] in its third word
    k = [j for j, w in enumerate(stream) if w[0] == isa.OP_XREDUCE][0]
    assert tuple(stream[k + 2][1:4]) == (2048, 3, 65)
    # a projection that sends its rows to the ranks' exchange blocks: two trailing words [table], [ranks, ex, n_ex]
    P2 = Program(1)
    P2.gemv(0, w_addr=1 << 30, n_rows=64, K=512, R=16, x=Src(1 << 20, 1024), out=Dst(4096, 64 * 8, "store"),
            mode=isa.GEMV_MODE_STORE_F32, peers=(1 << 23, 2, 3, 65))
    assert tuple(P2.c[0][-1][1:4]) == (2, 3, 65) and P2.c[0][-2][0] == isa.OP_EXT
