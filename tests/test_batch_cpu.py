"""Host-side logic of the batched (tensor-core) decode path, without a GPU: operand layouts,
the dealing of projection work to SMs, and the memory streams the program builder emits
(expanded here by a small interpreter of REPEAT loops)."""
import torch

from vdcores_b200 import isa
from vdcores_b200.batch import (BLOCK_ROWS, chunk_geometry, emit_projection, pack_blocks, pack_blocks_fp8, pack_kc,
                                plan_units, projection_blocks, unpack_kc)
from vdcores_b200.program import Program


def test_k_chunk_major_layout():
    x = torch.arange(32 * 64, dtype=torch.float32).view(32, 64)
    p = pack_kc(x)
    bp = 32
    for b, k in [(0, 0), (3, 9), (31, 63), (8, 8), (17, 40)]:
        off = ((k // 8) * (bp // 8) + b // 8) * 128 + (b % 8) * 16 + (k % 8) * 2       # bytes, as isa.h states it
        assert p[off // 2] == x[b, k]
    assert torch.equal(unpack_kc(p, 32, 64), x)
    # a K-range of the matrix is one contiguous piece
    assert torch.equal(p[16 * bp:48 * bp], pack_kc(x[:, 16:48].contiguous()))


def test_block_packing_keeps_k_ranges_contiguous():
    M, K = 256 + 256 + 96, 512
    w = torch.arange(M * K, dtype=torch.float32).view(M, K)
    pk = pack_blocks(w)
    for r0, n in projection_blocks(M):
        blk = pk[r0 * K:(r0 + n) * K]
        assert torch.equal(unpack_kc(blk, n, K), w[r0:r0 + n])
        kc = 64
        for c in (0, 3, K // kc - 1):
            assert torch.equal(blk[c * kc * n:(c + 1) * kc * n], pack_kc(w[r0:r0 + n, c * kc:(c + 1) * kc].contiguous()))


def test_fp8_block_packing_matches_the_in_kernel_conversion():
    """A 16-byte piece (16 k of one row) becomes the two adjacent 8-k pieces of the bf16 operand layout."""
    M, K, kc = 256, 256, 64
    codes = torch.randint(0, 256, (M, K), dtype=torch.uint8)
    pk = pack_blocks_fp8(codes)
    chunk = pk[0:M * kc]                                    # first W chunk of the block: [kc/16][M/8][8][16]
    out = torch.zeros(M * kc, dtype=torch.uint8)            # what the converting warps write (here: bytes, not bf16)
    pieces = chunk.view(-1, 16)
    for p in range(pieces.shape[0]):
        i16, row = divmod(p, M)
        out.view(-1, 8)[(2 * i16) * M + row] = pieces[p, :8]
        out.view(-1, 8)[(2 * i16 + 1) * M + row] = pieces[p, 8:]
    assert torch.equal(out, pack_kc(codes[:, :kc].contiguous()))


def test_plan_units_covers_every_step_once_and_balances():
    for M, K, S in [(6144, 4096, 148), (4096, 14336, 148), (28672, 4096, 148), (128256, 4096, 148), (640, 4096, 5),
                    (96, 512, 2)]:
        blocks = projection_blocks(M)
        kc, _ = chunk_geometry(blocks[0][1], 16, K)
        steps = K // kc
        load = [0] * S
        units = plan_units(blocks, steps, list(range(S)), load, kc * 2)
        seen = {}
        for sm, bi, c0, cnt in units:
            assert cnt > 0 and 0 <= c0 and c0 + cnt <= steps
            for c in range(c0, c0 + cnt):
                assert (bi, c) not in seen
                seen[(bi, c)] = sm
        assert len(seen) == len(blocks) * steps
        assert sum(load) == M * K * 2
        if S == 148:
            assert max(load) <= 1.15 * (sum(load) / S)


def expand_loads(minsts):
    """(address, bytes) of every 1-D load of one SM's memory stream, REPEAT loops unrolled."""
    out, i = [], 0
    deltas, count = {}, None
    while i < len(minsts):
        op, size, num_slots, arg, addr = minsts[i]
        opid = op >> isa.FLAG_BITS
        if opid == isa.op_id(isa.OP_REPEAT):
            lo, hi = num_slots & 0xFF, num_slots >> 8
            for lane in range(lo, hi):
                deltas[lane] = addr
            if size:
                count = size
            i += 1
            if count is not None and size:
                body = []
                while True:
                    body.append(minsts[i])
                    i += 1
                    if body[-1][0] & isa.F_JUMP:
                        break
                for it in range(count):
                    for j, (bop, bsize, _, _, baddr) in enumerate(body):
                        if bop >> isa.FLAG_BITS == isa.op_id(isa.OP_ALLOC_TMA_LOAD_1D):
                            out.append((baddr + it * deltas.get(j, 0), bsize))
                deltas, count = {}, None
            continue
        if opid == isa.op_id(isa.OP_ALLOC_TMA_LOAD_1D):
            out.append((addr, size))
        i += 1
    return out


def test_emitted_streams_read_every_weight_byte_once_and_the_right_activations():
    M, K, B, Bp, S = 1280, 2048, 12, 16, 7
    W_ADDR, X_ADDR, NORM = 1 << 30, 1 << 28, 1 << 27
    P = Program(S)
    bar = P.new_barrier()
    units = emit_projection(P, sms=list(range(S)), load=[0] * S, w_addr=W_ADDR, M=M, K=K, x_addr=X_ADDR, B=B, Bpad=Bp,
                            mode=isa.GEMM_MODE_STORE_ROWS, out_addr=1 << 26, scratch_addr=1 << 25, counter_addr=1 << 24,
                            release=bar, norm_addr=NORM, eps=1e-5, ld=M, stats_addr=1 << 23)
    assert P.bar_counts[bar] == len(projection_blocks(M))          # one release per block (its last arriver)
    w_bytes, x_total, n_total = [], 0, 0
    for sm in range(S):
        for addr, n in expand_loads(P.m[sm]):
            if W_ADDR <= addr < W_ADDR + M * K * 2:
                w_bytes.append((addr, n))
            elif X_ADDR <= addr < X_ADDR + Bp * K * 2:
                x_total += n
            elif NORM <= addr < NORM + K * 2:
                n_total += n
            else:
                raise AssertionError(hex(addr))
    w_bytes.sort()
    pos = W_ADDR
    for addr, n in w_bytes:                                        # contiguous, no gap, no overlap
        assert addr == pos
        pos += n
    assert pos == W_ADDR + M * K * 2
    k_streamed = sum(cnt for _, _, _, cnt in units) * chunk_geometry(BLOCK_ROWS, Bp, K)[0]
    assert x_total == Bp * k_streamed * 2                          # every unit reads the activations of its K-range
    assert n_total == k_streamed * 2                               # and the matching slice of the norm weights
    # compute side: one task per unit, eleven words each
    assert sum(1 for sm in range(S) for c in P.c[sm] if c[0] == isa.OP_GEMM_TC_BF16) == len(units)
    assert all(len(P.c[sm]) % 11 == 0 for sm in range(S))
