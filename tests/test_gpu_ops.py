"""Operator-level parity tests on a B200: a tiny program per task, run through
the C ABI, compared with the CPU oracle on the same seeded inputs.  They mirror
the reference's single-op harnesses (reference app/python/gemv_out.py,
rmsnorm.py, silu_mul.py, argmax.py, attention_split_kv.py), but assert."""
import math

import numpy as np
import pytest
import torch

from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16
TIMEOUT_NS = 300_000_000  # every device wait gives up after 0.3 s instead of hanging


def run_program(P, dev):
    from vdcores_b200 import isa, runtime
    n = max(max(len(x) for x in P.m), max(len(x) for x in P.c)) + 2
    P.insts_per_sm = ((n + 15) // 16) * 16
    c, m, bars = P.finalize()
    ct, mt = torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev)
    bt = torch.from_numpy(bars).to(dev)
    prof = torch.zeros(P.num_sms * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    runtime.launch_dae(P.num_sms, 0, ct, mt, None, bt, prof, torch.cuda.current_stream().cuda_stream,
                       timeout_ns=TIMEOUT_NS, insts_per_sm=P.insts_per_sm)
    assert int(bt.abs().sum()) == 0, "every barrier must have counted down to zero"
    return prof.view(P.num_sms, -1)


def seeded(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(BF16)


@pytest.mark.parametrize("M,K,R,n_sms", [(64, 256, 16, 1), (512, 4096, 4, 8), (96, 14336, 1, 3), (256, 768, 16, 2)])
def test_gemv_store(cuda_device, M, K, R, n_sms):
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    w, x = seeded((M, K), 1, 0.02), seeded((K,), 2)
    wd, xd = w.to(dev), x.to(dev)
    y = torch.zeros(M, dtype=BF16, device=dev)
    P = Program(n_sms)
    per = M // n_sms
    for sm in range(n_sms):
        r0 = sm * per
        P.gemv(sm, w_addr=wd.data_ptr() + r0 * K * 2, n_rows=per, K=K, R=R, x=Src(xd.data_ptr(), K * 2),
               out=Dst(y.data_ptr() + r0 * 2, per * 2, "store", release=None))
    run_program(P, dev)
    ref = O.linear(x[None], w)[0]
    assert O.rel_l2(y.cpu(), ref) < 2e-3


def test_gemv_norm_residual_and_barrier_chain(cuda_device):
    """Two dependent stages on different SMs: y = W1 rmsnorm(x); h += W2 y."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    K, M = 512, 256
    w1, w2 = seeded((M, K), 3, 0.05), seeded((K, M), 4, 0.05)
    x, nw = seeded((K,), 5), (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(6))).to(BF16)
    h0 = seeded((K,), 7)
    d = lambda t: t.to(dev)
    w1d, w2d, xd, nwd = d(w1), d(w2), d(x), d(nw)
    y = torch.zeros(M, dtype=BF16, device=dev)
    h = h0.clone().to(dev)
    P = Program(4)
    b1 = P.new_barrier()
    b2 = P.new_barrier()
    for sm in range(2):
        r0 = sm * (M // 2)
        P.gemv(sm, w_addr=w1d.data_ptr() + r0 * K * 2, n_rows=M // 2, K=K, R=16, x=Src(xd.data_ptr(), K * 2),
               out=Dst(y.data_ptr() + r0 * 2, M, "store", release=b1), norm_w=Src(nwd.data_ptr(), K * 2), eps=1e-5)
    for i, sm in enumerate((2, 3)):
        r0 = i * (K // 2)
        P.gemv(sm, w_addr=w2d.data_ptr() + r0 * M * 2, n_rows=K // 2, K=M, R=16,
               x=Src(y.data_ptr(), M * 2, wait=b1), out=Dst(h.data_ptr() + r0 * 2, K, "add_bf16", release=b2))
    run_program(P, dev)
    y_ref = O.linear(O.rms_norm(x, nw, 1e-5)[None], w1)[0]
    h_ref = h0 + O.linear(y_ref[None], w2)[0]
    assert O.rel_l2(y.cpu(), y_ref) < 3e-3
    assert O.rel_l2(h.cpu(), h_ref) < 3e-3


def test_gemv_silu_pairs(cuda_device):
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    K, F = 1024, 384
    gate, up, x = seeded((F, K), 8, 0.05), seeded((F, K), 9, 0.05), seeded((K,), 10)
    wgu = torch.stack((gate, up), dim=1).reshape(2 * F, K).contiguous().to(dev)
    xd = x.to(dev)
    act = torch.zeros(F, dtype=BF16, device=dev)
    P = Program(3)
    per = 2 * F // 3
    for sm in range(3):
        r0 = sm * per
        P.gemv(sm, w_addr=wgu.data_ptr() + r0 * K * 2, n_rows=per, K=K, R=8, x=Src(xd.data_ptr(), K * 2),
               out=Dst(act.data_ptr() + r0, per, "store"), mode=isa.GEMV_MODE_SILU_PAIRS)
    run_program(P, dev)
    ref = O.silu_mul(O.linear(x[None], gate), O.linear(x[None], up))[0]
    assert O.rel_l2(act.cpu(), ref) < 5e-3


def test_gemv_argmax_and_final(cuda_device):
    """Vocabulary projection with per-SM candidates, then the final reduction,
    token log and state advance; a planted tie must resolve to the lower id."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    K, V, n_sms = 256, 2048, 4
    w, x = seeded((V, K), 11, 0.05), seeded((K,), 12)
    w[1500] = w[300]                       # identical logits at rows 300 and 1500
    ref = O.linear(x[None], w)[0]
    big = ref.float().abs().max() * 4
    scale = float(big / ref[300].float().abs().clamp_min(1e-3))
    w[300] = (w[300].float() * scale * math.copysign(1.0, float(ref[300]))).to(BF16)
    w[1500] = w[300]
    ref = O.linear(x[None], w)[0]
    assert int(torch.argmax(ref.float())) == 300
    wd, xd = w.to(dev), x.to(dev)
    logits = torch.zeros(V, dtype=BF16, device=dev)
    rec = torch.zeros(n_sms, 4, dtype=torch.float32, device=dev)
    state = torch.zeros(isa.ST_PAGETABLE + 4, dtype=torch.int32, device=dev)
    st = torch.zeros(isa.ST_PAGETABLE + 4, dtype=torch.int32)
    st[isa.ST_POS], st[isa.ST_NKVH], st[isa.ST_MAXPAGES] = 63, 2, 4
    st[isa.ST_PAGETABLE:] = torch.tensor([3, 1, 0, 2])
    state.copy_(st)
    log = torch.full((8,), -1, dtype=torch.int32, device=dev)
    P = Program(n_sms)
    b = P.new_barrier()
    per = V // n_sms
    for sm in range(n_sms):
        r0 = sm * per
        P.gemv(sm, w_addr=wd.data_ptr() + r0 * K * 2, n_rows=per, K=K, R=16, x=Src(xd.data_ptr(), K * 2),
               out=Dst(logits.data_ptr() + r0 * 2, per * 2, "store", release=b), mode=isa.GEMV_MODE_ARGMAX,
               pair_out=Dst(rec[sm].data_ptr(), 16, release=b), row_base=r0)
    P.argmax_final(1, records=Src(rec.data_ptr(), n_sms * 16, wait=b), n=n_sms, state_addr=state.data_ptr(),
                   log_addr=log.data_ptr())
    run_program(P, dev)
    assert O.rel_l2(logits.cpu(), ref) < 2e-3
    s = state.cpu()
    assert int(log[0]) == 300 and int(s[isa.ST_TOKEN]) == 300
    assert int(s[isa.ST_POS]) == 64 and int(s[isa.ST_NPAGES]) == 2 and int(s[isa.ST_STEP]) == 1
    assert int(s[isa.ST_NEWROW]) == 1 * 64 * 2 + 0      # page_table[1] == 1, row 0


@pytest.mark.parametrize("G,n_kv,pos,qk_norm,pages_per_split", [
    (4, 2, 200, False, 2),     # tail page half full, 2 splits busy of 3
    (4, 2, 63, False, 1),      # new row is the last row of page 0
    (4, 2, 64, False, 1),      # new row opens page 1
    (8, 1, 300, True, 2),      # Qwen3 style: per-head QK norm, group of 8
    (4, 1, 0, True, 4),        # empty cache: only the new row
])
def test_attention_split_merge_paged(cuda_device, G, n_kv, pos, qk_norm, pages_per_split):
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    D, theta, eps = 128, 500000.0, 1e-6
    max_pages = 8
    n_q = G * n_kv
    g = torch.Generator().manual_seed(100 + pos)
    q = torch.randn(n_q * D, generator=g).to(BF16)
    k_new = torch.randn(n_kv * D, generator=g).to(BF16)
    v_new = torch.randn(n_kv * D, generator=g).to(BF16)
    kc = torch.randn(pos + 1, n_kv, D, generator=g).to(BF16)
    vc = torch.randn(pos + 1, n_kv, D, generator=g).to(BF16)
    qn = (1 + 0.1 * torch.randn(D, generator=g)).to(BF16)
    kn = (1 + 0.1 * torch.randn(D, generator=g)).to(BF16)

    # oracle
    cos, sin = O.rope_cos_sin(torch.tensor([pos]), D, theta)
    qh, kh = q.view(n_q, D), k_new.view(n_kv, D)
    if qk_norm:
        qh, kh = O.rms_norm(qh, qn, eps), O.rms_norm(kh, kn, eps)
    qh, kh = O.apply_rope(qh, cos, sin), O.apply_rope(kh, cos, sin)
    kref, vref = kc.clone(), vc.clone()
    kref[pos], vref[pos] = kh, v_new.view(n_kv, D)
    ref = O.gqa_decode_attention(qh, kref, vref)

    # device buffers: paged pools with a shuffled page table; the new row is NOT in the pool yet
    table = torch.randperm(max_pages, generator=g).to(torch.int32)
    kpool = torch.zeros(max_pages, n_kv, 64, D, dtype=BF16)
    vpool = torch.zeros(max_pages, n_kv, 64, D, dtype=BF16)
    for p in range(pos):
        kpool[table[p // 64], :, p % 64] = kc[p]
        vpool[table[p // 64], :, p % 64] = vc[p]
    from vdcores_b200.decode import kv_page_swizzle       # page rows live in HBM in the bank-friendly piece order
    kpool, vpool = kv_page_swizzle(kpool).to(dev), kv_page_swizzle(vpool).to(dev)
    # projection output stored per KV head group: [G query heads | key | value]
    qkv = torch.cat([torch.cat((q.view(n_kv, G * D)[h], k_new.view(n_kv, D)[h], v_new.view(n_kv, D)[h]))
                     for h in range(n_kv)]).to(dev)
    fr = torch.arange(max_pages * 64, dtype=torch.float32)[:, None] * O.rope_inv_freq(D, theta)[None]
    rope = torch.cat((fr.cos().to(BF16).float(), fr.sin().to(BF16).float()), 1).contiguous().to(dev)
    nw = torch.cat((qn, kn)).to(dev)
    st = torch.zeros(isa.ST_PAGETABLE + max_pages, dtype=torch.int32)
    st[isa.ST_POS], st[isa.ST_NPAGES] = pos, pos // 64 + 1
    st[isa.ST_NEWROW] = int(table[pos // 64]) * 64 * n_kv + pos % 64
    st[isa.ST_NKVH], st[isa.ST_MAXPAGES] = n_kv, max_pages
    st[isa.ST_PAGETABLE:] = table
    state = st.to(dev)
    n_splits = (max_pages + pages_per_split - 1) // pages_per_split
    rec_floats = G * D + 16 * ((2 * G + 15) // 16)
    part = torch.zeros(n_kv, n_splits, rec_floats, dtype=torch.float32, device=dev)
    cnt = torch.zeros(n_kv, dtype=torch.int32, device=dev)
    out = torch.zeros(n_q * D, dtype=BF16, device=dev)

    n_sms = 5
    P = Program(n_sms)
    b_out = P.new_barrier()
    P.add_releases(b_out, n_kv)
    page_bytes = 64 * D * 2
    page_shift = int(math.log2(n_kv * page_bytes))
    sa = state.data_ptr()
    grp = (G + 2) * D * 2
    units = [(h, s) for s in range(n_splits) for h in range(n_kv)]
    for i, (h, s) in enumerate(units):
        P.attn_decode(
            i % n_sms, G=G, state_addr=sa,
            rope=Src(rope.data_ptr(), 512, indirect=(sa + 4 * isa.ST_POS, 9, None)),
            norm_w=Src(nw.data_ptr(), 512) if qk_norm else None,
            qkv=Src(qkv.data_ptr() + h * grp, grp),
            k_page_addr=kpool.data_ptr() + h * page_bytes, v_page_addr=vpool.data_ptr() + h * page_bytes,
            page_shift=page_shift, base_page=s * pages_per_split, max_pages=pages_per_split,
            records_addr=part[h].data_ptr(), counter_addr=cnt[h].data_ptr(),
            out_addr=out.data_ptr() + h * G * D * 2, split=s, n_splits=n_splits, release=b_out, qk_eps=eps)
    run_program(P, dev)
    assert int(cnt.abs().sum()) == 0, "the last arrival resets the head's counter"
    assert O.rel_l2(out.cpu(), ref) < 6e-3
    # the new K (normed + rotated) and V rows landed in the right page, nothing else changed
    page, row = int(table[pos // 64]), pos % 64
    kpool, vpool = kv_page_swizzle(kpool), kv_page_swizzle(vpool)
    assert O.rel_l2(kpool[page, :, row].cpu(), kh) < 6e-3
    assert torch.equal(vpool[page, :, row].cpu(), v_new.view(n_kv, D))
    if pos > 0:
        p0 = 0
        assert torch.equal(kpool[int(table[0]), :, p0].cpu(), kc[0])


def test_copy_with_token_gather(cuda_device):
    """Embedding-row gather: the source address is offset by a token id read from device memory."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    H, V = 512, 64
    table = seeded((V, H), 20).to(dev)
    tok = torch.tensor([37, 0, 0, 0], dtype=torch.int32, device=dev)
    dst = torch.zeros(H, dtype=BF16, device=dev)
    P = Program(2)
    b = P.new_barrier()
    P.copy(1, Src(table.data_ptr(), H * 2, indirect=(tok.data_ptr(), None, H * 2)),
           Dst(dst.data_ptr(), H * 2, release=b), H * 2)
    run_program(P, dev)
    assert torch.equal(dst, table[37])


def test_wait_budget_returns_status_instead_of_hanging(cuda_device):
    """A load that waits on a barrier nobody releases: the kernel must give up
    within the budget and report which barrier, and the context stays usable."""
    from vdcores_b200 import isa, runtime
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    src = torch.zeros(1024, dtype=BF16, device=dev)
    dst = torch.zeros(1024, dtype=BF16, device=dev)
    P = Program(2)
    b = P.new_barrier()
    P.bar_counts[b] = 1                                    # nobody counts it down
    P.copy(0, Src(src.data_ptr(), 2048, wait=b), Dst(dst.data_ptr(), 2048), 2048)
    P.insts_per_sm = 16
    c, m, bars = P.finalize()
    prof = torch.zeros(2 * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    with pytest.raises(runtime.VdcError) as ei:
        runtime.launch_dae(2, 0, torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev), None,
                           torch.from_numpy(bars).to(dev), prof, 0, timeout_ns=50_000_000, insts_per_sm=16)
    assert ei.value.code == isa.ERR_TIMEOUT and ei.value.status["bar"] == b
    # the context is still healthy
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


@pytest.mark.parametrize("own,depth", [(0, 0), (3, 6)])
def test_gemv_chunks_drawn_from_a_shared_counter(cuda_device, own, depth):
    """Six SMs run the same projection over the whole matrix: each streams the chunks it owns, then they draw the
    rest from one counter (OP_DYN_CHUNKS).  Every row must be computed exactly once, whoever took its chunk."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    M, K, R, S = 1024, 2048, 8, 6
    w, x = seeded((M, K), 51, 0.02), seeded((K,), 52)
    h0 = seeded((M,), 53)
    wd, xd = w.to(dev), x.to(dev)
    h = h0.clone().to(dev)
    P = Program(S)
    ctr, done = P.new_barrier(), P.new_barrier()
    for sm in range(S):
        P.gemv(sm, w_addr=wd.data_ptr(), n_rows=M, K=K, R=R, x=Src(xd.data_ptr(), K * 2),
               out=Dst(h.data_ptr(), M * 2, "add_bf16", release=done), shared_counter=ctr, own_chunks=(sm * own, own),
               shared_first=S * own, shared_depth=depth)
    n = max(max(len(a) for a in P.m), max(len(a) for a in P.c)) + 2
    P.insts_per_sm = ((n + 15) // 16) * 16
    c, m, bars = P.finalize()
    bt = torch.from_numpy(bars).to(dev)
    prof = torch.zeros(S * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    from vdcores_b200 import runtime
    runtime.launch_dae(S, 0, torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev), None, bt, prof, 0,
                       timeout_ns=TIMEOUT_NS, insts_per_sm=P.insts_per_sm)
    assert int(bt[done]) == 0
    drawn = int(bt[ctr])
    assert M // R - S * own <= drawn <= M // R - S * own + 2 * S     # every chunk once, at most two overshoots per SM
    ref = h0 + O.linear(x[None], w)[0]
    assert O.rel_l2(h.cpu(), ref) < 3e-3


def test_gemv_gives_up_together_when_its_activation_never_arrives(cuda_device):
    """A projection whose activation barrier nobody releases, next to one that streams normally:
    the waiting task reports the barrier, the streaming task's warp pairs leave their loop together
    (no member is left alone at a pair barrier), the kernel retires and the context stays usable."""
    from vdcores_b200 import isa, runtime
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    K, M = 1024, 2048
    w, x = seeded((M, K), 41, 0.02).to(dev), seeded((K,), 42).to(dev)
    y = torch.zeros(2 * M, dtype=BF16, device=dev)
    P = Program(2)
    b = P.new_barrier()
    P.bar_counts[b] = 1                                    # nobody counts it down
    P.gemv(0, w_addr=w.data_ptr(), n_rows=M, K=K, R=16, x=Src(x.data_ptr(), K * 2, wait=b),
           out=Dst(y.data_ptr(), M * 2, "store"))
    for _ in range(8):                                      # SM 1 keeps streaming while SM 0 waits
        P.gemv(1, w_addr=w.data_ptr(), n_rows=M, K=K, R=16, x=Src(x.data_ptr(), K * 2),
               out=Dst(y.data_ptr() + M * 2, M * 2, "store"))
    P.insts_per_sm = 64
    c, m, bars = P.finalize()
    prof = torch.zeros(2 * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    with pytest.raises(runtime.VdcError) as ei:
        runtime.launch_dae(2, 0, torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev), None,
                           torch.from_numpy(bars).to(dev), prof, 0, timeout_ns=50_000_000, insts_per_sm=64)
    assert ei.value.code == isa.ERR_TIMEOUT and ei.value.status["bar"] == b and ei.value.status["sm"] == 0
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    # a task that expects one more weight chunk than its memory stream delivers: the pair that owns
    # the missing chunk gives up inside the streaming loop, both of its warps together
    P3 = Program(1)
    P3.gemv(0, w_addr=w.data_ptr(), n_rows=M, K=K, R=16, x=Src(x.data_ptr(), K * 2), out=Dst(y.data_ptr(), M * 2, "store"))
    op, n_chunks, a1, a2 = P3.c[0][0]
    P3.c[0][0] = (op, n_chunks + 1, a1, a2)
    P3.insts_per_sm = 16
    c, m, bars = P3.finalize()
    with pytest.raises(runtime.VdcError) as ei:
        runtime.launch_dae(1, 0, torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev), None,
                           torch.from_numpy(bars).to(dev), prof, 0, timeout_ns=20_000_000, insts_per_sm=16)
    assert ei.value.code == isa.ERR_TIMEOUT
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    # and the same streams run to completion once the barrier is released by a third SM
    P2 = Program(3)
    b2 = P2.new_barrier()
    P2.gemv(0, w_addr=w.data_ptr(), n_rows=M, K=K, R=16, x=Src(x.data_ptr(), K * 2, wait=b2),
            out=Dst(y.data_ptr(), M * 2, "store"))
    P2.copy(2, Src(x.data_ptr(), 256), Dst(y.data_ptr() + M * 2, 256, release=b2), 256)
    y.zero_()
    run_program(P2, dev)
    assert O.rel_l2(y[:M].cpu(), O.linear(x.cpu()[None], w.cpu())[0]) < 2e-3


@pytest.mark.parametrize("M,K,R,n_sms", [(256, 4096, 8, 4), (64, 14336, 2, 2), (128, 512, 16, 1)])
def test_gemv_fp8_store(cuda_device, M, K, R, n_sms):
    """e4m3 weights with per-row fp32 scales, dequantised in registers; the oracle
    multiplies the same codes and scales in fp32."""
    from vdcores_b200.decode import quantize_fp8_rows
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    w, x = seeded((M, K), 31, 0.02), seeded((K,), 32)
    lin = O.QLinear.make(w, "fp8")
    q, sc = quantize_fp8_rows(w)             # on the CPU: the same conversion the oracle used
    assert torch.equal(q, lin.q.view(torch.uint8)) and torch.equal(sc, lin.scale)
    q, sc, xd = q.to(dev), sc.to(dev), x.to(dev)
    y = torch.zeros(M, dtype=BF16, device=dev)
    P = Program(n_sms)
    per = M // n_sms
    for sm in range(n_sms):
        r0 = sm * per
        P.gemv(sm, w_addr=q.data_ptr() + r0 * K, n_rows=per, K=K, R=R, x=Src(xd.data_ptr(), K * 2),
               out=Dst(y.data_ptr() + r0 * 2, per * 2, "store"), fp8_scales=sc.data_ptr() + 4 * r0)
    run_program(P, dev)
    assert O.rel_l2(y.cpu(), lin(x[None])[0]) < 3e-3


@pytest.mark.parametrize("M,K,R,n_sms", [(128, 4096, 8, 2), (32, 12288, 4, 2), (64, 1024, 16, 1)])
def test_gemv_nvfp4_store(cuda_device, M, K, R, n_sms):
    """NVFP4 rows (e2m1 pairs + e4m3 block scales per 16 + fp32 tensor scale); block
    dots in half precision, fp32 across blocks.  Against the oracle's fp32 dequantised product."""
    from vdcores_b200.decode import quantize_nvfp4_rows
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    w, x = seeded((M, K), 41, 0.02), seeded((K,), 42)
    lin = O.QLinear.make(w, "nvfp4")
    rows, ts = quantize_nvfp4_rows(w)
    assert torch.equal(rows[:, :K // 2], lin.q)
    rows, xd = rows.to(dev), x.to(dev)
    sc = ts.expand(M).contiguous().to(dev)
    rb = K // 2 + K // 16
    y = torch.zeros(M, dtype=BF16, device=dev)
    P = Program(n_sms)
    per = M // n_sms
    for sm in range(n_sms):
        r0 = sm * per
        P.gemv(sm, w_addr=rows.data_ptr() + r0 * rb, n_rows=per, K=K, R=R, x=Src(xd.data_ptr(), K * 2),
               out=Dst(y.data_ptr() + r0 * 2, per * 2, "store"), nvfp4_scales=sc.data_ptr() + 4 * r0)
    run_program(P, dev)
    assert O.rel_l2(y.cpu(), lin(x[None])[0]) < 5e-3
