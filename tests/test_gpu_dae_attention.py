"""The reference's decode-attention operators on their own tile contracts, driven through this repository's
``dae`` package on a B200 the way app/python/attention_simple_decoding.py and attention_split_kv.py of the
reference drive them: Q through a five-dimensional tensor map that replicates the query rows into a 64-row
K-major tile, K blocks K-major and V blocks MN-major with the 128-byte swizzle, the fused QK-norm + interleaved
RoPE path with its side-input row and the k-store write-back, the split variant with its log-sum-exp table and
ATTN_SPLIT_POST_REDUCE.  Checked against the torch expressions of those scripts (`gqa_ref`), mean relative
difference under the 5 % budget of the reference's model script, plus a tighter rel-L2 bar."""
import os
import sys
from math import sqrt

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "vdcores_b200"))
D, KVT = 128, 64
BF16 = torch.bfloat16


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def k_map(n_kv):
    """K blocks of [64 positions x 128] from a [1, S, n_kv, 128] cache (tiled axis: the positions)."""
    from functools import partial
    import dae.model as M
    return partial(M.build_tma_wgmma_k, iN=-3), partial(M.cord_func_K_major, iN=-3)


def v_map(n_kv):
    """V blocks MN-major: per 8 positions two atoms of 64 dims x 8 rows."""
    from functools import partial
    import dae.model as M
    return partial(M.build_tma_wgmma_mn, iK=-3), partial(M.cord_func_MN_major, iK=-3)


def q_map(n_rows_src, row_stride_bytes, replicas, n_items):
    """The query rows of one item (n_rows_src rows, row_stride apart), replicated `replicas` times through a zero
    stride into a 64-row tile: app/python/attention_simple_decoding.py:93-113 (1 row x 64) and
    attention_split_kv.py (4 rows x 16)."""
    from dae import runtime

    def build(mat, tile_k, tile_n):
        return 5, runtime.build_tma_desc(mat, [64, n_rows_src, replicas, 2, n_items],
                                         [row_stride_bytes, 0, 128, n_rows_src * row_stride_bytes],
                                         [64, n_rows_src, replicas, 2, 1], [1] * 5, 128, 0)

    def cords(mat, rank):
        return lambda req, item: [0, 0, 0, item]
    return build, cords


def rope_rows(n, theta, dev):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    fr = torch.outer(torch.arange(n, device=dev, dtype=torch.float32), inv)
    rope = torch.empty(n, D, device=dev, dtype=BF16)
    rope[:, 0::2], rope[:, 1::2] = fr.cos().to(BF16), fr.sin().to(BF16)
    return rope


def norm_rope(x, w, rope_row):
    """RMS-norm with weight, then rotation of the pairs (2i, 2i+1) by (cos, sin); fp32, one rounding."""
    x = x.float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    e, o = x[..., 0::2], x[..., 1::2]
    c, s = rope_row[..., 0::2].float(), rope_row[..., 1::2].float()
    return torch.stack((e * c - o * s, e * s + o * c), -1).flatten(-2).to(BF16)


def gqa(Q, K, V, n_active):
    """Q [n_kv, G, 128], K / V [S, n_kv, 128]; positions >= n_active masked."""
    Kh, Vh = K.permute(1, 0, 2).float(), V.permute(1, 0, 2).float()
    s = torch.matmul(Q.float(), Kh.transpose(-1, -2)) / sqrt(D)
    s = s.masked_fill(torch.arange(K.shape[0], device=K.device)[None, None, :] >= n_active, float("-inf"))
    return torch.matmul(torch.softmax(s, -1), Vh)


@pytest.mark.parametrize("n_blocks,last_len,fused", [(1, 48, True), (3, 17, True), (2, 64, False)])
def test_attention_simple_decoding(cuda_device, n_blocks, last_len, fused):
    """One SM per query head (32 heads over 8 KV heads), as app/python/attention_simple_decoding.py."""
    from dae.launcher import Launcher
    import dae.instructions as I
    gpu = cuda_device
    torch.manual_seed(0)
    n_q, n_kv, S = 32, 8, n_blocks * KVT
    G = n_q // n_kv
    n_active = (n_blocks - 1) * KVT + last_len
    pos = n_active - 1
    matQ = torch.rand(1, n_q * D, dtype=BF16, device=gpu) - 0.5
    matK = torch.rand(S, n_kv * D, dtype=BF16, device=gpu) - 0.5
    matV = torch.rand(S, n_kv * D, dtype=BF16, device=gpu) - 0.5
    matO = torch.zeros(1, n_q * D, dtype=BF16, device=gpu)
    Kv, Vv = matK.view(1, S, n_kv, D), matV.view(1, S, n_kv, D)
    qw = 0.75 + 0.5 * torch.rand(D, dtype=BF16, device=gpu)
    kw = 0.75 + 0.5 * torch.rand(D, dtype=BF16, device=gpu)
    rope = rope_rows(S, 1.0e6, gpu)
    side = torch.empty(S, 3 * D, dtype=BF16, device=gpu)
    side[:, :D], side[:, D:2 * D], side[:, 2 * D:] = qw, kw, rope
    k_raw = Kv[0, pos].clone()
    if fused and pos > 0:           # the cache holds finished rows for the earlier positions
        Kv[0, :pos] = norm_rope(Kv[0, :pos], kw, rope[:pos].view(pos, 1, D))
    dae = Launcher(n_q, device=gpu)
    dae.timeout_ns = 300_000_000
    tQ = I.TmaTensor(dae, matQ.view(1, n_q, D))._build("load", D, 64, *q_map(1, D * 2, 64, n_q))
    tK = I.TmaTensor(dae, Kv)._build("load", D, KVT, *k_map(n_kv))
    tV = I.TmaTensor(dae, Vv)._build("load", D, KVT, *v_map(n_kv))
    tSide = I.TmaTensor(dae, side).tensor1d("load", 3 * D)
    kst = I.TmaTensor(dae, matK.view(S, n_kv * D)).tensor1d("store", D)

    def sm_task(sm):
        head, kvh = sm, sm // G
        return [
            I.ATTENTION_M64N64K16_F16_F32_64_64_hdim(n_blocks, last_len, need_norm=fused, need_rope=fused),
            tSide.cord(pos * 3 * D) if fused else [],
            kst.cord((pos * n_kv + kvh) * D) if fused else [],
            tQ.cord(0, head),
            I.RepeatM.on(n_blocks - 1, [tK.cord(0, 0, kvh, 0), tK.cord2tma(0, KVT, 0, 0)],
                         [tV.cord(0, 0, kvh, 0), tV.cord2tma(0, KVT, 0, 0)]),
            tK.cord(0, KVT * (n_blocks - 1), kvh, 0),
            tV.cord(0, KVT * (n_blocks - 1), kvh, 0),
            I.TmaStore1D(matO.view(1, n_q, D)[0, head, ...]),
        ]

    dae.i(sm_task, I.TerminateC(), I.TerminateM())
    dae.launch()
    Q = matQ.view(n_kv, G, D)
    K_ref = Kv[0].clone()
    if fused:
        Q = norm_rope(Q, qw, rope[pos].view(1, 1, D))
        k_new = norm_rope(k_raw, kw, rope[pos].view(1, D))
        assert rel_l2(Kv[0, pos], k_new) < 1e-2, "the finished key row was stored into the cache"
        K_ref[pos] = k_new
    ref = gqa(Q, K_ref, Vv[0], n_active).reshape(n_q, D)
    got = matO.view(n_q, D)
    assert rel_l2(got, ref) < 1e-2
    diff = float(((got.float() - ref).abs().mean() / ref.abs().mean()) * 100)
    assert diff < 5.0


def test_attention_split_kv_and_post_reduce(cuda_device):
    """app/python/attention_split_kv.py: one SM per (split, KV head) with the head group's four query rows in
    one tile, a log-sum-exp table in global memory, and the first SMs reducing the splits."""
    from dae.launcher import Launcher
    import dae.instructions as I
    gpu = cuda_device
    torch.manual_seed(1)
    n_q, n_kv, splits, blocks_per_split, last_len = 32, 8, 2, 2, 40
    G, S = n_q // n_kv, splits * blocks_per_split * KVT
    n_active = S - KVT + last_len
    matQ = torch.rand(1, n_q * D, dtype=BF16, device=gpu) - 0.5
    matK = torch.rand(S, n_kv * D, dtype=BF16, device=gpu) - 0.5
    matV = torch.rand(S, n_kv * D, dtype=BF16, device=gpu) - 0.5
    matO = torch.zeros(1, n_q * D, dtype=BF16, device=gpu)
    matO_split = torch.zeros(n_kv, splits, G, D, dtype=BF16, device=gpu)      # per KV head: the splits' rows together
    matP = torch.zeros(n_kv, G, 16, dtype=torch.float32, device=gpu)
    Kv, Vv = matK.view(1, S, n_kv, D), matV.view(1, S, n_kv, D)
    num_sms = n_kv * splits
    dae = Launcher(num_sms, device=gpu)
    dae.timeout_ns = 300_000_000
    import dae.model as M
    tQ = I.TmaTensor(dae, matQ.view(1, n_kv, G, D))._build("load", D, 64, M.tma_gqa_load_q, M.cord_gqa_load_q)
    tK = I.TmaTensor(dae, Kv)._build("load", D, KVT, *k_map(n_kv))
    tV = I.TmaTensor(dae, Vv)._build("load", D, KVT, *v_map(n_kv))
    bar = dae.new_bar(num_sms)

    def sm_task(sm):
        split, head = divmod(sm, n_kv)
        start = split * blocks_per_split * KVT
        ll = last_len if split == splits - 1 else KVT
        insts = [
            I.ATTENTION_M64N64K16_F16_F32_64_64_hdim_split(blocks_per_split, split, G, ll, start, need_norm=False, need_rope=False),
            tQ.cord(0, head),
            I.RepeatM.on(blocks_per_split, [tK.cord(0, start, head, 0), tK.cord2tma(0, KVT, 0, 0)],
                         [tV.cord(0, start, head, 0), tV.cord2tma(0, KVT, 0, 0)]),
            I.TmaStore1D(matO_split[head, split, ...], numSlots=2),
            I.RawAddress(matP[head], 24).bar(bar).writeback(),
        ]
        if sm < n_kv:
            insts += [
                I.ATTN_SPLIT_POST_REDUCE(splits),
                I.RawAddress(matP[head], 25).bar(bar),
                I.TmaLoad1D(matO_split[head, ...]),
                I.TmaStore1D(matO.view(n_kv, G, D)[head, ...]),
            ]
        return insts

    dae.i(sm_task, I.TerminateC(), I.TerminateM())
    dae.launch()
    Q = matQ.view(n_kv, G, D)
    # every split alone: locally normalised output and log2-sum-exp of the scaled scores
    for s in range(splits):
        lo, hi = s * blocks_per_split * KVT, (s + 1) * blocks_per_split * KVT
        act = hi - lo if s < splits - 1 else n_active - lo
        ref_s = gqa(Q, Kv[0, lo:hi], Vv[0, lo:hi], act)
        assert rel_l2(matO_split[:, s], ref_s) < 1e-2
        sc = torch.matmul(Q.float(), Kv[0, lo:hi].permute(1, 0, 2).float().transpose(-1, -2)) / sqrt(D)
        sc = sc.masked_fill(torch.arange(hi - lo, device=gpu)[None, None, :] >= act, float("-inf"))
        lse2 = torch.logsumexp(sc, -1) * 1.4426950408889634
        assert torch.allclose(matP[:, :, s], lse2, atol=2e-2), "log2-sum-exp table"
    ref = gqa(Q, Kv[0], Vv[0], n_active).reshape(n_q, D)
    assert rel_l2(matO.view(n_q, D), ref) < 1.5e-2


def test_sched_attention_decoding(cuda_device):
    """The schedule class (python/dae/schedule.py:250-325 of the reference) with the fused QK-norm + RoPE path: one
    SM per head, barriers "q", "k", "o" bound late."""
    from dae.launcher import Launcher
    import dae.instructions as I
    import dae.schedule as Sd
    gpu = cuda_device
    torch.manual_seed(2)
    n_heads, n_blocks, last_len = 8, 2, 33                 # one query head per KV head
    S = n_blocks * KVT
    seq_len = (n_blocks - 1) * KVT + last_len
    pos = seq_len - 1
    matQ = torch.rand(1, n_heads, D, dtype=BF16, device=gpu) - 0.5
    matK = torch.rand(S, n_heads * D, dtype=BF16, device=gpu) - 0.5
    matV = torch.rand(S, n_heads * D, dtype=BF16, device=gpu) - 0.5
    matO = torch.zeros(1, n_heads, D, dtype=BF16, device=gpu)
    Kv, Vv = matK.view(1, S, n_heads, D), matV.view(1, S, n_heads, D)
    qw = 0.75 + 0.5 * torch.rand(D, dtype=BF16, device=gpu)
    kw = 0.75 + 0.5 * torch.rand(D, dtype=BF16, device=gpu)
    rope = rope_rows(S, 1.0e6, gpu)
    side = torch.empty(S, 3 * D, dtype=BF16, device=gpu)
    side[:, :D], side[:, D:2 * D], side[:, 2 * D:] = qw, kw, rope
    k_raw = Kv[0, pos].clone()
    Kv[0, :pos] = norm_rope(Kv[0, :pos], kw, rope[:pos].view(pos, 1, D))
    dae = Launcher(n_heads, device=gpu)
    dae.timeout_ns = 300_000_000
    tQ = I.TmaTensor(dae, matQ)._build("load", D, 64, *q_map(1, D * 2, 64, n_heads))
    tK = I.TmaTensor(dae, Kv)._build("load", D, KVT, *k_map(n_heads))
    tV = I.TmaTensor(dae, Vv)._build("load", D, KVT, *v_map(n_heads))
    tSide = I.TmaTensor(dae, side).tensor1d("load", 3 * D)
    kst = [I.TmaTensor(dae, matK.view(S, n_heads * D)).tensor1d("store", D)]
    sched = Sd.SchedAttentionDecoding(1, seq_len, KVT, n_heads, matO, (tQ, tK, tV), side_input=tSide, k_store=kst,
                                      token_pos=pos).place(n_heads)
    dae.s(sched)
    dae.i(I.TerminateC(), I.TerminateM())
    dae.launch()
    Q = norm_rope(matQ[0].view(n_heads, 1, D), qw, rope[pos].view(1, 1, D))
    K_ref = Kv[0].clone()
    K_ref[pos] = norm_rope(k_raw, kw, rope[pos].view(1, D))
    ref = gqa(Q, K_ref, Vv[0], seq_len).reshape(n_heads, D)
    assert rel_l2(matO[0], ref) < 1e-2
