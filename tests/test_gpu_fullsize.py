"""One decoder layer at the full shapes of the quantised and mixture-of-experts configurations, on a
B200 against the CPU oracle: FP8-e4m3 Llama-3.1-8B layer at position 2048, NVFP4 Qwen3-8B layer
(FFN 12288, per-head QK norm, theta 1e6) at position 4096, Qwen3-30B-A3B layer (hidden 2048, 32q/4kv
heads, 128 experts of width 768, top-8) at position 1024.  The small-model tests never reach these
row lengths, expert counts or group sizes.  Bars: hidden state rel-L2 3e-2 / 6e-2 / 1e-2, new K/V
rows at twice that, and for the mixture the selected experts and their weights.

Same structure as the reference's single-layer correctness run (reference
app/python/llama3/sched.py:574-622), on seeded random weights of the named shapes."""
import dataclasses

import pytest
import torch

from oracle import decode_oracle as O
from tests.helpers import dense_weights, engine_config

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def one_layer_case(cfg: O.DecodeConfig, pos: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    lw = O.LayerWeights.random(cfg, gen)
    # norm weights away from 1 so that the affine part counts
    r = lambda n: (1.0 + 0.1 * torch.randn(n, generator=gen)).to(BF16)
    lw.ln1, lw.ln2 = r(cfg.hidden), r(cfg.hidden)
    if cfg.qk_norm:
        lw.q_norm, lw.k_norm = r(cfg.head_dim), r(cfg.head_dim)
    if lw.router is not None:       # N(0, 0.02) router logits are nearly flat: spread them out
        lw.router = (lw.router.float() * 8).to(BF16)
    hidden = torch.randn(cfg.hidden, generator=gen).to(BF16)
    kc = torch.randn(pos + 1, cfg.n_kv_heads, cfg.head_dim, generator=gen).to(BF16)
    vc = torch.randn(pos + 1, cfg.n_kv_heads, cfg.head_dim, generator=gen).to(BF16)
    return lw, hidden, kc, vc


@pytest.mark.parametrize("name,tol", [("llama8b_fp8", 3e-2), ("qwen3_8b_nvfp4", 6e-2), ("qwen3_30b_a3b", 1e-2)])
def test_full_shape_layer_matches_oracle(cuda_device, name, tol):
    from vdcores_b200.decode import DecodeEngine
    if name == "llama8b_fp8":
        base, wkind, pos = dataclasses.replace(O.LLAMA31_8B, n_layers=1, vocab=8), "fp8", 2048
    elif name == "qwen3_8b_nvfp4":
        base, wkind, pos = dataclasses.replace(O.QWEN3_8B, n_layers=1, vocab=8, wkind="bf16"), "nvfp4", 4096
    else:
        base, wkind, pos = dataclasses.replace(O.QWEN3_30B_A3B, n_layers=1, vocab=8), "bf16", 1024
    lw_b, hidden, kc, vc = one_layer_case(base, pos, seed=21)
    cfg = dataclasses.replace(base, wkind=wkind)
    lw = lw_b
    if wkind != "bf16":
        lw = dataclasses.replace(lw_b)
        for n in ("wq", "wk", "wv", "wo", "gate", "up", "down"):
            setattr(lw, n, O.QLinear.make(getattr(lw_b, n).w, wkind))
    # ---- oracle
    cap = {}
    kc_o, vc_o = kc.clone(), vc.clone()
    out_ref = O.decode_layer(cfg, lw, hidden, pos, kc_o, vc_o, cap)
    # ---- device: the layer input enters as the embedding row of token 0
    embed = torch.zeros(8, cfg.hidden, dtype=BF16)
    embed[0] = hidden
    w = O.ModelWeights(base, embed, [lw_b], torch.ones(cfg.hidden, dtype=BF16), torch.zeros(8, cfg.hidden, dtype=BF16))
    max_seq = ((pos + 1 + 63) // 64) * 64
    eng = DecodeEngine(engine_config(base), max_seq=max_seq, device=cuda_device, taps=True, wkind=wkind,
                       page_perm_seed=9, timeout_ns=500_000_000)
    eng.load_weights(dense_weights(w))
    eng.load_kv([kc[:pos]], [vc[:pos]])
    eng.set_state(pos, 0)
    eng.generate(1)
    out = eng.taps[0].cpu()
    r = O.rel_l2(out, out_ref)
    assert r < tol, f"{name}: hidden state rel-L2 {r:.3e}"
    k_dev, v_dev = eng.read_kv(0, pos + 1)
    assert O.rel_l2(k_dev[pos].cpu(), kc_o[pos]) < 2 * tol
    assert O.rel_l2(v_dev[pos].cpu(), vc_o[pos]) < 2 * tol
    # rows of the cache that existed before the step are untouched
    assert torch.equal(k_dev[:pos].cpu(), kc[:pos]) and torch.equal(v_dev[:pos].cpu(), vc[:pos])
    if cfg.n_experts:
        w_ref, idx_ref = O.moe_route(cap["post_attn_rms"][None], lw.router, cfg.top_k)
        probs = torch.softmax(cap["post_attn_rms"].float() @ lw.router.float().t(), dim=-1)
        p_k = float(torch.topk(probs, cfg.top_k).values[-1])
        route = eng.route.cpu()
        ids = route[:cfg.top_k].tolist()
        wts = route[16:16 + cfg.top_k].view(torch.float32).tolist()
        assert len(set(ids)) == cfg.top_k
        # experts clearly above the k-th probability must be selected, selected ones must not be clearly below it
        must = {e for e in range(cfg.n_experts) if float(probs[e]) > 1.01 * p_k}
        assert must <= set(ids), (sorted(must), ids)
        assert all(float(probs[e]) >= 0.99 * p_k for e in ids), ids
        if set(ids) == set(idx_ref[0].tolist()):
            ref = dict(zip(idx_ref[0].tolist(), w_ref[0].float().tolist()))
            for e, wt in zip(ids, wts):
                assert abs(wt - ref[e]) <= 2e-2 * max(ref.values()), (e, wt, ref[e])
