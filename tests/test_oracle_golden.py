"""The CPU oracle against the golden fixtures produced from Hugging Face
transformers and the reference's attention helper (tests/golden/make_golden.py).
No GPU, no transformers, no reference tree needed."""
import os

import numpy as np
import pytest
import torch

from oracle import decode_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BF16 = torch.bfloat16


def load(name):
    return np.load(os.path.join(GOLD, name))


def weights_from_state_dict(z, cfg: O.DecodeConfig) -> O.ModelWeights:
    # weights are stored as bf16 bit patterns ("wb." keys): the Hugging Face models were bf16
    g = lambda k: torch.from_numpy(z["wb." + k].view(np.int16)).view(BF16)
    layers = []
    for i in range(cfg.n_layers):
        p = f"model.layers.{i}."
        mk = lambda k: O.QLinear.make(g(p + k), "bf16")
        lw = O.LayerWeights(ln1=g(p + "input_layernorm.weight"), ln2=g(p + "post_attention_layernorm.weight"),
                            wq=mk("self_attn.q_proj.weight"), wk=mk("self_attn.k_proj.weight"),
                            wv=mk("self_attn.v_proj.weight"), wo=mk("self_attn.o_proj.weight"))
        if cfg.qk_norm:
            lw.q_norm, lw.k_norm = g(p + "self_attn.q_norm.weight"), g(p + "self_attn.k_norm.weight")
        if cfg.n_experts:
            lw.router = g(p + "mlp.gate.weight")
            gu, dn = g(p + "mlp.experts.gate_up_proj"), g(p + "mlp.experts.down_proj")
            for e in range(cfg.n_experts):
                lw.experts.append((O.QLinear.make(gu[e, :cfg.ffn].contiguous(), "bf16"),
                                   O.QLinear.make(gu[e, cfg.ffn:].contiguous(), "bf16"),
                                   O.QLinear.make(dn[e].contiguous(), "bf16")))
        else:
            lw.gate, lw.up, lw.down = mk("mlp.gate_proj.weight"), mk("mlp.up_proj.weight"), mk("mlp.down_proj.weight")
        layers.append(lw)
    return O.ModelWeights(cfg, g("model.embed_tokens.weight"), layers, g("model.norm.weight"), g("lm_head.weight"))


CFGS = {
    "llama_small.npz": O.DecodeConfig(hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                                      n_layers=3, eps=1e-5, theta=500000.0),
    "qwen3_small.npz": O.DecodeConfig(hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                                      n_layers=3, eps=1e-6, theta=1e6, qk_norm=True),
    "qwen3moe_small.npz": O.DecodeConfig(hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=128, vocab=512,
                                         n_layers=3, eps=1e-6, theta=1e6, qk_norm=True, n_experts=16, top_k=4),
}


@pytest.mark.parametrize("name", list(CFGS))
def test_decode_step_matches_hf_fixture(name):
    """Prefill 36 tokens, decode the 37th: every hooked module output of the
    last step, the KV cache and the logits agree with HF within bf16 noise."""
    z, cfg = load(name), CFGS[name]
    w = weights_from_state_dict(z, cfg)
    prompt = z["prompt"].tolist()
    orc = O.DecodeOracle(w, 64)
    orc.prefill(prompt[:-1])
    caps = []
    logits, nxt, gap = orc.step(prompt[-1], caps)
    T = len(prompt)
    for i in range(cfg.n_layers):
        # the bar on hidden states (layer outputs) is rel-L2 1e-2; the module outputs in
        # between are increments on top of them and get twice that (the reference itself
        # accepts 5 % mean relative difference there, app/python/llama3/sched.py:585-607)
        assert O.rel_l2(caps[i]["hidden_state_out"], torch.from_numpy(z[f"{i}.hidden_state_out"])) < 1e-2, i
        for key in ("input_rms", "q_proj", "k_proj", "v_proj", "o_proj", "post_attn_rms"):
            assert O.rel_l2(caps[i][key], torch.from_numpy(z[f"{i}.{key}"])) < 2e-2, (i, key)
        if not cfg.n_experts:
            for key in ("gate_proj", "up_proj", "down_proj"):
                assert O.rel_l2(caps[i][key], torch.from_numpy(z[f"{i}.{key}"])) < 2e-2, (i, key)
        else:
            assert O.rel_l2(caps[i]["down_proj"], torch.from_numpy(z[f"{i}.mlp_out"])) < 2e-2
        kc = torch.from_numpy(z[f"{i}.k_cache"]).permute(1, 0, 2)       # [T, kv, d], post-RoPE
        vc = torch.from_numpy(z[f"{i}.v_cache"]).permute(1, 0, 2)
        assert O.rel_l2(orc.k[i][:T], kc) < 1e-2 and O.rel_l2(orc.v[i][:T], vc) < 1e-2
    ref_logits = torch.from_numpy(z["logits"])
    assert O.rel_l2(logits, ref_logits) < 1e-2
    top2 = torch.topk(ref_logits, 2).values
    if float(top2[0] - top2[1]) > 1e-2:
        assert nxt == int(ref_logits.argmax())


def test_attention_matches_reference_helper():
    """Second witness: the reference's own pure-torch attention helper
    (app/python/llama3/llama_attention_reference.py) on 9 positions."""
    z = load("llama_small_refattn.npz")
    q, k, v = (torch.from_numpy(z[n]).to(BF16) for n in ("q", "k", "v"))
    ref = torch.from_numpy(z["pre_o"])
    T, d = q.shape[0], 64
    cos, sin = O.rope_cos_sin(torch.arange(T), d, 500000.0)
    qh = O.apply_rope(q.view(T, 8, d), cos[:, None], sin[:, None])
    kh = O.apply_rope(k.view(T, 2, d), cos[:, None], sin[:, None])
    vh = v.view(T, 2, d)
    for t in range(T):
        out = O.gqa_decode_attention(qh[t], kh[: t + 1], vh[: t + 1])
        assert O.rel_l2(out, ref[t]) < 1e-2, t


def test_full_size_layer_matches_hf_fixture():
    """BASELINE config 1: one Llama-3.1-8B-shaped layer, seed 0, position 1024."""
    z = load("llama8b_layer_pos1024.npz")
    cfg = O.DecodeConfig(n_layers=1, vocab=8)
    gen = torch.Generator().manual_seed(0)
    lw = O.LayerWeights.random(cfg, gen)
    hidden = torch.randn(cfg.hidden, generator=gen).to(BF16)
    kc = torch.zeros(1025, 8, 128, dtype=BF16)
    vc = torch.zeros(1025, 8, 128, dtype=BF16)
    kc[:1024] = torch.randn(1024, 8, 128, generator=gen).to(BF16)
    vc[:1024] = torch.randn(1024, 8, 128, generator=gen).to(BF16)
    # the regenerated inputs are the ones the fixture was made from
    assert np.array_equal(hidden[:8].float().numpy(), z["hidden_in_head"])
    assert np.array_equal(lw.wq.w[0, :8].float().numpy(), z["wq_head"])
    O.FAST_LINEAR = True
    try:
        out = O.decode_layer(cfg, lw, hidden, 1024, kc, vc)
    finally:
        O.FAST_LINEAR = False
    assert O.rel_l2(out, torch.from_numpy(z["hidden_out"])) < 1e-2
    assert O.rel_l2(kc[1024], torch.from_numpy(z["k_new"])) < 1e-2
    assert O.rel_l2(vc[1024], torch.from_numpy(z["v_new"])) < 1e-2


def test_codecs_against_fixture():
    z = load("codecs.npz")
    x = torch.from_numpy(z["x"]).to(BF16)
    q, s = O.fp8_quantize(x)
    assert np.array_equal(q.view(torch.uint8).numpy(), z["fp8_bits"]) and np.allclose(s.numpy(), z["fp8_scale"])
    p, bs, ts = O.nvfp4_quantize(x)
    assert np.array_equal(p.numpy(), z["fp4_packed"])
    assert np.array_equal(bs.view(torch.uint8).numpy(), z["fp4_bscale_bits"])
    # dequantised values stay close to the source: e4m3 has 3 mantissa bits, e2m1 one
    assert O.rel_l2(O.fp8_dequantize(q, s), x) < 4e-2
    assert O.rel_l2(O.nvfp4_dequantize(p, bs, ts), x) < 0.15
    # the e2m1 grid is the OCP one
    assert sorted(set(O.e2m1_decode(torch.arange(16, dtype=torch.uint8)).abs().tolist())) == [0, .5, 1, 1.5, 2, 3, 4, 6]


def test_e2m1_rounding_edges():
    x = torch.tensor([0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -5.0])
    got = O.e2m1_decode(O.e2m1_encode(x))
    # ties go to the even code: 0.25->0, 0.75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4, 7 saturates to 6
    assert got.tolist() == [0.0, 0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0, -4.0]


def test_moe_routing_renormalises():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(3, 64, generator=g).to(BF16)
    r = torch.randn(16, 64, generator=g).to(BF16)
    w, idx = O.moe_route(x, r, 4)
    assert idx.shape == (3, 4) and torch.allclose(w.float().sum(-1), torch.ones(3), atol=2e-2)
    assert all(len(set(row.tolist())) == 4 for row in idx)


def test_bytes_per_token_matches_the_published_accounting():
    # Llama-3.1-8B bf16 at 2112 cached positions: 15.287 GB; single layer at 1025: 440.42 MB
    assert abs(O.bytes_per_token(O.LLAMA31_8B, 2112) / 1e9 - 15.287) < 0.01
