"""Generates the golden fixtures in this directory.

Run once, in a container that has the reference tree and Hugging Face
``transformers`` (the reference's own oracle, see
app/python/llama3/reference.py:51-92 of the reference):

    python tests/golden/make_golden.py [--reference-root <path to reference>]

It runs random-init HF models (``LlamaForCausalLM``, ``Qwen3ForCausalLM``,
``Qwen3MoeForCausalLM``) on the CPU in bf16, captures the same module outputs
that ``reference_pass`` hooks, and stores them as small ``.npz`` files together
with the seeds needed to regenerate the inputs.  Where the reference tree is
available its pure-torch attention helper
(app/python/llama3/llama_attention_reference.py) is run on the same q/k/v and
stored as a second witness.  The fixtures travel with the repository; neither
transformers nor the reference is needed to *use* them.
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import decode_oracle as O  # noqa: E402


def cast_params_bf16(model):
    """bf16 parameters, fp32 buffers (rotary inv_freq stays fp32, as it does
    after from_pretrained(dtype=bfloat16) in the reference's scripts)."""
    for p in model.parameters():
        p.data = p.data.to(torch.bfloat16)
    return model.eval()


def hook_layers(model):
    cap = {}
    handles = []

    def post(name):
        def fn(mod, inp, out):
            cap[name] = (out[0] if isinstance(out, tuple) else out).detach()
        return fn

    def pre(name):
        def fn(mod, inp):
            cap[name] = inp[0].detach()
        return fn

    for i, layer in enumerate(model.model.layers):
        handles.append(layer.register_forward_pre_hook(pre(f"{i}.hidden_state_in")))
        handles.append(layer.input_layernorm.register_forward_hook(post(f"{i}.input_rms")))
        handles.append(layer.post_attention_layernorm.register_forward_hook(post(f"{i}.post_attn_rms")))
        at = layer.self_attn
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            handles.append(getattr(at, n).register_forward_hook(post(f"{i}.{n}")))
        mlp = layer.mlp
        for n in ("gate_proj", "up_proj", "down_proj"):
            if hasattr(mlp, n):
                handles.append(getattr(mlp, n).register_forward_hook(post(f"{i}.{n}")))
        handles.append(layer.mlp.register_forward_hook(post(f"{i}.mlp_out")))
        handles.append(layer.register_forward_hook(post(f"{i}.hidden_state_out")))
    handles.append(model.model.norm.register_forward_hook(post("final_rms")))
    handles.append(model.lm_head.register_forward_hook(post("lm_head")))
    return cap, handles


def oracle_weights_from_hf(model, cfg: O.DecodeConfig) -> O.ModelWeights:
    layers = []
    for l in model.model.layers:
        a = l.self_attn
        mk = lambda lin: O.QLinear.make(lin.weight.detach().clone(), "bf16")
        lw = O.LayerWeights(ln1=l.input_layernorm.weight.detach().clone(),
                            ln2=l.post_attention_layernorm.weight.detach().clone(),
                            wq=mk(a.q_proj), wk=mk(a.k_proj), wv=mk(a.v_proj), wo=mk(a.o_proj))
        if cfg.qk_norm:
            lw.q_norm = a.q_norm.weight.detach().clone()
            lw.k_norm = a.k_norm.weight.detach().clone()
        if cfg.n_experts:
            lw.router = l.mlp.gate.weight.detach().clone()
            ex = l.mlp.experts
            gu = ex.gate_up_proj.detach()      # [E, 2F, H]
            dn = ex.down_proj.detach()         # [E, H, F]
            F = cfg.ffn
            for e in range(cfg.n_experts):
                lw.experts.append((O.QLinear.make(gu[e, :F].clone(), "bf16"),
                                   O.QLinear.make(gu[e, F:].clone(), "bf16"),
                                   O.QLinear.make(dn[e].clone(), "bf16")))
        else:
            lw.gate, lw.up, lw.down = mk(l.mlp.gate_proj), mk(l.mlp.up_proj), mk(l.mlp.down_proj)
        layers.append(lw)
    return O.ModelWeights(cfg, model.model.embed_tokens.weight.detach().clone(), layers,
                          model.model.norm.weight.detach().clone(), model.lm_head.weight.detach().clone())


def randomise_norms(model, gen):
    """HF initialises norm weights to 1; perturb them so the affine part is tested."""
    for n, p in model.named_parameters():
        if "norm" in n:
            p.data = (1.0 + 0.1 * torch.randn(p.shape, generator=gen)).to(p.dtype)


def small_model_fixture(kind: str, path: str, ref_attn=None):
    import transformers as T
    torch.manual_seed(1234)
    gen = torch.Generator().manual_seed(99)
    common = dict(hidden_size=256, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2,
                  head_dim=64, vocab_size=512, tie_word_embeddings=False, attention_bias=False)
    if kind == "llama":
        hf_cfg = T.LlamaConfig(intermediate_size=512, rms_norm_eps=1e-5,
                               rope_parameters={"rope_type": "default", "rope_theta": 500000.0}, **common)
        model = T.LlamaForCausalLM(hf_cfg)
        cfg = O.DecodeConfig(hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                             n_layers=3, eps=1e-5, theta=500000.0)
    elif kind == "qwen3":
        hf_cfg = T.Qwen3Config(intermediate_size=512, rms_norm_eps=1e-6,
                               rope_parameters={"rope_type": "default", "rope_theta": 1e6}, **common)
        model = T.Qwen3ForCausalLM(hf_cfg)
        cfg = O.DecodeConfig(hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                             n_layers=3, eps=1e-6, theta=1e6, qk_norm=True)
    elif kind == "qwen3moe":
        hf_cfg = T.Qwen3MoeConfig(intermediate_size=512, moe_intermediate_size=128, num_experts=16,
                                  num_experts_per_tok=4, norm_topk_prob=True, decoder_sparse_step=1,
                                  mlp_only_layers=[], rms_norm_eps=1e-6,
                                  rope_parameters={"rope_type": "default", "rope_theta": 1e6}, **common)
        model = T.Qwen3MoeForCausalLM(hf_cfg)
        cfg = O.DecodeConfig(hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=128, vocab=512,
                             n_layers=3, eps=1e-6, theta=1e6, qk_norm=True, n_experts=16, top_k=4)
    else:
        raise ValueError(kind)
    randomise_norms(model, gen)
    cast_params_bf16(model)
    model.config._attn_implementation = "eager"

    prompt = torch.randint(0, cfg.vocab, (1, 37), generator=gen)
    with torch.no_grad():
        pre = model(input_ids=prompt[:, :-1], use_cache=True)
        cap, handles = hook_layers(model)
        out = model(input_ids=prompt[:, -1:], past_key_values=pre.past_key_values, use_cache=True)
        for h in handles:
            h.remove()
    store = {k: v.float().reshape(-1).numpy() for k, v in cap.items()}
    store["prompt"] = prompt[0].numpy()
    store["logits"] = out.logits[0, -1].float().numpy()
    cache = out.past_key_values
    for i in range(cfg.n_layers):
        store[f"{i}.k_cache"] = cache.layers[i].keys[0].float().numpy()      # [kv, T, d] post-RoPE
        store[f"{i}.v_cache"] = cache.layers[i].values[0].float().numpy()
    # state dict so the test can rebuild the oracle weights without transformers: the model is
    # bf16, so the bit patterns are stored ("wb." keys, uint16), half the size of fp32 and exact
    sd = {"wb." + k: v.detach().to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
          for k, v in model.state_dict().items()}
    np.savez_compressed(path, **store, **sd)

    # self-check: the oracle restatement agrees with HF on this fixture
    w = oracle_weights_from_hf(model, cfg)
    orc = O.DecodeOracle(w, 64)
    orc.prefill(prompt[0, :-1].tolist())
    caps = []
    logits, nxt, gap = orc.step(int(prompt[0, -1]), caps)
    worst = 0.0
    for i in range(cfg.n_layers):
        r = O.rel_l2(caps[i]["hidden_state_out"], cap[f"{i}.hidden_state_out"].reshape(-1))
        worst = max(worst, r)
    rl = O.rel_l2(logits, out.logits[0, -1])
    print(f"[{kind}] oracle vs HF: worst layer rel-L2 {worst:.2e}, logits rel-L2 {rl:.2e}, "
          f"token {nxt} vs {int(out.logits[0, -1].float().argmax())} (gap {gap:.3f})")
    assert worst < 1e-2 and rl < 1e-2

    if ref_attn is not None and kind == "llama":
        # second witness: the reference's own attention helper on layer 0's q/k/v
        # of a fresh 9-token prefill (it has no KV-cache interface).
        with torch.no_grad():
            cap2, handles = hook_layers(model)
            model(input_ids=prompt[:, :9])
            for h in handles:
                h.remove()
        q = cap2["0.q_proj"]
        k = cap2["0.k_proj"]
        v = cap2["0.v_proj"]
        lt = ref_attn.LayerAttentionTensors(
            query_states=q, key_states=k, value_states=v,
            o_proj_weight=model.model.layers[0].self_attn.o_proj.weight, o_proj_bias=None,
            num_heads=8, num_key_value_heads=2, head_dim=64, attention_dropout=0.0, rope_theta=500000.0)
        T_ = 9
        mask = torch.full((T_, T_), float("-inf")).triu(1)[None, None]
        pre_o = ref_attn.attention_reference_pre_o_proj(lt, torch.arange(T_)[None], attention_mask=mask)
        np.savez_compressed(path.replace(".npz", "_refattn.npz"),
                            q=q[0].float().numpy(), k=k[0].float().numpy(), v=v[0].float().numpy(),
                            pre_o=pre_o[0].float().numpy())
        print("[llama] stored the reference attention helper's output for 9 positions")


def full_layer_fixture(path: str):
    """BASELINE config 1: one Llama-3.1-8B-shaped layer, position 1024, seed 0.
    Only the outputs are stored; the inputs are regenerated from the seed."""
    import transformers as T
    from transformers.cache_utils import DynamicCache
    cfg = O.DecodeConfig(n_layers=1, vocab=8)
    gen = torch.Generator().manual_seed(0)
    lw = O.LayerWeights.random(cfg, gen)
    hidden = torch.randn(cfg.hidden, generator=gen).to(torch.bfloat16)
    kc = torch.randn(1024, cfg.n_kv_heads, cfg.head_dim, generator=gen).to(torch.bfloat16)
    vc = torch.randn(1024, cfg.n_kv_heads, cfg.head_dim, generator=gen).to(torch.bfloat16)

    hf_cfg = T.LlamaConfig(hidden_size=4096, intermediate_size=14336, num_hidden_layers=1,
                           num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=8,
                           rms_norm_eps=1e-5, tie_word_embeddings=False,
                           rope_parameters={"rope_type": "default", "rope_theta": 500000.0})
    with torch.device("meta"):
        model = T.LlamaForCausalLM(hf_cfg)
    model = model.to_empty(device="cpu")
    model.model.rotary_emb.inv_freq = O.rope_inv_freq(128, 500000.0)
    model.model.rotary_emb.original_inv_freq = model.model.rotary_emb.inv_freq
    cast_params_bf16(model)
    model.config._attn_implementation = "eager"
    l = model.model.layers[0]
    l.input_layernorm.weight.data = lw.ln1
    l.post_attention_layernorm.weight.data = lw.ln2
    l.self_attn.q_proj.weight.data = lw.wq.w
    l.self_attn.k_proj.weight.data = lw.wk.w
    l.self_attn.v_proj.weight.data = lw.wv.w
    l.self_attn.o_proj.weight.data = lw.wo.w
    l.mlp.gate_proj.weight.data = lw.gate.w
    l.mlp.up_proj.weight.data = lw.up.w
    l.mlp.down_proj.weight.data = lw.down.w
    cache = DynamicCache(config=hf_cfg)
    cache.update(kc.permute(1, 0, 2)[None].clone(), vc.permute(1, 0, 2)[None].clone(), 0)
    pos = torch.tensor([[1024]])
    with torch.no_grad():
        pe = model.model.rotary_emb(hidden[None, None], pos)
        out = l(hidden[None, None], position_embeddings=pe, past_key_values=cache,
                position_ids=pos, attention_mask=None, use_cache=True)
    out = out[0] if isinstance(out, tuple) else out
    k_new = cache.layers[0].keys[0, :, 1024]
    v_new = cache.layers[0].values[0, :, 1024]
    np.savez_compressed(path, hidden_out=out.reshape(-1).float().numpy(),
                        k_new=k_new.float().numpy(), v_new=v_new.float().numpy(),
                        hidden_in_head=hidden[:8].float().numpy(),
                        wq_head=lw.wq.w[0, :8].float().numpy())
    kfull = torch.zeros(1025, 8, 128, dtype=torch.bfloat16)
    vfull = torch.zeros(1025, 8, 128, dtype=torch.bfloat16)
    kfull[:1024], vfull[:1024] = kc, vc
    o = O.decode_layer(cfg, lw, hidden, 1024, kfull, vfull)
    r = O.rel_l2(o, out.reshape(-1))
    print(f"[config1] oracle vs HF LlamaDecoderLayer: rel-L2 {r:.2e}")
    assert r < 1e-2


def codec_fixture(path: str):
    """Quantisation codecs against torch's own float8 / float4 element types."""
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(64, 256, generator=gen) * 0.02
    q, s = O.fp8_quantize(x.to(torch.bfloat16))
    p, bs, ts = O.nvfp4_quantize(x.to(torch.bfloat16))
    store = dict(x=x.numpy(), fp8_bits=q.view(torch.uint8).numpy(), fp8_scale=s.numpy(),
                 fp4_packed=p.numpy(), fp4_bscale_bits=bs.view(torch.uint8).numpy(), fp4_tscale=ts.numpy())
    # e2m1 grid pinned against torch.float4_e2m1fn_x2 where this torch can decode it
    try:
        allcodes = torch.arange(256, dtype=torch.uint8)
        f4 = allcodes.view(torch.float4_e2m1fn_x2)
        lo = O.e2m1_decode(allcodes & 0xF)
        hi = O.e2m1_decode(allcodes >> 4)
        store["e2m1_lo"] = lo.numpy()
        store["e2m1_hi"] = hi.numpy()
        _ = f4  # torch (2.11) has the dtype but no CPU cast; the table is the OCP MX e2m1 grid
    except Exception as e:  # pragma: no cover
        print("float4 dtype unavailable:", e)
    np.savez_compressed(path, **store)
    print("[codec] stored fp8 / nvfp4 encodings of a seeded 64x256 tensor")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=os.environ.get("VDCORES_REFERENCE_ROOT", ""),
                    help="checkout of the reference project (for its pure-torch attention helper); "
                         "default: $VDCORES_REFERENCE_ROOT")
    args = ap.parse_args()
    ref_attn = None
    p = os.path.join(args.reference_root, "app/python/llama3/llama_attention_reference.py")
    if args.reference_root and os.path.exists(p):
        spec = importlib.util.spec_from_file_location("llama_attention_reference", p)
        ref_attn = importlib.util.module_from_spec(spec)
        sys.modules["llama_attention_reference"] = ref_attn
        spec.loader.exec_module(ref_attn)
    torch.set_num_threads(os.cpu_count())
    small_model_fixture("llama", os.path.join(HERE, "llama_small.npz"), ref_attn)
    small_model_fixture("qwen3", os.path.join(HERE, "qwen3_small.npz"))
    small_model_fixture("qwen3moe", os.path.join(HERE, "qwen3moe_small.npz"))
    codec_fixture(os.path.join(HERE, "codecs.npz"))
    full_layer_fixture(os.path.join(HERE, "llama8b_layer_pos1024.npz"))


if __name__ == "__main__":
    main()
