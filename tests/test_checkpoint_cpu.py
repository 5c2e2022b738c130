"""Checkpoint directories (config.json + safetensors, sharded or not) -> DecodeConfig / DenseWeights, against the
files Hugging Face's own writer produces for tiny random models."""
import json
import os

import pytest
import torch

from vdcores_b200 import checkpoint


def _write_sharded(tmp, state, n_shards=2):
    from safetensors.torch import save_file
    names = sorted(state)
    weight_map = {}
    for i in range(n_shards):
        part = {k: state[k].contiguous() for k in names[i::n_shards]}
        fn = f"model-{i + 1:05d}-of-{n_shards:05d}.safetensors"
        save_file(part, os.path.join(tmp, fn))
        weight_map.update({k: fn for k in part})
    with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)


def test_llama_directory_written_by_transformers(tmp_path):
    tr = pytest.importorskip("transformers")
    cfg = tr.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
                         num_key_value_heads=1, head_dim=128, vocab_size=320, rms_norm_eps=1e-5, rope_theta=500000.0,
                         tie_word_embeddings=False)
    torch.manual_seed(0)
    model = tr.LlamaForCausalLM(cfg).to(torch.bfloat16)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    c = checkpoint.read_config(str(tmp_path))
    assert (c.hidden, c.n_heads, c.n_kv_heads, c.head_dim, c.ffn, c.vocab, c.n_layers) == (256, 2, 1, 128, 512, 320, 2)
    assert c.eps == 1e-5 and c.theta == 500000.0 and not c.qk_norm and c.n_experts == 0
    w = checkpoint.read_weights(str(tmp_path))
    sd = model.state_dict()
    assert torch.equal(w.embed, sd["model.embed_tokens.weight"]) and torch.equal(w.lm_head, sd["lm_head.weight"])
    assert torch.equal(w.norm, sd["model.norm.weight"])
    for l in range(2):
        p = f"model.layers.{l}."
        for mine, theirs in ((w.wq, "self_attn.q_proj"), (w.wk, "self_attn.k_proj"), (w.wv, "self_attn.v_proj"),
                             (w.wo, "self_attn.o_proj"), (w.gate, "mlp.gate_proj"), (w.up, "mlp.up_proj"),
                             (w.down, "mlp.down_proj"), (w.ln1, "input_layernorm"), (w.ln2, "post_attention_layernorm")):
            assert torch.equal(mine[l], sd[p + theirs + ".weight"]), theirs
    assert w.q_norm is None and w.router is None


def test_sharded_qwen3_moe_names_and_tied_embeddings(tmp_path):
    g = torch.Generator().manual_seed(1)
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
    H, F, E, V, L = 256, 128, 4, 96, 2
    state = {"model.embed_tokens.weight": r(V, H), "model.norm.weight": r(H)}
    for l in range(L):
        p = f"model.layers.{l}."
        state.update({p + "input_layernorm.weight": r(H), p + "post_attention_layernorm.weight": r(H),
                      p + "self_attn.q_proj.weight": r(256, H), p + "self_attn.k_proj.weight": r(128, H),
                      p + "self_attn.v_proj.weight": r(128, H), p + "self_attn.o_proj.weight": r(H, 256),
                      p + "self_attn.q_norm.weight": r(128), p + "self_attn.k_norm.weight": r(128),
                      p + "mlp.gate.weight": r(E, H)})
        for e in range(E):
            q = p + f"mlp.experts.{e}."
            state.update({q + "gate_proj.weight": r(F, H), q + "up_proj.weight": r(F, H), q + "down_proj.weight": r(H, F)})
    _write_sharded(str(tmp_path), state)
    with open(os.path.join(str(tmp_path), "config.json"), "w") as f:
        json.dump({"model_type": "qwen3_moe", "hidden_size": H, "num_attention_heads": 2, "num_key_value_heads": 1,
                   "head_dim": 128, "intermediate_size": 999, "moe_intermediate_size": F, "num_experts": E,
                   "num_experts_per_tok": 2, "vocab_size": V, "num_hidden_layers": L, "rms_norm_eps": 1e-6,
                   "rope_theta": 1000000.0, "tie_word_embeddings": True}, f)
    c = checkpoint.read_config(str(tmp_path))
    assert c.qk_norm and c.n_experts == E and c.top_k == 2 and c.ffn == F and c.theta == 1e6
    w = checkpoint.read_weights(str(tmp_path), c)
    assert torch.equal(w.lm_head, state["model.embed_tokens.weight"])          # tied: no lm_head tensor on disk
    assert torch.equal(w.router[1], state["model.layers.1.mlp.gate.weight"])
    assert torch.equal(w.down[1][3], state["model.layers.1.mlp.experts.3.down_proj.weight"])
    assert torch.equal(w.k_norm[0], state["model.layers.0.self_attn.k_norm.weight"])
    with pytest.raises(KeyError, match="not in the checkpoint"):
        checkpoint.tensor_reader(str(tmp_path))("model.layers.9.mlp.gate.weight")
