"""Hugging Face checkpoints on disk -> the engines' weight layout.

The reference takes its weights from `AutoModelForCausalLM.from_pretrained` and re-packs them in its model scripts
(app/python/llama3/sched.py:31-38 load, :143-149 RoPE row permutation for its interleaved rotation, :169-170
vocabulary padding).  Here a checkpoint directory (config.json + *.safetensors, sharded or not) is read tensor by
tensor without building the Hugging Face model: `read_config` gives the DecodeConfig, `read_weights` the
DenseWeights that DecodeEngine.load_weights / BatchDecodeEngine.load_weights take.  No row permutation is needed:
the attention task rotates half-split pairs (i, i + 64) exactly like Hugging Face's rotate_half, and the argmax
works on the unpadded vocabulary.  Llama-3 / Qwen3 / Qwen3-MoE naming."""
import json
import os
from typing import Callable, Dict, List

import torch

from .decode import DecodeConfig, DenseWeights


def read_config(path: str) -> DecodeConfig:
    """DecodeConfig from a checkpoint directory's config.json (LlamaConfig / Qwen3Config / Qwen3MoeConfig keys)."""
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    head_dim = c.get("head_dim") or c["hidden_size"] // heads
    moe = int(c.get("num_experts", 0) or 0)
    qk_norm = c.get("model_type", "").startswith("qwen3")
    theta = c.get("rope_theta") or (c.get("rope_parameters") or {}).get("rope_theta", 10000.0)
    kw = dict(n_experts=moe, top_k=int(c["num_experts_per_tok"])) if moe else {}
    return DecodeConfig(hidden=c["hidden_size"], n_heads=heads, n_kv_heads=c.get("num_key_value_heads", heads),
                        head_dim=head_dim, ffn=c["moe_intermediate_size"] if moe else c["intermediate_size"],
                        vocab=c["vocab_size"], n_layers=c["num_hidden_layers"], eps=c.get("rms_norm_eps", 1e-5),
                        theta=float(theta), qk_norm=qk_norm,
                        qk_norm_eps=c.get("rms_norm_eps", 1e-6) if qk_norm else 1e-6, **kw)


def tensor_reader(path: str) -> Callable[[str], torch.Tensor]:
    """get(name) over every *.safetensors file of the directory (model.safetensors.index.json when present)."""
    from safetensors import safe_open
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            where: Dict[str, str] = json.load(f)["weight_map"]
    else:
        where = {}
        for fn in sorted(os.listdir(path)):
            if fn.endswith(".safetensors"):
                with safe_open(os.path.join(path, fn), framework="pt") as f:
                    where.update({k: fn for k in f.keys()})
    if not where:
        raise FileNotFoundError(f"no safetensors tensors under {path}")
    handles = {}

    def get(name: str) -> torch.Tensor:
        if name not in where:
            raise KeyError(f"{name} is not in the checkpoint at {path}")
        fn = where[name]
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), framework="pt")
        return handles[fn].get_tensor(name)

    get.names = set(where)
    return get


def read_weights(path: str, cfg: DecodeConfig = None) -> DenseWeights:
    """DenseWeights (bf16, [out, in]) of a Llama-3 / Qwen3 / Qwen3-MoE checkpoint directory."""
    cfg = cfg or read_config(path)
    get = tensor_reader(path)
    bf = lambda name: get(name).to(torch.bfloat16)
    L = range(cfg.n_layers)
    lay = lambda l, s: f"model.layers.{l}.{s}.weight"
    # tied embeddings: the vocabulary projection is the embedding table
    lm_head = bf("lm_head.weight") if "lm_head.weight" in get.names else bf("model.embed_tokens.weight")
    if cfg.n_experts:
        E = range(cfg.n_experts)
        exp = lambda l, s: [bf(f"model.layers.{l}.mlp.experts.{e}.{s}.weight") for e in E]
        gate, up, down = ([exp(l, s) for l in L] for s in ("gate_proj", "up_proj", "down_proj"))
        router: List[torch.Tensor] = [bf(lay(l, "mlp.gate")) for l in L]
    else:
        gate, up, down = ([bf(lay(l, f"mlp.{s}")) for l in L] for s in ("gate_proj", "up_proj", "down_proj"))
        router = None
    return DenseWeights(
        embed=bf("model.embed_tokens.weight"), lm_head=lm_head, norm=bf("model.norm.weight"),
        ln1=[bf(lay(l, "input_layernorm")) for l in L], ln2=[bf(lay(l, "post_attention_layernorm")) for l in L],
        wq=[bf(lay(l, "self_attn.q_proj")) for l in L], wk=[bf(lay(l, "self_attn.k_proj")) for l in L],
        wv=[bf(lay(l, "self_attn.v_proj")) for l in L], wo=[bf(lay(l, "self_attn.o_proj")) for l in L],
        gate=gate, up=up, down=down,
        q_norm=[bf(lay(l, "self_attn.q_norm")) for l in L] if cfg.qk_norm else None,
        k_norm=[bf(lay(l, "self_attn.k_norm")) for l in L] if cfg.qk_norm else None,
        router=router)
