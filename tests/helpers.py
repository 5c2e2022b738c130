"""Shared helpers for the tests: conversions between the oracle's weight
containers and the engine's, and small model configurations."""
import torch

from oracle import decode_oracle as O


def small_cfg(kind: str) -> O.DecodeConfig:
    if kind == "llama":
        return O.DecodeConfig(hidden=512, n_heads=8, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
                              n_layers=3, eps=1e-5, theta=500000.0)
    if kind == "qwen3":
        return O.DecodeConfig(hidden=512, n_heads=8, n_kv_heads=1, head_dim=128, ffn=768, vocab=1024,
                              n_layers=2, eps=1e-6, theta=1e6, qk_norm=True)
    if kind == "moe":           # Qwen3-MoE style: QK norm, group of 8, 16 experts of width 256, top-4
        return O.DecodeConfig(hidden=512, n_heads=8, n_kv_heads=1, head_dim=128, ffn=256, vocab=1024,
                              n_layers=2, eps=1e-6, theta=1e6, qk_norm=True, n_experts=16, top_k=4)
    if kind == "moe2":          # the same with two KV heads, so that attention can be split over two ranks
        return O.DecodeConfig(hidden=512, n_heads=8, n_kv_heads=2, head_dim=128, ffn=256, vocab=1024,
                              n_layers=2, eps=1e-6, theta=1e6, qk_norm=True, n_experts=16, top_k=4)
    if kind == "qwen3_1k":      # K multiples of 1024, as the NVFP4 rows need
        return O.DecodeConfig(hidden=1024, n_heads=8, n_kv_heads=1, head_dim=128, ffn=1024, vocab=1024,
                              n_layers=2, eps=1e-6, theta=1e6, qk_norm=True)
    raise ValueError(kind)


def perturb_norms(w: O.ModelWeights, seed: int = 7):
    """Norm weights are 1 at init; move them so the affine part is exercised."""
    g = torch.Generator().manual_seed(seed)
    r = lambda t: (1.0 + 0.1 * torch.randn(t.shape, generator=g)).to(t.dtype)
    w.norm = r(w.norm)
    for lw in w.layers:
        if lw.router is not None:       # N(0, 0.02) router logits are nearly flat: spread them out
            lw.router = (lw.router.float() * 40).to(lw.router.dtype)
        lw.ln1, lw.ln2 = r(lw.ln1), r(lw.ln2)
        if lw.q_norm is not None:
            lw.q_norm, lw.k_norm = r(lw.q_norm), r(lw.k_norm)
    return w


def engine_config(cfg: O.DecodeConfig):
    from vdcores_b200.decode import DecodeConfig
    return DecodeConfig(hidden=cfg.hidden, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                        ffn=cfg.ffn, vocab=cfg.vocab, n_layers=cfg.n_layers, eps=cfg.eps, theta=cfg.theta,
                        qk_norm=cfg.qk_norm, qk_norm_eps=cfg.qk_norm_eps, n_experts=cfg.n_experts, top_k=cfg.top_k)


def dense_weights(w: O.ModelWeights):
    from vdcores_b200.decode import DenseWeights
    L = w.layers
    if w.cfg.n_experts:
        return DenseWeights(
            embed=w.embed, lm_head=w.lm_head, norm=w.norm,
            ln1=[l.ln1 for l in L], ln2=[l.ln2 for l in L],
            wq=[l.wq.w for l in L], wk=[l.wk.w for l in L], wv=[l.wv.w for l in L], wo=[l.wo.w for l in L],
            gate=[[e[0].w for e in l.experts] for l in L], up=[[e[1].w for e in l.experts] for l in L],
            down=[[e[2].w for e in l.experts] for l in L], router=[l.router for l in L],
            q_norm=[l.q_norm for l in L] if w.cfg.qk_norm else None,
            k_norm=[l.k_norm for l in L] if w.cfg.qk_norm else None)
    return DenseWeights(
        embed=w.embed, lm_head=w.lm_head, norm=w.norm,
        ln1=[l.ln1 for l in L], ln2=[l.ln2 for l in L],
        wq=[l.wq.w for l in L], wk=[l.wk.w for l in L], wv=[l.wv.w for l in L], wo=[l.wo.w for l in L],
        gate=[l.gate.w for l in L], up=[l.up.w for l in L], down=[l.down.w for l in L],
        q_norm=[l.q_norm for l in L] if w.cfg.qk_norm else None,
        k_norm=[l.k_norm for l in L] if w.cfg.qk_norm else None)
