"""CPU oracle for the decode hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the decode-step math that the
reference checks its megakernel against.  Only tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it; the
product package never does.

What it follows (paths are inside the reference project):

* the per-module hook points of ``reference_pass``
  (app/python/llama3/reference.py:31-100; app/python/qwen3/reference.py:97-126),
  i.e. Hugging Face ``transformers`` ``LlamaDecoderLayer`` / ``Qwen3DecoderLayer``
  semantics (third-party dependency, version not pinned by the reference; the
  fixtures under tests/golden were produced with transformers 5.5.0);
* half-rotation RoPE and the fp32 softmax of
  app/python/llama3/llama_attention_reference.py:27-125;
* the GQA head grouping of python/dae/model.py:355-375;
* fp32 RMSNorm as app/python/qwen3/reference.py:49-53 and per-head QK norm as
  app/python/qwen3/runtime_context.py:61-73.

Rounding points: every linear layer accumulates in fp32 and rounds its output
to bf16 (module boundary), RMSNorm rounds the normalised value to bf16 before
the bf16 multiply by the weight, the KV cache holds bf16, softmax is fp32 and
its probabilities are rounded to bf16 before the PV product (as the reference
attention helper does).  FP8 / NVFP4 / MoE variants have no counterpart in the
reference: for those this file *is* the specification (parity unpinned by the
reference, pinned only against torch's own float8 / float4 conversions and HF's
Qwen3-MoE block in the golden script).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

BF16 = torch.bfloat16
# When True, bf16 linear layers run through torch's own bf16 kernels (fp32
# accumulation inside the host BLAS) instead of upcasting the weights first.
# Used only where the oracle is *timed* as the CPU baseline.
FAST_LINEAR = False


# --------------------------------------------------------------------------- #
# element-wise pieces
# --------------------------------------------------------------------------- #
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """HF LlamaRMSNorm / Qwen3RMSNorm: fp32 statistics, round, then multiply."""
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xn = (xf * torch.rsqrt(var + eps)).to(x.dtype)
    return weight * xn


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float,
                 dtype=BF16) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of shape [len(positions), head_dim] (half tables duplicated),
    computed in fp32 and rounded to ``dtype`` like build_rope_cache of the
    reference attention helper."""
    freqs = positions.float()[:, None] * rope_inv_freq(head_dim, theta)[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [..., heads, head_dim]; cos/sin broadcastable [..., 1, head_dim]."""
    return (x * cos) + (rotate_half(x) * sin)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x @ w.T with fp32 accumulation, rounded to x.dtype."""
    if FAST_LINEAR and w.dtype == x.dtype:
        return torch.nn.functional.linear(x, w)
    return (x.float() @ w.float().t()).to(x.dtype)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.silu(gate) * up


def gqa_decode_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Single-query grouped attention.

    q: [n_q_heads, d]; k, v: [T, n_kv_heads, d] (the cache including the
    current position).  Returns [n_q_heads * d] in q.dtype.
    """
    n_q, d = q.shape
    n_kv = k.shape[1]
    g = n_q // n_kv
    qf = q.float().view(n_kv, g, d)
    kf = k.float().permute(1, 0, 2)                      # [kv, T, d]
    vf = v.permute(1, 0, 2)                              # [kv, T, d]
    s = torch.matmul(qf, kf.transpose(1, 2)) / math.sqrt(d)   # [kv, g, T]
    p = torch.softmax(s, dim=-1, dtype=torch.float32).to(q.dtype)
    o = torch.matmul(p.float(), vf.float())              # [kv, g, d]
    return o.to(q.dtype).reshape(n_q * d)


# --------------------------------------------------------------------------- #
# quantisation codecs (no counterpart in the reference)
# --------------------------------------------------------------------------- #
FP8_MAX = 448.0
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def fp8_quantize(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel e4m3: scale[out] = max|w[out,:]|/448 (fp32)."""
    wf = w.float()
    scale = wf.abs().amax(dim=1).clamp_min(1e-12) / FP8_MAX
    q = (wf / scale[:, None]).to(torch.float8_e4m3fn)
    return q, scale


def fp8_dequantize(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.float() * scale[:, None]


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest (ties to the even code) onto the e2m1 grid.
    Returns uint8 codes 0..15: bit 3 sign, bits 0..2 index into E2M1_VALUES."""
    a = x.abs().clamp(max=6.0)
    # midpoints between code values; ties go to the code with an even index
    mids = (E2M1_VALUES[1:] + E2M1_VALUES[:-1]) / 2
    idx = torch.zeros_like(a, dtype=torch.int64)
    for i, m in enumerate(mids):
        up_on_tie = (i + 1) % 2 == 0          # moving to an even index on a tie
        idx = idx + ((a > m) | ((a == m) & up_on_tie)).long()
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return (idx | (sign.long() << 3)).to(torch.uint8)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    mag = E2M1_VALUES[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def nvfp4_quantize(w: torch.Tensor):
    """NVFP4: e2m1 values, one e4m3 scale per 16 elements along K, one fp32
    tensor scale.  Returns (packed uint8 [M, K/2] with element 2i in the low
    nibble, block scales float8_e4m3fn [M, K/16], tensor scale fp32 scalar)."""
    wf = w.float()
    M, K = wf.shape
    assert K % 16 == 0
    tscale = (wf.abs().max().clamp_min(1e-12) / (6.0 * FP8_MAX)).float()
    blocks = wf.view(M, K // 16, 16)
    bmax = blocks.abs().amax(dim=-1)
    bscale = (bmax / 6.0 / tscale).to(torch.float8_e4m3fn)
    denom = (bscale.float() * tscale).clamp_min(1e-30)
    codes = e2m1_encode(blocks / denom[..., None]).view(M, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, bscale, tscale


def nvfp4_dequantize(packed: torch.Tensor, bscale: torch.Tensor, tscale: torch.Tensor) -> torch.Tensor:
    M, Kh = packed.shape
    codes = torch.empty(M, Kh * 2, dtype=torch.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    vals = e2m1_decode(codes).view(M, Kh * 2 // 16, 16)
    return (vals * (bscale.float() * tscale)[..., None]).view(M, Kh * 2)


@dataclass
class QLinear:
    """A linear weight in one of the storage formats of the configs."""
    kind: str                                   # "bf16" | "fp8" | "nvfp4"
    w: Optional[torch.Tensor] = None            # bf16 [M, K]
    q: Optional[torch.Tensor] = None            # fp8 [M, K] or packed u8 [M, K/2]
    scale: Optional[torch.Tensor] = None        # fp32 [M] (fp8) / e4m3 [M, K/16] (nvfp4)
    tscale: Optional[torch.Tensor] = None       # fp32 scalar (nvfp4)

    @staticmethod
    def make(w_bf16: torch.Tensor, kind: str) -> "QLinear":
        if kind == "bf16":
            return QLinear("bf16", w=w_bf16)
        if kind == "fp8":
            q, s = fp8_quantize(w_bf16)
            return QLinear("fp8", q=q, scale=s)
        if kind == "nvfp4":
            p, bs, ts = nvfp4_quantize(w_bf16)
            return QLinear("nvfp4", q=p, scale=bs, tscale=ts)
        raise ValueError(kind)

    def dense(self) -> torch.Tensor:
        if self.kind == "bf16":
            return self.w.float()
        if self.kind == "fp8":
            return fp8_dequantize(self.q, self.scale)
        return nvfp4_dequantize(self.q, self.scale, self.tscale)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if FAST_LINEAR and self.kind == "bf16":
            return torch.nn.functional.linear(x, self.w)
        return (x.float() @ self.dense().t()).to(x.dtype)

    def nbytes(self) -> int:
        n = 0
        for t in (self.w, self.q, self.scale):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


# --------------------------------------------------------------------------- #
# model pieces
# --------------------------------------------------------------------------- #
@dataclass
class DecodeConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    n_layers: int = 32
    eps: float = 1e-5
    theta: float = 500000.0
    qk_norm: bool = False            # Qwen3: per-head RMSNorm on q and k
    qk_norm_eps: float = 1e-6
    n_experts: int = 0               # >0: MoE FFN (Qwen3-30B-A3B shape)
    top_k: int = 8
    wkind: str = "bf16"              # storage format of the linear weights

    @property
    def q_width(self):
        return self.n_heads * self.head_dim

    @property
    def kv_width(self):
        return self.n_kv_heads * self.head_dim


LLAMA31_8B = DecodeConfig()
QWEN3_8B = DecodeConfig(ffn=12288, vocab=151936, n_layers=36, eps=1e-6, theta=1e6,
                        qk_norm=True, wkind="nvfp4")
QWEN3_30B_A3B = DecodeConfig(hidden=2048, n_heads=32, n_kv_heads=4, ffn=768, vocab=151936,
                             n_layers=48, eps=1e-6, theta=1e6, qk_norm=True, n_experts=128, top_k=8)


def randn_bf16(gen: torch.Generator, *shape, std: float = 0.02) -> torch.Tensor:
    """Seeded N(0, std) drawn in fp32 on the CPU, then rounded once to bf16."""
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * std).to(BF16)


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    wq: QLinear
    wk: QLinear
    wv: QLinear
    wo: QLinear
    gate: Optional[QLinear] = None
    up: Optional[QLinear] = None
    down: Optional[QLinear] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    router: Optional[torch.Tensor] = None            # [E, hidden] bf16
    experts: List[Tuple[QLinear, QLinear, QLinear]] = field(default_factory=list)

    @staticmethod
    def random(cfg: DecodeConfig, gen: torch.Generator) -> "LayerWeights":
        H, F = cfg.hidden, cfg.ffn
        mk = lambda m, k: QLinear.make(randn_bf16(gen, m, k), cfg.wkind)
        lw = LayerWeights(
            ln1=torch.ones(H, dtype=BF16), ln2=torch.ones(H, dtype=BF16),
            wq=mk(cfg.q_width, H), wk=mk(cfg.kv_width, H), wv=mk(cfg.kv_width, H),
            wo=mk(H, cfg.q_width))
        if cfg.qk_norm:
            lw.q_norm = torch.ones(cfg.head_dim, dtype=BF16)
            lw.k_norm = torch.ones(cfg.head_dim, dtype=BF16)
        if cfg.n_experts:
            lw.router = randn_bf16(gen, cfg.n_experts, H)
            lw.experts = [(mk(F, H), mk(F, H), mk(H, F)) for _ in range(cfg.n_experts)]
        else:
            lw.gate, lw.up, lw.down = mk(F, H), mk(F, H), mk(H, F)
        return lw


def moe_route(x: torch.Tensor, router: torch.Tensor, top_k: int):
    """Qwen3-MoE routing: fp32 softmax over all experts, top-k, renormalise."""
    logits = (x.float() @ router.float().t())
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    w, idx = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w.to(x.dtype), idx


def moe_ffn(x: torch.Tensor, lw: LayerWeights, top_k: int) -> torch.Tensor:
    """x: [hidden].  Σ_e w_e · down_e(silu(gate_e x) · up_e x), summed in fp32
    over the selected experts in ascending slot order and rounded once."""
    w, idx = moe_route(x[None, :], lw.router, top_k)
    acc = torch.zeros(x.shape[0], dtype=torch.float32)
    for slot in range(top_k):
        g, u, d = lw.experts[int(idx[0, slot])]
        y = d(silu_mul(g(x[None, :]), u(x[None, :])))[0]
        acc += y.float() * w[0, slot].float()
    return acc.to(x.dtype)


def decode_layer(cfg: DecodeConfig, lw: LayerWeights, hidden: torch.Tensor, pos: int,
                 k_cache: torch.Tensor, v_cache: torch.Tensor,
                 capture: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
    """One decode step of one layer for a single sequence.

    hidden: [hidden] bf16.  k_cache/v_cache: [T_max, n_kv_heads, head_dim] bf16
    holding rows 0..pos-1; row ``pos`` is written here (K post-RoPE, as HF's
    cache stores it).  Returns the layer output [hidden].  ``capture`` receives
    the same names reference_pass hooks.
    """
    cap = capture if capture is not None else {}
    d = cfg.head_dim
    cap["hidden_state_in"] = hidden
    x = rms_norm(hidden, lw.ln1, cfg.eps)
    cap["input_rms"] = x
    q = lw.wq(x[None])[0]
    k = lw.wk(x[None])[0]
    v = lw.wv(x[None])[0]
    cap["q_proj"], cap["k_proj"], cap["v_proj"] = q, k, v
    qh = q.view(cfg.n_heads, d)
    kh = k.view(cfg.n_kv_heads, d)
    if cfg.qk_norm:
        qh = rms_norm(qh, lw.q_norm, cfg.qk_norm_eps)
        kh = rms_norm(kh, lw.k_norm, cfg.qk_norm_eps)
    cos, sin = rope_cos_sin(torch.tensor([pos]), d, cfg.theta)
    qh = apply_rope(qh, cos, sin)
    kh = apply_rope(kh, cos, sin)
    k_cache[pos] = kh
    v_cache[pos] = v.view(cfg.n_kv_heads, d)
    cap["q_rope"], cap["k_rope"] = qh, kh
    attn = gqa_decode_attention(qh, k_cache[: pos + 1], v_cache[: pos + 1])
    cap["attn_pre_o"] = attn
    o = lw.wo(attn[None])[0]
    cap["o_proj"] = o
    hidden = hidden + o
    cap["post_attn_residual"] = hidden
    x2 = rms_norm(hidden, lw.ln2, cfg.eps)
    cap["post_attn_rms"] = x2
    if cfg.n_experts:
        y = moe_ffn(x2, lw, cfg.top_k)
    else:
        g = lw.gate(x2[None])[0]
        u = lw.up(x2[None])[0]
        cap["gate_proj"], cap["up_proj"] = g, u
        a = silu_mul(g, u)
        cap["silu_mul"] = a
        y = lw.down(a[None])[0]
    cap["down_proj"] = y
    hidden = hidden + y
    cap["hidden_state_out"] = hidden
    return hidden


@dataclass
class ModelWeights:
    cfg: DecodeConfig
    embed: torch.Tensor
    layers: List[LayerWeights]
    norm: torch.Tensor
    lm_head: torch.Tensor

    @staticmethod
    def random(cfg: DecodeConfig, seed: int = 0) -> "ModelWeights":
        gen = torch.Generator().manual_seed(seed)
        embed = randn_bf16(gen, cfg.vocab, cfg.hidden)
        layers = [LayerWeights.random(cfg, gen) for _ in range(cfg.n_layers)]
        lm_head = randn_bf16(gen, cfg.vocab, cfg.hidden)
        return ModelWeights(cfg, embed, layers, torch.ones(cfg.hidden, dtype=BF16), lm_head)


class DecodeOracle:
    """Token-at-a-time causal model with an explicit bf16 KV cache; prefill is
    the same step applied to each prompt position."""

    def __init__(self, weights: ModelWeights, max_seq: int):
        self.w = weights
        cfg = weights.cfg
        self.k = [torch.zeros(max_seq, cfg.n_kv_heads, cfg.head_dim, dtype=BF16) for _ in weights.layers]
        self.v = [torch.zeros(max_seq, cfg.n_kv_heads, cfg.head_dim, dtype=BF16) for _ in weights.layers]
        self.pos = 0

    def step(self, token: int, capture: Optional[List[Dict[str, torch.Tensor]]] = None):
        """Feeds one token at the current position; returns (logits bf16
        [vocab], greedy next token id, top-2 logit gap as float)."""
        cfg = self.w.cfg
        h = self.w.embed[token]
        for i, lw in enumerate(self.w.layers):
            cap = {} if capture is not None else None
            h = decode_layer(cfg, lw, h, self.pos, self.k[i], self.v[i], cap)
            if capture is not None:
                capture.append(cap)
        hn = rms_norm(h, self.w.norm, cfg.eps)
        logits = linear(hn[None], self.w.lm_head)[0]
        self.pos += 1
        top2 = torch.topk(logits.float(), 2).values
        nxt = int(torch.argmax(logits.float()))
        if capture is not None:
            capture.append({"final_hidden": h, "final_rms": hn, "lm_head": logits})
        return logits, nxt, float(top2[0] - top2[1])

    def prefill(self, tokens):
        out = None
        for t in tokens:
            out = self.step(int(t))
        return out


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """‖a−b‖₂ / ‖b‖₂ with b the oracle value."""
    af, bf = a.float().flatten(), b.float().flatten()
    den = float(bf.norm())
    return float((af - bf).norm()) / (den if den > 0 else 1.0)


def bytes_per_token(cfg: DecodeConfig, kv_positions: int) -> int:
    """Algorithmic HBM bytes one batch-1 decode step must read: linear weights
    with their scales, norm weights, lm_head, final norm, one embedding row and
    the KV cache rows of ``kv_positions`` cached positions."""
    per_w = {"bf16": 2.0, "fp8": 1.0, "nvfp4": 0.5 + 1.0 / 16}[cfg.wkind]
    H, F = cfg.hidden, cfg.ffn
    attn_w = (cfg.q_width + 2 * cfg.kv_width) * H + H * cfg.q_width
    lin = attn_w * per_w
    scales = 0
    if cfg.wkind == "fp8":
        scales += 4 * (cfg.q_width + 2 * cfg.kv_width + H)
    if cfg.n_experts:
        lin += cfg.top_k * 3 * F * H * per_w + cfg.n_experts * H * 2
        if cfg.wkind == "fp8":
            scales += cfg.top_k * 4 * (2 * F + H)
    else:
        lin += 3 * F * H * per_w
        if cfg.wkind == "fp8":
            scales += 4 * (2 * F + H)
    norms = 2 * H * 2 + (2 * cfg.head_dim * 2 if cfg.qk_norm else 0)
    layer = lin + scales + norms
    head = cfg.vocab * H * 2 + H * 2 + H * 2
    kv = 2 * cfg.kv_width * 2 * kv_positions * cfg.n_layers
    return int(cfg.n_layers * layer + head + kv)
