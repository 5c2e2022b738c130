"""Batch-1 decode engine: packs a Llama / Qwen3 style model for the megakernel,
builds the per-SM instruction program once, and runs one kernel launch per
generated token.

The program plays the role of the reference's model schedule scripts
(reference app/python/llama3/sched.py:255-571, app/python/qwen3/sched.py): the
same stages — fused-norm QKV projection, GQA decode attention, output
projection with residual add, fused-norm gate/up with SiLU·mul, down projection
with residual add, final norm + vocabulary projection + argmax — cross-SM
ordering through countdown barriers, weights prefetched ahead of the
activations they wait for.  Unlike the reference it is laid out for all SMs of
a B200, a paged KV cache, and position-independent instruction streams (the
position comes from a small state block in device memory), so one program
serves every step.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from . import isa, runtime
from .program import Dst, Program, Src

BF16 = torch.bfloat16


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
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    n_experts: int = 0          # > 0: every layer's FFN is a top-k mixture of experts of width `ffn`
    top_k: int = 8

    @property
    def q_width(self):
        return self.n_heads * self.head_dim

    @property
    def kv_width(self):
        return self.n_kv_heads * self.head_dim

    @property
    def group(self):
        return self.n_heads // self.n_kv_heads


LLAMA31_8B = DecodeConfig()
QWEN3_8B = DecodeConfig(ffn=12288, vocab=151936, n_layers=36, eps=1e-6, theta=1e6, qk_norm=True)
QWEN3_30B_A3B = DecodeConfig(hidden=2048, n_heads=32, n_kv_heads=4, ffn=768, vocab=151936, n_layers=48, eps=1e-6,
                             theta=1e6, qk_norm=True, n_experts=128, top_k=8)


@dataclass
class DenseWeights:
    """Unpacked bf16 weights, one entry per layer, in the usual [out, in] layout."""
    embed: torch.Tensor
    lm_head: torch.Tensor
    norm: torch.Tensor
    ln1: List[torch.Tensor]
    ln2: List[torch.Tensor]
    wq: List[torch.Tensor]
    wk: List[torch.Tensor]
    wv: List[torch.Tensor]
    wo: List[torch.Tensor]
    gate: List[torch.Tensor]
    up: List[torch.Tensor]
    down: List[torch.Tensor]
    q_norm: Optional[List[torch.Tensor]] = None
    k_norm: Optional[List[torch.Tensor]] = None
    # mixture of experts (gate/up/down then hold, per layer, a list with one matrix per expert)
    router: Optional[List[torch.Tensor]] = None


def kv_page_swizzle(pages: torch.Tensor) -> torch.Tensor:
    """Piece order of KV page rows in HBM.  `pages` is [..., 64 rows, 128] bf16; every 256-byte row is stored
    with its sixteen 16-byte pieces at index (piece XOR (row mod 8)).  A page reaches shared memory as one
    linear copy, and with this order the eight row addresses of an `ldmatrix` (same piece, eight consecutive
    rows) fall into eight different banks.  The map is its own inverse: it converts both ways."""
    assert pages.shape[-2] == isa.KV_PAGE and pages.shape[-1] == isa.HEAD_DIM
    rows = torch.arange(isa.KV_PAGE, device=pages.device)
    idx = torch.arange(isa.HEAD_DIM // 8, device=pages.device)[None, :] ^ (rows[:, None] & 7)      # [64, 16]
    v = pages.reshape(*pages.shape[:-1], isa.HEAD_DIM // 8, 8)
    return v[..., rows[:, None], idx, :].reshape(pages.shape)


def rows_per_chunk(K: int, even: bool = False, row_bytes: Optional[int] = None) -> int:
    """Largest power-of-two row count whose rows (bf16 unless row_bytes is given) fit one 32 KB bulk copy."""
    row_bytes = 2 * K if row_bytes is None else row_bytes
    r = 16
    while r > 1 and r * row_bytes > 32768:
        r //= 2
    if r * row_bytes > 32768 or (even and r < 2):
        raise ValueError(f"K={K} rows do not fit the 32 KB chunk limit")
    return r


FP8_MAX = 448.0


def quantize_fp8_rows(w: torch.Tensor):
    """Per-output-channel e4m3: scale[row] = max|w[row]| / 448 (fp32), q = e4m3(w / scale).
    Works on [..., rows, K]; returns (uint8 view of the codes, fp32 scales)."""
    wf = w.float()
    scale = wf.abs().amax(dim=-1).clamp_min(1e-12) / FP8_MAX
    q = (wf / scale[..., None]).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), scale.contiguous()


_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def quantize_nvfp4_rows(w: torch.Tensor):
    """NVFP4 of one [M, K] matrix: e2m1 values (round to nearest, ties to the even
    code), one e4m3 scale per 16 weights along K, one fp32 scale for the tensor.
    Returns (uint8 rows [M, K/2 + K/16]: packed pairs with element 2i in the low
    nibble, then the block scales; fp32 tensor scale)."""
    wf = w.float()
    M, K = wf.shape
    assert K % 16 == 0
    grid = torch.tensor(_E2M1, device=wf.device)
    tscale = (wf.abs().max().clamp_min(1e-12) / (6.0 * FP8_MAX)).float()
    blocks = wf.view(M, K // 16, 16)
    bscale = (blocks.abs().amax(dim=-1) / 6.0 / tscale).to(torch.float8_e4m3fn)
    v = blocks / (bscale.float() * tscale).clamp_min(1e-30)[..., None]
    a = v.abs().clamp(max=6.0)
    mids = (grid[1:] + grid[:-1]) / 2
    idx = torch.zeros_like(a, dtype=torch.int64)
    for i in range(7):
        idx += ((a > mids[i]) | ((a == mids[i]) & ((i + 1) % 2 == 0))).long()
    sign = (v < 0) | ((v == 0) & torch.signbit(v))
    codes = (idx | (sign.long() << 3)).to(torch.uint8).view(M, K)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    rows = torch.cat((packed, bscale.view(torch.uint8)), dim=1).contiguous()
    return rows, tscale


class DecodeEngine:
    GEMV_PROJECTIONS = True     # the layer projections run as GEMV tasks (batch 1)
    FULL_KERNEL = False         # batch 1 launches the kernel with the native batch-1 operators only

    def __init__(self, cfg: DecodeConfig, max_seq: int, device="cuda", num_sms: Optional[int] = None,
                 taps: bool = False, page_perm_seed: Optional[int] = None, max_steps: int = 4096,
                 timeout_ns: int = 0, l2_prefetch_bytes: int = 0, wkind: str = "bf16", shared_counters: bool = False,
                 split_down: bool = False, interleave: bool = True):
        assert cfg.head_dim == isa.HEAD_DIM, "the attention task is built for head_dim 128"
        assert cfg.group in (4, 8), "GQA group size must be 4 or 8"
        assert cfg.n_kv_heads & (cfg.n_kv_heads - 1) == 0, "n_kv_heads must be a power of two"
        assert cfg.hidden % 256 == 0 and cfg.ffn % 256 == 0 and cfg.q_width % 256 == 0
        assert wkind in ("bf16", "fp8", "nvfp4")
        self.cfg = cfg
        self.wkind = wkind                  # storage of the layer projections; embed / norms / lm_head stay bf16
        # the GEMV task walks K in warp steps of 256 / 512 / 1024 weights; the batched tensor-core path (a subclass)
        # needs multiples of 16 only
        kmult = {"bf16": 256, "fp8": 512, "nvfp4": 1024}[wkind] if self.GEMV_PROJECTIONS else 256
        assert cfg.hidden % kmult == 0 and cfg.ffn % kmult == 0 and cfg.q_width % kmult == 0
        self.dev = torch.device(device)
        props = torch.cuda.get_device_properties(self.dev)
        self.num_sms = num_sms or props.multi_processor_count
        self.max_seq = max_seq
        self.max_pages = (max_seq + isa.KV_PAGE - 1) // isa.KV_PAGE
        self.taps_enabled = taps
        self.max_steps = max_steps
        self.timeout_ns = timeout_ns
        self.l2_prefetch_bytes = l2_prefetch_bytes     # per SM; 0 disables the L2 prefetch
        # gate/up and down as two half-stages each (see _build_program).  Measured on B200, Llama-3.1-8B shape:
        # 270 tokens/s against 288 without (FP8 318 / 357, NVFP4 342 / 355): the two extra tasks per layer (activation
        # copy + norm, phase begin / end, fences: 4-5 us each) cost more than the idle time at the boundary they remove
        self.split_down_wanted = split_down
        # deal a stage's chunks round-robin to the SMs (chunk j to SM j mod 148, continuing from stage to stage) instead
        # of one contiguous range each: all SMs then walk the same window of a matrix together.  Measured on B200,
        # Llama-3.1-8B shape: 290.4 against 287.7 tokens/s
        self.interleave = interleave
        # dense projections: every SM owns most of its chunks and the SMs draw the tail of each stage from a counter
        # they share.  Off by default: measured on B200 (Llama-3.1-8B shape) it narrows the spread of the SMs' finishing
        # times (3.5 -> 2.8 us per stage) but the draws thin out the copies in flight and the step gets slower
        # (3.79 -> 4.10 ms; 3.99 ms when every chunk is drawn).
        self.shared_counters = shared_counters
        self.tail_fraction = 0.2        # share of a stage's chunks that is not owned by an SM beforehand
        self.shared_depth = 6           # ring entries an SM may hold when it draws a chunk from the tail
        self.stream = torch.cuda.current_stream(self.dev)
        runtime.init()

        L, H, F, V = cfg.n_layers, cfg.hidden, cfg.ffn, cfg.vocab
        z = lambda *s, dt=BF16: torch.zeros(*s, dtype=dt, device=self.dev)
        self.qkv_rows = cfg.q_width + 2 * cfg.kv_width
        self.hidden = z(H)
        self.qkv = z(self.qkv_rows)
        self.attn_out = z(cfg.q_width)
        self.act = z(max(1, cfg.top_k if cfg.n_experts else 1), F)
        self.logits = z(V)
        if cfg.n_experts:
            assert wkind == "bf16", "expert weights are bf16 only"
            self.router_logits = z(cfg.n_experts, dt=torch.float32)
            self.route = z(64, dt=torch.int32)          # int32 ids[16] | fp32 weights[16] | int32 local[16] | int32 count[16]
            self.moe_acc = z(H, dt=torch.float32)       # zero between layers: the last expert to arrive clears it
            self.moe_cnt = z(H, dt=torch.int32)
        G = cfg.group
        self.rec_floats = G * isa.HEAD_DIM + 16 * ((2 * G + 15) // 16)
        max_rec_per_load = 32768 // (self.rec_floats * 4)
        self.n_splits = max(1, min(self.num_sms // cfg.n_kv_heads, self.max_pages))
        self.pages_per_split = max((self.max_pages + self.n_splits - 1) // self.n_splits, int(os.environ.get("VDC_PPS", "1")))
        self.n_splits = (self.max_pages + self.pages_per_split - 1) // self.pages_per_split
        self.max_rec_per_load = max_rec_per_load
        self.attn_part = z(cfg.n_kv_heads, self.n_splits, self.rec_floats, dt=torch.float32)
        self.attn_cnt = z(L, cfg.n_kv_heads, dt=torch.int32)     # arrival counters, zero between steps
        # projection rows are stored per KV head group: [G query heads | key | value] x 128
        D_ = isa.HEAD_DIM
        perm = []
        for h in range(cfg.n_kv_heads):
            perm += list(range(h * G * D_, (h + 1) * G * D_))
            perm += list(range(cfg.q_width + h * D_, cfg.q_width + (h + 1) * D_))
            perm += list(range(cfg.q_width + cfg.kv_width + h * D_, cfg.q_width + cfg.kv_width + (h + 1) * D_))
        self.qkv_perm = torch.tensor(perm, dtype=torch.long)            # packed row -> standard row
        self.qkv_inv = torch.empty_like(self.qkv_perm)
        self.qkv_inv[self.qkv_perm] = torch.arange(len(perm))           # standard row -> packed row
        self.argmax_rec = z(self.num_sms, 4, dt=torch.float32)
        self.state = z(isa.ST_PAGETABLE + self.max_pages, dt=torch.int32)
        self.state_host = torch.zeros(isa.ST_PAGETABLE + self.max_pages, dtype=torch.int32).pin_memory()
        self.token_log = z(max_steps, dt=torch.int32)
        self.kpool = z(L, self.max_pages, cfg.n_kv_heads, isa.KV_PAGE, isa.HEAD_DIM)
        self.vpool = z(L, self.max_pages, cfg.n_kv_heads, isa.KV_PAGE, isa.HEAD_DIM)
        self.taps = z(L, H) if taps else None
        if page_perm_seed is None:
            self.page_table = torch.arange(self.max_pages, dtype=torch.int32)
        else:
            g = torch.Generator().manual_seed(page_perm_seed)
            self.page_table = torch.randperm(self.max_pages, generator=g).to(torch.int32)
        # rope table: cos[64] | sin[64] per position, values rounded to bf16 like HF's tables, kept as fp32
        pos = torch.arange(max_seq, dtype=torch.float32)
        inv = 1.0 / (cfg.theta ** (torch.arange(0, isa.HEAD_DIM, 2, dtype=torch.float32) / isa.HEAD_DIM))
        fr = pos[:, None] * inv[None, :]
        self.rope = torch.cat((fr.cos().to(BF16).float(), fr.sin().to(BF16).float()), dim=1).contiguous().to(self.dev)
        self.bars = z(isa.MAX_BARS, dt=torch.int32)
        self.profile = z(self.num_sms * isa.NUM_PROFILE_EVENTS, dt=torch.int64)
        self.w = None
        self.program = None
        self.pos = 0
        self.steps_done = 0

    # ------------------------------------------------------------------ weights
    def row_bytes(self, K: int) -> int:
        """Bytes one weight row of K inputs occupies in the layer projections' storage."""
        return {"bf16": 2 * K, "fp8": K, "nvfp4": K // 2 + K // 16}[self.wkind]

    def _encode(self, w: torch.Tensor):
        """One [M, K] bf16 matrix -> (stored rows, fp32 per-row scale or None), on w's device."""
        if self.wkind == "bf16":
            return w, None
        if self.wkind == "fp8":
            return quantize_fp8_rows(w)
        rows, ts = quantize_nvfp4_rows(w)
        return rows, ts.expand(w.shape[0]).contiguous()

    def _dense(self, name: str, l: int) -> torch.Tensor:
        """Layer l's projection as a bf16 matrix (PyTorch prefill path)."""
        w = getattr(self, name)[l]
        if self.wkind == "fp8":
            return (w.view(torch.float8_e4m3fn).float() * self.scales[name][l][:, None]).to(BF16)
        if self.wkind == "nvfp4":
            K = w.shape[1] * 16 // 9
            codes = w[:, :K // 2]
            grid = torch.tensor(_E2M1 + [-x for x in _E2M1], device=w.device)
            vals = torch.stack((grid[(codes & 0xF).long()], grid[(codes >> 4).long()]), dim=-1).view(w.shape[0], K)
            bs = w[:, K // 2:].contiguous().view(torch.float8_e4m3fn).float()
            return (vals.view(w.shape[0], K // 16, 16) * (bs * self.scales[name][l][:, None])[..., None]
                    ).view(w.shape[0], K).to(BF16)
        return w

    def load_weights(self, w: DenseWeights):
        """Encodes (bf16 / fp8 / NVFP4, each source matrix on its own, like the
        oracle) and packs on the device the weights arrive on, then moves the result
        to the GPU: CPU weights give the exact CPU conversions (torch's fp8 cast is
        not bit-identical between CPU and CUDA)."""
        cfg, dev = self.cfg, self.dev
        L = cfg.n_layers
        to = lambda t: t.to(dtype=BF16).contiguous()
        pm = self.qkv_perm.to(w.wq[0].device)
        cat = lambda parts: (torch.cat([p[0] for p in parts], 0),
                             None if parts[0][1] is None else torch.cat([p[1] for p in parts], 0))
        packed = {"wqkv": [], "wo": [], "wgu": [], "wd": []}
        for l in range(L):
            rows, sc = cat([self._encode(to(w.wq[l])), self._encode(to(w.wk[l])), self._encode(to(w.wv[l]))])
            packed["wqkv"].append((rows[pm], None if sc is None else sc[pm]))
            packed["wo"].append(self._encode(to(w.wo[l])))
            if cfg.n_experts:
                # [E, 2F, H] with gate/up interleaved per expert, [E, H, F]
                packed["wgu"].append((torch.stack([torch.stack((to(g), to(u)), dim=1).reshape(2 * cfg.ffn, cfg.hidden)
                                                   for g, u in zip(w.gate[l], w.up[l])]), None))
                packed["wd"].append((torch.stack([to(d) for d in w.down[l]]), None))
                continue
            # gate and up rows interleaved: row 2j = gate_j, row 2j+1 = up_j
            (g, gs), (u, us) = self._encode(to(w.gate[l])), self._encode(to(w.up[l]))
            packed["wgu"].append((torch.stack((g, u), dim=1).reshape(2 * cfg.ffn, g.shape[1]),
                                  None if gs is None else torch.stack((gs, us), dim=1).reshape(-1)))
            packed["wd"].append(self._encode(to(w.down[l])))
        self.scales = {}
        for name, parts in packed.items():
            setattr(self, name, torch.stack([p[0] for p in parts]).to(dev))
            if parts[0][1] is not None:
                self.scales[name] = torch.stack([p[1] for p in parts]).to(dev)
        self.router = torch.stack([to(t) for t in w.router]).to(dev) if cfg.n_experts else None
        self.embed = to(w.embed).to(dev)
        self.lm_head = to(w.lm_head).to(dev)
        self.norm_w = to(w.norm).to(dev)
        self.ln1 = torch.stack([to(t) for t in w.ln1]).to(dev)
        self.ln2 = torch.stack([to(t) for t in w.ln2]).to(dev)
        if cfg.qk_norm:
            self.qknorm = torch.stack([torch.cat((to(w.q_norm[l]), to(w.k_norm[l]))) for l in range(L)]).to(dev)
        else:
            self.qknorm = None
        self.w = True
        self._build_program()

    def _quantize(self):
        """Random-weight path: replaces the packed bf16 projections by their stored form."""
        self.scales = {}
        if self.wkind == "bf16":
            return
        for name in ("wqkv", "wo", "wgu", "wd"):
            w = getattr(self, name)
            parts = [self._encode(w[l]) for l in range(w.shape[0])]
            setattr(self, name, torch.stack([p[0] for p in parts]))
            self.scales[name] = torch.stack([p[1] for p in parts])
            del w

    def init_random_weights(self, seed: int = 0, std: float = 0.02):
        """Random N(0, std) weights generated on the device (benchmarks)."""
        cfg, dev = self.cfg, self.dev
        g = torch.Generator(device=dev).manual_seed(seed)
        L, H, F, V = cfg.n_layers, cfg.hidden, cfg.ffn, cfg.vocab

        def rnd(*shape):
            t = torch.empty(*shape, dtype=BF16, device=dev)
            t.normal_(0.0, std, generator=g)
            return t
        self.embed = rnd(V, H)
        self.lm_head = rnd(V, H)
        self.norm_w = torch.ones(H, dtype=BF16, device=dev)
        self.ln1 = torch.ones(L, H, dtype=BF16, device=dev)
        self.ln2 = torch.ones(L, H, dtype=BF16, device=dev)
        self.wqkv = rnd(L, self.qkv_rows, H)
        self.wo = rnd(L, H, cfg.q_width)
        if cfg.n_experts:
            self.wgu = rnd(L, cfg.n_experts, 2 * F, H)
            self.wd = rnd(L, cfg.n_experts, H, F)
            self.router = rnd(L, cfg.n_experts, H)
        else:
            self.wgu = rnd(L, 2 * F, H)
            self.wd = rnd(L, H, F)
            self.router = None
        self.qknorm = torch.ones(L, 2 * isa.HEAD_DIM, dtype=BF16, device=dev) if cfg.qk_norm else None
        self.w = True
        self._quantize()
        self._build_program()

    def weight_bytes(self) -> int:
        ts = [self.lm_head, self.norm_w, self.ln1, self.ln2, self.wqkv, self.wo]
        ts += list(self.scales.values())
        if self.qknorm is not None:
            ts.append(self.qknorm)
        n = sum(t.numel() * t.element_size() for t in ts) + self.cfg.hidden * 2
        if self.cfg.n_experts:      # a token reads the router and top_k of the experts of every layer
            n += self.router.numel() * 2
            n += (self.wgu.numel() + self.wd.numel()) * 2 * self.cfg.top_k // self.cfg.n_experts
        else:
            n += sum(t.numel() * t.element_size() for t in (self.wgu, self.wd))
        return n

    def algorithmic_bytes(self, pos: int) -> int:
        """HBM bytes one decode step at position `pos` has to read: every weight
        once, one embedding row, and the KV rows of pos+1 positions."""
        cfg = self.cfg
        return self.weight_bytes() + 2 * cfg.kv_width * 2 * (pos + 1) * cfg.n_layers

    # ------------------------------------------------------------------ program
    def _ranges(self, load, n_units: int, unit_bytes: int):
        """Splits n_units into one contiguous range per SM; the SMs that carry
        the fewest bytes so far take the larger share."""
        S = self.num_sms
        base, rem = divmod(n_units, S)
        order = sorted(range(S), key=lambda s: (load[s], s))
        extra = set(order[:rem])
        out, u = [], 0
        for sm in range(S):
            cnt = base + (1 if sm in extra else 0)
            if cnt:
                out.append((sm, u, cnt))
                load[sm] += cnt * unit_bytes
            u += cnt
        assert u == n_units
        return out

    def _halve_k(self, w: torch.Tensor, K: int):
        """The stored rows of [L, M, K] weights as two tensors over the K-halves (each contiguous, rows in the
        engine's storage format: for NVFP4 the half's code bytes followed by the half's block scales)."""
        if self.wkind == "bf16":
            return w[:, :, :K // 2].contiguous(), w[:, :, K // 2:].contiguous()
        if self.wkind == "fp8":
            return w[:, :, :K // 2].contiguous(), w[:, :, K // 2:].contiguous()
        codes, bs = w[:, :, :K // 2], w[:, :, K // 2:]
        return (torch.cat((codes[:, :, :K // 4], bs[:, :, :K // 32]), dim=2).contiguous(),
                torch.cat((codes[:, :, K // 4:], bs[:, :, K // 32:]), dim=2).contiguous())

    def _pick(self, load, n: int, cost: int = 0):
        order = sorted(range(self.num_sms), key=lambda s: (load[s], s))
        sms = [order[i % self.num_sms] for i in range(n)]
        for sm in sms:
            load[sm] += cost
        return sms

    def _build_program(self):
        """Plans every task of one decode step per SM (stage by stage, balancing
        the bytes each SM streams), then emits the instruction streams.  After
        the weight loads of a task have been issued, the memory core prefetches
        the next `l2_prefetch_bytes` of that SM's weight stream into L2, so HBM
        keeps streaming while the compute core waits on a cross-SM dependency."""
        cfg = self.cfg
        L, H, F, V, G = cfg.n_layers, cfg.hidden, cfg.ffn, cfg.vocab, cfg.group
        D = isa.HEAD_DIM
        S = self.num_sms
        P = Program(S, insts_per_sm=isa.MAX_INSTS)
        st = self.state.data_ptr()
        page_bytes = isa.KV_PAGE * D * 2
        page_stride = cfg.n_kv_heads * page_bytes
        page_shift = int(math.log2(page_stride))
        assert 1 << page_shift == page_stride
        hid, qkv, ao, act = (t.data_ptr() for t in (self.hidden, self.qkv, self.attn_out, self.act))
        embed_src = lambda: Src(self.embed.data_ptr(), H * 2, indirect=(st + 4 * isa.ST_TOKEN, None, H * 2))
        rb = self.row_bytes
        rpc = lambda K, even=False: rows_per_chunk(K, even, row_bytes=rb(K))
        skey = {'fp8': 'fp8_scales', 'nvfp4': 'nvfp4_scales'}.get(self.wkind)
        sk = lambda name, l, r0: {skey: self.scales[name][l].data_ptr() + 4 * r0} if skey else {}
        load = [0] * S
        plan = [[] for _ in range(S)]      # per SM: (emit(sm), weight segment or None)
        kmult = {"bf16": 256, "fp8": 512, "nvfp4": 1024}[self.wkind]
        self.split_down = (self.split_down_wanted and not cfg.n_experts and not self.shared_counters
                           and F % 2 == 0 and (F // 2) % kmult == 0)
        if self.split_down:
            self.wd_half = self._halve_k(self.wd, F)
            self.down_partial = torch.zeros(H, dtype=torch.float32, device=self.dev)

        def add_gemv(sm, wseg, **kw):
            plan[sm].append((lambda sm=sm, kw=kw: P.gemv(sm, **kw), wseg))

        rot = [0]      # interleaved dealing: the SM that gets the next stage's first chunk

        def stage_ranges(n_units, unit_bytes):
            """(sm, first unit, units, extra gemv arguments) per SM: fixed contiguous ranges; with `interleave` the
            chunks dealt round-robin (SM after SM, continuing where the previous stage stopped); or with shared
            counters the whole matrix on every SM (the SMs draw its chunks from one counter)."""
            if self.interleave and not self.shared_counters:
                out = []
                for sm in range(S):
                    u0 = (sm - rot[0]) % S
                    cnt = (n_units - u0 + S - 1) // S if u0 < n_units else 0
                    if cnt:
                        out.append((sm, u0, cnt, dict(chunk_stride=S) if cnt > 1 else None))
                        load[sm] += cnt * unit_bytes
                rot[0] = (rot[0] + n_units) % S
                return out
            if not self.shared_counters:
                return [(sm, u0, cnt, None) for sm, u0, cnt in self._ranges(load, n_units, unit_bytes)]
            # every SM owns the same number of chunks; the last `tail_fraction` of the stage is drawn from a counter
            own = int(n_units * (1.0 - self.tail_fraction)) // S
            ctr = P.new_barrier()
            for sm in range(S):
                load[sm] += n_units * unit_bytes // S
            return [(sm, 0, n_units, dict(shared_counter=ctr, own_chunks=(sm * own, own), shared_first=S * own,
                                          shared_depth=self.shared_depth)) for sm in range(S)]

        b_hid = None
        for l in range(L):
            # ---- QKV projection with fused input RMSNorm
            b_qkv = P.new_barrier()
            R = rpc(H)
            for sm, u0, cnt, ctr in stage_ranges(self.qkv_rows // R, R * rb(H)):
                r0, n = u0 * R, cnt * R
                x = Src(hid, H * 2, wait=b_hid) if l > 0 else embed_src()
                wa = self.wqkv[l].data_ptr() + r0 * rb(H)
                add_gemv(sm, (wa, n * rb(H)), w_addr=wa, n_rows=n, K=H, R=R, x=x, **sk('wqkv', l, r0),
                         out=Dst(qkv + r0 * 2, n * 2, "store", release=b_qkv),
                         norm_w=Src(self.ln1[l].data_ptr(), H * 2), eps=cfg.eps, **(ctr or {}))
            if l == 0:
                sm = self._pick(load, 1)[0]
                plan[sm].append((lambda sm=sm, b=b_qkv: P.copy(sm, embed_src(), Dst(hid, H * 2, release=b), H * 2), None))
            elif self.taps_enabled:
                sm = self._pick(load, 1)[0]
                plan[sm].append((lambda sm=sm, b=b_qkv, bw=b_hid, t=self.taps[l - 1].data_ptr():
                                 P.copy(sm, Src(hid, H * 2, wait=bw), Dst(t, H * 2, release=b), H * 2), None))

            # ---- split-K GQA decode attention over the paged cache; the unit that finishes a
            # head last merges its split records and releases the barrier
            b_merge = P.new_barrier()
            P.add_releases(b_merge, cfg.n_kv_heads)
            units = [(h, s) for s in range(self.n_splits) for h in range(cfg.n_kv_heads)]
            kp, vp = self.kpool[l].data_ptr(), self.vpool[l].data_ptr()
            grp = (G + 2) * D * 2
            for (h, s), sm in zip(units, self._pick(load, len(units), 2 * page_bytes * self.pages_per_split)):
                kw = dict(
                    G=G, state_addr=st,
                    rope=Src(self.rope.data_ptr(), D * 4, indirect=(st + 4 * isa.ST_POS, 9, None)),
                    norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                    qkv=Src(qkv + h * grp, grp, wait=b_qkv),
                    k_page_addr=kp + h * page_bytes, v_page_addr=vp + h * page_bytes, page_shift=page_shift,
                    base_page=s * self.pages_per_split, max_pages=self.pages_per_split,
                    records_addr=self.attn_part[h].data_ptr(), counter_addr=self.attn_cnt[l, h].data_ptr(),
                    out_addr=ao + h * G * D * 2, split=s, n_splits=self.n_splits, release=b_merge,
                    qk_eps=cfg.qk_norm_eps)
                plan[sm].append((lambda sm=sm, kw=kw: P.attn_decode(sm, **kw), None))

            # ---- output projection, residual add into hidden
            b_o = P.new_barrier()
            K = cfg.q_width
            R = rpc(K)
            for sm, u0, cnt, ctr in stage_ranges(H // R, R * rb(K)):
                r0, n = u0 * R, cnt * R
                wa = self.wo[l].data_ptr() + r0 * rb(K)
                add_gemv(sm, (wa, n * rb(K)), w_addr=wa, n_rows=n, K=K, R=R, x=Src(ao, K * 2, wait=b_merge),
                         **sk('wo', l, r0),
                         out=Dst(hid + r0 * 2, n * 2, "add_bf16", release=b_o), **(ctr or {}))

            if cfg.n_experts:
                b_hid = self._plan_moe(P, plan, load, l, b_o, add_gemv)
                continue
            # ---- gate/up projection with fused post-attention RMSNorm and SiLU·mul, then the down projection with
            # the residual add into hidden.  With `split_down` both run as two half-stages: the SMs first produce
            # the first half of the activation vector (gate/up rows 0..F-1), then the second; the down projection
            # runs over the first half of its K (fp32 partial rows, kept by the SM that owns the rows) and then over
            # the second.  The first down pass waits for a barrier that opened half a gate/up stage earlier and the
            # second for one that opens while the first pass streams, so no SM idles at the gate/up -> down boundary.
            R = rpc(H, True)
            if self.split_down:
                halves = [(P.new_barrier(), 0), (P.new_barrier(), F)]
            else:
                halves = [(P.new_barrier(), None)]
            for b_half, first_row in halves:
                n_units = (2 * F if first_row is None else F) // R
                for sm, u0, cnt, ctr in stage_ranges(n_units, R * rb(H)):
                    r0, n = (first_row or 0) + u0 * R, cnt * R
                    wa = self.wgu[l].data_ptr() + r0 * rb(H)
                    add_gemv(sm, (wa, n * rb(H)), w_addr=wa, n_rows=n, K=H, R=R, x=Src(hid, H * 2, wait=b_o),
                             **sk('wgu', l, r0),
                             out=Dst(act + (r0 // 2) * 2, n, "store", release=b_half), mode=isa.GEMV_MODE_SILU_PAIRS,
                             norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps, **(ctr or {}))
            b_hid = P.new_barrier()
            if self.split_down:
                Kh = F // 2
                R = rpc(Kh)
                ranges = stage_ranges(H // R, 2 * R * rb(Kh))      # one SM owns a row block in both passes
                part = self.down_partial.data_ptr()
                for half, (b_half, _) in enumerate(halves):
                    wmat = self.wd_half[half][l]
                    for sm, u0, cnt, ctr in ranges:
                        r0, n = u0 * R, cnt * R
                        wa = wmat.data_ptr() + r0 * rb(Kh)
                        x = Src(act + half * Kh * 2, Kh * 2, wait=b_half)
                        if half == 0:
                            add_gemv(sm, (wa, n * rb(Kh)), w_addr=wa, n_rows=n, K=Kh, R=R, x=x, **sk('wd', l, r0),
                                     out=Dst(part + r0 * 4, n * 4, "store"), mode=isa.GEMV_MODE_STORE_F32)
                        else:
                            add_gemv(sm, (wa, n * rb(Kh)), w_addr=wa, n_rows=n, K=Kh, R=R, x=x, **sk('wd', l, r0),
                                     out=Dst(hid + r0 * 2, n * 2, "add_bf16", release=b_hid), partial_in=part + r0 * 4)
            else:
                b_gu = halves[0][0]
                R = rpc(F)
                for sm, u0, cnt, ctr in stage_ranges(H // R, R * rb(F)):
                    r0, n = u0 * R, cnt * R
                    wa = self.wd[l].data_ptr() + r0 * rb(F)
                    add_gemv(sm, (wa, n * rb(F)), w_addr=wa, n_rows=n, K=F, R=R, x=Src(act, F * 2, wait=b_gu),
                             **sk('wd', l, r0),
                             out=Dst(hid + r0 * 2, n * 2, "add_bf16", release=b_hid), **(ctr or {}))

        # ---- final norm + vocabulary projection + per-SM argmax candidates
        b_logits = P.new_barrier()
        R = rows_per_chunk(H)
        if self.taps_enabled:
            sm = self._pick(load, 1)[0]
            b_tap = P.new_barrier()
            plan[sm].append((lambda sm=sm: P.copy(sm, Src(hid, H * 2, wait=b_hid),
                                                  Dst(self.taps[L - 1].data_ptr(), H * 2, release=b_tap), H * 2), None))
        lm_ranges = stage_ranges(V // R, R * H * 2)
        for i, (sm, u0, cnt, ctr) in enumerate(lm_ranges):
            r0, n = u0 * R, cnt * R
            wa = self.lm_head.data_ptr() + r0 * H * 2
            add_gemv(sm, (wa, n * H * 2), w_addr=wa, n_rows=n, K=H, R=R, x=Src(hid, H * 2, wait=b_hid),
                     out=Dst(self.logits.data_ptr() + r0 * 2, n * 2, "store", release=b_logits),
                     mode=isa.GEMV_MODE_ARGMAX, norm_w=Src(self.norm_w.data_ptr(), H * 2), eps=cfg.eps,
                     pair_out=Dst(self.argmax_rec[i].data_ptr(), 16, release=b_logits), row_base=r0,
                     **(ctr or {}))
        sm = self._pick(load, 1)[0]
        plan[sm].append((lambda sm=sm: P.argmax_final(
            sm, records=Src(self.argmax_rec.data_ptr(), len(lm_ranges) * 16, wait=b_logits), n=len(lm_ranges),
            state_addr=st, log_addr=self.token_log.data_ptr()), None))

        # ---- emission.  Before every task the compute core is told to pull the next
        # `l2_prefetch_bytes` of this SM's weight stream into L2 (beyond the part the
        # memory core already holds in flight): it reaches that point exactly when it
        # is about to wait for an activation from the other SMs, so HBM keeps streaming
        # through the dependency bubble and the stalled stage later reads from L2.
        in_flight = (isa.NUM_SLOTS - 4) * isa.SLOT_BYTES
        for sm in range(S):
            segs = [w for _, w in plan[sm] if w is not None]
            seg_idx = 0          # segments before this index belong to tasks already emitted
            pf_seg, pf_off = 0, 0
            for emit, w in plan[sm]:
                if self.l2_prefetch_bytes > 0:
                    # frontier never behind the current task's start (+ what the memory core covers itself)
                    if pf_seg < seg_idx:
                        pf_seg, pf_off = seg_idx, 0
                    ahead = sum(segs[j][1] for j in range(seg_idx, pf_seg)) + pf_off
                    budget = in_flight + self.l2_prefetch_bytes - ahead
                    while budget > 0 and pf_seg < len(segs):
                        addr, nbytes = segs[pf_seg]
                        n = min(budget, nbytes - pf_off)
                        if n <= 0:
                            break
                        # the first `in_flight` bytes after the demand pointer are fetched by TMA anyway
                        skip = max(0, in_flight - (ahead)) if pf_seg == seg_idx and pf_off == 0 else 0
                        skip = min(skip, n)
                        if n - skip >= 4096:
                            P.l2_prefetch(sm, addr + pf_off + skip, n - skip)
                        budget -= n
                        ahead += n
                        pf_off += n
                        if pf_off >= nbytes:
                            pf_seg, pf_off = pf_seg + 1, 0
                emit()
                if w is not None:
                    seg_idx += 1

        st_ = P.stats()
        n_insts = max(st_["max_minsts"], st_["max_cinsts"]) + 2
        P.insts_per_sm = ((n_insts + 63) // 64) * 64
        c, m, bars = P.finalize()
        self.program = P
        self.insts_per_sm = P.insts_per_sm
        self.cinsts = torch.from_numpy(c).to(self.dev)
        self.minsts = torch.from_numpy(m).to(self.dev)
        self.bars_init = torch.from_numpy(bars).to(self.dev)
        self.launches_per_step = 1

    def _plan_moe(self, P, plan, load, l, b_o, add_gemv):
        """Router, top-k routing and the selected experts' gate/up and down projections of layer l."""
        cfg = self.cfg
        H, F, E, TK = cfg.hidden, cfg.ffn, cfg.n_experts, cfg.top_k
        hid = self.hidden.data_ptr()
        ids_addr = self.route.data_ptr()
        wts_addr = ids_addr + 64
        # ---- router logits (fp32) over all SMs that get a chunk
        b_rl = P.new_barrier()
        R = rows_per_chunk(H)
        for sm, u0, cnt in self._ranges(load, E // R, R * H * 2):
            r0, n = u0 * R, cnt * R
            wa = self.router[l].data_ptr() + r0 * H * 2
            add_gemv(sm, None, w_addr=wa, n_rows=n, K=H, R=R, x=Src(hid, H * 2, wait=b_o),
                     out=Dst(self.router_logits.data_ptr() + r0 * 4, n * 4, "store", release=b_rl),
                     mode=isa.GEMV_MODE_STORE_F32, norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps)
        # ---- softmax / top-k on one SM
        b_route = P.new_barrier()
        sm = self._pick(load, 1)[0]
        plan[sm].append((lambda sm=sm: P.moe_route(sm, logits=Src(self.router_logits.data_ptr(), E * 4, wait=b_rl),
                                                   route_addr=ids_addr, n_experts=E, top_k=TK, release=b_route), None))
        # ---- the selected experts' gate/up: units are (slot, chunk), contiguous per SM, split at slot borders
        b_gu = P.new_barrier()
        R = rows_per_chunk(H, even=True)
        per = 2 * F // R
        stride_gu = 2 * F * H * 2
        for sm, u0, cnt in self._ranges(load, TK * per, R * H * 2):
            u, end = u0, u0 + cnt
            while u < end:
                slot, c0 = divmod(u, per)
                n_c = min(end - u, per - c0)
                r0, n = c0 * R, n_c * R
                add_gemv(sm, None, w_addr=self.wgu[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R,
                         x=Src(hid, H * 2, wait=b_o), out=Dst(self.act[slot].data_ptr() + (r0 // 2) * 2, n, "store", release=b_gu),
                         mode=isa.GEMV_MODE_SILU_PAIRS, norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps,
                         w_indirect=(ids_addr + 4 * slot, stride_gu), wait_issue=b_route)
                u += n_c
        # ---- the selected experts' down projections, weighted and accumulated per output row;
        # the last expert to reach a row folds the sum into the hidden state
        b_hid = P.new_barrier()
        R = rows_per_chunk(F)
        per = H // R
        stride_d = H * F * 2
        for sm, u0, cnt in self._ranges(load, TK * per, R * F * 2):
            u, end = u0, u0 + cnt
            while u < end:
                slot, c0 = divmod(u, per)
                n_c = min(end - u, per - c0)
                r0, n = c0 * R, n_c * R
                add_gemv(sm, None, w_addr=self.wd[l].data_ptr() + r0 * F * 2, n_rows=n, K=F, R=R,
                         x=Src(self.act[slot].data_ptr(), F * 2, wait=b_gu), out=Dst(hid + r0 * 2, n * 2, "store", release=b_hid),
                         mode=isa.GEMV_MODE_MOE_DOWN, w_indirect=(ids_addr + 4 * slot, stride_d), wait_issue=b_route,
                         moe=dict(weight_addr=wts_addr + 4 * slot, acc_addr=self.moe_acc.data_ptr() + 4 * r0,
                                  cnt_addr=self.moe_cnt.data_ptr() + 4 * r0, top_k=TK))
                u += n_c
        return b_hid

    # ------------------------------------------------------------------ state
    def set_state(self, pos: int, token: int):
        """Positions [0, pos) are cached; `token` is decoded next at position pos."""
        assert pos < self.max_seq
        s = self.state_host
        s.zero_()
        page = pos // isa.KV_PAGE
        s[isa.ST_POS] = pos
        s[isa.ST_NPAGES] = page + 1
        s[isa.ST_TOKEN] = token
        s[isa.ST_STEP] = 0
        s[isa.ST_NEWROW] = int(self.page_table[page]) * isa.KV_PAGE * self.cfg.n_kv_heads + pos % isa.KV_PAGE
        s[isa.ST_NKVH] = self.cfg.n_kv_heads
        s[isa.ST_MAXPAGES] = self.max_pages
        s[isa.ST_PAGETABLE:] = self.page_table
        self.state.copy_(s, non_blocking=True)
        self.attn_cnt.zero_()
        if self.cfg.n_experts:
            self.moe_acc.zero_()
            self.moe_cnt.zero_()
        self.pos = pos
        self.steps_done = 0

    def load_kv(self, k: List[torch.Tensor], v: List[torch.Tensor]):
        """Fills the paged pools from per-layer contiguous caches [T, n_kv_heads, 128]."""
        cfg = self.cfg
        pt = self.page_table.long().to(self.dev)
        for l in range(cfg.n_layers):
            for src, pool in ((k[l], self.kpool[l]), (v[l], self.vpool[l])):
                T = src.shape[0]
                n_pages = (T + isa.KV_PAGE - 1) // isa.KV_PAGE
                pad = torch.zeros(n_pages * isa.KV_PAGE, cfg.n_kv_heads, isa.HEAD_DIM, dtype=BF16, device=self.dev)
                pad[:T] = src.to(self.dev)
                pool[pt[:n_pages]] = kv_page_swizzle(
                    pad.view(n_pages, isa.KV_PAGE, cfg.n_kv_heads, isa.HEAD_DIM).permute(0, 2, 1, 3))

    def read_kv(self, layer: int, T: int):
        """Contiguous [T, n_kv_heads, 128] views of layer `layer`'s cache (tests)."""
        n_pages = (T + isa.KV_PAGE - 1) // isa.KV_PAGE
        pt = self.page_table.long().to(self.dev)[:n_pages]
        out = []
        for pool in (self.kpool[layer], self.vpool[layer]):
            t = kv_page_swizzle(pool[pt]).permute(0, 2, 1, 3).reshape(n_pages * isa.KV_PAGE, self.cfg.n_kv_heads, isa.HEAD_DIM)
            out.append(t[:T])
        return out

    # ------------------------------------------------------------------ prefill (PyTorch, not the timed path)
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> int:
        """Runs the prompt through plain PyTorch ops on the GPU, fills the KV
        pools and returns the greedy next token.  The decode path starts after it."""
        cfg, dev = self.cfg, self.dev
        D, G = isa.HEAD_DIM, cfg.group
        T = tokens.numel()
        ids = tokens.to(dev).long()
        h = self.embed[ids]
        cos = self.rope[:T, :64].to(BF16)
        sin = self.rope[:T, 64:].to(BF16)
        cos = torch.cat((cos, cos), -1)[:, None, :]
        sin = torch.cat((sin, sin), -1)[:, None, :]

        def norm(x, w, eps):
            xf = x.float()
            return w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(BF16)

        def rot(x):
            return torch.cat((-x[..., D // 2:], x[..., :D // 2]), -1)
        ks, vs = [], []
        for l in range(cfg.n_layers):
            x = norm(h, self.ln1[l], cfg.eps)
            qkv = (x @ self._dense('wqkv', l).t())[:, self.qkv_inv.to(dev)]
            q = qkv[:, :cfg.q_width].view(T, cfg.n_heads, D)
            k = qkv[:, cfg.q_width:cfg.q_width + cfg.kv_width].view(T, cfg.n_kv_heads, D)
            v = qkv[:, cfg.q_width + cfg.kv_width:].view(T, cfg.n_kv_heads, D)
            if cfg.qk_norm:
                q = norm(q, self.qknorm[l, :D], cfg.qk_norm_eps)
                k = norm(k, self.qknorm[l, D:], cfg.qk_norm_eps)
            q = q * cos + rot(q) * sin
            k = k * cos + rot(k) * sin
            ks.append(k)
            vs.append(v)
            o = torch.nn.functional.scaled_dot_product_attention(
                q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], is_causal=True,
                enable_gqa=True)[0].transpose(0, 1).reshape(T, cfg.q_width)
            h = h + o @ self._dense('wo', l).t()
            x = norm(h, self.ln2[l], cfg.eps)
            if cfg.n_experts:
                probs = torch.softmax(x.float() @ self.router[l].float().t(), dim=-1)
                tw, ti = torch.topk(probs, cfg.top_k, dim=-1)
                tw = (tw / tw.sum(-1, keepdim=True)).to(BF16)
                y = torch.zeros(T, cfg.hidden, dtype=torch.float32, device=dev)
                for e in ti.unique().tolist():
                    rows, slots = (ti == e).nonzero(as_tuple=True)
                    gu = x[rows] @ self.wgu[l, e].t()
                    a = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
                    y.index_add_(0, rows, (a @ self.wd[l, e].t()).float() * tw[rows, slots].float()[:, None])
                h = h + y.to(BF16)
                continue
            gu = x @ self._dense('wgu', l).t()
            a = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
            h = h + a @ self._dense('wd', l).t()
        self.load_kv(ks, vs)
        hn = norm(h[-1], self.norm_w, cfg.eps)
        logits = hn @ self.lm_head.t()
        tok = int(torch.argmax(logits.float()))
        self.set_state(T, tok)
        return tok

    def prefill_device(self, tokens: torch.Tensor) -> int:
        """The prompt goes through the decode megakernel itself, one position per launch: the same program as a
        decode step, with the next prompt id written over the step's own argmax before the next launch (an 8-byte
        device-to-device copy on the engine's stream: {next id, step counter 0}).  No PyTorch arithmetic and no
        host round trip inside the loop; the KV rows and the returned first generated id have exactly the decode
        path's numerics.  Cost: one decode step per prompt position (PrefillEngine in prefill.py does 64
        positions per launch)."""
        T = int(tokens.numel())
        assert 1 <= T < self.max_seq
        forced = torch.zeros(T, 2, dtype=torch.int32)
        forced[:T - 1, 0] = tokens[1:].to(torch.int32)
        forced = forced.to(self.dev)
        self.set_state(0, int(tokens[0]))
        word = self.state[isa.ST_TOKEN:isa.ST_STEP + 1]
        assert isa.ST_STEP == isa.ST_TOKEN + 1
        with torch.cuda.stream(self.stream):
            for t in range(T):
                runtime.launch_async(self.num_sms, self.insts_per_sm, self.cinsts, self.minsts, None, self.bars,
                                     self.bars_init, self.profile, self.stream.cuda_stream, self.timeout_ns)
                if t + 1 < T:
                    word.copy_(forced[t], non_blocking=True)
        runtime.read_status(self.stream.cuda_stream)
        tok = int(self.token_log[0])
        self.set_state(T, tok)
        return tok

    # ------------------------------------------------------------------ decode
    def step_async(self):
        """Enqueues one decode step (one kernel launch); no synchronisation."""
        assert self.program is not None, "load weights first"
        if self.pos >= self.max_seq or self.steps_done >= self.max_steps:
            raise RuntimeError("out of KV pages or token-log space")
        runtime.launch_async(self.num_sms, self.insts_per_sm, self.cinsts, self.minsts, None, self.bars,
                             self.bars_init, self.profile, self.stream.cuda_stream, self.timeout_ns,
                             full=self.FULL_KERNEL)
        self.pos += 1
        self.steps_done += 1

    def generate(self, n_steps: int) -> List[int]:
        """Greedy decode of n_steps tokens, device resident; returns the ids."""
        first = self.steps_done
        for _ in range(n_steps):
            self.step_async()
        runtime.read_status(self.stream.cuda_stream)
        return self.token_log[first:first + n_steps].tolist()

    def generate_sampled(self, n_steps: int, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                         seed: int = 0) -> List[int]:
        """Decode with temperature / top-k / nucleus sampling instead of the kernel's own argmax.  Every step is
        the same launch as a greedy step; the draw from the step's logits (a softmax over one vocabulary row: PyTorch
        ops on the engine's stream, not part of the megakernel) replaces the id the kernel left in the state block
        before the next launch, without a host round trip.  top_k = 1 or temperature -> 0 reproduce generate()."""
        assert temperature >= 0.0 and 0.0 < top_p <= 1.0 and top_k >= 0
        g = torch.Generator(device=self.dev).manual_seed(seed)
        out = torch.empty(n_steps, dtype=torch.int32, device=self.dev)
        word = self.state[isa.ST_TOKEN:isa.ST_TOKEN + 1]
        with torch.cuda.stream(self.stream):
            for i in range(n_steps):
                self.step_async()
                lg = self.logits.float()
                if temperature < 1e-6 or top_k == 1:
                    tok = torch.argmax(lg).reshape(1)
                else:
                    lg = lg / temperature
                    if top_k:
                        lg = lg.masked_fill(lg < torch.topk(lg, top_k).values[-1], float("-inf"))
                    p = torch.softmax(lg, -1)
                    if top_p < 1.0:
                        ps, idx = torch.sort(p, descending=True)
                        keep = torch.cumsum(ps, 0) - ps < top_p        # the smallest prefix whose mass reaches top_p
                        p = torch.zeros_like(p).scatter_(0, idx[keep], ps[keep])
                    tok = torch.multinomial(p, 1, generator=g)
                out[i] = tok[0]
                word.copy_(tok.to(torch.int32))
        runtime.read_status(self.stream.cuda_stream)
        return out.tolist()

    def step_host(self, token: int) -> int:
        """One decode step driven from host buffers: the token id goes up, the
        next id comes back (synchronous)."""
        if not hasattr(self, "_tok_in"):
            self._tok_in = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._tok_out = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._tok_in[0] = token
        self.state[isa.ST_TOKEN:isa.ST_TOKEN + 1].copy_(self._tok_in, non_blocking=True)
        idx = self.steps_done
        self.step_async()
        self._tok_out.copy_(self.token_log[idx:idx + 1], non_blocking=True)
        runtime.read_status(self.stream.cuda_stream)
        return int(self._tok_out[0])
