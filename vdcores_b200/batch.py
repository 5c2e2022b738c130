"""Batched greedy decode (2..128 sequences in lock-step) on the tensor cores.

The reference pads every decode batch to 8 request slots and pushes it through
its 64x8 WGMMA GEMV tile (reference include/task/gemv.cuh:13-128,
python/dae/schedule.py:404-570).  Here the projections of a batch run on the
tcgen05 tensor cores: the batch sits on the 128 lanes of the accumulator in
tensor memory, each SM owns groups of 16 weight rows of every projection, and
activations live in HBM in the k-chunk-major layout the tensor cores read
without swizzling (csrc/isa.h).  Attention, RoPE, QK-norm and the KV cache are
the batch-1 tasks, one unit per (sequence, KV head, split), each sequence with
its own state block and page table.
"""
from __future__ import annotations

import math
from typing import List

import torch

from . import isa, runtime
from .decode import BF16, DecodeConfig, DecodeEngine
from .program import Dst, Program, Src, slots_for


def pack_kc(x: torch.Tensor) -> torch.Tensor:
    """[R, K] -> flat k-chunk-major [K/8][R/8][8][8] (R, K multiples of 8)."""
    R, K = x.shape
    return x.reshape(R // 8, 8, K // 8, 8).permute(2, 0, 1, 3).contiguous().view(-1)


def unpack_kc(flat: torch.Tensor, R: int, K: int) -> torch.Tensor:
    return flat.view(K // 8, R // 8, 8, 8).permute(1, 2, 0, 3).reshape(R, K)


def choose_kc(N: int, Bpad: int, K: int, max_slots: int = 6) -> int:
    """Largest K-range per chunk (a multiple of 16 dividing K) whose X and W chunks fit in
    max_slots shared-memory slots together, so that at least three pairs are in flight."""
    best = 0
    for kc in range(16, K + 1, 16):
        if K % kc:
            continue
        xb, wb = Bpad * kc * 2, N * kc * 2
        if xb > 32768 or wb > 32768:
            break
        if slots_for(xb + max(0, 2048 - Bpad * 16)) + slots_for(wb) <= max_slots:
            best = kc
    assert best, (N, Bpad, K)
    return best


class BatchDecodeEngine(DecodeEngine):
    """`batch` sequences decoded together, one kernel launch per step.  Dense bf16 models."""

    def __init__(self, cfg: DecodeConfig, batch: int, max_seq: int, device="cuda:0", num_sms=None, taps=False,
                 page_perm_seed=None, max_steps: int = 256, timeout_ns: int = 2_000_000_000):
        assert 1 <= batch <= 128 and not cfg.n_experts
        self.batch = batch
        self.bpad = next(p for p in (16, 32, 64, 128) if batch <= p)
        super().__init__(cfg, max_seq, device=device, num_sms=num_sms, taps=False, page_perm_seed=None,
                         max_steps=max_steps, timeout_ns=timeout_ns, wkind="bf16")
        B, Bp, L, H, F = batch, self.bpad, cfg.n_layers, cfg.hidden, cfg.ffn
        z = lambda *s, dt=BF16: torch.zeros(*s, dtype=dt, device=self.dev)
        self.hidden = z(Bp * H)                       # k-chunk-major [Bpad, H]
        self.attn_out = z(Bp * cfg.q_width)           # k-chunk-major [Bpad, q_width]
        self.act = z(Bp * F)                          # k-chunk-major [Bpad, F]
        self.qkv = z(B, self.qkv_rows)                # per sequence: [G q heads | k | v] per KV head
        self.keys = z(B, dt=torch.int64)              # argmax keys (u64), zero between steps
        # per-sequence sums of squares of the hidden matrix after the embedding / each residual add
        # (the RMSNorm statistics of the projection that reads it); zero between steps
        self.stats = z(2 * L + 1, 128, dt=torch.float32)
        units = B * cfg.n_kv_heads
        self.n_splits = 1 if units >= self.num_sms else max(1, min(self.num_sms // units, self.max_pages))
        self.pages_per_split = (self.max_pages + self.n_splits - 1) // self.n_splits
        self.n_splits = (self.max_pages + self.pages_per_split - 1) // self.pages_per_split
        self.attn_part = z(B, cfg.n_kv_heads, self.n_splits, self.rec_floats, dt=torch.float32)
        self.attn_cnt = z(L, B, cfg.n_kv_heads, dt=torch.int32)
        self.state_words = isa.ST_PAGETABLE + self.max_pages
        self.state = z(B, self.state_words, dt=torch.int32)
        self.state_host = torch.zeros(B, self.state_words, dtype=torch.int32).pin_memory()
        self.token_log = z(B, max_steps, dt=torch.int32)
        self.kpool = z(L, B * self.max_pages, cfg.n_kv_heads, isa.KV_PAGE, isa.HEAD_DIM)
        self.vpool = z(L, B * self.max_pages, cfg.n_kv_heads, isa.KV_PAGE, isa.HEAD_DIM)
        tables = []
        for b in range(B):
            if page_perm_seed is None:
                t = torch.arange(self.max_pages, dtype=torch.int32)
            else:
                t = torch.randperm(self.max_pages, generator=torch.Generator().manual_seed(page_perm_seed + b)).to(torch.int32)
            tables.append(t + b * self.max_pages)
        self.page_tables = torch.stack(tables)        # [B, max_pages] global page ids
        self.taps_enabled = taps
        if taps:
            assert Bp * H * 2 <= 32768, "taps copy the hidden matrix with one bulk load"
            self.taps = z(L, Bp * H)
        self._cur = 0
        self.positions = [0] * B

    # ------------------------------------------------------------------ weights
    def _units(self, load, n_rows: int, K: int):
        """Deals the projection's groups of 16 rows to the SMs; returns [(sm, first row, N)], N <= 256."""
        assert n_rows % 16 == 0
        out = []
        for sm, u0, cnt in self._ranges(load, n_rows // 16, 16 * K * 2):
            while cnt > 0:
                n = min(cnt, 16)
                out.append((sm, u0 * 16, n * 16))
                u0 += n
                cnt -= n
        return out

    @staticmethod
    def _pack_units(w: torch.Tensor, units) -> torch.Tensor:
        """Rows of w regrouped unit by unit into k-chunk-major blocks; unit (r0, N) starts at element r0 * K."""
        M, K = w.shape
        out = torch.empty(M * K, dtype=w.dtype, device=w.device)
        i = 0
        while i < len(units):
            j = i
            while j + 1 < len(units) and units[j + 1][2] == units[i][2]:
                j += 1
            r0, N = units[i][1], units[i][2]
            n_u = j - i + 1
            blk = w[r0:r0 + n_u * N].reshape(n_u, N // 8, 8, K // 8, 8).permute(0, 3, 1, 2, 4)
            out[r0 * K:(r0 + n_u * N) * K] = blk.reshape(-1)
            i = j + 1
        return out

    def weight_bytes(self) -> int:
        ts = [self.lm_head, self.norm_w, self.ln1, self.ln2, self.wqkv, self.wo, self.wgu, self.wd]
        return sum(t.numel() * t.element_size() for t in ts)

    def algorithmic_bytes(self, pos: int) -> int:
        """HBM bytes of one step with every sequence at position `pos`: each weight once, one
        embedding row and the KV rows of pos+1 positions per sequence."""
        cfg = self.cfg
        return self.weight_bytes() + self.batch * (cfg.hidden * 2 + 2 * cfg.kv_width * 2 * (pos + 1) * cfg.n_layers)

    # ------------------------------------------------------------------ program
    def _build_program(self):
        cfg = self.cfg
        L, H, F, V, G = cfg.n_layers, cfg.hidden, cfg.ffn, cfg.vocab, cfg.group
        D, S, B, Bp = isa.HEAD_DIM, self.num_sms, self.batch, self.bpad
        P = Program(S, insts_per_sm=isa.MAX_INSTS)
        st, sw = self.state.data_ptr(), self.state_words
        page_bytes = isa.KV_PAGE * D * 2
        page_stride = cfg.n_kv_heads * page_bytes
        page_shift = int(math.log2(page_stride))
        assert 1 << page_shift == page_stride
        hid, qkv, ao, act = (t.data_ptr() for t in (self.hidden, self.qkv, self.attn_out, self.act))
        load = [0] * S
        packed = {"wqkv": [], "wo": [], "wgu": [], "wd": []}

        stat = lambda i: self.stats[i].data_ptr()

        def gemm_stage(w, name, K, x_addr, x_wait, mode, out_addr, release, norm=None, ld=0, keys=0, stats=0):
            units = self._units(load, w.shape[0], K)
            pk = self._pack_units(w, units)
            if name is not None:
                packed[name].append(pk)
            for sm, r0, N in units:
                P.gemm_tc(sm, w_addr=pk.data_ptr() + r0 * K * 2, N=N, K=K, Kc=choose_kc(N, Bp, K), x_addr=x_addr, B=B,
                          Bpad=Bp, out_addr=out_addr, mode=mode, x_wait=x_wait,
                          norm_w=Src(norm.data_ptr(), K * 2) if norm is not None else None, eps=cfg.eps, n0=r0, ld=ld,
                          keys_addr=keys, stats_addr=stats, release=release)
            return pk

        def tap(l, wait, release):
            sm = self._pick(load, 1)[0]
            n = Bp * H * 2
            P.copy(sm, Src(hid, n, wait=wait), Dst(self.taps[l].data_ptr(), n, release=release), n)

        # ---- embedding rows into the hidden matrix
        b_hid = P.new_barrier()
        for b, sm in enumerate(self._pick(load, B)):
            P.embed_pack(sm, b0=b, count=1, Bpad=Bp, state_addr=st, state_stride_words=sw, hidden=H,
                         table_addr=self.embed.data_ptr(), out_addr=hid, stats_addr=stat(0), release=b_hid)
        for l in range(L):
            # ---- QKV projection with fused input RMSNorm
            b_qkv = P.new_barrier()
            gemm_stage(self.wqkv[l], "wqkv", H, hid, b_hid, isa.GEMM_MODE_STORE_ROWS, qkv, b_qkv, norm=self.ln1[l],
                       ld=self.qkv_rows, stats=stat(2 * l))
            if self.taps_enabled and l > 0:
                tap(l - 1, b_hid, b_qkv)
            # ---- attention: one unit per (sequence, KV head, split)
            b_merge = P.new_barrier()
            P.add_releases(b_merge, B * cfg.n_kv_heads)
            units = [(b, h, s) for s in range(self.n_splits) for b in range(B) for h in range(cfg.n_kv_heads)]
            kp, vp = self.kpool[l].data_ptr(), self.vpool[l].data_ptr()
            grp = (G + 2) * D * 2
            for (b, h, s), sm in zip(units, self._pick(load, len(units), 2 * page_bytes * self.pages_per_split)):
                sb = st + 4 * sw * b
                P.attn_decode(
                    sm, G=G, state_addr=sb,
                    rope=Src(self.rope.data_ptr(), D * 4, indirect=(sb + 4 * isa.ST_POS, 9, None)),
                    norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                    qkv=Src(qkv + (b * self.qkv_rows) * 2 + h * grp, grp, wait=b_qkv),
                    k_page_addr=kp + h * page_bytes, v_page_addr=vp + h * page_bytes, page_shift=page_shift,
                    base_page=s * self.pages_per_split, max_pages=self.pages_per_split,
                    records_addr=self.attn_part[b, h].data_ptr(), counter_addr=self.attn_cnt[l, b, h].data_ptr(),
                    out_addr=ao + (h * G * D) * Bp * 2, split=s, n_splits=self.n_splits, release=b_merge,
                    qk_eps=cfg.qk_norm_eps, packed=(b, Bp))
            # ---- output projection, residual add into the hidden matrix
            b_o = P.new_barrier()
            gemm_stage(self.wo[l], "wo", cfg.q_width, ao, b_merge, isa.GEMM_MODE_ADD_PACKED, hid, b_o,
                       stats=stat(2 * l + 1))
            # ---- gate/up projection with fused post-attention RMSNorm and SiLU-mul
            b_gu = P.new_barrier()
            gemm_stage(self.wgu[l], "wgu", H, hid, b_o, isa.GEMM_MODE_SILU_PAIRS, act, b_gu, norm=self.ln2[l],
                       stats=stat(2 * l + 1))
            # ---- down projection, residual add
            b_hid = P.new_barrier()
            gemm_stage(self.wd[l], "wd", F, act, b_gu, isa.GEMM_MODE_ADD_PACKED, hid, b_hid, stats=stat(2 * l + 2))
        # ---- final norm, vocabulary projection, per-sequence argmax
        b_lm = P.new_barrier()
        self.lm_head_packed = gemm_stage(self.lm_head, None, H, hid, b_hid, isa.GEMM_MODE_ARGMAX, 0, b_lm,
                                         norm=self.norm_w, keys=self.keys.data_ptr(), stats=stat(2 * L))
        if self.taps_enabled:
            tap(L - 1, b_hid, b_lm)
        sm = self._pick(load, 1)[0]
        P.batch_advance(sm, batch=B, state_addr=st, state_stride_words=sw, keys_addr=self.keys.data_ptr(),
                        log_addr=self.token_log.data_ptr(), log_stride=self.max_steps, wait=b_lm,
                        stats_addr=self.stats.data_ptr(), n_stats=self.stats.numel())
        self.packed = {k: v for k, v in packed.items()}     # keeps the device copies alive
        n = max(max(len(x) for x in P.m), max(len(x) for x in P.c)) + 2
        P.insts_per_sm = ((n + 15) // 16) * 16
        c, m, bars = P.finalize()
        self.program = P
        self.insts_per_sm = P.insts_per_sm
        self.cinsts = torch.from_numpy(c).to(self.dev)
        self.minsts = torch.from_numpy(m).to(self.dev)
        self.bars_init = torch.from_numpy(bars).to(self.dev)
        self.bars.copy_(self.bars_init)
        self.launches_per_step = 1

    # ------------------------------------------------------------------ state
    def set_state(self, pos: int, token: int, b: int = None):
        """Sequence b (default: the one being prefilled) has positions [0, pos) cached and decodes `token` next."""
        b = self._cur if b is None else b
        assert pos < self.max_seq
        s = self.state_host[b]
        s.zero_()
        page = pos // isa.KV_PAGE
        table = self.page_tables[b]
        s[isa.ST_POS] = pos
        s[isa.ST_NPAGES] = page + 1
        s[isa.ST_TOKEN] = token
        s[isa.ST_NEWROW] = int(table[page]) * isa.KV_PAGE * self.cfg.n_kv_heads + pos % isa.KV_PAGE
        s[isa.ST_NKVH] = self.cfg.n_kv_heads
        s[isa.ST_MAXPAGES] = self.max_pages
        s[isa.ST_PAGETABLE:] = table
        self.state[b].copy_(s, non_blocking=True)
        self.attn_cnt.zero_()
        self.keys.zero_()
        self.stats.zero_()
        self.positions[b] = pos
        self.pos = max(self.positions)
        self.steps_done = 0

    def load_kv(self, k: List[torch.Tensor], v: List[torch.Tensor], b: int = None):
        """Fills sequence b's pages from per-layer contiguous caches [T, n_kv_heads, 128]."""
        b = self._cur if b is None else b
        cfg = self.cfg
        pt = self.page_tables[b].long().to(self.dev)
        for l in range(cfg.n_layers):
            for src, pool in ((k[l], self.kpool[l]), (v[l], self.vpool[l])):
                T = src.shape[0]
                n_pages = (T + isa.KV_PAGE - 1) // isa.KV_PAGE
                pad = torch.zeros(n_pages * isa.KV_PAGE, cfg.n_kv_heads, isa.HEAD_DIM, dtype=BF16, device=self.dev)
                pad[:T] = src.to(self.dev)
                pool[pt[:n_pages]] = pad.view(n_pages, isa.KV_PAGE, cfg.n_kv_heads, isa.HEAD_DIM).permute(0, 2, 1, 3)

    def read_kv(self, layer: int, T: int, b: int = 0):
        n_pages = (T + isa.KV_PAGE - 1) // isa.KV_PAGE
        pt = self.page_tables[b].long().to(self.dev)[:n_pages]
        out = []
        for pool in (self.kpool[layer], self.vpool[layer]):
            t = pool[pt].permute(0, 2, 1, 3).reshape(n_pages * isa.KV_PAGE, self.cfg.n_kv_heads, isa.HEAD_DIM)
            out.append(t[:T])
        return out

    def read_hidden(self, flat: torch.Tensor) -> torch.Tensor:
        """A k-chunk-major [Bpad, hidden] matrix as [batch, hidden] (tests)."""
        return unpack_kc(flat, self.bpad, self.cfg.hidden)[:self.batch]

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> List[int]:
        """tokens [batch, T]: each prompt goes through the PyTorch prefill; returns the first greedy tokens."""
        assert tokens.shape[0] == self.batch
        out = []
        for b in range(self.batch):
            self._cur = b
            out.append(DecodeEngine.prefill(self, tokens[b]))
        return out

    # ------------------------------------------------------------------ decode
    def generate(self, n_steps: int) -> List[List[int]]:
        """n_steps greedy steps, device resident; returns [n_steps][batch] token ids."""
        first = self.steps_done
        for _ in range(n_steps):
            self.step_async()
        runtime.read_status(self.stream.cuda_stream)
        self.positions = [p + n_steps for p in self.positions]
        return self.token_log[:, first:first + n_steps].t().tolist()

    def step_host(self, tokens: List[int]) -> List[int]:
        """One step driven from host buffers: batch token ids go up, the next ids come back."""
        if not hasattr(self, "_tok_in"):
            self._tok_in = torch.zeros(self.batch, dtype=torch.int32).pin_memory()
            self._tok_out = torch.zeros(self.batch, dtype=torch.int32).pin_memory()
        self._tok_in.copy_(torch.as_tensor(tokens, dtype=torch.int32))
        self.state[:, isa.ST_TOKEN].copy_(self._tok_in, non_blocking=True)
        idx = self.steps_done
        self.step_async()
        self._tok_out.copy_(self.token_log[:, idx], non_blocking=True)
        runtime.read_status(self.stream.cuda_stream)
        self.positions = [p + 1 for p in self.positions]
        return self._tok_out.tolist()
