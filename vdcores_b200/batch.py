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
from .decode import BF16, DecodeConfig, DecodeEngine, kv_page_swizzle
from .program import Dst, Program, Src, slots_for


def pack_kc(x: torch.Tensor) -> torch.Tensor:
    """[R, K] -> flat k-chunk-major [K/8][R/8][8][8] (R, K multiples of 8)."""
    R, K = x.shape
    return x.reshape(R // 8, 8, K // 8, 8).permute(2, 0, 1, 3).contiguous().view(-1)


def unpack_kc(flat: torch.Tensor, R: int, K: int) -> torch.Tensor:
    return flat.view(K // 8, R // 8, 8, 8).permute(1, 2, 0, 3).reshape(R, K)


BLOCK_ROWS = 256    # weight rows per projection block = accumulator columns of one tensor-core task


def projection_blocks(M: int):
    """[(first row, rows)] of a projection with M output rows (a multiple of 16)."""
    assert M % 16 == 0
    return [(r, min(BLOCK_ROWS, M - r)) for r in range(0, M, BLOCK_ROWS)]


def pack_blocks(w: torch.Tensor) -> torch.Tensor:
    """[M, K] -> flat: every block of 256 rows (the last one may be smaller) k-chunk-major, so
    that any K-range of a block is one contiguous piece; block (r0, N) starts at element r0 * K."""
    M, K = w.shape
    out = torch.empty(M * K, dtype=w.dtype, device=w.device)
    full = M // BLOCK_ROWS
    if full:
        out[:full * BLOCK_ROWS * K] = (w[:full * BLOCK_ROWS].reshape(full, BLOCK_ROWS // 8, 8, K // 8, 8)
                                       .permute(0, 3, 1, 2, 4).reshape(-1))
    if M % BLOCK_ROWS:
        out[full * BLOCK_ROWS * K:] = pack_kc(w[full * BLOCK_ROWS:])
    return out


def pack_blocks_fp8(codes: torch.Tensor) -> torch.Tensor:
    """[M, K] e4m3 bytes -> flat: per block of 256 rows the layout [K/16][N/8][8 rows][16 k],
    which a 16-byte load turns into two adjacent bf16 pieces of the tensor-core operand layout."""
    M, K = codes.shape
    out = torch.empty(M * K, dtype=codes.dtype, device=codes.device)
    for r0, n in projection_blocks(M):
        out[r0 * K:(r0 + n) * K] = codes[r0:r0 + n].reshape(n // 8, 8, K // 16, 16).permute(2, 0, 1, 3).reshape(-1)
    return out


def pack_blocks_nvfp4(rows: torch.Tensor, K: int) -> torch.Tensor:
    """[M, K/2 + K/16] NVFP4 rows (e2m1 pairs, then the e4m3 block scales) -> flat: per block of 256 rows
    and per 16 inputs, the rows' 8 code bytes followed by the rows' scale bytes ([K/16][N x 8 | N]), so that
    any K-range of a block is one contiguous piece of 9 N bytes per 16 inputs."""
    M = rows.shape[0]
    codes, bs = rows[:, :K // 2].reshape(M, K // 16, 8), rows[:, K // 2:]
    out = torch.empty(M * K * 9 // 16, dtype=rows.dtype, device=rows.device)
    for r0, n in projection_blocks(M):
        blk = torch.cat((codes[r0:r0 + n].permute(1, 0, 2).reshape(K // 16, n * 8), bs[r0:r0 + n].t()), dim=1)
        out[r0 * K * 9 // 16:(r0 + n) * K * 9 // 16] = blk.reshape(-1)
    return out


def chunk_geometry(N: int, Bpad: int, K: int):
    """(Kc, G): inputs per W chunk (N * Kc * 2 bytes <= 32 KB, Kc divides K) and W chunks per X chunk
    (the X chunk fills at most one 8 KB slot when it can)."""
    kc = 256 if N <= 64 else 128 if N <= 128 else 64
    while K % kc or Bpad * kc * 2 > 16384:
        kc //= 2
    assert kc >= 16
    return kc, max(1, min(4, 8192 // (Bpad * kc * 2)))


def plan_units(blocks, steps: int, sms, load, step_bytes_per_row: int):
    """Deals the (block, W chunk) steps of a projection to the SMs, in `sms` order, as contiguous
    ranges of about equal bytes.  Returns [(sm, block index, first chunk, chunk count)]."""
    remaining = sum(n for _, n in blocks) * steps     # in rows x steps
    units, bi, ci = [], 0, 0
    for i, sm in enumerate(sms):
        quota = -(-remaining // (len(sms) - i))
        got = 0
        while bi < len(blocks) and got < quota:
            n = blocks[bi][1]
            take = min(max(1, round((quota - got) / n)), steps - ci)
            units.append((sm, bi, ci, take))
            got += take * n
            ci += take
            if ci == steps:
                bi, ci = bi + 1, 0
        remaining -= got
        load[sm] += got * step_bytes_per_row
    assert bi == len(blocks) and remaining == 0
    return units


def emit_projection(P: Program, *, sms, load, w_addr, M, K, x_addr, B, Bpad, mode, out_addr, scratch_addr,
                    counter_addr, x_wait=None, release=None, norm_addr=None, eps=0.0, ld=0, keys_addr=0, stats_addr=0,
                    wfmt="bf16", scales_addr=0):
    """Emits every unit of the projection y[B, M] = x[B, K] W^T (W packed by pack_blocks at w_addr,
    x k-chunk-major at x_addr).  scratch_addr: fp32 [blocks][B][256]; counter_addr: int32 [blocks]."""
    blocks = projection_blocks(M)
    Kc, G = chunk_geometry(blocks[0][1], Bpad, K)
    wb16 = {"bf16": 32, "fp8": 16, "nvfp4": 9}[wfmt]       # bytes per 16 weights of one row
    units = plan_units(blocks, K // Kc, sms, load, Kc * wb16 // 16)
    slices = [0] * len(blocks)
    for _, bi, _, _ in units:
        slices[bi] += 1
    if release is not None:
        P.add_releases(release, len(blocks))
    for sm, bi, c0, cnt in units:
        r0, N = blocks[bi]
        k0 = c0 * Kc
        P.gemm_tc(sm, w_addr=w_addr + (r0 * K + k0 * N) * wb16 // 16, N=N, K=K, k_len=cnt * Kc, Kc=Kc, G=G,
                  wfmt=wfmt, scales_addr=scales_addr + 4 * r0 if scales_addr else 0,
                  x_addr=x_addr + k0 * Bpad * 2, B=B, Bpad=Bpad, out_addr=out_addr, mode=mode, x_wait=x_wait,
                  norm_w=Src(norm_addr + k0 * 2, cnt * Kc * 2) if norm_addr is not None else None, eps=eps, n0=r0,
                  ld=ld, keys_addr=keys_addr, stats_addr=stats_addr, release=release,
                  scratch_addr=scratch_addr + bi * B * BLOCK_ROWS * 4, counter_addr=counter_addr + 4 * bi,
                  n_slices=slices[bi])
    return units


class BatchDecodeEngine(DecodeEngine):
    """`batch` sequences decoded together, one kernel launch per step.  Dense models; the layer
    projections are bf16, e4m3 with per-row scales (wkind "fp8") or NVFP4 (wkind "nvfp4": e2m1 values, e4m3 block
    scales, fp32 tensor scale), everything else bf16."""
    GEMV_PROJECTIONS = False
    FULL_KERNEL = True       # the attention variants for long page walks live in the full kernel only
    SHARED_CACHE = False     # True: the batch rows are consecutive positions of ONE sequence (prefill.PrefillEngine)
    WITH_VOCAB_PROJECTION = True   # False: the program ends after the last layer (prefill chunks before the last)

    def __init__(self, cfg: DecodeConfig, batch: int, max_seq: int, device="cuda:0", num_sms=None, taps=False,
                 page_perm_seed=None, max_steps: int = 256, timeout_ns: int = 2_000_000_000, wkind: str = "bf16"):
        assert 1 <= batch <= 128 and not cfg.n_experts and wkind in ("bf16", "fp8", "nvfp4")
        self.batch = batch
        self.bpad = next(p for p in (16, 32, 64, 128) if batch <= p)
        super().__init__(cfg, max_seq, device=device, num_sms=num_sms, taps=False, page_perm_seed=None,
                         max_steps=max_steps, timeout_ns=timeout_ns, wkind=wkind)
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
        if self.SHARED_CACHE and cfg.group == 4:      # split records of two positions x four heads (eight query rows)
            self.attn_part_pair = z((B + 1) // 2, cfg.n_kv_heads, self.n_splits, 8 * isa.HEAD_DIM + 16, dt=torch.float32)
        self.attn_cnt = z(L, B, cfg.n_kv_heads, dt=torch.int32)
        self.state_words = isa.ST_PAGETABLE + self.max_pages
        self.state = z(B, self.state_words, dt=torch.int32)
        self.state_host = torch.zeros(B, self.state_words, dtype=torch.int32).pin_memory()
        self.token_log = z(B, max_steps, dt=torch.int32)
        self._alloc_cache(page_perm_seed)
        self.taps_enabled = taps
        if taps:
            assert Bp * H * 2 <= 32768, "taps copy the hidden matrix with one bulk load"
            self.taps = z(L, Bp * H)
        self._cur = 0
        self.positions = [0] * B

    def _alloc_cache(self, page_perm_seed):
        """Paged pools and page tables: every sequence owns max_pages pages of one pool."""
        cfg, B, L = self.cfg, self.batch, self.cfg.n_layers
        z = lambda *s: torch.zeros(*s, dtype=BF16, device=self.dev)
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

    # ------------------------------------------------------------------ weights
    def load_weights(self, w):
        self._pack_cache = None         # packed copies of the previous weights
        super().load_weights(w)

    def init_random_weights(self, seed: int = 0, std: float = 0.02):
        self._pack_cache = None
        super().init_random_weights(seed, std)

    def weight_bytes(self) -> int:
        ts = [self.lm_head, self.norm_w, self.ln1, self.ln2, self.wqkv, self.wo, self.wgu, self.wd]
        ts += list(self.scales.values())
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
        # fp32 scratch / counters per projection kind and the packed weights outlive a rebuild of the program
        self.scratch = getattr(self, "scratch", None) or {}
        self._pack_cache = getattr(self, "_pack_cache", None) or {}

        stat = lambda i: self.stats[i].data_ptr()

        def gemm_stage(w, name, K, x_addr, x_wait, mode, out_addr, release, norm=None, ld=0, keys=0, stats=0):
            M = w.shape[0]
            wf = self.wkind if name is not None else "bf16"     # the vocabulary projection stays bf16
            fp8 = wf != "bf16"
            key = (name, len(packed[name]) if name is not None else 0)
            if key not in self._pack_cache:     # a second program of the same engine (prefill) shares the packed copies
                self._pack_cache[key] = (pack_blocks_fp8(w) if wf == "fp8" else pack_blocks_nvfp4(w, K) if wf == "nvfp4"
                                         else pack_blocks(w))
            pk = self._pack_cache[key]
            if name is not None:
                packed[name].append(pk)
            kind = name or "lm"
            n_blocks = len(projection_blocks(M))
            if kind not in self.scratch:      # fp32 partial sums and arrival counters, zero between uses
                self.scratch[kind] = (torch.zeros(n_blocks * B * BLOCK_ROWS, dtype=torch.float32, device=self.dev),
                                      torch.zeros(n_blocks, dtype=torch.int32, device=self.dev))
            scr, cnt = self.scratch[kind]
            sms = sorted(range(S), key=lambda i: (load[i], i))
            emit_projection(P, sms=sms, load=load, w_addr=pk.data_ptr(), M=M, K=K, x_addr=x_addr, B=B, Bpad=Bp,
                            mode=mode, out_addr=out_addr, scratch_addr=scr.data_ptr(), counter_addr=cnt.data_ptr(),
                            x_wait=x_wait, release=release, norm_addr=norm.data_ptr() if norm is not None else None,
                            eps=cfg.eps, ld=ld, keys_addr=keys, stats_addr=stats, wfmt=wf,
                            scales_addr=self.scales[name][len(packed[name]) - 1].data_ptr() if fp8 else 0)
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
            P.add_releases(b_merge, (B // 2 if self.SHARED_CACHE and G == 4 and B % 2 == 0 else B) * cfg.n_kv_heads)
            units = [(b, h, s) for s in range(self.n_splits) for b in range(B) for h in range(cfg.n_kv_heads)]
            kp, vp = self.kpool[l].data_ptr(), self.vpool[l].data_ptr()
            grp = (G + 2) * D * 2
            b_rows = None
            if self.SHARED_CACHE:
                # the rows of all the chunk's positions go to the pools first: position p attends to rows the
                # tasks of positions < p write in this same launch
                b_rows = P.new_barrier()
                P.add_releases(b_rows, B * cfg.n_kv_heads)
                for (b, h), sm in zip([(b, h) for b in range(B) for h in range(cfg.n_kv_heads)],
                                      self._pick(load, B * cfg.n_kv_heads)):
                    sb = st + 4 * sw * b
                    P.attn_decode(
                        sm, G=G, state_addr=sb,
                        rope=Src(self.rope.data_ptr(), D * 4, indirect=(sb + 4 * isa.ST_POS, 9, None)),
                        norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                        qkv=Src(qkv + (b * self.qkv_rows) * 2 + h * grp, grp, wait=b_qkv),
                        k_page_addr=kp + h * page_bytes, v_page_addr=vp + h * page_bytes, page_shift=page_shift,
                        base_page=0, max_pages=0, records_addr=0, counter_addr=0, out_addr=0, split=0, n_splits=1,
                        release=b_rows, qk_eps=cfg.qk_norm_eps, append=True)
            pairs = self.SHARED_CACHE and G == 4 and B % 2 == 0
            if pairs:
                # two consecutive prompt positions per unit: half the units walk the same pages (prefill only)
                units = [(b, h, s) for s in range(self.n_splits) for b in range(0, B, 2) for h in range(cfg.n_kv_heads)]
            for (b, h, s), sm in zip(units, self._pick(load, len(units), 2 * page_bytes * self.pages_per_split)):
                sb = st + 4 * sw * b
                if pairs:
                    P.attn_decode(
                        sm, G=8, state_addr=sb, pair=(sw, self.qkv_rows),
                        rope=Src(self.rope.data_ptr(), D * 4, indirect=(sb + 4 * isa.ST_POS, 9, None)),
                        norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                        qkv=Src(qkv + (b * self.qkv_rows) * 2 + h * grp, grp, wait=b_rows), wait_issue=b_rows,
                        k_page_addr=kp + h * page_bytes, v_page_addr=vp + h * page_bytes, page_shift=page_shift,
                        base_page=s * self.pages_per_split, max_pages=self.pages_per_split,
                        records_addr=self.attn_part_pair[b // 2, h].data_ptr(),
                        counter_addr=self.attn_cnt[l, b, h].data_ptr(),
                        out_addr=ao + (h * G * D) * Bp * 2, split=s, n_splits=self.n_splits, release=b_merge,
                        qk_eps=cfg.qk_norm_eps, packed=(b, Bp))
                    continue
                P.attn_decode(
                    sm, G=G, state_addr=sb,
                    rope=Src(self.rope.data_ptr(), D * 4, indirect=(sb + 4 * isa.ST_POS, 9, None)),
                    norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                    qkv=Src(qkv + (b * self.qkv_rows) * 2 + h * grp, grp, wait=b_qkv if b_rows is None else b_rows),
                    wait_issue=b_rows,
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
        if self.WITH_VOCAB_PROJECTION:
            b_lm = P.new_barrier()
            self.lm_head_packed = gemm_stage(self.lm_head, None, H, hid, b_hid, isa.GEMM_MODE_ARGMAX, 0, b_lm,
                                             norm=self.norm_w, keys=self.keys.data_ptr(), stats=stat(2 * L))
            if self.taps_enabled:
                tap(L - 1, b_hid, b_lm)
        else:
            b_lm = b_hid        # a prefill chunk that is not the prompt's last: nobody reads its logits
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
                pool[pt[:n_pages]] = kv_page_swizzle(
                    pad.view(n_pages, isa.KV_PAGE, cfg.n_kv_heads, isa.HEAD_DIM).permute(0, 2, 1, 3))

    def read_kv(self, layer: int, T: int, b: int = 0):
        n_pages = (T + isa.KV_PAGE - 1) // isa.KV_PAGE
        pt = self.page_tables[b].long().to(self.dev)[:n_pages]
        out = []
        for pool in (self.kpool[layer], self.vpool[layer]):
            t = kv_page_swizzle(pool[pt]).permute(0, 2, 1, 3).reshape(n_pages * isa.KV_PAGE, self.cfg.n_kv_heads, isa.HEAD_DIM)
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
