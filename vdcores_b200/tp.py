"""Tensor- and expert-parallel batch-1 decode: one process per GPU, the model split the
Megatron way — QKV and gate/up by output rows (heads / FFN columns), O and down
by input columns, vocabulary rows of the lm_head — with an all-reduce (sum) of
the fp32 partial hidden-state update after the O projection and after the down
projection of every layer, over NCCL (`torch.distributed`).

Mixture-of-experts layers are expert parallel: every rank keeps n_experts / world
consecutive experts whole, computes the router and the top-k selection on the
replicated hidden state, runs only the selected experts it owns (the others'
tasks see a chunk count of zero and stream nothing) and adds their weighted
outputs into its fp32 partial sum, which the same all-reduce combines.

The reference has no multi-GPU path at all; this is new.  Each rank runs the
same megakernel tasks as the single-GPU engine on its shard.  A layer becomes
two launches (attention half, MLP half) separated by the collectives; the whole
step is replayed as one CUDA graph when capture is available.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from . import isa, runtime
from .decode import BF16, DecodeConfig, DecodeEngine, DenseWeights, kv_page_swizzle, rows_per_chunk
from .program import Dst, Program, Src


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n].contiguous()


def shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[1] // world
    return t[:, rank * n:(rank + 1) * n].contiguous()


def kv_layout(cfg: DecodeConfig, rank: int, world: int):
    """(first KV head, KV heads, query heads per KV head) of a rank.  With more ranks than KV
    heads a KV head is replicated over world / n_kv_heads consecutive ranks, each of which
    takes a share of its query heads."""
    if cfg.n_kv_heads % world == 0:
        nkv = cfg.n_kv_heads // world
        return rank * nkv, nkv, cfg.group
    assert world % cfg.n_kv_heads == 0, "ranks must divide, or be a multiple of, the KV heads"
    rep = world // cfg.n_kv_heads
    assert cfg.group % rep == 0 and cfg.group // rep in (4, 8), "query heads per KV head and rank must be 4 or 8"
    return rank // rep, 1, cfg.group // rep


def shard_kv_rows(cfg: DecodeConfig, t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    h0, nkv, _ = kv_layout(cfg, rank, world)
    d = cfg.head_dim
    return t[h0 * d:(h0 + nkv) * d].contiguous()


def shard_dense_weights(cfg: DecodeConfig, w: DenseWeights, rank: int, world: int) -> DenseWeights:
    """The rank's shard in the usual [out, in] layout: q/k/v by heads, gate/up by
    FFN rows, o/down by input columns, lm_head by vocabulary rows; embedding and
    norms replicated."""
    assert cfg.n_heads % world == 0 and cfg.ffn % world == 0 and cfg.vocab % world == 0
    L = cfg.n_layers
    if cfg.n_experts:
        assert cfg.n_experts % world == 0
        e0, e1 = rank * cfg.n_experts // world, (rank + 1) * cfg.n_experts // world
        return DenseWeights(
            embed=w.embed, lm_head=shard_rows(w.lm_head, rank, world), norm=w.norm, ln1=w.ln1, ln2=w.ln2,
            wq=[shard_rows(w.wq[l], rank, world) for l in range(L)],
            wk=[shard_kv_rows(cfg, w.wk[l], rank, world) for l in range(L)],
            wv=[shard_kv_rows(cfg, w.wv[l], rank, world) for l in range(L)],
            wo=[shard_cols(w.wo[l], rank, world) for l in range(L)],
            gate=[w.gate[l][e0:e1] for l in range(L)], up=[w.up[l][e0:e1] for l in range(L)],
            down=[w.down[l][e0:e1] for l in range(L)], router=w.router,
            q_norm=w.q_norm, k_norm=w.k_norm)
    return DenseWeights(
        embed=w.embed, lm_head=shard_rows(w.lm_head, rank, world), norm=w.norm, ln1=w.ln1, ln2=w.ln2,
        wq=[shard_rows(w.wq[l], rank, world) for l in range(L)],
        wk=[shard_kv_rows(cfg, w.wk[l], rank, world) for l in range(L)],
        wv=[shard_kv_rows(cfg, w.wv[l], rank, world) for l in range(L)],
        wo=[shard_cols(w.wo[l], rank, world) for l in range(L)],
        gate=[shard_rows(w.gate[l], rank, world) for l in range(L)],
        up=[shard_rows(w.up[l], rank, world) for l in range(L)],
        down=[shard_cols(w.down[l], rank, world) for l in range(L)],
        q_norm=w.q_norm, k_norm=w.k_norm)


class TPDecodeEngine:
    def __init__(self, cfg: DecodeConfig, max_seq: int, rank: int, world: int, device, group=None,
                 max_steps: int = 4096, timeout_ns: int = 0, use_graph: bool = True):
        assert cfg.n_heads % world == 0 and cfg.ffn % world == 0 and cfg.vocab % world == 0
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        self.dev = torch.device(device)
        self.max_seq = max_seq
        self.max_pages = (max_seq + isa.KV_PAGE - 1) // isa.KV_PAGE
        self.max_steps, self.timeout_ns, self.use_graph = max_steps, timeout_ns, use_graph
        self.num_sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        self.stream = torch.cuda.current_stream(self.dev)
        runtime.init()
        D = isa.HEAD_DIM
        # this rank's KV heads and the query heads it serves per KV head (a KV head is replicated
        # when there are more ranks than KV heads)
        self.kv0, self.nkv, self.G = kv_layout(cfg, rank, world)
        G = self.G
        self.nq = cfg.n_heads // world
        assert self.nq == self.nkv * G
        self.F = cfg.ffn // world
        self.V = cfg.vocab // world
        self.qw, self.kvw = self.nq * D, self.nkv * D
        assert self.nkv & (self.nkv - 1) == 0 and self.qw % 256 == 0 and (cfg.n_experts or self.F % 256 == 0)
        L, H = cfg.n_layers, cfg.hidden
        z = lambda *s, dt=BF16: torch.zeros(*s, dtype=dt, device=self.dev)
        self.hidden = z(H)
        self.qkv = z(self.qw + 2 * self.kvw)
        self.attn_out = z(self.qw)
        self.act = z(self.F)
        self.partial = z(H, dt=torch.float32)
        self.logits = z(self.V)
        if cfg.n_experts:
            assert cfg.n_experts % world == 0 and cfg.top_k <= 16
            self.E_local = cfg.n_experts // world
            self.act = z(cfg.top_k, cfg.ffn)
            self.router_logits = z(cfg.n_experts, dt=torch.float32)
            self.route = z(64, dt=torch.int32)      # int32 ids[16] | fp32 weights[16] | int32 local[16] | int32 count[16]
        self.rec_floats = G * D + 16 * ((2 * G + 15) // 16)
        self.n_splits = max(1, min(self.num_sms // self.nkv, self.max_pages))
        # a page costs about a microsecond on the tensor cores, one more split record costs the merge a load
        # per output: with few KV heads per rank two pages per unit beat one
        self.pages_per_split = max(2, (self.max_pages + self.n_splits - 1) // self.n_splits)
        self.n_splits = (self.max_pages + self.pages_per_split - 1) // self.pages_per_split
        self.attn_part = z(self.nkv, self.n_splits, self.rec_floats, dt=torch.float32)
        self.attn_cnt = z(L, self.nkv, dt=torch.int32)
        self.argmax_rec = z(self.num_sms, 4, dt=torch.float32)
        self.best_local = z(4, dt=torch.float32)
        self.best_all = z(world, 4, dt=torch.float32)
        self.state = z(isa.ST_PAGETABLE + self.max_pages, dt=torch.int32)
        self.state_host = torch.zeros(isa.ST_PAGETABLE + self.max_pages, dtype=torch.int32).pin_memory()
        self.token_log = z(max_steps, dt=torch.int32)
        self.kpool = z(L, self.max_pages, self.nkv, isa.KV_PAGE, D)
        self.vpool = z(L, self.max_pages, self.nkv, isa.KV_PAGE, D)
        self.page_table = torch.arange(self.max_pages, dtype=torch.int32)
        pos = torch.arange(max_seq, dtype=torch.float32)
        inv = 1.0 / (cfg.theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        fr = pos[:, None] * inv[None, :]
        self.rope = torch.cat((fr.cos().to(BF16).float(), fr.sin().to(BF16).float()), dim=1).contiguous().to(self.dev)
        self.bars = z(isa.MAX_BARS, dt=torch.int32)
        self.profile = z(self.num_sms * isa.NUM_PROFILE_EVENTS, dt=torch.int64)
        self.programs = []
        self.graph = None
        self.pos = 0
        self.steps_done = 0
        self.launches_per_step = 2 * L + 2

    # ------------------------------------------------------------------ weights
    def load_shard(self, w: DenseWeights):
        """Takes this rank's shard (see shard_dense_weights) and builds the programs."""
        cfg, dev = self.cfg, self.dev
        L, G, D = cfg.n_layers, self.G, isa.HEAD_DIM
        to = lambda t: t.to(device=dev, dtype=BF16).contiguous()
        self.embed = to(w.embed)
        self.lm_head = to(w.lm_head)
        self.norm_w = to(w.norm)
        self.ln1 = torch.stack([to(t) for t in w.ln1])
        self.ln2 = torch.stack([to(t) for t in w.ln2])
        perm = []
        for h in range(self.nkv):
            perm += list(range(h * G * D, (h + 1) * G * D))
            perm += list(range(self.qw + h * D, self.qw + (h + 1) * D))
            perm += list(range(self.qw + self.kvw + h * D, self.qw + self.kvw + (h + 1) * D))
        pm = torch.tensor(perm, dtype=torch.long, device=dev)
        self.wqkv = torch.stack([torch.cat((to(w.wq[l]), to(w.wk[l]), to(w.wv[l])), dim=0)[pm] for l in range(L)])
        self.wo = torch.stack([to(w.wo[l]) for l in range(L)])
        if cfg.n_experts:
            # this rank's experts: [L, E_local, 2F, H] with gate/up rows interleaved, [L, E_local, H, F]
            self.wgu = torch.stack([torch.stack([torch.stack((to(g), to(u)), dim=1).reshape(2 * cfg.ffn, cfg.hidden)
                                                 for g, u in zip(w.gate[l], w.up[l])]) for l in range(L)])
            self.wd = torch.stack([torch.stack([to(d) for d in w.down[l]]) for l in range(L)])
            self.router = torch.stack([to(t) for t in w.router])
            self.qknorm = (torch.stack([torch.cat((to(w.q_norm[l]), to(w.k_norm[l]))) for l in range(L)])
                           if cfg.qk_norm else None)
            self._build_programs()
            return
        self.wgu = torch.stack([torch.stack((to(w.gate[l]), to(w.up[l])), dim=1).reshape(2 * self.F, cfg.hidden)
                                for l in range(L)])
        self.wd = torch.stack([to(w.down[l]) for l in range(L)])
        self.qknorm = (torch.stack([torch.cat((to(w.q_norm[l]), to(w.k_norm[l]))) for l in range(L)])
                       if cfg.qk_norm else None)
        self._build_programs()

    def weight_bytes(self) -> int:
        ts = [self.lm_head, self.norm_w, self.ln1, self.ln2, self.wqkv, self.wo]
        if self.qknorm is not None:
            ts.append(self.qknorm)
        n = sum(t.numel() * t.element_size() for t in ts) + self.cfg.hidden * 2
        if self.cfg.n_experts:
            # a token reads the router and, on average over a uniform router, top_k / world of this rank's experts
            n += self.router.numel() * 2
            n += (self.wgu.numel() + self.wd.numel()) * 2 * self.cfg.top_k // self.cfg.n_experts
        else:
            n += sum(t.numel() * t.element_size() for t in (self.wgu, self.wd))
        return n

    def algorithmic_bytes(self, pos: int) -> int:
        """Per-GPU HBM bytes of one step: this rank's weights once, one embedding
        row, its share of the KV cache."""
        return self.weight_bytes() + 2 * self.kvw * 2 * (pos + 1) * self.cfg.n_layers

    # ------------------------------------------------------------------ programs
    def _ranges(self, load, n_units: int, unit_bytes: int):
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
        return out

    def _finish(self, P: Program):
        n = max(max(len(x) for x in P.m), max(len(x) for x in P.c)) + 2
        P.insts_per_sm = ((n + 15) // 16) * 16
        c, m, bars = P.finalize()
        self.programs.append((torch.from_numpy(c).to(self.dev), torch.from_numpy(m).to(self.dev),
                              torch.from_numpy(bars).to(self.dev), P.insts_per_sm))

    def _build_programs(self):
        cfg = self.cfg
        L, H, G, D, S = cfg.n_layers, cfg.hidden, self.G, isa.HEAD_DIM, self.num_sms
        st = self.state.data_ptr()
        page_bytes = isa.KV_PAGE * D * 2
        page_shift = int(math.log2(self.nkv * page_bytes))
        hid, qkv, ao, act, part = (t.data_ptr() for t in (self.hidden, self.qkv, self.attn_out, self.act, self.partial))
        self.programs = []
        load = [0] * S
        for l in range(L):
            # ---- attention half: QKV (local heads) -> attention -> O projection over the local columns
            P = Program(S)
            b_qkv, b_merge = P.new_barrier(), P.new_barrier()
            R = rows_per_chunk(H)
            rows = self.qw + 2 * self.kvw
            for sm, u0, cnt in self._ranges(load, rows // R, R * H * 2):
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wqkv[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2),
                       out=Dst(qkv + r0 * 2, n * 2, "store", release=b_qkv),
                       norm_w=Src(self.ln1[l].data_ptr(), H * 2), eps=cfg.eps)
            P.add_releases(b_merge, self.nkv)
            units = [(h, s) for s in range(self.n_splits) for h in range(self.nkv)]
            order = sorted(range(S), key=lambda s: (load[s], s))
            grp = (G + 2) * D * 2
            for i, (h, s) in enumerate(units):
                sm = order[i % S]
                P.attn_decode(
                    sm, G=G, state_addr=st,
                    rope=Src(self.rope.data_ptr(), D * 4, indirect=(st + 4 * isa.ST_POS, 9, None)),
                    norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                    qkv=Src(qkv + h * grp, grp, wait=b_qkv),
                    k_page_addr=self.kpool[l].data_ptr() + h * page_bytes,
                    v_page_addr=self.vpool[l].data_ptr() + h * page_bytes, page_shift=page_shift,
                    base_page=s * self.pages_per_split, max_pages=self.pages_per_split,
                    records_addr=self.attn_part[h].data_ptr(), counter_addr=self.attn_cnt[l, h].data_ptr(),
                    out_addr=ao + h * G * D * 2, split=s, n_splits=self.n_splits, release=b_merge,
                    qk_eps=cfg.qk_norm_eps)
            K = self.qw
            R = rows_per_chunk(K)
            for sm, u0, cnt in self._ranges(load, H // R, R * K * 2):
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wo[l].data_ptr() + r0 * K * 2, n_rows=n, K=K, R=R,
                       x=Src(ao, K * 2, wait=b_merge), out=Dst(part + r0 * 4, n * 4, "store"),
                       mode=isa.GEMV_MODE_STORE_F32)
            self._finish(P)
            if cfg.n_experts:
                self._build_moe_half(l, load)
                continue
            # ---- MLP half: gate/up over the local FFN rows -> down over the local columns
            P = Program(S)
            b_gu = P.new_barrier()
            R = rows_per_chunk(H, even=True)
            for sm, u0, cnt in self._ranges(load, 2 * self.F // R, R * H * 2):
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wgu[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2),
                       out=Dst(act + (r0 // 2) * 2, n, "store", release=b_gu), mode=isa.GEMV_MODE_SILU_PAIRS,
                       norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps)
            K = self.F
            R = rows_per_chunk(K)
            for sm, u0, cnt in self._ranges(load, H // R, R * K * 2):
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wd[l].data_ptr() + r0 * K * 2, n_rows=n, K=K, R=R,
                       x=Src(act, K * 2, wait=b_gu), out=Dst(part + r0 * 4, n * 4, "store"),
                       mode=isa.GEMV_MODE_STORE_F32)
            self._finish(P)
        # ---- vocabulary shard: candidates per SM, then this rank's best as one record
        P = Program(S)
        b_logits = P.new_barrier()
        R = rows_per_chunk(H)
        lm = self._ranges(load, self.V // R, R * H * 2)
        for i, (sm, u0, cnt) in enumerate(lm):
            r0, n = u0 * R, cnt * R
            P.gemv(sm, w_addr=self.lm_head.data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2),
                   out=Dst(self.logits.data_ptr() + r0 * 2, n * 2, "store", release=b_logits),
                   mode=isa.GEMV_MODE_ARGMAX, norm_w=Src(self.norm_w.data_ptr(), H * 2), eps=cfg.eps,
                   pair_out=Dst(self.argmax_rec[i].data_ptr(), 16, release=b_logits), row_base=self.rank * self.V + r0)
        P.argmax_final(0, records=Src(self.argmax_rec.data_ptr(), len(lm) * 16, wait=b_logits), n=len(lm),
                       state_addr=st, log_addr=self.best_local.data_ptr(), local_only=True)
        self._finish(P)
        # ---- global winner among the ranks' records, token log, state advance (identical on every rank)
        P = Program(1)
        P.argmax_final(0, records=Src(self.best_all.data_ptr(), self.world * 16), n=self.world, state_addr=st,
                       log_addr=self.token_log.data_ptr())
        self._finish(P)

    def _build_moe_half(self, l: int, load):
        """Router and selection on the replicated hidden state, then the selected experts this
        rank owns: gate/up with fused norm and SiLU-mul, down projections added (times the
        routing weight) into the fp32 partial sum, which the host zeroes before the launch."""
        cfg = self.cfg
        H, F, E, TK, S = cfg.hidden, cfg.ffn, cfg.n_experts, cfg.top_k, self.num_sms
        hid, part = self.hidden.data_ptr(), self.partial.data_ptr()
        ids = self.route.data_ptr()
        wts, lid, cnt = ids + 64, ids + 128, ids + 192
        P = Program(S)
        b_rl, b_route, b_gu = P.new_barrier(), P.new_barrier(), P.new_barrier()
        R = rows_per_chunk(H)
        for sm, u0, n_u in self._ranges(load, E // R, R * H * 2):
            r0, n = u0 * R, n_u * R
            P.gemv(sm, w_addr=self.router[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2),
                   out=Dst(self.router_logits.data_ptr() + r0 * 4, n * 4, "store", release=b_rl),
                   mode=isa.GEMV_MODE_STORE_F32, norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps)
        sm = min(range(S), key=lambda i: (load[i], i))
        P.moe_route(sm, logits=Src(self.router_logits.data_ptr(), E * 4, wait=b_rl), route_addr=ids, n_experts=E,
                    top_k=TK, release=b_route, rank=self.rank, world=self.world)
        # units are (slot, chunk), contiguous per SM, split at slot borders
        R = rows_per_chunk(H, even=True)
        per = 2 * F // R
        for sm, u0, n_u in self._ranges(load, TK * per, R * H * 2 // max(1, self.world)):
            u, end = u0, u0 + n_u
            while u < end:
                slot, c0 = divmod(u, per)
                n_c = min(end - u, per - c0)
                r0, n = c0 * R, n_c * R
                P.gemv(sm, w_addr=self.wgu[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2),
                       out=Dst(self.act[slot].data_ptr() + (r0 // 2) * 2, n, "store", release=b_gu),
                       mode=isa.GEMV_MODE_SILU_PAIRS, norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps,
                       w_indirect=(lid + 4 * slot, 2 * F * H * 2), wait_issue=b_route, dyn_count_addr=cnt + 4 * slot)
                u += n_c
        R = rows_per_chunk(F)
        per = H // R
        for sm, u0, n_u in self._ranges(load, TK * per, R * F * 2 // max(1, self.world)):
            u, end = u0, u0 + n_u
            while u < end:
                slot, c0 = divmod(u, per)
                n_c = min(end - u, per - c0)
                r0, n = c0 * R, n_c * R
                P.gemv(sm, w_addr=self.wd[l].data_ptr() + r0 * F * 2, n_rows=n, K=F, R=R,
                       x=Src(self.act[slot].data_ptr(), F * 2, wait=b_gu), out=Dst(part + r0 * 4, n * 4, "store"),
                       mode=isa.GEMV_MODE_MOE_DOWN, w_indirect=(lid + 4 * slot, H * F * 2), wait_issue=b_route,
                       dyn_count_addr=cnt + 4 * slot,
                       moe=dict(weight_addr=wts + 4 * slot, acc_addr=0, cnt_addr=0, top_k=TK))
                u += n_c
        self._finish(P)

    # ------------------------------------------------------------------ state / cache
    def set_state(self, pos: int, token: int):
        s = self.state_host
        s.zero_()
        page = pos // isa.KV_PAGE
        s[isa.ST_POS], s[isa.ST_NPAGES], s[isa.ST_TOKEN] = pos, page + 1, token
        s[isa.ST_NEWROW] = int(self.page_table[page]) * isa.KV_PAGE * self.nkv + pos % isa.KV_PAGE
        s[isa.ST_NKVH], s[isa.ST_MAXPAGES] = self.nkv, self.max_pages
        s[isa.ST_PAGETABLE:] = self.page_table
        self.state.copy_(s, non_blocking=True)
        self.attn_cnt.zero_()
        self.pos, self.steps_done = pos, 0

    def load_kv(self, k: List[torch.Tensor], v: List[torch.Tensor]):
        """Per-layer contiguous caches [T, n_kv_heads (all), 128]: keeps this rank's heads."""
        h0 = self.kv0
        for l in range(self.cfg.n_layers):
            for src, pool in ((k[l], self.kpool[l]), (v[l], self.vpool[l])):
                T = src.shape[0]
                n_pages = (T + isa.KV_PAGE - 1) // isa.KV_PAGE
                pad = torch.zeros(n_pages * isa.KV_PAGE, self.nkv, isa.HEAD_DIM, dtype=BF16, device=self.dev)
                pad[:T] = src[:, h0:h0 + self.nkv].to(self.dev)
                pool[:n_pages] = kv_page_swizzle(pad.view(n_pages, isa.KV_PAGE, self.nkv, isa.HEAD_DIM).permute(0, 2, 1, 3))

    # ------------------------------------------------------------------ decode
    def _launch(self, i: int):
        c, m, b0, n = self.programs[i]
        num_sms = 1 if i == len(self.programs) - 1 else self.num_sms
        # the stream that is current now: inside a graph capture that is the capturing stream
        runtime.launch_async(num_sms, n, c, m, None, self.bars, b0, self.profile,
                             torch.cuda.current_stream(self.dev).cuda_stream, self.timeout_ns)

    def _all_reduce_add(self):
        dist.all_reduce(self.partial, group=self.group)
        self.hidden.add_(self.partial)           # bf16(hidden + fp32 sum of the ranks' partial products)

    def _step_body(self):
        L = self.cfg.n_layers
        tok = self.state[isa.ST_TOKEN:isa.ST_TOKEN + 1].long()
        torch.index_select(self.embed, 0, tok, out=self.hidden.view(1, -1))
        for l in range(L):
            self._launch(2 * l)
            self._all_reduce_add()
            if self.cfg.n_experts:
                self.partial.zero_()         # the experts' down projections add into it
            self._launch(2 * l + 1)
            self._all_reduce_add()
        self._launch(2 * L)
        dist.all_gather_into_tensor(self.best_all.view(-1), self.best_local, group=self.group)
        self._launch(2 * L + 1)

    def step_async(self):
        if self.pos >= self.max_seq or self.steps_done >= self.max_steps:
            raise RuntimeError("out of KV pages or token-log space")
        if self.use_graph and self.graph is None and self.steps_done >= 2:
            # two eager steps first (NCCL sets up its channels on first use), then capture one step
            try:
                torch.cuda.synchronize(self.dev)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step_body()
                self.graph = g
                # the captured step has not run: fall through and replay it below
            except Exception as e:           # capture not available: stay eager
                self.use_graph = False
                self.graph_error = repr(e)
                torch.cuda.synchronize(self.dev)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step_body()
        self.pos += 1
        self.steps_done += 1

    def step_host(self, token: int) -> int:
        """One step from host buffers: token id up, next id down (synchronous)."""
        if not hasattr(self, "_tok_in"):
            self._tok_in = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._tok_out = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._tok_in[0] = token
        self.state[isa.ST_TOKEN:isa.ST_TOKEN + 1].copy_(self._tok_in, non_blocking=True)
        idx = self.steps_done
        self.step_async()
        self._tok_out.copy_(self.token_log[idx:idx + 1], non_blocking=True)
        torch.cuda.synchronize(self.dev)
        return int(self._tok_out[0])

    def load_from_full(self, full: DecodeEngine, cached_positions: int):
        """Takes this rank's shard out of a single-GPU engine that holds the whole
        model (packed layout) and its KV cache for `cached_positions` positions."""
        r, cfg = self.rank, self.cfg
        D = isa.HEAD_DIM
        self.embed, self.norm_w, self.ln1, self.ln2 = full.embed, full.norm_w, full.ln1, full.ln2
        self.lm_head = full.lm_head[r * self.V:(r + 1) * self.V].contiguous()
        # the full engine stores [group's query heads | key | value] per KV head; this rank keeps, for each
        # of its KV heads, its share of the query heads and the key / value rows
        grp_rows = (cfg.group + 2) * D
        q_share = (r % max(1, self.world // cfg.n_kv_heads)) * self.G * D if self.world > cfg.n_kv_heads else 0
        idx = []
        for h in range(self.kv0, self.kv0 + self.nkv):
            base = h * grp_rows
            idx += list(range(base + q_share, base + q_share + self.G * D))
            idx += list(range(base + cfg.group * D, base + (cfg.group + 2) * D))
        self.wqkv = full.wqkv[:, torch.tensor(idx, dtype=torch.long, device=full.wqkv.device)].contiguous()
        self.wo = full.wo[:, :, r * self.qw:(r + 1) * self.qw].contiguous()
        if cfg.n_experts:
            e0 = r * self.E_local
            self.wgu = full.wgu[:, e0:e0 + self.E_local].contiguous()
            self.wd = full.wd[:, e0:e0 + self.E_local].contiguous()
            self.router = full.router
        else:
            self.wgu = full.wgu[:, r * 2 * self.F:(r + 1) * 2 * self.F].contiguous()
            self.wd = full.wd[:, :, r * self.F:(r + 1) * self.F].contiguous()
        self.qknorm = full.qknorm
        ks, vs = [], []
        for l in range(cfg.n_layers):
            k, v = full.read_kv(l, cached_positions)
            ks.append(k)
            vs.append(v)
        self.load_kv(ks, vs)
        self._build_programs()

    def close(self):
        """Drops the captured step (it holds NCCL kernels) before the process group
        is destroyed; call on every rank, then barrier, then destroy."""
        torch.cuda.synchronize(self.dev)
        self.graph = None
        torch.cuda.synchronize(self.dev)

    def generate(self, n_steps: int) -> List[int]:
        first = self.steps_done
        for _ in range(n_steps):
            self.step_async()
        torch.cuda.synchronize(self.dev)
        runtime.read_status(self.stream.cuda_stream)
        return self.token_log[first:first + n_steps].tolist()


class TPFusedEngine(TPDecodeEngine):
    """Tensor-parallel decode of a dense model with the exchange inside the kernel: one launch
    per step and rank, no collective library call in the step.  Every rank owns an exchange
    block (allocated by the library, mapped by all ranks through CUDA IPC); the row-split
    projections (O, down) store their fp32 partial rows into every rank's block as tagged
    8-byte entries {value, exchange tag} with plain peer stores over NVLink; an XREDUCE task
    per slice of the hidden state polls the entries of its slice and folds the ranks' partial
    sums into the replicated hidden state as soon as the last one lands — no fence, counter
    or collective stands between a partial row and its consumers.  The vocabulary shard's
    best candidate travels the same way.  Bounded waits throughout: a rank that never
    arrives makes the others time out and report, not hang."""

    SLICE = 128     # hidden elements per XREDUCE task

    def __init__(self, *args, **kw):
        kw["use_graph"] = False
        super().__init__(*args, **kw)
        assert not self.cfg.n_experts, "the fused exchange covers dense models"
        H, Pn, L = self.cfg.hidden, self.world, self.cfg.n_layers
        # exchange block of tagged 8-byte entries {payload, tag}: xbuf[2][ranks][H] | best[ranks][value, row index]
        self.n_ex = 2 * L + 1                       # exchanges per step: two per layer and the vocabulary winner
        self.off_best = 2 * Pn * H * 8
        n_bytes = self.off_best + Pn * 16
        # the block is an allocation of its own made by the library, so that its CUDA IPC handle names exactly it
        with torch.cuda.device(self.dev):
            self._block = runtime.PeerBlock((n_bytes + 255) // 256 * 256)
            self.xchg = self._block.tensor(torch.float32)
        self._peer_mappings = []
        bases = [0] * Pn
        bases[self.rank] = self._block.ptr
        if Pn > 1:
            handles = [None] * Pn
            dist.all_gather_object(handles, (self.dev.index, self._block.handle), group=self.group)
            # a rank that cannot map a peer still takes part in the agreement below, so that all ranks give up
            # together instead of one leaving the others at a barrier
            error = None
            try:
                for r in range(Pn):
                    if r == self.rank:
                        continue
                    peer_dev, handle = handles[r]
                    if not torch.cuda.can_device_access_peer(self.dev.index, peer_dev):
                        raise RuntimeError(f"device {self.dev.index} has no peer access to device {peer_dev}")
                    with torch.cuda.device(self.dev):      # mapped with THIS device current: its kernels store there
                        bases[r] = runtime.ipc_open(handle)
                    self._peer_mappings.append(bases[r])
            except Exception as e:     # noqa: BLE001 (reported below, on every rank)
                error = e
            torch.cuda.synchronize(self.dev)
            agreed = torch.tensor([0 if error else 1], dtype=torch.int32, device=self.dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)
            if int(agreed.item()) == 0:
                self.close()
                raise RuntimeError(f"exchange blocks could not be mapped on every rank (this rank: {error!r})")
        # what the sending tasks read: every rank's block, then this rank's state block (for the step number)
        self.peer_table = torch.tensor(bases + [self.state.data_ptr()], dtype=torch.int64, device=self.dev)
        self.best_rec = torch.zeros(Pn, 4, dtype=torch.int32, device=self.dev)
        self.launches_per_step = 1

    # ------------------------------------------------------------------ program
    def _build_programs(self):
        cfg = self.cfg
        L, H, G, D, S, Pn = cfg.n_layers, cfg.hidden, self.G, isa.HEAD_DIM, self.num_sms, self.world
        st = self.state.data_ptr()
        page_bytes = isa.KV_PAGE * D * 2
        page_shift = int(math.log2(self.nkv * page_bytes))
        hid, qkv, ao, act = (t.data_ptr() for t in (self.hidden, self.qkv, self.attn_out, self.act))
        xb = self.xchg.data_ptr()
        table = self.peer_table.data_ptr()
        load = [0] * S
        P = Program(S, insts_per_sm=isa.MAX_INSTS)

        def exchange(half: int, release: int):
            """XREDUCE tasks for exchange number `half` (two per layer), one per slice of the hidden state."""
            par = half & 1
            order = sorted(range(S), key=lambda s: (load[s], s))
            for i, e0 in enumerate(range(0, H, self.SLICE)):
                n = min(self.SLICE, H - e0)
                P.xreduce(order[i % S], n=n, n_ranks=Pn, xbuf_addr=xb + (par * Pn * H + e0) * 8, hidden_elems=H,
                          ex=half, n_ex=self.n_ex, hidden_addr=hid + e0 * 2, state_addr=st, release=release)

        def peers(half: int):
            return (table, Pn, half, self.n_ex)

        def my_slot(half: int, r0: int) -> int:
            return (((half & 1) * Pn + self.rank) * H + r0) * 8      # byte offset of an entry inside an exchange block

        # ---- embedding row of the current token into the hidden state
        b_hid = P.new_barrier()
        sm0 = 0
        P.copy(sm0, Src(self.embed.data_ptr(), H * 2, indirect=(st + 4 * isa.ST_TOKEN, None, H * 2)),
               Dst(hid, H * 2, release=b_hid), H * 2)
        for l in range(L):
            b_qkv, b_merge = P.new_barrier(), P.new_barrier()
            R = rows_per_chunk(H)
            rows = self.qw + 2 * self.kvw
            for sm, u0, cnt in self._ranges(load, rows // R, R * H * 2):
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wqkv[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2, wait=b_hid),
                       out=Dst(qkv + r0 * 2, n * 2, "store", release=b_qkv),
                       norm_w=Src(self.ln1[l].data_ptr(), H * 2), eps=cfg.eps)
            P.add_releases(b_merge, self.nkv)
            units = [(h, s) for s in range(self.n_splits) for h in range(self.nkv)]
            order = sorted(range(S), key=lambda s: (load[s], s))
            grp = (G + 2) * D * 2
            for i, (h, s) in enumerate(units):
                P.attn_decode(
                    order[i % S], G=G, state_addr=st,
                    rope=Src(self.rope.data_ptr(), D * 4, indirect=(st + 4 * isa.ST_POS, 9, None)),
                    norm_w=Src(self.qknorm[l].data_ptr(), 2 * D * 2) if cfg.qk_norm else None,
                    qkv=Src(qkv + h * grp, grp, wait=b_qkv),
                    k_page_addr=self.kpool[l].data_ptr() + h * page_bytes,
                    v_page_addr=self.vpool[l].data_ptr() + h * page_bytes, page_shift=page_shift,
                    base_page=s * self.pages_per_split, max_pages=self.pages_per_split,
                    records_addr=self.attn_part[h].data_ptr(), counter_addr=self.attn_cnt[l, h].data_ptr(),
                    out_addr=ao + h * G * D * 2, split=s, n_splits=self.n_splits, release=b_merge,
                    qk_eps=cfg.qk_norm_eps)
            # ---- O projection over the local columns: partial rows to every rank, then the exchange
            K = self.qw
            R = rows_per_chunk(K)
            tasks = self._ranges(load, H // R, R * K * 2)
            for sm, u0, cnt in tasks:
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wo[l].data_ptr() + r0 * K * 2, n_rows=n, K=K, R=R, x=Src(ao, K * 2, wait=b_merge),
                       out=Dst(my_slot(2 * l, r0), n * 8, "store"), mode=isa.GEMV_MODE_STORE_F32, peers=peers(2 * l))
            b_h1 = P.new_barrier()
            exchange(2 * l, b_h1)
            # ---- gate/up over the local FFN rows, down over the local columns
            b_gu = P.new_barrier()
            R = rows_per_chunk(H, even=True)
            for sm, u0, cnt in self._ranges(load, 2 * self.F // R, R * H * 2):
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wgu[l].data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2, wait=b_h1),
                       out=Dst(act + (r0 // 2) * 2, n, "store", release=b_gu), mode=isa.GEMV_MODE_SILU_PAIRS,
                       norm_w=Src(self.ln2[l].data_ptr(), H * 2), eps=cfg.eps)
            K = self.F
            R = rows_per_chunk(K)
            tasks = self._ranges(load, H // R, R * K * 2)
            for sm, u0, cnt in tasks:
                r0, n = u0 * R, cnt * R
                P.gemv(sm, w_addr=self.wd[l].data_ptr() + r0 * K * 2, n_rows=n, K=K, R=R, x=Src(act, K * 2, wait=b_gu),
                       out=Dst(my_slot(2 * l + 1, r0), n * 8, "store"), mode=isa.GEMV_MODE_STORE_F32,
                       peers=peers(2 * l + 1))
            b_hid = P.new_barrier()
            exchange(2 * l + 1, b_hid)
        # ---- vocabulary shard, this rank's best candidate to every rank, global winner
        b_logits = P.new_barrier()
        R = rows_per_chunk(H)
        lm = self._ranges(load, self.V // R, R * H * 2)
        for i, (sm, u0, cnt) in enumerate(lm):
            r0, n = u0 * R, cnt * R
            P.gemv(sm, w_addr=self.lm_head.data_ptr() + r0 * H * 2, n_rows=n, K=H, R=R, x=Src(hid, H * 2, wait=b_hid),
                   out=Dst(self.logits.data_ptr() + r0 * 2, n * 2, "store", release=b_logits),
                   mode=isa.GEMV_MODE_ARGMAX, norm_w=Src(self.norm_w.data_ptr(), H * 2), eps=cfg.eps,
                   pair_out=Dst(self.argmax_rec[i].data_ptr(), 16, release=b_logits), row_base=self.rank * self.V + r0)
        last = 2 * L
        P.argmax_final(0, records=Src(self.argmax_rec.data_ptr(), len(lm) * 16, wait=b_logits), n=len(lm),
                       state_addr=st, log_addr=self.off_best + 16 * self.rank, local_only=True, peers=peers(last))
        b_best = P.new_barrier()
        P.xwait(0, n_ranks=Pn, ex=last, n_ex=self.n_ex, entries_addr=xb + self.off_best, state_addr=st,
                records_addr=self.best_rec.data_ptr(), release=b_best)
        P.argmax_final(0, records=Src(self.best_rec.data_ptr(), Pn * 16, wait=b_best), n=Pn, state_addr=st,
                       log_addr=self.token_log.data_ptr())
        n = max(max(len(x) for x in P.m), max(len(x) for x in P.c)) + 2
        P.insts_per_sm = ((n + 63) // 64) * 64
        c, m, bars = P.finalize()
        self.program = P
        self.programs = [(torch.from_numpy(c).to(self.dev), torch.from_numpy(m).to(self.dev),
                          torch.from_numpy(bars).to(self.dev), P.insts_per_sm)]

    # ------------------------------------------------------------------ state / decode
    def set_state(self, pos: int, token: int):
        super().set_state(pos, token)
        # the arrival counters count from step 0 again; nobody may still be writing
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.xchg.zero_()
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier(group=self.group)

    def _step_body(self):
        c, m, b0, n = self.programs[0]
        runtime.launch_async(self.num_sms, n, c, m, None, self.bars, b0, self.profile,
                             torch.cuda.current_stream(self.dev).cuda_stream, self.timeout_ns)

    def close(self):
        """Unmaps the other ranks' blocks, waits for every rank to have done so, then frees this rank's."""
        torch.cuda.synchronize(self.dev)
        with torch.cuda.device(self.dev):
            for base in self._peer_mappings:
                runtime.ipc_close(base)
        self._peer_mappings = []
        if self.world > 1:
            dist.barrier(group=self.group)
        self.xchg = None
        if self._block is not None:
            self._block.free()
            self._block = None
