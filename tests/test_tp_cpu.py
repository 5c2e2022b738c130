"""Host-side logic of the tensor-parallel split, with two gloo ranks on the CPU:
each rank evaluates one decode layer on its shard of the weights (plain torch
math on the shard tensors), partial hidden-state updates are all-reduced, and
the result must equal the oracle's full layer."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import decode_oracle as O
from tests.helpers import dense_weights, engine_config, perturb_norms, small_cfg


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, q):
    from vdcores_b200.tp import shard_dense_weights
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        cfg = small_cfg("llama")
        w = perturb_norms(O.ModelWeights.random(cfg, seed=5))
        ecfg = engine_config(cfg)
        sh = shard_dense_weights(ecfg, dense_weights(w), rank, world)
        g = torch.Generator().manual_seed(9)
        hidden = torch.randn(cfg.hidden, generator=g).to(torch.bfloat16)
        T, pos, d = 40, 40, cfg.head_dim
        kc = torch.randn(T + 1, cfg.n_kv_heads, d, generator=g).to(torch.bfloat16)
        vc = torch.randn(T + 1, cfg.n_kv_heads, d, generator=g).to(torch.bfloat16)
        nkv, nq = cfg.n_kv_heads // world, cfg.n_heads // world
        # --- this rank's half layer, on shard tensors only
        x = O.rms_norm(hidden, sh.ln1[0], cfg.eps)
        q_ = O.linear(x[None], sh.wq[0])[0].view(nq, d)
        k_ = O.linear(x[None], sh.wk[0])[0].view(nkv, d)
        v_ = O.linear(x[None], sh.wv[0])[0].view(nkv, d)
        cos, sin = O.rope_cos_sin(torch.tensor([pos]), d, cfg.theta)
        q_, k_ = O.apply_rope(q_, cos, sin), O.apply_rope(k_, cos, sin)
        kl = kc[:, rank * nkv:(rank + 1) * nkv].clone()
        vl = vc[:, rank * nkv:(rank + 1) * nkv].clone()
        kl[pos], vl[pos] = k_, v_
        attn = O.gqa_decode_attention(q_, kl, vl)
        part = attn.float() @ sh.wo[0].float().t()                 # fp32 partial over the local columns
        dist.all_reduce(part)
        h1 = hidden + part.to(torch.bfloat16)
        x2 = O.rms_norm(h1, sh.ln2[0], cfg.eps)
        a = O.silu_mul(O.linear(x2[None], sh.gate[0]), O.linear(x2[None], sh.up[0]))[0]
        part2 = a.float() @ sh.down[0].float().t()
        dist.all_reduce(part2)
        h2 = h1 + part2.to(torch.bfloat16)
        # --- the oracle's full layer
        kf, vf = kc.clone(), vc.clone()
        ref = O.decode_layer(cfg, w.layers[0], hidden, pos, kf, vf)
        q.put((rank, O.rel_l2(h2, ref), float((h2.float() - ref.float()).abs().max())))
    finally:
        dist.destroy_process_group()


def test_two_rank_split_reproduces_the_full_layer():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=120) for _ in range(2)]
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    for rank, r, mx in res:
        assert r < 3e-3, (rank, r, mx)


def test_shard_shapes():
    from vdcores_b200.tp import shard_dense_weights
    cfg = small_cfg("llama")
    w = O.ModelWeights.random(cfg, seed=1)
    ecfg = engine_config(cfg)
    for world in (1, 2):
        parts = [shard_dense_weights(ecfg, dense_weights(w), r, world) for r in range(world)]
        assert torch.equal(torch.cat([p.wq[0] for p in parts], 0), w.layers[0].wq.w)
        assert torch.equal(torch.cat([p.wo[1] for p in parts], 1), w.layers[1].wo.w)
        assert torch.equal(torch.cat([p.down[2] for p in parts], 1), w.layers[2].down.w)
        assert torch.equal(torch.cat([p.lm_head for p in parts], 0), w.lm_head)
        assert parts[0].gate[0].shape == (cfg.ffn // world, cfg.hidden)
    # more ranks than KV heads: the KV head is replicated, its query heads are shared out
    from vdcores_b200.tp import kv_layout
    cfg = small_cfg("moe")          # 8 query heads on 1 KV head
    w = O.ModelWeights.random(cfg, seed=2)
    ecfg = engine_config(cfg)
    parts = [shard_dense_weights(ecfg, dense_weights(w), r, 2) for r in range(2)]
    assert [kv_layout(ecfg, r, 2) for r in range(2)] == [(0, 1, 4), (0, 1, 4)]
    assert torch.equal(parts[0].wk[0], w.layers[0].wk.w) and torch.equal(parts[1].wv[1], w.layers[1].wv.w)
    assert torch.equal(torch.cat([p.wq[0] for p in parts], 0), w.layers[0].wq.w)
    assert len(parts[1].gate[0]) == cfg.n_experts // 2


def _ep_rank(rank, world, port, q):
    """Expert parallelism: every rank routes on the replicated hidden state, evaluates only the
    selected experts it owns and the weighted partial sums are all-reduced."""
    from vdcores_b200.tp import shard_dense_weights
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        cfg = small_cfg("moe2")
        w = perturb_norms(O.ModelWeights.random(cfg, seed=5))
        lw = w.layers[0]
        sh = shard_dense_weights(engine_config(cfg), dense_weights(w), rank, world)
        per = cfg.n_experts // world
        assert len(sh.gate[0]) == per and torch.equal(sh.gate[0][0], lw.experts[rank * per][0].w)
        g = torch.Generator().manual_seed(10)
        x = torch.randn(cfg.hidden, generator=g).to(torch.bfloat16)
        wts, idx = O.moe_route(x[None], sh.router[0], cfg.top_k)
        part = torch.zeros(cfg.hidden, dtype=torch.float32)
        n_local = 0
        for slot in range(cfg.top_k):
            e = int(idx[0, slot])
            if e // per != rank:
                continue                      # another rank's expert: this rank streams nothing for the slot
            n_local += 1
            le = e % per
            a = O.silu_mul(O.linear(x[None], sh.gate[0][le]), O.linear(x[None], sh.up[0][le]))
            part += O.linear(a, sh.down[0][le])[0].float() * wts[0, slot].float()
        dist.all_reduce(part)
        ref = O.moe_ffn(x, lw, cfg.top_k)
        q.put((rank, n_local, O.rel_l2(part.to(torch.bfloat16), ref)))
    finally:
        dist.destroy_process_group()


def test_two_rank_expert_parallel_sum_reproduces_the_moe_block():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_ep_rank, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=120) for _ in range(2)]
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    assert sum(n for _, n, _ in res) == small_cfg("moe2").top_k      # every selected expert has exactly one owner
    for rank, n_local, r in res:
        assert r < 3e-3, (rank, r)


def test_exchange_protocol_two_buffers_suffice():
    """Model of the in-kernel tensor-parallel exchange (TPFusedEngine): every rank writes the partial rows of
    exchange h as tagged entries {payload, tag = step * n_ex + h + 1} into slot [h % 2][rank] of every rank's
    block (one remote store per entry, in any order, no fence and no counter); a rank folds exchange h once every
    writer's entry in its own block carries that tag, and only then produces exchange h + 1.  Under random
    interleavings of the ranks and of each rank's individual remote writes, over several steps that reuse the
    exchange numbers: a fold never sees a payload of another exchange under the tag it waits for, no slot is
    overwritten before its owner has folded it, and nobody deadlocks."""
    import random
    for seed in range(200):
        rng = random.Random(seed)
        n_ranks, n_ex, n_steps = rng.choice([2, 3, 4, 8]), 5, 3
        total = n_ex * n_steps
        # [owner][parity][writer] -> (tag, payload); payload names the (global exchange, writer) it belongs to
        xbuf = [[[(0, None)] * n_ranks for _ in range(2)] for _ in range(n_ranks)]
        folded = [[-1] * 2 for _ in range(n_ranks)]          # last global exchange each owner folded, per parity
        state = [{"g": 0, "todo": None} for _ in range(n_ranks)]

        def tag_of(g):
            step, h = divmod(g, n_ex)
            return step * n_ex + h + 1

        def start(r):
            steps = [("write", p) for p in range(n_ranks)]
            rng.shuffle(steps)
            state[r]["todo"] = steps + [("fold", None)]

        for r in range(n_ranks):
            start(r)
        live = set(range(n_ranks))
        guard = 0
        while live:
            guard += 1
            assert guard < 200000, "deadlock in the model"
            r = rng.choice(sorted(live))
            g = state[r]["g"]
            kind, p = state[r]["todo"][0]
            if kind == "write":
                # the slot's previous content (exchange g - 2 of this writer) must have been folded by its owner
                old_tag, old = xbuf[p][g & 1][r]
                assert old is None or folded[p][g & 1] >= old[0], (seed, r, p, g, old)
                xbuf[p][g & 1][r] = (tag_of(g), (g, r))
                state[r]["todo"].pop(0)
                continue
            if any(t != tag_of(g) for t, _ in xbuf[r][g & 1]):
                continue                                 # bounded poll in the kernel; here: let another rank run
            assert all(pl == (g, w) for w, (_, pl) in enumerate(xbuf[r][g & 1])), (seed, r, g)
            folded[r][g & 1] = g
            state[r]["g"] = g + 1
            if g + 1 == total:
                live.discard(r)
            else:
                start(r)
