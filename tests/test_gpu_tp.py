"""Tensor-parallel decode engine on a B200 against the CPU oracle.

With one GPU the engine runs as a one-rank NCCL group: that still exercises the
per-layer split into two launches, the fp32 partial outputs, the collectives and
the two-stage argmax.  With two or more GPUs a two-rank run is spawned as well."""
import os
import socket

import pytest
import torch

from oracle import decode_oracle as O
from tests.helpers import dense_weights, engine_config, perturb_norms, small_cfg

pytestmark = pytest.mark.gpu


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_rank(rank, world, port, n_steps, results, kind="llama", fused=False):
    import torch.distributed as dist
    from vdcores_b200.tp import TPDecodeEngine, TPFusedEngine, shard_dense_weights
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=dev)
    try:
        cfg = small_cfg(kind)
        w = perturb_norms(O.ModelWeights.random(cfg, seed=3))
        g = torch.Generator().manual_seed(11)
        prompt = torch.randint(0, cfg.vocab, (70,), generator=g)
        orc = O.DecodeOracle(w, 256)
        orc.prefill(prompt[:-1].tolist())
        ecfg = engine_config(cfg)
        cls = TPFusedEngine if fused else TPDecodeEngine
        eng = cls(ecfg, max_seq=256, rank=rank, world=world, device=dev, timeout_ns=1_000_000_000)
        eng.load_shard(shard_dense_weights(ecfg, dense_weights(w), rank, world))
        eng.load_kv([k[:69] for k in orc.k], [v[:69] for v in orc.v])
        tok = int(prompt[-1])
        eng.set_state(69, tok)
        out = []
        for step in range(n_steps):
            logits_ref, nxt_ref, gap = orc.step(tok)
            if fused and world > 1:
                dist.barrier()          # the ranks' launches start together: the in-kernel waits are bounded
            got = eng.generate(1)[0]
            V = cfg.vocab // world
            r = O.rel_l2(eng.logits.cpu(), logits_ref[rank * V:(rank + 1) * V])
            out.append((got, nxt_ref, gap, r))
            tok = nxt_ref
            if got != nxt_ref:
                eng.state[2:3].copy_(torch.tensor([tok], dtype=torch.int32))
        results[rank] = (out, eng.graph is not None, getattr(eng, "graph_error", None))
        eng.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def check(results, world, bar=1e-2):
    for rank in range(world):
        out, used_graph, err = results[rank]
        for step, (got, ref, gap, r) in enumerate(out):
            assert r < bar, f"rank {rank} step {step}: logits rel-L2 {r:.3e}"
            if gap > 1e-2:
                assert got == ref, f"rank {rank} step {step}: token {got} vs {ref}"
    # every rank logged the same tokens
    assert len({tuple(g for g, *_ in results[r][0]) for r in range(world)}) == 1


def test_tp_one_rank_group(cuda_device):
    results = {}
    run_rank(0, 1, free_port(), 5, results)
    check(results, 1)


def test_fused_exchange_one_rank(cuda_device):
    """The in-kernel exchange (peer stores, arrival counters, XREDUCE) with a single rank:
    one launch per step, no collective call in the step."""
    results = {}
    run_rank(0, 1, free_port(), 5, results, fused=True)
    check(results, 1)


def test_expert_parallel_one_rank_group(cuda_device):
    """The mixture-of-experts model through the expert-parallel path with one rank: router,
    selection, dynamically counted expert tasks, fp32 partial sum, collectives."""
    results = {}
    run_rank(0, 1, free_port(), 4, results, kind="moe")
    # sixteen random-init experts: a step whose router has two experts nearly tied at the top-k edge may pick the
    # other one than the oracle (both are right to rounding), which moves that step's logits by about 1e-2
    check(results, 1, bar=2e-2)


def _worker(rank, world, port, n_steps, q, kind="llama"):
    res = {}
    fused = kind == "llama-fused"
    run_rank(rank, world, port, n_steps, res, kind="llama" if fused else kind, fused=fused)
    q.put((rank, res[rank]))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind", ["llama", "llama-fused", "moe2", "moe"])
def test_tp_two_ranks(kind):
    """Two ranks: tensor parallel for the dense model, with the collectives ("llama") and with the exchange
    inside the kernel over mapped peer memory ("llama-fused"); attention tensor parallel and experts
    expert parallel (8 of 16 experts per rank) for the mixture-of-experts models — "moe" has a
    single KV head, which both ranks then hold, each serving four of its eight query heads."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 4, q, kind), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = dict(q.get(timeout=180) for _ in range(2))
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():      # a rank that never reported must not outlive the test
                p.kill()
    check(results, 2, bar=1e-2 if kind.startswith("llama") else 2e-2)
