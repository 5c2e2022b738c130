#!/usr/bin/env python
"""Decode benchmark: tokens/s at batch 1 on the Llama-3.1-8B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode step (one megakernel launch) after a 2048-token
prompt has been prefilled into the paged KV cache.  Weights are random
N(0, 0.02) bf16 of the named shape, the prompt is uniform random ids (synthetic
stand-ins for a checkpoint and a dataset; there is no network).  Prints ONE
JSON line.  `value` is timed with the state resident on the device; `e2e` goes
through the host-buffer step API (token id up, next id down, every step).
`--impl reference` times the CPU oracle of the same math on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 2048
METRIC = "decode tokens/s at batch 1 (Llama-3.1-8B shape)"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index = index
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.3)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.lines = []
        if self.proc is not None:
            time.sleep(0.1)
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
                self.lines = [l for l in out.splitlines() if l.strip()]
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in getattr(self, "lines", []):
            f = [x.strip() for x in l.split(",")]
            try:
                sm.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except Exception:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [x for x in sm if x > 0.5 * mx] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def oracle_cfg(model, wkind):
    from oracle import decode_oracle as O
    import dataclasses
    base = {"llama31-8b": O.LLAMA31_8B, "qwen3-8b": O.QWEN3_8B, "qwen3-30b-a3b": O.QWEN3_30B_A3B}[model]
    return dataclasses.replace(base, wkind=wkind)


def cpu_oracle_tokens_per_s(model="llama31-8b", wkind="bf16", n_layers_sample=2, steps=2, threads=None,
                            budget_s=25.0):
    """Times the CPU oracle (the reference's PyTorch decode math) on a bounded sample of the workload:
    `n_layers_sample` layers of the named shape plus the final norm and vocabulary projection, up to
    `steps` decode steps at the prompt length, stopping early once `budget_s` is spent.  The layer
    time is scaled to the model's depth.  Returns (tokens/s, threads, description, steps timed)."""
    import dataclasses
    import torch
    from oracle import decode_oracle as O
    threads = threads or os.cpu_count()
    torch.set_num_threads(threads)
    full = oracle_cfg(model, wkind)
    n_layers_sample = min(n_layers_sample, full.n_layers)
    cfg = dataclasses.replace(full, n_layers=n_layers_sample)
    if cfg.n_experts:
        cfg = dataclasses.replace(cfg, n_experts=max(cfg.top_k, 16))   # a token touches top_k experts: 16 are enough to draw from
    gen = torch.Generator().manual_seed(0)
    layers = [O.LayerWeights.random(cfg, gen) for _ in range(n_layers_sample)]
    lm_head = O.randn_bf16(gen, cfg.vocab, cfg.hidden)
    norm = torch.ones(cfg.hidden, dtype=torch.bfloat16)
    T = PROMPT_LEN + steps + 1
    kc = [O.randn_bf16(gen, T, cfg.n_kv_heads, cfg.head_dim, std=1.0) for _ in layers]
    vc = [O.randn_bf16(gen, T, cfg.n_kv_heads, cfg.head_dim, std=1.0) for _ in layers]
    h0 = O.randn_bf16(gen, cfg.hidden, std=1.0)
    O.FAST_LINEAR = True        # bf16 kernels of the host BLAS, fp32 accumulation inside them

    def one(pos):
        h = h0
        t0 = time.perf_counter()
        for i, lw in enumerate(layers):
            h = O.decode_layer(cfg, lw, h, pos, kc[i], vc[i])
        t1 = time.perf_counter()
        logits = O.linear(O.rms_norm(h, norm, cfg.eps)[None], lm_head)[0]
        int(torch.argmax(logits.float()))
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1
    one(PROMPT_LEN)                                   # warm-up
    tl, th = [], []
    t_start = time.perf_counter()
    for s in range(steps):
        a, b = one(PROMPT_LEN + 1 + s)
        tl.append(a)
        th.append(b)
        if time.perf_counter() - t_start > budget_s:
            break
    per_token = statistics.mean(tl) / n_layers_sample * full.n_layers + statistics.mean(th)
    desc = (f"{model} shape, {wkind}: {n_layers_sample} of {full.n_layers} layers + final norm/lm_head/argmax, "
            f"{len(tl)} steps at context {PROMPT_LEN}, layer time scaled x{full.n_layers / n_layers_sample:g}, "
            f"host BLAS bf16 linears (FAST_LINEAR)")
    return 1.0 / per_token, threads, desc, len(tl)


def run_reference(args):
    """The reference arm: its PyTorch decode math on the host CPU (rank 0 only).  Every step of the
    arm is a bounded sample: `layers` of the model's layers are run and the layer time is scaled."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    global PROMPT_LEN
    PROMPT_LEN = {"llama31-8b": 2048, "qwen3-8b": 4096, "qwen3-30b-a3b": 1024}[args.model]
    sample_layers = 8 if args.model == "llama31-8b" else 4
    tps, cores, sample, timed = cpu_oracle_tokens_per_s(args.model, args.wkind, n_layers_sample=sample_layers,
                                                        steps=max(1, args.steps), budget_s=60.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": timed, "steps_requested": args.steps, "warmup": 1, "ms_per_step": 1000.0 / tps,
        "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": args.wkind, "data": "synthetic",
        "config": {"workload": f"{args.model} shape, {args.wkind}, batch 1, {PROMPT_LEN}-token prompt, greedy decode",
                   "timing": "CPU oracle of the reference's PyTorch decode math; each step is a bounded sample "
                             "(see cpu_baseline.sample), stopped after 60 s of timed steps"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def dbg(msg):
    if os.environ.get("VDC_BENCH_DEBUG"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from vdcores_b200 import runtime
    from vdcores_b200.decode import LLAMA31_8B, DecodeEngine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K, W = args.steps, max(args.warmup, 3)
    import dataclasses
    from vdcores_b200.decode import QWEN3_8B
    from vdcores_b200.decode import QWEN3_30B_A3B
    cfg = {"llama31-8b": LLAMA31_8B, "qwen3-8b": QWEN3_8B, "qwen3-30b-a3b": QWEN3_30B_A3B}[args.model]
    global PROMPT_LEN
    PROMPT_LEN = {"llama31-8b": 2048, "qwen3-8b": 4096, "qwen3-30b-a3b": 1024}[args.model]
    if args.layers != 32:
        cfg = dataclasses.replace(cfg, n_layers=args.layers)
    max_seq = ((PROMPT_LEN + max(W + K, 32) + 8 + 63) // 64) * 64      # 32: steps of the sharded engines' agreement check
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (PROMPT_LEN,), generator=g)
    prefill_info = {"impl": "PyTorch ops (library GEMMs)", "prompt_tokens": PROMPT_LEN}
    tf, tp_fallback = None, None
    if world == 1 and args.batch > 1:
        # batched decode: the projections run on the tensor cores, one state block per sequence
        from vdcores_b200.batch import BatchDecodeEngine
        eng = BatchDecodeEngine(cfg, args.batch, max_seq=max_seq, device=dev, max_steps=W + K + 8, wkind=args.wkind)
        eng.init_random_weights(seed=0)
        prompt = torch.randint(0, cfg.vocab, (args.batch, PROMPT_LEN), generator=g)
        first = eng.prefill(prompt)
        tokens_per_step, scaling, parallelism = args.batch, "strong", "single GPU"
    elif world == 1:
        eng = DecodeEngine(cfg, max_seq=max_seq, device=dev, max_steps=W + K + 8, wkind=args.wkind)
        eng.init_random_weights(seed=0)
        first, prefill_info = run_prefill(eng, prompt, args.prefill == "device")
        tokens_per_step, scaling, parallelism = 1, "strong", "single GPU"
    else:
        # tensor parallel: every rank builds the same full model (same seed), prefills it with the
        # PyTorch path, keeps its shard of the weights and of the KV cache, and drops the rest
        from vdcores_b200.tp import TPDecodeEngine, TPFusedEngine
        N_CHECK = 32
        full = DecodeEngine(cfg, max_seq=max_seq, device=dev, max_steps=max(W + K, N_CHECK) + 8)
        full.init_random_weights(seed=0)
        first, prefill_info = run_prefill(full, prompt, args.prefill == "device")
        if "ms" in prefill_info:
            # The megakernel prefill adds the K-slices of a projection block with fp32 atomics: the cache is not
            # bit-identical from one GPU to the next, and a random-init model turns the last bits into other greedy
            # ids.  Every rank's shard and every rank's single-GPU trajectory must come from one cache: rank 0's.
            t = torch.tensor([first], dtype=torch.int64, device=dev)
            for buf in (full.kpool, full.vpool, t):
                dist.broadcast(buf, 0)
            first = int(t)
            full.set_state(PROMPT_LEN, first)
        # dense models: one launch per step and rank, the partial sums cross NVLink as peer stores inside the
        # kernel; mixture-of-experts models (and --tp-impl nccl): two launches per layer around NCCL collectives
        fused = args.tp_impl == "fused" and not cfg.n_experts
        kw = dict(max_seq=max_seq, rank=rank, world=world, device=dev, max_steps=2 * (W + K) + 16 + N_CHECK)
        eng = None
        if fused:
            try:
                eng = TPFusedEngine(cfg, **kw)
            except RuntimeError as e:          # raised on every rank together: no peer mapping on this machine
                dbg(f"in-kernel exchange unavailable, using the NCCL engine: {e}")
                fused = False
        if eng is None:
            eng = TPDecodeEngine(cfg, **kw)
        dbg('prefill done')
        eng.load_from_full(full, PROMPT_LEN)
        dbg('shard loaded')
        # The single-GPU engine every rank still holds decodes the same prompt: its greedy ids and, per step, the gap
        # between its two largest logits.  The sharded engine is then checked teacher-forced (fed the single-GPU ids, so
        # both see the same sequence) below: a random-init model has near-ties, and a free-running comparison would stop
        # meaning anything after the first one.
        full.set_state(PROMPT_LEN, first)
        single_gpu_tokens, single_gpu_gaps = [], []
        for _ in range(N_CHECK):
            single_gpu_tokens += full.generate(1)
            top2 = torch.topk(full.logits.float(), 2).values
            single_gpu_gaps.append(float((top2[0] - top2[1]) / top2[0].abs().clamp_min(1e-6)))

        def teacher_forced(e):
            # The two engines round differently (the sharded one adds fp32 partial sums to the residual, the single-GPU
            # one a bf16 projection output), which moves bf16 logits by a few ulps (0.4 % each): ids may differ only
            # where the single-GPU engine's two best logits are closer than 5 % of the best one
            e.set_state(PROMPT_LEN, first)
            feed, agree, beyond, worst = first, 0, [], 0.0
            for i in range(N_CHECK):
                got = e.step_host(feed)
                agree += int(got == single_gpu_tokens[i])
                if got != single_gpu_tokens[i]:
                    worst = max(worst, single_gpu_gaps[i])
                    if single_gpu_gaps[i] > 0.05:
                        beyond.append(i)
                feed = single_gpu_tokens[i]
            return {"steps": N_CHECK, "agree": agree, "disagree_beyond_near_ties": len(beyond),
                    "max_rel_gap_at_a_disagreement": worst}

        # ---- teacher-forced agreement with the single-GPU engine (untimed).  The in-kernel exchange has to pass it on
        # every rank; if a launch gives up a wait (a bounded wait returns a status, the context stays usable) or the
        # ids disagree beyond near-ties on any rank, all ranks switch to the NCCL engine together and say so.
        tf, tp_fallback = None, None
        if fused:
            ok = 1
            try:
                tf = teacher_forced(eng)
                ok = int(tf["disagree_beyond_near_ties"] == 0)
            except RuntimeError as e:
                dbg(f"in-kernel exchange failed a step: {e}")
                ok = 0
            if os.environ.get("VDCORES_BENCH_FAIL_EXCHANGE_CHECK"):     # exercises the switch-over (host-side injection)
                ok = 0
            flag = torch.tensor([ok], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag) == 0:
                tp_fallback = "the in-kernel exchange did not pass the agreement check on this machine; NCCL engine used"
                dbg(tp_fallback)
                retired = eng             # kept alive: its peer mappings are torn down at exit, not mid-run
                fused, tf = False, None
                eng = TPDecodeEngine(cfg, **kw)
                eng.load_from_full(full, PROMPT_LEN)
        if tf is None:
            tf = teacher_forced(eng)
        del full
        torch.cuda.empty_cache()
        tokens_per_step, scaling = 1, "strong"
        parallelism = ((f"tp{world}, in-kernel exchange over peer memory" if fused else f"tp{world}, NCCL collectives")
                       if not cfg.n_experts else f"attention tp{world}, experts ep{world}, NCCL collectives")
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    batched = world == 1 and args.batch > 1

    def reset():
        if batched:
            for b in range(args.batch):
                eng.set_state(PROMPT_LEN, first[b], b=b)
        else:
            eng.set_state(PROMPT_LEN, first)

    # ---- device-resident arm: K launches back to back, CUDA events on the launching stream
    reset()
    for _ in range(W):
        eng.step_async()
    runtime.read_status(stream.cuda_stream)
    dbg(f'warm-up done, graph={getattr(eng, "graph", None) is not None} {getattr(eng, "graph_error", "")}')
    pos0 = eng.pos
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clk:
        torch.cuda.profiler.start()          # lets a profiler capture only the timed region
        e0.record(stream)
        for _ in range(K):
            eng.step_async()
        e1.record(stream)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    barrier()
    runtime.read_status(stream.cuda_stream)
    ms = e0.elapsed_time(e1)
    dbg(f'timed region done: {ms:.2f} ms')
    tokens = eng.token_log[0, W:W + K].tolist() if batched else eng.token_log[W:W + K].tolist()
    # ---- end-to-end arm: host token in, host token out, every step
    e2e_ms = float("nan")
    if not args.no_e2e:
        reset()
        tok = first
        for _ in range(W):
            tok = eng.step_host(tok)
        barrier()
        t0 = time.perf_counter()
        for _ in range(K):
            tok = eng.step_host(tok)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        barrier()
        e2e_ms = (t1 - t0) * 1000.0
    dbg('e2e done')
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if world > 1:
        # symmetric teardown on every rank: the captured step holds NCCL kernels
        eng.close()
        dist.barrier()
        dist.destroy_process_group()
        dbg('process group destroyed')
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    mid_pos = pos0 + K // 2
    bytes_per_launch = eng.algorithmic_bytes(mid_pos)
    achieved = bytes_per_launch / (ms / K * 1e-3) / 1e9
    line = {
        "metric": (METRIC if args.batch == 1 else METRIC.replace("batch 1", f"batch {args.batch}")) if args.model == "llama31-8b" else METRIC.replace("Llama-3.1-8B", {"qwen3-8b": "Qwen3-8B", "qwen3-30b-a3b": "Qwen3-30B-A3B"}[args.model]),
        "value": tokens_per_step * K / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": args.wkind, "data": "synthetic",
        "config": {"workload": (f"{args.model} shape ({cfg.n_layers} layers, hidden {cfg.hidden}, {cfg.n_heads}q/"
                                f"{cfg.n_kv_heads}kv heads, FFN {cfg.ffn}, vocab {cfg.vocab}), {args.wkind} projections, "
                                f"batch {args.batch}, {PROMPT_LEN}-token prompt{'s' if args.batch > 1 else ''} prefilled, greedy decode"),
                   "l2": f"inputs larger than L2: every step streams {bytes_per_launch / 1e9:.2f} GB per GPU through a 126 MB L2",
                   "parallelism": parallelism,
                   "num_sms": eng.num_sms, "kv_splits": eng.n_splits, "first_tokens": tokens[:4],
                   **({"layers": args.layers, "note": "reduced-depth profiling case, not a benchmark result"}
                      if args.layers != 32 else {})},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # dram__bytes_read+write per launch: ncu measured 1.006 x the algorithmic bytes on a
                     # 4-layer case of the same program (profiles/), scaled here by the bytes of this launch
                     "traffic": bytes_per_launch * 1.006 / 1e9, "traffic_unit": "GB", "peak_kind": f"of {peak_kind}", "frac_of_8TBs": achieved / 8000.0,
                     "bytes_per_launch": bytes_per_launch},
        "e2e": ({"value": tokens_per_step * K / (e2e_ms * 1e-3), "unit": "tokens/s",
                 "h2d_bytes_per_step": 4 * tokens_per_step, "d2h_bytes_per_step": 4 * tokens_per_step}
                if not args.no_e2e else None),
        "gpu_launches": K * eng.launches_per_step,
        "prefill": prefill_info,      # untimed set-up of the decode measurement; reported for the time to first token
        # greedy ids of the sharded engine, fed the single-GPU engine's ids, against that engine's next ids: true when
        # they agree on every step whose two best single-GPU logits are more than a near-tie apart
        **({"tokens_match_single_gpu": tf["disagree_beyond_near_ties"] == 0, "teacher_forced": tf} if tf else {}),
        **({"tp_fallback": tp_fallback} if tp_fallback else {}),
        "clocks": clk.summary(),
    }
    if not args.no_cpu_baseline:
        tps, cores, sample, _ = cpu_oracle_tokens_per_s(args.model, args.wkind, n_layers_sample=2, steps=3, budget_s=20.0)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line))


def run_prefill(eng, prompt, on_device):
    """Fills eng's KV pools with the prompt and returns (first generated id, what ran and how long it took)."""
    import torch
    T = int(prompt.numel())
    if not on_device:
        return eng.prefill(prompt), {"impl": "PyTorch ops (library GEMMs)", "prompt_tokens": T}
    if eng.cfg.n_experts:
        # mixture-of-experts models: the decode program itself over the prompt, one position per launch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first = eng.prefill_device(prompt)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return first, {"impl": "megakernel, one prompt position per launch (the decode program)", "prompt_tokens": T,
                       "ms": dt * 1e3, "tokens_per_s": T / dt, "launches": T}
    # the prompt goes through the megakernel too: 128 positions per launch into this engine's own pools
    from vdcores_b200.prefill import PrefillEngine
    pre = PrefillEngine(eng, chunk=128).adopt_weights()
    pre.prefill(prompt)                          # first call: one-time set-up of the kernel
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first = pre.prefill(prompt)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    del pre
    torch.cuda.empty_cache()
    return first, {"impl": "megakernel, 128 prompt positions per launch", "prompt_tokens": T, "ms": dt * 1e3,
                   "tokens_per_s": T / dt, "launches": (T + 127) // 128}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="vdcores_b200", choices=["vdcores_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer arm (profiling runs)")
    ap.add_argument("--wkind", default="bf16", choices=["bf16", "fp8", "nvfp4"],
                    help="storage of the layer projections (fp8: e4m3 + per-row fp32 scales; reported, not the headline)")
    ap.add_argument("--model", default="llama31-8b", choices=["llama31-8b", "qwen3-8b", "qwen3-30b-a3b"],
                    help="shape of the random-init model (qwen3-8b: 36 layers, FFN 12288, per-head QK norm, 4096-token prompt)")
    ap.add_argument("--batch", type=int, default=1,
                    help="sequences decoded in lock-step (> 1: tensor-core projections, bf16, one GPU)")
    ap.add_argument("--tp-impl", default="fused", choices=["fused", "nccl"],
                    help="N > 1, dense models: exchange inside the kernel (peer stores) or NCCL collectives between launches")
    ap.add_argument("--prefill", default="device", choices=["device", "torch"],
                    help="batch 1: prompt through the megakernel (device) or PyTorch ops (torch)")
    ap.add_argument("--layers", type=int, default=32,
                    help="profiling only: a model with fewer layers of the same shape (the JSON line says so)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
