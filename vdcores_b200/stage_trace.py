"""Where the time of a batch-1 decode step goes: per-task and per-stage timelines from the kernel's own stamps.

    python -m vdcores_b200.stage_trace [--layers 4] [--prompt 2048] [--batch 1]

Every launch leaves, per SM, the global-timer start and end of its first 56 tasks in the profile rows; this
program decodes a few steps of a Llama-3.1-8B-shaped model with `--layers` layers (random weights), reads the
rows of the last step and prints SM 0's task list and, for the k-th GEMV / attention task of every SM, when the
first and last SM started and ended it (i.e. the stage and its skew).

With a library built by `python -m vdcores_b200.build --trace VDC_TRACE_ATTN` (or VDC_TRACE_GEMV) and selected
through VDCORES_LIB, the stamps inside the attention task (barrier seen, prologue, page arrivals, arrival at the
head's counter, merge) or inside the GEMV task are printed as well.  With --batch B > 1 the program is the batched
one (projections on the tensor cores); a library built with --trace VDC_TC_PROFILE adds where the projection task's
issuing warp and the task as a whole spend their cycles (sums per SM over one launch); one built with --trace
VDC_TRACE_CHUNKS prints the life of SM 0's ring entries --entries LO:HI (published by the control warp, copy issued
by the load port, seen by the consuming warp, slots given back)."""
import argparse
import collections
import dataclasses
import os

import numpy as np
import torch

from . import isa, runtime
from .decode import LLAMA31_8B, DecodeEngine

ATTN_LABELS = {0: "start", 1: "barrier seen", 2: "prologue done", 3: "K page 0", 4: "V page 0", 5: "page 0 done",
               6: "K page 1", 7: "V page 1", 8: "page 1 done", 11: "pages done", 12: "arrived", 13: "merged"}
GEMV_LABELS = ["task start", "pops done", "barrier open", "x ready", "phase begun", "last chunk done (thread 0)",
               "phase end", "released"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--entries", default="60:120", help="ring entries of SM 0 to list (VDC_TRACE_CHUNKS library)")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    cfg = dataclasses.replace(LLAMA31_8B, n_layers=args.layers)
    max_seq = ((args.prompt + 64 + 63) // 64) * 64
    if args.batch > 1:
        from .batch import BatchDecodeEngine
        eng = BatchDecodeEngine(cfg, args.batch, max_seq=max_seq, device=dev, max_steps=64)
        eng.init_random_weights(0)
        for b in range(args.batch):           # the cache contents do not matter for the timing: zero rows
            eng.set_state(args.prompt, 5 + b, b=b)
    else:
        eng = DecodeEngine(cfg, max_seq=max_seq, device=dev, max_steps=64)
        eng.init_random_weights(0)
        g = torch.Generator().manual_seed(0)
        first = eng.prefill(torch.randint(0, cfg.vocab, (args.prompt,), generator=g))
        eng.set_state(args.prompt, first)
    trace = os.environ.get("VDCORES_LIB", "")
    if "trace_chunks" in trace:               # that build stamps 1500 ring entries of SM 0 behind the per-SM rows
        eng.profile = torch.zeros(isa.MAX_SMS * isa.NUM_PROFILE_EVENTS + 1500 * 4, dtype=torch.int64, device=dev)
    for _ in range(args.steps - 1):
        eng.step_async()
    runtime.read_status(eng.stream.cuda_stream)
    eng.profile.zero_()                       # the cycle sums of the traced builds accumulate: keep one launch
    eng.step_async()
    runtime.read_status(eng.stream.cuda_stream)
    raw = eng.profile.cpu().numpy().astype(np.int64)
    pv = raw[:eng.num_sms * isa.NUM_PROFILE_EVENTS].reshape(eng.num_sms, -1)
    t0 = pv[:, 0].min()
    names = {v: k for k, v in isa.OPCODES.items()}
    print(f"{args.layers} layers, context {args.prompt}: kernel {(pv[:, 1].max() - t0) / 1e3:.1f} us, "
          f"CTA start skew {(pv[:, 0].max() - t0) / 1e3:.2f} us")
    rows = []
    n_traced = 24 if "trace_gemv" in trace else 56
    if "tc_profile" in trace:
        # the task stamps (rows 16 + 2 j) must stay clear of the projection task's sums in rows 100-106
        n_tasks = max(sum(1 for w in eng.program.c[sm] if w[0] not in (isa.OP_EXT, isa.OP_TERMINATEC))
                      for sm in range(eng.num_sms))
        assert n_tasks <= 42, f"{n_tasks} tasks on one SM: use fewer layers (--layers 2) with the VDC_TC_PROFILE library"
    for sm in range(eng.num_sms):
        ops = [w[0] for w in eng.program.c[sm] if w[0] not in (isa.OP_EXT, isa.OP_TERMINATEC)]
        for j, o in enumerate(ops[:n_traced]):
            rows.append((sm, j, o, (pv[sm, 16 + 2 * j] - t0) / 1e3, (pv[sm, 17 + 2 * j] - t0) / 1e3))
    print("SM 0 (us since kernel start):")
    for r in rows:
        if r[0] == 0 and r[1] < 20:
            print(f"   {r[1]:2d} {names.get(r[2], hex(r[2])):28s} {r[3]:8.1f} -> {r[4]:8.1f}  ({r[4] - r[3]:6.1f})")
    by = collections.defaultdict(list)
    for sm in range(eng.num_sms):
        k = collections.Counter()
        for r in rows:
            if r[0] == sm:
                by[(names.get(r[2], hex(r[2])), k[r[2]])].append(r)
                k[r[2]] += 1
    print("k-th task of a kind over all SMs: first/last start | first/last end | mean duration (us)")
    for key in sorted(by, key=lambda q: min(r[3] for r in by[q]))[:4 * args.layers + 6]:
        st = np.array([r[3] for r in by[key]])
        en = np.array([r[4] for r in by[key]])
        print(f"   {key[0]:26s}#{key[1]:2d} n={len(st):3d}  {st.min():7.1f} .. {st.max():7.1f} | {en.min():7.1f} .. {en.max():7.1f}"
              f" | {np.mean(en - st):6.1f}")
    if "trace_attn" in trace:
        a = []
        for sm in range(eng.num_sms):
            t = pv[sm, 100:114]
            if t[0]:
                a.append([(t[k] - t[0]) / 1e3 if t[k] >= t[0] else np.nan for k in sorted(ATTN_LABELS)])
        a = np.array(a)
        print("inside the attention task (us after its start; last attention task of every SM; median / min / max):")
        for i, k in enumerate(sorted(ATTN_LABELS)):
            col = a[:, i][~np.isnan(a[:, i])]
            if len(col):
                print(f"   {ATTN_LABELS[k]:16s} {np.median(col):6.2f} {col.min():6.2f} {col.max():6.2f}   (n={len(col)})")
    if "trace_chunks" in trace:
        lo, hi = (int(v) for v in args.entries.split(":"))
        ch = raw[isa.MAX_SMS * isa.NUM_PROFILE_EVENTS:][:6000].reshape(1500, 4)
        print("ring entries of SM 0: published (us since kernel start, +gap to the previous entry) | copy issued | "
              "seen by the consumer | slots given back (us after published; - = not stamped for this kind of entry)")
        prev = 0
        for n in range(1500):
            a = ch[n]
            if a[0] == 0:
                continue
            if lo <= n < hi:
                d = [f"{(x - a[0]) / 1e3:6.2f}" if x else "     -" for x in a[1:]]
                print(f"   {n:5d}  {(a[0] - t0) / 1e3:8.2f} (+{(a[0] - prev) / 1e3 if prev else 0:5.2f}) | {d[0]} | {d[1]} | {d[2]}")
            prev = a[0]
    if "tc_profile" in trace:
        clk = 1965.0      # SM cycles per microsecond at the clock the B200s of this pool run at
        print("projection task, microseconds per SM in this launch (issuing warp, then the whole task):")
        for row, label in ((8, "waiting for chunks (incl. the stage's input barrier)"), (14, "   of that, X chunks after a task's first"),
                           (15, "   of that, W chunks after a task's first"), (9, "waiting for the normalised X chunk"),
                           (10, "issuing MMAs"), (11, "waiting for the previous chunk's commit"), (100, "set-up"),
                           (101, "streaming loop"), (102, "epilogue from tensor memory"), (103, "partial sums to scratch"),
                           (104, "arrival at the block's counter"), (105, "last arrival's epilogue")):
            print(f"   {label:56s} {pv[:, row].mean() / clk:8.1f}")
        print(f"   weight chunks per SM {pv[:, 12].mean():.0f}, blocks finished per SM {pv[:, 106].mean():.1f}")
    if "trace_gemv" in trace:
        stage = ["qkv", "o", "gate/up", "down"]
        for o in range(8):
            t = (pv[:, 64 + o * 8: 64 + o * 8 + 8] - t0) / 1e3
            print(f"inside GEMV task {o + 4} (layer {1 + o // 4}, {stage[o % 4]}): us since kernel start, min / median / max over SMs")
            for i in range(8):
                col = t[:, i][t[:, i] > 0]
                if len(col):
                    print(f"   {GEMV_LABELS[i]:28s} {col.min():8.2f} {np.median(col):8.2f} {col.max():8.2f}")


if __name__ == "__main__":
    main()
