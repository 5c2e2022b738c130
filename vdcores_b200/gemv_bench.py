"""Rate of the row-block GEMV task alone: one stage over all SMs, weights larger than L2.

    python -m vdcores_b200.gemv_bench [--rows 2048] [--k 4096] [--reps 4] [--formats bf16,fp8,nvfp4]

Every SM streams `rows` rows of K inputs in the chosen storage (bf16; e4m3 with fp32 per-row scales; NVFP4 rows
of e2m1 pairs + e4m3 block scales) through `Program.gemv` and writes bf16 outputs; the weights are random code
bytes (finite in every format), the timing is CUDA events around one launch, best of the repetitions after the
first.  Prints one line per format: bytes, time, GB/s and the fraction of the measured copy peak.  This is the
per-task figure next to which the whole decode step (bench.py) is read; it is not the headline metric."""
import argparse
import json
import os

import torch

from . import isa, runtime
from .decode import rows_per_chunk
from .program import Dst, Program, Src


def measured_copy_peak() -> float:
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0      # earlier measurement on the same pool


def run(fmt: str, rows_per_sm: int, K: int, reps: int, dev) -> dict:
    S = torch.cuda.get_device_properties(dev).multi_processor_count
    row_bytes = {"bf16": 2 * K, "fp8": K, "nvfp4": K // 2 + K // 16}[fmt]
    R = rows_per_chunk(K, row_bytes=row_bytes)
    rows_per_sm = rows_per_sm // R * R
    g = torch.Generator(device="cpu").manual_seed(0)
    w = torch.randint(0, 120, (S * rows_per_sm, row_bytes), dtype=torch.uint8, generator=g).to(dev)
    x = torch.randn(K, device=dev).to(torch.bfloat16)
    y = torch.zeros(S * rows_per_sm, dtype=torch.bfloat16, device=dev)
    scales = torch.ones(S * rows_per_sm, dtype=torch.float32, device=dev)
    P = Program(S)
    for sm in range(S):
        kw = {}
        if fmt == "fp8":
            kw["fp8_scales"] = scales.data_ptr() + 4 * sm * rows_per_sm
        if fmt == "nvfp4":
            kw["nvfp4_scales"] = scales.data_ptr() + 4 * sm * rows_per_sm
        P.gemv(sm, w_addr=w.data_ptr() + sm * rows_per_sm * row_bytes, n_rows=rows_per_sm, K=K, R=R,
               x=Src(x.data_ptr(), K * 2), out=Dst(y.data_ptr() + sm * rows_per_sm * 2, rows_per_sm * 2, "store"), **kw)
    n = max(max(len(a) for a in P.m), max(len(a) for a in P.c)) + 2
    P.insts_per_sm = ((n + 15) // 16) * 16
    c, m, bars = P.finalize()
    ct, mt, bt = (torch.from_numpy(a).to(dev) for a in (c, m, bars))
    prof = torch.zeros(S * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b = bt.clone()
        e0.record()
        runtime.launch_dae(S, 0, ct, mt, None, b, prof, torch.cuda.current_stream().cuda_stream,
                           timeout_ns=2_000_000_000, insts_per_sm=P.insts_per_sm)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = min(times[1:]) if len(times) > 1 else times[0]
    nbytes = S * rows_per_sm * row_bytes
    return {"format": fmt, "rows_per_chunk": R, "bytes": nbytes, "us": ms * 1e3, "gbs": nbytes / ms / 1e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048, help="rows per SM")
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--formats", default="bf16,fp8,nvfp4")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    runtime.init()
    peak = measured_copy_peak()
    for fmt in args.formats.split(","):
        r = run(fmt, args.rows, args.k, args.reps, dev)
        print(f"{r['format']:6s} R={r['rows_per_chunk']:2d} {r['bytes'] / 1e6:8.1f} MB  {r['us']:8.1f} us  {r['gbs']:8.1f} GB/s"
              f"  ({r['gbs'] / peak:.3f} of the measured copy peak)", flush=True)


if __name__ == "__main__":
    main()
