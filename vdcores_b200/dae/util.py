"""Script helpers of the ``dae`` API (reference python/dae/util.py): result comparison, instruction dumps and
the command-line front end the operator scripts end with (-l launch, -b [N] bench, -i [SM] dump, -p profile)."""
import argparse

import numpy as np
import torch

from .launcher import extract_compute_operator_names

DEFAULT_COMPUTE_OPS_FILE = "dae_compute_ops.vdcore.build"


def tensor_diff(name: str, t1: torch.Tensor, t2: torch.Tensor, ref=None):
    """Mean absolute difference relative to the mean magnitude of `ref` (default t1), in percent; printed the
    way the reference prints it, and returned so that tests can assert on it."""
    ref = t1 if ref is None else ref
    diff = (t1 - t2).abs().float().mean().item() / ref.abs().float().mean().item() * 100
    print(f"Ave Diff {name}: {diff} %. ")
    if diff > 1.5:
        print(f"{name} t1:", t1)
        print(f"{name} t2:", t2)
    print(f"{name} checksum t1: {(t1.float().sum().item(), t1.shape)}, t2: {(t2.float().sum().item(), t2.shape)}")
    return diff


def dump_insts(dae, smid: int):
    dae.build_instructions()
    b = dae.builder[smid]
    for title, insts in (("Compute", b.built_cinsts), ("Memory", b.built_minsts)):
        print(f"[sm={smid}] {title} Instructions:")
        for i, inst in enumerate(insts):
            print(f"{i:02}: {inst}")


def write_compute_operator_file(dae, path: str = DEFAULT_COMPUTE_OPS_FILE):
    names = extract_compute_operator_names(dae)
    with open(path, "w", encoding="utf-8") as f:
        f.writelines(n + "\n" for n in names)
    print(f"[compute-ops] wrote {len(names)} operators to {path}")
    return path


class ProfileParser:
    """Reads the per-SM profile rows after a launch: `name` prints the mean of the next column in microseconds,
    `+name` relative to the kernel start, `=N` jumps to column N, `name:K` repeats K times, `@raw` prints rows."""

    def __init__(self, dae):
        self.data = dae.profile.cpu().view(torch.int64).numpy()
        self.count, self.history, self.raw = 2, None, False

    def parse(self, prof: str):
        if prof == "@raw":
            self.raw = True
            return
        if prof.startswith("@"):
            raise ValueError(f"Unknown profile option: {prof}")
        if prof.startswith("="):
            self.count, self.history = int(prof[1:]), None
            return
        if ":" in prof:
            name, repeat = prof.split(":")
            for i in range(int(repeat)):
                self.parse(f"{name}r{i}")
            return
        col = self.data[:, self.count].astype(np.float64)
        if prof.startswith("+"):
            col = col - self.data[:, 0]
        if self.raw:
            print(f"[profile] {prof}: {col}")
        us = float(np.mean(col)) / 1e3
        shown = us - self.history if ("^" in prof and self.history is not None) else us
        print(f"[profile] {prof}: {shown:.3f} us")
        self.history = us
        self.count += 1


def dae_app(dae, total_bytes=None, argv=None):
    ap = argparse.ArgumentParser(description="VDCores frontend")
    mode = ap.add_mutually_exclusive_group()
    mode.add_argument("-b", "--bench", type=int, nargs="?", const=1, default=None, help="Run benchmark N times (default: 1)")
    mode.add_argument("-l", "--launch", action="store_true", help="Launch configuration")
    ap.add_argument("-i", "--instdump", type=int, nargs="?", const=0, default=None, help="Dump instructions for SM ID")
    ap.add_argument("-p", "--profile", type=str, nargs="+", default=None, help="Profile with the runtime's counters")
    ap.add_argument("-w", "--write-compute-ops", type=str, nargs="?", const=DEFAULT_COMPUTE_OPS_FILE, default=None,
                    help="Write the launcher's compute-operator list to a file")
    args = ap.parse_args(argv)
    did = False
    if args.instdump is not None:
        dump_insts(dae, args.instdump)
        print()
        did = True
    if args.write_compute_ops is not None:
        write_compute_operator_file(dae, args.write_compute_ops)
        did = True
    ran = False
    if args.launch:
        print(f"[launch] VDCores with {dae.num_sms} SMs...")
        dae.launch()
        ran = True
    elif args.bench is not None:
        torch.cuda.synchronize()
        print(f"[bench] VDCores with {dae.num_sms} SMs...")
        dae.bench(args.bench, total_bytes=total_bytes)
        torch.cuda.synchronize()
        ran = True
    elif not did:
        print("DAE NO EXECUTION MODE.")
    if ran and args.profile is not None:
        pp = ProfileParser(dae)
        for p in args.profile:
            pp.parse(p)
