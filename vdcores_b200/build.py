"""Builds libvdcores_b200.so in-tree with nvcc for sm_100a:  python -m vdcores_b200.build"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libvdcores_b200.so")
SOURCES = [os.path.join(HERE, "csrc", f) for f in ("megakernel.cu", "capi.cu")]
# VDC_NO_STREAMER: the optional HBM->L2 streamer warp stays out of the build (it did not pay for
# the registers it costs: 13 warps cap the kernel at 128 registers per thread instead of 168).
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
         "-Xcompiler", "-fPIC", "-DVDC_NO_STREAMER"]


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    csrc = os.path.join(HERE, "csrc")
    deps = [os.path.join(csrc, f) for f in os.listdir(csrc)] + [os.path.join(HERE, "..", "include", "vdcores.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if force or needs_build():
        nvcc = os.environ.get("NVCC", "nvcc")
        cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB, *SOURCES]
        subprocess.check_call(cmd)
    return LIB


def build_trace(define: str) -> str:
    """A second library with one of the tracing switches compiled in (VDC_TRACE_ATTN: stamps inside the attention
    task, VDC_TRACE_GEMV: inside the GEMV task, VDC_TRACE_CHUNKS: life of SM 0's ring entries, VDC_TC_PROFILE: cycle
    sums inside the tensor-core projection task, profile rows 8-15 and 100-106); select it with
    VDCORES_LIB=<path>.  The stamps go into the launch's profile rows (vdcores_b200.stage_trace prints them)."""
    assert define in ("VDC_TRACE_ATTN", "VDC_TRACE_GEMV", "VDC_TRACE_CHUNKS", "VDC_TC_PROFILE")
    out = os.path.join(HERE, f"libvdcores_b200_{define.lower()}.so")
    subprocess.check_call([os.environ.get("NVCC", "nvcc"), *FLAGS, f"-D{define}", "-o", out, *SOURCES])
    return out


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build_trace(sys.argv[sys.argv.index("--trace") + 1]))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
