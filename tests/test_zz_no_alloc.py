"""The allocation-free launch entry point (vdc_launch_static) against the regular
one (vdc_launch).  It exists for hosts that cannot afford a cudaMalloc inside a
library call — everything on the GPU already belongs to their own memory pool —
so its scratch is a static device array in the library.  Both entry points run
the same kernel on the same program, so the outputs must be identical; the call
is made twice in a row because the static array keeps the previous call's
contents and must be re-initialised correctly.  Collected last on purpose."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def build_case(dev):
    """Two dependent GEMV stages on four SMs (norm, residual add, a barrier chain)."""
    from vdcores_b200.program import Dst, Program, Src
    g = torch.Generator().manual_seed(42)
    K, M = 512, 256
    w1 = (torch.randn(M, K, generator=g) * 0.05).to(BF16).to(dev)
    w2 = (torch.randn(K, M, generator=g) * 0.05).to(BF16).to(dev)
    x = torch.randn(K, generator=g).to(BF16).to(dev)
    nw = (1 + 0.1 * torch.randn(K, generator=g)).to(BF16).to(dev)
    h0 = torch.randn(K, generator=g).to(BF16).to(dev)
    y = torch.zeros(M, dtype=BF16, device=dev)
    h = h0.clone()
    P = Program(4)
    b1, b2 = P.new_barrier(), P.new_barrier()
    for sm in range(2):
        r0 = sm * (M // 2)
        P.gemv(sm, w_addr=w1.data_ptr() + r0 * K * 2, n_rows=M // 2, K=K, R=16, x=Src(x.data_ptr(), K * 2),
               out=Dst(y.data_ptr() + r0 * 2, M, "store", release=b1), norm_w=Src(nw.data_ptr(), K * 2), eps=1e-5)
    for i, sm in enumerate((2, 3)):
        r0 = i * (K // 2)
        P.gemv(sm, w_addr=w2.data_ptr() + r0 * M * 2, n_rows=K // 2, K=M, R=16,
               x=Src(y.data_ptr(), M * 2, wait=b1), out=Dst(h.data_ptr() + r0 * 2, K, "add_bf16", release=b2))
    P.insts_per_sm = 32
    c, m, bars = P.finalize()
    keep = (w1, w2, x, nw)
    return (torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev), torch.from_numpy(bars).to(dev)), y, h, h0, keep


def test_static_launch_matches_regular_launch_twice(cuda_device):
    from vdcores_b200 import isa, runtime
    dev = cuda_device
    (c, m, bars_init), y, h, h0, keep = build_case(dev)
    stream = torch.cuda.current_stream().cuda_stream

    # the existing entry point: caller-owned barriers and profile, status block from vdc_init
    bars = bars_init.clone()
    prof = torch.zeros(4 * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    runtime.launch_dae(4, 0, c, m, None, bars, prof, stream, timeout_ns=300_000_000, insts_per_sm=32)
    y_ref, h_ref = y.clone(), h.clone()
    assert float(y_ref.float().abs().sum()) > 0

    for call in range(2):
        y.zero_()
        h.copy_(h0)
        st = runtime.launch_static(4, 32, c, m, None, bars_init, stream, timeout_ns=300_000_000)
        assert st["abort"] == 0 and st["code"] == 0
        assert torch.equal(y, y_ref), f"call {call}: first stage differs"
        assert torch.equal(h, h_ref), f"call {call}: residual stage differs"
    # the barrier image the caller passed in is an input: untouched
    assert int(bars_init.sum()) == 4


def test_static_launch_rejects_what_its_scratch_cannot_hold(cuda_device):
    from vdcores_b200 import isa, runtime
    (c, m, bars_init), *_ = build_case(cuda_device)
    with pytest.raises(runtime.VdcError) as ei:
        runtime.launch_static(161, 32, c, m, None, bars_init, 0)
    assert ei.value.code == isa.ERR_ARG and "160" in str(ei.value)
