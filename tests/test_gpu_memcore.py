"""Memory-virtual-core paths on a B200, each against a plain torch expression: tiled
`cp.async.bulk.tensor` loads and stores through tensor maps built by vdc_build_tma_desc (2-D and
3-D, no swizzle and 128-byte swizzle), tensor-map and 1-D reduce-adds (bf16 and fp32), the
register hand-over between two tasks (REG_STORE -> REG_LOAD), the memory-stream LOOP with its
resource-group shift together with the compute-stream LOOPC, and the stream access-policy call.

Reference behaviour these follow: include/dae/pipeline/ldwarp.cuh:63-183 (tensor loads, registers),
stwarp.cuh:38-145 (tensor stores, reduce-add), allocwarp.cuh:148-166 (LOOP + group shift),
compute_dispatch.cuh:311-321 (LOOPC), src/torch_runtime.cu:147-258 (descriptors, cache policy)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
TIMEOUT_NS = 300_000_000


def launch(P, dev, tmas=None, stream=None):
    from vdcores_b200 import isa, runtime
    n = max(max(len(x) for x in P.m), max(len(x) for x in P.c)) + 2
    P.insts_per_sm = ((n + 15) // 16) * 16
    c, m, bars = P.finalize()
    ct, mt, bt = (torch.from_numpy(a).to(dev) for a in (c, m, bars))
    prof = torch.zeros(P.num_sms * isa.NUM_PROFILE_EVENTS, dtype=torch.int64, device=dev)
    td = torch.stack(tmas).to(dev) if tmas else None
    s = torch.cuda.current_stream().cuda_stream if stream is None else stream
    runtime.launch_dae(P.num_sms, 0, ct, mt, td, bt, prof, s, timeout_ns=TIMEOUT_NS, insts_per_sm=P.insts_per_sm)
    assert int(bt.abs().sum()) == 0, "every barrier must have counted down to zero"


def desc2d(t, box_cols, box_rows, swizzle):
    """Row-major [rows, cols] tensor; boxes of box_rows x box_cols elements."""
    from vdcores_b200 import runtime
    rows, cols = t.shape
    return runtime.build_tma_desc(t, [cols, rows], [cols * t.element_size()], [box_cols, box_rows], [1, 1], swizzle, 0)


def seeded(shape, seed, dtype=BF16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("swizzle", [0, 128])
def test_tensor_copy_2d(cuda_device, swizzle):
    """Four 32 x 64 boxes of a [32, 256] bf16 matrix travel load -> COPY -> store through two maps."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Program
    dev = cuda_device
    src = seeded((32, 256), 1).to(dev)
    dst = torch.zeros_like(src)
    tmas = [desc2d(src, 64, 32, swizzle), desc2d(dst, 64, 32, swizzle)]
    nbytes = 32 * 64 * 2
    P = Program(1)
    for j in range(4):
        P.tensor_load(0, tma_id=0, rank=2, coords=[64 * j, 0], nbytes=nbytes)
        P.tensor_store(0, tma_id=1, rank=2, coords=[64 * j, 0], nbytes=nbytes)
    P.comp(0, isa.OP_COPY, 4, nbytes // 4)
    launch(P, dev, tmas)
    assert torch.equal(dst, src)


def test_swizzle_128_puts_16_byte_pieces_where_the_tile_contract_says(cuda_device):
    """A 128-byte-swizzled box in shared memory, written out linearly: row r of the box holds its eight
    16-byte pieces at position (piece XOR (r mod 8)) — the K-major tile layout the reference's tasks read
    (python/dae/tma_utils.py:276-313)."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program
    dev = cuda_device
    src = seeded((16, 64), 2).to(dev)                       # one box: 16 rows x 128 bytes
    raw = torch.zeros(16 * 64, dtype=BF16, device=dev)
    P = Program(1)
    P.tensor_load(0, tma_id=0, rank=2, coords=[0, 0], nbytes=2048)
    P.store(0, Dst(raw.data_ptr(), 2048))
    P.comp(0, isa.OP_COPY, 1, 512)
    launch(P, dev, [desc2d(src, 64, 16, 128)])
    pieces = src.view(16, 8, 8)                             # [row][piece][8 elements]
    want = torch.empty_like(pieces)
    for r in range(16):
        for p in range(8):
            want[r, p ^ (r % 8)] = pieces[r, p]
    assert torch.equal(raw.view(16, 8, 8), want)


def test_tensor_copy_3d(cuda_device):
    """[3, 16, 128] bf16: a rank-3 map, boxes of 16 x 64 from every (batch, column half)."""
    from vdcores_b200 import isa, runtime
    from vdcores_b200.program import Program
    dev = cuda_device
    src = seeded((3, 16, 128), 3).to(dev)
    dst = torch.zeros_like(src)
    mk = lambda t: runtime.build_tma_desc(t, [128, 16, 3], [128 * 2, 16 * 128 * 2], [64, 16, 1], [1, 1, 1], 128, 0)
    nbytes = 16 * 64 * 2
    P = Program(2)
    for sm in range(2):                                     # SM 0 takes the left halves, SM 1 the right ones
        for b in range(3):
            P.tensor_load(sm, tma_id=0, rank=3, coords=[64 * sm, 0, b], nbytes=nbytes, port=b & 1)
            P.tensor_store(sm, tma_id=1, rank=3, coords=[64 * sm, 0, b], nbytes=nbytes)
        P.comp(sm, isa.OP_COPY, 3, nbytes // 4)
    launch(P, dev, [mk(src), mk(dst)])
    assert torch.equal(dst, src)


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
def test_reduce_add_2d_and_1d(cuda_device, dtype):
    """Tensor-map reduce-add of a box into a matrix that already holds values, twice from two SMs (the
    split-K sum plus residual add of the reference's projections), and the 1-D form."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    es = 2 if dtype == BF16 else 4
    cols = 128 // es                                        # one 128-byte box row
    # values on a coarse grid: the sums are exact in bf16 whatever the order
    g = torch.Generator().manual_seed(4)
    q = lambda *s: (torch.randint(-8, 9, s, generator=g).float() / 4).to(dtype)
    part = q(2, 16, cols).to(dev)
    acc = q(16, 2 * cols).to(dev)
    acc0 = acc.clone()
    P = Program(2)
    tmas = [desc2d(part[0], cols, 16, 0), desc2d(part[1], cols, 16, 0), desc2d(acc, cols, 16, 0)]
    for sm in range(2):                                     # both add into the right half of acc
        P.tensor_load(sm, tma_id=sm, rank=2, coords=[0, 0], nbytes=2048)
        P.tensor_store(sm, tma_id=2, rank=2, coords=[cols, 0], nbytes=2048, reduce=True)
        P.comp(sm, isa.OP_COPY, 1, 512)
    launch(P, dev, tmas)
    want = acc0.clone()
    want[:, cols:] = (acc0[:, cols:].float() + part[0].float() + part[1].float()).to(dtype)
    assert torch.equal(acc, want)
    # 1-D reduce-add through the bulk (untiled) form
    vec = q(1024).to(dev)
    tgt = q(1024).to(dev)
    tgt0 = tgt.clone()
    P = Program(1)
    P.copy(0, Src(vec.data_ptr(), 1024 * es), Dst(tgt.data_ptr(), 1024 * es, "add_bf16" if dtype == BF16 else "add_f32"),
           1024 * es)
    launch(P, dev)
    assert torch.equal(tgt, (tgt0.float() + vec.float()).to(dtype))


def test_register_hand_over_between_tasks(cuda_device):
    """Task 1 copies a loaded tile into slots that stay resident (REG_STORE: no write-back happens);
    task 2 receives the same slots through REG_LOAD and copies them to the output."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    src = seeded((2, 4096), 5).to(dev)
    out = torch.zeros_like(src)
    P = Program(2)
    for sm in range(2):
        P.load(sm, Src(src[sm].data_ptr(), 8192))
        P.reg_store(sm, 1, 8192)
        P.comp(sm, isa.OP_COPY, 1, 2048)
        P.reg_load(sm, 1)
        P.store(sm, Dst(out[sm].data_ptr(), 8192))
        P.comp(sm, isa.OP_COPY, 1, 2048)
    launch(P, dev)
    assert torch.equal(out, src)


def test_layer_loop_shifts_resource_groups(cuda_device):
    """One "layer" is emitted once and replayed three times: LOOP in the memory stream moves the tensor-map
    ids by 3 and the barrier ids by 1 per trip, LOOPC replays the compute instruction.  SM 0 copies
    src[l] -> mid[l] and releases barrier l; SM 1 waits for barrier l and copies mid[l] -> out[l]."""
    from vdcores_b200 import isa
    from vdcores_b200.program import Program
    dev = cuda_device
    L = 3
    src = seeded((L, 16, 64), 6).to(dev)
    mid = torch.zeros_like(src)
    out = torch.zeros_like(src)
    tmas = []
    for l in range(L):                                      # the resource group of layer l: three maps
        tmas += [desc2d(src[l], 64, 16, 128), desc2d(mid[l], 64, 16, 128), desc2d(out[l], 64, 16, 128)]
    P = Program(2)
    bars = [P.new_barrier() for _ in range(L)]
    for b in bars:
        P.bar_counts[b] = 1                                 # one release per layer, by the GROUP-flagged store
    # SM 0: body = {load map 0, store map 1 releasing barrier 0}, replayed with shifted ids
    P.tensor_load(0, tma_id=0, rank=2, coords=[0, 0], nbytes=2048, group=True)
    P.tensor_store(0, tma_id=1, rank=2, coords=[0, 0], nbytes=2048, release=bars[0], group=True)
    P.loop_m(0, L, 0, bar_shift=1, tma_shift=3)
    P.comp(0, isa.OP_COPY, 1, 512)
    P.loop_c(0, L, 0)
    # SM 1: body = {load map 1 behind barrier 0, store map 2}
    P.tensor_load(1, tma_id=1, rank=2, coords=[0, 0], nbytes=2048, wait=bars[0], port=1, group=True)
    P.tensor_store(1, tma_id=2, rank=2, coords=[0, 0], nbytes=2048, group=True)
    P.loop_m(1, L, 0, bar_shift=1, tma_shift=3)
    P.comp(1, isa.OP_COPY, 1, 512)
    P.loop_c(1, L, 0)
    launch(P, dev, tmas)
    assert torch.equal(mid, src) and torch.equal(out, src)


def test_cache_policy_window_on_a_stream(cuda_device):
    """vdc_set_cache_policy on a stream of its own (persisting hits over the source, as the reference's
    launcher does for its barriers and instruction tables), a launch on that stream, then a streaming window."""
    from vdcores_b200 import isa, runtime
    from vdcores_b200.program import Dst, Program, Src
    dev = cuda_device
    src = seeded((4, 4096), 7).to(dev)
    out = torch.zeros_like(src)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        runtime.init()
        runtime.set_cache_policy(src, side.cuda_stream, 1.0, 2, 0)      # persisting
        P = Program(4)
        for sm in range(4):
            P.copy(sm, Src(src[sm].data_ptr(), 8192), Dst(out[sm].data_ptr(), 8192), 8192)
        launch(P, dev, stream=side.cuda_stream)
        runtime.set_cache_policy(src[:1], side.cuda_stream, 0.0, 0, 1)  # streaming, over a slice
    side.synchronize()
    assert torch.equal(out, src)
    with pytest.raises(runtime.VdcError):
        runtime._check(runtime._lib.vdc_set_cache_policy(None, 0, 0, 1.0, 2, 0))
