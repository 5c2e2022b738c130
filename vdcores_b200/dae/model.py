"""Layer helpers of the ``dae`` API (reference python/dae/model.py): a layer owns its tensors, builds the
tensor maps its schedule needs, and can compare the device result with a PyTorch expression.  Here: the
projection layer, and the tensor-map recipes of the attention operators for caches whose tiled axis is not the
second-to-last one ([request, position, head, dim] views: `iN` / `iK` name the tiled axis).  The prefill
attention layer (GQALayer over SchedAttention) is outside the decode path and not built."""
import torch

from . import runtime
from .instructions import TmaTensor
from .schedule import SchedGemv
from .tma_utils import Major
from .util import tensor_diff


def uniform_rand_scaled(*shape: int, dtype=torch.float16, device="cuda", scale=0.1):
    return (torch.rand(*shape, dtype=dtype, device=device) - 0.5) * scale


def get_other_dims(dim: int, i: int):
    """Axes of a `dim`-dimensional tensor other than axis i (either sign) and the last one."""
    return [j for j in range(dim - 1) if j != i and j - dim != i]


def _others(mat: torch.Tensor, axis: int):
    """(folded extent, stride of the innermost one) of the axes other than `axis` and the last."""
    dims = get_other_dims(mat.dim(), axis)
    n = 1
    for j in dims:
        n *= mat.shape[j]
    return dims, n, mat.stride(dims[-1])


def _rest(mat: torch.Tensor, dims, cords) -> int:
    """Coordinate along the folded axis: the other axes' offset in units of the innermost one's stride."""
    return int(sum(mat.stride(j) * cords[j] for j in dims) // mat.stride(dims[-1]))


def _desc(mat, dims, strides_elems, box):
    es = mat.element_size()
    return len(dims), runtime.build_tma_desc(mat, dims, [s * es for s in strides_elems], box, [1] * len(dims), 128, 0)


def build_tma_wgmma_k(mat: torch.Tensor, tileK: int, tileN: int, iN: int = -2):
    """K-major operand tiles ([tileN rows along axis iN] x tileK columns, as tileK/64 blocks of 128-byte rows,
    128-byte swizzle) of a tensor whose last axis is K."""
    assert iN != -1 and iN < mat.dim() - 1, "iN must not be the last dim"
    block = 128 // mat.element_size()
    assert tileK % block == 0, "tileK must be multiple of blockK"
    dims, strides, box = [block, mat.shape[iN], mat.shape[-1] // block], [mat.stride(iN), block], [block, tileN, tileK // block]
    if mat.dim() > 2:
        _, n, st = _others(mat, iN)
        dims, strides, box = dims + [n], strides + [st], box + [1]
    return _desc(mat, dims, strides, box)


def cord_func_K_major(mat: torch.Tensor, rank: int, iN: int = -2):
    assert iN != -1 and iN < mat.dim() - 1, "iN must not be the last dim"

    def cord_func(*cords):
        assert mat.dim() == len(cords), f"cords length {len(cords)} does not match mat rank {mat.dim()}"
        if rank == 3:
            assert iN == -2
            return [0, cords[-2], cords[-1] // 64]
        if rank == 4:
            return [0, cords[iN], cords[-1] // 64, _rest(mat, get_other_dims(mat.dim(), iN), cords)]
        raise ValueError(f"Unsupported rank {rank} for k-major cord function")
    return cord_func


def build_tma_wgmma_mn(mat: torch.Tensor, tileM: int, tileK: int, iK: int = -2):
    """MN-major operand tiles (tileK rows along axis iK x tileM contiguous columns, delivered as atoms of 8 rows x
    64 columns, 128-byte swizzle)."""
    assert iK != -1 and iK < mat.dim() - 1, "iK must not be the last dim"
    assert mat.dim() >= 2, "Input matrix must be at least 2D"
    K, M = mat.shape[iK], mat.shape[-1]
    block = 128 // mat.element_size()
    assert tileM % block == 0, f"tileM {tileM} must be multiple of blockM {block}"
    if block != tileM:
        dims, strides = [block, 8, M // block, K // 8], [mat.stride(iK), block, mat.stride(iK) * 8]
        box = [block, 8, tileM // block, tileK // 8]
    else:
        dims, strides, box = [M, K], [mat.stride(iK)], [tileM, tileK]
    if mat.dim() > 2:
        _, n, st = _others(mat, iK)
        dims, strides, box = dims + [n], strides + [st], box + [1]
    return _desc(mat, dims, strides, box)


def _mn_cords(mat, rank, iK, cords):
    if rank == 2:
        assert iK == -2
        return [cords[-1], cords[-2]]
    rest = _rest(mat, get_other_dims(mat.dim(), iK), cords)
    if rank == 3:
        return [cords[-1], cords[iK], rest]
    if rank == 4:
        assert iK == -2
        return [0, 0, cords[-1] // 64, cords[-2] // 8]
    if rank == 5:      # the innermost coordinate is fixed to zero by the load
        return [0, cords[-1] // 64, cords[iK] // 8, rest]
    raise ValueError(f"Unsupported rank {rank} for mn-major cord function")


def cord_func_MN_major(mat: torch.Tensor, rank: int, iK: int = -2):
    assert iK != -1 and iK < mat.dim() - 1, "iK must not be the last dim"

    def cord_func(*cords):
        assert mat.dim() == len(cords), f"cords length {len(cords)} does not match mat rank {mat.dim()}"
        return _mn_cords(mat, rank, iK, cords)
    return cord_func


def cord_func_MN_major_cord2(mat: torch.Tensor, rank: int, iK: int = -2):
    """The same with only the last two coordinates given (the leading ones zero)."""
    assert iK != -1 and iK < mat.dim() - 1, "iK must not be the last dim"

    def cord_func(*cords):
        assert len(cords) == 2, f"expect input cords to be length 2, but got {len(cords)}"
        return _mn_cords(mat, rank, iK, [0] * (mat.dim() - 2) + list(cords))
    return cord_func


def tma_gqa_load_q(mat: torch.Tensor, tileK: int, tileN: int):
    """The query rows of one KV head's group ([request, kv head, group, head_dim]) as a 64-row K-major tile: the
    group's rows repeated 64 / group times through a zero stride."""
    assert mat.element_size() == 2, "Only support float16/bfloat16 output"
    assert tileN == 64, "tileN must be 64"
    n_req, n_kv, group, head_dim = mat.shape
    assert tileK == head_dim, "tileK must match HEAD_DIM"
    assert head_dim % 64 == 0, "HEAD_DIM must be a multiple of 64"
    assert 64 % group == 0, "HEAD_GROUP_SIZE must divide the 64-row Q tile"
    dims = [64, group, 64 // group, head_dim // 64, n_req * n_kv]
    return _desc(mat, dims, [head_dim, 0, 64, head_dim * group], dims[:4] + [1])


def cord_gqa_load_q(mat: torch.Tensor, rank: int):
    assert rank == 5, "Only support 5D TMA load for load Q"
    n_kv = mat.shape[1]

    def cfunc(*cords):
        assert len(cords) == 2, f"cords should be (req, head), but got {cords}"
        return [0, 0, 0, cords[0] * n_kv + cords[1]]
    return cfunc


class Layer:
    def __init__(self, dae, name: str):
        self.dae = dae
        self.name = name

    def schedule(self):
        raise NotImplementedError("Layer.schedule() must be implemented by subclass")

    def reference(self):
        raise NotImplementedError("Layer.reference() must be implemented by subclass")

    def diff(self):
        raise NotImplementedError("Layer.diff() must be implemented by subclass")


class GemvLayerBase(Layer):
    """C[N, M] (+)= B[N, K] A[M, K]^T with tile atom `Atom`; tmas = (load A, load B, store / reduce C)."""

    def __init__(self, dae, Atom, name: str, MNK, tmas, reduce=True):
        super().__init__(dae, name)
        self.Atom, self.reduce, self.MNK, self.tmas = Atom, reduce, MNK, tmas

    @staticmethod
    def _tma_funcs(self, Atom, reduce):
        TileM, TileN, TileK = Atom.MNK
        return [lambda t: t.wgmma_load(TileM, TileK, Major.K),
                lambda t: t.wgmma_load(TileN, TileK * Atom.n_batch, Major.K),
                lambda t: t.wgmma("reduce" if reduce else "store", TileN, TileM, Major.MN)]

    def schedule(self, num_gemv_sms=None, base_sm=0, **kwargs):
        sched = SchedGemv(self.Atom, self.MNK, self.tmas, **kwargs)
        return sched if num_gemv_sms is None else sched.place(num_gemv_sms, base_sm=base_sm)

    def schedule_(self, num_gemv_sms=None, base_sm=0, **kwargs):
        return self.schedule(num_gemv_sms=num_gemv_sms, base_sm=base_sm, exec=False, **kwargs)

    def reference(self):
        matA, matB, _ = self.tensors
        return matA @ matB.t()

    def diff(self):
        return tensor_diff(f"GEMV Layer: {self.name}", self.reference(), self.tensors[2].t())


class GemvLayer(GemvLayerBase):
    def __init__(self, dae, Atom, name: str, tensors, reduce=True):
        assert len(tensors) == 3, "GemvLayer requires 3 TmaTensors (A, B, C)"
        Layer.__init__(self, dae, name)
        self.Atom, self.reduce, self.tensors = Atom, reduce, tensors
        matA, matB, matC = tensors
        assert matA.dim() == matB.dim() == matC.dim() == 2, "A, B and C must be 2D"
        assert matA.shape[1] == matB.shape[1], "matA and matB K dimensions must match"
        assert matA.shape[0] == matC.shape[1], "matA and matC M dimensions must match"
        assert matB.shape[0] == matC.shape[0] == Atom.MNK[1], "matB / matC N dimension must match Atom.N"
        self.MNK = (matA.shape[0], matB.shape[0], matA.shape[1])
        self.tmas = tuple(f(TmaTensor(dae, t)) for f, t in zip(GemvLayerBase._tma_funcs(self, Atom, reduce), tensors))


def layers_like(constr, *cargs):
    return lambda *args, **kwargs: constr(*cargs, *args, **kwargs)
