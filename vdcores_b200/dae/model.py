"""Layer helpers of the ``dae`` API (reference python/dae/model.py): a layer owns its tensors, builds the
tensor maps its schedule needs, and can compare the device result with a PyTorch expression.  The
projection layer is here; the attention layer helpers follow the attention operator."""
import torch

from .instructions import TmaTensor
from .schedule import SchedGemv
from .tma_utils import Major
from .util import tensor_diff


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
