"""Tensor-map recipes and coordinate helpers of the ``dae`` API (reference python/dae/tma_utils.py).

A recipe takes a tensor and a tile and returns ``(rank, descriptor)``; the matching coordinate
function turns logical tensor coordinates into the (at most four) 16-bit coordinates a memory
instruction carries.  The tile layouts are the contract with the compute tasks: K-major tiles are
boxes of 64 contiguous 2-byte elements (128 bytes) by `tile` rows with 128-byte swizzle, so row r
of a box holds its 16-byte pieces at piece XOR (r mod 8)."""
from enum import Enum
from math import prod

import torch

from . import runtime


class Major(Enum):
    MN = 1
    K = 2


def get_tensor_address(tensor: torch.Tensor) -> int:
    assert tensor.is_contiguous(), "memory instructions address contiguous tensors"
    assert tensor.device.type == "cuda", "memory instructions address device memory"
    return tensor.data_ptr()


def addr2cords(address: int):
    return [(address >> (16 * i)) & 0xFFFF for i in range(4)]


def cords2addr(cords) -> int:
    return sum((int(c) & 0xFFFF) << (16 * i) for i, c in enumerate(cords))


def bytes2slots(nbytes: int) -> int:
    return -(-nbytes // runtime.config.slot_size)


# --------------------------------------------------------------------------- coordinate adapters
class CordAdapter:
    """Wraps an instruction template and changes what `.cord(...)` means for it."""

    def __init__(self, inner):
        self.inner = inner

    def cord(self, *cords):
        raise NotImplementedError

    def __getattr__(self, name):
        return getattr(self.inner, name)


class StaticCordAdapter(CordAdapter):
    def cord(self, *cords):
        return self.inner


def wrap_static(*tmas):
    return tuple(StaticCordAdapter(t) for t in tmas)


class ToConvertedCordAdapter(CordAdapter):
    def __init__(self, inner, convert):
        super().__init__(inner)
        self.convert = convert

    def cord(self, *cords):
        return self.inner.cord(*self.convert(*cords))


class ToLinearCordAdapter(ToConvertedCordAdapter):
    def __init__(self, inner, delta: int):
        super().__init__(inner, lambda sm: (sm * delta,))


class ToRopeTableCordAdapter(ToConvertedCordAdapter):
    def __init__(self, inner, batch_seq_len: int, tile_repeats: int = 2):
        super().__init__(inner, lambda sm: (sm % tile_repeats, batch_seq_len))


class ToSplitMCordAdapter(ToConvertedCordAdapter):
    def __init__(self, inner, num_sms: int, tile_m: int):
        super().__init__(inner, lambda sm: (0, (sm % num_sms) * tile_m))


class ToAttnKVStoreCordAdapter(ToConvertedCordAdapter):
    def __init__(self, inner, num_sms: int, tile_m: int, position: int):
        super().__init__(inner, lambda sm: ((sm % num_sms) * tile_m, position, 0))


class ToAttnVStoreCordAdapter(ToConvertedCordAdapter):
    def __init__(self, inner, position: int):
        super().__init__(inner, lambda _, m: (m, position, 0))


class ToAttnCurrentKStore1DAdapter(ToConvertedCordAdapter):
    def __init__(self, inner, position: int, max_seq_len: int, num_kv_heads: int, head_dim: int, dtype_size: int = 2):
        row = num_kv_heads * head_dim

        def convert(sm):
            req, head = divmod(sm, num_kv_heads)
            return (((req * max_seq_len + position) * row + head * head_dim) * dtype_size,)
        super().__init__(inner, convert)


# --------------------------------------------------------------------------- tensor-map recipes
def _encode(mat, dims, strides, box, swizzle):
    return len(dims), runtime.build_tma_desc(mat, dims, strides, box, [1] * len(dims), swizzle, 0)


def _fold_leading(mat):
    """Index of the 2-D matrix a coordinate tuple selects when the leading dimensions are folded into one."""
    def rest(cords):
        lead = sum(int(s) * int(c) for s, c in zip(mat.stride()[:-2], cords[:-2]))
        return lead // prod(mat.shape[-2:])
    return rest


def cord_id(mat: torch.Tensor, rank: int):
    def cordf(*cords):
        assert len(cords) == rank, f"{len(cords)} coordinates for a rank-{rank} map"
        return list(cords)
    return cordf


def build_tma_1d(mat: torch.Tensor, size1: int, size2: int):
    """A flat tensor as rows of 64 elements: boxes of size1*size2 elements, addressed by element offset."""
    total, tile = mat.numel(), size1 * size2
    assert total % 64 == 0 and tile % 64 == 0, "1-D maps move multiples of 64 elements"
    return _encode(mat, [64, total // 64], [64 * 2], [64, tile // 64], 0)


def cord_func_tma_1d(mat: torch.Tensor, rank: int):
    assert rank == 2

    def cordf(offset):
        assert offset % 64 == 0, "1-D map offsets are multiples of 64 elements"
        return [0, offset // 64]
    return cordf


def build_tma_wgmma_kmajor(mat: torch.Tensor, tileK: int, tileN: int):
    """[..., N, K] with K contiguous -> boxes of tileN rows x tileK columns, delivered as tileK/64 blocks of
    [tileN rows x 128 bytes], 128-byte swizzled (the K-major operand tile of the projection tasks)."""
    assert mat.dim() >= 2
    N, K = mat.shape[-2], mat.shape[-1]
    es = mat.element_size()
    blockK = 128 // es
    assert tileK % blockK == 0, "tileK must cover whole 128-byte blocks"
    dims, strides, box = [blockK, N, K // blockK], [K * es, blockK * es], [blockK, tileN, tileK // blockK]
    if mat.dim() > 2:
        dims.append(prod(mat.shape[:-2]))
        strides.append(N * K * es)
        box.append(1)
    return _encode(mat, dims, strides, box, 128)


def cord_func_2d_kmajor(mat: torch.Tensor, rank: int):
    rest = _fold_leading(mat)

    def cordf(*cords):
        assert len(cords) == mat.dim()
        if rank == 3:
            return [0, cords[-2], cords[-1] // 64]
        if rank == 4:
            return [0, cords[-2], cords[-1] // 64, rest(cords)]
        raise ValueError(f"no K-major coordinates for rank {rank}")
    return cordf


def build_tma_wgmma_mnmajor(mat: torch.Tensor, tileM: int, tileK: int):
    """[..., K, M] with M contiguous -> boxes of tileK rows x tileM columns, 128-byte swizzled (the MN-major
    64 x 8 result tile of the projection tasks when tileM == 64 two-byte elements)."""
    assert mat.dim() >= 2
    K, M = mat.shape[-2], mat.shape[-1]
    es = mat.element_size()
    blockM, blockK = 128 // es, 8
    assert tileM % blockM == 0
    if tileM != blockM:
        dims = [blockM, blockK, M // blockM, K // blockK]
        strides = [M * es, blockM * es, M * blockK * es]
        box = [blockM, blockK, tileM // blockM, tileK // blockK]
    else:
        dims, strides, box = [M, K], [M * es], [tileM, tileK]
    if mat.dim() > 2:
        dims.append(prod(mat.shape[:-2]))
        strides.append(K * M * es)
        box.append(1)
    return _encode(mat, dims, strides, box, 128)


def cord_func_2d_mnmajor(mat: torch.Tensor, rank: int):
    rest = _fold_leading(mat)

    def cordf(*cords):
        assert len(cords) == mat.dim()
        if rank == 2:
            return [cords[-1], cords[-2]]
        if rank == 3:
            return [cords[-1], cords[-2], rest(cords)]
        if rank == 4:
            return [0, 0, cords[-1] // 64, cords[-2] // 8]
        if rank == 5:       # the innermost coordinate of a rank-5 map is fixed to 0 by the memory core
            return [0, cords[-1] // 64, cords[-2] // 8, rest(cords)]
        raise ValueError(f"no MN-major coordinates for rank {rank}")
    return cordf


def tma_store_attn_kv(mat: torch.Tensor, TileM: int, TileK: int):
    """KV cache [reqs, max_seq, kv_width]: a projection's 64-row x 8-request result tile goes to one position."""
    assert (TileM, TileK) == (64, 8) and mat.dim() == 3 and mat.element_size() == 2
    es = mat.element_size()
    reqs, seq, width = mat.shape
    return _encode(mat, [width, seq, reqs], [es * width, es * width * seq], [TileM, 1, TileK], 128)


def tma_load_tbl(mat: torch.Tensor, TileM: int, TileN: int):
    """Rope table [max_seq, head_dim]: one 64-wide half of a position's row, repeated for TileN requests."""
    assert mat.element_size() == 2 and TileM == 64 and mat.shape[-1] % 64 == 0
    s, head_dim, seq = mat.element_size(), mat.shape[-1], mat.shape[0]
    return _encode(mat, [64, TileN, head_dim // 64, seq], [head_dim * s, 64 * s, head_dim * TileN * s],
                   [64, TileN, 1, 1], 128)


def cord_load_tbl(mat: torch.Tensor, rank: int):
    assert rank == 4

    def cordf(half, position):
        return [0, 0, half, position]
    return cordf
