"""ctypes binding of libvdcores_b200.so with the surface of the reference's
``dae.runtime`` extension module (reference src/torch_runtime.cu:260-314):
``launch_dae``, ``build_tma_desc``, ``set_cache_policy``, ``set_smem_size``,
``opcode``, ``config``, ``compute_family_specs``, ``supported_compute_ops``.

There is no fallback: if the shared library is missing the import raises, and
every compute entry point needs a B200.
"""
from __future__ import annotations

import ctypes
import os
import types

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("VDCORES_LIB") or os.path.join(_HERE, "libvdcores_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m vdcores_b200.build` "
        "(needs nvcc); there is no CPU or PyTorch fallback for the decode path")

_lib = ctypes.CDLL(LIB_PATH)


class Status(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("abort", "code", "sm", "role", "pc", "opcode", "bar", "aux")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


_u64, _i32, _vp = ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p
_lib.vdc_version.restype = _i32
_lib.vdc_init.restype = _i32
_lib.vdc_set_smem_size.argtypes = [_i32]
_lib.vdc_launch.argtypes = [_i32, _i32, _vp, _vp, _vp, _vp, _vp, _u64, _u64, ctypes.POINTER(Status)]
_lib.vdc_launch_async.argtypes = [_i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64]
_lib.vdc_launch_async_full.argtypes = [_i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64]
_lib.vdc_launch_static.argtypes = [_i32, _i32, _vp, _vp, _vp, _vp, _u64, _u64, ctypes.POINTER(Status)]
_lib.vdc_read_status.argtypes = [_u64, ctypes.POINTER(Status), _i32]
_lib.vdc_build_tma_desc.argtypes = [_vp, _vp, _i32, _i32, ctypes.POINTER(_u64), ctypes.POINTER(_u64),
                                    ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32), _i32, _i32]
_lib.vdc_set_cache_policy.argtypes = [_vp, ctypes.c_size_t, _u64, ctypes.c_float, _i32, _i32]
_lib.vdc_enable_peer_access.argtypes = [_i32]
_lib.vdc_enable_peer_access.restype = _i32
_lib.vdc_ipc_open.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_uint64)]
_lib.vdc_ipc_open.restype = _i32
_lib.vdc_ipc_close.argtypes = [_u64]
_lib.vdc_ipc_close.restype = _i32
_lib.vdc_peer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_uint64)]
_lib.vdc_peer_alloc.restype = _i32
_lib.vdc_peer_free.argtypes = [_u64]
_lib.vdc_peer_free.restype = _i32
_lib.vdc_ipc_export.argtypes = [_u64, ctypes.c_char_p, ctypes.c_size_t]
_lib.vdc_ipc_export.restype = _i32
_lib.vdc_opcode_name.restype = ctypes.c_char_p
_lib.vdc_opcode_name.argtypes = [_i32]
_lib.vdc_opcode_value.argtypes = [_i32]
_lib.vdc_opcode_is_compute.argtypes = [_i32]
_lib.vdc_config.restype = ctypes.c_int64
_lib.vdc_config.argtypes = [ctypes.c_char_p]
_lib.vdc_family_specs.restype = ctypes.c_char_p
_lib.vdc_last_error.restype = ctypes.c_char_p
_lib.vdc_validate_streams.argtypes = [_i32, _i32, _vp, _vp, ctypes.POINTER(_i32), ctypes.POINTER(_i32)]
_lib.vdc_validate_streams.restype = _i32

EXPORTED_SYMBOLS = [
    "vdc_version", "vdc_init", "vdc_set_smem_size", "vdc_launch", "vdc_launch_async", "vdc_launch_async_full",
    "vdc_launch_static",
    "vdc_read_status",
    "vdc_build_tma_desc", "vdc_set_cache_policy", "vdc_enable_peer_access", "vdc_ipc_open", "vdc_ipc_close", "vdc_peer_alloc", "vdc_peer_free", "vdc_ipc_export", "vdc_opcode_count", "vdc_opcode_name", "vdc_opcode_value",
    "vdc_opcode_is_compute", "vdc_config", "vdc_family_specs", "vdc_last_error", "vdc_validate_streams",
]


class VdcError(RuntimeError):
    def __init__(self, code, message, status=None):
        super().__init__(f"vdcores error {code}: {message}")
        self.code = code
        self.status = status


def last_error() -> str:
    return _lib.vdc_last_error().decode()


def _check(rc, status=None):
    if rc != 0:
        raise VdcError(rc, last_error(), status.as_dict() if status is not None else None)


# ---- opcode / config namespaces (same attribute names as the reference) ----
opcode = types.SimpleNamespace()
supported_compute_ops = []
for _i in range(_lib.vdc_opcode_count()):
    _n = _lib.vdc_opcode_name(_i).decode()
    setattr(opcode, _n, _lib.vdc_opcode_value(_i))
    if _lib.vdc_opcode_is_compute(_i):
        supported_compute_ops.append(_n)

config = types.SimpleNamespace(**{
    k: int(_lib.vdc_config(k.encode()))
    for k in ("slot_size", "num_slots", "max_insts", "num_profile_events", "max_tmas", "max_bars",
              "num_special_slots", "compute_threads", "threads", "kv_page", "head_dim", "dynamic_smem")})

compute_family_specs = [
    dict(zip(("family", "definition"), line.split("\t", 1)))
    for line in _lib.vdc_family_specs().decode().split("\n") if line]

_initialised = set()


def init():
    """Prepares the current CUDA device (idempotent)."""
    dev = torch.cuda.current_device()
    if dev not in _initialised:
        _check(_lib.vdc_init())
        _initialised.add(dev)


def set_smem_size(nbytes: int) -> int:
    _check(_lib.vdc_set_smem_size(int(nbytes)))
    return 0


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def launch_dae(num_sms, smem_size, compute_insts, memory_insts, tma_descs, bars, profile, stream=0,
               timeout_ns=0, insts_per_sm=None):
    """Synchronous launch, same argument order as the reference's launch_dae
    (src/torch_runtime.cu:68-100).  Raises VdcError with the device status when
    a device-side wait gave up."""
    init()
    for name, t in (("compute_insts", compute_insts), ("memory_insts", memory_insts), ("bars", bars),
                    ("profile", profile)):
        if not (t.is_cuda and t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous CUDA tensor")
    if insts_per_sm is None:
        insts_per_sm = compute_insts.shape[0] // num_sms
    if compute_insts.numel() * compute_insts.element_size() != num_sms * insts_per_sm * 8:
        raise ValueError("compute_insts must hold num_sms * insts_per_sm 8-byte instructions")
    if memory_insts.numel() * memory_insts.element_size() != num_sms * insts_per_sm * 16:
        raise ValueError("memory_insts must hold num_sms * insts_per_sm 16-byte instructions")
    st = Status()
    rc = _lib.vdc_launch(num_sms, insts_per_sm, _ptr(compute_insts), _ptr(memory_insts), _ptr(tma_descs),
                         _ptr(bars), _ptr(profile), int(stream), int(timeout_ns), ctypes.byref(st))
    _check(rc, st)
    return 0


def validate_streams(num_sms, insts_per_sm, compute_insts, memory_insts):
    """Host-side check of a program's instruction words before the upload (numpy arrays or CPU tensors of
    num_sms * insts_per_sm 8-byte / 16-byte instructions).  Raises ValueError naming the SM, the instruction
    and what is wrong with it; needs no GPU."""
    import numpy as np
    c = np.ascontiguousarray(np.asarray(compute_insts)).view(np.uint8).reshape(-1)
    m = np.ascontiguousarray(np.asarray(memory_insts)).view(np.uint8).reshape(-1)
    if c.size != num_sms * insts_per_sm * 8 or m.size != num_sms * insts_per_sm * 16:
        raise ValueError("streams must hold num_sms * insts_per_sm instructions")
    sm, pc = _i32(-1), _i32(-1)
    rc = _lib.vdc_validate_streams(num_sms, insts_per_sm, c.ctypes.data_as(_vp), m.ctypes.data_as(_vp),
                                   ctypes.byref(sm), ctypes.byref(pc))
    if rc != 0:
        raise ValueError(last_error())


def launch_async(num_sms, insts_per_sm, compute_insts, memory_insts, tma_descs, bars, bars_init, profile,
                 stream=0, timeout_ns=0, full=False):
    """Enqueues one launch; full=True selects the kernel with every operator (batched engines, prefill)."""
    init()
    fn = _lib.vdc_launch_async_full if full else _lib.vdc_launch_async
    _check(fn(num_sms, insts_per_sm, _ptr(compute_insts), _ptr(memory_insts), _ptr(tma_descs),
                                 _ptr(bars), _ptr(bars_init), _ptr(profile), int(stream), int(timeout_ns)))


def launch_static(num_sms, insts_per_sm, compute_insts, memory_insts, tma_descs, bars_init, stream=0, timeout_ns=0):
    """Synchronous launch whose scratch (status, barriers, profile) is a static
    device array inside the library: for hosts that cannot let a library call
    allocate device memory.  Needs no init(); at most 160 SMs; calls on one device
    share the array, so do not overlap them."""
    st = Status()
    rc = _lib.vdc_launch_static(num_sms, insts_per_sm, _ptr(compute_insts), _ptr(memory_insts), _ptr(tma_descs),
                                _ptr(bars_init), int(stream), int(timeout_ns), ctypes.byref(st))
    _check(rc, st)
    return st.as_dict()


def read_status(stream=0, clear=True):
    st = Status()
    rc = _lib.vdc_read_status(int(stream), ctypes.byref(st), 1 if clear else 0)
    _check(rc, st)
    return st.as_dict()


_DTYPES = {torch.uint8: 0, torch.float16: 1, torch.bfloat16: 2, torch.float32: 3, torch.int32: 4}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = 0


def build_tma_desc(base, shape, strides_bytes, box_dim, elem_strides, swizzle_bytes=0, interleave=0):
    """Returns a CPU uint8[128] tensor holding the encoded tensor map
    (reference build_tma_desc, src/torch_runtime.cu:147-220)."""
    r = len(shape)
    if base.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {base.dtype}")
    out = torch.zeros(128, dtype=torch.uint8)
    A64 = _u64 * max(r, 1)
    A32 = ctypes.c_uint32 * max(r, 1)
    strides = list(strides_bytes) + [0] * (r - len(strides_bytes))
    rc = _lib.vdc_build_tma_desc(ctypes.c_void_p(out.data_ptr()), _ptr(base), _DTYPES[base.dtype], r,
                                 A64(*[int(x) for x in shape]), A64(*[int(x) for x in strides]),
                                 A32(*[int(x) for x in box_dim]), A32(*[int(x) for x in elem_strides]),
                                 int(swizzle_bytes), int(interleave))
    _check(rc)
    return out


def enable_peer_access(peer_device: int):
    """Kernels of the current device may then access `peer_device`'s memory mapped into this process."""
    _check(_lib.vdc_enable_peer_access(int(peer_device)))


def ipc_open(handle: bytes) -> int:
    """Maps another process's exported device allocation for the current device; returns its address."""
    out = ctypes.c_uint64(0)
    _check(_lib.vdc_ipc_open(handle, len(handle), ctypes.byref(out)))
    return int(out.value)


class PeerBlock:
    """Device memory allocated by the library as a block of its own (cudaMalloc), zeroed; `handle` is its
    64-byte CUDA IPC handle for other processes' ipc_open.  `tensor(dtype)` views it as a torch tensor."""

    def __init__(self, nbytes: int):
        out = ctypes.c_uint64(0)
        _check(_lib.vdc_peer_alloc(int(nbytes), ctypes.byref(out)))
        self.ptr, self.nbytes = int(out.value), int(nbytes)
        buf = ctypes.create_string_buffer(64)
        _check(_lib.vdc_ipc_export(self.ptr, buf, 64))
        self.handle = bytes(buf.raw)
        self.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 2}

    def tensor(self, dtype=torch.uint8):
        return torch.as_tensor(self, device=f"cuda:{torch.cuda.current_device()}").view(dtype)

    def free(self):
        if self.ptr:
            _check(_lib.vdc_peer_free(self.ptr))
            self.ptr = 0


def ipc_close(ptr: int):
    _check(_lib.vdc_ipc_close(int(ptr)))


def set_cache_policy(tensor, stream, hit_ratio, hit_policy, miss_policy):
    _check(_lib.vdc_set_cache_policy(_ptr(tensor), tensor.numel() * tensor.element_size(), int(stream),
                                     float(hit_ratio), int(hit_policy), int(miss_policy)))
