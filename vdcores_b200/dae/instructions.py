"""Instruction classes of the ``dae`` API and their wire encodings (reference
python/dae/instructions.py, instruction_utils.py): a compute instruction is {u16 opcode, u16 args[3]},
a memory instruction {u16 opcode|flags, u16 size, u16 nslot|bar<<6, u16 arg, four u16 coordinates or a
64-bit address}.  Flag bits: 2 write-back, 4 resource group, 8 jump, 16 barrier, 32 port 1."""
import copy

import torch

from .op_families import ComputeOpFamilyRef, family_name, family_ref
from .runtime import config, opcode
from .tma_utils import (Major, addr2cords, build_tma_1d, build_tma_wgmma_kmajor, build_tma_wgmma_mnmajor, bytes2slots,
                        cord_func_2d_kmajor, cord_func_2d_mnmajor, cord_func_tma_1d, cords2addr, get_tensor_address)


# --------------------------------------------------------------------------- helpers
def decode_opcode(op: int) -> str:
    table = vars(opcode)
    for probe in (op, op | 2):      # the write-back bit may have been toggled after the opcode was chosen
        for name, value in table.items():
            if value == probe:
                return name
    return f"UNKNOWN_OPCODE[0x{op:04x}]"


dedcode_opcode = decode_opcode      # historic spelling kept for older scripts


def encode_bfloat16_u16(value: float) -> int:
    return int(torch.tensor(value, dtype=torch.bfloat16).view(torch.uint16).item())


class Instruction:
    def tensor(self, tensor=None):
        raise NotImplementedError()


# --------------------------------------------------------------------------- compute instructions
class ComputeInstruction(Instruction):
    """opcode: an integer from ``runtime.opcode``, or a family member (name or ``family_ref``) that is
    looked up in the runtime's opcode table when the instruction is encoded."""

    def __init__(self, opcode, args):
        if isinstance(opcode, int):
            self.opcode, self.op_family_name = opcode, None
        else:
            self.opcode, self.op_family_name = None, family_name(opcode)
        self.args = args

    def opcode_value(self) -> int:
        if self.opcode is not None:
            return self.opcode
        try:
            return int(getattr(opcode, self.op_family_name))
        except AttributeError as exc:
            raise ValueError(f"Missing runtime opcode for op-family instruction {self.op_family_name}. "
                             "Rebuild dae.runtime with this generated compute op.") from exc

    def compute_operator_name(self) -> str:
        return self.op_family_name if self.op_family_name is not None else decode_opcode(self.opcode)

    def tensor(self, tensor=None):
        words = torch.empty(4, dtype=torch.uint16) if tensor is None else tensor.view(torch.uint16)
        assert words.numel() == 4 and len(self.args) <= 3
        words.zero_()
        words[0] = self.opcode_value()
        for i, a in enumerate(self.args):
            assert 0 <= a < 2 ** 16, "args must be uint16"
            words[1 + i] = a
        return words.view(torch.uint8)

    def __repr__(self):
        return f"ComputeInstruction(opcode={self.compute_operator_name()}, args={self.args})"


class TerminateC(ComputeInstruction):
    def __init__(self):
        super().__init__(opcode.OP_TERMINATEC, [])


def _gemv_family(name, family, M, K, n_batch, **fixed):
    """A projection-tile instruction class: C[M, 8] += A[M, K] B[8, K]^T per k-tile; the activation tile is
    re-loaded every n_batch tiles."""
    def __init__(self, kTiles: int, nprefeth=0, residual: bool = False):
        fields = dict(M=M, N=8, K=K, **fixed)
        if family == "GEMV_WGMMA":
            fields.update(BLOAD=n_batch, RESIDUAL=residual)
            ComputeInstruction.__init__(self, family_ref(family, **fields), [kTiles, nprefeth])
        else:
            ComputeInstruction.__init__(self, family_ref(family, **fields), [kTiles])
    return type(name, (ComputeInstruction,), {"MNK": (M, 8, K), "n_batch": n_batch, "__init__": __init__})


Gemv_M64N8 = _gemv_family("Gemv_M64N8", "GEMV_WGMMA", 64, 256, 4)
Gemv_M64N8K64 = _gemv_family("Gemv_M64N8K64", "GEMV_WGMMA", 64, 64, 1)
Gemv_M64N8B2 = _gemv_family("Gemv_M64N8B2", "GEMV_WGMMA", 64, 256, 2)
Gemv_M128N8 = _gemv_family("Gemv_M128N8", "GEMV_WGMMA", 128, 128, 4)
Gemv_M64N8_MMA = _gemv_family("Gemv_M64N8_MMA", "GEMV_MMA", 64, 256, 1)


def _plain(name, op_name, arg_names=(), doc=None, **attrs):
    """A compute instruction class whose constructor arguments are its args, in order."""
    def __init__(self, *values, **kw):
        vals = list(values) + [kw[n] for n in arg_names[len(values):]]
        assert len(vals) == len(arg_names), f"{name}({', '.join(arg_names)})"
        ComputeInstruction.__init__(self, getattr(opcode, op_name), [int(v) for v in vals])
    return type(name, (ComputeInstruction,), {"__init__": __init__, "__doc__": doc, **attrs})


class ROPE_INTERLEAVE_512(ComputeInstruction):
    def __init__(self):
        super().__init__(opcode.OP_ROPE_INTERLEAVE_512, [])


def _attention(name, op_name, head_dim, split=False):
    if split:
        def __init__(self, num_kv_block, split_idx, num_active_q, last_kv_active_token_len, kv_start_idx,
                     need_norm: bool = True, need_rope: bool = True):
            assert split_idx < 16, "split_idx must be less than 16 to fit in the instruction encoding"
            ComputeInstruction.__init__(self, getattr(opcode, op_name),
                                        [num_kv_block | (split_idx << 12),
                                         num_active_q | (last_kv_active_token_len << 8), kv_start_idx])
    else:
        def __init__(self, num_kv_block, last_kv_active_token_len, need_norm: bool = True, need_rope: bool = True):
            flags = (1 if need_norm else 0) | (2 if need_rope else 0)
            ComputeInstruction.__init__(self, getattr(opcode, op_name), [num_kv_block, last_kv_active_token_len, flags])
    return type(name, (ComputeInstruction,), {"HEAD_DIM": head_dim, "__init__": __init__})


ATTENTION_M64N64K16_F16_F32_64_64_hdim = _attention(
    "ATTENTION_M64N64K16_F16_F32_64_64_hdim", "OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim", 128)
ATTENTION_M64N64K16_F16_F32_64_64_hdim_MMA = _attention(
    "ATTENTION_M64N64K16_F16_F32_64_64_hdim_MMA", "OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim_MMA", 128)
ATTENTION_M64N64K16_F16_F32_64_64_hdim_split = _attention(
    "ATTENTION_M64N64K16_F16_F32_64_64_hdim_split", "OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim_split", 128, split=True)
ATTENTION_M64N64K16_F16_F32_64_64_hdim_split_MMA = _attention(
    "ATTENTION_M64N64K16_F16_F32_64_64_hdim_split_MMA", "OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim_split_MMA", 128,
    split=True)


class ATTN_SPLIT_POST_REDUCE(ComputeInstruction):
    HEAD_DIM = 128
    Q_TILE = 4

    def __init__(self, num_split: int):
        super().__init__(opcode.OP_ATTN_SPLIT_POST_REDUCE, [num_split])


SILU_MUL_SHARED_BF16_K_4096_INTER = _plain("SILU_MUL_SHARED_BF16_K_4096_INTER", "OP_SILU_MUL_SHARED_BF16_K_4096_INTER",
                                           ("num_token",))
SILU_MUL_SHARED_BF16_K_64_SW128 = _plain("SILU_MUL_SHARED_BF16_K_64_SW128", "OP_SILU_MUL_SHARED_BF16_K_64_SW128",
                                         ("num_token",))


def _rms(name, op_name):
    def __init__(self, num_token: int, epsilon: float):
        ComputeInstruction.__init__(self, getattr(opcode, op_name), [num_token, encode_bfloat16_u16(epsilon)])
    return type(name, (ComputeInstruction,), {"__init__": __init__})


RMS_NORM_F16_K_4096_SMEM = _rms("RMS_NORM_F16_K_4096_SMEM", "OP_RMS_NORM_F16_K_4096_SMEM")
RMS_NORM_F16_K_128_SMEM = _rms("RMS_NORM_F16_K_128_SMEM", "OP_RMS_NORM_F16_K_128_SMEM")
RMS_NORM_F16_K_2048_SMEM = _rms("RMS_NORM_F16_K_2048_SMEM", "OP_RMS_NORM_F16_K_2048_SMEM")
RMS_NORM_F16_K_5120_SMEM = _rms("RMS_NORM_F16_K_5120_SMEM", "OP_RMS_NORM_F16_K_5120_SMEM")


def select_attention_decode_instruction(head_dim: int):
    if head_dim == ATTENTION_M64N64K16_F16_F32_64_64_hdim.HEAD_DIM:
        return ATTENTION_M64N64K16_F16_F32_64_64_hdim
    raise NotImplementedError(f"Missing attention decode kernel support for head_dim={head_dim}. "
                              "Add a dedicated opcode/instruction path before launching this model.")


def select_rms_smem_instruction(hidden_size: int):
    table = {4096: RMS_NORM_F16_K_4096_SMEM, 2048: RMS_NORM_F16_K_2048_SMEM, 5120: RMS_NORM_F16_K_5120_SMEM,
             128: RMS_NORM_F16_K_128_SMEM}
    if hidden_size not in table:
        raise NotImplementedError(f"Missing shared-memory RMS kernel support for hidden_size={hidden_size}. "
                                  "Add a dedicated opcode/instruction path before launching this model.")
    return table[hidden_size]


def ensure_cc0_supported_hidden_size(hidden_size: int):
    if hidden_size * 2 <= 0:
        raise NotImplementedError(f"Missing CC0 embedding-stride support for hidden_size={hidden_size}.")


ARGMAX_PARTIAL_bf16_1152_50688_132 = _plain("ARGMAX_PARTIAL_bf16_1152_50688_132", "OP_ARGMAX_PARTIAL_bf16_1152_50688_132",
                                            ("num_active_token",), CHUNK_SIZE=1152, I_STRIDE=50688, SMS=132)
ARGMAX_REDUCE_bf16_1152_132 = _plain("ARGMAX_REDUCE_bf16_1152_132", "OP_ARGMAX_REDUCE_bf16_1152_132",
                                     ("num_active_token",), CHUNK_SIZE=1152, SMS=132)
ARGMAX_PARTIAL_bf16_1024_65536_128 = _plain("ARGMAX_PARTIAL_bf16_1024_65536_128", "OP_ARGMAX_PARTIAL_bf16_1024_65536_128",
                                            ("num_active_token",), CHUNK_SIZE=1024, I_STRIDE=65536, SMS=128)
ARGMAX_REDUCE_bf16_1024_128 = _plain("ARGMAX_REDUCE_bf16_1024_128", "OP_ARGMAX_REDUCE_bf16_1024_128",
                                     ("num_active_token",), CHUNK_SIZE=1024, SMS=128)
Dummy = _plain("Dummy", "OP_DUMMY", ("iters",))


class Copy(ComputeInstruction):
    def __init__(self, iters: int, size: int):
        assert size % 4 == 0, "Copy size must be multiple of 4 bytes (size of uint32)"
        super().__init__(opcode.OP_COPY, [iters, size // 4])


class LoopC(ComputeInstruction):
    def __init__(self, count: int, pc: int):
        super().__init__(opcode.OP_LOOPC, [count, pc])

    @classmethod
    def toNext(cls, ptrs, count):
        return lambda sm_id: cls(count, ptrs[sm_id])


# --------------------------------------------------------------------------- memory instructions
class MemoryInstruction(Instruction):
    def __init__(self, opcode: int, num_slots: int, arg: int, size: int, cords=(), address=None):
        self.opcode = opcode
        self.num_slots = num_slots
        self.arg = arg
        self.size = size
        self.annotation = {}
        self.set_cords(list(cords))
        if address is not None:
            self.cords = addr2cords(address)

    def set_cords(self, cords):
        assert len(cords) <= 4, "Maximum 4 cords are supported"
        self.cords = list(cords) + [0] * (4 - len(cords))
        assert all(0 <= c < 2 ** 16 - 1 for c in self.cords), "cord values must be a uint16"

    def delta(self, delta):
        """Moves the instruction: by a byte count (the coordinates taken as a 64-bit address) or coordinate-wise."""
        if isinstance(delta, int):
            self.cords = addr2cords(cords2addr(self.cords) + delta)
        elif isinstance(delta, list):
            assert len(delta) <= 4, "Maximum 4 cords are supported"
            self.cords = [c + d for c, d in zip(self.cords, delta + [0] * (4 - len(delta)))]
        else:
            raise ValueError("delta must be int or list[int]")
        return self

    def group(self, enable=True):
        if enable:
            self.opcode |= 4
        return self

    def jump(self):
        self.opcode |= 8
        return self

    def bar(self, bar_id=None):
        if bar_id is not None:
            self.opcode |= 16
            self.num_slots |= bar_id << 6
        return self

    def writeback(self):
        self.opcode |= 2
        return self

    def port(self, port_id: int):
        if port_id not in (0, 1):
            raise ValueError("Only port 0 and 1 are supported")
        if port_id == 1:
            self.opcode |= 32
        return self

    def copy(self):
        other = MemoryInstruction(self.opcode, self.num_slots, self.arg, self.size, cords=list(self.cords))
        other.annotation = dict(self.annotation)
        return other

    def tensor(self, tensor=None):
        words = torch.empty(8, dtype=torch.uint16) if tensor is None else tensor.view(torch.uint16)
        assert words.numel() == 8
        for i, v in enumerate([self.opcode, self.size, self.num_slots, self.arg, *self.cords]):
            words[i] = v
        return words.view(torch.uint8)

    def __repr__(self):
        op, slots, flags = self.opcode, self.num_slots, []
        for bit, label in ((8, "JUMP"), (4, "GROUP"), (16, None), (2, "WB"), (32, "PORT1")):
            if op & bit:
                if bit == 16:
                    flags.append(f"BAR[{slots >> 6}]")
                    slots &= 0x3F
                else:
                    flags.append(label)
                op &= ~bit
        return (f"MemoryInstruction(opcode={decode_opcode(op)}, num_slots={slots}, arg={self.arg}, size={self.size}, "
                f"cords={self.cords}, flags={flags}, anno={self.annotation})")


class TerminateM(MemoryInstruction):
    def __init__(self):
        super().__init__(opcode.OP_TERMINATE, 0, 0, 0, address=0)


class LoopM(MemoryInstruction):
    """Memory-stream loop back to `pc`, `count` trips in all; after every trip the barrier ids and tensor-map
    ids of GROUP-flagged instructions move on by the resource group's width."""

    def __init__(self, count: int, pc: int, reg=0, bar_shift: int = 0, tma_shift: int = 0, resource_group=None):
        if resource_group is not None:
            tma_shift, bar_shift = resource_group.get_shift()
        assert 0 <= reg < 32, "reg must be in [0,31]"
        assert tma_shift < 2 ** 16, "tma_shift must be less than 65536"
        assert bar_shift < 2 ** 10, "bar_shift must be less than 1024"
        super().__init__(opcode.OP_LOOP, reg, 0, count, cords=[pc, 0, bar_shift << 6, tma_shift])

    @classmethod
    def toNext(cls, ptrs, count: int, **kwargs):
        return lambda sm_id: cls(count, ptrs[sm_id], **kwargs)


class RepeatM(MemoryInstruction):
    """Header of a hardware loop over the following instructions: lanes [reg, reg_end) of the control warp
    take `delta` as the per-trip address (or coordinate) increment of body instructions reg..reg_end-1."""

    def __init__(self, count: int, reg: int = 0, reg_end=None, delta_addr=None, delta_cords=()):
        reg_end = reg + 1 if reg_end is None else reg_end
        assert 0 <= reg < 32 and 0 <= reg_end <= 32 and reg_end > reg
        super().__init__(opcode.OP_REPEAT, (reg_end << 8) | reg, 0, count, address=delta_addr, cords=list(delta_cords))

    @classmethod
    def on(cls, count: int, *steps):
        """steps: (instruction, per-trip delta) pairs.  Equal consecutive deltas share one header; the last
        header carries the count, the last body instruction the jump flag."""
        if not steps or count == 0:
            return []
        runs = []
        for i, (_, delta) in enumerate(steps):
            cords = delta if isinstance(delta, list) else addr2cords(delta) if isinstance(delta, int) else None
            if cords is None:
                raise ValueError("delta must be int or list[int]")
            if runs and runs[-1][2] == cords:
                runs[-1][1] = i + 1
            else:
                runs.append([i, i + 1, cords])
        insts = []
        if count > 1:
            insts = [cls(0, reg=lo, reg_end=hi, delta_cords=c) for lo, hi, c in runs]
            insts[-1].size = count
        insts += [inst for inst, _ in steps]
        if count > 1:
            insts[-1].jump()
        return insts

    @classmethod
    def on1(cls, count: int, *steps):
        """The loop with its first trip already peeled off: every template moves on by one delta."""
        assert count > 0, "count must be greater than 0 to use on1"
        return cls.on(count - 1, *[(inst.delta(delta), delta) for inst, delta in steps])

    @classmethod
    def onSync(cls, bar_inst_offset: int, bar_id, count: int, *steps, asyncPort: bool = True):
        """The first trip is emitted on its own with instruction `bar_inst_offset` waiting for `bar_id`
        (on port 1 when asyncPort, so the wait does not hold up port 0); the rest loops without waits."""
        if bar_id is None:
            return cls.on(count, *steps)
        first = []
        for i, (inst, _) in enumerate(steps):
            if i == bar_inst_offset:
                inst.port(1 if asyncPort else 0)
            peeled = inst.copy()
            if i == bar_inst_offset:
                peeled.bar(bar_id)
            first.append(peeled)
        return first + cls.on1(count, *steps)


class RawAddress(MemoryInstruction):
    def __init__(self, tensor: torch.Tensor, slot_id: int):
        assert tensor.device.type == "cuda"
        lo, hi = config.num_slots, config.num_slots + config.num_special_slots - 1
        assert lo <= slot_id <= hi, f"slot_id must be in the range of special slots [{lo}, {hi}]"
        super().__init__(opcode.OP_ALLOC_WB_RAW_ADDRESS, slot_id, slot_id, 0, address=tensor.data_ptr())


class IssueBarrier(MemoryInstruction):
    def __init__(self, bar: int):
        super().__init__(opcode.OP_ISSUE_BARRIER, 0, 0, 0, address=0)
        self.bar(bar)


class CC0(MemoryInstruction):
    """The next 1-D load's address moves on by token id x embedding row bytes (token read from tokens[idx])."""

    def __init__(self, tokens: torch.Tensor, idx: int, hidden_size: int = 4096, dtype_size: int = 2):
        addr = get_tensor_address(tokens[idx])
        row_bytes = hidden_size * dtype_size
        if row_bytes <= 0:
            raise ValueError(f"CC0 requires a positive embedding row size in bytes, got {row_bytes}")
        if row_bytes & (row_bytes - 1) == 0:
            super().__init__(opcode.OP_CC0, 0, row_bytes.bit_length() - 1, 0, address=addr)
        else:
            super().__init__(opcode.OP_CC0_ROW_BYTES, 0, 0, row_bytes, address=addr)


class RegStore(MemoryInstruction):
    def __init__(self, reg_id: int, shape: torch.Tensor = None, size=None):
        if size is None:
            assert shape is not None, "Either shape or size must be provided for RegStore"
            size = shape.numel() * shape.element_size()
        super().__init__(opcode.OP_ALLOC_WB_REG_STORE, bytes2slots(size), 0, reg_id, address=0)
        self.mode = "reduce"

    def cord(self, *args):
        return self


class RegLoad(MemoryInstruction):
    def __init__(self, reg_id: int, slot_id=None):
        slot_id = reg_id if slot_id is None else slot_id
        assert slot_id < config.num_special_slots, f"slot_id must be less than {config.num_special_slots} for RegLoad"
        super().__init__(opcode.OP_ALLOC_REG_LOAD, config.num_slots + slot_id, 0, reg_id, address=0)

    def cord(self, *args):
        return self


class _Tma1D(MemoryInstruction):
    _OP = None

    def __init__(self, t: torch.Tensor, bytes=None, numSlots=None):
        nbytes = t.numel() * t.element_size() if bytes is None else bytes
        super().__init__(getattr(opcode, self._OP), bytes2slots(nbytes) if numSlots is None else numSlots, 0, nbytes,
                         address=get_tensor_address(t))

    def cord(self, addr):
        moved = copy.copy(self)
        moved.cords = list(self.cords)
        return moved.delta(addr)


class TmaLoad1D(_Tma1D):
    _OP = "OP_ALLOC_TMA_LOAD_1D"


class TmaStore1D(_Tma1D):
    _OP = "OP_ALLOC_WB_TMA_STORE_1D"


class TmaTensor(MemoryInstruction):
    """A tensor-map instruction template bound to one tensor: `wgmma` / `tensor1d` choose the map recipe and
    register the descriptor with the launcher, `.cord(...)` stamps out instructions at logical coordinates."""

    _OPS = {
        "load": {1: "OP_ALLOC_TMA_LOAD_TENSOR_1D", 2: "OP_ALLOC_TMA_LOAD_2D", 3: "OP_ALLOC_TMA_LOAD_3D",
                 4: "OP_ALLOC_TMA_LOAD_4D", 5: "OP_ALLOC_TMA_LOAD_5D_FIX0"},
        "store": {1: "OP_ALLOC_WB_TMA_STORE_1D", 2: "OP_ALLOC_WB_TMA_STORE_2D", 3: "OP_ALLOC_WB_TMA_STORE_3D",
                  4: "OP_ALLOC_WB_TMA_STORE_4D", 5: "OP_ALLOC_WB_TMA_STORE_5D_FIX0"},
        "reduce": {2: "OP_ALLOC_WB_TMA_REDUCE_ADD_2D", 3: "OP_ALLOC_WB_TMA_REDUCE_ADD_3D"},
    }

    def __init__(self, launcher, mat: torch.Tensor):
        super().__init__(0, 0, 0, 0)
        self.launcher = launcher
        self.mat = mat
        self.cord_func = None

    def _rank2opcode(self, rank: int, action: str) -> int:
        try:
            return getattr(opcode, self._OPS[action][rank])
        except KeyError as exc:
            raise ValueError(f"Unsupported rank {rank} and action {action}") from exc

    def _build(self, action, tileM, tileN, tma_func, cord_func_builder):
        self.mode = action
        self.size = self.mat.element_size() * tileM * tileN
        self.num_slots = bytes2slots(self.size)
        self.rank, self.desc = tma_func(self.mat, tileM, tileN)
        self.opcode = self._rank2opcode(self.rank, action)
        self.cord_func = cord_func_builder(self.mat, self.rank)
        if not hasattr(self.launcher, "new_tma"):
            raise ValueError("launcher must expose new_tma()")
        self.arg = self.launcher.new_tma(self.desc)
        return self

    def cord2tma(self, *cords):
        if self.cord_func is None:
            raise ValueError("cord_func is not set, please call wgmma_load/wgmma_store first")
        return self.cord_func(*cords)

    def cord(self, *cords):
        inst = copy.copy(self)
        inst.set_cords(self.cord2tma(*cords))
        return inst

    def tensor1d(self, action: str, size: int):
        assert action in ("load", "store"), f"action must be one of ['load', 'store'], got {action}"
        return self._build(action, size, 1, build_tma_1d, cord_func_tma_1d)

    def wgmma(self, action: str, tileN: int, tileM: int, major: Major):
        assert action in ("load", "store", "reduce"), f"action must be load, store or reduce, got {action}"
        if major == Major.K:
            return self._build(action, tileM, tileN, build_tma_wgmma_kmajor, cord_func_2d_kmajor)
        return self._build(action, tileM, tileN, build_tma_wgmma_mnmajor, cord_func_2d_mnmajor)

    def wgmma_load(self, tileN: int, tileM: int, major: Major):
        return self.wgmma("load", tileN, tileM, major)

    def wgmma_store(self, tileN: int, tileM: int, major: Major):
        return self.wgmma("store", tileN, tileM, major)


__all__ = [n for n, v in list(globals().items())
           if not n.startswith("_") and (isinstance(v, type) or callable(v)) and getattr(v, "__module__", "") == __name__]
__all__ += ["Major"]
