"""ISA constants for the host side, read from csrc/isa.h so that the header is
the single source of truth (a test checks them against the built library's
opcode table)."""
import os
import re

_H = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "isa.h")
_src = open(_H).read()

_defs = {}
for _m in re.finditer(r"^#define\s+VDC_(\w+)\s+(0x[0-9A-Fa-f]+|\d+)\s*(?://.*)?$", _src, re.M):
    _defs[_m.group(1)] = int(_m.group(2), 0)

SLOT_BYTES = _defs["SLOT_BYTES"]
NUM_SLOTS = _defs["NUM_SLOTS"]
NUM_SPECIAL_SLOTS = _defs["NUM_SPECIAL_SLOTS"]
MAX_INSTS = _defs["MAX_INSTS"]
MAX_SMS = _defs["MAX_SMS"]
NUM_PROFILE_EVENTS = _defs["NUM_PROFILE_EVENTS"]
MAX_TMAS = _defs["MAX_TMAS"]
MAX_BARS = _defs["MAX_BARS"]
QUEUE_LEN = _defs["QUEUE_LEN"]
COMPUTE_THREADS = _defs["COMPUTE_WARPS"] * 32
KV_PAGE = _defs["KV_PAGE"]
HEAD_DIM = _defs["HEAD_DIM"]
FLAG_BITS = _defs["FLAG_BITS"]

F_ALLOCATE, F_WRITEBACK, F_GROUP = _defs["F_ALLOCATE"], _defs["F_WRITEBACK"], _defs["F_GROUP"]
F_JUMP, F_BARRIER, F_PORT = _defs["F_JUMP"], _defs["F_BARRIER"], _defs["F_PORT"]

GEMV_MODE_STORE = _defs["GEMV_MODE_STORE"]
GEMV_MODE_SILU_PAIRS = _defs["GEMV_MODE_SILU_PAIRS"]
GEMV_MODE_ARGMAX = _defs["GEMV_MODE_ARGMAX"]
GEMV_MODE_STORE_F32 = _defs["GEMV_MODE_STORE_F32"]
GEMV_MODE_MOE_DOWN = _defs["GEMV_MODE_MOE_DOWN"]
GEMV_NORM_BIT = _defs["GEMV_NORM_BIT"]
GEMV_ACC_BIT = _defs["GEMV_ACC_BIT"]
GEMV_DYN_BIT = _defs["GEMV_DYN_BIT"]
GEMV_PEERS_BIT = _defs["GEMV_PEERS_BIT"]
GEMV_DYNROWS_BIT = _defs["GEMV_DYNROWS_BIT"]
GEMV_PARTIAL_BIT = _defs["GEMV_PARTIAL_BIT"]
GEMV_STRIDE_BIT = _defs["GEMV_STRIDE_BIT"]
TC_STAGES = _defs["TC_STAGES"]
STREAM_END = _defs["STREAM_END"]
ATTN_QKNORM_BIT = _defs["ATTN_QKNORM_BIT"]
ATTN_PACKED_BIT = _defs["ATTN_PACKED_BIT"]
ATTN_APPEND_BIT = _defs["ATTN_APPEND_BIT"]
ATTN_PAIR_BIT = _defs["ATTN_PAIR_BIT"]
GEMM_MODE_STORE_ROWS = _defs["GEMM_MODE_STORE_ROWS"]
GEMM_MODE_SILU_PAIRS = _defs["GEMM_MODE_SILU_PAIRS"]
GEMM_MODE_ARGMAX = _defs["GEMM_MODE_ARGMAX"]
GEMM_MODE_ADD_PACKED = _defs["GEMM_MODE_ADD_PACKED"]

ST_POS, ST_NPAGES, ST_TOKEN, ST_STEP = _defs["ST_POS"], _defs["ST_NPAGES"], _defs["ST_TOKEN"], _defs["ST_STEP"]
ST_NEWROW, ST_NKVH, ST_MAXPAGES, ST_ERR = _defs["ST_NEWROW"], _defs["ST_NKVH"], _defs["ST_MAXPAGES"], _defs["ST_ERR"]
ST_PAGETABLE = _defs["ST_PAGETABLE"]

OK, ERR_TIMEOUT, ERR_BAD_OPCODE, ERR_CUDA, ERR_ARG = (_defs[k] for k in
                                                       ("OK", "ERR_TIMEOUT", "ERR_BAD_OPCODE", "ERR_CUDA", "ERR_ARG"))

_flagval = {"VDC_F_ALLOCATE": F_ALLOCATE, "VDC_F_WRITEBACK": F_WRITEBACK, "0": 0}
OPCODES = {}
MEMORY_OPS, COMPUTE_OPS = [], []
for _m in re.finditer(r"X\((OP_\w+),\s*VDC_MOP\((\d+),\s*([^)]*)\)\)", _src):
    _flags = 0
    for _t in _m.group(3).split("|"):
        _flags |= _flagval[_t.strip()]
    OPCODES[_m.group(1)] = (int(_m.group(2)) << FLAG_BITS) | _flags
    MEMORY_OPS.append(_m.group(1))
OP_WORDS = {}      # compute opcode value -> 8-byte words it occupies before optional trailing words
for _m in re.finditer(r"X\((OP_\w+),\s*(0x[0-9A-Fa-f]+),\s*(\d+)\)", _src):
    OPCODES[_m.group(1)] = int(_m.group(2), 16)
    OP_WORDS[int(_m.group(2), 16)] = int(_m.group(3))
    COMPUTE_OPS.append(_m.group(1))
globals().update(OPCODES)


def op_id(opcode: int) -> int:
    return opcode >> FLAG_BITS
