"""Per-SM instruction streams for the decode megakernel.

A ``Program`` holds, for every SM, the memory-core stream (16-byte
instructions) and the compute-core stream (8-byte instructions) in the wire
format of the reference ISA (reference include/dae/context.cuh:51-113), and
derives the initial value of every global countdown barrier from the stores
that release it, the way the reference's launcher does from its schedules
(reference python/dae/schedule.py:39-55, python/dae/launcher.py:343-351).

The task helpers (``gemv``, ``attn_decode`` ...) emit the memory and the
compute instructions of one task on one SM in the order the device task pops
its operands.
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from . import isa

MINST = np.dtype([("opcode", "<u2"), ("size", "<u2"), ("num_slots", "<u2"), ("arg", "<u2"), ("address", "<u8")])
CINST = np.dtype([("opcode", "<u2"), ("a0", "<u2"), ("a1", "<u2"), ("a2", "<u2")])
assert MINST.itemsize == 16 and CINST.itemsize == 8

SLOT = isa.SLOT_BYTES


def slots_for(nbytes: int) -> int:
    return max(1, (nbytes + SLOT - 1) // SLOT)


def f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


@dataclass
class Src:
    """A 1-D bulk load: `nbytes` from device address `addr`.

    wait: global barrier id that must reach zero first (None: no wait).
    indirect: (word_address, shift, row_bytes): the address is offset by the
      32-bit word read at issue time, `word << shift` when row_bytes is None,
      `word * row_bytes` otherwise (embedding row / KV page gather)."""
    addr: int
    nbytes: int
    wait: Optional[int] = None
    indirect: Optional[tuple] = None
    port: Optional[int] = None


@dataclass
class Dst:
    """A write-back: bulk store (kind 'store') or bulk reduce-add ('add_bf16',
    'add_f32') of `nbytes` to `addr`; `release` names the barrier it counts
    down once the data is globally visible."""
    addr: int
    nbytes: int
    kind: str = "store"
    release: Optional[int] = None
    indirect: Optional[tuple] = None


class Program:
    def __init__(self, num_sms: int, insts_per_sm: int = isa.MAX_INSTS):
        self.num_sms = num_sms
        self.insts_per_sm = insts_per_sm
        self.m: List[list] = [[] for _ in range(num_sms)]
        self.c: List[list] = [[] for _ in range(num_sms)]
        self.bar_counts = {}
        self.bytes_loaded = [0] * num_sms       # bulk-load bytes issued per SM (for balancing)
        self._next_bar = 0
        self._finalized = False

    # ------------------------------------------------------------------ barriers
    def new_barrier(self) -> int:
        b = self._next_bar
        self._next_bar += 1
        if b >= isa.MAX_BARS:
            raise ValueError("out of global barriers")
        self.bar_counts[b] = 0
        return b

    # ------------------------------------------------------------------ raw emitters
    def mem(self, sm, opcode, *, size=0, nslot=0, bar=0, arg=0, address=0, flags=0, reg_range=None):
        if reg_range is not None:
            num_slots = (reg_range[0] & 0xFF) | ((reg_range[1] & 0xFF) << 8)
        else:
            assert 0 <= nslot < 64 and 0 <= bar < isa.MAX_BARS
            num_slots = nslot | (bar << 6)
        assert 0 <= size <= 0xFFFF and 0 <= arg <= 0xFFFF
        self.m[sm].append((opcode | flags, size, num_slots, arg, address & 0xFFFFFFFFFFFFFFFF))

    def comp(self, sm, opcode, a0=0, a1=0, a2=0):
        for a in (a0, a1, a2):
            assert 0 <= a <= 0xFFFF, a
        self.c[sm].append((opcode, a0, a1, a2))

    # ------------------------------------------------------------------ operand emitters
    def load(self, sm, src: Src, default_port=0):
        assert src.nbytes % 16 == 0 and src.addr % 16 == 0, (src.nbytes, src.addr)
        assert 0 < src.nbytes <= 32768
        if src.indirect is not None:
            waddr, shift, row_bytes = src.indirect
            if row_bytes is None:
                self.mem(sm, isa.OP_CC0, arg=shift, address=waddr)
            else:
                self.mem(sm, isa.OP_CC0_ROW_BYTES, size=row_bytes, address=waddr)
        flags = 0
        port = src.port if src.port is not None else (1 if src.wait is not None else default_port)
        if port:
            flags |= isa.F_PORT
        bar = 0
        if src.wait is not None:
            flags |= isa.F_BARRIER
            bar = src.wait
        self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=src.nbytes, nslot=slots_for(src.nbytes), bar=bar,
                 address=src.addr, flags=flags)
        self.bytes_loaded[sm] += src.nbytes

    def load_x(self, sm, src: Src):
        """An activation vector for a compute task.  A plain source becomes an XVEC hand-over: slots are
        allocated, the task waits for `src.wait` itself and copies the vector from global memory with
        ordinary loads.  A gathered source (an embedding row) still goes through the copy engine."""
        if src.indirect is not None:
            return self.load(sm, src, default_port=1)
        assert src.nbytes % 16 == 0 and src.addr % 16 == 0 and 0 < src.nbytes <= 32768
        flags, bar = 0, 0
        if src.wait is not None:
            flags, bar = isa.F_BARRIER, src.wait
        self.mem(sm, isa.OP_ALLOC_XVEC, size=src.nbytes, nslot=slots_for(src.nbytes), bar=bar, address=src.addr,
                 flags=flags)

    def store(self, sm, dst: Dst):
        assert dst.nbytes % 16 == 0 and dst.addr % 16 == 0, (dst.nbytes, dst.addr)
        assert 0 < dst.nbytes <= SLOT * 4
        if dst.indirect is not None:
            waddr, shift, row_bytes = dst.indirect
            if row_bytes is None:
                self.mem(sm, isa.OP_CC0, arg=shift, address=waddr)
            else:
                self.mem(sm, isa.OP_CC0_ROW_BYTES, size=row_bytes, address=waddr)
        flags, bar, arg = 0, 0, 0
        if dst.release is not None:
            flags |= isa.F_BARRIER
            bar = dst.release
            self.bar_counts[bar] += 1
        if dst.kind == "store":
            op = isa.OP_ALLOC_WB_TMA_STORE_1D
        elif dst.kind == "add_bf16":
            op = isa.OP_ALLOC_WB_TMA_REDUCE_ADD_1D
        elif dst.kind == "add_f32":
            op, arg = isa.OP_ALLOC_WB_TMA_REDUCE_ADD_1D, 1
        else:
            raise ValueError(dst.kind)
        self.mem(sm, op, size=dst.nbytes, nslot=slots_for(dst.nbytes), bar=bar, arg=arg, address=dst.addr, flags=flags)

    def raw_address(self, sm, addr, special_slot, release=None, wait=None):
        """Hands a 64-bit value to the compute task through special slot
        `special_slot` (24..32).  With `release` the store warp counts that
        barrier down when the task pushes the slot back; with `wait` the load
        port holds the hand-over until that barrier reached zero."""
        assert isa.NUM_SLOTS <= special_slot < isa.NUM_SLOTS + isa.NUM_SPECIAL_SLOTS
        flags, bar = 0, 0
        if release is not None:
            flags |= isa.F_BARRIER | isa.F_WRITEBACK
            bar = release
            self.bar_counts[bar] += 1
        elif wait is not None:
            flags |= isa.F_BARRIER | isa.F_PORT
            bar = wait
        self.mem(sm, isa.OP_ALLOC_WB_RAW_ADDRESS, nslot=special_slot, bar=bar, arg=special_slot, address=addr,
                 flags=flags)

    def repeat(self, sm, count, deltas, dynamic=False):
        """Loop header for the next len(deltas) memory instructions: instruction
        i gets `address += iteration * deltas[i]`.  The caller sets F_JUMP on the
        last body instruction.  dynamic: the count comes from the last DYN_COUNT."""
        n = len(deltas)
        assert 1 <= n <= 32
        # one header per run of equal consecutive deltas; the last header carries the count
        runs = []
        for i, d in enumerate(deltas):
            if runs and runs[-1][2] == d:
                runs[-1][1] = i + 1
            else:
                runs.append([i, i + 1, d])
        for k, (lo, hi, d) in enumerate(runs):
            last = k == len(runs) - 1
            size = (0xFFFF if dynamic else count) if last else 0
            self.mem(sm, isa.OP_REPEAT, size=size, arg=(n if (last and dynamic) else 0), address=d,
                     reg_range=(lo, hi))

    def prefetch_l2(self, sm, addr, nbytes):
        """Pulls [addr, addr+nbytes) into L2 (no shared-memory slot, no completion)."""
        assert addr % 16 == 0 and nbytes % 16 == 0
        while nbytes > 0:
            n = min(nbytes, 65536)
            self.mem(sm, isa.OP_PREFETCH_L2, size=n & 0xFFFF, arg=n >> 16, address=addr)
            addr += n
            nbytes -= n

    def stream_list(self, sm, list_addr, n_segments, window_bytes):
        """Starts the SM's HBM->L2 streamer on a device array of n_segments
        {u64 address, u32 bytes, u32 pad} records: the weight bytes this SM will
        load with stream=True, in order."""
        assert n_segments <= 0xFFFF and window_bytes % 1024 == 0 and window_bytes >> 10 <= 0xFFFF
        self.mem(sm, isa.OP_STREAM_LIST, size=n_segments, address=list_addr, reg_range=None)
        op, size, _, arg, addr = self.m[sm][-1]
        self.m[sm][-1] = (op, size, window_bytes >> 10, arg, addr)

    def l2_prefetch(self, sm, addr, nbytes):
        """Compute-stream hint: when the compute core reaches this point all its
        threads issue L2 prefetches for [addr, addr+nbytes) and continue."""
        assert 0 <= addr < 1 << 48 and 0 < nbytes < 1 << 32
        self.comp(sm, isa.OP_L2_PREFETCH, addr & 0xFFFF, (addr >> 16) & 0xFFFF, (addr >> 32) & 0xFFFF)
        self.comp(sm, isa.OP_EXT, nbytes & 0xFFFF, nbytes >> 16, 0)

    def dyn_count(self, sm, word_addr, base, maximum):
        self.mem(sm, isa.OP_DYN_COUNT, size=maximum, address=word_addr, reg_range=None, nslot=0, bar=0)
        # base travels in the num_slots field
        op, size, _, arg, addr = self.m[sm][-1]
        assert 0 <= base <= 0xFFFF
        self.m[sm][-1] = (op, size, base, arg, addr)

    # ------------------------------------------------------------------ tensor-map copies, registers, loops
    @staticmethod
    def _coords(coords):
        assert 1 <= len(coords) <= 4 and all(0 <= c < 0xFFFF for c in coords)
        c = list(coords) + [0] * (4 - len(coords))
        return c[0] | (c[1] << 16) | (c[2] << 32) | (c[3] << 48)

    def tensor_load(self, sm, *, tma_id, rank, coords, nbytes, wait=None, port=0, group=False, jump=False):
        """Tiled `cp.async.bulk.tensor` load of one box of tensor map `tma_id` (rank 1..5; a rank-5 map takes
        four coordinates, its innermost one is fixed to 0) at `coords` (innermost first) into fresh slots.
        group: the map id and the barrier id shift with the enclosing LOOP (reference
        python/dae/instructions.py TmaTensor, include/dae/pipeline/ldwarp.cuh:63-168)."""
        op = {1: isa.OP_ALLOC_TMA_LOAD_TENSOR_1D, 2: isa.OP_ALLOC_TMA_LOAD_2D, 3: isa.OP_ALLOC_TMA_LOAD_3D,
              4: isa.OP_ALLOC_TMA_LOAD_4D, 5: isa.OP_ALLOC_TMA_LOAD_5D_FIX0}[rank]
        flags = (isa.F_PORT if port else 0) | (isa.F_GROUP if group else 0) | (isa.F_JUMP if jump else 0)
        bar = 0
        if wait is not None:
            flags |= isa.F_BARRIER
            bar = wait
        self.mem(sm, op, size=nbytes, nslot=slots_for(nbytes), bar=bar, arg=tma_id, address=self._coords(coords),
                 flags=flags)
        self.bytes_loaded[sm] += nbytes

    def tensor_store(self, sm, *, tma_id, rank, coords, nbytes, reduce=False, release=None, group=False, jump=False,
                     n_releases=1):
        """Tiled store (or reduce-add, ranks 2 and 3: the element type comes from the map) of the slots a task
        writes back (reference include/dae/pipeline/stwarp.cuh:38-145).  n_releases: how many times the
        instruction executes (a loop body), for the barrier's initial count."""
        if reduce:
            op = {2: isa.OP_ALLOC_WB_TMA_REDUCE_ADD_2D, 3: isa.OP_ALLOC_WB_TMA_REDUCE_ADD_3D}[rank]
        else:
            op = {2: isa.OP_ALLOC_WB_TMA_STORE_2D, 3: isa.OP_ALLOC_WB_TMA_STORE_3D, 4: isa.OP_ALLOC_WB_TMA_STORE_4D,
                  5: isa.OP_ALLOC_WB_TMA_STORE_5D_FIX0}[rank]
        flags = (isa.F_GROUP if group else 0) | (isa.F_JUMP if jump else 0)
        bar = 0
        if release is not None:
            flags |= isa.F_BARRIER
            bar = release
            if not group:
                self.bar_counts[bar] += n_releases
        self.mem(sm, op, size=nbytes, nslot=slots_for(nbytes), bar=bar, arg=tma_id, address=self._coords(coords),
                 flags=flags)

    def reg_store(self, sm, reg, nbytes):
        """Slots for a task's result that stays in shared memory: the producing task's write-back is skipped,
        a later reg_load(reg) hands the same slots to the consuming task, which frees them (reference
        python/dae/instructions.py RegStore / RegLoad, include/dae/pipeline/ldwarp.cuh:169-183)."""
        assert 0 <= reg < 4
        self.mem(sm, isa.OP_ALLOC_WB_REG_STORE, size=reg, nslot=slots_for(nbytes))

    def reg_load(self, sm, reg, special_slot=None):
        assert 0 <= reg < 4
        slot = isa.NUM_SLOTS + (reg if special_slot is None else special_slot)
        self.mem(sm, isa.OP_ALLOC_REG_LOAD, size=reg, nslot=slot)

    def loop_m(self, sm, count, pc, *, bar_shift=0, tma_shift=0, reg=0):
        """Memory-stream loop: jumps back to instruction `pc` count-1 times; before every further trip the
        barrier ids and tensor-map ids of GROUP-flagged instructions move on by bar_shift / tma_shift
        (reference python/dae/instructions.py LoopM, include/dae/pipeline/allocwarp.cuh:148-166)."""
        assert 0 <= reg < 32 and 0 <= bar_shift < 1024 and 0 <= tma_shift < 1 << 16 and 0 <= pc < 0xFFFF
        self.m[sm].append((isa.OP_LOOP, count, reg, 0, pc | ((bar_shift << 6) << 32) | (tma_shift << 48)))

    def loop_c(self, sm, count, pc):
        """Compute-stream loop: jumps back to compute instruction `pc` count-1 times (reference LoopC,
        include/dae/compute_dispatch.cuh:311-321)."""
        self.comp(sm, isa.OP_LOOPC, count, pc)

    # ------------------------------------------------------------------ tasks
    def copy(self, sm, src: Src, dst: Dst, nbytes: int):
        self.load(sm, src)
        self.store(sm, dst)
        self.comp(sm, isa.OP_COPY, 1, nbytes // 4)

    def gemv(self, sm, *, w_addr, n_rows, K, R, x: Src, out: Dst, mode=isa.GEMV_MODE_STORE,
             norm_w: Optional[Src] = None, eps: float = 0.0, pair_out: Optional[Dst] = None, row_base: int = 0,
             stream: bool = False, fp8_scales: Optional[int] = None, nvfp4_scales: Optional[int] = None,
             w_indirect: Optional[tuple] = None, wait_issue: Optional[int] = None, moe: Optional[dict] = None,
             dyn_count_addr: Optional[int] = None, peers: Optional[tuple] = None, shared_counter: Optional[int] = None,
             own_chunks: Optional[tuple] = None, shared_first: int = 0, shared_depth: int = 0,
             partial_in: Optional[int] = None, chunk_stride: int = 1):
        """y[0:n_rows] = W[0:n_rows, :K] @ x for the contiguous row block at w_addr
        (bf16; e4m3 with fp8_scales = address of the block's fp32 per-row scales;
        or NVFP4 rows — K/2 code bytes + K/16 block scales — with nvfp4_scales =
        address of the fp32 per-row tensor scales), streamed as chunks of R rows.  The task writes y straight to
        out.addr (kind 'store') or adds it there (kind 'add_bf16'); in SILU_PAIRS
        mode rows (2j, 2j+1) are (gate_j, up_j) and n_rows/2 values are written.
        shared_counter: a barrier id used as a counter that starts at 0.  w_addr / n_rows / out / scales then
        describe the WHOLE matrix on every SM that runs the task: the SM first streams the chunks it owns
        (own_chunks = (first, count)), then draws chunks shared_first, shared_first + 1, ... from the counter
        until the matrix is exhausted, never holding more than shared_depth unconsumed ring entries when it
        draws (0: no limit), so the SMs that finish early take the tail of the stage.
        partial_in: address of fp32 sums of the same rows over another K-range (written by an earlier STORE_F32
        task of this SM); they are added to the task's sums before the result is rounded.
        chunk_stride s > 1: the task's chunk i is chunk i * s of the matrix that starts at w_addr (rows, outputs
        and scales likewise): the chunks of a stage dealt round-robin to s SMs; n_rows counts the task's own rows."""
        assert fp8_scales is None or nvfp4_scales is None
        if nvfp4_scales is not None:
            row_bytes, kmult, op, scales = K // 2 + K // 16, 1024, isa.OP_GEMV_ROWS_NVFP4, nvfp4_scales
        elif fp8_scales is not None:
            row_bytes, kmult, op, scales = K, 512, isa.OP_GEMV_ROWS_FP8, fp8_scales
        else:
            row_bytes, kmult, op, scales = 2 * K, 256, isa.OP_GEMV_ROWS_BF16, None
        assert K % kmult == 0 and row_bytes * R <= 32768 and R in (1, 2, 4, 8, 16)
        assert n_rows % R == 0 and n_rows > 0
        assert mode != isa.GEMV_MODE_SILU_PAIRS or R % 2 == 0
        assert out.kind in ("store", "add_bf16") and out.addr % 2 == 0
        assert mode != isa.GEMV_MODE_STORE_F32 or (out.kind == "store" and out.addr % 4 == 0)
        n_chunks = n_rows // R
        assert n_chunks < 0xFFFF
        chunk_bytes = R * row_bytes
        assert x.nbytes == K * 2
        if norm_w is not None:
            self.load(sm, norm_w, default_port=1)
        self.load_x(sm, x)
        self.raw_address(sm, out.addr, 24, release=out.release)
        if mode == isa.GEMV_MODE_ARGMAX:
            assert pair_out is not None and row_base % R == 0
            self.raw_address(sm, pair_out.addr, 25, release=pair_out.release)
        if wait_issue is not None:
            # the weight address depends on data another SM produces (an expert id): the memory
            # stream of this SM stops here until that barrier has opened
            self.mem(sm, isa.OP_ISSUE_BARRIER, bar=wait_issue)
        if dyn_count_addr is not None:
            # the task takes min(n_chunks, word) chunks (an expert of another rank: none); the hand-over
            # of the word's address follows the barrier that orders the word
            assert wait_issue is not None
            self.raw_address(sm, dyn_count_addr, 27)
        if w_indirect is not None:
            waddr, stride = w_indirect
            assert 0 < stride < 1 << 32
            if dyn_count_addr is not None:
                self.dyn_count(sm, dyn_count_addr, 0, n_chunks)
            self.mem(sm, isa.OP_CC0_STRIDE32, size=stride & 0xFFFF, arg=stride >> 16, address=waddr)
        elif dyn_count_addr is not None:
            self.dyn_count(sm, dyn_count_addr, 0, n_chunks)
        if shared_counter is not None:
            assert dyn_count_addr is None and w_indirect is None and moe is None and peers is None and row_base == 0
            assert shared_counter in self.bar_counts and self.bar_counts[shared_counter] == 0
            own_first, own_n = own_chunks if own_chunks is not None else (0, 0)
            n_shared = n_chunks - shared_first
            assert 0 <= own_first and own_first + own_n <= shared_first <= n_chunks and 0 <= shared_depth < 1 << 16
            if own_n:
                self.repeat(sm, own_n, [chunk_bytes])
                self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=chunk_bytes, nslot=slots_for(chunk_bytes),
                         address=w_addr + own_first * chunk_bytes, flags=isa.F_JUMP)
            self.mem(sm, isa.OP_DYN_CHUNKS, size=n_shared & 0xFFFF, arg=n_shared >> 16, bar=shared_counter,
                     address=shared_depth)
            self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=chunk_bytes, nslot=slots_for(chunk_bytes),
                     address=w_addr + shared_first * chunk_bytes)
            self.bytes_loaded[sm] += chunk_bytes * (own_n + n_shared // max(1, self.num_sms))
        else:
            self.repeat(sm, n_chunks, [chunk_bytes * chunk_stride], dynamic=dyn_count_addr is not None)
            self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D_STREAM if stream else isa.OP_ALLOC_TMA_LOAD_1D, size=chunk_bytes,
                     nslot=slots_for(chunk_bytes), address=w_addr, flags=isa.F_JUMP)
            self.bytes_loaded[sm] += chunk_bytes * n_chunks
        rb8 = row_base // R     # index of the first chunk within the whole matrix
        a1 = R | (mode << 8) | (isa.GEMV_NORM_BIT if norm_w is not None else 0) | \
            (isa.GEMV_ACC_BIT if out.kind == "add_bf16" else 0) | (isa.GEMV_DYN_BIT if dyn_count_addr is not None else 0) | \
            (isa.GEMV_PEERS_BIT if peers is not None else 0) | (isa.GEMV_DYNROWS_BIT if shared_counter is not None else 0) | \
            (isa.GEMV_PARTIAL_BIT if partial_in is not None else 0) | (isa.GEMV_STRIDE_BIT if chunk_stride > 1 else 0)
        assert chunk_stride == 1 or (shared_counter is None and moe is None and peers is None and 1 < chunk_stride <= 0xFFFF)
        a2 = (K // 256) | ((rb8 >> 16) << 8)
        e = f32_bits(eps)
        if moe is not None:
            assert mode == isa.GEMV_MODE_MOE_DOWN and scales is None
            self.comp(sm, isa.OP_GEMV_ROWS_MOE_DOWN, n_chunks, a1, a2)
            self.comp(sm, isa.OP_EXT, e >> 16, e & 0xFFFF, moe["top_k"])
            for addr in (moe["weight_addr"], moe["acc_addr"], moe["cnt_addr"]):   # acc_addr 0: fp32 partial-sum output
                assert addr % 4 == 0 and 0 <= addr < 1 << 48
                self.comp(sm, isa.OP_EXT, addr & 0xFFFF, (addr >> 16) & 0xFFFF, (addr >> 32) & 0xFFFF)
            return
        self.comp(sm, op, n_chunks, a1, a2)
        self.comp(sm, isa.OP_EXT, e >> 16, e & 0xFFFF, rb8 & 0xFFFF)
        if scales is not None:
            assert scales % 4 == 0 and 0 <= scales < 1 << 48
            self.comp(sm, isa.OP_EXT, scales & 0xFFFF, (scales >> 16) & 0xFFFF, (scales >> 32) & 0xFFFF)
        if chunk_stride > 1:
            self.comp(sm, isa.OP_EXT, chunk_stride, 0, 0)
        if partial_in is not None:
            assert moe is None and partial_in % 4 == 0 and 0 < partial_in < 1 << 48
            self.comp(sm, isa.OP_EXT, partial_in & 0xFFFF, (partial_in >> 16) & 0xFFFF, (partial_in >> 32) & 0xFFFF)
        if peers is not None:
            # (table address, ranks, counter byte offset): out.addr is then the byte offset of the task's
            # first row inside an exchange block, the rows go to every rank's block
            assert mode == isa.GEMV_MODE_STORE_F32
            self._peer_words(sm, peers)
        if shared_counter is not None:
            assert 0 < w_addr < 1 << 48
            self.comp(sm, isa.OP_EXT, w_addr & 0xFFFF, (w_addr >> 16) & 0xFFFF, (w_addr >> 32) & 0xFFFF)

    def _peer_words(self, sm, peers):
        """peers = (address of the table {every rank's exchange block base, state block}, ranks, exchange number,
        exchanges per step)."""
        table, n, ex, n_ex = peers
        assert 0 <= table < 1 << 48 and table % 8 == 0 and 1 <= n <= 255 and 0 <= ex < n_ex <= 0xFFFF
        self.comp(sm, isa.OP_EXT, table & 0xFFFF, (table >> 16) & 0xFFFF, (table >> 32) & 0xFFFF)
        self.comp(sm, isa.OP_EXT, n, ex, n_ex)

    def xreduce(self, sm, *, n, n_ranks, xbuf_addr, hidden_elems, ex, n_ex, hidden_addr, state_addr,
                release: Optional[int] = None):
        """hidden[i] = bf16(hidden[i] + sum over ranks of the partial sums) for n elements: xbuf_addr is this
        rank's first tagged entry {fp32 bits, tag} of rank 0 for the slice, the ranks' entry arrays lie
        hidden_elems entries apart; every entry is polled until it carries the tag of exchange `ex` of the
        current step (state.STEP * n_ex + ex + 1)."""
        assert 0 < n <= 0xFFFF and hidden_elems % 2 == 0 and hidden_elems // 2 <= 0xFFFF and 0 <= ex < n_ex <= 0xFFFF
        if release is not None:
            self.bar_counts[release] += 1
        a48 = lambda a: (a & 0xFFFF, (a >> 16) & 0xFFFF, (a >> 32) & 0xFFFF)
        self.comp(sm, isa.OP_XREDUCE, n, n_ranks, 0xFFFF if release is None else release)
        self.comp(sm, isa.OP_EXT, *a48(xbuf_addr))
        self.comp(sm, isa.OP_EXT, hidden_elems // 2, ex, n_ex)
        for a in (hidden_addr, state_addr):
            assert 0 <= a < 1 << 48
            self.comp(sm, isa.OP_EXT, *a48(a))

    def xwait(self, sm, *, n_ranks, ex, n_ex, entries_addr, state_addr, records_addr, release: int):
        """Waits for the ranks' candidate entries ({value, tag}, {row index, tag} per rank) of exchange `ex`,
        writes them as compact records {f32, i32, 0, 0} to records_addr and counts `release` down."""
        assert 0 < n_ranks <= 128 and 0 <= ex < n_ex <= 0xFFFF
        self.bar_counts[release] += 1
        a48 = lambda a: (a & 0xFFFF, (a >> 16) & 0xFFFF, (a >> 32) & 0xFFFF)
        self.comp(sm, isa.OP_XWAIT, release, n_ranks, ex)
        for a in (entries_addr, state_addr, records_addr):
            assert 0 <= a < 1 << 48
            self.comp(sm, isa.OP_EXT, *a48(a))
        self.comp(sm, isa.OP_EXT, n_ex, 0, 0)

    def add_releases(self, bar: int, n: int):
        """Declares n count-downs of `bar` that tasks perform themselves (not
        through a store instruction), so that its initial value includes them."""
        self.bar_counts[bar] += n

    def attn_decode(self, sm, *, G, state_addr, rope: Src, norm_w: Optional[Src], qkv: Src, k_page_addr, v_page_addr,
                    page_shift, base_page, max_pages, records_addr, counter_addr, out_addr, split, n_splits,
                    release, qk_eps: float = 1e-6, packed: Optional[tuple] = None, append: bool = False,
                    wait_issue: Optional[int] = None, pair: Optional[tuple] = None):
        """One (KV head, split) unit of the decode attention.  k_page_addr /
        v_page_addr: this head's rows inside page 0 of the layer's K / V pool;
        the page table in the state block selects the page.  The unit that
        completes the head last merges the n_splits records at records_addr,
        writes G*128 bf16 to out_addr and counts `release` down once (declare it
        with add_releases(release, 1) per head).  packed=(b, Bpad): out_addr is the
        head's first k group inside a k-chunk-major [Bpad, q_width] matrix and the
        outputs go to its row b (batched decode).  append: the unit only writes the new key / value rows to the
        pools and counts `release` down (max_pages must be 0).  wait_issue: the page loads are not issued before
        this barrier opens (pages that tasks of the same launch are still writing: chunked prefill).
        pair=(state_stride_words, qkv_stride_elems): G must be 8 and the model's group 4; the unit serves the
        position of state_addr / qkv and the next one (their state block and projection row lie that far on), both
        with their cache rows in the pools already; needs `packed`, whose b is the first position's slot."""
        page_bytes = isa.KV_PAGE * isa.HEAD_DIM * 2
        assert not append or max_pages == 0
        g_row = G // 2 if pair else G       # query heads in one projection row's head group
        assert pair is None or (G == 8 and packed is not None and not append and pair[0] <= 0xFFFF
                                and pair[1] % 8 == 0 and pair[1] // 8 <= 0xFFFF)
        if wait_issue is not None and max_pages:
            self.mem(sm, isa.OP_ISSUE_BARRIER, bar=wait_issue)
        assert qkv.nbytes == (g_row + 2) * isa.HEAD_DIM * 2 and qkv.addr % 16 == 0 and qkv.indirect is None
        # the rope row is table + position * 512 bytes: the task reads the position from the state block itself
        assert rope.indirect is None or (rope.indirect[0] == state_addr + 4 * isa.ST_POS and rope.indirect[1] == 9)
        # The page ids of up to 32 pages are fetched with one load (a word per lane of the control
        # warp); each trip of the loop then takes its page from there, so no load sits between
        # two page copies.  Longer ranges are cut into segments of 32 pages.
        for seg in range(0, max_pages, 32):
            n = min(32, max_pages - seg)
            self.dyn_count(sm, state_addr + 4 * isa.ST_NPAGES, base_page + seg, n)
            self.mem(sm, isa.OP_PT_LOAD32, size=n, address=state_addr + 4 * (isa.ST_PAGETABLE + base_page + seg))
            self.repeat(sm, 0, [0, 0, 0, 0], dynamic=True)
            self.mem(sm, isa.OP_PT_APPLY, arg=page_shift)
            self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=page_bytes, nslot=slots_for(page_bytes), address=k_page_addr)
            self.mem(sm, isa.OP_PT_APPLY, arg=page_shift)
            self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=page_bytes, nslot=slots_for(page_bytes), address=v_page_addr,
                     flags=isa.F_JUMP)
        self.bytes_loaded[sm] += 2 * page_bytes * max_pages
        e = f32_bits(qk_eps)
        op = isa.OP_ATTN_DECODE_PAGED_G4 if G == 4 else isa.OP_ATTN_DECODE_PAGED_G8
        flags = ((isa.ATTN_QKNORM_BIT if norm_w is not None else 0) | (isa.ATTN_PACKED_BIT if packed else 0) |
                 (isa.ATTN_APPEND_BIT if append else 0) | (isa.ATTN_PAIR_BIT if pair else 0))
        self.comp(sm, op, max_pages, base_page, flags)
        self.comp(sm, isa.OP_EXT, e >> 16, e & 0xFFFF, n_splits)
        a48 = lambda a: (a & 0xFFFF, (a >> 16) & 0xFFFF, (a >> 32) & 0xFFFF)
        for addr in (state_addr, k_page_addr, v_page_addr, records_addr, counter_addr, out_addr):
            assert 0 <= addr < 1 << 48
            self.comp(sm, isa.OP_EXT, *a48(addr))
        self.comp(sm, isa.OP_EXT, split, release, (packed[0] | (packed[1] // 16) << 8) if packed else 0)
        for addr in (rope.addr, norm_w.addr if norm_w is not None else 0, qkv.addr):
            assert 0 <= addr < 1 << 48
            self.comp(sm, isa.OP_EXT, *a48(addr))
        self.comp(sm, isa.OP_EXT, 0xFFFF if qkv.wait is None else qkv.wait, pair[0] if pair else 0,
                  pair[1] // 8 if pair else 0)

    # ------------------------------------------------------------------ batched decode (tensor cores)
    def gemm_tc(self, sm, *, w_addr, N, K, k_len, Kc, G, x_addr, B, Bpad, out_addr, mode, x_wait: Optional[int] = None,
                norm_w: Optional[Src] = None, eps: float = 0.0, n0: int = 0, ld: int = 0, keys_addr: int = 0,
                stats_addr: int = 0, release: Optional[int] = None, scratch_addr: int = 0, counter_addr: int = 0,
                n_slices: int = 1, wfmt: str = "bf16", scales_addr: int = 0):
        """One unit of a batched projection: D[b, n] = sum_k X[b, k] W[n, k] over a K-range
        of k_len inputs for a block of N weight rows (k-chunk-major [K/8][N/8][8][8] bf16;
        w_addr points at the range's first W chunk) against the k-chunk-major activation
        matrix (x_addr points at the range's first k group).  The range is streamed as
        W chunks of Kc inputs, G of them per X chunk.  `mode` selects the epilogue
        (isa.GEMM_MODE_*); n0 is the block's first output row; K the projection's whole K.
        stats_addr: fp32 per-sequence sums of squares, read when norm_w (the norm weights
        of the range) is given, accumulated over the updated rows in ADD_PACKED mode.
        With n_slices > 1 the block's K is shared by that many units: partial sums meet in
        scratch_addr, counter_addr counts arrivals.  The caller declares `release` once per
        block with add_releases.  wfmt "fp8": the weights are e4m3 bytes (chunk layout
        [Kc/16][N/8][8][16]) with fp32 per-row scales at scales_addr; wfmt "nvfp4": per 16 inputs
        [N rows x 8 bytes of e2m1 pairs | N e4m3 block scales], fp32 per-row (tensor) scales at
        scales_addr; isa.TC_STAGES bf16 staging buffers are allocated for the task in both cases."""
        assert wfmt in ("bf16", "fp8", "nvfp4") and (wfmt == "bf16" or (scales_addr and scales_addr % 16 == 0))
        wb16 = {"bf16": 32, "fp8": 16, "nvfp4": 9}[wfmt]       # bytes per 16 weights of one row
        assert N % 16 == 0 and 16 <= N <= 256 and Bpad in (16, 32, 64, 128) and 1 <= B <= Bpad
        assert Kc % 16 == 0 and k_len % Kc == 0 and k_len > 0 and n0 % 16 == 0 and ld % 16 == 0 and K % 16 == 0
        assert norm_w is None or stats_addr
        assert n_slices == 1 or (scratch_addr and counter_addr)
        n_w = k_len // Kc
        wbytes = N * Kc * wb16 // 16
        assert N * Kc * 2 <= 32768 and n_w <= 0xFFFF and 1 <= G <= 15 and Kc // 16 <= 255
        assert Bpad * G * Kc * 2 <= 32768
        wslots = slots_for(wbytes)
        if norm_w is not None:
            assert norm_w.nbytes == k_len * 2
            self.load(sm, norm_w, default_port=1)
        if wfmt != "bf16":
            for _ in range(isa.TC_STAGES):      # staging buffers: slots only, nothing is loaded or stored
                self.mem(sm, isa.OP_ALLOC_WB_TMA_STORE_1D, size=0, nslot=slots_for(N * Kc * 2), address=0)

        def group(first_w, count, wait=None, jump=False):
            # one X chunk and the `count` W chunks that go with it
            xb = Bpad * count * Kc * 2
            flags = isa.F_PORT | (isa.F_BARRIER if wait is not None else 0)
            self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=xb, nslot=slots_for(xb), bar=wait or 0,
                     address=x_addr + first_w * Kc * Bpad * 2, flags=flags)
            for i in range(count):
                self.mem(sm, isa.OP_ALLOC_TMA_LOAD_1D, size=wbytes, nslot=wslots, address=w_addr + (first_w + i) * wbytes,
                         flags=isa.F_JUMP if (jump and i == count - 1) else 0)

        n_full, tail = divmod(n_w, G)
        if n_full == 0:
            group(0, tail, wait=x_wait)
        else:
            group(0, G, wait=x_wait)          # the first X chunk carries the wait on the producers
            if n_full > 1:
                self.repeat(sm, n_full - 1, [Bpad * G * Kc * 2] + [G * wbytes] * G)
                group(G, G, jump=True)
            if tail:
                group(n_full * G, tail)
        self.bytes_loaded[sm] += (Bpad * Kc * 2 + wbytes) * n_w
        e = f32_bits(eps)
        a48 = lambda a: (a & 0xFFFF, (a >> 16) & 0xFFFF, (a >> 32) & 0xFFFF)
        for a in (out_addr, keys_addr, stats_addr, scratch_addr, counter_addr, scales_addr):
            assert 0 <= a < 1 << 48
        assert out_addr % 16 == 0 and keys_addr % 8 == 0 and stats_addr % 4 == 0 and scratch_addr % 16 == 0
        self.comp(sm, isa.OP_GEMM_TC_BF16, n_w, (N // 16) | (mode << 8) | ((1 << 12) if norm_w is not None else 0) |
                  ({"bf16": 0, "fp8": 1, "nvfp4": 2}[wfmt] << 13), (Kc // 16) | (G << 8))
        self.comp(sm, isa.OP_EXT, e >> 16, e & 0xFFFF, B)
        self.comp(sm, isa.OP_EXT, *a48(out_addr))
        self.comp(sm, isa.OP_EXT, *a48(keys_addr))
        self.comp(sm, isa.OP_EXT, n0 & 0xFFFF, n0 >> 16, 0xFFFF if release is None else release)
        self.comp(sm, isa.OP_EXT, ld // 16, Bpad, K // 16)
        self.comp(sm, isa.OP_EXT, *a48(stats_addr))
        self.comp(sm, isa.OP_EXT, *a48(scratch_addr))
        self.comp(sm, isa.OP_EXT, *a48(counter_addr))
        self.comp(sm, isa.OP_EXT, n_slices, 0, 0)
        self.comp(sm, isa.OP_EXT, *a48(scales_addr))

    def embed_pack(self, sm, *, b0, count, Bpad, state_addr, state_stride_words, hidden, table_addr, out_addr,
                   stats_addr, release: Optional[int] = None):
        """Copies embedding row state[b].TOKEN of sequences b0..b0+count-1 into row b
        of the k-chunk-major [Bpad, hidden] matrix at out_addr."""
        assert hidden % 8 == 0 and hidden // 8 <= 0xFFFF and state_stride_words <= 0xFFFF
        if release is not None:
            self.bar_counts[release] += 1
        a48 = lambda a: (a & 0xFFFF, (a >> 16) & 0xFFFF, (a >> 32) & 0xFFFF)
        self.comp(sm, isa.OP_EMBED_PACK, b0, count, Bpad)
        self.comp(sm, isa.OP_EXT, state_stride_words, hidden // 8, 0xFFFF if release is None else release)
        for a in (state_addr, table_addr, out_addr, stats_addr):
            assert 0 <= a < 1 << 48
            self.comp(sm, isa.OP_EXT, *a48(a))

    def batch_advance(self, sm, *, batch, state_addr, state_stride_words, keys_addr, log_addr, log_stride, wait,
                      stats_addr=0, n_stats=0):
        """Turns the argmax keys into next tokens, logs them and advances every
        sequence's state block, once barrier `wait` has opened."""
        assert batch <= isa.COMPUTE_THREADS and log_stride <= 0xFFFF and state_stride_words <= 0xFFFF
        self.raw_address(sm, state_addr, 25, wait=wait)
        a48 = lambda a: (a & 0xFFFF, (a >> 16) & 0xFFFF, (a >> 32) & 0xFFFF)
        self.comp(sm, isa.OP_BATCH_ADVANCE, batch, state_stride_words, log_stride)
        self.comp(sm, isa.OP_EXT, *a48(keys_addr))
        self.comp(sm, isa.OP_EXT, *a48(log_addr))
        self.comp(sm, isa.OP_EXT, *a48(stats_addr))
        self.comp(sm, isa.OP_EXT, n_stats & 0xFFFF, n_stats >> 16, 0)

    def moe_route(self, sm, *, logits: Src, route_addr: int, n_experts: int, top_k: int, release=None,
                  rank: int = 0, world: int = 1):
        """Softmax over n_experts fp32 router logits, top-k, renormalise: writes int32
        ids[16], fp32 weights[16], int32 local[16], int32 count[16] at route_addr (256 bytes).
        With world > 1 (expert parallelism, n_experts / world consecutive experts per rank)
        local / count describe this rank's share of the selection (see isa.h)."""
        assert n_experts <= 256 and top_k <= 16 and logits.nbytes == n_experts * 4
        assert 0 <= rank < max(world, 1) <= 255 and n_experts % max(world, 1) == 0
        self.load(sm, logits)
        self.raw_address(sm, route_addr, 25, release=release)
        self.comp(sm, isa.OP_MOE_ROUTE, n_experts, top_k, rank | (world << 8))

    def argmax_final(self, sm, *, records: Src, n: int, state_addr, log_addr, release=None, local_only=False,
                     peers: Optional[tuple] = None):
        """Reduces n candidate records {f32 value, i32 index, pad, pad}.  Normally
        the winner is logged as the next token and the state block advances;
        with local_only the winner is written to log_addr as one more record."""
        self.load(sm, records)
        self.raw_address(sm, state_addr, 25)
        self.raw_address(sm, log_addr, 26, release=release)
        if peers is not None:       # log_addr: byte offset of this rank's record inside an exchange block
            assert local_only
            self.comp(sm, isa.OP_ARGMAX_FINAL, n, 2)
            self._peer_words(sm, peers)
            return
        self.comp(sm, isa.OP_ARGMAX_FINAL, n, 1 if local_only else 0)

    # ------------------------------------------------------------------ output
    def finalize(self, check: bool = True):
        """Appends the terminators and returns (compute u8[S*N,8], memory
        u8[S*N,16], bars int32[MAX_BARS]) as numpy arrays.  With `check` the
        streams go through the library's own walk of the instruction words
        (runtime.validate_streams) first, so that a malformed program raises
        here, on the host, instead of ending a launch with a device-side status.
        (validate() adds the checks that need the whole program: barriers and sizes.)"""
        if not self._finalized:
            for sm in range(self.num_sms):
                self.mem(sm, isa.OP_TERMINATE)
                self.comp(sm, isa.OP_TERMINATEC)
            self._finalized = True
        n = self.insts_per_sm
        cm = np.zeros((self.num_sms, n), dtype=CINST)
        mm = np.zeros((self.num_sms, n), dtype=MINST)
        for sm in range(self.num_sms):
            if len(self.c[sm]) > n or len(self.m[sm]) > n:
                raise ValueError(f"SM {sm}: {len(self.c[sm])} compute / {len(self.m[sm])} memory instructions "
                                 f"exceed the ring of {n}")
            if self.c[sm]:
                cm[sm, :len(self.c[sm])] = np.array(self.c[sm], dtype=CINST)
            if self.m[sm]:
                mm[sm, :len(self.m[sm])] = np.array(self.m[sm], dtype=MINST)
        bars = np.zeros(isa.MAX_BARS, dtype=np.int32)
        for b, cnt in self.bar_counts.items():
            bars[b] = cnt
        c8, m8 = cm.view(np.uint8).reshape(self.num_sms * n, 8), mm.view(np.uint8).reshape(self.num_sms * n, 16)
        if check:
            from . import runtime
            runtime.validate_streams(self.num_sms, n, c8, m8)
        return c8, m8, bars

    def validate(self):
        """Static checks of the streams before they go to the device; raises ValueError.
        * every allocation fits the slot pool, every load size fits its slots;
        * every barrier some instruction waits for is counted down by somebody (a wait on a
          barrier nobody releases would only end at the device-side timeout), and nobody
          releases a barrier that was never declared."""
        waited, released = set(), set(b for b, n in self.bar_counts.items() if n > 0)
        op_id = isa.op_id
        loads = {op_id(isa.OP_ALLOC_TMA_LOAD_1D), op_id(isa.OP_ALLOC_TMA_LOAD_1D_STREAM)}
        for sm in range(self.num_sms):
            for i, (op, size, num_slots, arg, addr) in enumerate(self.m[sm]):
                oid = op_id(op)
                if oid == op_id(isa.OP_REPEAT) or oid == op_id(isa.OP_DYN_COUNT) or oid == op_id(isa.OP_STREAM_LIST):
                    continue
                nslot, bar = num_slots & 63, num_slots >> 6
                if op & isa.F_ALLOCATE and nslot < isa.NUM_SLOTS:
                    if nslot == 0:
                        raise ValueError(f"SM {sm} instruction {i}: allocation of zero slots")
                    if oid in loads and size > nslot * SLOT:
                        raise ValueError(f"SM {sm} instruction {i}: {size} bytes into {nslot} slots")
                if op & isa.F_ALLOCATE and nslot >= isa.NUM_SLOTS + isa.NUM_SPECIAL_SLOTS:
                    raise ValueError(f"SM {sm} instruction {i}: slot id {nslot} out of range")
                if op & isa.F_BARRIER:
                    if bar not in self.bar_counts:
                        raise ValueError(f"SM {sm} instruction {i}: barrier {bar} was never declared")
                    if not (op & isa.F_WRITEBACK):
                        waited.add(bar)
                if oid == op_id(isa.OP_ISSUE_BARRIER):
                    waited.add(bar)
        dead = sorted(waited - released)
        if dead:
            raise ValueError(f"barriers {dead} are waited for but never released")
        return True

    def stats(self):
        return {"max_minsts": max(len(x) for x in self.m), "max_cinsts": max(len(x) for x in self.c),
                "barriers": self._next_bar,
                "bytes_loaded_max": max(self.bytes_loaded), "bytes_loaded_min": min(self.bytes_loaded)}
