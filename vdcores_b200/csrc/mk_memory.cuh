// Memory virtual core of the megakernel: control warp, load ports, store warp.
#pragma once
#include "mk_common.cuh"

namespace vdc {

// ------------------------------------------------------------------------- //
// memory virtual core: control warp
// ------------------------------------------------------------------------- //
__device__ __forceinline__ VdcMInst load_minst(const VdcMInst* p) {
  uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  VdcMInst m;
  *reinterpret_cast<uint4*>(&m) = v;
  return m;
}

// Oldest ring entry that some consumer may still read: the CTA-wide head, or
// the next entry of the slowest warp while a per-warp phase is running.
__device__ __forceinline__ unsigned ring_head(const Shared* sh, int lane) {
  // cta_head is read first: it is only raised after every warp_next was set
  // (warp_phase_begin), so the minimum below never runs ahead of a consumer.
  const unsigned ch = sh->cta_head;
  __threadfence_block();
  unsigned v = lane < kCW ? sh->warp_next[lane] : 0xFFFFFFFFu;
  v = v < ch ? v : ch;
  return __reduce_min_sync(0xffffffffu, v);
}

__device__ void control_warp(const Ctx& c, const VdcMInst* __restrict__ insts, int n_insts, int lane) {
  Shared* sh = c.sh;
  uint32_t pc = 0, next_pc = 0;
  uint32_t shift = 0;
  uint64_t delta = 0, accum = 0;  // per-lane REPEAT registers
  int loop_counter = 0, loop_start = 0, jmp_cnt = 0;
  int dyn = 0;
  uint64_t ind_off = 0;
  bool ind_pending = false;
  unsigned tail = 0;        // ring entries published
  unsigned head_cache = 0;  // last known ring head
  bool running = true;
  unsigned demand = 0;      // bytes of the weight stream whose loads were issued
  long long t_fetch = 0, t_alloc = 0, t_pub = 0, n_inst = 0;

  // two-entry register cache of the instruction stream: the instruction being
  // executed (re-used by single-instruction REPEAT bodies) and its successor
  VdcMInst cur = load_minst(insts);
  uint32_t cur_pc = 0;
  VdcMInst nxt = load_minst(insts + (1 % n_insts));
  uint32_t nxt_pc = 1;

  while (running) {
    pc = next_pc;
    const long long tf0 = clock64();
    if (pc != cur_pc) {
      if (pc == nxt_pc) cur = nxt;
      else cur = load_minst(insts + (pc % (uint32_t)n_insts));
      cur_pc = pc;
    }
    if (nxt_pc != pc + 1) {
      nxt = load_minst(insts + ((pc + 1) % (uint32_t)n_insts));  // consumed on the next trip at the earliest
      nxt_pc = pc + 1;
    }
    VdcMInst inst = cur;
    next_pc = pc + 1;

    if (loop_counter > 0) inst.address += __shfl_sync(0xffffffffu, accum, (int)((pc - (uint32_t)loop_start) & 31u));
    if (inst.opcode & VDC_F_GROUP) inst.shifter += shift;
    const uint16_t opid = inst.opcode >> VDC_FLAG_BITS;
    t_fetch += clock64() - tf0;
    n_inst++;

    if (inst.opcode & VDC_F_ALLOCATE) {
      if (ind_pending) {
        inst.address += ind_off;
        ind_pending = false;
      }
      const int req = inst.num_slots & 63;
      int slot, word;
      const long long ta0 = clock64();
      if (req >= kSlots) {
        slot = req;  // special slot: nothing is allocated, the id itself is handed over
        word = req;
      } else {
        const uint32_t want = ((1u << req) - 1u) << lane;
        const bool lane_ok = req > 0 && lane + req <= kSlots;
        uint32_t it = 0;
        uint64_t t0 = 0;
        bool ok = true;
        while (true) {
          const uint32_t avail = *reinterpret_cast<volatile uint32_t*>(&sh->slot_avail);  // same word for all lanes
          const uint32_t cand = __ballot_sync(0xffffffffu, lane_ok && (avail & want) == want);
          if (cand) {
            slot = __ffs(cand) - 1;
            break;
          }
          __nanosleep(20);
          if ((++it & 63u) == 0) {
            int ab = 0;
            if (lane == 0) {
              ab = ld_relaxed_gpu(&c.status->abort);
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > 2 * c.timeout_ns) {
                raise_abort(c, VDC_ERR_TIMEOUT, 1, (int)pc, inst.opcode, -1, req);
                ab = 1;
              }
            }
            if (__shfl_sync(0xffffffffu, ab, 0)) {
              ok = false;
              break;
            }
          }
        }
        if (!ok) break;
        const uint32_t mask = ((1u << req) - 1u) << slot;
        if (lane == 0) atomicAnd(&sh->slot_avail, ~mask);
        word = (int)mask;
      }
      t_alloc += clock64() - ta0;

      const long long tp0 = clock64();
      // a ring entry is recycled only after every consumer moved past it
      if (tail - head_cache >= (unsigned)kQ) {
        uint32_t it = 0;
        uint64_t t0 = 0;
        bool ok = true;
        while (true) {
          head_cache = ring_head(sh, lane);
          if (tail - head_cache < (unsigned)kQ) break;
          if ((++it & 63u) == 0) {
            int ab = 0;
            if (lane == 0) {
              ab = ld_relaxed_gpu(&c.status->abort);
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > 2 * c.timeout_ns) {
                raise_abort(c, VDC_ERR_TIMEOUT, 1, (int)pc, inst.opcode, -1, -2);
                ab = 1;
              }
            }
            if (__shfl_sync(0xffffffffu, ab, 0)) {
              ok = false;
              break;
            }
          }
        }
        if (!ok) break;
      }
      if (lane == 0) {
        const unsigned e = tail % kQ;
        if ((inst.opcode & VDC_F_WRITEBACK) || req >= kSlots) sh->st_insts[slot] = inst;
        sh->ring[e] = inst;
        sh->ring_word[e] = word;
        __threadfence_block();
        sh->ring_tail = tail + 1;
        if (opid == 28) sh->demand_pos = demand + inst.size;
      }
      if (opid == 28) demand += inst.size;
      tail++;
      t_pub += clock64() - tp0;

      if ((inst.opcode & VDC_F_JUMP) && loop_counter > 0) {
        --loop_counter;
        if (loop_counter > 0) next_pc = (uint32_t)loop_start;
        accum += delta;
      }
    } else {
      switch (opid) {
        case 1: {  // TERMINATE: an end marker travels through the ring to both load ports
          running = false;
          bool ok = true;
          uint32_t it = 0;
          while (tail - head_cache >= (unsigned)kQ) {
            head_cache = ring_head(sh, lane);
            if ((++it & 1023u) == 0 && __shfl_sync(0xffffffffu, ld_relaxed_gpu(&c.status->abort), 0)) {
              ok = false;
              break;
            }
          }
          if (ok && lane == 0) {
            sh->ring[tail % kQ] = inst;
            __threadfence_block();
            sh->ring_tail = tail + 1;
          }
          break;
        }
        case 2: {  // REPEAT: per-lane address deltas for the following body
          int count = inst.size;
          if (count == 0xFFFF) count = dyn;
          const int reg_start = inst.num_slots & 0xFF, reg_end = inst.num_slots >> 8;
          if (lane >= reg_start && lane < reg_end) {
            delta = inst.address;
            accum = 0;
          }
          loop_counter = count;
          loop_start = (int)pc + 1;
          if (inst.size == 0xFFFF && count == 0) next_pc = pc + 1 + inst.arg;  // empty dynamic loop: skip body
          break;
        }
        case 3: {  // LOOP: jump back `size-1` times, shifting GROUP-flagged bar/TMA ids each time
          const int reg = inst.num_slots & 31;
          if (lane == reg) {
            if (++jmp_cnt < (int)inst.size) {
              next_pc = inst.coords[0];
              shift += (uint32_t)inst.coords[2] | ((uint32_t)inst.coords[3] << 16);
            } else {
              jmp_cnt = 0;
              shift = 0;
            }
          }
          next_pc = __shfl_sync(0xffffffffu, next_pc, reg);
          shift = __shfl_sync(0xffffffffu, shift, reg);
          break;
        }
        case 5: {  // ISSUE_BARRIER: stall the whole memory stream on a global barrier
          int ok = 1;
          if (lane == 0) ok = wait_global_barrier(c, inst.num_slots >> 6, 1, (int)pc, inst.opcode);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) running = false;
          break;
        }
        case 6:    // CC0: next allocating instruction's address += word << arg
        case 7: {  // CC0_ROW_BYTES:                        ... += word * size
          int word = 0;
          if (lane == 0) word = ld_relaxed_gpu(reinterpret_cast<const int*>(inst.address));
          word = __shfl_sync(0xffffffffu, word, 0);
          ind_off = (opid == 6) ? ((uint64_t)(uint32_t)word << inst.arg) : ((uint64_t)(uint32_t)word * inst.size);
          ind_pending = true;
          break;
        }
        case 25: {  // DYN_COUNT: dyn = clamp(word - base, 0, max)
          int word = 0;
          if (lane == 0) word = ld_relaxed_gpu(reinterpret_cast<const int*>(inst.address));
          word = __shfl_sync(0xffffffffu, word, 0);
          int v = word - (int)inst.num_slots;
          dyn = v < 0 ? 0 : (v > (int)inst.size ? (int)inst.size : v);
          break;
        }
        case 27: {  // STREAM_LIST: hand the weight-stream segment list to the streamer warp
          if (lane == 0) {
            sh->pf_list = inst.address;
            sh->pf_n = inst.size;
            sh->pf_window = (uint32_t)inst.num_slots << 10;  // KB
            __threadfence_block();
            sh->pf_go = 1;
          }
          break;
        }
        case 26: {  // PREFETCH_L2: pull [address, address + (arg << 16 | size)) into L2, no slot involved
          if (lane == 0) {
            const uint32_t bytes = ((uint32_t)inst.arg << 16) | inst.size;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(inst.address), "r"(bytes) : "memory");
          }
          break;
        }
        default:
          break;  // OP_SHIFT_RESOURCE and unknown control ids are no-ops, as in the reference
      }
    }
  }
  if (lane == 0) {
    sh->pf_exit = 1;
    uint64_t* pr = c.profile + c.sm * VDC_NUM_PROFILE_EVENTS;
    pr[3] = (uint64_t)t_fetch;
    pr[4] = (uint64_t)t_alloc;
    pr[5] = (uint64_t)t_pub;
    pr[6] = (uint64_t)n_inst;
  }
  // When the loop was left through an abort the load ports get no end marker:
  // their own waits observe the global abort flag and return.
}

// ------------------------------------------------------------------------- //
// memory virtual core: load port (single lane)
// ------------------------------------------------------------------------- //
__device__ __forceinline__ void tensor_load(int rank, void* dst, const CUtensorMap* desc, const uint16_t* cd,
                                            uint64_t* bar, bool fix0) {
  const uint32_t d = smem_u32(dst), b = smem_u32(bar);
  if (rank == 1) {
    asm volatile("cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2}], [%3];" ::
                     "r"(d), "l"(desc), "r"((int)(*reinterpret_cast<const uint32_t*>(cd))), "r"(b)
                 : "memory");
  } else if (rank == 2) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(d),
        "l"(desc), "r"((int)cd[0]), "r"((int)cd[1]), "r"(b)
        : "memory");
  } else if (rank == 3) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(d),
        "l"(desc), "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"(b)
        : "memory");
  } else if (rank == 4) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(d),
        "l"(desc), "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"((int)cd[3]), "r"(b)
        : "memory");
  } else if (fix0) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(d),
        "l"(desc), "r"(0), "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"((int)cd[3]), "r"(b)
        : "memory");
  }
}

__device__ void load_port(const Ctx& c, int port) {
  Shared* sh = c.sh;
  unsigned cursor = 0;  // next ring entry to look at (both ports walk every entry)
  int reg_file[4] = {0, 0, 0, 0};
  const int role = 3 + port;
  long long t_idle = 0, t_bar = 0, t_issue = 0;
  unsigned n_mine = 0;
  uint64_t* pr = c.profile + c.sm * VDC_NUM_PROFILE_EVENTS + 8 + port * 4;
  unsigned seen_tail = 0;
  while (true) {
    if (seen_tail == cursor) {
      const long long ti0 = clock64();
      if (!wait_until(c, [&] { return (seen_tail = sh->ring_tail) != cursor; }, role, (int)cursor, 0, -1, 0)) return;
      t_idle += clock64() - ti0;
      __threadfence_block();
    }
    const unsigned e = cursor % kQ;
    const VdcMInst inst = sh->ring[e];
    cursor++;
    const uint16_t opcode = inst.opcode;
    if ((opcode >> VDC_FLAG_BITS) == 1) {  // end marker
      pr[0] = (uint64_t)t_idle;
      pr[1] = (uint64_t)t_bar;
      pr[2] = (uint64_t)t_issue;
      pr[3] = n_mine;
      return;
    }
    if (((opcode & VDC_F_PORT) ? 1 : 0) != port) continue;
    n_mine++;
    const int word = sh->ring_word[e];
    const int req = inst.num_slots & 63;
    const int slot = req >= kSlots ? req : __ffs(word) - 1;
    uint64_t* bar = &sh->full[e];

    if ((opcode & VDC_F_BARRIER) && !(opcode & VDC_F_WRITEBACK)) {
      const long long tb0 = clock64();
      if (!wait_global_barrier(c, inst.num_slots >> 6, role, (int)cursor, opcode)) return;
      t_bar += clock64() - tb0;
    }
    const long long ts0 = clock64();
    void* dst = slot < kSlots ? slot_ptr(c, slot) : nullptr;
    switch (opcode >> VDC_FLAG_BITS) {
      case 28:  // 1-D bulk load of weight-stream bytes (counted by the L2 streamer)
      case 9:   // 1-D bulk load from a raw address
        mbar_arrive_expect_tx(bar, inst.size);
        bulk_load_1d(dst, reinterpret_cast<const void*>(inst.address), inst.size, bar);
        break;
      case 10:
        mbar_arrive_expect_tx(bar, inst.size);
        tensor_load(1, dst, c.tmas + inst.arg, inst.coords, bar, false);
        break;
      case 11:
        mbar_arrive_expect_tx(bar, inst.size);
        tensor_load(2, dst, c.tmas + inst.arg, inst.coords, bar, false);
        break;
      case 12:
        mbar_arrive_expect_tx(bar, inst.size);
        tensor_load(3, dst, c.tmas + inst.arg, inst.coords, bar, false);
        break;
      case 13:
        mbar_arrive_expect_tx(bar, inst.size);
        tensor_load(4, dst, c.tmas + inst.arg, inst.coords, bar, false);
        break;
      case 14:
        mbar_arrive_expect_tx(bar, inst.size);
        tensor_load(5, dst, c.tmas + inst.arg, inst.coords, bar, true);
        break;
      case 15:  // REG_STORE: remember the slot mask; the producer gets it with bit 31 set
        sh->ring_word[e] = word | (int)0x80000000;
        reg_file[inst.size & 3] = word;
        __threadfence_block();
        mbar_arrive(bar);
        break;
      case 8:  // REG_LOAD: hand the remembered mask to the consumer
        sh->ring_word[e] = reg_file[inst.size & 3];
        __threadfence_block();
        mbar_arrive(bar);
        break;
      default:  // write-back slots and raw addresses carry no load
        mbar_arrive(bar);
        break;
    }
    t_issue += clock64() - ts0;
  }
}

// ------------------------------------------------------------------------- //
// memory virtual core: store warp (single lane)
// ------------------------------------------------------------------------- //
__device__ __forceinline__ void tensor_store(int rank, const CUtensorMap* desc, const uint16_t* cd, const void* src,
                                             bool reduce, bool fix0) {
  const uint32_t s = smem_u32(src);
  if (!reduce) {
    if (rank == 2)
      asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(desc),
                   "r"((int)cd[0]), "r"((int)cd[1]), "r"(s)
                   : "memory");
    else if (rank == 3)
      asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(desc),
                   "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"(s)
                   : "memory");
    else if (rank == 4)
      asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(desc),
                   "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"((int)cd[3]), "r"(s)
                   : "memory");
    else if (rank == 5 && fix0)
      asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];" ::"l"(desc),
                   "r"(0), "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"((int)cd[3]), "r"(s)
                   : "memory");
  } else {
    if (rank == 2)
      asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%1, %2}], [%3];" ::"l"(desc),
                   "r"((int)cd[0]), "r"((int)cd[1]), "r"(s)
                   : "memory");
    else if (rank == 3)
      asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(desc),
                   "r"((int)cd[0]), "r"((int)cd[1]), "r"((int)cd[2]), "r"(s)
                   : "memory");
  }
}

__device__ void store_warp(const Ctx& c) {
  Shared* sh = c.sh;
  unsigned head = 0;
  while (true) {
    if (!wait_until(c, [&] { return sh->st_tail != head; }, 2, (int)head, 0, -1, 0)) break;
    __threadfence_block();
    const int mask = sh->st_q[head % kQ];
    head++;
    sh->st_head = head;
    if (mask == 0) break;
    const int slot = __ffs(mask) - 1;
    const VdcMInst inst = sh->st_insts[slot];
    const void* src = slot < kSlots ? slot_ptr(c, slot) : nullptr;
    bool copied = true;
    switch (inst.opcode >> VDC_FLAG_BITS) {
      case 16: bulk_store_1d(reinterpret_cast<void*>(inst.address), src, inst.size); break;
      case 17: tensor_store(2, c.tmas + inst.arg, inst.coords, src, false, false); break;
      case 18: tensor_store(3, c.tmas + inst.arg, inst.coords, src, false, false); break;
      case 19: tensor_store(4, c.tmas + inst.arg, inst.coords, src, false, false); break;
      case 20: tensor_store(5, c.tmas + inst.arg, inst.coords, src, false, true); break;
      case 21: tensor_store(2, c.tmas + inst.arg, inst.coords, src, true, false); break;
      case 22: tensor_store(3, c.tmas + inst.arg, inst.coords, src, true, false); break;
      case 24:
        if (inst.arg == 1) bulk_reduce_add_f32_1d(reinterpret_cast<void*>(inst.address), src, inst.size);
        else bulk_reduce_add_bf16_1d(reinterpret_cast<void*>(inst.address), src, inst.size);
        break;
      default: copied = false; break;  // raw-address hand-back: no copy, only the barrier below
    }
    if (copied) bulk_commit();
    if (inst.opcode & VDC_F_BARRIER) {
      bulk_wait_all();
      fence_proxy_async();
      __threadfence();
      red_release_gpu_add(c.bars + (inst.num_slots >> 6), -1);
    } else if (copied) {
      bulk_wait_read();
    }
    if (copied) atomicOr(&sh->slot_avail, (uint32_t)mask & kSlotMaskAll);
  }
  bulk_wait_all();
}


// ------------------------------------------------------------------------- //
// memory virtual core: HBM -> L2 streamer warp
// ------------------------------------------------------------------------- //
// Walks the SM's weight-stream segment list and issues L2 prefetches (one 128-byte
// line per lane, 4 KB per step), staying at most pf_window bytes ahead of the
// bytes the control warp has issued loads for.  While the compute core waits on
// a cross-SM dependency the loads stall but the frontier still moves, so HBM
// keeps streaming into L2 and the stalled stage later reads from L2.
__device__ void streamer_warp(const Ctx& c, int lane) {
  Shared* sh = c.sh;
  // wait for the list (or for the end of the program)
  while (true) {
    int go = sh->pf_go, ex = sh->pf_exit;
    if (__shfl_sync(0xffffffffu, go, 0)) break;
    if (__shfl_sync(0xffffffffu, ex, 0)) return;
    __nanosleep(200);
  }
  __threadfence_block();
  const uint4* list = reinterpret_cast<const uint4*>((unsigned long long)sh->pf_list);
  const unsigned n = sh->pf_n, window = sh->pf_window;
  unsigned pos = 0;  // stream position of the next piece
  for (unsigned s = 0; s < n; ++s) {
    const uint4 seg = __ldg(list + s);
    const unsigned long long base = (unsigned long long)seg.x | ((unsigned long long)seg.y << 32);
    const unsigned bytes = seg.z;
    for (unsigned off = 0; off < bytes; off += 4096) {
      const unsigned piece = bytes - off < 4096u ? bytes - off : 4096u;
      const unsigned end = pos + piece;
      bool skip = false;
      unsigned it = 0;
      while (true) {
        unsigned d = sh->demand_pos;
        int ex = sh->pf_exit;
        d = __shfl_sync(0xffffffffu, d, 0);
        if (__shfl_sync(0xffffffffu, ex, 0)) return;
        if (end <= d) {  // the loads already went past this piece
          skip = true;
          break;
        }
        if (end - d <= window) break;
        __nanosleep(100);
        if ((++it & 255u) == 0 && __shfl_sync(0xffffffffu, ld_relaxed_gpu(&c.status->abort), 0)) return;
      }
      const unsigned o = off + lane * 128;
      if (!skip && o < bytes) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + o));
      pos = end;
    }
  }
}

}  // namespace vdc
