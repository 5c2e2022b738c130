// Memory virtual core of the megakernel: control warp, load ports, store warp.
#pragma once
#include "mk_common.cuh"

namespace vdc {

// ------------------------------------------------------------------------- //
// memory virtual core: control warp
// ------------------------------------------------------------------------- //
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

#ifndef VDC_CTRL_FASTPATH
#define VDC_CTRL_FASTPATH 0
#endif
#ifndef VDC_CTRL_PAGELOOP
#define VDC_CTRL_PAGELOOP 1   // lane-0 fast path for the attention page loop
#endif
#ifndef VDC_ALLOC_SLEEP
#define VDC_ALLOC_SLEEP 20   // ns between two looks at the slot mask while no slot is free
#endif
#ifndef VDC_FAST_SLEEP
#define VDC_FAST_SLEEP 20
#endif
#ifndef VDC_FAST_FIRSTFIT
#define VDC_FAST_FIRSTFIT 0
#endif
// The control warp keeps instructions as four 32-bit words in registers:
//   w.x = opcode | size << 16,  w.y = num_slots | arg << 16 (the "shifter"),
//   w.z / w.w = low / high half of the address (or the four 16-bit coordinates).
// The instruction stream lives in global memory; the control warp keeps a
// 64-instruction window of it in shared memory (filled 32 lanes at a time), so
// that loop bodies are re-read from shared memory, never from L2.
__device__ __forceinline__ void icache_fill(Shared* sh, const VdcMInst* insts, uint32_t base, int n_insts, int lane) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(insts + ((base + lane) % (uint32_t)n_insts)));
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(insts + ((base + 32 + lane) % (uint32_t)n_insts)));
  __syncwarp();
  *reinterpret_cast<uint4*>(&sh->icache[lane]) = a;
  *reinterpret_cast<uint4*>(&sh->icache[32 + lane]) = b;
  __syncwarp();
}

// Bounded warp-wide back-off used by the control warp's two resource waits.
// Returns non-zero when the wait must be given up.
__device__ __forceinline__ int control_backoff(const Ctx& c, int lane, uint32_t& it, uint64_t& t0, uint32_t pc,
                                               uint32_t opcode, int aux) {
  if ((++it & 63u) != 0) return 0;
  int ab = 0;
  if (lane == 0) {
    ab = ld_relaxed_gpu(&c.status->abort);
    const uint64_t now = globaltimer_ns();
    if (t0 == 0) t0 = now;
    else if (now - t0 > 2 * c.timeout_ns) {
      raise_abort(c, VDC_ERR_TIMEOUT, 1, (int)pc, (int)opcode, -1, aux);
      ab = 1;
    }
  }
  return __shfl_sync(0xffffffffu, ab, 0);
}

__device__ void control_warp(const Ctx& c, const VdcMInst* __restrict__ insts, int n_insts, int lane) {
  Shared* sh = c.sh;
  uint32_t pc = 0, next_pc = 0;
  uint32_t shift = 0;
  uint64_t delta = 0, accum = 0;  // per-lane REPEAT registers
  int loop_counter = 0, loop_start = 0, jmp_cnt = 0;
  int dyn = 0;
  int loop_iter = 0;     // trips of the current REPEAT completed so far
  uint32_t tbl = 0;      // per-lane word of the table PT_LOAD32 fetched
  uint64_t ind_off = 0;
  bool ind_pending = false;
  unsigned tail = 0;        // ring entries published
  unsigned head_cache = 0;  // last known ring head
  unsigned demand = 0;      // bytes of the weight stream whose loads were issued
  unsigned n_inst = 0, n_alloc_retry = 0, n_ring_wait = 0;
  const long long t_begin = clock64();
  bool running = true;

  uint32_t ic_base = 0;  // first instruction index held in the shared-memory window
  icache_fill(sh, insts, 0, n_insts, lane);

#ifdef VDC_CTRL_PROFILE
  long long tp_fetch = 0, tp_alloc = 0, tp_pub = 0, tp_ctl = 0, tp_mark = clock64();
#define CTP(var) { const long long _n = clock64(); var += _n - tp_mark; tp_mark = _n; }
#else
#define CTP(var)
#endif
  while (running) {
    pc = next_pc;
    if (pc - ic_base >= 64u) {
      ic_base = pc & ~31u;
      icache_fill(sh, insts, ic_base, n_insts, lane);
    }
    uint4 w = *reinterpret_cast<const uint4*>(&sh->icache[pc - ic_base]);
    next_pc = pc + 1;
    n_inst++;

    if (loop_counter > 0) {
      const uint64_t a = __shfl_sync(0xffffffffu, accum, (int)((pc - (uint32_t)loop_start) & 31u));
      const uint64_t addr = (((uint64_t)w.w << 32) | w.z) + a;
      w.z = (uint32_t)addr;
      w.w = (uint32_t)(addr >> 32);
    }
    const uint32_t opcode = w.x & 0xFFFFu;
    if (opcode & VDC_F_GROUP) w.y += shift;
    const uint32_t opid = opcode >> VDC_FLAG_BITS;
    const uint32_t size = w.x >> 16;
    const uint32_t num_slots = w.y & 0xFFFFu;

    CTP(tp_fetch);
    if (opcode & VDC_F_ALLOCATE) {
      if (ind_pending) {
        const uint64_t addr = (((uint64_t)w.w << 32) | w.z) + ind_off;
        w.z = (uint32_t)addr;
        w.w = (uint32_t)(addr >> 32);
        // one shot, except for a loop body that is about to jump back: every trip of a
        // weight-stream loop behind an indirection (an expert's rows) needs the offset
        if (!((opcode & VDC_F_JUMP) && loop_counter > 1)) ind_pending = false;
      }
      const int req = (int)(num_slots & 63u);
      int slot, word;
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
            // activation vectors live for a whole task: they go to the top of the pool, so that the
            // weight chunks below them keep whole groups of slots
            slot = opid == 32 ? 31 - __clz(cand) : __ffs(cand) - 1;
            break;
          }
          n_alloc_retry++;
          if (VDC_ALLOC_SLEEP) __nanosleep(VDC_ALLOC_SLEEP);
          if (control_backoff(c, lane, it, t0, pc, opcode, req)) {
            ok = false;
            break;
          }
        }
        if (!ok) break;
        const uint32_t mask = ((1u << req) - 1u) << slot;
        if (lane == 0) atomicAnd(&sh->slot_avail, ~mask);
        word = (int)mask;
      }

      CTP(tp_alloc);
      // a ring entry is recycled only after every consumer moved past it
      if (tail - head_cache >= (unsigned)kQ) {
        uint32_t it = 0;
        uint64_t t0 = 0;
        bool ok = true;
        while (true) {
          head_cache = ring_head(sh, lane);
          if (tail - head_cache < (unsigned)kQ) break;
          n_ring_wait++;
          if (control_backoff(c, lane, it, t0, pc, opcode, -2)) {
            ok = false;
            break;
          }
        }
        if (!ok) break;
      }
      if (lane == 0) {
        const unsigned e = tail % kQ;
        if ((opcode & VDC_F_WRITEBACK) || req >= kSlots) *reinterpret_cast<uint4*>(&sh->st_insts[slot]) = w;
        *reinterpret_cast<uint4*>(&sh->ring[e]) = w;
        sh->ring_word[e] = word;
        __threadfence_block();
        sh->ring_tail = tail + 1;
        if (opid == 28) sh->demand_pos = demand + size;
        CHUNK_STAMP(c, tail, 0);
      }
      if (opid == 28) demand += size;
      tail++;

      if ((opcode & VDC_F_JUMP) && loop_counter > 0) {
        --loop_counter;
        ++loop_iter;
        if (loop_counter > 0) next_pc = (uint32_t)loop_start;
        accum += delta;
      }
      CTP(tp_pub);
    } else {
      const uint64_t address = ((uint64_t)w.w << 32) | w.z;
      const uint32_t arg = w.y >> 16;
      switch (opid) {
        case 1: {  // TERMINATE: an end marker travels through the ring to both load ports
          running = false;
          bool ok = true;
          uint32_t it = 0;
          uint64_t t0 = 0;
          while (tail - head_cache >= (unsigned)kQ) {
            head_cache = ring_head(sh, lane);
            if (control_backoff(c, lane, it, t0, pc, opcode, -3)) {
              ok = false;
              break;
            }
          }
          if (ok && lane == 0) {
            *reinterpret_cast<uint4*>(&sh->ring[tail % kQ]) = w;
            __threadfence_block();
            sh->ring_tail = tail + 1;
          }
          break;
        }
        case 2: {  // REPEAT: per-lane address deltas for the following body
          int count = (int)size;
          if (count == 0xFFFF) count = dyn;
          const int reg_start = (int)(num_slots & 0xFF), reg_end = (int)(num_slots >> 8);
          if (lane >= reg_start && lane < reg_end) {
            delta = address;
            accum = 0;
          }
          loop_counter = count;
          loop_iter = 0;
          loop_start = (int)pc + 1;
          if (size == 0xFFFF && count == 0) {
            ind_pending = false;     // an indirection meant for the skipped body must not reach a later load
            next_pc = pc + 1 + arg;  // empty dynamic loop: skip body
            break;
          }
          // Fast path for the dominant case, a body of one plain 1-D load (a weight
          // stream): lane 0 runs the whole loop alone, without warp-wide votes.
          // (Measured on B200: issuing the chunk loads this fast makes them arrive in
          // bursts, the warps then compute and free in lock-step, and a GEMV stage
          // streams ~7 % slower than with the paced general path; off by default.)
          // Page loop of the decode attention: a body of {PT_APPLY, page load, PT_APPLY, page load}.
          // Lane 0 runs all its trips alone from the table words PT_LOAD32 fetched: per page copy
          // one look at the slot mask, one ring entry, no warp-wide votes and no instruction fetch.
          if (VDC_CTRL_PAGELOOP && count > 0 && pc + 4 - ic_base < 64u && !ind_pending) {
            const uint4 a0 = *reinterpret_cast<const uint4*>(&sh->icache[pc + 1 - ic_base]);
            const uint4 l0 = *reinterpret_cast<const uint4*>(&sh->icache[pc + 2 - ic_base]);
            const uint4 a1 = *reinterpret_cast<const uint4*>(&sh->icache[pc + 3 - ic_base]);
            const uint4 l1 = *reinterpret_cast<const uint4*>(&sh->icache[pc + 4 - ic_base]);
            auto is_apply = [](const uint4& v) { return ((v.x & 0xFFFFu) >> VDC_FLAG_BITS) == 31u; };
            auto is_load = [](const uint4& v, bool jump) {
              const uint32_t op = v.x & 0xFFFFu;
              const int rq = (int)(v.y & 63u);
              return (op >> VDC_FLAG_BITS) == 9u && (op & VDC_F_ALLOCATE) && !(op & (VDC_F_GROUP | VDC_F_BARRIER)) &&
                     ((op & VDC_F_JUMP) != 0) == jump && rq > 0 && rq < kSlots;
            };
            if (is_apply(a0) && is_load(l0, false) && is_apply(a1) && is_load(l1, true) && count <= 32 &&
                reg_start == 0 && reg_end == 4 && address == 0) {
              sh->pt_words[lane] = tbl;
              __syncwarp();
              int ok = 1;
              if (lane == 0) {
                const uint32_t sh0 = a0.y >> 16, sh1 = a1.y >> 16;
                int pos = 0;
                for (int k = 0; k < 2 * count && ok; ++k) {
                  const uint4& b = (k & 1) ? l1 : l0;
                  const int breq = (int)(b.y & 63u);
                  const uint32_t unit = (1u << breq) - 1u;
                  const uint64_t addr = (((uint64_t)b.w << 32) | b.z) + ((uint64_t)sh->pt_words[k >> 1] << ((k & 1) ? sh1 : sh0));
                  uint32_t it = 0, mask;
                  uint64_t t0 = 0;
                  while (true) {
                    const uint32_t avail = *reinterpret_cast<volatile uint32_t*>(&sh->slot_avail);
                    if (pos + breq > kSlots) pos = 0;
                    mask = unit << pos;
                    if ((avail & mask) == mask) break;
                    bool found = false;
                    for (int p2 = 0; p2 + breq <= kSlots; ++p2) {
                      mask = unit << p2;
                      if ((avail & mask) == mask) {
                        pos = p2;
                        found = true;
                        break;
                      }
                    }
                    if (found) break;
                    n_alloc_retry++;
                    __nanosleep(20);
                    if ((++it & 63u) == 0) {
                      const uint64_t now = globaltimer_ns();
                      if (t0 == 0) t0 = now;
                      if (ld_relaxed_gpu(&c.status->abort) != 0) ok = 0;
                      else if (now - t0 > 2 * c.timeout_ns) {
                        raise_abort(c, VDC_ERR_TIMEOUT, 1, (int)pc + 2, (int)(b.x & 0xFFFFu), -1, breq);
                        ok = 0;
                      }
                      if (!ok) break;
                    }
                  }
                  if (!ok) break;
                  atomicAnd(&sh->slot_avail, ~mask);
                  pos += breq;
                  while (tail - head_cache >= (unsigned)kQ) {  // ring full: recompute the head alone
                    unsigned h = sh->cta_head;
                    __threadfence_block();
                    for (int wv = 0; wv < kCW; ++wv) {
                      const unsigned v = sh->warp_next[wv];
                      h = v < h ? v : h;
                    }
                    head_cache = h;
                    if ((++it & 1023u) == 0 && ld_relaxed_gpu(&c.status->abort) != 0) {
                      ok = 0;
                      break;
                    }
                  }
                  if (!ok) break;
                  const unsigned e = tail % kQ;
                  *reinterpret_cast<uint4*>(&sh->ring[e]) = make_uint4(b.x, b.y, (uint32_t)addr, (uint32_t)(addr >> 32));
                  sh->ring_word[e] = (int)mask;
                  __threadfence_block();
                  CHUNK_STAMP(c, tail, 0);
                  sh->ring_tail = ++tail;
                }
              }
              ok = __shfl_sync(0xffffffffu, ok, 0);
              tail = __shfl_sync(0xffffffffu, tail, 0);
              head_cache = __shfl_sync(0xffffffffu, head_cache, 0);
              n_inst += 4u * (unsigned)count;
              loop_counter = 0;
              next_pc = pc + 5;
              if (!ok) running = false;
              break;
            }
          }
          if (VDC_CTRL_FASTPATH && count > 0 && pc + 1 - ic_base < 64u && !ind_pending) {
            const uint4 b = *reinterpret_cast<const uint4*>(&sh->icache[pc + 1 - ic_base]);
            const uint32_t bop = b.x & 0xFFFFu, bid = bop >> VDC_FLAG_BITS;
            const int breq = (int)(b.y & 63u);
            if ((bid == 9 || bid == 28) && (bop & VDC_F_JUMP) && !(bop & (VDC_F_GROUP | VDC_F_BARRIER)) && breq > 0 &&
                breq < kSlots && reg_start == 0 && reg_end >= 1) {
              int ok = 1;
              if (lane == 0) {
                uint64_t addr = ((uint64_t)b.w << 32) | b.z;
                const uint32_t bsize = b.x >> 16;
                const uint32_t unit = (1u << breq) - 1u;
                int pos = 0;  // where the previous allocation ended: frees come back in the same order
                for (int k = 0; k < count && ok; ++k) {
                  uint32_t it = 0;
                  uint64_t t0 = 0;
                  uint32_t mask;
                  while (true) {
                    const uint32_t avail = *reinterpret_cast<volatile uint32_t*>(&sh->slot_avail);
                    if (VDC_FAST_FIRSTFIT || pos + breq > kSlots) pos = 0;
                    mask = unit << pos;
                    if ((avail & mask) == mask) break;
                    bool found = false;
                    for (int p2 = 0; p2 + breq <= kSlots; ++p2) {
                      mask = unit << p2;
                      if ((avail & mask) == mask) {
                        pos = p2;
                        found = true;
                        break;
                      }
                    }
                    if (found) break;
                    n_alloc_retry++;
                    __nanosleep(VDC_FAST_SLEEP);
                    if ((++it & 63u) == 0) {
                      const uint64_t now = globaltimer_ns();
                      if (t0 == 0) t0 = now;
                      if (ld_relaxed_gpu(&c.status->abort) != 0) ok = 0;
                      else if (now - t0 > 2 * c.timeout_ns) {
                        raise_abort(c, VDC_ERR_TIMEOUT, 1, (int)pc + 1, (int)bop, -1, breq);
                        ok = 0;
                      }
                      if (!ok) break;
                    }
                  }
                  if (!ok) break;
                  atomicAnd(&sh->slot_avail, ~mask);
                  pos += breq;
                  while (tail - head_cache >= (unsigned)kQ) {  // ring full: recompute the head alone
                    unsigned h = sh->cta_head;
                    __threadfence_block();
                    for (int wv = 0; wv < kCW; ++wv) {
                      const unsigned v = sh->warp_next[wv];
                      h = v < h ? v : h;
                    }
                    head_cache = h;
                    if ((++it & 1023u) == 0 && ld_relaxed_gpu(&c.status->abort) != 0) {
                      ok = 0;
                      break;
                    }
                  }
                  if (!ok) break;
                  const unsigned e = tail % kQ;
                  *reinterpret_cast<uint4*>(&sh->ring[e]) = make_uint4(b.x, b.y, (uint32_t)addr, (uint32_t)(addr >> 32));
                  sh->ring_word[e] = (int)mask;
                  __threadfence_block();
                  sh->ring_tail = ++tail;
                  if (bid == 28) {
                    demand += bsize;
                    sh->demand_pos = demand;
                  }
                  addr += address;  // the REPEAT delta
                }
              }
              ok = __shfl_sync(0xffffffffu, ok, 0);
              tail = __shfl_sync(0xffffffffu, tail, 0);
              head_cache = __shfl_sync(0xffffffffu, head_cache, 0);
              demand = __shfl_sync(0xffffffffu, demand, 0);
              n_inst += (unsigned)count;
              loop_counter = 0;
              next_pc = pc + 2;
              if (!ok) running = false;
            }
          }
          break;
        }
        case 3: {  // LOOP: jump back `size-1` times, shifting GROUP-flagged bar/TMA ids each time
          const int reg = (int)(num_slots & 31u);
          if (lane == reg) {
            if (++jmp_cnt < (int)size) {
              next_pc = w.z & 0xFFFFu;  // coords[0]
              shift += w.w;            // coords[2] | coords[3] << 16
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
          if (lane == 0) ok = wait_global_barrier(c, (int)(num_slots >> 6), 1, (int)pc, (int)opcode);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) running = false;
          break;
        }
        case 29:   // CC0_STRIDE32:                         ... += word * (size | arg << 16)
        case 6:    // CC0: next allocating instruction's address += word << arg
        case 7: {  // CC0_ROW_BYTES:                        ... += word * size
          int word = 0;
          if (lane == 0) word = ld_relaxed_gpu(reinterpret_cast<const int*>(address));
          word = __shfl_sync(0xffffffffu, word, 0);
          ind_off = (opid == 6) ? ((uint64_t)(uint32_t)word << arg)
                                : (opid == 7 ? (uint64_t)(uint32_t)word * size
                                             : (uint64_t)(uint32_t)word * (uint64_t)(size | (arg << 16)));
          ind_pending = true;
          break;
        }
        case 33: {  // DYN_CHUNKS: stream the template load for chunk indices drawn from a shared counter
          const int total = (int)(size | (arg << 16));
          int* counter = c.bars + (num_slots >> 6);
          if (pc + 1 - ic_base >= 64u) {
            ic_base = (pc + 1) & ~31u;
            icache_fill(sh, insts, ic_base, n_insts, lane);
          }
          const uint4 t = *reinterpret_cast<const uint4*>(&sh->icache[pc + 1 - ic_base]);
          const uint32_t t_op = t.x & 0xFFFFu, t_bytes = t.x >> 16;
          const int req = (int)(t.y & 63u);
          const uint64_t t_addr = ((uint64_t)t.w << 32) | t.z;
          const uint32_t want = ((1u << req) - 1u) << lane;
          const bool lane_ok = req > 0 && req < kSlots && lane + req <= kSlots;
          // the address field limits how many ring entries may be unconsumed when a chunk is drawn (0: no
          // limit): near the end of a stage an SM must not sit on chunks that an idle SM could take
          const unsigned depth = (uint32_t)address != 0u ? (uint32_t)address : 0x7FFFFFFFu;
          int idx = 0, taken = 0;
          bool ok = true;
          {
            uint32_t it = 0;
            uint64_t t0 = 0;
            while (tail - (head_cache = ring_head(sh, lane)) > depth)
              if (control_backoff(c, lane, it, t0, pc, opcode, -5)) {
                ok = false;
                break;
              }
          }
          if (ok && lane == 0) idx = atomicAdd(counter, 1);
          idx = ok ? __shfl_sync(0xffffffffu, idx, 0) : total;
          while (ok && idx < total) {
            int nxt = 0;
            {
              uint32_t it = 0;
              uint64_t t0 = 0;
              while (tail + 1u - (head_cache = ring_head(sh, lane)) > depth)
                if (control_backoff(c, lane, it, t0, pc, opcode, -5)) {
                  ok = false;
                  break;
                }
              if (!ok) break;
            }
            if (lane == 0) nxt = atomicAdd(counter, 1);  // the next draw travels while this chunk is placed
            int slot = 0;
            uint32_t it = 0;
            uint64_t t0 = 0;
            while (true) {
              const uint32_t avail = *reinterpret_cast<volatile uint32_t*>(&sh->slot_avail);
              const uint32_t cand = __ballot_sync(0xffffffffu, lane_ok && (avail & want) == want);
              if (cand) {
                slot = __ffs(cand) - 1;
                break;
              }
              n_alloc_retry++;
              if (VDC_ALLOC_SLEEP) __nanosleep(VDC_ALLOC_SLEEP);
              if (control_backoff(c, lane, it, t0, pc + 1, t_op, req)) {
                ok = false;
                break;
              }
            }
            if (!ok) break;
            const uint32_t mask = ((1u << req) - 1u) << slot;
            if (lane == 0) atomicAnd(&sh->slot_avail, ~mask);
            while (tail - head_cache >= (unsigned)kQ) {
              head_cache = ring_head(sh, lane);
              if (tail - head_cache < (unsigned)kQ) break;
              n_ring_wait++;
              if (control_backoff(c, lane, it, t0, pc + 1, t_op, -2)) {
                ok = false;
                break;
              }
            }
            if (!ok) break;
            if (lane == 0) {
              const unsigned e = tail % kQ;
              const uint64_t a = t_addr + (uint64_t)(uint32_t)idx * t_bytes;
              *reinterpret_cast<uint4*>(&sh->ring[e]) = make_uint4(t.x, t.y, (uint32_t)a, (uint32_t)(a >> 32));
              sh->ring_word[e] = (int)mask;
              __threadfence_block();
              sh->ring_tail = tail + 1;
              CHUNK_STAMP(c, tail, 0);
            }
            tail++;
            taken++;
            n_inst++;
            idx = __shfl_sync(0xffffffffu, nxt, 0);
          }
          for (int k = 0; ok && k < 4; ++k) {  // end markers, one per consuming warp pair
            uint32_t it = 0;
            uint64_t t0 = 0;
            while (tail - head_cache >= (unsigned)kQ) {
              head_cache = ring_head(sh, lane);
              if (tail - head_cache < (unsigned)kQ) break;
              if (control_backoff(c, lane, it, t0, pc, opcode, -4)) {
                ok = false;
                break;
              }
            }
            if (!ok) break;
            if (lane == 0) {
              const unsigned e = tail % kQ;
              *reinterpret_cast<uint4*>(&sh->ring[e]) = make_uint4(33u << VDC_FLAG_BITS, 0u, (uint32_t)taken, (uint32_t)k);
              sh->ring_word[e] = VDC_STREAM_END;
              __threadfence_block();
              sh->ring_tail = tail + 1;
            }
            tail++;
          }
          if (!ok) running = false;
          next_pc = pc + 2;
          break;
        }
        case 30: {  // PT_LOAD32: lane i keeps 32-bit word i of the table at `address` (size words, at most 32)
          tbl = lane < (int)size ? (uint32_t)ld_relaxed_gpu(reinterpret_cast<const int*>(address) + lane) : 0u;
          break;
        }
        case 31: {  // PT_APPLY: next allocating instruction's address += table word of this loop trip << arg
          const uint32_t word = __shfl_sync(0xffffffffu, tbl, loop_iter & 31);
          ind_off = (uint64_t)word << arg;
          ind_pending = true;
          break;
        }
        case 25: {  // DYN_COUNT: dyn = clamp(word - base, 0, max)
          int word = 0;
          if (lane == 0) word = ld_relaxed_gpu(reinterpret_cast<const int*>(address));
          word = __shfl_sync(0xffffffffu, word, 0);
          const int v = word - (int)num_slots;
          dyn = v < 0 ? 0 : (v > (int)size ? (int)size : v);
          break;
        }
        case 27: {  // STREAM_LIST: hand the weight-stream segment list to the streamer warp
          if (lane == 0) {
            sh->pf_list = address;
            sh->pf_n = size;
            sh->pf_window = num_slots << 10;  // KB
            __threadfence_block();
            sh->pf_go = 1;
          }
          break;
        }
        case 26: {  // PREFETCH_L2: pull [address, address + (arg << 16 | size)) into L2, no slot involved
          if (lane == 0) {
            const uint32_t bytes = (arg << 16) | size;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(address), "r"(bytes) : "memory");
          }
          break;
        }
        default:
          break;  // OP_SHIFT_RESOURCE and unknown control ids are no-ops, as in the reference
      }
      CTP(tp_ctl);
    }
  }
#ifdef VDC_CTRL_PROFILE
  if (lane == 0) {
    uint64_t* pr = c.profile + c.sm * VDC_NUM_PROFILE_EVENTS;
    pr[120] = tp_fetch; pr[121] = tp_alloc; pr[122] = tp_pub; pr[123] = tp_ctl;
  }
#endif
  if (lane == 0) {
    sh->pf_exit = 1;
    c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 6] = n_inst;
    c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 3] = (uint64_t)(clock64() - t_begin);
    c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 4] = n_alloc_retry;
    c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 5] = n_ring_wait;
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
  unsigned seen_tail = 0;
  while (true) {
    if (seen_tail == cursor) {
      if (!wait_until(c, [&] { return (seen_tail = sh->ring_tail) != cursor; }, role, (int)cursor, 0, -1, 0)) return;
      __threadfence_block();
    }
    const unsigned e = cursor % kQ;
    const VdcMInst inst = sh->ring[e];
    cursor++;
    const uint16_t opcode = inst.opcode;
    if ((opcode >> VDC_FLAG_BITS) == 1) return;  // end marker
    if (((opcode & VDC_F_PORT) ? 1 : 0) != port) continue;
    const int word = sh->ring_word[e];
    const int req = inst.num_slots & 63;
    const int slot = req >= kSlots ? req : __ffs(word) - 1;
    uint64_t* bar = &sh->full[e];

    // (an XVEC hand-over carries its barrier to the compute task, which waits for it itself)
    if ((opcode & VDC_F_BARRIER) && !(opcode & VDC_F_WRITEBACK) && (opcode >> VDC_FLAG_BITS) != 32) {
      if (!wait_global_barrier(c, inst.num_slots >> 6, role, (int)cursor, opcode)) return;
    }
    void* dst = slot < kSlots ? slot_ptr(c, slot) : nullptr;
    switch (opcode >> VDC_FLAG_BITS) {
      case 28:  // 1-D bulk load of weight-stream bytes (counted by the L2 streamer)
      case 9:   // 1-D bulk load from a raw address
        mbar_arrive_expect_tx(bar, inst.size);
        bulk_load_1d(dst, reinterpret_cast<const void*>(inst.address), inst.size, bar);
        CHUNK_STAMP(c, cursor - 1, 1);
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
