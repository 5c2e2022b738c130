// Persistent decode megakernel for sm_100a.
//
// One CTA per SM.  Each CTA runs two instruction streams:
//   * the memory virtual core  (control warp + two load ports + store warp)
//     fetches 16-byte memory instructions, allocates 8 KB shared-memory slots,
//     issues TMA bulk / tensor copies whose completion is signalled on
//     mbarriers, waits on / releases global countdown barriers, and writes
//     results back with bulk stores or bulk reduce-adds;
//   * the compute virtual core (8 warps) executes 8-byte compute instructions;
//     each task pops the slots the memory core filled for it, does its math on
//     CUDA cores, and either frees the slots or hands them to the store warp.
//
// It plays the role of the reference's dae2 kernel and pipeline warps
// (include/dae/dae2.cuh:28-177, include/dae/pipeline/{allocwarp,ldwarp,stwarp}.cuh)
// and honours the same instruction encodings, but queues, allocator, waits and
// all compute tasks are written for B200: every wait is bounded and reports
// through a status block instead of spinning forever, compute tasks are
// bandwidth-oriented CUDA-core kernels (128-bit shared loads, warp-shuffle
// reductions, fp32 accumulation) rather than WGMMA tiles.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "isa.h"

namespace vdc {

constexpr int kSlots = VDC_NUM_SLOTS;
constexpr int kQ = VDC_QUEUE_LEN;
constexpr int kCT = VDC_COMPUTE_THREADS;
constexpr int kCW = VDC_COMPUTE_WARPS;
constexpr uint32_t kSlotEnd = 0xFFu;
constexpr int kPopAbort = 0x40000000;
constexpr uint32_t kSlotMaskAll = (1u << kSlots) - 1;

// ------------------------------------------------------------------------- //
// PTX helpers
// ------------------------------------------------------------------------- //
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_load_1d(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_bf16_1d(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_f32_1d(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory"); }

__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------- //
// shared state of one CTA
// ------------------------------------------------------------------------- //
struct __align__(16) Shared {
  VdcMInst st_insts[kSlots + VDC_NUM_SPECIAL_SLOTS];  // instruction that owns each slot
  uint64_t full[kQ];                                   // m2c: completion barrier per queue entry
  int m2c_data[kQ];                                    // m2c: slot mask (or special slot id) per entry
  VdcMInst ent_insts[kQ];                              // m2c: the instruction behind each entry
  int ld_q[2][kQ];                                     // control warp -> load port commands
  int st_q[kQ];                                        // compute -> store warp slot masks
  volatile unsigned m2c_head;                          // entries consumed by the compute core
  volatile unsigned ld_head[2], ld_tail[2];
  volatile unsigned st_head, st_tail;
  unsigned slot_avail;                                 // bit i set = slot i free
  volatile int pop_val[2];
  volatile uint32_t pop_meta[2];
  volatile uint64_t pop_addr[2];
  float red[4096 + 64];                                // task scratch (reductions)
  float scores[VDC_KV_PAGE * 8];
  float probs[VDC_KV_PAGE * 8];
  float wmax[kCW * 8];
  float qrot[8 * VDC_HEAD_DIM];
  float misc[64];
};

struct Ctx {
  Shared* sh;
  uint8_t* slots;  // 1 KB aligned base of the slot area
  const CUtensorMap* tmas;
  int* bars;
  vdc_status* status;
  uint64_t* profile;
  uint64_t timeout_ns;
  int sm;
};

__device__ __forceinline__ void* slot_ptr(const Ctx& c, int slot) { return c.slots + (size_t)slot * VDC_SLOT_BYTES; }

__device__ __noinline__ void raise_abort(const Ctx& c, int code, int role, int pc, int opcode, int bar, int aux) {
  if (atomicCAS(&c.status->abort, 0, 1) == 0) {
    c.status->code = code;
    c.status->sm = c.sm;
    c.status->role = role;
    c.status->pc = pc;
    c.status->opcode = opcode;
    c.status->bar = bar;
    c.status->aux = aux;
    __threadfence();
  }
}

// Bounded polling.  `ready` is re-evaluated until it holds; every 64 polls the
// global abort flag and the wall-clock budget are checked.  Returns false when
// the wait was given up (by this thread or because another one aborted).
template <class Pred>
__device__ __forceinline__ bool wait_until(const Ctx& c, Pred ready, int role, int pc, int opcode, int bar,
                                           unsigned sleep_ns) {
  // Waits on a named global barrier use the budget as given; queue waits (a
  // role idling for work) get twice as long, so that when something is stuck
  // the wait that names the culprit is the one that reports.
  const uint64_t budget = bar >= 0 ? c.timeout_ns : 2 * c.timeout_ns;
  if (ready()) return true;
  uint32_t it = 0;
  uint64_t t0 = 0;
  while (true) {
    if (ready()) return true;
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((++it & 63u) == 0) {
      if (ld_relaxed_gpu(&c.status->abort) != 0) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget) {
        raise_abort(c, VDC_ERR_TIMEOUT, role, pc, opcode, bar, (int)it);
        return false;
      }
    }
  }
}

__device__ __forceinline__ bool wait_global_barrier(const Ctx& c, int bar, int role, int pc, int opcode) {
  const int* p = c.bars + bar;
  bool ok = wait_until(c, [&] { return ld_acquire_gpu(p) == 0; }, role, pc, opcode, bar, 32);
  fence_proxy_async();  // later bulk copies (async proxy) must observe what the releasing stores wrote
  return ok;
}

// ------------------------------------------------------------------------- //
// memory virtual core: control warp
// ------------------------------------------------------------------------- //
__device__ __forceinline__ VdcMInst load_minst(const VdcMInst* p) {
  uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  VdcMInst m;
  *reinterpret_cast<uint4*>(&m) = v;
  return m;
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
  unsigned m2c_tail = 0;
  unsigned ld_tail[2] = {0, 0};
  bool running = true;

  while (running) {
    pc = next_pc;
    VdcMInst inst = load_minst(insts + (pc % (uint32_t)n_insts));
    if (lane == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(insts + ((pc + 16) % (uint32_t)n_insts)));
    next_pc = pc + 1;

    uint64_t acc_i = __shfl_sync(0xffffffffu, accum, (int)((pc - (uint32_t)loop_start) & 31u));
    if (loop_counter > 0) inst.address += acc_i;
    if (inst.opcode & VDC_F_GROUP) inst.shifter += shift;
    const int port = (inst.opcode & VDC_F_PORT) ? 1 : 0;
    const uint16_t opid = inst.opcode >> VDC_FLAG_BITS;

    if (inst.opcode & VDC_F_ALLOCATE) {
      if (ind_pending) {
        inst.address += ind_off;
        ind_pending = false;
      }
      const int req = inst.num_slots & 63;
      int slot, m2c_word;
      if (req >= kSlots) {
        slot = req;  // special slot: nothing is allocated, the id itself is handed over
        m2c_word = req;
      } else {
        const uint32_t want = ((1u << req) - 1u) << lane;
        bool ok = true;
        uint32_t it = 0;
        uint64_t t0 = 0;
        while (true) {
          uint32_t avail = *reinterpret_cast<volatile uint32_t*>(&sh->slot_avail);
          avail = __shfl_sync(0xffffffffu, avail, 0);
          uint32_t cand = __ballot_sync(0xffffffffu, req > 0 && lane + req <= kSlots && (avail & want) == want);
          if (cand) {
            slot = __ffs(cand) - 1;
            break;
          }
          __nanosleep(20);
          if ((++it & 63u) == 0) {
            int ab = 0;
            if (lane == 0) {
              ab = ld_relaxed_gpu(&c.status->abort);
              uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > 2 * c.timeout_ns) {
                raise_abort(c, VDC_ERR_TIMEOUT, 1, (int)pc, inst.opcode, -1, req);
                ab = 1;
              }
            }
            ab = __shfl_sync(0xffffffffu, ab, 0);
            if (ab) {
              ok = false;
              break;
            }
          }
        }
        if (!ok) break;
        const uint32_t mask = ((1u << req) - 1u) << slot;
        if (lane == 0) atomicAnd(&sh->slot_avail, ~mask);
        m2c_word = (int)mask;
      }

      int ok = 1;
      if (lane == 0) {
        // queue entries are recycled only after the consumer moved past them
        ok = wait_until(c, [&] { return m2c_tail - sh->m2c_head < (unsigned)kQ; }, 1, (int)pc, inst.opcode, -1, 0);
        if (ok) ok = wait_until(c, [&] { return ld_tail[port] - sh->ld_head[port] < (unsigned)kQ; }, 1, (int)pc,
                                inst.opcode, -1, 0);
        if (ok) {
          const unsigned e = m2c_tail % kQ;
          sh->st_insts[slot] = inst;
          sh->m2c_data[e] = m2c_word;
          sh->ent_insts[e] = inst;
          sh->ld_q[port][ld_tail[port] % kQ] = (int)((uint32_t)slot | (e << 8) | ((uint32_t)inst.opcode << 16));
          __threadfence_block();
          sh->ld_tail[port] = ld_tail[port] + 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      m2c_tail++;
      ld_tail[port]++;

      if ((inst.opcode & VDC_F_JUMP) && loop_counter > 0) {
        --loop_counter;
        if (loop_counter > 0) next_pc = (uint32_t)loop_start;
        accum += delta;
      }
    } else {
      switch (opid) {
        case 1: {  // TERMINATE
          running = false;
          if (lane == 0) {
            for (int p = 0; p < 2; ++p) {
              bool ok = wait_until(c, [&] { return ld_tail[p] - sh->ld_head[p] < (unsigned)kQ; }, 1, (int)pc,
                                   inst.opcode, -1, 0);
              if (ok) {
                sh->ld_q[p][ld_tail[p] % kQ] = (int)kSlotEnd;
                __threadfence_block();
                sh->ld_tail[p] = ld_tail[p] + 1;
              }
            }
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
        default:
          break;  // OP_SHIFT_RESOURCE and unknown control ids are no-ops, as in the reference
      }
    }
  }
  // When the loop was left through an abort the load ports are not sent an end
  // marker: their own waits observe the global abort flag and return.
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
  unsigned head = 0;
  int reg_file[4] = {0, 0, 0, 0};
  const int role = 3 + port;
  while (true) {
    if (!wait_until(c, [&] { return sh->ld_tail[port] != head; }, role, (int)head, 0, -1, 0)) return;
    __threadfence_block();
    const uint32_t cmd = (uint32_t)sh->ld_q[port][head % kQ];
    head++;
    sh->ld_head[port] = head;
    const uint32_t slot = cmd & 0xFF;
    if (slot == kSlotEnd) return;
    const uint32_t e = (cmd >> 8) & 0xFF;
    const uint16_t opcode = (uint16_t)(cmd >> 16);
    const VdcMInst inst = sh->ent_insts[e];  // per-entry copy: special slots may be re-targeted meanwhile
    uint64_t* bar = &sh->full[e];

    if ((opcode & VDC_F_BARRIER) && !(opcode & VDC_F_WRITEBACK)) {
      if (!wait_global_barrier(c, inst.num_slots >> 6, role, (int)head, opcode)) return;
    }
    void* dst = slot < (uint32_t)kSlots ? slot_ptr(c, (int)slot) : nullptr;
    switch (opcode >> VDC_FLAG_BITS) {
      case 9:  // 1-D bulk load from a raw address
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
      case 15: {  // REG_STORE: remember the slot mask; the producer gets it with bit 31 set
        const int mask = sh->m2c_data[e];
        sh->m2c_data[e] = mask | (int)0x80000000;
        reg_file[inst.size & 3] = mask;
        __threadfence_block();
        mbar_arrive(bar);
        break;
      }
      case 8:  // REG_LOAD: hand the remembered mask to the consumer
        sh->m2c_data[e] = reg_file[inst.size & 3];
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
// compute virtual core: queue access
// ------------------------------------------------------------------------- //
struct Compute {
  const Ctx& c;
  Shared* sh;
  int tid, warp, lane;
  unsigned head;     // m2c entries popped so far (uniform across the 256 threads)
  unsigned st_tail;  // store-queue pushes so far (thread 0)
  uint32_t pc;
  bool aborted;
  uint64_t stall;    // cycles thread 0 spent waiting for data

  __device__ __forceinline__ int pop() {
    if (tid == 0) {
      const unsigned e = head % kQ;
      const uint32_t parity = (head / kQ) & 1u;
      uint64_t* bar = &sh->full[e];
      int v;
      if (mbar_try_wait(bar, parity)) {
        v = sh->m2c_data[e];
      } else {
        const long long t0 = clock64();
        bool ok = wait_until(c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)pc, 0, -1, 0);
        stall += (uint64_t)(clock64() - t0);
        v = ok ? sh->m2c_data[e] : kPopAbort;
      }
      sh->pop_val[head & 1u] = v;
      sh->pop_addr[head & 1u] = sh->ent_insts[e].address;
      sh->pop_meta[head & 1u] = (uint32_t)sh->ent_insts[e].opcode | ((uint32_t)sh->ent_insts[e].num_slots << 16);
      __threadfence_block();
      sh->m2c_head = head + 1;
    }
    compute_sync();
    const int v = sh->pop_val[head & 1u];
    head++;
    if (v == kPopAbort) aborted = true;
    return v;
  }
  // Address / (opcode | num_slots << 16) of the instruction behind the last pop.
  __device__ __forceinline__ uint64_t addr() const { return sh->pop_addr[(head - 1u) & 1u]; }
  __device__ __forceinline__ uint32_t meta() const { return sh->pop_meta[(head - 1u) & 1u]; }
  // Counts down the global barrier named by a popped raw-address instruction
  // that carries BARRIER|WRITEBACK.  Caller guarantees every writer executed
  // __threadfence() and a compute_sync() since its last global write.
  __device__ __forceinline__ void release(uint32_t m) {
    if (tid == 0 && (m & VDC_F_BARRIER) && (m & VDC_F_WRITEBACK)) {
      __threadfence();
      red_release_gpu_add(c.bars + (m >> 22), -1);
    }
  }
  // Caller guarantees (with a compute_sync) that no thread still reads the slots.
  __device__ __forceinline__ void free_slots(int mask) {
    if (tid == 0 && mask > 0) atomicOr(&sh->slot_avail, (uint32_t)mask & kSlotMaskAll);
  }
  // Hands slots to the store warp.  Caller guarantees all writers executed
  // fence_proxy_async_smem() and a compute_sync() since their last write.
  __device__ __forceinline__ void push_store(int mask) {
    if (mask < 0) return;  // RegStore'd result stays resident
    if (tid == 0) {
      bool ok = wait_until(c, [&] { return st_tail - sh->st_head < (unsigned)kQ; }, 0, (int)pc, 0, -1, 0);
      if (ok) {
        sh->st_q[st_tail % kQ] = mask;
        __threadfence_block();
        sh->st_tail = st_tail + 1;
        st_tail++;
      }
    }
  }
};

__device__ __forceinline__ int first_slot(int mask) { return __ffs(mask & 0x7fffffff) - 1; }

// ------------------------------------------------------------------------- //
// task: row-block GEMV  y[r] = sum_k W[r,k] x[k]   (batch-1 decode projections)
// ------------------------------------------------------------------------- //
// Pop order: [norm weight], x, out, [argmax pair out], then n_chunks weight
// chunks of R rows x K bf16 (row-major, contiguous).  All eight warps split K
// in 256-element steps; each lane keeps R fp32 partial sums.
template <int R>
__device__ __forceinline__ void gemv_accumulate(const uint8_t* w, const uint8_t* x, int K, int warp, int lane,
                                                float (&acc)[R]) {
  const int iters = K >> 8;
  for (int it = warp; it < iters; it += kCW) {
    const int off = (it << 9) + (lane << 4);  // byte offset of this lane's 8 elements
    const uint4 xv = lds128(x + off);
    float xf[8] = {bf_lo(xv.x), bf_hi(xv.x), bf_lo(xv.y), bf_hi(xv.y), bf_lo(xv.z), bf_hi(xv.z), bf_lo(xv.w), bf_hi(xv.w)};
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint4 wv = lds128(w + (size_t)r * K * 2 + off);
      float a = acc[r];
      a = fmaf(bf_lo(wv.x), xf[0], a);
      a = fmaf(bf_hi(wv.x), xf[1], a);
      a = fmaf(bf_lo(wv.y), xf[2], a);
      a = fmaf(bf_hi(wv.y), xf[3], a);
      a = fmaf(bf_lo(wv.z), xf[4], a);
      a = fmaf(bf_hi(wv.z), xf[5], a);
      a = fmaf(bf_lo(wv.w), xf[6], a);
      a = fmaf(bf_hi(wv.w), xf[7], a);
      acc[r] = a;
    }
  }
}

struct ArgBest {
  float val;
  int idx;
};

template <int R>
__device__ void task_gemv_rows(Compute& q, int n_chunks, int mode, bool accumulate, bool norm, int K, int row_base) {
  Shared* sh = q.sh;
  const Ctx& c = q.c;
  int normw_mask = 0;
  if (norm) normw_mask = q.pop();
  const int x_mask = q.pop();
  q.pop();  // output vector: raw address
  __nv_bfloat16* outg = reinterpret_cast<__nv_bfloat16*>(q.addr());
  const uint32_t out_meta = q.meta();
  float* recg = nullptr;
  uint32_t rec_meta = 0;
  if (mode == VDC_GEMV_MODE_ARGMAX) {
    q.pop();  // candidate record: raw address
    recg = reinterpret_cast<float*>(q.addr());
    rec_meta = q.meta();
  }
  if (q.aborted) return;
  uint8_t* x = (uint8_t*)slot_ptr(c, first_slot(x_mask));

  if (norm) {
    // RMSNorm of the activation vector in place: bf16(w * bf16(x * rstd)), fp32 statistics
    const uint8_t* nw = (const uint8_t*)slot_ptr(c, first_slot(normw_mask));
    float ss = 0.f;
    for (int i = q.tid * 8; i < K; i += kCT * 8) {
      const uint4 v = lds128(x + i * 2);
      const float f[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = warp_sum(ss);
    if (q.lane == 0) sh->misc[q.warp] = ss;
    compute_sync();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; ++w) tot += sh->misc[w];
    const float rstd = rsqrtf(tot / (float)K + sh->misc[32]);  // misc[32]: eps, set by the dispatcher
    for (int i = q.tid * 2; i < K; i += kCT * 2) {
      const uint32_t xv = *reinterpret_cast<const uint32_t*>(x + i * 2);
      const uint32_t wv = *reinterpret_cast<const uint32_t*>(nw + i * 2);
      const float a = bf16_round(bf_lo(wv) * bf16_round(bf_lo(xv) * rstd));
      const float b = bf16_round(bf_hi(wv) * bf16_round(bf_hi(xv) * rstd));
      *reinterpret_cast<uint32_t*>(x + i * 2) = (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xffff0000u);
    }
    compute_sync();
    q.free_slots(normw_mask);
  }

  // part[buf][r][warp]
  float* part = sh->red;
  ArgBest best = {-INFINITY, 0x7fffffff};
  int prev_mask = 0;
  for (int i = 0; i <= n_chunks; ++i) {
    int w_mask = 0;
    if (i < n_chunks) {
      w_mask = q.pop();
      if (q.aborted) return;
    } else {
      compute_sync();
    }
    // chunk i-1 is complete on every warp once the sync inside pop() has passed
    if (i > 0) {
      q.free_slots(prev_mask);
      const float* pp = part + ((i - 1) & 1) * (R * kCW);
      const int row0 = (i - 1) * R;
      if (mode == VDC_GEMV_MODE_SILU_PAIRS) {
        if (q.tid < R / 2) {
          float g = 0.f, u = 0.f;
#pragma unroll
          for (int w = 0; w < kCW; ++w) {
            g += pp[(2 * q.tid) * kCW + w];
            u += pp[(2 * q.tid + 1) * kCW + w];
          }
          g = bf16_round(g);
          u = bf16_round(u);
          const float sg = bf16_round(g / (1.f + __expf(-g)));
          outg[row0 / 2 + q.tid] = __float2bfloat16_rn(sg * u);
        }
      } else if (q.tid < R) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kCW; ++w) v += pp[q.tid * kCW + w];
        const __nv_bfloat16 b = __float2bfloat16_rn(v);
        if (accumulate) atomicAdd(outg + row0 + q.tid, b);  // residual add: bf16(old + bf16(W x))
        else outg[row0 + q.tid] = b;
        if (mode == VDC_GEMV_MODE_ARGMAX) {
          const float bv = __bfloat162float(b);
          if (bv > best.val) {  // rows are visited in ascending order: first maximum wins
            best.val = bv;
            best.idx = row0 + q.tid;
          }
        }
      }
    }
    if (i < n_chunks) {
      const uint8_t* w = (const uint8_t*)slot_ptr(c, first_slot(w_mask));
      float acc[R];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
      gemv_accumulate<R>(w, x, K, q.warp, q.lane, acc);
      float* pw = part + (i & 1) * (R * kCW);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float sum = warp_sum(acc[r]);
        if (q.lane == 0) pw[r * kCW + q.warp] = sum;
      }
      prev_mask = w_mask;
    }
  }

  if (mode == VDC_GEMV_MODE_ARGMAX && q.warp == 0) {
    // threads 0..R-1 hold candidates; the lowest row index wins ties
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best.val, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best.idx, o);
      if (ov > best.val || (ov == best.val && oi < best.idx)) {
        best.val = ov;
        best.idx = oi;
      }
    }
    if (q.lane == 0) {
      recg[0] = best.val;
      reinterpret_cast<int*>(recg)[1] = best.idx + row_base;
      recg[2] = 0.f;
      recg[3] = 0.f;
    }
  }
  if (q.tid < 32) __threadfence();  // the writers of the output vector all sit in warp 0
  compute_sync();
  q.release(out_meta);
  q.release(rec_meta);
  q.free_slots(x_mask);
}

// ------------------------------------------------------------------------- //
// task: split-K GQA decode attention over 64-position KV pages
// ------------------------------------------------------------------------- //
// Pop order: state (raw address), rope row (cos[64] sin[64] fp32), [q/k norm
// weights 2x128 bf16], q (G x 128 bf16, raw projection output), k_new, v_new
// (128 bf16 each, raw projection output of the token being decoded), k_row_out,
// v_row_out (write-back slots for the new cache rows), `count` x (K page, V page),
// out (write-back: G x 128 fp32 unnormalised O, then m[G], l[G]).
// count = clamp(n_pages - base, 0, max_pages) is read from the state block; the
// memory stream uses the same rule (DYN_COUNT + REPEAT).
template <int G>
__device__ void task_attn_decode(Compute& q, int max_pages, int base_page, int flags) {
  constexpr int D = VDC_HEAD_DIM;
  constexpr int LPP = (G == 4) ? 8 : 16;  // lanes per position in the QK phase
  constexpr int DPL = D / LPP;            // dims per lane: 16 or 8
  constexpr int PPW = 32 / LPP;           // positions per warp per round
  constexpr int ROUNDS = VDC_KV_PAGE / (PPW * kCW);
  Shared* sh = q.sh;
  const Ctx& c = q.c;
  const bool qk_norm = flags & VDC_ATTN_QKNORM_BIT;

  q.pop();  // decode state block: raw address
  const int* state = reinterpret_cast<const int*>(q.addr());
  const int rope_mask = q.pop();
  int nw_mask = 0;
  if (qk_norm) nw_mask = q.pop();
  const int q_mask = q.pop();
  const int kn_mask = q.pop();
  const int vn_mask = q.pop();
  const int kro_mask = q.pop();
  const int vro_mask = q.pop();
  if (q.aborted) return;

  const int pos = ld_relaxed_gpu(state + VDC_ST_POS);
  const int n_pages = ld_relaxed_gpu(state + VDC_ST_NPAGES);
  int count = n_pages - base_page;
  count = count < 0 ? 0 : (count > max_pages ? max_pages : count);
  const bool owner = count > 0 && base_page + count == n_pages;
  const int tail_valid = (pos % VDC_KV_PAGE) + 1;  // valid rows of the last page, new row included

  const float* rope = (const float*)slot_ptr(c, first_slot(rope_mask));
  const __nv_bfloat16* nw = qk_norm ? (const __nv_bfloat16*)slot_ptr(c, first_slot(nw_mask)) : nullptr;
  const __nv_bfloat16* qraw = (const __nv_bfloat16*)slot_ptr(c, first_slot(q_mask));
  const __nv_bfloat16* knew = (const __nv_bfloat16*)slot_ptr(c, first_slot(kn_mask));
  __nv_bfloat16* krow = (__nv_bfloat16*)slot_ptr(c, first_slot(kro_mask));
  __nv_bfloat16* vrow = (__nv_bfloat16*)slot_ptr(c, first_slot(vro_mask));
  const float eps = sh->misc[33];

  // --- prologue: optional per-head RMSNorm, then half-rotation RoPE.  One warp
  // per head: heads 0..G-1 are the queries, "head" G is the new key row.
  for (int head = q.warp; head <= G; head += kCW) {
    const bool is_k = head == G;
    const __nv_bfloat16* src = is_k ? knew : qraw + head * D;
    const int i0 = q.lane * 2;  // pairs (i0, i0+64), (i0+1, i0+65)
    float a0 = __bfloat162float(src[i0]), a1 = __bfloat162float(src[i0 + 1]);
    float b0 = __bfloat162float(src[i0 + 64]), b1 = __bfloat162float(src[i0 + 65]);
    if (qk_norm) {
      float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
      const float rstd = rsqrtf(ss / (float)D + eps);
      const __nv_bfloat16* w = nw + (is_k ? D : 0);
      a0 = bf16_round(__bfloat162float(w[i0]) * bf16_round(a0 * rstd));
      a1 = bf16_round(__bfloat162float(w[i0 + 1]) * bf16_round(a1 * rstd));
      b0 = bf16_round(__bfloat162float(w[i0 + 64]) * bf16_round(b0 * rstd));
      b1 = bf16_round(__bfloat162float(w[i0 + 65]) * bf16_round(b1 * rstd));
    }
    const float c0 = rope[i0], c1 = rope[i0 + 1], s0 = rope[64 + i0], s1 = rope[64 + i0 + 1];
    // x*cos + rotate_half(x)*sin with every product and the sum rounded to bf16,
    // the way a bf16 tensor expression evaluates it
    const float r0 = bf16_round(bf16_round(a0 * c0) - bf16_round(b0 * s0));
    const float r1 = bf16_round(bf16_round(a1 * c1) - bf16_round(b1 * s1));
    const float r64 = bf16_round(bf16_round(b0 * c0) + bf16_round(a0 * s0));
    const float r65 = bf16_round(bf16_round(b1 * c1) + bf16_round(a1 * s1));
    if (is_k) {
      krow[i0] = __float2bfloat16_rn(r0);
      krow[i0 + 1] = __float2bfloat16_rn(r1);
      krow[i0 + 64] = __float2bfloat16_rn(r64);
      krow[i0 + 65] = __float2bfloat16_rn(r65);
    } else {
      float* dst = sh->qrot + head * D;
      dst[i0] = r0;
      dst[i0 + 1] = r1;
      dst[i0 + 64] = r64;
      dst[i0 + 65] = r65;
    }
  }
  if (q.tid < D / 8) {  // v_new row copied as is (16 threads x 16 bytes)
    reinterpret_cast<uint4*>(vrow)[q.tid] = reinterpret_cast<const uint4*>(slot_ptr(c, first_slot(vn_mask)))[q.tid];
  }
  fence_proxy_async_smem();
  compute_sync();
  q.free_slots(rope_mask | nw_mask | q_mask | kn_mask | vn_mask);

  // per-lane slice of the rotated queries
  const int sub = q.lane % LPP, pl = q.lane / LPP;
  float qreg[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int h = 0; h < DPL / 8; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) qreg[g][h * 8 + j] = sh->qrot[g * D + (sub + h * 8) * 8 + j];
  const float scale_log2 = 1.4426950408889634f * rsqrtf((float)D);

  float m_run[G], l_run[G], acc[G][2];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
    acc[g][0] = acc[g][1] = 0.f;
  }
  const int pg = q.tid >> 6, dp = q.tid & 63;  // PV phase: position group, dim pair

  int v_prev = 0;
  for (int blk = 0; blk < count; ++blk) {
    const int k_mask = q.pop();  // its sync also ends the previous block's PV phase
    if (q.aborted) return;
    q.free_slots(v_prev);
    uint8_t* kb = (uint8_t*)slot_ptr(c, first_slot(k_mask));
    const bool last = owner && blk == count - 1;
    const int valid = last ? tail_valid : VDC_KV_PAGE;
    if (last) {
      // the page in HBM does not hold the new row yet: patch it in shared memory
      if (q.tid < D / 8)
        reinterpret_cast<uint4*>(kb + (valid - 1) * D * 2)[q.tid] = reinterpret_cast<const uint4*>(krow)[q.tid];
      compute_sync();
    }
    // ---- phase 1: scores = q . k for 64 positions
    float wm[G];
#pragma unroll
    for (int g = 0; g < G; ++g) wm[g] = -INFINITY;
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
      const int p = rd * (PPW * kCW) + q.warp * PPW + pl;
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
      for (int h = 0; h < DPL / 8; ++h) {
        const uint4 kv = lds128(kb + p * (D * 2) + (sub + h * 8) * 16);
        const float kf[8] = {bf_lo(kv.x), bf_hi(kv.x), bf_lo(kv.y), bf_hi(kv.y),
                             bf_lo(kv.z), bf_hi(kv.z), bf_lo(kv.w), bf_hi(kv.w)};
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int j = 0; j < 8; ++j) s[g] = fmaf(qreg[g][h * 8 + j], kf[j], s[g]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = 1; o < LPP; o <<= 1) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
        s[g] = (p < valid) ? s[g] * scale_log2 : -INFINITY;
        wm[g] = fmaxf(wm[g], s[g]);
      }
      if (sub == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) sh->scores[p * G + g] = s[g];
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int o = LPP; o < 32; o <<= 1) wm[g] = fmaxf(wm[g], __shfl_xor_sync(0xffffffffu, wm[g], o));
      if (q.lane == 0) sh->wmax[q.warp * G + g] = wm[g];
    }
    compute_sync();  // (A) scores and warp maxima visible; K page fully read
    q.free_slots(k_mask);
    // ---- phase 2: running max, rescale factors, probabilities
    float alpha[G], m_new[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mb = sh->wmax[g];
#pragma unroll
      for (int w = 1; w < kCW; ++w) mb = fmaxf(mb, sh->wmax[w * G + g]);
      m_new[g] = fmaxf(m_run[g], mb);
      alpha[g] = (m_new[g] == -INFINITY) ? 1.f : exp2f(m_run[g] - m_new[g]);
      m_run[g] = m_new[g];
    }
    for (int t = q.tid; t < VDC_KV_PAGE * G; t += kCT) {
      const int g = t % G;
      const float s = sh->scores[t];
      // HF rounds probabilities to bf16 after the softmax; here they stay fp32
      sh->probs[t] = (m_new[g] == -INFINITY) ? 0.f : exp2f(s - m_new[g]);
    }
    const int v_mask = q.pop();  // (B) its sync publishes probs
    if (q.aborted) return;
    uint8_t* vb = (uint8_t*)slot_ptr(c, first_slot(v_mask));
    if (last) {
      if (q.tid < D / 8)
        reinterpret_cast<uint4*>(vb + (valid - 1) * D * 2)[q.tid] = reinterpret_cast<const uint4*>(vrow)[q.tid];
      compute_sync();
    }
    // ---- phase 3: O += P V over this thread's 16 positions, two dims per thread
#pragma unroll
    for (int g = 0; g < G; ++g) {
      acc[g][0] *= alpha[g];
      acc[g][1] *= alpha[g];
      l_run[g] *= alpha[g];
    }
    const int p_end = min(pg * 16 + 16, valid);
    for (int p = pg * 16; p < p_end; ++p) {
      const uint32_t vv = *reinterpret_cast<const uint32_t*>(vb + p * (D * 2) + dp * 4);
      const float v0 = bf_lo(vv), v1 = bf_hi(vv);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = sh->probs[p * G + g];
        l_run[g] += pr;
        acc[g][0] = fmaf(pr, v0, acc[g][0]);
        acc[g][1] = fmaf(pr, v1, acc[g][1]);
      }
    }
    v_prev = v_mask;
  }

  const int out_mask = q.pop();  // sync: everyone is done with the last V page
  if (q.aborted) return;
  q.free_slots(v_prev);
  float* out = (float*)slot_ptr(c, first_slot(out_mask));
  // cross position-group reduction: groups 1..3 publish, group 0 adds
  float* red = sh->red;  // [3][G][128] then l: [3][G]
  if (pg > 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      red[((pg - 1) * G + g) * D + dp * 2] = acc[g][0];
      red[((pg - 1) * G + g) * D + dp * 2 + 1] = acc[g][1];
      if (dp == 0) red[3 * G * D + (pg - 1) * G + g] = l_run[g];
    }
  }
  compute_sync();
  if (pg == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float o0 = acc[g][0], o1 = acc[g][1], l = l_run[g];
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        o0 += red[(r * G + g) * D + dp * 2];
        o1 += red[(r * G + g) * D + dp * 2 + 1];
        l += red[3 * G * D + r * G + g];
      }
      out[g * D + dp * 2] = o0;
      out[g * D + dp * 2 + 1] = o1;
      if (dp == 0) {
        out[G * D + g] = m_run[g];
        out[G * D + G + g] = l;
      }
    }
  }
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(out_mask);
  if (owner) {
    q.push_store(kro_mask);
    q.push_store(vro_mask);
  } else {
    q.free_slots(kro_mask | vro_mask);
  }
}

// ------------------------------------------------------------------------- //
// task: merge the split partials of one KV head:  O = sum_s 2^(m_s-m) O_s / sum_s 2^(m_s-m) l_s
// ------------------------------------------------------------------------- //
// Pop order: records part 1 (n1 records), [records part 2], out (G*128 bf16).
// Record = G*128 fp32 O, G fp32 m, G fp32 l, padded to a multiple of 64 bytes.
__device__ void task_attn_merge(Compute& q, int n_splits, int G, int n1) {
  constexpr int D = VDC_HEAD_DIM;
  const Ctx& c = q.c;
  const int rec_floats = G * D + 16 * ((2 * G + 15) / 16);
  const int m1 = q.pop();
  int m2 = 0;
  if (n_splits > n1) m2 = q.pop();
  const int out_mask = q.pop();
  if (q.aborted) return;
  const float* r1 = (const float*)slot_ptr(c, first_slot(m1));
  const float* r2 = m2 ? (const float*)slot_ptr(c, first_slot(m2)) : nullptr;
  __nv_bfloat16* out = (__nv_bfloat16*)slot_ptr(c, first_slot(out_mask));
  for (int o = q.tid; o < G * D; o += kCT) {
    const int g = o / D;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) {
      const float* r = s < n1 ? r1 + s * rec_floats : r2 + (s - n1) * rec_floats;
      m = fmaxf(m, r[G * D + g]);
    }
    float num = 0.f, den = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float* r = s < n1 ? r1 + s * rec_floats : r2 + (s - n1) * rec_floats;
      const float ms = r[G * D + g];
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      num = fmaf(w, r[o], num);
      den = fmaf(w, r[G * D + G + g], den);
    }
    out[o] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
  }
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(out_mask);
  q.free_slots(m1 | m2);
}

// ------------------------------------------------------------------------- //
// task: final argmax over the per-SM candidates, token hand-over, state advance
// ------------------------------------------------------------------------- //
// Pop order: candidate records (n x {f32 val, i32 idx, pad, pad}), state (raw
// address), token log (raw address, int32 per step), done (raw address slot that
// is pushed back so the store warp can release a barrier).
__device__ void task_argmax_final(Compute& q, int n) {
  const Ctx& c = q.c;
  const int rec_mask = q.pop();
  q.pop();
  int* state = reinterpret_cast<int*>(q.addr());
  q.pop();
  int* log = reinterpret_cast<int*>(q.addr());
  const uint32_t log_meta = q.meta();
  if (q.aborted) return;
  if (q.warp == 0) {
    const float* rec = (const float*)slot_ptr(c, first_slot(rec_mask));
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = q.lane; i < n; i += 32) {
      const float v = rec[i * 4];
      const int idx = reinterpret_cast<const int*>(rec)[i * 4 + 1];
      if (v > bv || (v == bv && idx < bi)) {
        bv = v;
        bi = idx;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (q.lane == 0) {
      const int step = state[VDC_ST_STEP];
      const int pos = state[VDC_ST_POS] + 1;
      log[step] = bi;
      state[VDC_ST_TOKEN] = bi;
      state[VDC_ST_STEP] = step + 1;
      state[VDC_ST_POS] = pos;
      const int page = pos / VDC_KV_PAGE;
      state[VDC_ST_NPAGES] = page + 1;
      if (page < state[VDC_ST_MAXPAGES]) {
        state[VDC_ST_NEWROW] = state[VDC_ST_PAGETABLE + page] * VDC_KV_PAGE * state[VDC_ST_NKVH] + pos % VDC_KV_PAGE;
      } else {
        state[VDC_ST_ERR] = 1;  // out of KV pages: the host must not launch another step
      }
      __threadfence();
    }
  }
  compute_sync();
  q.release(log_meta);
  q.free_slots(rec_mask);
}

// ------------------------------------------------------------------------- //
// compute virtual core: dispatch
// ------------------------------------------------------------------------- //
__device__ void compute_core(const Ctx& c, const VdcCInst* __restrict__ insts, int n_insts, int tid) {
  Compute q{c, c.sh, tid, tid >> 5, tid & 31, 0u, 0u, 0u, false, 0ull};
  uint32_t count = 0;
  bool finish = false;
  while (!finish && !q.aborted) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(insts + (q.pc % (uint32_t)n_insts)));
    VdcCInst ci;
    *reinterpret_cast<uint2*>(&ci) = raw;
    q.pc++;
    switch (ci.opcode) {
      case 0x7000:  // TERMINATEC
        if (tid == 0) {
          // mask 0 tells the store warp to drain and leave
          bool ok = wait_until(c, [&] { return q.st_tail - q.sh->st_head < (unsigned)kQ; }, 0, (int)q.pc, ci.opcode, -1, 0);
          if (ok) {
            q.sh->st_q[q.st_tail % kQ] = 0;
            __threadfence_block();
            q.sh->st_tail = q.st_tail + 1;
          }
          c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 1] = globaltimer_ns();
          c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 2] = q.stall;
        }
        finish = true;
        break;
      case 0x7001:  // LOOPC
        if (++count < ci.args[0]) q.pc = ci.args[1];
        else count = 0;
        compute_sync();
        break;
      case 0x7002:  // DUMMY: pass slots through untouched
        for (int i = 0; i < ci.args[0] && !q.aborted; ++i) {
          const int m = q.pop();
          if (q.aborted) break;
          __nanosleep(ci.args[1]);
          q.free_slots(m);
        }
        break;
      case 0x7003:  // COPY: args[0] x { pop src, pop dst, copy args[1] 32-bit words, write dst back }
        for (int i = 0; i < ci.args[0] && !q.aborted; ++i) {
          const int src_m = q.pop();
          const int dst_m = q.pop();
          if (q.aborted) break;
          const uint32_t* s = (const uint32_t*)slot_ptr(c, first_slot(src_m));
          uint32_t* d = (uint32_t*)slot_ptr(c, first_slot(dst_m));
          for (int j = tid; j < ci.args[1]; j += kCT) d[j] = s[j];
          fence_proxy_async_smem();
          compute_sync();
          q.push_store(dst_m);
          q.free_slots(src_m);
        }
        break;
      case 0x7200: {  // GEMV_ROWS_BF16 (two words)
        const int R = ci.args[1] & 31, mode = (ci.args[1] >> 8) & 7;
        const bool accumulate = ci.args[1] & VDC_GEMV_ACC_BIT;
        const bool norm = ci.args[1] & VDC_GEMV_NORM_BIT;
        const int K = (ci.args[2] & 0xFF) << 8;
        VdcCInst ex;
        *reinterpret_cast<uint2*>(&ex) = __ldg(reinterpret_cast<const uint2*>(insts + (q.pc % (uint32_t)n_insts)));
        q.pc++;
        if (tid == 0) q.sh->misc[32] = __uint_as_float(((uint32_t)ex.args[0] << 16) | ex.args[1]);  // norm eps
        const int row_base = ((int)ex.args[2] | ((int)(ci.args[2] >> 8) << 16)) * 8;  // first output row (argmax)
        switch (R) {
          case 1: task_gemv_rows<1>(q, ci.args[0], mode, accumulate, norm, K, row_base); break;
          case 2: task_gemv_rows<2>(q, ci.args[0], mode, accumulate, norm, K, row_base); break;
          case 4: task_gemv_rows<4>(q, ci.args[0], mode, accumulate, norm, K, row_base); break;
          case 8: task_gemv_rows<8>(q, ci.args[0], mode, accumulate, norm, K, row_base); break;
          case 16: task_gemv_rows<16>(q, ci.args[0], mode, accumulate, norm, K, row_base); break;
          default: raise_abort(c, VDC_ERR_BAD_OPCODE, 0, (int)q.pc, ci.opcode, -1, R); q.aborted = true; break;
        }
        break;
      }
      case 0x7210:
      case 0x7211: {
        VdcCInst ex;
        *reinterpret_cast<uint2*>(&ex) = __ldg(reinterpret_cast<const uint2*>(insts + (q.pc % (uint32_t)n_insts)));
        q.pc++;
        if (tid == 0) q.sh->misc[33] = __uint_as_float(((uint32_t)ex.args[0] << 16) | ex.args[1]);  // qk-norm eps
        compute_sync();
        if (ci.opcode == 0x7210) task_attn_decode<4>(q, ci.args[0], ci.args[1], ci.args[2]);
        else task_attn_decode<8>(q, ci.args[0], ci.args[1], ci.args[2]);
        break;
      }
      case 0x7212: task_attn_merge(q, ci.args[0], ci.args[1], ci.args[2]); break;
      case 0x7220: task_argmax_final(q, ci.args[0]); break;
      default:
        raise_abort(c, VDC_ERR_BAD_OPCODE, 0, (int)q.pc, ci.opcode, -1, 0);
        q.aborted = true;
        break;
    }
  }
}

// ------------------------------------------------------------------------- //
// the kernel
// ------------------------------------------------------------------------- //
__global__ void __launch_bounds__(VDC_THREADS, 1)
vdc_megakernel(const VdcCInst* __restrict__ cinsts, const VdcMInst* __restrict__ minsts,
               const CUtensorMap* __restrict__ tmas, int* bars, uint64_t* profile, vdc_status* status,
               int insts_per_sm, uint64_t timeout_ns) {
  __shared__ Shared sh;
  extern __shared__ uint8_t dyn_smem[];
  const int tid = threadIdx.x;
  Ctx c;
  c.sh = &sh;
  c.slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~(uintptr_t)1023);
  c.tmas = tmas;
  c.bars = bars;
  c.status = status;
  c.profile = profile;
  c.timeout_ns = timeout_ns;
  c.sm = blockIdx.x;

  if (tid < kQ) mbar_init(&sh.full[tid], 1);
  if (tid == 0) {
    sh.slot_avail = kSlotMaskAll;
    sh.m2c_head = 0;
    sh.ld_head[0] = sh.ld_head[1] = sh.ld_tail[0] = sh.ld_tail[1] = 0;
    sh.st_head = sh.st_tail = 0;
    profile[c.sm * VDC_NUM_PROFILE_EVENTS + 0] = globaltimer_ns();
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (tid < kCT) {
    compute_core(c, cinsts + (size_t)c.sm * insts_per_sm, insts_per_sm, tid);
  } else {
    const int w = (tid - kCT) >> 5, lane = tid & 31;
    if (w == 0) control_warp(c, minsts + (size_t)c.sm * insts_per_sm, insts_per_sm, lane);
    else if (w == 1) { if (lane == 0) store_warp(c); }
    else if (lane == 0) load_port(c, w - 2);
  }
  __syncthreads();
  // After an abort some bulk loads may still be in flight towards this CTA's
  // shared memory: give them a bounded time to land before the CTA retires.
  if (tid == 0 && ld_relaxed_gpu(&status->abort) != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  __syncthreads();
}

}  // namespace vdc

// ------------------------------------------------------------------------- //
// host entry used by the C ABI
// ------------------------------------------------------------------------- //
extern "C" size_t vdc_megakernel_dynamic_smem() { return (size_t)VDC_NUM_SLOTS * VDC_SLOT_BYTES + 1024; }

extern "C" cudaError_t vdc_megakernel_prepare() {
  return cudaFuncSetAttribute(vdc::vdc_megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)vdc_megakernel_dynamic_smem());
}

extern "C" cudaError_t vdc_megakernel_launch(int num_sms, const void* cinsts, const void* minsts, const void* tmas,
                                             int* bars, uint64_t* profile, vdc_status* status, int insts_per_sm,
                                             uint64_t timeout_ns, cudaStream_t stream) {
  vdc::vdc_megakernel<<<num_sms, VDC_THREADS, vdc_megakernel_dynamic_smem(), stream>>>(
      reinterpret_cast<const VdcCInst*>(cinsts), reinterpret_cast<const VdcMInst*>(minsts),
      reinterpret_cast<const CUtensorMap*>(tmas), bars, profile, status, insts_per_sm, timeout_ns);
  return cudaGetLastError();
}
