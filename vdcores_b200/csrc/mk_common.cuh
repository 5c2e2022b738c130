// Common definitions of the persistent decode megakernel for sm_100a.
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
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "isa.h"

namespace vdc {

#ifndef VDC_SPIN_SLEEP
#define VDC_SPIN_SLEEP 0
#endif
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
__device__ __forceinline__ float ld_relaxed_gpu_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
// One 8-byte entry of the in-kernel tensor-parallel exchange: {payload, sequence tag}.  An aligned 64-bit
// scalar store is a single copy, so a reader that finds the tag it expects has the payload that goes with it:
// no fence and no arrival counter stand between a partial result and its consumers on the other GPUs.
__device__ __forceinline__ void st_tagged_sys(unsigned long long addr, uint32_t payload, uint32_t tag) {
  const unsigned long long v = ((unsigned long long)tag << 32) | payload;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged_sys(const void* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ int atom_acquire_gpu_add(int* p, int v) {
  int old;
  asm volatile("atom.acquire.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_relaxed_gpu_add(int* p, int v) {
  asm volatile("red.relaxed.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
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
  VdcMInst st_insts[kSlots + VDC_NUM_SPECIAL_SLOTS];  // write-back instruction that owns each slot (store warp)
  // The instruction ring: the control warp publishes one entry per allocating
  // instruction; both load ports walk it (each takes the entries of its port),
  // the compute core consumes the entries in order through `full`.
  VdcMInst ring[kQ];
  VdcMInst icache[64];      // control warp's window of the memory instruction stream
  int ring_word[kQ];        // slot mask of the entry, or the special slot id
  uint64_t full[kQ];        // completion barrier of the entry (1 arrival + TMA bytes)
  int st_q[kQ];             // compute -> store warp slot masks
  volatile unsigned ring_tail;              // entries published so far
  volatile unsigned cta_head;               // entries consumed by CTA-wide pops (and finished per-warp phases)
  volatile unsigned warp_next[VDC_COMPUTE_WARPS];  // next entry of each warp inside a per-warp phase, else ~0u
  volatile unsigned st_head, st_tail;
  unsigned slot_avail;                      // bit i set = slot i free
  volatile int aborted;                     // some compute wait in this CTA gave up
  // HBM->L2 streamer: the control warp publishes how many bytes of the weight
  // stream it has issued loads for; the streamer warp keeps the L2 prefetch
  // frontier a bounded distance ahead of that.
  volatile unsigned demand_pos;
  volatile unsigned long long pf_list;      // device array of {u64 addr, u32 bytes, u32 pad}
  volatile unsigned pf_n;
  volatile unsigned pf_window;              // bytes the frontier may run ahead
  volatile int pf_go, pf_exit;
  uint32_t pt_words[32];                    // control warp: the table words PT_LOAD32 fetched (page loop)
  volatile int pop_val[8];                  // what thread 0 read for the CTA-wide pops (entry index mod 8)
  volatile uint32_t pop_meta[8];
  volatile uint32_t pop_size[8];
  volatile uint64_t pop_addr[8];
  volatile int pair_ok[4][2][2];            // GEMV warp pairs: [pair][trip parity][member] chunk arrived
  int att_done[8];                          // attention: warps finished with page pair i % 8
  alignas(16) float red[4096 + 64];                     // task scratch (reductions)
  alignas(16) __nv_bfloat16 qbf[8 * VDC_HEAD_DIM];  // attention: rotated query heads (bf16), tensor-core A operand
  alignas(16) float misc[64];
  uint4 newrows[32];                        // attention: rotated new key row, new value row (bf16, page-row swizzle)
  uint4 zero_row[16];                       // attention: stands in for value rows past the last valid position
  // tensor cores (batched decode): tensor memory is allocated by the first task that needs it
  uint32_t tmem_base;                       // written by tcgen05.alloc
  volatile int tmem_ready;
  uint64_t mma_bar[4];                      // completion of the tensor-core work of chunk i % 4
  uint64_t mma_final;                       // used once, before the tensor memory is given back
  uint64_t x_ready[16];                     // normalised X chunk i % 16 may be read by the tensor cores
  uint64_t w_ready[16];                     // converted W chunk i % 16 (e4m3 weights) may be read by them
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

#ifdef VDC_TRACE_CHUNKS
// Life of a ring entry on SM 0: stamps 0 published by the control warp, 1 copy issued by the load port,
// 2 seen by the consuming warp, 3 slots given back.  Written behind the per-SM profile rows.
#define CHUNK_STAMP(c, n, k)                                                                               \
  if ((c).sm == 0 && (n) < 1500u) (c).profile[VDC_MAX_SMS * VDC_NUM_PROFILE_EVENTS + (n) * 4 + (k)] = globaltimer_ns()
#else
#define CHUNK_STAMP(c, n, k)
#endif

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
    else if (VDC_SPIN_SLEEP) __nanosleep(VDC_SPIN_SLEEP);
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
  // every poll is an acquire load: the one that reads zero pairs with the producers' releasing reds, and no
  // separate fence (one more trip to L2) stands between the open barrier and the first dependent access
  bool ok = wait_until(c, [&] { return ld_acquire_gpu(p) == 0; }, role, pc, opcode, bar, 0);
  fence_proxy_async();  // later bulk copies (async proxy) must observe what the releasing stores wrote
  return ok;
}
// The same wait for a consumer that reads the produced data with ordinary loads (no bulk copy follows).
__device__ __forceinline__ bool wait_global_barrier_generic(const Ctx& c, int bar, int role, int pc, int opcode) {
  const int* p = c.bars + bar;
  bool ok = wait_until(c, [&] { return ld_acquire_gpu(p) == 0; }, role, pc, opcode, bar, 0);
  return ok;
}
// Tensor-core helpers of the decode attention (legacy warp-level MMA: the problem is 4..8 query rows
// by 64 positions per page, far below the 128-row tiles of the tcgen05 path the batched projections use).
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}
// D(16x8, fp32) += A(16x16, bf16, rows 8..15 zero) * B(16x8, bf16).  Only rows 0..7 of A carry data:
// a_lo / a_hi are this thread's pairs (row lane/4, k = 2(lane%4) + {0,1}) and (same row, k + 8).
__device__ __forceinline__ void mma_rows8(float& d0, float& d1, float& z0, float& z1, uint32_t a_lo, uint32_t a_hi,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
               : "+f"(d0), "+f"(d1), "+f"(z0), "+f"(z1) : "r"(a_lo), "r"(0u), "r"(a_hi), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ldcg128(const void* p) {  // 16 bytes past L1: another SM wrote them
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldcg32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}


}  // namespace vdc
