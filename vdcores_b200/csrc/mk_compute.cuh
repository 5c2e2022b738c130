// Compute virtual core of the megakernel: queue access and the decode tasks.
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "mk_common.cuh"

namespace vdc {

#ifndef VDC_GEMV_VARIANT
#define VDC_GEMV_VARIANT 1   // 1: bf16 x bf16 + f32 mixed-precision FMA (no unpacking); 0: unpack to f32 pairs
#endif
#ifndef VDC_GEMV_UNROLL4
#define VDC_GEMV_UNROLL4 2
#endif

// Tasks are inlined into the kernel: measured on B200, the same GEMV loop behind a real function call
// (its queue state then lives in local memory, shared-memory accesses go through generic pointers)
// streams at 3.5 TB/s instead of 6.4 TB/s.
#define VDC_TASK __device__ __forceinline__

// ------------------------------------------------------------------------- //
// compute virtual core: queue access
// ------------------------------------------------------------------------- //
struct Compute {
  const Ctx& c;
  Shared* sh;
  int tid, warp, lane;
  unsigned head;     // ring entries consumed so far (uniform across the 256 threads)
  unsigned st_tail;  // store-queue pushes so far (thread 0)
  uint32_t pc;
  bool aborted;
  uint64_t stall;    // cycles thread 0 spent waiting for data
  unsigned mma_count;  // tensor-core commits issued so far (thread 0)
  unsigned xr_count;   // X chunks normalised by earlier tensor-core tasks (phase of the x_ready barriers)
  unsigned wr_count;   // W chunks converted by earlier tensor-core tasks (phase of the w_ready barriers)
  int batch = 0;       // size of the last pop_many
#ifdef VDC_TRACE_GEMV
  unsigned gemv_ord = 0;
#endif

  // CTA-wide pop: thread 0 waits for the entry (bounded), everybody gets its
  // word after one compute_sync.  Returns kPopAbort once a wait was given up.
  __device__ __forceinline__ int pop() {
    if (tid == 0) {
      const unsigned e = head % kQ;
      const uint32_t parity = (head / kQ) & 1u;
      uint64_t* bar = &sh->full[e];
      bool ok = mbar_try_wait(bar, parity);
      if (!ok) {
        const long long t0 = clock64();
        ok = wait_until(c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)pc, 0, -1, 0);
        stall += (uint64_t)(clock64() - t0);
      }
      sh->pop_val[head & 7u] = ok ? sh->ring_word[e] : kPopAbort;
      sh->pop_addr[head & 7u] = sh->ring[e].address;
      sh->pop_meta[head & 7u] = (uint32_t)sh->ring[e].opcode | ((uint32_t)sh->ring[e].num_slots << 16);
      sh->pop_size[head & 7u] = sh->ring[e].size;
      if (!ok) sh->aborted = 1;
      __threadfence_block();
      sh->cta_head = head + 1;
    }
    compute_sync();
    const int v = sh->pop_val[head & 7u];
    head++;
    if (v == kPopAbort) aborted = true;
    return v;
  }
  // The next n (<= 4) entries in one go: thread 0 waits for each, one CTA barrier publishes them all.  Entry j of
  // the batch is then read with val_at / addr_at / meta_at(j).  A task that takes several operands pays one
  // barrier instead of one per operand.
  __device__ __forceinline__ void pop_many(int n) {
    if (tid == 0) {
      for (int j = 0; j < n; ++j) {
        const unsigned idx = head + (unsigned)j, e = idx % kQ;
        const uint32_t parity = (idx / kQ) & 1u;
        uint64_t* bar = &sh->full[e];
        bool ok = mbar_try_wait(bar, parity);
        if (!ok) {
          const long long t0 = clock64();
          ok = wait_until(c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)pc, 0, -1, 0);
          stall += (uint64_t)(clock64() - t0);
        }
        sh->pop_val[idx & 7u] = ok ? sh->ring_word[e] : kPopAbort;
        sh->pop_addr[idx & 7u] = sh->ring[e].address;
        sh->pop_meta[idx & 7u] = (uint32_t)sh->ring[e].opcode | ((uint32_t)sh->ring[e].num_slots << 16);
        sh->pop_size[idx & 7u] = sh->ring[e].size;
        if (!ok) sh->aborted = 1;
      }
      __threadfence_block();
      sh->cta_head = head + (unsigned)n;
    }
    compute_sync();
    for (int j = 0; j < n; ++j)
      if (sh->pop_val[(head + (unsigned)j) & 7u] == kPopAbort) aborted = true;
    head += (unsigned)n;
    batch = n;
  }
  __device__ __forceinline__ int val_at(int j) const { return sh->pop_val[(head - (unsigned)batch + (unsigned)j) & 7u]; }
  __device__ __forceinline__ uint64_t addr_at(int j) const { return sh->pop_addr[(head - (unsigned)batch + (unsigned)j) & 7u]; }
  __device__ __forceinline__ uint32_t meta_at(int j) const { return sh->pop_meta[(head - (unsigned)batch + (unsigned)j) & 7u]; }
  // Address / (opcode | num_slots << 16) of the instruction behind the last pop.
  __device__ __forceinline__ uint64_t addr() const { return sh->pop_addr[(head - 1u) & 7u]; }
  __device__ __forceinline__ uint32_t meta() const { return sh->pop_meta[(head - 1u) & 7u]; }
  __device__ __forceinline__ uint32_t size() const { return sh->pop_size[(head - 1u) & 7u]; }
  // CTA-wide wait on a global barrier by the compute core itself (thread 0 polls; the data it
  // orders is then read with ordinary loads).  Returns false once a wait was given up.
  __device__ __forceinline__ bool wait_barrier(int bar, int opcode) {
    if (tid == 0 && !wait_global_barrier_generic(c, bar, 0, (int)pc, opcode)) sh->aborted = 1;
    compute_sync();
    if (sh->aborted) aborted = true;
    return !aborted;
  }

  // Per-warp phase: the next `n` ring entries are consumed by the warps on their own
  // schedule (the GEMV task gives entry head+i to the warp pair i % 4).  begin/end are CTA-wide.
  __device__ __forceinline__ void warp_phase_begin(unsigned n, unsigned first) {
    // first: index of the first entry this warp will consume
    if (lane == 0) sh->warp_next[warp] = first < n ? head + first : 0xFFFFFFFFu;
    compute_sync();
    if (tid == 0) sh->cta_head = head + n;
  }
  // Waits for entry head+i (whole warp); returns its word or kPopAbort.
  __device__ __forceinline__ int warp_wait(unsigned i) {
    const unsigned idx = head + i;
    uint64_t* bar = &sh->full[idx % kQ];
    const uint32_t parity = (idx / kQ) & 1u;
    int ok = 1;
    if (lane == 0) {
      if (!mbar_try_wait(bar, parity)) {
        ok = wait_until(c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)pc, 0, -1, 0);
        if (!ok) sh->aborted = 1;
      }
      if (sh->aborted) ok = 0;  // another warp of this CTA gave up: stop consuming
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    // lanes other than 0 did not observe the barrier themselves: order their
    // reads after lane 0's acquire
    __syncwarp();
    return ok ? sh->ring_word[idx % kQ] : kPopAbort;
  }
  // Entry head+i is finished: free its slots and publish this warp's next entry.
  __device__ __forceinline__ void warp_done(unsigned i, unsigned n, int mask) {
    __syncwarp();
    if (lane == 0) {
      if (mask > 0) atomicOr(&sh->slot_avail, (uint32_t)mask & kSlotMaskAll);
      sh->warp_next[warp] = i + kCW < n ? head + i + kCW : 0xFFFFFFFFu;
    }
  }
  __device__ __forceinline__ void warp_phase_end(unsigned n) {
    compute_sync();
    head += n;
    if (sh->aborted) aborted = true;
  }

  // Counts down the global barrier named by a popped raw-address instruction
  // that carries BARRIER|WRITEBACK.  Caller guarantees every writer executed
  // __threadfence() and a compute_sync() since its last global write.
  __device__ __forceinline__ void release(uint32_t m) {
    // red.release.gpu is cumulative: it orders this thread's earlier writes and
    // those it observed through the CTA barrier, so no separate fence is needed
    if (tid == 0 && (m & VDC_F_BARRIER) && (m & VDC_F_WRITEBACK)) red_release_gpu_add(c.bars + (m >> 22), -1);
  }
  // The same count-down for a task whose every writing thread ran __threadfence() after its last global
  // write and then met thread 0 at a CTA barrier: the writes are performed at gpu scope before the barrier
  // lets thread 0 through, so the count-down itself carries no fence of its own (a fence here costs one more
  // trip to L2 on the path every consumer SM is waiting on).
  __device__ __forceinline__ void release_prefenced(uint32_t m) {
#ifdef VDC_STRICT_RELEASE
    release(m);
#else
    if (tid == 0 && (m & VDC_F_BARRIER) && (m & VDC_F_WRITEBACK)) red_relaxed_gpu_add(c.bars + (m >> 22), -1);
#endif
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
// Pop order: [norm weight], x, out (raw address), [argmax record (raw address)],
// then n_chunks weight chunks of R rows x K bf16 (row-major, contiguous).
// Operands are popped CTA-wide; the chunks are consumed by the eight warps
// independently (chunk i by warp i % 8), each warp doing the whole dot products
// of its chunk, so the streaming loop has no CTA-wide synchronisation.
struct ArgBest {
  float val;
  int idx;
};

__device__ __forceinline__ float2 bf2(uint32_t u) { return make_float2(bf_lo(u), bf_hi(u)); }

// One warp's dot products for a chunk of R rows, with packed fp32 FMAs.  Each
// row keeps NA independent partial sums so the FMA chains stay short when R is
// small (a single 28 KB row would otherwise be one long dependent chain).
template <int R>
__device__ __forceinline__ void gemv_chunk(const uint8_t* w, const uint8_t* x, int K, int lane, int it0, int it1,
                                           float (&out)[R]) {
  constexpr int NA = R >= 8 ? 1 : (R == 4 ? 2 : 4);
  constexpr int UNROLL = R >= 8 ? 1 : (R == 4 ? VDC_GEMV_UNROLL4 : 4);
  float2 acc[R][NA];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int a = 0; a < NA; ++a) acc[r][a] = make_float2(0.f, 0.f);
#pragma unroll UNROLL
  for (int it = it0; it < it1; ++it) {
    const int off = (it << 9) + (lane << 4);  // byte offset of this lane's 8 elements
    const uint4 xv = lds128(x + off);
    const float2 xf[4] = {bf2(xv.x), bf2(xv.y), bf2(xv.z), bf2(xv.w)};
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint4 wv = lds128(w + (size_t)r * K * 2 + off);
      acc[r][0 % NA] = __ffma2_rn(bf2(wv.x), xf[0], acc[r][0 % NA]);
      acc[r][1 % NA] = __ffma2_rn(bf2(wv.y), xf[1], acc[r][1 % NA]);
      acc[r][2 % NA] = __ffma2_rn(bf2(wv.z), xf[2], acc[r][2 % NA]);
      acc[r][3 % NA] = __ffma2_rn(bf2(wv.w), xf[3], acc[r][3 % NA]);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v = acc[r][0].x + acc[r][0].y;
#pragma unroll
    for (int a = 1; a < NA; ++a) v += acc[r][a].x + acc[r][a].y;
    out[r] = warp_sum(v);
  }
}

// Mixed-precision FMA of sm_100: d(f32) = a(bf16) * b(bf16) + c(f32), one rounding; the bf16 pairs are used
// as they come out of shared memory, nothing is converted.
__device__ __forceinline__ void fma_bf16x2(float& lo, float& hi, uint32_t w, uint32_t x) {
  asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %2;\n\t"
      "mov.b32 {xl, xh}, %3;\n\t"
      "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.bf16 %1, wh, xh, %1;\n\t}"
      : "+f"(lo), "+f"(hi)
      : "r"(w), "r"(x));
}
#if VDC_GEMV_VARIANT >= 1
template <int R>
__device__ __forceinline__ void gemv_chunk_mixed(const uint8_t* w, const uint8_t* x, int K, int lane, int it0, int it1,
                                                 float (&out)[R]) {
  constexpr int NA = R >= 8 ? 1 : (R == 4 ? 2 : 4);
  constexpr int UNROLL = R >= 8 ? 1 : (R == 4 ? VDC_GEMV_UNROLL4 : 4);
  float lo[R][NA], hi[R][NA];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int a = 0; a < NA; ++a) lo[r][a] = hi[r][a] = 0.f;
#pragma unroll UNROLL
  for (int it = it0; it < it1; ++it) {
    const int off = (it << 9) + (lane << 4);
    const uint4 xv = lds128(x + off);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint4 wv = lds128(w + (size_t)r * K * 2 + off);
      fma_bf16x2(lo[r][0 % NA], hi[r][0 % NA], wv.x, xv.x);
      fma_bf16x2(lo[r][1 % NA], hi[r][1 % NA], wv.y, xv.y);
      fma_bf16x2(lo[r][2 % NA], hi[r][2 % NA], wv.z, xv.z);
      fma_bf16x2(lo[r][3 % NA], hi[r][3 % NA], wv.w, xv.w);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v = lo[r][0] + hi[r][0];
#pragma unroll
    for (int a = 1; a < NA; ++a) v += lo[r][a] + hi[r][a];
    out[r] = warp_sum(v);
  }
}
#endif

// Same for e4m3 weights (one byte each, per-row fp32 scale applied by the caller).  The activation
// vector has been converted to fp16 in place (exact for normalised activations); 16 weights per lane and
// step become fp16 pairs with one conversion per pair and go straight into the mixed-precision FMA
// d(f32) = a(f16) * b(f16) + c(f32): half a conversion and one FMA per weight, nothing is widened.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t pair16) {   // widened pair (batched path's conversion)
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)pair16, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t pair16) {
  uint32_t d;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"((unsigned short)pair16));
  return d;
}
__device__ __forceinline__ void fma_f16x2(float& lo, float& hi, uint32_t w, uint32_t x) {
  asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %2;\n\t"
      "mov.b32 {xl, xh}, %3;\n\t"
      "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.f16 %1, wh, xh, %1;\n\t}"
      : "+f"(lo), "+f"(hi)
      : "r"(w), "r"(x));
}

template <int R>
__device__ __forceinline__ void gemv_chunk_fp8_rows(const uint8_t* w, const uint8_t* x16, int K, int lane, int it0, int it1,
                                                    float (&out)[R]) {
  constexpr int NA = R >= 8 ? 1 : (R == 4 ? 2 : 4);
  float lo[R][NA], hi[R][NA];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int a = 0; a < NA; ++a) lo[r][a] = hi[r][a] = 0.f;
#pragma unroll 1
  for (int it = it0; it < it1; ++it) {  // 512 weights per warp step
    const int e0 = (it << 9) + (lane << 4);  // first element of this lane
    const uint4 xa = lds128(x16 + e0 * 2), xb = lds128(x16 + e0 * 2 + 16);
    const uint32_t xx[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint4 wv = lds128(w + (size_t)r * K + e0);
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        fma_f16x2(lo[r][(2 * j) % NA], hi[r][(2 * j) % NA], e4m3x2_to_f16x2(ww[j] & 0xFFFFu), xx[2 * j]);
        fma_f16x2(lo[r][(2 * j + 1) % NA], hi[r][(2 * j + 1) % NA], e4m3x2_to_f16x2(ww[j] >> 16), xx[2 * j + 1]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v = lo[r][0] + hi[r][0];
#pragma unroll
    for (int a = 1; a < NA; ++a) v += lo[r][a] + hi[r][a];
    out[r] = warp_sum(v);
  }
}

// Option: a chunk of more than VDC_QROWS rows is walked in groups of VDC_QROWS rows, one pass over K per
// group (a smaller unrolled body).  Measured on B200 with groups of 2, 4 and no grouping: no difference for
// e4m3 and NVFP4 rows (the stream is bound by the chunks' lifetime in the slots, not by the loop), so off.
#ifndef VDC_QROWS
#define VDC_QROWS 16
#endif
template <int R>
__device__ __forceinline__ void gemv_chunk_fp8(const uint8_t* w, const uint8_t* x16, int K, int lane, int it0, int it1,
                                               float (&out)[R]) {
  if constexpr (R <= VDC_QROWS) {
    gemv_chunk_fp8_rows<R>(w, x16, K, lane, it0, it1, out);
  } else {
#pragma unroll 1
    for (int g = 0; g < R / VDC_QROWS; ++g) {
      float part[VDC_QROWS];
      gemv_chunk_fp8_rows<VDC_QROWS>(w + (size_t)g * VDC_QROWS * K, x16, K, lane, it0, it1, part);
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r / VDC_QROWS == g) out[r] = part[r % VDC_QROWS];
    }
  }
}

// NVFP4 rows: K/2 bytes of e2m1 pairs (element 2i in the low nibble) followed by
// K/16 e4m3 block scales, one per 16 weights.  The activation vector has been
// converted to fp16 in place.  Each lane takes 32 weights (two blocks) per step:
// the 16 products of a block are accumulated with half2 FMAs, the block sum is
// widened, multiplied by the block scale and accumulated in fp32.  The per-row
// fp32 scale (the tensor scale) is applied by the caller.
__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
  const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
  return *reinterpret_cast<const __half2*>(&h);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

template <int R>
__device__ __forceinline__ void gemv_chunk_nvfp4_rows(const uint8_t* w, const uint8_t* x16, int K, int lane, int it0,
                                                      int it1, float (&out)[R]) {
  const int row_bytes = (K >> 1) + (K >> 4);
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  for (int it = it0; it < it1; ++it) {  // 1024 weights per warp step
    const int e0 = (it << 10) + (lane << 5);  // first element of this lane
    uint4 xv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) xv[j] = lds128(x16 + e0 * 2 + 16 * j);
    const __half2* xh = reinterpret_cast<const __half2*>(xv);  // 16 half2 = 32 activations
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint8_t* row = w + (size_t)r * row_bytes;
      const uint4 cv = lds128(row + (e0 >> 1));
      const uint32_t sc2 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(row + (K >> 1) + (e0 >> 4)));  // two block scales
      const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
      uint32_t bs[2];   // the two block sums, fp16 pairs
#pragma unroll
      for (int b = 0; b < 2; ++b) {  // two blocks of 16 weights = 8 bytes each
        __half2 s0 = __float2half2_rn(0.f), s1 = s0;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const uint32_t word = cw[b * 2 + (j >> 2)];
          s0 = __hfma2(e2m1x2_to_half2((word >> (8 * (j & 3))) & 0xFFu), xh[b * 8 + j], s0);
          s1 = __hfma2(e2m1x2_to_half2((word >> (8 * ((j + 1) & 3))) & 0xFFu), xh[b * 8 + j + 1], s1);
        }
        const __half2 t = __hadd2(s0, s1);
        bs[b] = *reinterpret_cast<const uint32_t*>(&t);
      }
      // acc += (lo + hi of block b) * scale_b: the scale pair is {scale_0, scale_1}; two mixed FMAs per block
      {
        const uint32_t s00 = __byte_perm(sc2, 0, 0x1010), s11 = __byte_perm(sc2, 0, 0x3232);
        float a0 = 0.f, a1 = 0.f;
        fma_f16x2(a0, a1, bs[0], s00);
        fma_f16x2(a0, a1, bs[1], s11);
        acc[r] += a0 + a1;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) out[r] = warp_sum(acc[r]);
}

template <int R>
__device__ __forceinline__ void gemv_chunk_nvfp4(const uint8_t* w, const uint8_t* x16, int K, int lane, int it0,
                                                 int it1, float (&out)[R]) {
  if constexpr (R <= VDC_QROWS) {
    gemv_chunk_nvfp4_rows<R>(w, x16, K, lane, it0, it1, out);
  } else {
    const int row_bytes = (K >> 1) + (K >> 4);
#pragma unroll 1
    for (int g = 0; g < R / VDC_QROWS; ++g) {
      float part[VDC_QROWS];
      gemv_chunk_nvfp4_rows<VDC_QROWS>(w + (size_t)g * VDC_QROWS * row_bytes, x16, K, lane, it0, it1, part);
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r / VDC_QROWS == g) out[r] = part[r % VDC_QROWS];
    }
  }
}

// wfmt: 0 bf16, 1 e4m3 (scales = fp32 per-row scales of the task's rows), 2 NVFP4 (scales likewise).
struct MoeDown {           // mode MOE_DOWN: per-row accumulation over the selected experts
  const float* weight;     // this expert's routing weight
  float* acc;              // fp32 accumulators of the task's rows
  int* cnt;                // arrival counters of the task's rows
  int top_k;
};

// Tensor parallel without a collective library: the exchange blocks of all ranks are mapped into
// this process; a task writes its fp32 partial rows into its own slot of every rank's block with
// tagged 8-byte peer stores ({fp32 bits, exchange tag}); the consumers poll the entries themselves.
struct PeerOut {
  const unsigned long long* table;  // base address of each rank's exchange block; entry [n] is the state block
  int n;                            // ranks
  uint32_t ex;                      // exchange number | exchanges per step << 16
};
// The tag of exchange number (ex & 0xFFFF) in the current step: unique over a run, never zero (a zeroed
// exchange block matches nothing).
__device__ __forceinline__ uint32_t exchange_tag(const int* state, uint32_t ex) {
  return (uint32_t)ld_relaxed_gpu(state + VDC_ST_STEP) * (ex >> 16) + (ex & 0xFFFFu) + 1u;
}

template <int R>
VDC_TASK void task_gemv_rows(Compute& q, int n_chunks, int mode, bool accumulate, bool norm, int K, int row_base,
                               const float* scales = nullptr, int wfmt = 0, const MoeDown* moe = nullptr,
                               bool dyn = false, const PeerOut* peers = nullptr, uint64_t dyn_base = 0,
                               const float* partial = nullptr, int chunk_stride = 1) {
  Shared* sh = q.sh;
  const Ctx& c = q.c;
#ifdef VDC_TRACE_GEMV
  // eight stamps for each of the GEMV tasks 4..11 of this SM (layers 1 and 2 of a dense model)
  const unsigned g_ord = q.gemv_ord++;
#define GEMV_STAMP(i)                                                                         \
  if (q.tid == 0 && g_ord >= 4 && g_ord < 12)                                                  \
  c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 64 + (g_ord - 4) * 8 + (i)] = globaltimer_ns()
#else
#define GEMV_STAMP(i)
#endif
  GEMV_STAMP(0);
  // operands: [norm weights], activation vector, output (raw address), [argmax record (raw address)]
  q.pop_many((norm ? 1 : 0) + 2 + (mode == VDC_GEMV_MODE_ARGMAX ? 1 : 0));
  int k_op = 0;
  int normw_mask = 0;
  if (norm) normw_mask = q.val_at(k_op++);
  const int x_mask = q.val_at(k_op);
  const uint32_t x_meta = q.meta_at(k_op);
  const uint64_t x_addr = q.addr_at(k_op);
  ++k_op;
  __nv_bfloat16* outg = reinterpret_cast<__nv_bfloat16*>(q.addr_at(k_op));
  const uint32_t out_meta = q.meta_at(k_op);
  ++k_op;
  float* recg = nullptr;
  uint32_t rec_meta = 0;
  if (mode == VDC_GEMV_MODE_ARGMAX) {
    recg = reinterpret_cast<float*>(q.addr_at(k_op));
    rec_meta = q.meta_at(k_op);
  }
  if (dyn) {
    // the count word was written by another SM; this hand-over was published only after the
    // barrier that orders it had opened
    q.pop();
    if (q.aborted) return;
    const int lim = ld_relaxed_gpu(reinterpret_cast<const int*>(q.addr()));
    n_chunks = min(n_chunks, max(lim, 0));
  }
  if (q.aborted) return;
  uint8_t* x = (uint8_t*)slot_ptr(c, first_slot(x_mask));

  float ss = 0.f;
  if (((x_meta & 0xFFFFu) >> VDC_FLAG_BITS) == 32u) {
    // XVEC hand-over: the slots are empty.  Wait for the producers' barrier here, then every
    // thread copies its share of the vector from global memory (past L1) into the slots.
    GEMV_STAMP(1);
    if ((x_meta & VDC_F_BARRIER) && !q.wait_barrier((int)(x_meta >> 22), 0x7200)) return;
    GEMV_STAMP(2);
    const uint8_t* xg = reinterpret_cast<const uint8_t*>(x_addr);
    // up to eight loads per thread are in flight before the first one is used
    for (int i0 = q.tid * 8; i0 < K; i0 += kCT * 8 * 8) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * kCT * 8;
        v[j] = i < K ? ldcg128(xg + i * 2) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * kCT * 8;
        if (i < K) {
          *reinterpret_cast<uint4*>(x + i * 2) = v[j];
          if (norm) {
            const float f[8] = {bf_lo(v[j].x), bf_hi(v[j].x), bf_lo(v[j].y), bf_hi(v[j].y),
                                bf_lo(v[j].z), bf_hi(v[j].z), bf_lo(v[j].w), bf_hi(v[j].w)};
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
          }
        }
      }
    }
  } else if (norm) {
    for (int i = q.tid * 8; i < K; i += kCT * 8) {
      const uint4 v = lds128(x + i * 2);
      const float f[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
  }
  if (norm) {
    // RMSNorm of the activation vector in place: bf16(w * bf16(x * rstd)), fp32 statistics
    const uint8_t* nw = (const uint8_t*)slot_ptr(c, first_slot(normw_mask));
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
    // the sync inside warp_phase_begin publishes the normalised vector
  }
  if (wfmt != 0) {
    // e4m3 weights meet the activations in the mixed fp16 FMA, NVFP4 block dots run in half precision: the
    // activation vector becomes fp16 in place
    compute_sync();  // the vector was written (copied or normalised) by other threads
    for (int i = q.tid * 2; i < K; i += kCT * 2) {
      const uint32_t xv = *reinterpret_cast<const uint32_t*>(x + i * 2);
      const __half2 h = __floats2half2_rn(bf_lo(xv), bf_hi(xv));
      *reinterpret_cast<__half2*>(x + i * 2) = h;
    }
  }

  ArgBest best = {-INFINITY, 0x7fffffff};
  const uint32_t peer_tag =
      peers != nullptr ? exchange_tag(reinterpret_cast<const int*>(__ldg(peers->table + peers->n)), peers->ex) : 0u;
  // Chunk i belongs to the pair of warps (i % 4, i % 4 + 4): each member takes one half of K
  // for all R rows, the halves meet in shared memory at a two-warp named barrier, and the
  // lower warp finishes the chunk.  A chunk therefore stays resident for half the time one
  // warp alone would need, which is what the in-flight window of 24 slots can afford.
  const int pair = q.warp & 3, member = q.warp >> 2;
  const int steps = wfmt == 2 ? K >> 10 : (wfmt == 1 ? K >> 9 : K >> 8);
  const int it0 = member == 0 ? 0 : (steps + 1) / 2, it1 = member == 0 ? (steps + 1) / 2 : steps;
  float* pair_part = sh->red + pair * (2 * 2 * 16);  // [buffer][member][row]
  GEMV_STAMP(3);
  const bool dyn_rows = dyn_base != 0;
  // (chunks drawn from the shared counter: their number is only known at the end marker)
  q.warp_phase_begin(dyn_rows ? 0x10000000u : (unsigned)n_chunks, (unsigned)pair);  // its sync also publishes the vector
  GEMV_STAMP(4);
  if (norm) q.free_slots(normw_mask);
  if (dyn_rows) n_chunks = 0x0FFFFFFF;
  for (int i = pair, trip = 0; i < n_chunks; i += 4, ++trip) {
    const int w_mask = q.warp_wait((unsigned)i);
    if (q.lane == 0 && member == 0) CHUNK_STAMP(c, q.head + (unsigned)i, 2);
    if (w_mask == VDC_STREAM_END) {  // both members of the pair read the same entry: they leave together
      // the k-th of the four consecutive markers sits k entries behind the last chunk of the phase
      n_chunks = i - (int)(sh->ring[(q.head + (unsigned)i) % kQ].address >> 32);
      break;
    }
    const bool arrived = w_mask != kPopAbort;
    float acc[R];
    int row0 = i * R * chunk_stride;
    if (dyn_rows && arrived) {
      const uint32_t chunk_bytes = (uint32_t)R * (uint32_t)(wfmt == 2 ? (K >> 1) + (K >> 4) : (wfmt == 1 ? K : 2 * K));
      row0 = (int)((sh->ring[(q.head + (unsigned)i) % kQ].address - dyn_base) / chunk_bytes) * R;
    }
    if (arrived) {
      const uint8_t* w = (const uint8_t*)slot_ptr(c, first_slot(w_mask));
      if (wfmt == 2) gemv_chunk_nvfp4<R>(w, x, K, q.lane, it0, it1, acc);
      else if (wfmt == 1) gemv_chunk_fp8<R>(w, x, K, q.lane, it0, it1, acc);
#if VDC_GEMV_VARIANT >= 1
      else gemv_chunk_mixed<R>(w, x, K, q.lane, it0, it1, acc);
#else
      else gemv_chunk<R>(w, x, K, q.lane, it0, it1, acc);
#endif
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
    }
    float* pp = pair_part + (trip & 1) * 32;
    if (member == 1) {
      float v = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (q.lane == r) v = acc[r];
      if (q.lane < R) pp[16 + q.lane] = v;
    }
    // Both members always meet at the pair's barrier and decide together whether to go on: a
    // member whose wait was given up must not leave its partner alone at a later barrier.
    if (q.lane == 0) sh->pair_ok[pair][trip & 1][member] = arrived ? 1 : 0;
    asm volatile("bar.sync %0, 64;" ::"r"(2 + pair) : "memory");
    if (!(sh->pair_ok[pair][trip & 1][0] && sh->pair_ok[pair][trip & 1][1])) break;
    if (member == 1) {  // the partner finishes the chunk; it also frees the slots
      if (q.lane == 0) sh->warp_next[q.warp] = i + 4 < n_chunks ? q.head + i + 4 : 0xFFFFFFFFu;
      continue;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] += pp[16 + r];
    if (wfmt != 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] *= __ldg(scales + row0 + r);
    }
    if (partial != nullptr) {   // the rows' sums over the other K-range, left by an earlier task of this SM
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] += __ldcg(partial + row0 + r);
    }
    __syncwarp();
    if (q.lane == 0) {
      atomicOr(&sh->slot_avail, (uint32_t)w_mask & kSlotMaskAll);
      sh->warp_next[q.warp] = i + 4 < n_chunks ? q.head + i + 4 : 0xFFFFFFFFu;
      CHUNK_STAMP(c, q.head + (unsigned)i, 3);
    }
    if (mode == VDC_GEMV_MODE_SILU_PAIRS) {
      float g = 0.f, u = 0.f;
#pragma unroll
      for (int j = 0; j < R / 2; ++j)
        if (q.lane == j) {
          g = acc[2 * j];
          u = acc[2 * j + 1];
        }
      if (q.lane < R / 2) {
        g = bf16_round(g);
        u = bf16_round(u);
        const float sg = bf16_round(g / (1.f + __expf(-g)));
        outg[row0 / 2 + q.lane] = __float2bfloat16_rn(sg * u);
      }
    } else {
      float v = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (q.lane == r) v = acc[r];
      if (q.lane < R && mode == VDC_GEMV_MODE_STORE_F32 && peers != nullptr) {
        // `outg` is the byte offset of the task's first row entry inside an exchange block
        const unsigned long long off = reinterpret_cast<unsigned long long>(outg) + (unsigned long long)(row0 + q.lane) * 8ull;
        for (int pr = 0; pr < peers->n; ++pr) st_tagged_sys(__ldg(peers->table + pr) + off, __float_as_uint(v), peer_tag);
      } else if (q.lane < R && mode == VDC_GEMV_MODE_STORE_F32) {
        reinterpret_cast<float*>(outg)[row0 + q.lane] = v;
      } else if (q.lane < R && mode == VDC_GEMV_MODE_MOE_DOWN && moe->acc == nullptr) {
        // expert parallel: this rank's share of the weighted sum, fp32, all-reduced by the host side
        atomicAdd(reinterpret_cast<float*>(outg) + row0 + q.lane, ld_relaxed_gpu_f32(moe->weight) * bf16_round(v));
      } else if (q.lane < R && mode == VDC_GEMV_MODE_MOE_DOWN) {
        const int row = row0 + q.lane;
        atomicAdd(moe->acc + row, ld_relaxed_gpu_f32(moe->weight) * bf16_round(v));  // rewritten every layer: no read-only path
        __threadfence();
        if (atomicAdd(moe->cnt + row, 1) == moe->top_k - 1) {
          // every selected expert has added its share: fold the sum into the residual stream
          __threadfence();
          const float total = atomicExch(moe->acc + row, 0.f);
          moe->cnt[row] = 0;
          outg[row] = __float2bfloat16_rn(__bfloat162float(outg[row]) + bf16_round(total));
        }
      } else if (q.lane < R) {
        const __nv_bfloat16 bq = __float2bfloat16_rn(v);
        if (accumulate) atomicAdd(outg + row0 + q.lane, bq);  // residual add: bf16(old + bf16(W x))
        else outg[row0 + q.lane] = bq;
        if (mode == VDC_GEMV_MODE_ARGMAX) {
          const float bv = __bfloat162float(bq);
          if (bv > best.val || (bv == best.val && row0 + q.lane < best.idx)) {
            best.val = bv;
            best.idx = row0 + q.lane;
          }
        }
      }
    }
  }
  if (mode == VDC_GEMV_MODE_ARGMAX) {
    // candidates sit in lanes 0..R-1 of every warp; the lowest row index wins ties
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
      sh->misc[40 + q.warp] = best.val;
      reinterpret_cast<int*>(sh->misc)[48 + q.warp] = best.idx;
    }
  }
  GEMV_STAMP(5);
  // Output rows were written by the lower warp of every pair.  Each of them drains its own global writes
  // here, while the other warps still compute; the CTA barrier inside warp_phase_end then lets thread 0
  // count the barrier down without a fence of its own (release_prefenced).
  if (member == 0 && (out_meta & VDC_F_BARRIER)) __threadfence();
  if (dyn_rows) {
    // every pair has met its end marker and knows the chunk count; the ring moves on past the four markers
    if (q.lane == 0) sh->warp_next[q.warp] = 0xFFFFFFFFu;
    compute_sync();
    if (q.tid == 0) sh->cta_head = q.head + (unsigned)n_chunks + 4u;
    q.warp_phase_end((unsigned)n_chunks + 4u);
  } else {
    q.warp_phase_end((unsigned)n_chunks);
  }
  GEMV_STAMP(6);
  if (q.aborted) return;
  if (mode == VDC_GEMV_MODE_ARGMAX && q.tid == 0) {
    float bv = sh->misc[40];
    int bi = reinterpret_cast<int*>(sh->misc)[48];
    for (int w = 1; w < kCW; ++w) {
      const float ov = sh->misc[40 + w];
      const int oi = reinterpret_cast<int*>(sh->misc)[48 + w];
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    recg[0] = bv;
    reinterpret_cast<int*>(recg)[1] = bi + row_base;
    recg[2] = 0.f;
    recg[3] = 0.f;
  }
  q.release_prefenced(out_meta);   // every writing warp fenced before warp_phase_end
  q.release(rec_meta);
  q.free_slots(x_mask);
  GEMV_STAMP(7);
}

// ------------------------------------------------------------------------- //
// task: split-K GQA decode attention over 64-position KV pages, merge included
// ------------------------------------------------------------------------- //
// One task handles one KV head and one split (a range of pages) of the cache.
// The memory stream delivers only the pages: `count` x (K page, V page) with
// count = clamp(n_pages - base, 0, max_pages) read from the state block (the
// memory stream applies the same rule through DYN_COUNT + REPEAT).  Everything
// else travels in the instruction words and is read with ordinary loads: the
// state block, the rope table, the q/k norm weights, the head group's
// projection output (G query heads, the new key row, the new value row:
// (G+2) x 128 bf16, contiguous) behind the barrier the task waits for itself,
// this head's K / V pages (for the new cache rows), the head's split records,
// its arrival counter, its slice of the attention output, and the barrier the
// merged output releases.
//
// The page loop has no CTA-wide synchronisation: the eight warps share the 64
// positions of a page (G = 4: eight each; G = 8: the warps form two groups of
// four query heads, sixteen positions each), every warp waits for the page
// entries itself, keeps its own online-softmax state (scores and probabilities
// never leave registers; exp2 domain) and its own partial output, and the warp
// that finishes a page last gives its slots back.  The warps' states meet once,
// in shared memory, after the last page.
//
// Each task leaves {G x 128 fp32 unnormalised O, m[G], l[G]} in its record and
// bumps the head's counter; the task that arrives last merges all records
// (O = sum_s 2^(m_s-m) O_s / sum_s 2^(m_s-m) l_s), writes the bf16 output,
// resets the counter and counts the barrier down.
#ifdef VDC_TRACE_ATTN
#define ATTN_STAMP(i) if (q.tid == 0) c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 100 + (i)] = globaltimer_ns()
#else
#define ATTN_STAMP(i)
#endif

struct AttnArgs {
  int max_pages, base_page, flags;
  float qk_eps;
  int n_splits, split, bar;
  const int* state;
  uint8_t* k_rows;   // this head's rows inside K page 0 of the layer (new row = + NEWROW * 256)
  uint8_t* v_rows;
  float* records;    // [n_splits][rec_floats] of this head
  int* counter;
  __nv_bfloat16* out;  // G*128 outputs of this head
  int b, bpad;         // bpad != 0: `out` is this head's first k group in a k-chunk-major [bpad, *] matrix, row b
  const float* rope;           // table [position][cos 64 | sin 64] fp32
  const __nv_bfloat16* nw;     // q norm | k norm weights (2 x 128), or null
  const __nv_bfloat16* qkv;    // the head group's projection output
  int wait_bar;                // barrier that orders qkv (0xFFFF: none)
  int state_stride, qkv_stride;  // pair units: int32 words to the second position's state block, elements to its row
};

// kPair (chunked prefill, models with four query heads per KV head): the unit serves TWO consecutive prompt
// positions of one KV head.  Rows 0..3 of the MMA tile are the first position's query heads, rows 4..7 the
// second's (the tile has eight usable rows either way); both walk the same pages, each row masks the page rows
// past its own position, and all cache rows, the two positions' own included, are in HBM already (the chunk's
// cache-append stage ran first), so nothing is patched in from shared memory and nothing is written back.
template <int G, bool kPair = false, bool kTwo = false>
VDC_TASK void task_attn_decode(Compute& q, const AttnArgs& a) {
  constexpr int D = VDC_HEAD_DIM;
  constexpr int GQ = kPair ? G / 2 : G;      // query heads per position
  constexpr int PPW = VDC_KV_PAGE / kCW;     // positions of a page per warp: one 8-column MMA tile
  static_assert(PPW == 8 && D == 128 && G <= 8, "the page loop maps one MMA tile of 8 positions to each warp");
  constexpr int REC = G * D + 16 * ((2 * G + 15) / 16);
  Shared* sh = q.sh;
  const Ctx& c = q.c;
  const bool qk_norm = a.flags & VDC_ATTN_QKNORM_BIT;

  ATTN_STAMP(0);
  if (q.tid < 8) sh->att_done[q.tid] = 0;
  if (q.tid >= 32 && q.tid < 48) sh->zero_row[q.tid - 32] = make_uint4(0u, 0u, 0u, 0u);
  if (a.wait_bar != 0xFFFF && !q.wait_barrier(a.wait_bar, 0x7210)) return;
  ATTN_STAMP(1);

  const int pos = ld_relaxed_gpu(a.state + VDC_ST_POS);
  const int n_pages = ld_relaxed_gpu(a.state + VDC_ST_NPAGES);
  int count = n_pages - a.base_page;
  count = count < 0 ? 0 : (count > a.max_pages ? a.max_pages : count);
  const bool owner = count > 0 && a.base_page + count == n_pages;
  const int tail_valid = (pos % VDC_KV_PAGE) + 1;  // valid rows of the last page, new row included
  // pair units: the second position (the first one again in a prompt's ragged tail) lies in the same page
  const int pos_b = kPair ? ld_relaxed_gpu(a.state + a.state_stride + VDC_ST_POS) : pos;
  const int tail_valid_b = (pos_b % VDC_KV_PAGE) + 1;
  const int sw_new = pos & 7;                      // piece swizzle of the new row (its row index mod 8)

  const __nv_bfloat16* knew = a.qkv + G * D;
  const __nv_bfloat16* vnew = knew + D;
  __nv_bfloat16* krow = reinterpret_cast<__nv_bfloat16*>(sh->newrows);  // rotated new key row
  __nv_bfloat16* vrow = krow + D;
  const float scale_log2 = 1.4426950408889634f * rsqrtf((float)D);

  // --- prologue: optional per-head RMSNorm, then half-rotation RoPE.  One warp
  // per head: heads 0..G-1 are the queries, "head" G is the new key row.
  for (int head = q.warp; head <= (kPair ? G - 1 : G); head += kCW) {
    const bool is_k = !kPair && head == G;
    const bool second = kPair && head >= GQ;
    const __nv_bfloat16* src = is_k ? knew : (second ? a.qkv + a.qkv_stride + (head - GQ) * D : a.qkv + head * D);
    const float* rope = second ? a.rope + (size_t)pos_b * D : a.rope + (size_t)pos * D;
    const int i0 = q.lane * 2;  // pairs (i0, i0+64), (i0+1, i0+65)
    const uint32_t lo = ldcg32(src + i0), hi = ldcg32(src + i0 + 64);
    float a0 = bf_lo(lo), a1 = bf_hi(lo), b0 = bf_lo(hi), b1 = bf_hi(hi);
    if (qk_norm) {
      float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
      const float rstd = rsqrtf(ss / (float)D + a.qk_eps);
      const __nv_bfloat16* w = a.nw + (is_k ? D : 0);
      a0 = bf16_round(__bfloat162float(w[i0]) * bf16_round(a0 * rstd));
      a1 = bf16_round(__bfloat162float(w[i0 + 1]) * bf16_round(a1 * rstd));
      b0 = bf16_round(__bfloat162float(w[i0 + 64]) * bf16_round(b0 * rstd));
      b1 = bf16_round(__bfloat162float(w[i0 + 65]) * bf16_round(b1 * rstd));
    }
    const float2 cs = __ldg(reinterpret_cast<const float2*>(rope + i0));
    const float2 sn = __ldg(reinterpret_cast<const float2*>(rope + 64 + i0));
    // x*cos + rotate_half(x)*sin with every product and the sum rounded to bf16,
    // the way a bf16 tensor expression evaluates it
    const float r0 = bf16_round(bf16_round(a0 * cs.x) - bf16_round(b0 * sn.x));
    const float r1 = bf16_round(bf16_round(a1 * cs.y) - bf16_round(b1 * sn.y));
    const float r64 = bf16_round(bf16_round(b0 * cs.x) + bf16_round(a0 * sn.x));
    const float r65 = bf16_round(bf16_round(b1 * cs.y) + bf16_round(a1 * sn.y));
    // the key row takes the piece order of its row inside the page; query rows stay linear
    uint32_t* dst = reinterpret_cast<uint32_t*>(is_k ? krow : sh->qbf + head * D);
    const int sw = is_k ? sw_new : 0;
    const int e_lo = (((i0 >> 3) ^ sw) << 3) | (i0 & 7), e_hi = ((((i0 + 64) >> 3) ^ sw) << 3) | (i0 & 7);
    dst[e_lo >> 1] = pack_bf16x2(r0, r1);
    dst[e_hi >> 1] = pack_bf16x2(r64, r65);
  }
  if (!kPair && q.tid >= kCT - D / 8) {
    const int t = q.tid - (kCT - D / 8);
    reinterpret_cast<uint4*>(vrow)[t ^ sw_new] = ldcg128(reinterpret_cast<const uint4*>(vnew) + t);
  }
  if (a.flags & VDC_ATTN_APPEND_BIT) {
    // cache append only (chunked prefill): the rows go to the pools now; the attention tasks of the chunk's
    // positions start behind the barrier counted down here and find every row of the chunk in HBM
    compute_sync();
    if (q.tid >= 64 && q.tid < 64 + 2 * (D / 8)) {
      const int t = q.tid - 64;
      const size_t off = (size_t)ld_relaxed_gpu(a.state + VDC_ST_NEWROW) * (D * 2);
      uint8_t* dst = (t < D / 8 ? a.k_rows : a.v_rows) + off;
      reinterpret_cast<uint4*>(dst)[t % (D / 8)] = reinterpret_cast<const uint4*>(sh->newrows)[t];
    }
    __threadfence();
    compute_sync();
    if (q.tid == 0) red_relaxed_gpu_add(c.bars + a.bar, -1);
    return;
  }
  const unsigned n_ent = 2u * (unsigned)count;  // ring entries: K page, V page, K page, ...
  q.warp_phase_begin(n_ent, 0u);              // its CTA barrier also publishes qbf / krow / vrow / zero_row
  ATTN_STAMP(2);

  // Tensor-core page loop.  A warp owns positions 8w..8w+7 of every page: one 16x8x16 MMA tile column.
  // Scores: S[g][p] = sum_d Q[g][d] K[p][d], Q rows 0..G-1 of the A operand (rows G..15 zero), eight
  // k-steps; thread (gid = lane / 4, t = lane % 4) ends up with row gid, positions 2t and 2t + 1.
  // Output: O[g][d] += P[g][p] V[p][d] with the warp's eight positions as the lower half of a k-step
  // (upper half zero), sixteen 8-dim tiles; thread holds row gid, dims 8 nt + 2t, + 1.
  // Page rows are 256 bytes with their 16-byte pieces stored at (piece XOR (row mod 8)), in HBM and
  // therefore in the slot: the eight row addresses of one ldmatrix fall into eight different banks.
  const int gid = q.lane >> 2, t4 = q.lane & 3;
  const int lrow = q.lane & 7, lmi = q.lane >> 3;    // ldmatrix: this lane supplies row lrow of matrix lmi
  const int slice = q.warp * PPW;
  uint32_t qa[8][2];
  {
    const uint32_t* qb = reinterpret_cast<const uint32_t*>(sh->qbf) + gid * (D / 2);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = gid < G ? qb[8 * ks + t4] : 0u;
      qa[ks][1] = gid < G ? qb[8 * ks + 4 + t4] : 0u;
    }
  }
  const uint32_t krow_s = (uint32_t)__cvta_generic_to_shared(krow);
  const uint32_t vrow_s = (uint32_t)__cvta_generic_to_shared(vrow);
  const uint32_t zero_s = (uint32_t)__cvta_generic_to_shared(sh->zero_row);
  float m_run = -INFINITY, l_run = 0.f, acc[16][2], z0 = 0.f, z1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = 0.f;
  int blk = 0;
  if constexpr (kTwo) {
    // Two pages per trip (units that walk many pages: batched decode, prefill).  The warp's eight positions of the
    // second page fill the upper half of the P·V k-step that a single page leaves zero, and one softmax update
    // serves both pages: 32 instead of 48 MMAs and half the quad shuffles per two pages.  Ring entries of a trip:
    // K, V of the first page, K, V of the second.  An odd last page takes the single-page body below.
    bool stop = false;
    for (; blk + 1 < count && !stop; blk += 2) {
      const unsigned e0i = 2u * (unsigned)blk;
      const int ka_mask = q.warp_wait(e0i);
      if (ka_mask == kPopAbort) { stop = true; break; }
      const int kb_mask = q.warp_wait(e0i + 2u);
      if (kb_mask == kPopAbort) { stop = true; break; }
      const bool last_b = owner && blk + 1 == count - 1;      // only the second page can be the walk's last
      const int valid_b = last_b ? (kPair ? tail_valid_b : tail_valid) : VDC_KV_PAGE;
      const int valid_b_row = kPair ? (last_b ? (gid >= GQ ? tail_valid_b : tail_valid) : VDC_KV_PAGE) : valid_b;
      const int newpos_b = (!kPair && last_b) ? tail_valid - 1 : -1;
      const int p_l = slice + lrow;
      const uint32_t ka_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(ka_mask)));
      const uint32_t kb_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(kb_mask)));
      const uint32_t ka_base = ka_s + (uint32_t)p_l * (D * 2);
      const uint32_t kb_base = p_l == newpos_b ? krow_s : kb_s + (uint32_t)p_l * (D * 2);
      float s0 = 0.f, s1 = 0.f, u0 = 0.f, u1 = 0.f, t0 = 0.f, t1 = 0.f, w0 = 0.f, w1 = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t kr[4], ks[4];
        ldsm_x4(kr, ka_base + (uint32_t)(((4 * j + lmi) ^ lrow) << 4));
        ldsm_x4(ks, kb_base + (uint32_t)(((4 * j + lmi) ^ lrow) << 4));
        mma_rows8(s0, s1, z0, z1, qa[2 * j][0], qa[2 * j][1], kr[0], kr[1]);
        mma_rows8(t0, t1, z0, z1, qa[2 * j][0], qa[2 * j][1], ks[0], ks[1]);
        mma_rows8(u0, u1, z0, z1, qa[2 * j + 1][0], qa[2 * j + 1][1], kr[2], kr[3]);
        mma_rows8(w0, w1, z0, z1, qa[2 * j + 1][0], qa[2 * j + 1][1], ks[2], ks[3]);
      }
      const int p0 = slice + 2 * t4;
      s0 = (s0 + u0) * scale_log2;                            // the first page is never the last: all rows exist
      s1 = (s1 + u1) * scale_log2;
      t0 = p0 < valid_b_row ? (t0 + w0) * scale_log2 : -INFINITY;
      t1 = p0 + 1 < valid_b_row ? (t1 + w1) * scale_log2 : -INFINITY;
      float mx = fmaxf(fmaxf(s0, s1), fmaxf(t0, t1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);                   // finite: the first page has 64 real scores
      const float alpha = exp2f(m_run - m_new);
      const float e0 = exp2f(s0 - m_new), e1 = exp2f(s1 - m_new), e2 = exp2f(t0 - m_new), e3 = exp2f(t1 - m_new);
      float sum = (e0 + e1) + (e2 + e3);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      m_run = m_new;
      l_run = l_run * alpha + sum;
      const uint32_t pa = pack_bf16x2(e0, e1), pb = pack_bf16x2(e2, e3);
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        acc[nt][0] *= alpha;
        acc[nt][1] *= alpha;
      }
      const int va_mask = q.warp_wait(e0i + 1u);
      if (va_mask == kPopAbort) { stop = true; break; }
      const int vb_mask = q.warp_wait(e0i + 3u);
      if (vb_mask == kPopAbort) { stop = true; break; }
      const uint32_t va_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(va_mask)));
      const uint32_t vb_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(vb_mask)));
      const uint32_t va_base = va_s + (uint32_t)p_l * (D * 2);
      const uint32_t vb_base = p_l == newpos_b ? vrow_s : (p_l >= valid_b ? zero_s : vb_s + (uint32_t)p_l * (D * 2));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t vr[4], vs2[4];
        ldsm_x4_trans(vr, va_base + (uint32_t)(((4 * j + lmi) ^ lrow) << 4));
        ldsm_x4_trans(vs2, vb_base + (uint32_t)(((4 * j + lmi) ^ lrow) << 4));
#pragma unroll
        for (int mi = 0; mi < 4; ++mi) mma_rows8(acc[4 * j + mi][0], acc[4 * j + mi][1], z0, z1, pa, pb, vr[mi], vs2[mi]);
      }
      __syncwarp();
      if (q.lane == 0) {
        // counters 0..3 serve the trips (the slot pool holds three trips, so a warp is at most two trips ahead
        // of the slowest one), counter 4 the single odd page below: the two must never share a counter, or a
        // warp that races through the tail page hands back the wrong trip's slots and the pool leaks
        if (atomicAdd(&sh->att_done[(blk >> 1) & 3], 1) == kCW - 1) {
          sh->att_done[(blk >> 1) & 3] = 0;
          atomicOr(&sh->slot_avail, (uint32_t)(ka_mask | va_mask | kb_mask | vb_mask) & kSlotMaskAll);
        }
        sh->warp_next[q.warp] = q.head + e0i + 4u;
      }
    }
    if (stop) blk = count;      // a wait gave up: skip the tail, the phase end below sees the abort
  }
  for (; blk < count; ++blk) {
    const int k_mask = q.warp_wait(2u * (unsigned)blk);
    if (k_mask == kPopAbort) break;
    if (q.tid == 0) CHUNK_STAMP(c, q.head + 2u * (unsigned)blk, 2);
    ATTN_STAMP(3 + 3 * (blk & 1));
    const bool last = owner && blk == count - 1;
    // rows of the page that exist for the later of the unit's positions / for this thread's query row
    const int valid = last ? (kPair ? tail_valid_b : tail_valid) : VDC_KV_PAGE;
    const int valid_row = kPair ? (last ? (gid >= GQ ? tail_valid_b : tail_valid) : VDC_KV_PAGE) : valid;
    const int newpos = (!kPair && last) ? tail_valid - 1 : -1;  // this row of the page is not in HBM yet
    const int p_l = slice + lrow;                   // the page row this lane addresses
    // ---- scores of the warp's eight positions
    const uint32_t kb_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(k_mask)));
    const uint32_t k_base = p_l == newpos ? krow_s : kb_s + (uint32_t)p_l * (D * 2);
    float s0 = 0.f, s1 = 0.f, u0 = 0.f, u1 = 0.f;   // two accumulation chains: even and odd k-steps
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t kr[4];
      ldsm_x4(kr, k_base + (uint32_t)(((4 * j + lmi) ^ lrow) << 4));
      mma_rows8(s0, s1, z0, z1, qa[2 * j][0], qa[2 * j][1], kr[0], kr[1]);
      mma_rows8(u0, u1, z0, z1, qa[2 * j + 1][0], qa[2 * j + 1][1], kr[2], kr[3]);
    }
    s0 += u0;
    s1 += u1;
    // ---- online softmax (exp2 domain); a row's eight positions sit in the four lanes of a quad
    const int p0 = slice + 2 * t4;
    s0 = p0 < valid_row ? s0 * scale_log2 : -INFINITY;
    s1 = p0 + 1 < valid_row ? s1 * scale_log2 : -INFINITY;
    float mx = fmaxf(s0, s1);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const bool none = m_new == -INFINITY;
    const float alpha = none ? 1.f : exp2f(m_run - m_new);
    const float e0 = none ? 0.f : exp2f(s0 - m_new), e1 = none ? 0.f : exp2f(s1 - m_new);
    float sum = e0 + e1;
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    m_run = m_new;
    l_run = l_run * alpha + sum;
    // probabilities enter the PV product rounded to bf16, as a bf16 attention module hands them over
    const uint32_t pa = pack_bf16x2(e0, e1);
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      acc[nt][0] *= alpha;
      acc[nt][1] *= alpha;
    }
    // ---- O += P V
    const int v_mask = q.warp_wait(2u * (unsigned)blk + 1u);
    if (v_mask == kPopAbort) break;
    if (q.tid == 0) CHUNK_STAMP(c, q.head + 2u * (unsigned)blk + 1u, 2);
    ATTN_STAMP(4 + 3 * (blk & 1));
    const uint32_t vb_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(v_mask)));
    const uint32_t v_base = p_l == newpos ? vrow_s : (p_l >= valid ? zero_s : vb_s + (uint32_t)p_l * (D * 2));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t vr[4];
      ldsm_x4_trans(vr, v_base + (uint32_t)(((4 * j + lmi) ^ lrow) << 4));
#pragma unroll
      for (int mi = 0; mi < 4; ++mi) mma_rows8(acc[4 * j + mi][0], acc[4 * j + mi][1], z0, z1, pa, 0u, vr[mi], 0u);
    }
    // ---- the warp is done with this page pair; the last of the eight gives the slots back
    __syncwarp();
    if (q.lane == 0) {
      const int di = kTwo ? 4 : (blk & 7);
      if (atomicAdd(&sh->att_done[di], 1) == kCW - 1) {
        sh->att_done[di] = 0;
        atomicOr(&sh->slot_avail, (uint32_t)(k_mask | v_mask) & kSlotMaskAll);
        CHUNK_STAMP(c, q.head + 2u * (unsigned)blk + 1u, 3);
      }
      sh->warp_next[q.warp] = q.head + 2u * (unsigned)blk + 2u;
    }
    ATTN_STAMP(5 + 3 * (blk & 1));
  }
  if (q.lane == 0) sh->warp_next[q.warp] = 0xFFFFFFFFu;
  // ---- the warps' states meet in shared memory, four query rows at a time: red[warp][4][128], then m and l
  float* red = sh->red;
  float* ml = red + kCW * 4 * D;   // [warp][m of 4 rows | l of 4 rows]
  float* rec = a.records + (size_t)a.split * REC;
#pragma unroll
  for (int pass = 0; pass < (G + 3) / 4; ++pass) {
    if (pass > 0) compute_sync();  // the previous pass has been folded
    if ((gid >> 2) == pass) {
      float* dst = red + (q.warp * 4 + (gid & 3)) * D + 2 * t4;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2*>(dst + 8 * nt) = make_float2(acc[nt][0], acc[nt][1]);
      if (t4 == 0) {
        ml[q.warp * 8 + (gid & 3)] = m_run;
        ml[q.warp * 8 + 4 + (gid & 3)] = l_run;
      }
    }
    if (pass == 0) {
      q.warp_phase_end(n_ent);  // CTA barrier: every warp is done with the pages and has published its state
      if (q.aborted) return;
      ATTN_STAMP(11);
    } else {
      compute_sync();
    }
    for (int o = q.tid; o < 4 * D; o += kCT) {
      const int gg = o / D, d = o % D, g = pass * 4 + gg;
      if (g >= G) break;
      float m = -INFINITY;
#pragma unroll
      for (int k = 0; k < kCW; ++k) m = fmaxf(m, ml[k * 8 + gg]);
      float num = 0.f, l = 0.f;
#pragma unroll
      for (int k = 0; k < kCW; ++k) {
        const float mw = ml[k * 8 + gg];
        const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
        num = fmaf(wgt, red[(k * 4 + gg) * D + d], num);
        l = fmaf(wgt, ml[k * 8 + 4 + gg], l);
      }
      rec[g * D + d] = num;
      if (d == 0) {
        rec[G * D + g] = m;
        rec[G * D + G + g] = l;
      }
    }
  }
  if (!kPair && owner && q.tid >= 64 && q.tid < 64 + 2 * (D / 8)) {
    // the new cache rows go to HBM (already in the page-row piece order); the next step's page loads
    // (a later launch) see them
    const int t = q.tid - 64;
    const size_t off = (size_t)ld_relaxed_gpu(a.state + VDC_ST_NEWROW) * (D * 2);
    uint8_t* dst = (t < D / 8 ? a.k_rows : a.v_rows) + off;
    reinterpret_cast<uint4*>(dst)[t % (D / 8)] = reinterpret_cast<const uint4*>(sh->newrows)[t];
  }
  // arrival: every writer drains its own record writes (in parallel) before the barrier lets thread 0
  // bump the head's counter, so the bump needs no releasing fence of its own; its acquire side orders the
  // merge's reads behind the other splits' bumps
  __threadfence();
  compute_sync();
  if (q.tid == 0) {
    const int old = atom_acquire_gpu_add(a.counter, 1);
    sh->misc[34] = (old == a.n_splits - 1) ? 1.f : 0.f;
  }
  compute_sync();
  ATTN_STAMP(12);
  if (sh->misc[34] == 0.f) return;

  // ---- last arrival for this head: merge the split records (read past L1: other SMs wrote them).
  // Two outputs per thread.  The numerators of the first sixteen splits are requested before anything
  // else; meanwhile one warp per query row turns the splits' maxima and sums into weights in shared
  // memory, so the whole merge costs about one L2 round trip.
  const int ns = a.n_splits;
  float* wts = red;                  // [n_splits][G] weights 2^(m_s - m), then den[G]
  const int o = q.tid * 2;           // G * 128 outputs over 256 threads: G / 4 rounds
  float2 vs[16];
#pragma unroll
  for (int k = 0; k < 16; ++k)
    vs[k] = k < ns ? __ldcg(reinterpret_cast<const float2*>(a.records + (size_t)k * REC + o)) : make_float2(0.f, 0.f);
  if (q.warp < G) {
    const int g = q.warp;
    // lane-strided over the splits; the first two rounds stay in registers
    float mr[2] = {-INFINITY, -INFINITY}, lr[2] = {0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int sidx = q.lane + 32 * k;
      if (sidx < ns) {
        mr[k] = __ldcg(a.records + (size_t)sidx * REC + G * D + g);
        lr[k] = __ldcg(a.records + (size_t)sidx * REC + G * D + G + g);
      }
    }
    float m = fmaxf(mr[0], mr[1]);
    for (int sidx = q.lane + 64; sidx < ns; sidx += 32) m = fmaxf(m, __ldcg(a.records + (size_t)sidx * REC + G * D + g));
#pragma unroll
    for (int sh_ = 16; sh_ > 0; sh_ >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, sh_));
    float den = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int sidx = q.lane + 32 * k;
      if (sidx < ns) {
        const float w = (mr[k] == -INFINITY) ? 0.f : exp2f(mr[k] - m);
        wts[sidx * G + g] = w;
        den = fmaf(w, lr[k], den);
      }
    }
    for (int sidx = q.lane + 64; sidx < ns; sidx += 32) {
      const float* r = a.records + (size_t)sidx * REC;
      const float ms = __ldcg(r + G * D + g);
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      wts[sidx * G + g] = w;
      den = fmaf(w, __ldcg(r + G * D + G + g), den);
    }
    den = warp_sum(den);
    if (q.lane == 0) wts[ns * G + g] = den;
  }
  compute_sync();
#pragma unroll
  for (int rnd = 0; rnd < (G * D) / (2 * kCT); ++rnd) {
    const int oo = o + rnd * 2 * kCT, g = oo / D;
    float n0 = 0.f, n1 = 0.f;
    if (rnd == 0) {
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float w = k < ns ? wts[k * G + g] : 0.f;
        n0 = fmaf(w, vs[k].x, n0);
        n1 = fmaf(w, vs[k].y, n1);
      }
    }
#pragma unroll 8
    for (int sidx = rnd == 0 ? 16 : 0; sidx < ns; ++sidx) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(a.records + (size_t)sidx * REC + oo));
      const float w = wts[sidx * G + g];
      n0 = fmaf(w, v.x, n0);
      n1 = fmaf(w, v.y, n1);
    }
    const float den = wts[ns * G + g];
    const __nv_bfloat16 r0 = __float2bfloat16_rn(den > 0.f ? n0 / den : 0.f);
    const __nv_bfloat16 r1 = __float2bfloat16_rn(den > 0.f ? n1 / den : 0.f);
    if (a.bpad) {
      // pair units: query rows GQ.. are the next sequence slot's heads
      const int bb = (kPair && g >= GQ) ? a.b + 1 : a.b, ob = (kPair && g >= GQ) ? oo - GQ * D : oo;
      uint8_t* dst = reinterpret_cast<uint8_t*>(a.out) + (size_t)(ob >> 3) * a.bpad * 16 + (bb >> 3) * 128 + (bb & 7) * 16 +
                     (ob & 7) * 2;
      *reinterpret_cast<__nv_bfloat162*>(dst) = __halves2bfloat162(r0, r1);
    } else {
      *reinterpret_cast<__nv_bfloat162*>(a.out + oo) = __halves2bfloat162(r0, r1);
    }
  }
  __threadfence();   // every writer drains its outputs in parallel
  compute_sync();
  ATTN_STAMP(13);
  if (q.tid == 0) {
    *a.counter = 0;  // this layer's counter is next used by the next step, a later launch
    red_relaxed_gpu_add(c.bars + a.bar, -1);  // every writer fenced before the barrier above
  }
}

// ------------------------------------------------------------------------- //
// task: MoE routing — softmax over all experts, top-k, renormalise
// ------------------------------------------------------------------------- //
// Pop order: router logits (n_experts fp32), route record (raw address: int32
// ids[16], fp32 weights[16], int32 local[16], int32 count[16]).  One warp does the work.
__device__ void task_moe_route(Compute& q, int n_experts, int top_k, int rank, int world) {
  const Ctx& c = q.c;
  const int lg_mask = q.pop();
  q.pop();
  int* ids = reinterpret_cast<int*>(q.addr());
  float* wts = reinterpret_cast<float*>(ids + 16);
  const uint32_t meta = q.meta();
  if (q.aborted) return;
  if (q.warp == 0) {
    const float* lg = (const float*)slot_ptr(c, first_slot(lg_mask));
    constexpr int kMaxPerLane = 8;  // up to 256 experts
    float v[kMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = q.lane + 32 * j;
      v[j] = e < n_experts ? lg[e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      v[j] = (v[j] == -INFINITY) ? 0.f : __expf(v[j] - mx);  // unnormalised probabilities
      sum += v[j];
    }
    sum = warp_sum(sum);
    float sel_sum = 0.f, my_w = 0.f;
    int my_id = 0;
    for (int k = 0; k < top_k; ++k) {
      float bv = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = q.lane + 32 * j;
        if (e < n_experts && v[j] > bv) {  // ascending e within a lane: first maximum wins
          bv = v[j];
          bi = e;
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
      if ((bi & 31) == q.lane) v[bi >> 5] = -1.f;  // taken
      const float p = bv / sum;
      sel_sum += p;
      if (q.lane == k) {
        my_w = p;
        my_id = bi;
      }
    }
    if (q.lane < top_k) {
      ids[q.lane] = my_id;
      wts[q.lane] = bf16_round(my_w / sel_sum);
      // expert parallelism: which of this rank's experts, and whether the slot is this rank's at all
      const int per_rank = world > 1 ? n_experts / world : n_experts;
      const bool mine = world <= 1 || my_id / per_rank == rank;
      ids[32 + q.lane] = mine ? my_id % per_rank : 0;
      ids[48 + q.lane] = mine ? 0x7FFF : 0;
    }
  }
  compute_sync();
  q.release(meta);
  q.free_slots(lg_mask);
}

// ------------------------------------------------------------------------- //
// task: final argmax over the per-SM candidates, token hand-over, state advance
// ------------------------------------------------------------------------- //
// Pop order: candidate records (n x {f32 val, i32 idx, pad, pad}), state (raw
// address), token log (raw address, int32 per step), done (raw address slot that
// is pushed back so the store warp can release a barrier).
__device__ void task_argmax_final(Compute& q, int n, int local_only, const PeerOut* peers = nullptr) {
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
    if (q.lane == 0 && local_only && peers != nullptr) {
      // vocabulary shard under in-kernel tensor parallelism: this rank's best candidate goes into its two
      // tagged entries ({value, tag}, {row index, tag}) of every rank's exchange block (`log` holds their
      // byte offset)
      const unsigned long long off = reinterpret_cast<unsigned long long>(log);
      const uint32_t tag = exchange_tag(reinterpret_cast<const int*>(__ldg(peers->table + peers->n)), peers->ex);
      for (int pr = 0; pr < peers->n; ++pr) {
        const unsigned long long base = __ldg(peers->table + pr) + off;
        st_tagged_sys(base, __float_as_uint(bv), tag);
        st_tagged_sys(base + 8, (uint32_t)bi, tag);
      }
    } else if (q.lane == 0 && local_only) {
      // tensor-parallel vocabulary shard: leave this rank's best candidate as one
      // record; the ranks' records are reduced by a second, global call
      reinterpret_cast<float*>(log)[0] = bv;
      log[1] = bi;
      log[2] = 0;
      log[3] = 0;
      __threadfence();
    } else if (q.lane == 0) {
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
// tasks: in-kernel tensor-parallel exchange (peer stores instead of a collective library)
// ------------------------------------------------------------------------- //
// Bounded wait (any thread) until the tagged entry at `p` carries `tag`; returns its payload.  A wait that
// gives up raises the abort and marks the CTA.
__device__ __forceinline__ uint32_t tagged_wait(Compute& q, const void* p, uint32_t tag, int opcode) {
  unsigned long long v = ld_tagged_sys(p);
  if ((uint32_t)(v >> 32) != tag) {
    const bool ok = wait_until(q.c, [&] { return (uint32_t)((v = ld_tagged_sys(p)) >> 32) == tag; }, 0, (int)q.pc, opcode, -1, 20);
    if (!ok) q.sh->aborted = 1;
  }
  return (uint32_t)v;
}

// XREDUCE: hidden[i] = bf16(hidden[i] + sum over ranks of the partial sums) for a slice of n elements.  Every
// thread polls its own element's entry of every rank ({fp32 bits, tag} written by the ranks' projections),
// so the slice is folded as soon as the last partial row lands; counts `bar` down.  Pops nothing.
__device__ void task_xreduce(Compute& q, int n, int n_ranks, int bar, const unsigned long long* xbuf, size_t rank_stride,
                             uint32_t ex, __nv_bfloat16* hidden, const int* state) {
  const uint32_t tag = exchange_tag(state, ex);
  for (int i = q.tid; i < n; i += kCT) {
    float sum = 0.f;
    for (int r = 0; r < n_ranks; ++r)   // rank order: every rank folds the same sum
      sum += __uint_as_float(tagged_wait(q, xbuf + (size_t)r * rank_stride + i, tag, 0x7330));
    hidden[i] = __float2bfloat16_rn(__bfloat162float(hidden[i]) + sum);
  }
  __threadfence();   // every writer drains its own outputs; thread 0 then counts down without a fence
  compute_sync();
  if (q.sh->aborted) {
    q.aborted = true;
    return;
  }
  if (q.tid == 0 && bar != 0xFFFF) red_relaxed_gpu_add(q.c.bars + bar, -1);
}

// XWAIT: collects the ranks' best candidates (two tagged entries per rank: value, row index) into compact
// records {f32 value, i32 index, 0, 0} at `rec_out` and counts `bar` down.  Pops nothing.
__device__ void task_xwait(Compute& q, int bar, int n_ranks, uint32_t ex, const unsigned long long* entries,
                           const int* state, uint32_t* rec_out) {
  const uint32_t tag = exchange_tag(state, ex);
  if (q.tid < 2 * n_ranks) {
    const uint32_t v = tagged_wait(q, entries + q.tid, tag, 0x7331);
    rec_out[(q.tid >> 1) * 4 + (q.tid & 1)] = v;
    rec_out[(q.tid >> 1) * 4 + 2 + (q.tid & 1)] = 0u;
    __threadfence();
  }
  compute_sync();
  if (q.sh->aborted) {
    q.aborted = true;
    return;
  }
  if (q.tid == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");  // a bulk copy reads the records
    red_release_gpu_add(q.c.bars + bar, -1);
  }
}

}  // namespace vdc
