// Batched-decode tasks of the compute virtual core: projections on the tcgen05
// tensor cores with the accumulator in tensor memory, embedding gather into
// the k-chunk-major activation layout, and the per-sequence state advance.
//
// The reference pads every decode batch to 8 slots and runs its WGMMA GEMV
// tile on it (include/task/gemv.cuh:13-128).  Here a batch of 2..128 sequences
// sits on the 128 lanes of a tcgen05 accumulator and the weight rows of the
// task sit on its columns, so that weight rows can be dealt to the SMs in
// groups of 16 and each sequence's outputs land in one thread's registers.
#pragma once
#include "mk_compute.cuh"

namespace vdc {

constexpr uint32_t kTmemCols = 512;

// ------------------------------------------------------------------------- //
// tcgen05 helpers
// ------------------------------------------------------------------------- //
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Warp-wide: allocates `ncols` columns of tensor memory, the base address lands in *dst (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Shared-memory operand descriptor, no swizzle, K-major: 8 rows x 16 bytes form one contiguous
// 128-byte core matrix; `lbo` = byte distance between the two core matrices a 16-element k-step
// spans, `sbo` = byte distance between consecutive 8-row groups.  Bit 46 marks the sm_100 format.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
         (1ull << 46);
}
// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, both K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc_bf16_m128(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}
// One thread issues: D[tmem] (+)= A[smem] * B[smem]^T for one k-step of 16.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every tensor-core operation this thread issued so far is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// Warp-wide: 16 consecutive fp32 columns of this thread's lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Byte offset of the 16-byte piece holding (b, k..k+7) in a k-chunk-major [Bpad, K] matrix.
__device__ __forceinline__ size_t kc_piece(int bpad, int b, int k) {
  return ((size_t)(k >> 3) * (size_t)(bpad >> 3) + (size_t)(b >> 3)) * 128 + (size_t)(b & 7) * 16;
}

// Bounded wait on one of the tensor-core completion barriers (thread 0 only).
__device__ __forceinline__ bool mma_wait(Compute& q, unsigned commit_index) {
  uint64_t* bar = &q.sh->mma_bar[commit_index & 3u];
  const uint32_t parity = (commit_index >> 2) & 1u;
  if (mbar_try_wait(bar, parity)) return true;
  const bool ok = wait_until(q.c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)q.pc, 0x7300, -1, 0);
  if (!ok) q.sh->aborted = 1;
  return ok;
}

// ------------------------------------------------------------------------- //
// task: batched projection on the tensor cores
// ------------------------------------------------------------------------- //
// One unit = a block of N weight rows (N <= 256, the accumulator's columns) times a K-range.
// The memory stream delivers groups of one X chunk (all sequences, G * KS * 16 inputs) and
// the G W chunks that go with it.  A block whose K is cut into several units (n_slices > 1)
// is summed in an fp32 scratch area in global memory; the unit that arrives last applies
// the epilogue, clears the scratch and releases the barrier.
struct GemmTc {
  int n_w;       // W chunks of this unit
  int N, KS, G;  // weight rows, k-steps of 16 per W chunk, W chunks per X chunk
  int mode;
  bool norm;
  float eps;
  int B, Bpad, Kfull;
  uint8_t* out;
  unsigned long long* keys;
  float* stats;  // fp32 per sequence: sum of squares of the input rows (norm) / of the updated rows (ADD_PACKED)
  int n0, ld, bar;
  float* scratch;  // [B][N] fp32 partial sums of this block (n_slices > 1)
  int* counter;    // arrivals of this block's units
  int n_slices;
  int wfmt;             // 0: bf16 weights; 1: e4m3, 2: NVFP4 (both converted to bf16 in shared memory)
  const float* scales;  // e4m3: fp32 per-row scales of the block, applied in the epilogue
};

constexpr int kStages = VDC_TC_STAGES;  // bf16 staging buffers of the converted-weight paths

struct EpiAcc {
  float ssq;   // ADD_PACKED: squares of the new values
  float best;  // ARGMAX
  int best_row;
};

// Epilogue of 16 consecutive output rows (row .. row+15) of sequence b.
__device__ __forceinline__ void gemm_epilogue16(const GemmTc& g, int b, int row, float (&v)[16], EpiAcc& acc) {
  if (g.scales != nullptr) {
    // e4m3 weights: the accumulator holds sums over the codes; one fp32 scale per output row
    const float4* sc = reinterpret_cast<const float4*>(g.scales + (row - g.n0));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 t = __ldg(sc + j);
      v[4 * j] *= t.x; v[4 * j + 1] *= t.y; v[4 * j + 2] *= t.z; v[4 * j + 3] *= t.w;
    }
  }
  if (g.mode == VDC_GEMM_MODE_STORE_ROWS) {
    uint4* dst = reinterpret_cast<uint4*>(g.out + ((size_t)b * g.ld + row) * 2);
    dst[0] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    dst[1] = make_uint4(pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]), pack_bf16x2(v[12], v[13]),
                        pack_bf16x2(v[14], v[15]));
  } else if (g.mode == VDC_GEMM_MODE_SILU_PAIRS) {
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gt = bf16_round(v[2 * j]), up = bf16_round(v[2 * j + 1]);
      a[j] = bf16_round(gt / (1.f + __expf(-gt))) * up;
    }
    *reinterpret_cast<uint4*>(g.out + kc_piece(g.Bpad, b, row >> 1)) =
        make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
  } else if (g.mode == VDC_GEMM_MODE_ADD_PACKED) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(g.out + kc_piece(g.Bpad, b, row + 8 * h));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // every element gets exactly one add per projection, so old + v is its final value
        const __nv_bfloat162 add = __floats2bfloat162_rn(v[8 * h + 2 * j], v[8 * h + 2 * j + 1]);
        const float2 nv = __bfloat1622float2(__hadd2(atomicAdd(dst + j, add), add));
        acc.ssq = fmaf(nv.x, nv.x, fmaf(nv.y, nv.y, acc.ssq));
      }
    }
  } else {  // ARGMAX over bf16-rounded logits, the lowest row wins ties
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float l = bf16_round(v[j]);
      if (l > acc.best) {
        acc.best = l;
        acc.best_row = row + j;
      }
    }
  }
}

// Publishes what gemm_epilogue16 accumulated for sequence b and resets it.
__device__ __forceinline__ void gemm_epilogue_flush(const GemmTc& g, int b, EpiAcc& acc) {
  if (g.mode == VDC_GEMM_MODE_ARGMAX && acc.best_row != 0x7fffffff) {
    uint32_t u = __float_as_uint(acc.best);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // order-preserving map of the float
    atomicMax(g.keys + b, ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)acc.best_row));
  }
  if (g.mode == VDC_GEMM_MODE_ADD_PACKED && g.stats != nullptr) atomicAdd(g.stats + b, acc.ssq);
  acc.ssq = 0.f;
  acc.best = -INFINITY;
  acc.best_row = 0x7fffffff;
}

#ifdef VDC_TC_PROFILE
#define TCS(i) if (q.tid == 0) { const long long _n = clock64(); c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 100 + (i)] += _n - tcs_mark; tcs_mark = _n; }
#else
#define TCS(i)
#endif
VDC_TASK void task_gemm_tc(Compute& q, const GemmTc& g) {
  Shared* sh = q.sh;
  const Ctx& c = q.c;
#ifdef VDC_TC_PROFILE
  long long tcs_mark = clock64();
#endif
  // Tensor memory is taken the first time a program needs it and given back when the kernel ends.
  if (!sh->tmem_ready) {
    if (q.warp == 0) tmem_alloc(&sh->tmem_base, kTmemCols);
    if (q.tid >= 32 && q.tid < 36) mbar_init(&sh->mma_bar[q.tid - 32], 1);
    if (q.tid == 36) mbar_init(&sh->mma_final, 1);
    if (q.tid >= 64 && q.tid < 80) mbar_init(&sh->x_ready[q.tid - 64], 1);
    if (q.tid >= 96 && q.tid < 112) mbar_init(&sh->w_ready[q.tid - 96], 1);
    if (q.tid >= 32 && q.tid < 112) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    compute_sync();
    tc_fence_after();
    if (q.tid == 0) sh->tmem_ready = 1;
  }
  int normw_mask = 0;
  if (g.norm) normw_mask = q.pop();
  int stage_mask[kStages] = {};
  if (g.wfmt != 0) {
#pragma unroll
    for (int st = 0; st < kStages; ++st) stage_mask[st] = q.pop();  // allocate-only entries: bf16 staging buffers
  }
  if (q.aborted) return;
  const unsigned mma_base = q.mma_count;  // commits issued before this task (uniform across the CTA)
  const uint8_t* nw = g.norm ? (const uint8_t*)slot_ptr(c, first_slot(normw_mask)) : nullptr;
  const uint32_t tmem = sh->tmem_base;
  const uint32_t idesc = umma_idesc_bf16_m128(g.N);
  const uint32_t lbo_a = (uint32_t)g.Bpad * 16u, lbo_b = (uint32_t)g.N * 16u;
  const int n_x = (g.n_w + g.G - 1) / g.G;                      // X chunks = groups
  const unsigned n_ent = (unsigned)(g.n_w + n_x);               // ring entries: X, G x W, X, G x W, ...
  auto x_entry = [&](int grp) { return (unsigned)(grp * (g.G + 1)); };
  auto w_entry = [&](int j) { return (unsigned)((j / g.G) * (g.G + 1) + 1 + j % g.G); };

  // The streaming loop has no CTA-wide synchronisation.  Warp 0 consumes the ring entries in
  // order: it waits for the chunks, one lane issues the tensor-core work and, once the
  // previous chunk's reads are done, recycles its slots.  With norm the other seven warps
  // run ahead of it, normalising the X chunks in place and signalling each chunk's barrier.
  TCS(0);
  q.warp_phase_begin(n_ent, q.warp == 0 ? 0u : n_ent);
  if (q.warp > 0 && (g.norm || g.wfmt != 0)) {
    // The seven warps work as a team of 224 threads, ahead of the issuer: they normalise each X
    // chunk in place and, for e4m3 weights, convert each W chunk into a bf16 staging buffer.
    // One warp does the (bounded) waiting and tells the team, so that all leave together on an abort.
    constexpr int kTeam = (kCW - 1) * 32;
    const int t = q.tid - 32;
    float* rs = sh->red;  // per-sequence rsqrt(mean x^2 + eps)
    int* told = reinterpret_cast<int*>(sh->misc) + 36;
    for (int j = 0; j < g.n_w; ++j) {
      const int grp = j / g.G, jj = j % g.G;
      if (g.norm && jj == 0) {
        if (q.warp == 1) {
          const int m = q.warp_wait(x_entry(grp));
          if (q.lane == 0) told[0] = m;
        }
        asm volatile("bar.sync 6, %0;" ::"n"(kTeam) : "memory");
        const int xm = told[0];
        if (xm == kPopAbort) break;
        if (grp == 0) {
          // Any X chunk of this task was loaded after the producers of the input matrix had
          // finished, and with them the sums of squares they left (read past L1).
          if (t < g.Bpad) rs[t] = rsqrtf(__ldcg(g.stats + t) / (float)g.Kfull + g.eps);
          asm volatile("bar.sync 6, %0;" ::"n"(kTeam) : "memory");
        }
        uint8_t* xs = (uint8_t*)slot_ptr(c, first_slot(xm));
        const int w_in_grp = min(g.G, g.n_w - grp * g.G);
        const int pieces = w_in_grp * g.KS * 2 * g.Bpad;  // 16-byte pieces of this X chunk
        const int kc0 = grp * g.G * g.KS * 2;             // the chunk's first 8-element k group within the unit
        // RMSNorm in place, rounded like a bf16 tensor expression: bf16(w * bf16(x * rstd))
        for (int p = t; p < pieces; p += kTeam) {
          const uint4 v = lds128(xs + p * 16);
          const uint4 w = lds128(nw + (kc0 + p / g.Bpad) * 16);
          const float rstd = rs[p & (g.Bpad - 1)];
          const uint32_t xv[4] = {v.x, v.y, v.z, v.w}, wv[4] = {w.x, w.y, w.z, w.w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            o[i] = pack_bf16x2(bf16_round(bf_lo(xv[i]) * rstd) * bf_lo(wv[i]), bf16_round(bf_hi(xv[i]) * rstd) * bf_hi(wv[i]));
          *reinterpret_cast<uint4*>(xs + p * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_proxy_async_smem();  // the tensor cores read shared memory through the async proxy
        asm volatile("bar.sync 6, %0;" ::"n"(kTeam) : "memory");
        if (t == 0) mbar_arrive(&sh->x_ready[(q.xr_count + (unsigned)grp) & 15u]);
      }
      if (g.wfmt != 0) {
        // W chunk j: [Kc/16][N/8][8 rows][16 k] e4m3 bytes -> staging buffer j % kStages as
        // [Kc/8][N/8][8 rows][8 k] bf16 (exact), once the tensor cores are done with the
        // buffer's previous occupant (chunk j - kStages)
        if (q.warp == 1) {
          int m = q.warp_wait(w_entry(j));
          if (m != kPopAbort && j >= kStages) {
            int ok = 1;
            if (q.lane == 0) ok = mma_wait(q, mma_base + (unsigned)(j - kStages)) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, ok, 0)) m = kPopAbort;
          }
          if (q.lane == 0) told[1] = m;
        }
        asm volatile("bar.sync 6, %0;" ::"n"(kTeam) : "memory");
        const int wm = told[1];
        if (wm == kPopAbort) break;
        const uint8_t* src = (const uint8_t*)slot_ptr(c, first_slot(wm));
        uint8_t* dst = (uint8_t*)slot_ptr(c, first_slot(stage_mask[j % kStages]));
        const int pieces = g.KS * g.N;  // (16-k group, row) pairs of the chunk: 16 weights each
        if (g.wfmt == 1) {
          for (int p = t; p < pieces; p += kTeam) {   // e4m3: one 16-byte piece per pair
            const uint4 v = lds128(src + p * 16);
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 lo = e4m3x2_to_float2(wv[i] & 0xFFFFu), hi = e4m3x2_to_float2(wv[i] >> 16);
              o[2 * i] = pack_bf16x2(lo.x, lo.y);
              o[2 * i + 1] = pack_bf16x2(hi.x, hi.y);
            }
            const int i16 = p / g.N, row = p - i16 * g.N;
            *reinterpret_cast<uint4*>(dst + ((size_t)(2 * i16) * g.N + row) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + ((size_t)(2 * i16 + 1) * g.N + row) * 16) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        } else {
          // NVFP4: per 16-k group [N x 8 bytes of e2m1 pairs | N e4m3 block scales]; code times block scale is
          // exact in bf16 (two significant bits times four), the per-row tensor scale waits for the epilogue
          for (int p = t; p < pieces; p += kTeam) {
            const int i16 = p / g.N, row = p - i16 * g.N;
            const uint8_t* grp = src + (size_t)i16 * 9 * g.N;
            const uint2 cv = *reinterpret_cast<const uint2*>(grp + row * 8);
            const float sc = e4m3_to_float(grp[8 * g.N + row]);
            const uint32_t cw[2] = {cv.x, cv.y};
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 f = __half22float2(e2m1x2_to_half2((cw[i >> 2] >> (8 * (i & 3))) & 0xFFu));
              o[i] = pack_bf16x2(f.x * sc, f.y * sc);
            }
            *reinterpret_cast<uint4*>(dst + ((size_t)(2 * i16) * g.N + row) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + ((size_t)(2 * i16 + 1) * g.N + row) * 16) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 6, %0;" ::"n"(kTeam) : "memory");  // also: everybody has read told[] and the chunk
        if (t == 0) {
          atomicOr(&sh->slot_avail, (uint32_t)wm & kSlotMaskAll);  // the e4m3 chunk's slots are free already
          mbar_arrive(&sh->w_ready[(q.wr_count + (unsigned)j) & 15u]);
        }
      }
    }
  }
  if (q.warp == 0) {
    int w_prev = 0, x_prev = 0;  // lane 0: slots whose tensor-core reads may still be in flight
    int xm = 0;
#ifdef VDC_TC_PROFILE
    long long t_data = 0, t_xr = 0, t_mma = 0, t_wait = 0, t_xw = 0, t_ww = 0;
#endif
    for (int j = 0; j < g.n_w; ++j) {
      const int grp = j / g.G, jj = j % g.G;
#ifdef VDC_TC_PROFILE
      const long long td0 = clock64();
#endif
      int x_done = 0;
      if (jj == 0) x_done = xm;  // the previous group's X chunk: its last W chunk is the previous chunk
#ifdef VDC_TC_PROFILE
      const long long tq0 = clock64();
#endif
      if (jj == 0) {
        xm = q.warp_wait(x_entry(grp));
        if (xm == kPopAbort) break;
        if (q.lane == 0) CHUNK_STAMP(c, q.head + x_entry(grp), 2);
      }
#ifdef VDC_TC_PROFILE
      if (j > 0) t_xw += clock64() - tq0;
      const long long tq1 = clock64();
#endif
      const int wm = q.warp_wait(w_entry(j));
#ifdef VDC_TC_PROFILE
      if (j > 0) t_ww += clock64() - tq1;
#endif
      if (wm == kPopAbort) break;
      if (q.lane == 0) CHUNK_STAMP(c, q.head + w_entry(j), 2);
      if (g.wfmt != 0) {
        // the converted chunk, not the loaded one, is the operand
        int ok = 1;
        if (q.lane == 0) {
          const unsigned gch = q.wr_count + (unsigned)j;
          uint64_t* bar = &sh->w_ready[gch & 15u];
          const uint32_t parity = (gch >> 4) & 1u;
          if (!mbar_try_wait(bar, parity)) {
            ok = wait_until(c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)q.pc, 0x7300, -1, 0);
            if (!ok) sh->aborted = 1;
          }
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      }
#ifdef VDC_TC_PROFILE
      t_data += clock64() - td0;
      const long long tx0 = clock64();
#endif
      if (g.norm && jj == 0) {
        int ok = 1;
        if (q.lane == 0) {
          const unsigned gch = q.xr_count + (unsigned)grp;
          uint64_t* bar = &sh->x_ready[gch & 15u];
          const uint32_t parity = (gch >> 4) & 1u;
          if (!mbar_try_wait(bar, parity)) {
            ok = wait_until(c, [&] { return mbar_try_wait(bar, parity); }, 0, (int)q.pc, 0x7300, -1, 0);
            if (!ok) sh->aborted = 1;
          }
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      }
#ifdef VDC_TC_PROFILE
      t_xr += clock64() - tx0;
      const long long tm0 = clock64();
#endif
      if (q.lane == 0) {
        tc_fence_after();
        uint64_t adesc = umma_desc(smem_u32(slot_ptr(c, first_slot(xm))) + (uint32_t)(jj * g.KS) * 2u * lbo_a, lbo_a, 128u);
        const int b_slot = g.wfmt != 0 ? first_slot(stage_mask[j % kStages]) : first_slot(wm);
        uint64_t bdesc = umma_desc(smem_u32(slot_ptr(c, b_slot)), lbo_b, 128u);
        const uint64_t step_a = (uint64_t)((2u * lbo_a) >> 4), step_b = (uint64_t)((2u * lbo_b) >> 4);
        umma_bf16(tmem, adesc, bdesc, idesc, (uint32_t)(j != 0));
#pragma unroll 4
        for (int kk = 1; kk < g.KS; ++kk) {
          adesc += step_a;  // the start-address field: 16 k further in both operands
          bdesc += step_b;
          umma_bf16(tmem, adesc, bdesc, idesc, 1u);
        }
        umma_commit(&sh->mma_bar[q.mma_count & 3u]);
#ifdef VDC_TC_PROFILE
        t_mma += clock64() - tm0;
        const long long tw0 = clock64();
#endif
        // the previous chunk's reads are certainly done once its commit arrived
        if (j > 0) {
          int done = (g.wfmt != 0 ? 0 : w_prev) | x_done;  // e4m3 chunks were freed by the converting team
          if (!mma_wait(q, q.mma_count - 1)) done = 0;
          if (done) atomicOr(&sh->slot_avail, (uint32_t)done & kSlotMaskAll);
          CHUNK_STAMP(c, q.head + w_entry(j - 1), 3);
          sh->warp_next[0] = q.head + x_entry(grp);  // ring entries before this group may be recycled
        }
        w_prev = wm & (int)kSlotMaskAll;
        q.mma_count++;
#ifdef VDC_TC_PROFILE
        t_wait += clock64() - tw0;
#endif
      }
      __syncwarp();
    }
    if (q.lane == 0) {
      x_prev = xm == kPopAbort ? 0 : (xm & (int)kSlotMaskAll);
      if (g.wfmt != 0) w_prev = 0;
      if (q.mma_count > 0 && mma_wait(q, q.mma_count - 1) && (w_prev | x_prev))
        atomicOr(&sh->slot_avail, (uint32_t)(w_prev | x_prev) & kSlotMaskAll);
      sh->warp_next[0] = 0xFFFFFFFFu;
#ifdef VDC_TC_PROFILE
      uint64_t* pr = c.profile + c.sm * VDC_NUM_PROFILE_EVENTS;
      pr[8] += t_data; pr[9] += t_xr; pr[10] += t_mma; pr[11] += t_wait; pr[12] += g.n_w;
      pr[13] += (uint64_t)g.n_w * g.KS;
      pr[14] += t_xw; pr[15] += t_ww;   // waits for X / W chunks after a task's first chunk
#endif
    }
  }
  tc_fence_before();
  q.warp_phase_end(n_ent);  // CTA barrier: accumulator complete (lane 0 saw the last commit)
  tc_fence_after();
  if (g.norm) q.xr_count += (unsigned)n_x;
  if (g.wfmt != 0) q.wr_count += (unsigned)g.n_w;
  q.mma_count = mma_base + (unsigned)g.n_w;  // every thread keeps the count (thread 0 counted along)
  if (q.aborted) return;
  if (g.wfmt != 0) {
    int all = 0;
#pragma unroll
    for (int st = 0; st < kStages; ++st) all |= stage_mask[st];
    q.free_slots(all);
  }
  TCS(1);

  // Lane b of the accumulator belongs to sequence b; warps w and w+4 share the lane quarter
  // w % 4 and split the columns.
  const int quarter = q.warp & 3, half = q.warp >> 2;
  const int b = quarter * 32 + q.lane;
  const int ng = g.N >> 4;
  const int g0 = half ? (ng + 1) / 2 : 0, g1 = half ? ng : (ng + 1) / 2;
  EpiAcc acc{0.f, -INFINITY, 0x7fffffff};
  if (g.n_slices <= 1) {
    // ---- the unit covers the whole K: epilogue straight from tensor memory
    if (quarter * 32 < g.B) {
      for (int gi = g0; gi < g1; ++gi) {
        uint32_t r[16];
        tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(gi * 16), r);
        if (b >= g.B) continue;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        gemm_epilogue16(g, b, g.n0 + gi * 16, v, acc);
      }
      if (b < g.B) gemm_epilogue_flush(g, b, acc);
    }
    tc_fence_before();
    compute_sync();  // every lane read its columns: the next task may overwrite the accumulator
    if (q.tid == 0 && g.bar != 0xFFFF) red_release_gpu_add(c.bars + g.bar, -1);
    q.free_slots(normw_mask);
    TCS(2);
    return;
  }
  // ---- a K-slice: add the partial sums to the block's fp32 scratch area
  if (quarter * 32 < g.B) {
    for (int gi = g0; gi < g1; ++gi) {
      uint32_t r[16];
      tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(gi * 16), r);
      if (b >= g.B) continue;
      float* dst = g.scratch + (size_t)b * g.N + gi * 16;
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(__uint_as_float(r[j])),
                     "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3]))
                     : "memory");
    }
  }
  tc_fence_before();
  compute_sync();
  TCS(3);
  if (q.tid == 0) {
    // The sums are complete once every unit of the block arrived.  The bump releases this CTA's
    // adds (ordered before it by the CTA barrier; a release is cumulative) and acquires the
    // other units' for the reads of the last arriver.
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(g.counter) : "memory");
    sh->misc[35] = (old == g.n_slices - 1) ? 1.f : 0.f;
  }
  compute_sync();
  q.free_slots(normw_mask);
  TCS(4);
  if (sh->misc[35] == 0.f) return;
  // ---- last arrival for this block: epilogue from the scratch area (read past L1), cleared for its next use
  const int items = g.B * ng;
  for (int item = q.tid; item < items; item += kCT) {
    const int bb = item / ng, gi = item % ng;
    float4* src = reinterpret_cast<float4*>(g.scratch + (size_t)bb * g.N + gi * 16);
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 t = __ldcg(src + j);
      v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) src[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    gemm_epilogue16(g, bb, g.n0 + gi * 16, v, acc);
    gemm_epilogue_flush(g, bb, acc);
  }
  compute_sync();
  if (q.tid == 0) {
    *g.counter = 0;  // ready for the block's next use; ordered before it by the barrier chain
    // the releasing count-down is cumulative: it publishes what the CTA barrier ordered before it
    if (g.bar != 0xFFFF) red_release_gpu_add(c.bars + g.bar, -1);
  }
  TCS(5);
#ifdef VDC_TC_PROFILE
  if (q.tid == 0) c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 106] += 1;
#endif
}

// ------------------------------------------------------------------------- //
// task: embedding rows of this SM's sequences into the k-chunk-major hidden state
// ------------------------------------------------------------------------- //
__device__ void task_embed_pack(Compute& q, int b0, int count, int bpad, int stride_words, int h8, int bar,
                                const int* state, const uint8_t* table, uint8_t* out, float* stats) {
  for (int i = 0; i < count; ++i) {
    const int b = b0 + i;
    const int token = ld_relaxed_gpu(state + (size_t)b * stride_words + VDC_ST_TOKEN);
    const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)token * h8 * 16);
    float ss = 0.f;
    for (int p = q.tid; p < h8; p += kCT) {
      const uint4 v = __ldg(row + p);
      *reinterpret_cast<uint4*>(out + kc_piece(bpad, b, p * 8)) = v;
      const uint32_t xv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) ss = fmaf(bf_lo(xv[j]), bf_lo(xv[j]), fmaf(bf_hi(xv[j]), bf_hi(xv[j]), ss));
    }
    ss = warp_sum(ss);
    if (q.lane == 0) q.sh->misc[q.warp] = ss;
    compute_sync();
    if (q.tid == 0) {
      float t = 0.f;
      for (int w = 0; w < kCW; ++w) t += q.sh->misc[w];
      stats[b] = t;  // sum of squares of the row: the first projection's RMSNorm uses it
    }
    compute_sync();
  }
  __threadfence();
  compute_sync();
  if (q.tid == 0 && bar != 0xFFFF) red_release_gpu_add(q.c.bars + bar, -1);
}

// ------------------------------------------------------------------------- //
// task: next token, token log and state advance of every sequence
// ------------------------------------------------------------------------- //
__device__ void task_batch_advance(Compute& q, int batch, int stride_words, int log_stride, unsigned long long* keys,
                                   int* log, float* stats, int n_stats) {
  q.pop();
  int* state0 = reinterpret_cast<int*>(q.addr());
  if (q.aborted) return;
  if (q.tid < batch) {
    int* state = state0 + (size_t)q.tid * stride_words;
    const unsigned long long key = __ldcg(keys + q.tid);
    const int token = (int)(0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull));
    keys[q.tid] = 0ull;
    const int step = state[VDC_ST_STEP];
    const int pos = state[VDC_ST_POS] + 1;
    log[(size_t)q.tid * log_stride + step] = token;
    state[VDC_ST_TOKEN] = token;
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
  // every consumer of this step's per-sequence sums of squares is done: clear them for the next step
  for (int i = q.tid; i < n_stats; i += kCT) stats[i] = 0.f;
  __threadfence();
  compute_sync();
}

}  // namespace vdc
