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

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
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
struct GemmTc {
  int n_chunks, N, KS, mode;
  bool norm;
  float eps;
  int B, Bpad;
  uint8_t* out;
  unsigned long long* keys;
  float* stats;  // fp32 per sequence: sum of squares of the input rows (norm) / of the updated rows (ADD_PACKED)
  int n0, ld, bar;
};

__device__ void task_gemm_tc(Compute& q, const GemmTc& g) {
  Shared* sh = q.sh;
  const Ctx& c = q.c;
  // Tensor memory is taken the first time a program needs it and given back when the kernel ends.
  if (!sh->tmem_ready) {
    if (q.warp == 0) tmem_alloc(&sh->tmem_base, kTmemCols);
    if (q.tid >= 32 && q.tid < 36) mbar_init(&sh->mma_bar[q.tid - 32], 1);
    if (q.tid == 36) mbar_init(&sh->mma_final, 1);
    if (q.tid >= 64 && q.tid < 80) mbar_init(&sh->x_ready[q.tid - 64], 1);
    if (q.tid >= 32 && q.tid < 80) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    compute_sync();
    tc_fence_after();
    if (q.tid == 0) sh->tmem_ready = 1;
  }
  int normw_mask = 0;
  if (g.norm) normw_mask = q.pop();
  if (q.aborted) return;
  const uint8_t* nw = g.norm ? (const uint8_t*)slot_ptr(c, first_slot(normw_mask)) : nullptr;
  const uint32_t tmem = sh->tmem_base;
  const uint32_t idesc = umma_idesc_bf16_m128(g.N);
  const uint32_t lbo_a = (uint32_t)g.Bpad * 16u, lbo_b = (uint32_t)g.N * 16u;
  const int pieces = g.KS * 2 * g.Bpad;  // 16-byte pieces of one X chunk
  const int K = g.n_chunks * g.KS * 16;
  const unsigned n_ent = 2u * (unsigned)g.n_chunks;  // ring entries of this task: X chunk, W chunk, X chunk, ...

  // The streaming loop has no CTA-wide synchronisation.  Warp 0 consumes the ring entries in
  // order: it waits for a chunk pair, one lane issues the tensor-core work and, once the
  // previous pair's reads are done, recycles that pair's slots and ring entries.  With norm
  // the other seven warps run ahead of it, each normalising every seventh X chunk in place
  // and signalling that chunk's barrier.
  q.warp_phase_begin(n_ent, q.warp == 0 ? 0u : n_ent);
  if (q.warp > 0 && g.norm) {
    float* rs = sh->red + q.warp * 128;  // this warp's copy of the per-sequence rsqrt(mean x^2 + eps)
    bool have_rstd = false;
    for (int ch = q.warp - 1; ch < g.n_chunks; ch += kCW - 1) {
      const int xm = q.warp_wait(2u * (unsigned)ch);
      if (xm == kPopAbort) break;
      if (!have_rstd) {
        // Any X chunk of this task was loaded after the producers of the input matrix had
        // finished, and with them the sums of squares they left (read past L1).
        for (int bb = q.lane; bb < g.Bpad; bb += 32) rs[bb] = rsqrtf(__ldcg(g.stats + bb) / (float)K + g.eps);
        __syncwarp();
        have_rstd = true;
      }
      uint8_t* xs = (uint8_t*)slot_ptr(c, first_slot(xm));
      const int kc0 = ch * g.KS * 2;  // index of the chunk's first 8-element k group
      // RMSNorm in place, rounded like a bf16 tensor expression: bf16(w * bf16(x * rstd))
      for (int p = q.lane; p < pieces; p += 32) {
        const uint4 v = lds128(xs + p * 16);
        const uint4 w = lds128(nw + (kc0 + p / g.Bpad) * 16);
        const float rstd = rs[p & (g.Bpad - 1)];
        const uint32_t xv[4] = {v.x, v.y, v.z, v.w}, wv[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o[j] = pack_bf16x2(bf16_round(bf_lo(xv[j]) * rstd) * bf_lo(wv[j]), bf16_round(bf_hi(xv[j]) * rstd) * bf_hi(wv[j]));
        *reinterpret_cast<uint4*>(xs + p * 16) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();  // the tensor cores read shared memory through the async proxy
      __syncwarp();
      if (q.lane == 0) mbar_arrive(&sh->x_ready[(q.xr_count + (unsigned)ch) & 15u]);
    }
  }
  if (q.warp == 0) {
    int prev_masks = 0;  // lane 0: slots of the chunk pair whose tensor-core reads are in flight
#ifdef VDC_TC_PROFILE
    long long t_data = 0, t_xr = 0, t_mma = 0, t_wait = 0;
#endif
    for (int ch = 0; ch < g.n_chunks; ++ch) {
#ifdef VDC_TC_PROFILE
      const long long td0 = clock64();
#endif
      const int xm = q.warp_wait(2u * (unsigned)ch);
      const int wm = q.warp_wait(2u * (unsigned)ch + 1u);
      if (xm == kPopAbort || wm == kPopAbort) break;
#ifdef VDC_TC_PROFILE
      t_data += clock64() - td0;
      const long long tx0 = clock64();
#endif
      if (g.norm) {
        int ok = 1;
        if (q.lane == 0) {
          const unsigned gch = q.xr_count + (unsigned)ch;
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
        uint64_t adesc = umma_desc(smem_u32(slot_ptr(c, first_slot(xm))), lbo_a, 128u);
        uint64_t bdesc = umma_desc(smem_u32(slot_ptr(c, first_slot(wm))), lbo_b, 128u);
        const uint64_t step_a = (uint64_t)((2u * lbo_a) >> 4), step_b = (uint64_t)((2u * lbo_b) >> 4);
        umma_bf16(tmem, adesc, bdesc, idesc, (uint32_t)(ch != 0));
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
        // the previous pair's reads are certainly done once its commit arrived
        if (ch > 0) {
          if (!mma_wait(q, q.mma_count - 1)) prev_masks = 0;
          if (prev_masks) atomicOr(&sh->slot_avail, (uint32_t)prev_masks & kSlotMaskAll);
          sh->warp_next[0] = q.head + 2u * (unsigned)ch;  // its ring entries may be recycled too
        }
        prev_masks = (xm | wm) & (int)kSlotMaskAll;
        q.mma_count++;
#ifdef VDC_TC_PROFILE
        t_wait += clock64() - tw0;
#endif
      }
      __syncwarp();
    }
    if (q.lane == 0) {
      if (q.mma_count > 0 && mma_wait(q, q.mma_count - 1) && prev_masks)
        atomicOr(&sh->slot_avail, (uint32_t)prev_masks & kSlotMaskAll);
      sh->warp_next[0] = 0xFFFFFFFFu;
#ifdef VDC_TC_PROFILE
      uint64_t* pr = c.profile + c.sm * VDC_NUM_PROFILE_EVENTS;
      pr[8] += t_data; pr[9] += t_xr; pr[10] += t_mma; pr[11] += t_wait; pr[12] += g.n_chunks;
      pr[13] += (uint64_t)g.n_chunks * g.KS;
#endif
    }
  }
  tc_fence_before();
  q.warp_phase_end(n_ent);  // CTA barrier: accumulator complete (lane 0 saw the last commit)
  tc_fence_after();
  if (g.norm) q.xr_count += (unsigned)g.n_chunks;
  if (q.aborted) return;

  // ---- epilogue: lane b of the accumulator belongs to sequence b; warps w and w+4 share the
  // lane quarter w % 4 and split the columns
  const int quarter = q.warp & 3, half = q.warp >> 2;
  const int b = quarter * 32 + q.lane;
  if (quarter * 32 < g.B) {
    float ssq = 0.f;  // ADD_PACKED: squares of the rows' new values over this thread's columns
    const int ng = g.N >> 4;
    const int g0 = half ? (ng + 1) / 2 : 0, g1 = half ? ng : (ng + 1) / 2;
    float best = -INFINITY;
    int best_row = 0x7fffffff;
    for (int gi = g0; gi < g1; ++gi) {
      uint32_t r[16];
      tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(gi * 16), r);
      if (b >= g.B) continue;
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
      const int row = g.n0 + gi * 16;  // first of the 16 output rows in v
      if (g.mode == VDC_GEMM_MODE_STORE_ROWS) {
        uint4* dst = reinterpret_cast<uint4*>(g.out + ((size_t)b * g.ld + row) * 2);
        dst[0] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                            pack_bf16x2(v[6], v[7]));
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
            ssq = fmaf(nv.x, nv.x, fmaf(nv.y, nv.y, ssq));
          }
        }
      } else {  // ARGMAX over bf16-rounded logits, the lowest row wins ties
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float l = bf16_round(v[j]);
          if (l > best) {
            best = l;
            best_row = row + j;
          }
        }
      }
    }
    if (g.mode == VDC_GEMM_MODE_ARGMAX && b < g.B && best_row != 0x7fffffff) {
      uint32_t u = __float_as_uint(best);
      u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // order-preserving map of the float
      atomicMax(g.keys + b, ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)best_row));
    }
    if (g.mode == VDC_GEMM_MODE_ADD_PACKED && g.stats != nullptr && b < g.B) atomicAdd(g.stats + b, ssq);
    __threadfence();
  }
  tc_fence_before();
  compute_sync();  // every lane read its columns: the next task may overwrite the accumulator
  if (q.tid == 0 && g.bar != 0xFFFF) red_release_gpu_add(c.bars + g.bar, -1);
  q.free_slots(normw_mask);
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
