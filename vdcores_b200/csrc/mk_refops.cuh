// Compute tasks that honour the tile contracts of the reference's operators, so that instruction
// streams built by its schedules run on this kernel: the same opcodes names, pop orders, shared-memory
// tile layouts (128-byte-swizzled K-major operand tiles, MN-major result tiles) and argument words.
// The arithmetic is B200 CUDA-core code (the reference's is sm_90a WGMMA / mma.sync through CuTe):
//   GEMV tile      reference include/task/gemv.cuh:13-204
//   RMSNorm        reference include/task/rms_norm.cuh:7-133   (statistics here in fp32, there in bf16)
//   RoPE           reference include/task/rope.cuh:142-170
//   SiLU * up      reference include/task/silu.cuh:126-190
//   argmax         reference include/task/argmax.cuh:60-175
#pragma once
#include "mk_compute.cuh"

namespace vdc {

// Byte offset of the 16-byte piece `piece` (0..7) of row `row` inside one 128-byte-swizzled block of
// 128-byte rows: the piece index is XORed with the row index modulo 8.
__device__ __forceinline__ uint32_t sw128(int row, int piece) { return (uint32_t)row * 128u + (uint32_t)((piece ^ (row & 7)) << 4); }

__device__ __forceinline__ void fma_bf16x8(float& acc, const uint4& a, const uint4& b) {
  float lo = 0.f, hi = 0.f;
  fma_bf16x2(lo, hi, a.x, b.x);
  fma_bf16x2(lo, hi, a.y, b.y);
  fma_bf16x2(lo, hi, a.z, b.z);
  fma_bf16x2(lo, hi, a.w, b.w);
  acc += lo + hi;
}

// ------------------------------------------------------------------------- //
// C[64, 8] (+)= sum over k-tiles of A[64, 256] B[8, 256]^T
// ------------------------------------------------------------------------- //
// Pop order: [fp32 C tile, M-contiguous, when `residual`], then per k-tile: the B tile when the tile index
// is a multiple of `bload` (bload sub-tiles of [8 x 256], 4 KB each), the A tile ([64 x 256]: four blocks
// of 64 rows x 128 bytes); last the result slot, written as bf16 MN-major 64 x 8 with 128-byte swizzle
// (row n, piece (m / 8) XOR n) and handed to the store warp.  Thread t owns row t / 4 and the two
// columns 2 (t mod 4), 2 (t mod 4) + 1.
VDC_TASK void task_ref_gemv(Compute& q, int k_tiles, int bload, bool residual) {
  const Ctx& c = q.c;
  const int row = q.tid >> 2, n0 = (q.tid & 3) * 2;
  float acc0 = 0.f, acc1 = 0.f;
  if (residual) {
    const int m = q.pop();
    if (q.aborted) return;
    const float* cin = (const float*)slot_ptr(c, first_slot(m));
    acc0 = cin[n0 * 64 + row];
    acc1 = cin[(n0 + 1) * 64 + row];
    compute_sync();
    q.free_slots(m);
  }
  int b_mask = 0;
  const uint8_t* b_tile = nullptr;
  for (int i = 0; i < k_tiles; ++i) {
    if (i % bload == 0) {
      b_mask = q.pop();
      if (q.aborted) return;
      b_tile = (const uint8_t*)slot_ptr(c, first_slot(b_mask));
    } else {
      b_tile += 8 * 256 * 2;
    }
    const int a_mask = q.pop();
    if (q.aborted) return;
    const uint8_t* a_tile = (const uint8_t*)slot_ptr(c, first_slot(a_mask));
#pragma unroll 4
    for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const uint4 a = lds128(a_tile + kb * (64 * 128) + sw128(row, p));
        const uint4 b0 = lds128(b_tile + kb * (8 * 128) + sw128(n0, p));
        const uint4 b1 = lds128(b_tile + kb * (8 * 128) + sw128(n0 + 1, p));
        fma_bf16x8(acc0, a, b0);
        fma_bf16x8(acc1, a, b1);
      }
    }
    compute_sync();  // every thread is done with the tiles
    q.free_slots(a_mask | ((i % bload == bload - 1 || i == k_tiles - 1) ? b_mask : 0));
  }
  const int c_mask = q.pop();
  if (q.aborted) return;
  uint8_t* out = (uint8_t*)slot_ptr(c, first_slot(c_mask));
  *reinterpret_cast<__nv_bfloat16*>(out + sw128(n0, row >> 3) + (row & 7) * 2) = __float2bfloat16_rn(acc0);
  *reinterpret_cast<__nv_bfloat16*>(out + sw128(n0 + 1, row >> 3) + (row & 7) * 2) = __float2bfloat16_rn(acc1);
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(c_mask);
}

// ------------------------------------------------------------------------- //
// RMSNorm of `num_token` rows of K bf16 in shared memory
// ------------------------------------------------------------------------- //
// Pop order: weight row, input rows, output rows.  y = bf16(bf16(x * rstd) * w), rstd from fp32 statistics;
// eps arrives as a bf16 bit pattern.
VDC_TASK void task_ref_rms(Compute& q, int K, int num_token, uint32_t eps_bf16) {
  const Ctx& c = q.c;
  Shared* sh = q.sh;
  const int w_mask = q.pop();
  const int in_mask = q.pop();
  const int out_mask = q.pop();
  if (q.aborted) return;
  const uint32_t* w = (const uint32_t*)slot_ptr(c, first_slot(w_mask));
  const uint32_t* in = (const uint32_t*)slot_ptr(c, first_slot(in_mask));
  uint32_t* out = (uint32_t*)slot_ptr(c, first_slot(out_mask));
  const float eps = __uint_as_float(eps_bf16 << 16);
  for (int t = 0; t < num_token; ++t) {
    const uint32_t* x = in + t * (K / 2);
    float ss = 0.f;
    for (int i = q.tid; i < K / 2; i += kCT) ss += bf_lo(x[i]) * bf_lo(x[i]) + bf_hi(x[i]) * bf_hi(x[i]);
    ss = warp_sum(ss);
    if (q.lane == 0) sh->misc[q.warp] = ss;
    compute_sync();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < kCW; ++k) tot += sh->misc[k];
    const float rstd = rsqrtf(tot / (float)K + eps);
    for (int i = q.tid; i < K / 2; i += kCT) {
      const float a = bf16_round(bf16_round(bf_lo(x[i]) * rstd) * bf_lo(w[i]));
      const float b = bf16_round(bf16_round(bf_hi(x[i]) * rstd) * bf_hi(w[i]));
      out[t * (K / 2) + i] = (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xffff0000u);
    }
    compute_sync();
  }
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(out_mask);
  q.free_slots(in_mask | w_mask);
}

// ------------------------------------------------------------------------- //
// interleaved RoPE on 512 bf16: (x_even + i x_odd) * (cos + i sin), pair by pair
// ------------------------------------------------------------------------- //
// Pop order: table (cos, sin pairs), input, output; all three in the same tile layout, so the product
// is element-wise over 256 pairs.
VDC_TASK void task_ref_rope512(Compute& q) {
  const Ctx& c = q.c;
  const int t_mask = q.pop();
  const int in_mask = q.pop();
  const int out_mask = q.pop();
  if (q.aborted) return;
  const __nv_bfloat162* tbl = (const __nv_bfloat162*)slot_ptr(c, first_slot(t_mask));
  const __nv_bfloat162* in = (const __nv_bfloat162*)slot_ptr(c, first_slot(in_mask));
  __nv_bfloat162* out = (__nv_bfloat162*)slot_ptr(c, first_slot(out_mask));
  if (q.tid < 256) out[q.tid] = __hcmadd(in[q.tid], tbl[q.tid], __floats2bfloat162_rn(0.f, 0.f));
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(out_mask);
  q.free_slots(in_mask | t_mask);
}

// ------------------------------------------------------------------------- //
// silu(gate) * up over n_pairs bf16 pairs (same layout for all three operands)
// ------------------------------------------------------------------------- //
// Pop order: output, gate, up.
VDC_TASK void task_ref_silu(Compute& q, int n_pairs) {
  const Ctx& c = q.c;
  const int out_mask = q.pop();
  const int g_mask = q.pop();
  const int u_mask = q.pop();
  if (q.aborted) return;
  uint32_t* out = (uint32_t*)slot_ptr(c, first_slot(out_mask));
  const uint32_t* g = (const uint32_t*)slot_ptr(c, first_slot(g_mask));
  const uint32_t* u = (const uint32_t*)slot_ptr(c, first_slot(u_mask));
  for (int i = q.tid; i < n_pairs; i += kCT) {
    const float g0 = bf_lo(g[i]), g1 = bf_hi(g[i]);
    const float a = (g0 / (1.0f + expf(-g0))) * bf_lo(u[i]);
    const float b = (g1 / (1.0f + expf(-g1))) * bf_hi(u[i]);
    const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    out[i] = *reinterpret_cast<const uint32_t*>(&r);
  }
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(out_mask);
  q.free_slots(g_mask | u_mask);
}

// ------------------------------------------------------------------------- //
// greedy argmax in two steps through global memory
// ------------------------------------------------------------------------- //
// CTA-wide (value, index) maximum in bf16 ordering; strict comparisons, the first maximum a thread meets wins.
__device__ __forceinline__ void ref_block_argmax(Compute& q, float& val, long long& idx) {
  Shared* sh = q.sh;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_down_sync(0xffffffffu, val, o);
    const long long oi = __shfl_down_sync(0xffffffffu, idx, o);
    if (ov > val) {
      val = ov;
      idx = oi;
    }
  }
  long long* sidx = reinterpret_cast<long long*>(sh->red);
  float* sval = sh->red + 2 * kCW;
  if (q.lane == 0) {
    sval[q.warp] = val;
    sidx[q.warp] = idx;
  }
  compute_sync();
  if (q.tid == 0) {
    float bv = -3.4e38f;
    long long bi = -1;
    for (int w = 0; w < kCW; ++w)
      if (sval[w] > bv) {
        bv = sval[w];
        bi = sidx[w];
      }
    val = bv;
    idx = bi;
  }
  compute_sync();
}

// Partial: pops three raw addresses — this SM's chunk of the logits (token b at + b * i_stride elements), its
// (value bf16, index int64) outputs (token b at + b * o_stride).
VDC_TASK void task_ref_argmax_partial(Compute& q, int chunk, int i_stride, int o_stride, int n_tokens) {
  q.pop();
  const uint32_t* in = reinterpret_cast<const uint32_t*>(q.addr());
  q.pop();
  __nv_bfloat16* oval = reinterpret_cast<__nv_bfloat16*>(q.addr());
  const uint32_t val_meta = q.meta();
  q.pop();
  long long* oidx = reinterpret_cast<long long*>(q.addr());
  const uint32_t idx_meta = q.meta();
  if (q.aborted) return;
  for (int b = 0; b < n_tokens; ++b) {
    float best = -3.4e38f;
    long long bi = -1;
    for (int i = q.tid; i < chunk / 2; i += kCT) {
      const uint32_t v = ldcg32(in + i + b * (i_stride / 2));
      if (bf_lo(v) > best) {
        best = bf_lo(v);
        bi = 2 * i;
      }
      if (bf_hi(v) > best) {
        best = bf_hi(v);
        bi = 2 * i + 1;
      }
    }
    ref_block_argmax(q, best, bi);
    if (q.tid == 0) {
      oval[b * o_stride] = __float2bfloat16_rn(best);
      oidx[b * o_stride] = bi;
      __threadfence();
    }
  }
  compute_sync();
  q.release(val_meta);
  q.release(idx_meta);
}

// Reduce: pops the partial values / indices of one token (n_partial each) and the final output (int64):
// final = winning chunk * chunk size + index inside the chunk.
VDC_TASK void task_ref_argmax_reduce(Compute& q, int chunk, int n_partial, int n_tokens) {
  q.pop();
  const __nv_bfloat16* pval = reinterpret_cast<const __nv_bfloat16*>(q.addr());
  q.pop();
  const long long* pidx = reinterpret_cast<const long long*>(q.addr());
  q.pop();
  long long* fin = reinterpret_cast<long long*>(q.addr());
  const uint32_t fin_meta = q.meta();
  if (q.aborted) return;
  for (int b = 0; b < n_tokens; ++b) {
    float best = -3.4e38f;
    long long packed = -1;
    for (int i = q.tid; i < n_partial; i += kCT) {
      const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(pval) + i + b * n_partial);
      const float v = __uint_as_float((uint32_t)raw << 16);
      if (v > best) {
        best = v;
        packed = ((long long)i << 32) | __ldcg(pidx + i + b * n_partial);
      }
    }
    ref_block_argmax(q, best, packed);
    if (q.tid == 0) {
      fin[b] = packed != -1 ? (packed >> 32) * chunk + (packed & 0xFFFFFFFFll) : -1;
      __threadfence();
    }
  }
  compute_sync();
  q.release(fin_meta);
}

}  // namespace vdc
