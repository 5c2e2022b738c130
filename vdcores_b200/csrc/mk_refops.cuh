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

// ------------------------------------------------------------------------- //
// Decode attention on the reference's tiles (reference include/task/attention.cuh:673-932, 934-1036)
// ------------------------------------------------------------------------- //
// Tiles as the reference's tensor maps deliver them (128-byte swizzle, 64-element = 128-byte rows):
//   Q  [64 rows x 128] K-major: two blocks of 64 rows x 128 bytes (dims 0..63 | 64..127); the plain op's rows all
//      hold the one query head, the split op's row r holds head r mod 4 of the KV head's group;
//   K  [64 positions x 128] K-major, same shape;   V  [64 positions x 128] MN-major: per 8 positions two 1 KB
//      atoms (dims 0..63 | 64..127), each 8 rows of 128 bytes;
//   O  [64 x 128] bf16 row-major (16 KB), of which the write-back copies the first rows.
// Pop order: [side input (q-norm weight | k-norm weight | rope row of cos/sin pairs, 3 x 128 bf16), k-store
// row (128 bf16, written back)] when the fused norm/rope flags are set; Q; per block K then V; O; [split: the
// raw address of the log-sum-exp table, fp32 [row][16 splits], counted down after the write].
// The arithmetic is the tensor-core page loop of the native attention task: a warp owns 8 of a block's 64
// positions, rows 0..7 of the MMA's A operand are the live query rows.
__device__ __forceinline__ uint32_t ktile_off(int row, int piece) {   // piece: 16-byte piece 0..15 of a 256-byte logical row
  return (uint32_t)(piece >> 3) * 8192u + sw128(row, piece & 7);
}

// RMS-norm (weight w) and interleaved RoPE (pairs (2i, 2i+1) rotated by the row's (cos, sin) pairs) of one
// 128-element row of a K-major tile, in place, by one warp; one rounding at the end, as the reference does.
__device__ __forceinline__ void ref_norm_rope_row(uint8_t* tile, int row, const uint32_t* w, const uint32_t* rope, bool need_norm,
                                                  bool need_rope, int lane, uint32_t* copy_to) {
  uint32_t v[2];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = lane + 32 * k;   // pair index: dims 2i, 2i+1
    v[k] = *reinterpret_cast<const uint32_t*>(tile + ktile_off(row, i >> 2) + (i & 3) * 4);
    ss += bf_lo(v[k]) * bf_lo(v[k]) + bf_hi(v[k]) * bf_hi(v[k]);
  }
  ss = warp_sum(ss);
  const float rcp = need_norm ? rsqrtf(ss / 128.f + 1.0e-6f) : 1.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = lane + 32 * k;
    float x = bf_lo(v[k]), y = bf_hi(v[k]);
    if (need_norm) {
      x *= rcp * bf_lo(w[i]);
      y *= rcp * bf_hi(w[i]);
    }
    if (need_rope) {
      const float cs = bf_lo(rope[i]), sn = bf_hi(rope[i]);
      const float e = x * cs - y * sn, o = x * sn + y * cs;
      x = e;
      y = o;
    }
    const uint32_t out = pack_bf16x2(x, y);
    *reinterpret_cast<uint32_t*>(tile + ktile_off(row, i >> 2) + (i & 3) * 4) = out;
    if (copy_to != nullptr) copy_to[i] = out;
  }
}

VDC_TASK void task_ref_attn_decode(Compute& q, int num_kv_blocks, int last_len, int flags, bool split, int split_idx,
                                   int num_active_q) {
  constexpr int D = 128;
  const Ctx& c = q.c;
  Shared* sh = q.sh;
  const bool need_norm = flags & 1, need_rope = flags & 2, fused = (flags & 3) != 0;
  const int n_q = split ? num_active_q : 1;
  int side_mask = 0, kst_mask = 0;
  const uint32_t* side = nullptr;
  uint32_t* kstore = nullptr;
  if (fused) {
    side_mask = q.pop();
    kst_mask = q.pop();
    if (q.aborted) return;
    side = (const uint32_t*)slot_ptr(c, first_slot(side_mask));
    kstore = (uint32_t*)slot_ptr(c, first_slot(kst_mask));
  }
  const int q_mask = q.pop();
  if (q.aborted) return;
  uint8_t* qt = (uint8_t*)slot_ptr(c, first_slot(q_mask));
  if (fused) {
    if (q.warp == 0) ref_norm_rope_row(qt, 0, side, side + 128, need_norm, need_rope, q.lane, nullptr);
    compute_sync();
  }
  const int gid = q.lane >> 2, t4 = q.lane & 3, lrow = q.lane & 7, lmi = q.lane >> 3;
  const int slice = q.warp * 8;
  uint32_t qa[8][2];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qa[ks][0] = gid < n_q ? *reinterpret_cast<const uint32_t*>(qt + ktile_off(gid, 2 * ks) + 4 * t4) : 0u;
    qa[ks][1] = gid < n_q ? *reinterpret_cast<const uint32_t*>(qt + ktile_off(gid, 2 * ks + 1) + 4 * t4) : 0u;
  }
  const float scale_log2 = 1.4426950408889634f * rsqrtf((float)D);
  float m_run = -INFINITY, l_run = 0.f, acc[16][2], z0 = 0.f, z1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = 0.f;
  for (int blk = 0; blk < num_kv_blocks; ++blk) {
    const int k_mask = q.pop();
    if (q.aborted) return;
    uint8_t* kt = (uint8_t*)slot_ptr(c, first_slot(k_mask));
    const bool last = blk == num_kv_blocks - 1;
    if (fused && last && last_len > 0) {
      // the newest position's key row arrives raw: normalise, rotate, and hand the finished row to the cache store
      if (q.warp == 0) ref_norm_rope_row(kt, last_len - 1, side + 64, side + 128, need_norm, need_rope, q.lane, kstore);
      compute_sync();
    }
    const int p_l = slice + lrow;
    const uint32_t kb_s = (uint32_t)__cvta_generic_to_shared(kt);
    float s0 = 0.f, s1 = 0.f, u0 = 0.f, u1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t kr[4];
      ldsm_x4(kr, kb_s + ktile_off(p_l, 4 * j + lmi));
      mma_rows8(s0, s1, z0, z1, qa[2 * j][0], qa[2 * j][1], kr[0], kr[1]);
      mma_rows8(u0, u1, z0, z1, qa[2 * j + 1][0], qa[2 * j + 1][1], kr[2], kr[3]);
    }
    s0 += u0;
    s1 += u1;
    const int valid = last ? last_len : 64;
    const int p0 = slice + 2 * t4;
    s0 = p0 < valid ? s0 * scale_log2 : -INFINITY;
    s1 = p0 + 1 < valid ? s1 * scale_log2 : -INFINITY;
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
    const uint32_t pa = pack_bf16x2(e0, e1);   // probabilities as bf16, like the reference's P tile
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      acc[nt][0] *= alpha;
      acc[nt][1] *= alpha;
    }
    const int v_mask = q.pop();
    if (q.aborted) return;
    const uint32_t vb_s = (uint32_t)__cvta_generic_to_shared(slot_ptr(c, first_slot(v_mask)));
    // MN-major: positions 8w..8w+7 are the two 1 KB atoms number 2w (dims 0..63) and 2w + 1 (dims 64..127)
    const uint32_t v_row = vb_s + (uint32_t)q.warp * 2048u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t vr[4];
      const int piece = 4 * j + lmi;
      ldsm_x4_trans(vr, v_row + (uint32_t)(piece >> 3) * 1024u + sw128(lrow, piece & 7));
#pragma unroll
      for (int mi = 0; mi < 4; ++mi) mma_rows8(acc[4 * j + mi][0], acc[4 * j + mi][1], z0, z1, pa, 0u, vr[mi], 0u);
    }
    compute_sync();  // every warp is done with the block's tiles
    q.free_slots(k_mask | v_mask);
  }
  q.free_slots(q_mask | side_mask);
  // the warps' states meet in shared memory (four query rows per pass), the finished rows go to the O tile
  const int o_mask = q.pop();
  if (q.aborted) return;
  __nv_bfloat16* ot = (__nv_bfloat16*)slot_ptr(c, first_slot(o_mask));
  float* red = sh->red;
  float* ml = red + kCW * 4 * D;
  for (int pass = 0; pass * 4 < n_q; ++pass) {
    if (pass > 0) compute_sync();
    if ((gid >> 2) == pass) {
      float* dst = red + (q.warp * 4 + (gid & 3)) * D + 2 * t4;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2*>(dst + 8 * nt) = make_float2(acc[nt][0], acc[nt][1]);
      if (t4 == 0) {
        ml[q.warp * 8 + (gid & 3)] = m_run;
        ml[q.warp * 8 + 4 + (gid & 3)] = l_run;
      }
    }
    compute_sync();
    for (int o = q.tid; o < 4 * D; o += kCT) {
      const int gg = o / D, d = o % D, g = pass * 4 + gg;
      if (g >= n_q) break;
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
      ot[g * D + d] = __float2bfloat16_rn(l == 0.f ? num : num / l);
      if (d == 0) {   // kept for the split table below
        sh->misc[16 + g] = m;
        sh->misc[24 + g] = l;
      }
    }
  }
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(o_mask);
  if (fused) q.push_store(kst_mask);
  if (split) {
    q.pop();
    float* lse = reinterpret_cast<float*>(q.addr());
    const uint32_t lse_meta = q.meta();
    if (q.aborted) return;
    if (q.tid < n_q) {
      lse[q.tid * 16 + split_idx] = sh->misc[16 + q.tid] + log2f(sh->misc[24 + q.tid]);
      __threadfence();
    }
    compute_sync();
    q.release(lse_meta);
  }
}

// Pops the log-sum-exp table (raw address behind the barrier the splits count down), the splits' outputs
// ([split][4 rows][128] bf16 in one tile) and the final [4 x 128] bf16 tile:
// out = sum_s 2^(lse_s - max) O_s / sum_s 2^(lse_s - max).
VDC_TASK void task_ref_attn_post_reduce(Compute& q, int num_split) {
  const Ctx& c = q.c;
  q.pop();
  const float* lse = reinterpret_cast<const float*>(q.addr());
  if (q.aborted) return;
  const int row = q.tid >> 6, i = q.tid & 63;      // 4 rows x 64 pairs = 256 threads
  float w[16], tot = 0.f, mx = -INFINITY;
  for (int s = 0; s < num_split; ++s) {
    w[s & 15] = __ldcg(lse + row * 16 + s);
    mx = fmaxf(mx, w[s & 15]);
  }
  for (int s = 0; s < num_split; ++s) {
    w[s & 15] = exp2f(w[s & 15] - mx);
    tot += w[s & 15];
  }
  const int in_mask = q.pop();
  if (q.aborted) return;
  const uint32_t* so = (const uint32_t*)slot_ptr(c, first_slot(in_mask));
  float ax = 0.f, ay = 0.f;
  for (int s = 0; s < num_split; ++s) {
    const uint32_t v = so[(s * 4 + row) * 64 + i];
    ax = fmaf(bf_lo(v), w[s & 15], ax);
    ay = fmaf(bf_hi(v), w[s & 15], ay);
  }
  compute_sync();
  q.free_slots(in_mask);
  const int out_mask = q.pop();
  if (q.aborted) return;
  uint32_t* out = (uint32_t*)slot_ptr(c, first_slot(out_mask));
  out[row * 64 + i] = pack_bf16x2(ax / tot, ay / tot);
  fence_proxy_async_smem();
  compute_sync();
  q.push_store(out_mask);
}

}  // namespace vdc
