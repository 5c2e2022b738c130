// Persistent decode megakernel for sm_100a: dispatch loop, kernel entry, host launch.
#include "mk_common.cuh"
#include "mk_memory.cuh"
#include "mk_compute.cuh"
#include "mk_tensor.cuh"
#include "mk_refops.cuh"

namespace vdc {

// The two trailing words of a task that writes to every rank's exchange block.
#define VDC_LOAD_PEERS(dst)                                                                             \
  {                                                                                                     \
    VdcCInst p0, p1;                                                                                    \
    *reinterpret_cast<uint2*>(&p0) = ld_word(q.pc);                                                     \
    *reinterpret_cast<uint2*>(&p1) = ld_word(q.pc + 1);                                                 \
    q.pc += 2;                                                                                          \
    (dst).table = reinterpret_cast<const unsigned long long*>(                                          \
        (uint64_t)p0.args[0] | ((uint64_t)p0.args[1] << 16) | ((uint64_t)p0.args[2] << 32));            \
    (dst).n = p1.args[0];                                                                               \
    (dst).ex = (uint32_t)p1.args[1] | ((uint32_t)p1.args[2] << 16);                                     \
  }

// ------------------------------------------------------------------------- //
// compute virtual core: dispatch
// ------------------------------------------------------------------------- //
// Words an instruction occupies before its optional trailing words: the one table in isa.h
// that the host-side emitters read too.
__device__ __forceinline__ int compute_op_words(uint16_t op) {
  switch (op) {
#define X(name, value, words) \
  case value:                 \
    return words;
    VDC_COMPUTE_OPS(X)
#undef X
    default:
      return 1;
  }
}

// The reference's operators (tile contracts of its schedules).  They are compiled into the full kernel only
// (vdc_launch, the entry point behind the reference's launch_dae); the kernel the native decode engines launch
// leaves them out: measured on B200, their presence in the dispatcher costs the batch-1 step 1.8 %.
__device__ __forceinline__ bool dispatch_ref_op(Compute& q, const VdcCInst& ci) {
  switch (ci.opcode) {
      case 0x7400: case 0x7401: task_ref_gemv(q, ci.args[0], 4, ci.opcode & 1); break;
      case 0x7402: case 0x7403: task_ref_gemv(q, ci.args[0], 2, ci.opcode & 1); break;
      case 0x7404: case 0x7405: task_ref_gemv(q, ci.args[0], 1, ci.opcode & 1); break;
      case 0x7408: task_ref_gemv(q, ci.args[0], 1, false); break;
      case 0x7410: task_ref_rms(q, 4096, ci.args[0], ci.args[1]); break;
      case 0x7411: task_ref_rms(q, 2048, ci.args[0], ci.args[1]); break;
      case 0x7412: task_ref_rms(q, 5120, ci.args[0], ci.args[1]); break;
      case 0x7413: task_ref_rms(q, 128, ci.args[0], ci.args[1]); break;
      case 0x7418: task_ref_rope512(q); break;
      case 0x7420: task_ref_silu(q, 32 * 8); break;                  // one 64 x 8 tile, whatever the token count
      case 0x7421: task_ref_silu(q, 6144 / 2 * ci.args[0]); break;
      case 0x7428: task_ref_argmax_partial(q, 1024, 65536, 128, ci.args[0]); break;
      case 0x7429: task_ref_argmax_reduce(q, 1024, 128, ci.args[0]); break;
      case 0x742A: task_ref_argmax_partial(q, 1152, 50688, 132, ci.args[0]); break;
      case 0x742B: task_ref_argmax_reduce(q, 1152, 132, ci.args[0]); break;
      case 0x7430: case 0x7431: task_ref_attn_decode(q, ci.args[0], ci.args[1], ci.args[2], false, 0, 1); break;
      case 0x7432: case 0x7433:   // [blocks | split << 12, active rows | last length << 8, first position]
        task_ref_attn_decode(q, ci.args[0] & 0xFFF, ci.args[1] >> 8, 0, true, ci.args[0] >> 12, ci.args[1] & 0xFF);
        break;
      case 0x7434: task_ref_attn_post_reduce(q, ci.args[0]); break;
      default: return false;
  }
  return true;
}

template <bool kRefOps>
__device__ __forceinline__ void compute_core(const Ctx& c, const VdcCInst* __restrict__ insts, int n_insts, int tid) {
  Compute q{c, c.sh, tid, tid >> 5, tid & 31, 0u, 0u, 0u, false, 0ull};
  uint32_t count = 0;
  int n_traced = 0;
  bool finish = false;
  // The next two instruction words are always in registers: their loads were
  // issued before the previous task started, so a task never begins by waiting
  // on an L2 round trip for its own instruction.
  auto ld_word = [&](uint32_t at) { return __ldg(reinterpret_cast<const uint2*>(insts + (at % (uint32_t)n_insts))); };
  uint2 w0 = ld_word(0), w1 = ld_word(1);
  uint32_t w_pc = 0;  // instruction index of w0
  while (!finish && !q.aborted) {
    if (w_pc != q.pc) {  // a LOOPC jump: refill
      w0 = ld_word(q.pc);
      w1 = ld_word(q.pc + 1);
      w_pc = q.pc;
    }
    VdcCInst ci, ex;
    *reinterpret_cast<uint2*>(&ci) = w0;
    *reinterpret_cast<uint2*>(&ex) = w1;
    const bool two_words = compute_op_words(ci.opcode) >= 2;
    q.pc += two_words ? 2 : 1;
    if (two_words) {
      w0 = ld_word(q.pc);
      w1 = ld_word(q.pc + 1);
    } else {
      w0 = w1;
      w1 = ld_word(q.pc + 1);
    }
    w_pc = q.pc;
    // task trace: (start, end) global-timer stamps of the first 56 tasks of this SM
#ifdef VDC_TRACE_GEMV
    const bool traced = tid == 0 && n_traced < 24 && ci.opcode != 0x7000;   // rows 64..127 hold the GEMV stamps
#else
    const bool traced = tid == 0 && n_traced < 56 && ci.opcode != 0x7000;
#endif
    if (traced) c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 16 + 2 * n_traced] = globaltimer_ns();
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
          if (ci.args[1]) __nanosleep(ci.args[1]);
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
      case 0x7200:    // GEMV_ROWS_BF16 (two words)
      case 0x7201:    // GEMV_ROWS_FP8 (three words: + address of the per-row scales)
      case 0x7202:    // GEMV_ROWS_NVFP4 (three words, likewise)
      case 0x7203: {  // GEMV_ROWS_MOE_DOWN (five words: + routing weight, accumulators, counters)
        const int R = ci.args[1] & 31, mode = (ci.args[1] >> 8) & 7;
        const bool accumulate = ci.args[1] & VDC_GEMV_ACC_BIT;
        const bool norm = ci.args[1] & VDC_GEMV_NORM_BIT;
        const bool dyn = ci.args[1] & VDC_GEMV_DYN_BIT;
        const bool to_peers = ci.args[1] & VDC_GEMV_PEERS_BIT;
        const int K = (ci.args[2] & 0xFF) << 8;
        if (tid == 0) q.sh->misc[32] = __uint_as_float(((uint32_t)ex.args[0] << 16) | ex.args[1]);  // norm eps
        const int row_base = ((int)ex.args[2] | ((int)(ci.args[2] >> 8) << 16)) * R;  // first output row (argmax)
        const float* scales = nullptr;
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        MoeDown moe_args;
        const MoeDown* moe = nullptr;
        if (ci.opcode == 0x7203) {
          VdcCInst e2, e3, e4;
          *reinterpret_cast<uint2*>(&e2) = ld_word(q.pc);
          *reinterpret_cast<uint2*>(&e3) = ld_word(q.pc + 1);
          *reinterpret_cast<uint2*>(&e4) = ld_word(q.pc + 2);
          q.pc += 3;
          moe_args.weight = reinterpret_cast<const float*>(addr48(e2));
          moe_args.acc = reinterpret_cast<float*>(addr48(e3));
          moe_args.cnt = reinterpret_cast<int*>(addr48(e4));
          moe_args.top_k = ex.args[2];
          moe = &moe_args;
        }
        const int wfmt = ci.opcode == 0x7203 ? 0 : ci.opcode - 0x7200;
        if (wfmt != 0) {
          VdcCInst e2;
          *reinterpret_cast<uint2*>(&e2) = ld_word(q.pc);
          q.pc += 1;
          scales = reinterpret_cast<const float*>((uint64_t)e2.args[0] | ((uint64_t)e2.args[1] << 16) |
                                                  ((uint64_t)e2.args[2] << 32));
        }
        int chunk_stride = 1;
        if (ci.args[1] & VDC_GEMV_STRIDE_BIT) {
          VdcCInst e2;
          *reinterpret_cast<uint2*>(&e2) = ld_word(q.pc);
          q.pc += 1;
          chunk_stride = e2.args[0];
        }
        const float* partial = nullptr;   // fp32 sums over another K-range of the same rows (a projection in two passes)
        if (ci.args[1] & VDC_GEMV_PARTIAL_BIT) {
          VdcCInst e2;
          *reinterpret_cast<uint2*>(&e2) = ld_word(q.pc);
          q.pc += 1;
          partial = reinterpret_cast<const float*>(addr48(e2));
        }
        PeerOut peer_args;
        const PeerOut* peers = nullptr;
        if (to_peers) {
          VDC_LOAD_PEERS(peer_args);
          peers = &peer_args;
        }
        uint64_t dyn_base = 0;
        if (ci.args[1] & VDC_GEMV_DYNROWS_BIT) {
          VdcCInst e2;
          *reinterpret_cast<uint2*>(&e2) = ld_word(q.pc);
          q.pc += 1;
          dyn_base = addr48(e2);
        }
        switch (R) {
          case 1: task_gemv_rows<1>(q, ci.args[0], mode, accumulate, norm, K, row_base, scales, wfmt, moe, dyn, peers, dyn_base, partial, chunk_stride); break;
          case 2: task_gemv_rows<2>(q, ci.args[0], mode, accumulate, norm, K, row_base, scales, wfmt, moe, dyn, peers, dyn_base, partial, chunk_stride); break;
          case 4: task_gemv_rows<4>(q, ci.args[0], mode, accumulate, norm, K, row_base, scales, wfmt, moe, dyn, peers, dyn_base, partial, chunk_stride); break;
          case 8: task_gemv_rows<8>(q, ci.args[0], mode, accumulate, norm, K, row_base, scales, wfmt, moe, dyn, peers, dyn_base, partial, chunk_stride); break;
          case 16: task_gemv_rows<16>(q, ci.args[0], mode, accumulate, norm, K, row_base, scales, wfmt, moe, dyn, peers, dyn_base, partial, chunk_stride); break;
          default: raise_abort(c, VDC_ERR_BAD_OPCODE, 0, (int)q.pc, ci.opcode, -1, R); q.aborted = true; break;
        }
        break;
      }
      case 0x7210:
      case 0x7211: {  // ATTN_DECODE_PAGED (thirteen words; the first two are in registers already)
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        VdcCInst e[11];
#pragma unroll
        for (int k = 0; k < 11; ++k) *reinterpret_cast<uint2*>(&e[k]) = ld_word(q.pc + (uint32_t)k);
        q.pc += 11;
        AttnArgs a;
        a.max_pages = ci.args[0];
        a.base_page = ci.args[1];
        a.flags = ci.args[2];
        a.qk_eps = __uint_as_float(((uint32_t)ex.args[0] << 16) | ex.args[1]);
        a.n_splits = ex.args[2];
        a.state = reinterpret_cast<const int*>(addr48(e[0]));
        a.k_rows = reinterpret_cast<uint8_t*>(addr48(e[1]));
        a.v_rows = reinterpret_cast<uint8_t*>(addr48(e[2]));
        a.records = reinterpret_cast<float*>(addr48(e[3]));
        a.counter = reinterpret_cast<int*>(addr48(e[4]));
        a.out = reinterpret_cast<__nv_bfloat16*>(addr48(e[5]));
        a.split = e[6].args[0];
        a.bar = e[6].args[1];
        a.b = (a.flags & VDC_ATTN_PACKED_BIT) ? (e[6].args[2] & 0xFF) : 0;
        a.bpad = (a.flags & VDC_ATTN_PACKED_BIT) ? (e[6].args[2] >> 8) * 16 : 0;
        a.rope = reinterpret_cast<const float*>(addr48(e[7]));
        a.nw = reinterpret_cast<const __nv_bfloat16*>(addr48(e[8]));
        a.qkv = reinterpret_cast<const __nv_bfloat16*>(addr48(e[9]));
        a.wait_bar = e[10].args[0];
        a.state_stride = e[10].args[1];
        a.qkv_stride = (int)e[10].args[2] * 8;
        // units that walk four pages or more take two pages per trip; like the pair units that variant is
        // compiled into the full kernel only (the batch-1 engines' units walk two pages)
        bool long_walk = false;
        if constexpr (kRefOps) long_walk = a.max_pages >= 4 && !(a.flags & VDC_ATTN_APPEND_BIT);
        if (long_walk && !(a.flags & VDC_ATTN_PAIR_BIT)) {
          if constexpr (kRefOps) {
            if (ci.opcode == 0x7210) task_attn_decode<4, false, true>(q, a);
            else task_attn_decode<8, false, true>(q, a);
          }
        } else if (ci.opcode == 0x7210) {
          task_attn_decode<4>(q, a);
        } else if (a.flags & VDC_ATTN_PAIR_BIT) {
          // pair units exist in the full kernel only (vdc_launch, vdc_launch_async_full): measured on B200, one more instantiation of
          // the attention task in the kernel the decode engines launch costs the batch-1 step 1.7 %
          if constexpr (kRefOps) {
            if (long_walk) task_attn_decode<8, true, true>(q, a);
            else task_attn_decode<8, true>(q, a);
          } else {
            raise_abort(c, VDC_ERR_BAD_OPCODE, 0, (int)q.pc, ci.opcode, -1, a.flags);
            q.aborted = true;
          }
        } else {
          task_attn_decode<8>(q, a);
        }
        break;
      }
      case 0x7230: {  // L2_PREFETCH: every thread touches its share of the range, nobody waits
        const uint64_t base = (uint64_t)ci.args[0] | ((uint64_t)ci.args[1] << 16) | ((uint64_t)ci.args[2] << 32);
        const uint32_t bytes = (uint32_t)ex.args[0] | ((uint32_t)ex.args[1] << 16);
        for (uint32_t off = (uint32_t)tid * 128u; off < bytes; off += kCT * 128u)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
        break;
      }
      case 0x7300: {  // GEMM_TC_BF16 (eleven words)
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        VdcCInst e[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) *reinterpret_cast<uint2*>(&e[k]) = ld_word(q.pc + (uint32_t)k);
        q.pc += 9;
        GemmTc g;
        g.n_w = ci.args[0];
        g.N = (ci.args[1] & 0xFF) * 16;
        g.mode = (ci.args[1] >> 8) & 0xF;
        g.norm = (ci.args[1] >> 12) & 1;
        g.KS = ci.args[2] & 0xFF;
        g.G = ci.args[2] >> 8;
        g.eps = __uint_as_float(((uint32_t)ex.args[0] << 16) | ex.args[1]);
        g.B = ex.args[2];
        g.out = reinterpret_cast<uint8_t*>(addr48(e[0]));
        g.keys = reinterpret_cast<unsigned long long*>(addr48(e[1]));
        g.n0 = (int)e[2].args[0] | ((int)e[2].args[1] << 16);
        g.bar = e[2].args[2];
        g.ld = (int)e[3].args[0] * 16;
        g.Bpad = e[3].args[1];
        g.Kfull = (int)e[3].args[2] * 16;
        g.stats = reinterpret_cast<float*>(addr48(e[4]));
        g.scratch = reinterpret_cast<float*>(addr48(e[5]));
        g.counter = reinterpret_cast<int*>(addr48(e[6]));
        g.n_slices = e[7].args[0];
        g.wfmt = (ci.args[1] >> 13) & 3;   // 0 bf16, 1 e4m3, 2 NVFP4
        g.scales = reinterpret_cast<const float*>(addr48(e[8]));
        const bool ok = g.N >= 16 && g.N <= 256 && g.B >= 1 && g.B <= g.Bpad &&
                        (g.Bpad == 16 || g.Bpad == 32 || g.Bpad == 64 || g.Bpad == 128) && g.KS >= 1 && g.G >= 1 &&
                        g.n_w >= 1 && (!g.norm || g.stats != nullptr) &&
                        (g.n_slices <= 1 || (g.scratch != nullptr && g.counter != nullptr)) &&
                        (g.wfmt == 0 || g.scales != nullptr);
        if (!ok) {
          raise_abort(c, VDC_ERR_BAD_OPCODE, 0, (int)q.pc, ci.opcode, -1, g.N);
          q.aborted = true;
          break;
        }
        task_gemm_tc(q, g);
        break;
      }
      case 0x7310: {  // EMBED_PACK (six words)
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        VdcCInst e[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) *reinterpret_cast<uint2*>(&e[k]) = ld_word(q.pc + (uint32_t)k);
        q.pc += 4;
        task_embed_pack(q, ci.args[0], ci.args[1], ci.args[2], ex.args[0], ex.args[1], ex.args[2],
                        reinterpret_cast<const int*>(addr48(e[0])), reinterpret_cast<const uint8_t*>(addr48(e[1])),
                        reinterpret_cast<uint8_t*>(addr48(e[2])), reinterpret_cast<float*>(addr48(e[3])));
        break;
      }
      case 0x7320: {  // BATCH_ADVANCE (five words)
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        VdcCInst e2, e3, e4;
        *reinterpret_cast<uint2*>(&e2) = ld_word(q.pc);
        *reinterpret_cast<uint2*>(&e3) = ld_word(q.pc + 1);
        *reinterpret_cast<uint2*>(&e4) = ld_word(q.pc + 2);
        q.pc += 3;
        task_batch_advance(q, ci.args[0], ci.args[1], ci.args[2], reinterpret_cast<unsigned long long*>(addr48(ex)),
                           reinterpret_cast<int*>(addr48(e2)), reinterpret_cast<float*>(addr48(e3)),
                           (int)e4.args[0] | ((int)e4.args[1] << 16));
        break;
      }
      case 0x7220: {
        PeerOut peer_args;
        if (ci.args[1] == 2) {
          VDC_LOAD_PEERS(peer_args);
          task_argmax_final(q, ci.args[0], 1, &peer_args);
        } else {
          task_argmax_final(q, ci.args[0], ci.args[1]);
        }
        break;
      }
      case 0x7330: {  // XREDUCE (five words)
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        VdcCInst e[4];
        e[0] = ex;
#pragma unroll
        for (int k = 1; k < 4; ++k) *reinterpret_cast<uint2*>(&e[k]) = ld_word(q.pc + (uint32_t)(k - 1));
        q.pc += 3;
        task_xreduce(q, ci.args[0], ci.args[1], ci.args[2], reinterpret_cast<const unsigned long long*>(addr48(e[0])),
                     (size_t)e[1].args[0] * 2, (uint32_t)e[1].args[1] | ((uint32_t)e[1].args[2] << 16),
                     reinterpret_cast<__nv_bfloat16*>(addr48(e[2])), reinterpret_cast<const int*>(addr48(e[3])));
        break;
      }
      case 0x7331: {  // XWAIT (five words)
        auto addr48 = [](const VdcCInst& w) {
          return (uint64_t)w.args[0] | ((uint64_t)w.args[1] << 16) | ((uint64_t)w.args[2] << 32);
        };
        VdcCInst e[4];
        e[0] = ex;
#pragma unroll
        for (int k = 1; k < 4; ++k) *reinterpret_cast<uint2*>(&e[k]) = ld_word(q.pc + (uint32_t)(k - 1));
        q.pc += 3;
        task_xwait(q, ci.args[0], ci.args[1], (uint32_t)ci.args[2] | ((uint32_t)e[3].args[0] << 16),
                   reinterpret_cast<const unsigned long long*>(addr48(e[0])), reinterpret_cast<const int*>(addr48(e[1])),
                   reinterpret_cast<uint32_t*>(addr48(e[2])));
        break;
      }
      case 0x7240: task_moe_route(q, ci.args[0], ci.args[1], ci.args[2] & 0xFF, ci.args[2] >> 8); break;
      default:
        if constexpr (kRefOps) {
          if (dispatch_ref_op(q, ci)) break;
        }
        raise_abort(c, VDC_ERR_BAD_OPCODE, 0, (int)q.pc, ci.opcode, -1, 0);
        q.aborted = true;
        break;
    }
    if (traced) c.profile[c.sm * VDC_NUM_PROFILE_EVENTS + 16 + 2 * n_traced + 1] = globaltimer_ns();
    if (ci.opcode != 0x7000) n_traced++;
  }
}

// ------------------------------------------------------------------------- //
// the kernel
// ------------------------------------------------------------------------- //
template <bool kRefOps>
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
  if (tid < kCW) sh.warp_next[tid] = 0xFFFFFFFFu;
  if (tid == 0) {
    sh.slot_avail = kSlotMaskAll;
    sh.ring_tail = 0;
    sh.cta_head = 0;
    sh.st_head = sh.st_tail = 0;
    sh.aborted = 0;
    sh.demand_pos = 0;
    sh.pf_go = 0;
    sh.pf_exit = 0;
    sh.tmem_ready = 0;
    profile[c.sm * VDC_NUM_PROFILE_EVENTS + 0] = globaltimer_ns();
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (tid < kCT) {
    compute_core<kRefOps>(c, cinsts + (size_t)c.sm * insts_per_sm, insts_per_sm, tid);
  } else {
    const int w = (tid - kCT) >> 5, lane = tid & 31;
    if (w == 0) control_warp(c, minsts + (size_t)c.sm * insts_per_sm, insts_per_sm, lane);
    else if (w == 1) { if (lane == 0) store_warp(c); }
#ifndef VDC_NO_STREAMER
    else if (w == 4) streamer_warp(c, lane);
#endif
    else if (lane == 0) load_port(c, w - 2);
  }
  __syncthreads();
  if (sh.tmem_ready && tid < 32) {
    // Tensor memory goes back only after every tensor-core operation has finished (an
    // aborted task may have left some in flight): bounded wait on one last commit.
    if (tid == 0) {
      umma_commit(&sh.mma_final);
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&sh.mma_final, 0) && globaltimer_ns() - t0 < 2000000ull) __nanosleep(200);
    }
    __syncwarp();
    tmem_dealloc(sh.tmem_base, kTmemCols);
  }
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
// Slots, 1 KB of alignment slack, and a 2 KB guard behind the last slot: the tensor cores read 128
// operand rows of an X chunk whatever the batch, and the rows past the batch fall behind the chunk.
extern "C" size_t vdc_megakernel_dynamic_smem() { return (size_t)VDC_NUM_SLOTS * VDC_SLOT_BYTES + 1024 + 2048; }

extern "C" cudaError_t vdc_megakernel_prepare() {
  cudaError_t e = cudaFuncSetAttribute(vdc::vdc_megakernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)vdc_megakernel_dynamic_smem());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(vdc::vdc_megakernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)vdc_megakernel_dynamic_smem());
}

extern "C" cudaError_t vdc_megakernel_launch(int num_sms, const void* cinsts, const void* minsts, const void* tmas,
                                             int* bars, uint64_t* profile, vdc_status* status, int insts_per_sm,
                                             uint64_t timeout_ns, cudaStream_t stream, int ref_ops) {
  // ref_ops: the full kernel, which also knows the reference's tile-contract operators
  if (ref_ops)
    vdc::vdc_megakernel<true><<<num_sms, VDC_THREADS, vdc_megakernel_dynamic_smem(), stream>>>(
        reinterpret_cast<const VdcCInst*>(cinsts), reinterpret_cast<const VdcMInst*>(minsts),
        reinterpret_cast<const CUtensorMap*>(tmas), bars, profile, status, insts_per_sm, timeout_ns);
  else
    vdc::vdc_megakernel<false><<<num_sms, VDC_THREADS, vdc_megakernel_dynamic_smem(), stream>>>(
        reinterpret_cast<const VdcCInst*>(cinsts), reinterpret_cast<const VdcMInst*>(minsts),
        reinterpret_cast<const CUtensorMap*>(tmas), bars, profile, status, insts_per_sm, timeout_ns);
  return cudaGetLastError();
}

