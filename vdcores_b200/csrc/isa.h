// Instruction-set constants shared by the host library and the megakernel.
//
// The encodings keep the reference's wire format so that instruction streams
// produced by its Python schedules stay valid:
//   * 8-byte compute instruction {u16 opcode, u16 args[3]}   (reference include/dae/context.cuh:51-54)
//   * 16-byte memory instruction {u16 opcode|flags, u16 size, u16 nslot|bar<<6, u16 arg, u64 address}
//     (reference include/dae/context.cuh:87-113), six flag bits (context.cuh:58-66)
//   * memory opcode ids 1..23 (reference include/dae/opcode.cuh.inc:1-32)
// Ids 24 and up, and every compute opcode, are this runtime's own.
#pragma once
#include <stdint.h>

#define VDC_SLOT_BYTES 8192
#define VDC_NUM_SLOTS 24
#define VDC_NUM_SPECIAL_SLOTS 9
#define VDC_MAX_INSTS 4096
#define VDC_NUM_PROFILE_EVENTS 128
#define VDC_MAX_TMAS 1024
#define VDC_MAX_BARS 1024
#define VDC_QUEUE_LEN 32

#define VDC_COMPUTE_WARPS 8
#define VDC_COMPUTE_THREADS (VDC_COMPUTE_WARPS * 32)
#ifdef VDC_NO_STREAMER
#define VDC_MEMORY_WARPS 4
#else
#define VDC_MEMORY_WARPS 5
#endif
#define VDC_THREADS ((VDC_COMPUTE_WARPS + VDC_MEMORY_WARPS) * 32)
#define VDC_MAX_SMS 160

// memory-instruction flag bits (low 6 bits of the opcode field)
#define VDC_F_ALLOCATE 0x01
#define VDC_F_WRITEBACK 0x02
#define VDC_F_GROUP 0x04
#define VDC_F_JUMP 0x08
#define VDC_F_BARRIER 0x10
#define VDC_F_PORT 0x20
#define VDC_FLAG_BITS 6
#define VDC_MOP(id, flags) ((uint16_t)(((id) << VDC_FLAG_BITS) | (flags)))

// X(name, value)
#define VDC_MEMORY_OPS(X)                                                              \
  X(OP_TERMINATE, VDC_MOP(1, 0))                                                       \
  X(OP_REPEAT, VDC_MOP(2, 0))                                                          \
  X(OP_LOOP, VDC_MOP(3, 0))                                                            \
  X(OP_SHIFT_RESOURCE, VDC_MOP(4, 0))                                                  \
  X(OP_ISSUE_BARRIER, VDC_MOP(5, 0))                                                   \
  X(OP_CC0, VDC_MOP(6, 0))                                                             \
  X(OP_CC0_ROW_BYTES, VDC_MOP(7, 0))                                                   \
  X(OP_ALLOC_REG_LOAD, VDC_MOP(8, VDC_F_ALLOCATE))                                     \
  X(OP_ALLOC_TMA_LOAD_1D, VDC_MOP(9, VDC_F_ALLOCATE))                                  \
  X(OP_ALLOC_TMA_LOAD_TENSOR_1D, VDC_MOP(10, VDC_F_ALLOCATE))                          \
  X(OP_ALLOC_TMA_LOAD_2D, VDC_MOP(11, VDC_F_ALLOCATE))                                 \
  X(OP_ALLOC_TMA_LOAD_3D, VDC_MOP(12, VDC_F_ALLOCATE))                                 \
  X(OP_ALLOC_TMA_LOAD_4D, VDC_MOP(13, VDC_F_ALLOCATE))                                 \
  X(OP_ALLOC_TMA_LOAD_5D_FIX0, VDC_MOP(14, VDC_F_ALLOCATE))                            \
  X(OP_ALLOC_WB_REG_STORE, VDC_MOP(15, VDC_F_ALLOCATE))                                \
  X(OP_ALLOC_WB_TMA_STORE_1D, VDC_MOP(16, VDC_F_ALLOCATE | VDC_F_WRITEBACK))           \
  X(OP_ALLOC_WB_TMA_STORE_2D, VDC_MOP(17, VDC_F_ALLOCATE | VDC_F_WRITEBACK))           \
  X(OP_ALLOC_WB_TMA_STORE_3D, VDC_MOP(18, VDC_F_ALLOCATE | VDC_F_WRITEBACK))           \
  X(OP_ALLOC_WB_TMA_STORE_4D, VDC_MOP(19, VDC_F_ALLOCATE | VDC_F_WRITEBACK))           \
  X(OP_ALLOC_WB_TMA_STORE_5D_FIX0, VDC_MOP(20, VDC_F_ALLOCATE | VDC_F_WRITEBACK))      \
  X(OP_ALLOC_WB_TMA_REDUCE_ADD_2D, VDC_MOP(21, VDC_F_ALLOCATE | VDC_F_WRITEBACK))      \
  X(OP_ALLOC_WB_TMA_REDUCE_ADD_3D, VDC_MOP(22, VDC_F_ALLOCATE | VDC_F_WRITEBACK))      \
  X(OP_ALLOC_WB_RAW_ADDRESS, VDC_MOP(23, VDC_F_ALLOCATE))                              \
  X(OP_ALLOC_WB_TMA_REDUCE_ADD_1D, VDC_MOP(24, VDC_F_ALLOCATE | VDC_F_WRITEBACK))      \
  X(OP_DYN_COUNT, VDC_MOP(25, 0))                                                      \
  X(OP_PREFETCH_L2, VDC_MOP(26, 0))                                                    \
  X(OP_STREAM_LIST, VDC_MOP(27, 0))                                                    \
  X(OP_ALLOC_TMA_LOAD_1D_STREAM, VDC_MOP(28, VDC_F_ALLOCATE))                          \
  X(OP_CC0_STRIDE32, VDC_MOP(29, 0))                                                   \
  X(OP_PT_LOAD32, VDC_MOP(30, 0))                                                      \
  X(OP_PT_APPLY, VDC_MOP(31, 0))                                                       \
  X(OP_ALLOC_XVEC, VDC_MOP(32, VDC_F_ALLOCATE))                                        \
  X(OP_DYN_CHUNKS, VDC_MOP(33, 0))

// OP_ALLOC_XVEC: allocates slots for an activation vector and hands {address, size, barrier} to the
// compute task, which waits for the barrier itself (BARRIER flag: the load port does NOT wait) and reads
// the vector from global memory with ordinary loads.  It takes the copy engine, one ring hop and one
// CTA barrier out of the path between "the producers' barrier opened" and "the stage computes".
//
// OP_DYN_CHUNKS: the next instruction (a plain 1-D load of one weight chunk) is issued for chunk indices
// drawn one at a time from a counter all SMs share (barrier word `bar`, starts at 0, atomically incremented)
// until the index reaches size | arg << 16; chunk i is read at the template's address + i * its size.  Four
// end markers follow the last chunk in the ring (one per consuming warp pair; the address field holds the
// number of chunks this SM drew, low half, and the marker's ordinal 0..3, high half).  SMs that stream faster take more chunks, so a stage ends everywhere within
// one chunk time instead of waiting for the SM with the slowest memory path.
#define VDC_STREAM_END 0x20000000   // ring word of an end marker
//
// Compute opcodes.  The first block keeps reference names (control ops); the 0x72xx / 0x73xx blocks are
// the B200-native decode set; the 0x74xx block carries the reference's operator names and tile contracts
// (include/dae/opcode.cuh.inc:56-82, tools/generate_selected_compute_ops.py:235-258), so that its
// instruction classes resolve and its schedules run: see mk_refops.cuh.
// X(name, value, words): `words` = 8-byte words the instruction occupies in the compute stream
// before any optional trailing words (flags of the first word announce those).
#define VDC_COMPUTE_OPS(X)                                                             \
  X(OP_TERMINATEC, 0x7000, 1)                                                          \
  X(OP_LOOPC, 0x7001, 1)                                                               \
  X(OP_DUMMY, 0x7002, 1)                                                               \
  X(OP_COPY, 0x7003, 1)                                                                \
  X(OP_GEMV_ROWS_BF16, 0x7200, 2)                                                      \
  X(OP_GEMV_ROWS_FP8, 0x7201, 3)                                                       \
  X(OP_GEMV_ROWS_NVFP4, 0x7202, 3)                                                     \
  X(OP_GEMV_ROWS_MOE_DOWN, 0x7203, 5)                                                  \
  X(OP_ATTN_DECODE_PAGED_G4, 0x7210, 13)                                               \
  X(OP_ATTN_DECODE_PAGED_G8, 0x7211, 13)                                               \
  X(OP_ARGMAX_FINAL, 0x7220, 1)                                                        \
  X(OP_L2_PREFETCH, 0x7230, 2)                                                         \
  X(OP_MOE_ROUTE, 0x7240, 1)                                                           \
  X(OP_GEMM_TC_BF16, 0x7300, 11)                                                       \
  X(OP_EMBED_PACK, 0x7310, 6)                                                          \
  X(OP_BATCH_ADVANCE, 0x7320, 5)                                                       \
  X(OP_XREDUCE, 0x7330, 5)                                                             \
  X(OP_XWAIT, 0x7331, 5)                                                               \
  X(OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_4__RESIDUAL_0, 0x7400, 1)                   \
  X(OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_4__RESIDUAL_1, 0x7401, 1)                   \
  X(OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_2__RESIDUAL_0, 0x7402, 1)                   \
  X(OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_2__RESIDUAL_1, 0x7403, 1)                   \
  X(OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_1__RESIDUAL_0, 0x7404, 1)                   \
  X(OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_1__RESIDUAL_1, 0x7405, 1)                   \
  X(OP_GEMV_MMA__M_64__N_8__K_256, 0x7408, 1)                                          \
  X(OP_RMS_NORM_F16_K_4096_SMEM, 0x7410, 1)                                            \
  X(OP_RMS_NORM_F16_K_2048_SMEM, 0x7411, 1)                                            \
  X(OP_RMS_NORM_F16_K_5120_SMEM, 0x7412, 1)                                            \
  X(OP_RMS_NORM_F16_K_128_SMEM, 0x7413, 1)                                             \
  X(OP_ROPE_INTERLEAVE_512, 0x7418, 1)                                                 \
  X(OP_SILU_MUL_SHARED_BF16_K_64_SW128, 0x7420, 1)                                     \
  X(OP_SILU_MUL_SHARED_BF16_K_4096_INTER, 0x7421, 1)                                   \
  X(OP_ARGMAX_PARTIAL_bf16_1024_65536_128, 0x7428, 1)                                  \
  X(OP_ARGMAX_REDUCE_bf16_1024_128, 0x7429, 1)                                         \
  X(OP_ARGMAX_PARTIAL_bf16_1152_50688_132, 0x742A, 1)                                  \
  X(OP_ARGMAX_REDUCE_bf16_1152_132, 0x742B, 1)                                         \
  X(OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim, 0x7430, 1)                              \
  X(OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim_MMA, 0x7431, 1)                          \
  X(OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim_split, 0x7432, 1)                        \
  X(OP_ATTENTION_M64N64K16_F16_F32_64_64_hdim_split_MMA, 0x7433, 1)                    \
  X(OP_ATTN_SPLIT_POST_REDUCE, 0x7434, 1)                                              \
  X(OP_EXT, 0x7FFF, 1)

// OP_L2_PREFETCH (two words): args = 48-bit address in three 16-bit pieces (low
// first); second word args[0..1] = byte count (low, high).  All compute threads
// issue L2 prefetches for the range and move on; nothing is popped.
//
// OP_EXT is never dispatched: it marks the continuation words of a multi-word
// compute instruction (the table above gives the counts).
//
// GEMV_ROWS_FP8 (3 words): as GEMV_ROWS_BF16 for e4m3 weights (K a multiple of 512, one byte per
// weight), third word = 48-bit address of the fp32 per-row scales of the task's first row.
//
// GEMV_ROWS_NVFP4 (3 words): rows of K/2 bytes e2m1 pairs + K/16 e4m3 block scales (K a multiple
// of 1024); third word as for FP8 (fp32 per-row scale = the tensor scale of the row's matrix).
//
// GEMV_ROWS_MOE_DOWN (5 words, bf16 weights): an expert's down projection.  Words 3..5 are 48-bit
// addresses: the expert's routing weight (fp32), the fp32 accumulator and the int32 arrival counter of
// the task's first output row.  Each row adds weight * bf16(W x) to its accumulator; the top_k-th
// arrival (args of word 2: [eps hi, eps lo] unused, args[2] = top_k) folds bf16(sum) into the hidden
// state (the output address) and clears both.
//
// In-kernel tensor parallelism (no collective library in the step).  Every rank owns an exchange block
// that all ranks map (CUDA IPC): fp32 partial rows xbuf[parity][rank][hidden], argmax records
// best[rank][4], int32 arrival counters that only ever grow.  A GEMV_ROWS task with VDC_GEMV_PEERS_BIT
// (mode STORE_F32; its output "address" is the byte offset of its first row inside a block) stores its
// rows into its slot of every rank's block and then adds 1 to every rank's counter with a system-scope
// release; its two extra words are the 48-bit address of a table {block base address of every rank,
// state block address} and [ranks, exchange number, exchanges per step].  The partial rows travel as tagged
// 8-byte entries {fp32 bits, tag}, tag = state.STEP * exchanges per step + exchange number + 1: a reader that
// finds its tag has the payload, no fence or counter is involved.  ARGMAX_FINAL with args[1] = 2 sends its
// record the same way (two entries: value, row index; same two extra words).
// XREDUCE (five words): [n elements, ranks, barrier] [48-bit address of this rank's entries xbuf[parity][0][first
// element]] [entries per rank / 2, exchange number, exchanges per step] [48-bit address of the first hidden
// element] [48-bit state block]: every thread polls (bounded) its element's entry of every rank, then
// hidden[i] = bf16(hidden[i] + sum over ranks in rank order).
// XWAIT (five words): [barrier, ranks, exchange number] [48-bit address of the ranks' candidate entries]
// [48-bit state block] [48-bit address of the compact records it writes] [exchanges per step, 0, 0].
//
// MOE_ROUTE: args = [n_experts, top_k, rank | world << 8].  Pops the fp32 router logits and a raw address;
// writes int32 ids[16], fp32 weights[16] (softmax over all experts, top-k, renormalised, rounded to bf16),
// int32 local[16] and int32 count[16]: with expert parallelism (world > 1, n_experts / world consecutive
// experts per rank) local = id modulo the experts per rank and count = 0x7FFF for the slots whose expert
// this rank owns, 0 / 0 for the others; without it local = id, count = 0x7FFF.  A GEMV_ROWS task with
// VDC_GEMV_DYN_BIT takes min(n_chunks, count) chunks, i.e. it is skipped for experts of other ranks.
// GEMV_ROWS_MOE_DOWN with a null accumulator address adds weight * bf16(W x) to the fp32 output
// (the rank's partial sum, all-reduced afterwards) instead of counting arrivals.
//
// ATTN_DECODE_PAGED (thirteen words): [max_pages, base_page, flags] [qk-norm eps hi, lo, n_splits]
// then six 48-bit addresses, low piece first: state block, this head's rows in K page 0,
// same for V, the head's split records, its arrival counter, its slice of the output;
// then [split index, barrier released by the merged output, packed-output info]; then three more
// 48-bit addresses: the rope table ([position][cos 64 | sin 64] fp32), the q / k norm weights
// (2 x 128 bf16, or 0) and the head group's projection output ((G + 2) x 128 bf16); last word
// [barrier that orders that output (0xFFFF: none), 0, 0].  The memory stream delivers only the pages.
//
// GEMV_ROWS args[1] layout: bits 0..4 rows per chunk (1,2,4,8,16), bits 8..10
// epilogue mode, bit 11 accumulate into the output (residual add), bit 12 fused
// RMSNorm of the activation vector.  args[2]: K/256 in the low byte.  Second
// word: fp32 bits of the norm eps (hi, lo), index of the first chunk within the
// whole matrix (argmax mode: candidate row = (first chunk + i) * R + r).
// Batched decode (2 <= batch <= 128) keeps every activation matrix [Bpad, K] bf16 in the
// "k-chunk major" layout the tensor cores read without swizzling: 16-byte pieces (8 consecutive k
// of one sequence) ordered [K/8][Bpad/8][8 sequences]; byte offset of (b, k) =
// ((k/8) * (Bpad/8) + b/8) * 128 + (b%8) * 16 + (k%8) * 2.  Bpad is 16, 32, 64 or 128.  Weights of
// a projection unit (N rows, N a multiple of 16, at most 256) are stored the same way, [K/8][N/8][8 rows].
// A K-range of either is one contiguous piece of memory, loaded with one 1-D bulk copy.
//
// GEMM_TC_BF16 (eleven words): D[b, n] = sum_k X[b, k] W[n, k] on the tcgen05 tensor cores for one unit =
// a block of N weight rows times a K-range; the batch sits on the accumulator's 128 lanes, the rows on
// its columns (fp32, in tensor memory).
//   word 0: [W chunks, N/16 | mode << 8 | norm << 12 | e4m3 << 13, k-steps of 16 per W chunk | W chunks per X chunk << 8]
//   word 1: [norm eps hi, lo, batch]      word 2: 48-bit output address
//   word 3: 48-bit address of the argmax keys (u64 per sequence; ARGMAX mode)
//   word 4: [first output row low 16 bits, high bits, barrier to release (0xFFFF: none)]
//   word 5: [row-major output leading dimension / 16, Bpad, whole K / 16]
//   word 6: 48-bit address of fp32 per-sequence sums of squares: read by a norm task (the producers
//           of its input left them there), accumulated by an ADD_PACKED epilogue over the rows it updated
//   word 7, 8: 48-bit addresses of the block's fp32 scratch sums [batch][N] and of its arrival counter
//   word 9: [units the block's K is cut into, 0, 0]
//   word 10: 48-bit address of the block's fp32 per-row scales (e4m3 weights), else 0
// e4m3 weights (one byte each, chunk layout [Kc/16][N/8][8 rows][16 k]) are converted, exactly, to bf16
// in shared memory by the seven non-issuing warps into two staging buffers (allocate-only entries popped
// before the groups); the accumulator sums over the codes and the epilogue applies the row scale.
// Pops [norm weights of the K-range], then per group one X chunk and its W chunks.  With norm the X
// chunks become bf16(w * bf16(x * rsqrt(sum/K + eps))) in shared memory before the tensor cores read
// them.  With several units per block each adds its partial sums to the scratch area; the unit that
// arrives last applies the epilogue, clears scratch and counter, and releases the barrier.
#define VDC_GEMM_MODE_STORE_ROWS 0    // bf16 out[b * ld + row]
#define VDC_GEMM_MODE_SILU_PAIRS 1    // rows (2j, 2j+1) = (gate_j, up_j): k-chunk-major act[b, j]
#define VDC_GEMM_MODE_ARGMAX 2        // atomicMax of (orderable bf16 logit, ~row) per sequence
#define VDC_GEMM_MODE_ADD_PACKED 3    // k-chunk-major out[b, row] += bf16(value)   (residual add)
//
// EMBED_PACK (six words): [first sequence, count, Bpad] [state stride in words, hidden/8, barrier]
// then 48-bit addresses of the first state block, the embedding table, the k-chunk-major output and
// the fp32 per-sequence sums of squares.  Copies embedding row state[b].TOKEN of each of its
// sequences into the output and stores the row's sum of squares; pops nothing.
//
// BATCH_ADVANCE (five words): [batch, state stride in words, token-log stride] then 48-bit addresses
// of the argmax keys, of the token log and of the sums of squares, then [count of those floats (lo, hi), 0]
// (they are cleared for the next step).  Pops one raw address (the first state block; it carries
// the wait on the vocabulary projection).  Thread b turns key b into the next token of sequence b,
// logs it, advances that sequence's state block and clears the key.
#define VDC_GEMV_MODE_STORE 0
#define VDC_GEMV_MODE_SILU_PAIRS 1
#define VDC_GEMV_MODE_ARGMAX 2
#define VDC_GEMV_MODE_STORE_F32 3   // fp32 partial results (tensor-parallel row-split projections)
#define VDC_GEMV_MODE_MOE_DOWN 4    // weighted fp32 accumulation over the selected experts
#define VDC_TC_STAGES 2  // bf16 staging buffers of a batched projection with converted (e4m3 / NVFP4) weights (3: measured no faster)
#define VDC_GEMV_STRIDE_BIT 0x0040   // one more word [s, 0, 0]: chunk i holds rows (i * s) * R ... of the task's matrix (chunks dealt round-robin to s SMs)
#define VDC_GEMV_PARTIAL_BIT 0x0080  // one more word: address of fp32 partial sums of the task's rows, added before rounding
#define VDC_GEMV_ACC_BIT 0x0800
#define VDC_GEMV_NORM_BIT 0x1000
#define VDC_GEMV_PEERS_BIT 0x4000  // STORE_F32 to every rank's exchange block; two more words (see below)
#define VDC_GEMV_DYN_BIT 0x2000    // the chunk count is min(n_chunks, int32 word): one more pop (a raw address: the word)
#define VDC_GEMV_DYNROWS_BIT 0x8000  // chunks come from OP_DYN_CHUNKS: row = chunk index * R, the index from the chunk's
                                     // address; one more word (last): 48-bit address of the matrix

// ATTN_DECODE args[2] bits
#define VDC_ATTN_QKNORM_BIT 0x1
#define VDC_ATTN_PACKED_BIT 0x2   // output goes to a k-chunk-major matrix; last word args[2] = b | Bpad/16 << 8
#define VDC_ATTN_PAIR_BIT 0x8     // G8 opcode only, chunked prefill of a model with 4 query heads per KV head: the unit serves two
                                  // consecutive positions (query rows 0..3 / 4..7), both with their cache rows in the pools already;
                                  // last word args[1] = int32 words from the first position's state block to the second's,
                                  // args[2] = elements / 8 from the first position's projection row to the second's; the packed
                                  // output's sequence slot b is the first position's, b + 1 the second's
#define VDC_ATTN_APPEND_BIT 0x4   // cache append only: the new key row (normed, rotated) and value row go to the pools, the
                                  // task counts `release` down once and ends; no pages, no records (chunked prefill: the
                                  // rows of a whole chunk of positions are in the pools before any of them attends)

// words of the per-sequence decode state block in device memory
#define VDC_ST_POS 0        // number of cached positions = position of the token being decoded
#define VDC_ST_NPAGES 1     // pos / 64 + 1
#define VDC_ST_TOKEN 2      // id of the token being decoded
#define VDC_ST_STEP 3       // decode steps completed
#define VDC_ST_NEWROW 4     // page_table[pos/64] * 64 * n_kv_heads + pos % 64   (256-byte row units)
#define VDC_ST_NKVH 5       // n_kv_heads (constant, used to advance NEWROW)
#define VDC_ST_MAXPAGES 6
#define VDC_ST_ERR 7
#define VDC_ST_PAGETABLE 8  // int32 page ids follow

#define VDC_KV_PAGE 64      // positions per KV page
#define VDC_HEAD_DIM 128

// status codes written to vdc_status.code
#define VDC_OK 0
#define VDC_ERR_TIMEOUT 1
#define VDC_ERR_BAD_OPCODE 2
#define VDC_ERR_CUDA 3
#define VDC_ERR_ARG 4

typedef struct vdc_status {
  int32_t abort;    // non-zero once any wait gave up; every other wait then returns
  int32_t code;     // VDC_ERR_*
  int32_t sm;       // CTA that raised it
  int32_t role;     // 0 compute, 1 control warp, 2 store warp, 3/4 load port 0/1
  int32_t pc;       // instruction index where it happened (role dependent)
  int32_t opcode;   // raw opcode field
  int32_t bar;      // global barrier id being waited for, or -1
  int32_t aux;
} vdc_status;

#ifdef __cplusplus
struct alignas(8) VdcCInst {
  uint16_t opcode;
  uint16_t args[3];
};
struct alignas(16) VdcMInst {
  uint16_t opcode;
  uint16_t size;
  union {
    struct {
      uint16_t num_slots;
      uint16_t arg;
    };
    uint32_t shifter;
  };
  union {
    uint64_t address;
    uint16_t coords[4];
  };
};
static_assert(sizeof(VdcCInst) == 8 && sizeof(VdcMInst) == 16, "wire format");
#endif
