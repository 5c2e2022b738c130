/* C ABI of libvdcores_b200.so — the B200 decode megakernel runtime.
 *
 * Every entry point takes plain pointers and sizes (device pointers where the
 * comment says "device"), returns 0 on success or a VDC_ERR_* code, allocates
 * nothing it does not own, and transfers no ownership.  Host use is single
 * threaded per device (one process per GPU).
 *
 * Each declaration names the reference interface it stands in for; paths are
 * inside the reference project.  The reference exposes these through a
 * pybind11 module called dae.runtime (src/torch_runtime.cu:260-314).
 */
#ifndef VDCORES_H
#define VDCORES_H

#include <stddef.h>
#include <stdint.h>

#include "../vdcores_b200/csrc/isa.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Library version (major*100 + minor). */
int vdc_version(void);

/* Prepares the current device: raises the kernel's dynamic shared-memory limit
 * and allocates the device-side status block.  Must be called once per device
 * before the first launch, with that device current.
 * Replaces: set_smem_size (src/runtime.cu:6-16, src/torch_runtime.cu:15-17). */
int vdc_init(void);

/* Kept for callers that pass an explicit size like the reference did; the
 * runtime sizes shared memory itself, so this only validates the value.
 * Replaces: set_smem_size (src/torch_runtime.cu:15-17). */
int vdc_set_smem_size(int bytes);

/* Synchronous launch of the persistent megakernel: device-synchronises, runs
 * one CTA per entry of the instruction tables, device-synchronises, and copies
 * the status block to *status (may be NULL).
 *   compute_insts : device, num_sms * insts_per_sm * 8 bytes
 *   memory_insts  : device, num_sms * insts_per_sm * 16 bytes
 *   tma_descs     : device, array of 128-byte tensor maps (may be NULL)
 *   bars          : device, int32[VDC_MAX_BARS] countdown barriers, MUTATED
 *   profile       : device, uint64[num_sms * VDC_NUM_PROFILE_EVENTS]
 *   stream        : cudaStream_t as an integer handle
 *   timeout_ns    : budget of every device-side wait; 0 selects 2 s
 * Returns VDC_ERR_TIMEOUT / VDC_ERR_BAD_OPCODE with details in *status when the
 * kernel gave up a wait instead of hanging, VDC_ERR_CUDA on a CUDA error.
 * Replaces: launch_dae (src/torch_runtime.cu:68-100, src/runtime.cu:18-43);
 * unlike it, num_sms may be anything up to the device's SM count. */
int vdc_launch(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
               const void* tma_descs, int* bars, uint64_t* profile, uint64_t stream, uint64_t timeout_ns,
               vdc_status* status);

/* Asynchronous variant for decode loops: optionally restores `bars` from
 * `bars_init` (device, same size; NULL to skip) on `stream`, then enqueues the
 * kernel and returns without synchronising.  Errors detected by the kernel are
 * fetched later with vdc_read_status.  No counterpart in the reference, whose
 * launches are always synchronous (src/runtime.cu:29,40). */
int vdc_launch_async(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                     const void* tma_descs, int* bars, const int* bars_init, uint64_t* profile, uint64_t stream,
                     uint64_t timeout_ns);

/* vdc_launch_async for the FULL kernel (every operator vdc_launch has, no synchronisation): what the batched decode
 * engine and the prefill launch.  The batch-1 engines stay on vdc_launch_async, whose kernel is smaller and, measured,
 * 1.7-1.8 % faster on their step.  No counterpart in the reference. */
int vdc_launch_async_full(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                          const void* tma_descs, int* bars, const int* bars_init, uint64_t* profile, uint64_t stream,
                          uint64_t timeout_ns);

/* Synchronises `stream` and copies the device status block to *status; returns
 * its code.  Clears the block when `clear` is non-zero. */
int vdc_read_status(uint64_t stream, vdc_status* status, int clear);

/* Encodes a tiled tensor map (128 bytes written to out_desc, host memory).
 *   dtype: 0 u8, 1 f16, 2 bf16, 3 f32, 4 i32, 5 u32;  rank 1..5, dims fastest first;
 *   strides_bytes has rank-1 entries; swizzle_bytes in {0,32,64,128};
 *   interleave_bytes in {0,16,32}.  L2 promotion 256 B, no out-of-bounds fill.
 * Replaces: build_tma_desc (src/torch_runtime.cu:147-220) and
 * create_tma_descriptor (src/runtime.cu:45-107). */
int vdc_build_tma_desc(void* out_desc, const void* base, int dtype, int rank, const uint64_t* shape,
                       const uint64_t* strides_bytes, const uint32_t* box_dim, const uint32_t* elem_strides,
                       int swizzle_bytes, int interleave_bytes);

/* Sets the stream's L2 access-policy window over [ptr, ptr+bytes), clamped to
 * the device maximum.  Policies are cudaAccessProperty values (0 normal,
 * 1 streaming, 2 persisting).
 * Replaces: set_cache_policy (src/torch_runtime.cu:229-258). */
int vdc_set_cache_policy(const void* ptr, size_t bytes, uint64_t stream, float hit_ratio, int hit_policy,
                         int miss_policy);

/* Lets kernels of the current device load from / store to memory of `peer_device` that is mapped
 * into this process (its own allocations there, or another process's imported through CUDA IPC).
 * The tensor-parallel engine calls it once per peer before its first step: its decode kernel
 * writes partial results straight into the other ranks' exchange blocks.  Already enabled: success.
 * No counterpart in the reference (it has no multi-GPU path). */
int vdc_enable_peer_access(int peer_device);

/* Exchange blocks of the in-kernel tensor-parallel exchange: vdc_peer_alloc allocates `bytes` of zeroed device
 * memory on the current device as an allocation of its own (so that its IPC handle names exactly that block),
 * vdc_ipc_export writes its 64-byte CUDA IPC handle for the other ranks' vdc_ipc_open, vdc_peer_free releases
 * it (after every importer has closed its mapping).  No counterpart in the reference (it has no multi-GPU path). */
int vdc_peer_alloc(size_t bytes, uint64_t* out_ptr);
int vdc_peer_free(uint64_t ptr);
int vdc_ipc_export(uint64_t ptr, void* handle_out, size_t handle_bytes);

/* Maps a device allocation exported by another process (the 64-byte CUDA IPC memory handle of
 * its base allocation) for kernels of the CURRENT device and returns its address in *out_ptr;
 * peer access to the exporting device is enabled as needed.  vdc_ipc_close unmaps it.  Used for
 * the other ranks' exchange blocks of the in-kernel tensor-parallel exchange.
 * No counterpart in the reference. */
int vdc_ipc_open(const void* handle, size_t handle_bytes, uint64_t* out_ptr);
int vdc_ipc_close(uint64_t ptr);

/* Opcode table: names and values of every memory and compute opcode.
 * Replaces: the `opcode` submodule (src/torch_runtime.cu:261-264). */
int vdc_opcode_count(void);
const char* vdc_opcode_name(int index);
int vdc_opcode_value(int index);
/* 1 when the opcode at `index` is a compute opcode the kernel can execute.
 * Replaces: supported_compute_ops (src/torch_runtime.cu:279-283). */
int vdc_opcode_is_compute(int index);

/* Named integer constants: slot_size, num_slots, max_insts, num_profile_events,
 * max_tmas, max_bars, num_special_slots, compute_threads, kv_page, head_dim.
 * Returns -1 for an unknown name.
 * Replaces: the `config` submodule (src/torch_runtime.cu:285-292). */
int64_t vdc_config(const char* name);

/* Compute-op family definitions as "FAMILY\tdefinition" lines separated by
 * '\n' (empty: this runtime compiles every op, nothing is generated at build
 * time).  Replaces: compute_family_specs (src/torch_runtime.cu:266-277). */
const char* vdc_family_specs(void);

/* Launch for hosts that must not allocate device memory.  Some embedders hand
 * every free byte of the GPU to their own pool at start-up (a serving engine
 * that sizes its KV cache to whatever is left), or run under a memory budget
 * that an outside allocator enforces; for them a cudaMalloc inside a library
 * call fails or eats into that pool, so vdc_init (which allocates the status
 * block) and scratch tensors are not an option.  This entry point runs the same
 * megakernel as vdc_launch, synchronously on `stream`, with its scratch — status
 * block, the VDC_MAX_BARS countdown barriers and the per-SM profile rows — in a
 * 164 KB device array that is part of the library image.  It calls no
 * cudaMalloc / cudaFree and no allocating library routine, and needs no vdc_init.
 *   bars_init : device, int32[VDC_MAX_BARS], initial barrier counts (input, not modified)
 *   other arguments as for vdc_launch; outputs are whatever the program's stores write.
 * Limits: num_sms <= 160 (more is rejected with VDC_ERR_ARG).  The first call
 * on a device does the one-time set-up (shared-memory attribute, address of the
 * array).  The call synchronises its stream (it returns the status), so it cannot be
 * part of a stream capture.  All calls on a device share
 * the one array: it keeps the last call's contents (status and barriers are
 * re-initialised at the start of every call), and two calls that overlap on the
 * GPU would race on it, so keep them on one stream or serialise them.
 * No counterpart in the reference. */
int vdc_launch_static(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                      const void* tma_descs, const int* bars_init, uint64_t stream, uint64_t timeout_ns,
                      vdc_status* status);

/* Host-side check of a program before it is uploaded: walks every SM's compute
 * and memory stream in HOST memory (the arrays vdc_launch takes, before the copy
 * to the device) and rejects what the kernel could only report after a launch:
 * an unknown opcode, a multi-word instruction whose continuation words are
 * missing or run past the stream, a GEMV with an unsupported rows-per-chunk
 * count, a slot request or special slot id out of range, a loop that does not jump
 * backwards, a stream without its terminator.  Touches no GPU state.  On a
 * finding returns VDC_ERR_BAD_OPCODE or VDC_ERR_ARG, writes the SM and the
 * instruction index to *bad_sm / *bad_pc (either may be null) and leaves a
 * sentence in vdc_last_error().
 * Replaces: the only checks the reference makes before a launch, the stream
 * lengths asserted against max_insts (python/dae/launcher.py:67-68); it has no
 * check of the instruction words themselves. */
int vdc_validate_streams(int num_sms, int insts_per_sm, const void* compute_insts_host, const void* memory_insts_host,
                         int* bad_sm, int* bad_pc);

/* Text of the last CUDA error seen by this library on the calling thread. */
const char* vdc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* VDCORES_H */
