// Host side of the C ABI declared in include/vdcores.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <string>

#include "../../include/vdcores.h"

extern "C" size_t vdc_megakernel_dynamic_smem();
extern "C" cudaError_t vdc_megakernel_prepare();
// ref_ops != 0 selects the full kernel (native operators + the reference's tile-contract operators); 0 the kernel
// with the native operators only, which the decode engines launch every step.
extern "C" cudaError_t vdc_megakernel_launch(int num_sms, const void* cinsts, const void* minsts, const void* tmas,
                                             int* bars, uint64_t* profile, vdc_status* status, int insts_per_sm,
                                             uint64_t timeout_ns, cudaStream_t stream, int ref_ops);

namespace {

thread_local std::string g_err;
constexpr int kMaxDevices = 16;
vdc_status* g_status[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

int fail_cuda(cudaError_t e, const char* what) {
  g_err = std::string(what) + ": " + cudaGetErrorString(e);
  return VDC_ERR_CUDA;
}
int fail_arg(const char* what) {
  g_err = what;
  return VDC_ERR_ARG;
}

struct OpEntry {
  const char* name;
  int value;
  int is_compute;
  int words;   // 8-byte words of a compute instruction before its optional trailing words
};
const OpEntry kOps[] = {
#define X(name, value) {#name, (int)(value), 0, 0},
    VDC_MEMORY_OPS(X)
#undef X
#define X(name, value, words) {#name, (int)(value), 1, words},
        VDC_COMPUTE_OPS(X)
#undef X
};
constexpr int kNumOps = sizeof(kOps) / sizeof(kOps[0]);

int current_device(int* dev) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (*dev < 0 || *dev >= kMaxDevices) return fail_arg("device index out of range");
  return VDC_OK;
}

int check_launch_args(int dev, int num_sms, int insts_per_sm, const void* ci, const void* mi, const int* bars,
                      const uint64_t* profile) {
  if (!g_status[dev]) return fail_arg("vdc_init was not called on this device");
  if (num_sms <= 0 || num_sms > g_sm_count[dev]) return fail_arg("num_sms must be in [1, SM count of the device]");
  if (insts_per_sm <= 0 || insts_per_sm > 65536) return fail_arg("insts_per_sm out of range");
  if (!ci || !mi || !bars || !profile) return fail_arg("null instruction, barrier or profile pointer");
  if (((uintptr_t)ci & 7) || ((uintptr_t)mi & 15) || ((uintptr_t)bars & 3) || ((uintptr_t)profile & 7))
    return fail_arg("misaligned instruction, barrier or profile pointer");
  return VDC_OK;
}

}  // namespace

extern "C" {

int vdc_version(void) { return 100; }

const char* vdc_last_error(void) { return g_err.c_str(); }

int vdc_init(void) {
  int dev;
  if (int r = current_device(&dev)) return r;
  if (g_status[dev]) return VDC_OK;
  cudaDeviceProp prop{};
  cudaError_t e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDeviceProperties");
  if (prop.major != 10) return fail_arg("this library is built for sm_100a (B200) only");
  g_sm_count[dev] = prop.multiProcessorCount;
  e = vdc_megakernel_prepare();
  if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
  vdc_status* st = nullptr;
  e = cudaMalloc(&st, sizeof(vdc_status));
  if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc(status)");
  e = cudaMemset(st, 0, sizeof(vdc_status));
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemset(status)");
  g_status[dev] = st;
  return VDC_OK;
}

int vdc_set_smem_size(int bytes) {
  if (bytes < 0 || (size_t)bytes > 232448) return fail_arg("shared-memory size beyond the 227 KB a B200 CTA can have");
  return VDC_OK;
}

static int launch_async_impl(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                             const void* tma_descs, int* bars, const int* bars_init, uint64_t* profile, uint64_t stream,
                             uint64_t timeout_ns, int ref_ops) {
  int dev;
  if (int r = current_device(&dev)) return r;
  if (int r = check_launch_args(dev, num_sms, insts_per_sm, compute_insts, memory_insts, bars, profile)) return r;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bars_init) {
    cudaError_t e = cudaMemcpyAsync(bars, bars_init, sizeof(int) * VDC_MAX_BARS, cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(bars)");
  }
  if (timeout_ns == 0) timeout_ns = 2000000000ull;
  cudaError_t e = vdc_megakernel_launch(num_sms, compute_insts, memory_insts, tma_descs, bars, profile,
                                        g_status[dev], insts_per_sm, timeout_ns, s, ref_ops);
  if (e != cudaSuccess) return fail_cuda(e, "megakernel launch");
  return VDC_OK;
}

// The decode engines' per-step launch: the kernel with the native operators only.
int vdc_launch_async(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                     const void* tma_descs, int* bars, const int* bars_init, uint64_t* profile, uint64_t stream,
                     uint64_t timeout_ns) {
  return launch_async_impl(num_sms, insts_per_sm, compute_insts, memory_insts, tma_descs, bars, bars_init, profile, stream,
                           timeout_ns, 0);
}

// The same without the synchronisation of vdc_launch, for the full kernel: the batched engines and the prefill
// run tasks (attention variants for long page walks) that the batch-1 kernel does not carry.
int vdc_launch_async_full(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                          const void* tma_descs, int* bars, const int* bars_init, uint64_t* profile, uint64_t stream,
                          uint64_t timeout_ns) {
  return launch_async_impl(num_sms, insts_per_sm, compute_insts, memory_insts, tma_descs, bars, bars_init, profile, stream,
                           timeout_ns, 1);
}

int vdc_read_status(uint64_t stream, vdc_status* status, int clear) {
  int dev;
  if (int r = current_device(&dev)) return r;
  if (!g_status[dev]) return fail_arg("vdc_init was not called on this device");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaStreamSynchronize");
  vdc_status h{};
  e = cudaMemcpy(&h, g_status[dev], sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpy(status)");
  if (clear && h.abort) {
    e = cudaMemset(g_status[dev], 0, sizeof(vdc_status));
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemset(status)");
  }
  if (status) *status = h;
  if (h.abort) {
    char buf[256];
    snprintf(buf, sizeof buf, "megakernel gave up: code=%d sm=%d role=%d pc=%d opcode=0x%x bar=%d aux=%d", h.code, h.sm,
             h.role, h.pc, h.opcode, h.bar, h.aux);
    g_err = buf;
    return h.code ? h.code : VDC_ERR_TIMEOUT;
  }
  return VDC_OK;
}

int vdc_launch(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
               const void* tma_descs, int* bars, uint64_t* profile, uint64_t stream, uint64_t timeout_ns,
               vdc_status* status) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize (before launch)");
  // the entry point behind the reference's launch_dae: the full kernel, which also runs its tile-contract operators
  if (int r = launch_async_impl(num_sms, insts_per_sm, compute_insts, memory_insts, tma_descs, bars, nullptr, profile,
                                stream, timeout_ns, 1))
    return r;
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize (after launch)");
  return vdc_read_status(stream, status, 1);
}

int vdc_build_tma_desc(void* out_desc, const void* base, int dtype, int rank, const uint64_t* shape,
                       const uint64_t* strides_bytes, const uint32_t* box_dim, const uint32_t* elem_strides,
                       int swizzle_bytes, int interleave_bytes) {
  if (!out_desc || !base || !shape || !box_dim || !elem_strides) return fail_arg("null argument");
  if (rank < 1 || rank > 5) return fail_arg("tensor-map rank must be 1..5");
  if ((uintptr_t)base & 15) return fail_arg("tensor-map base address must be 16-byte aligned");
  static const CUtensorMapDataType kTypes[] = {CU_TENSOR_MAP_DATA_TYPE_UINT8,   CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                               CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                               CU_TENSOR_MAP_DATA_TYPE_INT32,   CU_TENSOR_MAP_DATA_TYPE_UINT32};
  if (dtype < 0 || dtype > 5) return fail_arg("unsupported dtype code");
  CUtensorMapSwizzle swz;
  switch (swizzle_bytes) {
    case 0: swz = CU_TENSOR_MAP_SWIZZLE_NONE; break;
    case 32: swz = CU_TENSOR_MAP_SWIZZLE_32B; break;
    case 64: swz = CU_TENSOR_MAP_SWIZZLE_64B; break;
    case 128: swz = CU_TENSOR_MAP_SWIZZLE_128B; break;
    default: return fail_arg("swizzle_bytes must be 0, 32, 64 or 128");
  }
  CUtensorMapInterleave il;
  switch (interleave_bytes) {
    case 0: il = CU_TENSOR_MAP_INTERLEAVE_NONE; break;
    case 16: il = CU_TENSOR_MAP_INTERLEAVE_16B; break;
    case 32: il = CU_TENSOR_MAP_INTERLEAVE_32B; break;
    default: return fail_arg("interleave_bytes must be 0, 16 or 32");
  }
  cuuint64_t gdim[5] = {1, 1, 1, 1, 1}, gstride[5] = {0, 0, 0, 0, 0};
  cuuint32_t bdim[5] = {1, 1, 1, 1, 1}, estride[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    if (shape[i] == 0 || box_dim[i] == 0 || elem_strides[i] == 0) return fail_arg("shape, box and element strides must be positive");
    gdim[i] = shape[i];
    bdim[i] = box_dim[i];
    estride[i] = elem_strides[i];
    if (i < rank - 1) {
      if (!strides_bytes) return fail_arg("strides_bytes is required for rank > 1");
      gstride[i] = strides_bytes[i];
    }
  }
  // The driver entry point is resolved at run time so that the library has no
  // link-time dependency on libcuda (it must load on machines without a GPU).
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
      return fail_cuda(e == cudaSuccess ? cudaErrorNotSupported : e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    encode = reinterpret_cast<EncodeFn>(fn);
  }
  alignas(64) CUtensorMap map;
  CUresult r = encode(&map, kTypes[dtype], (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride, il,
                      swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    g_err = buf;
    return VDC_ERR_CUDA;
  }
  memcpy(out_desc, &map, sizeof(map));
  return VDC_OK;
}

int vdc_set_cache_policy(const void* ptr, size_t bytes, uint64_t stream, float hit_ratio, int hit_policy,
                         int miss_policy) {
  if (!ptr || bytes == 0) return fail_arg("empty range");
  int dev;
  if (int r = current_device(&dev)) return r;
  int max_window = 0;
  cudaError_t e = cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceGetAttribute");
  if (max_window > 0 && bytes > (size_t)max_window) bytes = (size_t)max_window;
  cudaStreamAttrValue attr{};
  attr.accessPolicyWindow.base_ptr = const_cast<void*>(ptr);
  attr.accessPolicyWindow.num_bytes = bytes;
  attr.accessPolicyWindow.hitRatio = hit_ratio;
  attr.accessPolicyWindow.hitProp = static_cast<cudaAccessProperty>(hit_policy);
  attr.accessPolicyWindow.missProp = static_cast<cudaAccessProperty>(miss_policy);
  e = cudaStreamSetAttribute(reinterpret_cast<cudaStream_t>(stream), cudaStreamAttributeAccessPolicyWindow, &attr);
  if (e != cudaSuccess) return fail_cuda(e, "cudaStreamSetAttribute");
  return VDC_OK;
}

int vdc_enable_peer_access(int peer_device) {
  int dev;
  if (int r = current_device(&dev)) return r;
  if (peer_device == dev) return VDC_OK;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceCanAccessPeer");
  if (!can) return fail_arg("the current device cannot map the peer's memory");
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();  // not an error for the caller: clear it
    return VDC_OK;
  }
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceEnablePeerAccess");
  return VDC_OK;
}

int vdc_peer_alloc(size_t bytes, uint64_t* out_ptr) {
  if (!out_ptr || bytes == 0) return fail_arg("bad peer allocation request");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);   // a block of its own: its IPC handle names exactly this allocation
  if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc(exchange block)");
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail_cuda(e, "cudaMemset(exchange block)");
  }
  *out_ptr = reinterpret_cast<uint64_t>(p);
  return VDC_OK;
}

int vdc_peer_free(uint64_t ptr) {
  cudaError_t e = cudaFree(reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) return fail_cuda(e, "cudaFree(exchange block)");
  return VDC_OK;
}

int vdc_ipc_export(uint64_t ptr, void* handle_out, size_t handle_bytes) {
  if (!ptr || !handle_out || handle_bytes != sizeof(cudaIpcMemHandle_t)) return fail_arg("bad IPC export request");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) return fail_cuda(e, "cudaIpcGetMemHandle");
  memcpy(handle_out, &h, sizeof(h));
  return VDC_OK;
}

int vdc_ipc_open(const void* handle, size_t handle_bytes, uint64_t* out_ptr) {
  if (!handle || !out_ptr || handle_bytes != sizeof(cudaIpcMemHandle_t)) return fail_arg("bad IPC handle");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  // opened with the importing device current: the mapping is made for this device, peer access
  // to the exporting device is enabled as needed
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail_cuda(e, "cudaIpcOpenMemHandle");
  *out_ptr = reinterpret_cast<uint64_t>(p);
  return VDC_OK;
}

int vdc_ipc_close(uint64_t ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) return fail_cuda(e, "cudaIpcCloseMemHandle");
  return VDC_OK;
}

int vdc_opcode_count(void) { return kNumOps; }
const char* vdc_opcode_name(int i) { return (i >= 0 && i < kNumOps) ? kOps[i].name : nullptr; }
int vdc_opcode_value(int i) { return (i >= 0 && i < kNumOps) ? kOps[i].value : -1; }
int vdc_opcode_is_compute(int i) { return (i >= 0 && i < kNumOps) ? kOps[i].is_compute : 0; }

namespace {
const OpEntry* find_op(int value, int is_compute) {
  for (int i = 0; i < kNumOps; ++i)
    if (kOps[i].is_compute == is_compute && kOps[i].value == value) return &kOps[i];
  return nullptr;
}
int fail_stream(int code, const char* stream, int sm, int pc, int opcode, const char* what, int* bad_sm, int* bad_pc) {
  static thread_local char msg[160];
  snprintf(msg, sizeof msg, "%s stream of SM %d, instruction %d (opcode 0x%04x): %s", stream, sm, pc, opcode, what);
  g_err = msg;
  if (bad_sm) *bad_sm = sm;
  if (bad_pc) *bad_pc = pc;
  return code;
}
}  // namespace

int vdc_validate_streams(int num_sms, int insts_per_sm, const void* compute_insts_host, const void* memory_insts_host,
                         int* bad_sm, int* bad_pc) {
  if (bad_sm) *bad_sm = -1;
  if (bad_pc) *bad_pc = -1;
  if (num_sms <= 0 || num_sms > VDC_MAX_SMS) return fail_arg("num_sms out of range");
  // VDC_MAX_INSTS is the ring the reference fixes; the native engines size theirs to the program, and the only
  // limit of the wire format is the 16-bit jump target
  if (insts_per_sm <= 0 || insts_per_sm > 65536) return fail_arg("insts_per_sm out of range");
  if (!compute_insts_host || !memory_insts_host) return fail_arg("null instruction stream");
  const VdcCInst* C = static_cast<const VdcCInst*>(compute_insts_host);
  const VdcMInst* M = static_cast<const VdcMInst*>(memory_insts_host);
  for (int sm = 0; sm < num_sms; ++sm) {
    // compute stream: walk instruction by instruction (the counts of the table plus the trailing words the
    // flags of the first word announce), until TERMINATEC
    const VdcCInst* c = C + (size_t)sm * insts_per_sm;
    bool ended = false;
    for (int pc = 0; pc < insts_per_sm;) {
      const int op = c[pc].opcode;
      const OpEntry* e = find_op(op, 1);
      if (!e || op == 0x7FFF)
        return fail_stream(VDC_ERR_BAD_OPCODE, "compute", sm, pc, op, e ? "continuation word where an instruction starts" : "unknown opcode", bad_sm, bad_pc);
      int words = e->words;
      if (op >= 0x7200 && op <= 0x7203) {
        const int f = c[pc].args[1], R = f & 31;
        if (R != 1 && R != 2 && R != 4 && R != 8 && R != 16)
          return fail_stream(VDC_ERR_ARG, "compute", sm, pc, op, "rows per chunk must be 1, 2, 4, 8 or 16", bad_sm, bad_pc);
        words += ((f & VDC_GEMV_STRIDE_BIT) ? 1 : 0) + ((f & VDC_GEMV_PARTIAL_BIT) ? 1 : 0) +
                 ((f & VDC_GEMV_PEERS_BIT) ? 2 : 0) + ((f & VDC_GEMV_DYNROWS_BIT) ? 1 : 0);
      }
      if (op == 0x7220 && c[pc].args[1] == 2) words += 2;
      if (pc + words > insts_per_sm)
        return fail_stream(VDC_ERR_ARG, "compute", sm, pc, op, "instruction runs past the end of the stream", bad_sm, bad_pc);
      for (int k = 1; k < words; ++k)
        if (c[pc + k].opcode != 0x7FFF)
          return fail_stream(VDC_ERR_BAD_OPCODE, "compute", sm, pc + k, c[pc + k].opcode, "continuation word expected", bad_sm, bad_pc);
      if (op == 0x7001 && c[pc].args[1] >= pc)
        return fail_stream(VDC_ERR_ARG, "compute", sm, pc, op, "loop target is not an earlier instruction", bad_sm, bad_pc);
      if (op == 0x7000) {
        ended = true;
        break;
      }
      pc += words;
    }
    if (!ended) return fail_stream(VDC_ERR_ARG, "compute", sm, insts_per_sm, 0, "no TERMINATEC", bad_sm, bad_pc);
    // memory stream: every word is an instruction; known id, the table's ALLOCATE bit, a slot
    // request the pool can serve, backward jumps, and a TERMINATE
    const VdcMInst* m = M + (size_t)sm * insts_per_sm;
    ended = false;
    for (int pc = 0; pc < insts_per_sm; ++pc) {
      const int op = m[pc].opcode, id = op >> VDC_FLAG_BITS;
      const OpEntry* e = nullptr;
      for (int i = 0; i < kNumOps && !e; ++i)
        if (!kOps[i].is_compute && (kOps[i].value >> VDC_FLAG_BITS) == id) e = &kOps[i];
      if (!e) return fail_stream(VDC_ERR_BAD_OPCODE, "memory", sm, pc, op, "unknown opcode", bad_sm, bad_pc);
      if ((e->value & VDC_F_ALLOCATE) != (op & VDC_F_ALLOCATE))
        return fail_stream(VDC_ERR_BAD_OPCODE, "memory", sm, pc, op, "ALLOCATE flag does not fit the opcode", bad_sm, bad_pc);
      if ((op & VDC_F_ALLOCATE) && (m[pc].num_slots & 63) >= VDC_NUM_SLOTS + VDC_NUM_SPECIAL_SLOTS)
        return fail_stream(VDC_ERR_ARG, "memory", sm, pc, op, "slot request or special slot id out of range", bad_sm, bad_pc);
      if (id == 3 && m[pc].coords[0] >= pc)
        return fail_stream(VDC_ERR_ARG, "memory", sm, pc, op, "loop target is not an earlier instruction", bad_sm, bad_pc);
      if (id == 1) {
        ended = true;
        break;
      }
    }
    if (!ended) return fail_stream(VDC_ERR_ARG, "memory", sm, insts_per_sm, 0, "no TERMINATE", bad_sm, bad_pc);
  }
  return VDC_OK;
}

int64_t vdc_config(const char* name) {
  if (!name) return -1;
  struct {
    const char* k;
    int64_t v;
  } const tbl[] = {{"slot_size", VDC_SLOT_BYTES},
                   {"num_slots", VDC_NUM_SLOTS},
                   {"max_insts", VDC_MAX_INSTS},
                   {"num_profile_events", VDC_NUM_PROFILE_EVENTS},
                   {"max_tmas", VDC_MAX_TMAS},
                   {"max_bars", VDC_MAX_BARS},
                   {"num_special_slots", VDC_NUM_SPECIAL_SLOTS},
                   {"compute_threads", VDC_COMPUTE_THREADS},
                   {"threads", VDC_THREADS},
                   {"kv_page", VDC_KV_PAGE},
                   {"head_dim", VDC_HEAD_DIM},
                   {"dynamic_smem", (int64_t)vdc_megakernel_dynamic_smem()}};
  for (auto& e : tbl)
    if (strcmp(e.k, name) == 0) return e.v;
  return -1;
}

// Families of parameterised compute ops, in the reference's definition syntax (include/dae/opcode.cuh.inc:36-37).
const char* vdc_family_specs(void) {
  return "GEMV_WGMMA\tFIELDS=M|N|K|BLOAD|RESIDUAL, M_MULTIPLE=64, N_FIXED=8, K_MULTIPLE=16, BLOAD_MIN=1, RESIDUAL_MAX=1\n"
         "GEMV_MMA\tFIELDS=M|N|K, M_FIXED=64, N_FIXED=8, K_MULTIPLE=16";
}

// ------------------------------------------------------------------------- //
// launch without any allocation
// ------------------------------------------------------------------------- //
// Scratch of vdc_launch_static: status block, countdown barriers and per-SM
// profile rows live in this file-scope device array, so the call needs neither
// vdc_init's cudaMalloc nor caller-provided scratch.  Every GPU that loads the
// library holds these 164 KB until the process exits.
#define VDC_STATIC_MAX_SMS 160
#define VDC_STATIC_STATUS_OFF 0
#define VDC_STATIC_BARS_OFF 256
#define VDC_STATIC_PROFILE_OFF (256 + 4 * VDC_MAX_BARS)
#define VDC_STATIC_BYTES (VDC_STATIC_PROFILE_OFF + 8 * VDC_NUM_PROFILE_EVENTS * VDC_STATIC_MAX_SMS)
static __device__ __align__(256) unsigned char g_static_scratch[VDC_STATIC_BYTES];

namespace {
unsigned char* g_static_ptr[kMaxDevices] = {nullptr};  // device address of g_static_scratch, per device
int g_static_sms[kMaxDevices] = {0};
}  // namespace

int vdc_launch_static(int num_sms, int insts_per_sm, const void* compute_insts, const void* memory_insts,
                      const void* tma_descs, const int* bars_init, uint64_t stream, uint64_t timeout_ns,
                      vdc_status* status) {
  int dev;
  if (int r = current_device(&dev)) return r;
  if (!g_static_ptr[dev]) {
    // Set-up, once per device, with that device current.  In host code the
    // array's name is only a stand-in; the device address comes from the runtime.
    int sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceGetAttribute(MultiProcessorCount)");
    e = vdc_megakernel_prepare();
    if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
    g_static_ptr[dev] = static_cast<unsigned char*>(p);
    g_static_sms[dev] = sms;
  }
  if (num_sms > VDC_STATIC_MAX_SMS)
    return fail_arg("vdc_launch_static: the static scratch holds profile rows for at most 160 SMs");
  if (num_sms <= 0 || num_sms > g_static_sms[dev]) return fail_arg("num_sms must be in [1, SM count of the device]");
  if (insts_per_sm <= 0 || insts_per_sm > 65536) return fail_arg("insts_per_sm out of range");
  if (!compute_insts || !memory_insts || !bars_init) return fail_arg("null instruction or barrier-image pointer");
  if (((uintptr_t)compute_insts & 7) || ((uintptr_t)memory_insts & 15) || ((uintptr_t)bars_init & 3))
    return fail_arg("misaligned instruction or barrier-image pointer");
  unsigned char* base = g_static_ptr[dev];
  vdc_status* d_status = reinterpret_cast<vdc_status*>(base + VDC_STATIC_STATUS_OFF);
  int* d_bars = reinterpret_cast<int*>(base + VDC_STATIC_BARS_OFF);
  uint64_t* d_profile = reinterpret_cast<uint64_t*>(base + VDC_STATIC_PROFILE_OFF);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the array keeps the previous call's contents: the status must start at zero,
  // the barriers at the caller's counts; the profile rows stay internal (the kernel writes only its start / end
  // stamps and the traced task pairs into them, nothing reads the rest)
  cudaError_t e = cudaMemsetAsync(d_status, 0, sizeof(vdc_status), s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(status)");
  e = cudaMemcpyAsync(d_bars, bars_init, sizeof(int) * VDC_MAX_BARS, cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(bars)");
  if (timeout_ns == 0) timeout_ns = 2000000000ull;
  e = vdc_megakernel_launch(num_sms, compute_insts, memory_insts, tma_descs, d_bars, d_profile, d_status, insts_per_sm,
                            timeout_ns, s, 1);   // an embedder's streams may hold any operator: the full kernel
  if (e != cudaSuccess) return fail_cuda(e, "megakernel launch");
  vdc_status h{};
  e = cudaMemcpyAsync(&h, d_status, sizeof(h), cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(status)");
  e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaStreamSynchronize");
  if (status) *status = h;
  if (h.abort) {
    char buf[256];
    snprintf(buf, sizeof buf, "megakernel gave up: code=%d sm=%d role=%d pc=%d opcode=0x%x bar=%d aux=%d", h.code, h.sm,
             h.role, h.pc, h.opcode, h.bar, h.aux);
    g_err = buf;
    return h.code ? h.code : VDC_ERR_TIMEOUT;
  }
  return VDC_OK;
}

}  // extern "C"
