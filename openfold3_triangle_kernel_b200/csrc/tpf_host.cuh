// Host-side helpers shared by the translation units of the C-ABI library:
// error reporting, TMA descriptor encoding (driver entry point resolved at run
// time, so the library loads on machines without a CUDA driver), launch checks.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "../../include/tpf_b200.h"  // TPF_OK / TPF_ERR_* codes

namespace tpf {


char* last_error_buffer();  // thread-local, 512 bytes (defined in tpf_cabi.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define TPF_REQUIRE(cond, code, ...)                  \
  do {                                                \
    if (!(cond)) return ::tpf::fail(code, __VA_ARGS__); \
  } while (0)

#define TPF_CUDA_OK(expr)                                                                             \
  do {                                                                                                \
    cudaError_t _e = (expr);                                                                          \
    if (_e != cudaSuccess)                                                                            \
      return ::tpf::fail(TPF_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                         __FILE__, __LINE__);                                                         \
  } while (0)

// Number of kernel launches this process has issued through the library (all host threads).
inline std::atomic<long long>& launch_counter() {
  static std::atomic<long long> n{0};
  return n;
}

// Every kernel of the library is launched with programmatic stream serialization: the launch is set up
// while the preceding kernel of the stream still runs, and the kernel itself holds at `griddep_wait()`
// (its first statement that can touch global memory) until that kernel has completed and its writes are
// visible.  Results are those of plain stream order; the launch latency between dependent kernels is hidden.
template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);  // the error is read by TPF_LAUNCH_OK()
}

// After every launch_kernel(...): count the launch and surface a launch error.
#define TPF_LAUNCH_OK()                          \
  do {                                           \
    ::tpf::launch_counter().fetch_add(1);        \
    TPF_CUDA_OK(cudaGetLastError());             \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

inline CUtensorMapSwizzle swizzle_enum(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                      : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                    : bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
}

// Encode a tiled tensor map of rank `rank` (2..5).  dims[0] is the
// contiguous dimension; strides_bytes[i] is the byte stride of dims[i+1].
inline int make_tmap(CUtensorMap* out, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  TPF_REQUIRE(fn != nullptr, TPF_ERR_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  TPF_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, TPF_ERR_INVALID_ARGUMENT,
              "tensor base address must be 16-byte aligned");
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i + 1 < rank) {
      s[i] = strides_bytes[i];
      TPF_REQUIRE((s[i] & 15) == 0, TPF_ERR_INVALID_ARGUMENT, "tensor stride %d (%llu bytes) must be a multiple of 16",
                  i + 1, (unsigned long long)s[i]);
    }
  }
  CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPF_REQUIRE(r == CUDA_SUCCESS, TPF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TPF_OK;
}

inline int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box, swizzle_bytes);
}
inline int make_tmap_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box, 0);
}

// ---- per-device host state --------------------------------------------------------------
// Function attributes, symbol addresses and the SM count belong to a device, not to the process;
// a process may drive several GPUs from several host threads.  Each cache below is a small table
// indexed by device ordinal whose entries are published with release / acquire ordering (two
// threads that race on the first use both do the idempotent set-up, then one flag store wins).
constexpr int kMaxDevices = 64;

inline int current_device(int* dev) {
  TPF_CUDA_OK(cudaGetDevice(dev));
  TPF_REQUIRE(*dev >= 0 && *dev < kMaxDevices, TPF_ERR_UNSUPPORTED, "device ordinal %d out of range", *dev);
  return TPF_OK;
}

struct PerDeviceOnce {
  std::atomic<bool> done[kMaxDevices];
};

// cudaFuncAttributeMaxDynamicSharedMemorySize for `kern` on the current device, once per device.
template <class Kernel>
inline int ensure_dynamic_smem(Kernel kern, int bytes, PerDeviceOnce& once) {
  int dev = 0;
  int rc = current_device(&dev);
  if (rc) return rc;
  if (once.done[dev].load(std::memory_order_acquire)) return TPF_OK;
  TPF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  once.done[dev].store(true, std::memory_order_release);
  return TPF_OK;
}

// Device address of a __device__ symbol on the current device, looked up once per device.
struct PerDeviceAddress {
  std::atomic<void*> addr[kMaxDevices];
};
template <class Symbol>
inline int device_symbol_address(const Symbol& sym, PerDeviceAddress& cache, void** out) {
  int dev = 0;
  int rc = current_device(&dev);
  if (rc) return rc;
  void* p = cache.addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    TPF_CUDA_OK(cudaGetSymbolAddress(&p, sym));
    TPF_REQUIRE(p != nullptr, TPF_ERR_CUDA, "symbol address lookup returned NULL");
    cache.addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return TPF_OK;
}

inline int sm_count() {
  static std::atomic<int> table[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = table[dev].load(std::memory_order_acquire);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  table[dev].store(n, std::memory_order_release);
  return n;
}

#define TPF_REQUIRE_ALIGNED16(ptr, who, name)                                                       \
  TPF_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, TPF_ERR_INVALID_ARGUMENT,               \
              "%s: %s must be 16-byte aligned", who, name)

}  // namespace tpf
