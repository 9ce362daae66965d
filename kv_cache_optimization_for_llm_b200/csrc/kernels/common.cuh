// Shared by every kernel module: element types, conversions, error reporting.
//
// Every exported launcher has C linkage, takes raw device pointers, sizes and the
// stream to launch on, and returns 0 or a negative KVB_ERR_* / positive cudaError_t.
// Nothing here allocates.  A kernel that meets an impossible index (an unmapped
// page, a position beyond its table) records a code in the caller's status word and
// skips the access instead of trapping, so the context stays usable.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KVB_EXPORT extern "C" __attribute__((visibility("default")))

enum KvbDtype { KVB_F32 = 0, KVB_BF16 = 1 };

enum KvbErr {
  KVB_ERR_BAD_DTYPE = -1,
  KVB_ERR_BAD_SIZE = -2,   // a size the kernel refuses (see the launcher's comment)
  KVB_ERR_ALIGN = -3,
};

// Codes a kernel may leave in the status word.
enum KvbStatus {
  KVB_STATUS_OK = 0,
  KVB_STATUS_UNMAPPED_PAGE = 1,
  KVB_STATUS_BAD_POSITION = 2,
  KVB_STATUS_BAD_TOKEN = 3,
  KVB_STATUS_WAIT_TIMEOUT = 4,
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch: a kernel launched through kvb_launch may be set up
// on the SMs while its predecessor in the stream still runs.  pdl_trigger() at the
// top of a kernel lets the next one begin that early; pdl_wait() holds a kernel until
// everything before it in the stream has finished and its writes are visible, so it
// comes before the first read of data that an earlier kernel produced and before the
// first write to global memory.  Both are no-ops for a kernel launched the plain way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#include <cstdlib>
#include <utility>

static inline bool kvb_pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("KVB200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t kvb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kvb_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// SMs of the current device, asked once per device: what launchers size their grids by.
static inline int kvb_sm_count() {
  static int count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    count[dev] = n;
  }
  return count[dev];
}

static inline int kvb_launch_result() {
  cudaError_t e = cudaPeekAtLastError();
  return (int)e;
}

#define KVB_DISPATCH_DTYPE(dtype, T, ...)                    \
  switch (dtype) {                                           \
    case KVB_F32: { using T = float; __VA_ARGS__; break; }   \
    case KVB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    default: return KVB_ERR_BAD_DTYPE;                       \
  }
