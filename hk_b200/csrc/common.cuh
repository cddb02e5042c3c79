// Shared helpers of the sm_100a kernels: element conversion, warp reductions and the
// C-ABI conventions every entry point follows.
//
// Conventions: an entry point takes raw device pointers, sizes and the CUDA stream to
// launch on; it returns 0 or a cudaError_t value (never throws, never synchronises,
// never allocates).  `dtype` arguments are HK_F32 (0) or HK_BF16 (1).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define HK_F32 0
#define HK_BF16 1
// Returned (instead of a cudaError_t) when an entry point refuses its arguments.
#define HK_ERR_UNSUPPORTED 100001

#define HK_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

static inline int hk_launch_status() { return (int)cudaGetLastError(); }

// Dynamic shared memory above 48 KB has to be allowed per kernel on every device that runs it.  A launcher keeps a
// `static HkSmemCache` per kernel: the largest size allowed so far on each device (devices beyond the table are
// set on every launch).  Returns 0 or a cudaError_t.
#define HK_MAX_DEVICES 64
struct HkSmemCache {
  size_t allowed[HK_MAX_DEVICES];
};
template <typename K>
static inline int hk_allow_smem(K kernel, size_t smem, HkSmemCache& cache) {
  if (smem <= 48 * 1024) return 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  const bool known = dev >= 0 && dev < HK_MAX_DEVICES;
  if (known && smem <= cache.allowed[dev]) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  if (known) cache.allowed[dev] = smem;
  return 0;
}

// A launch through cudaLaunchKernelEx (full stream order).
template <typename... KArgs, typename... Args>
static inline int hk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
