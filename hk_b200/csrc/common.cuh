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

// Programmatic dependent launch.  Measured over a decode step of the 8B layer sizes at batch 8 (4.28 ms with plain
// launches): the small-M product alone 4.26; + RMS norm 4.25; + the fused norm/rotation/cache write 4.24; + the TMA-fed
// decode attention 4.18; + the streaming product 4.17; the split-key combine launched this way made the step 4.58 (it
// moves in when the attention kernel says its keys are read, and then sits on the SMs), so that one stays a plain
// launch.  A kernel launched with `hk_launch_pdl` may start while the kernel before it
// in the stream is still running; it must call `pdl_wait()` before it reads or writes anything that an
// earlier kernel of the stream touches (what it may do before: set up shared memory, read weights and the
// step's host-written tables).  `pdl_launch_dependents()` lets the NEXT kernel start its own prologue early.
// Without the launch attribute both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A plain launch through the same interface (full stream order).
template <typename... KArgs, typename... Args>
static inline int hk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
static inline int hk_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
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
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
