// Generic attention over the paged cache, for every head size, group size and window, in
// float (the true 32-bit path) or bf16 storage with fp32 arithmetic.
//
// One block per (token, query head).  The token at position p of request slot s reads keys
// j in [max(0, p - window + 1), p] (window <= 0: all of [0, p]) through the slot's block table;
// its own key was written by the cache-write kernel earlier in the same step.  Four warps take
// the keys round-robin, each keeping an online softmax state (max, sum, weighted values); the
// four states are merged in a fixed order.  Nothing depends on which other tokens are in the
// batch, so the result at a position is the same under every way of cutting the work.
//
// Reference counterpart: `attention`, src/cuda_device.zig:1494-1594 (block per (token, head),
// warp per position, online softmax); scale on q first: src/engine/attention_kernel.zig:109.
#include <math_constants.h>

#include "common.cuh"

#define AG_WARPS 4
#define AG_MAX_PER_LANE 8  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ block_table,
                         int table_stride, const int* __restrict__ positions,
                         const int* __restrict__ slot_of_token, T* __restrict__ out, int H, int G, int hd,
                         int page_tokens, int window, float scale) {
  extern __shared__ float smem[];  // [AG_WARPS][hd] values, then [AG_WARPS] max, [AG_WARPS] sum
  float* acc_s = smem;
  float* m_s = smem + AG_WARPS * hd;
  float* l_s = m_s + AG_WARPS;

  int t = blockIdx.x / H, h = blockIdx.x % H;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int g = h / (H / G);
  int pos = positions[t];
  const int* bt = block_table + (size_t)slot_of_token[t] * table_stride;
  int lo = window > 0 ? max(0, pos - window + 1) : 0;

  float qr[AG_MAX_PER_LANE], acc[AG_MAX_PER_LANE];
  const T* qp = q + ((size_t)t * H + h) * hd;
#pragma unroll
  for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
    int d = lane + 32 * i;
    qr[i] = d < hd ? to_f32<T>(qp[d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -CUDART_INF_F, l = 0.f;
  for (int j = lo + wid; j <= pos; j += AG_WARPS) {
    int page = bt[j / page_tokens];
    if (page < 0) continue;  // never scheduled by the host; keeps the reads in bounds
    size_t off = (((size_t)page * G + g) * page_tokens + (j % page_tokens)) * hd;
    const T* kp = k_pages + off;
    const T* vp = v_pages + off;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
      int d = lane + 32 * i;
      if (d < hd) s = fmaf(qr[i], to_f32<T>(kp[d]), s);
    }
    s = warp_sum(s);
    float mn = fmaxf(m, s);
    float corr = expf(m - mn);
    float p = expf(s - mn);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
      int d = lane + 32 * i;
      if (d < hd) acc[i] = acc[i] * corr + p * to_f32<T>(vp[d]);
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
    int d = lane + 32 * i;
    if (d < hd) acc_s[wid * hd + d] = acc[i];
  }
  if (lane == 0) {
    m_s[wid] = m;
    l_s[wid] = l;
  }
  __syncthreads();
  float mm = m_s[0];
#pragma unroll
  for (int w = 1; w < AG_WARPS; ++w) mm = fmaxf(mm, m_s[w]);
  float f[AG_WARPS], lt = 0.f;
#pragma unroll
  for (int w = 0; w < AG_WARPS; ++w) {
    f[w] = m_s[w] == -CUDART_INF_F ? 0.f : expf(m_s[w] - mm);
    lt += l_s[w] * f[w];
  }
  T* op = out + ((size_t)t * H + h) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < AG_WARPS; ++w) a += acc_s[w * hd + d] * f[w];
    op[d] = from_f32<T>(a / lt);
  }
}

HK_API int hk_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                const int* block_table, int table_stride, const int* positions,
                                const int* slot_of_token, void* out, int n, int H, int G, int hd,
                                int page_tokens, int window, float scale, void* stream) {
  if (n <= 0) return 0;
  if (hd > 32 * AG_MAX_PER_LANE || hd < 1 || G < 1 || H % G != 0) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  size_t smem = (size_t)(AG_WARPS * hd + 2 * AG_WARPS) * sizeof(float);
  unsigned blocks = (unsigned)((long long)n * H);
  if (dtype == HK_F32)
    attention_generic_kernel<float><<<blocks, AG_WARPS * 32, smem, s>>>(
        (const float*)q, (const float*)k_pages, (const float*)v_pages, block_table, table_stride, positions,
        slot_of_token, (float*)out, H, G, hd, page_tokens, window, scale);
  else if (dtype == HK_BF16)
    attention_generic_kernel<bf16><<<blocks, AG_WARPS * 32, smem, s>>>(
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, table_stride, positions,
        slot_of_token, (bf16*)out, H, G, hd, page_tokens, window, scale);
  else
    return HK_ERR_UNSUPPORTED;
  return hk_launch_status();
}
