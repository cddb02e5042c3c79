// Generic matrix product for every shape: out[M, N] (fp32) = a[M, K] * w[N, K]^T, optionally
// added onto what `out` holds (the residual sum).  Operands are float (the true 32-bit path:
// plain FMA, no reduced-precision matrix mode) or bf16 (the fallback of the serving path for
// shapes the tensor-core kernels refuse).  Each output element accumulates k = 0..K-1 in
// order in one fp32 register, so a row's result does not depend on M or on the tile it is in.
//
// Reference counterpart: `gemm_<fmt>` tiled kernel, src/cuda_device.zig:237-285.
#include "common.cuh"

#define GG_BM 64
#define GG_BN 64
#define GG_BK 16

template <typename T>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const T* __restrict__ a, const T* __restrict__ w, float* __restrict__ out, int M,
                    int N, int K, long long lda, long long ldw, long long ldo, int accumulate) {
  __shared__ float As[GG_BK][GG_BM + 4];
  __shared__ float Ws[GG_BK][GG_BN + 4];
  int tid = threadIdx.x;
  int m0 = blockIdx.y * GG_BM, n0 = blockIdx.x * GG_BN;
  int tx = tid & 15, ty = tid >> 4;  // thread computes rows ty*4.., cols tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int i = tid + j * 256;
      int r = i >> 4, c = i & 15;
      int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32<T>(a[(size_t)gm * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? to_f32<T>(w[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GG_BK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* o = out + (size_t)gm * ldo + gn;
      *o = accumulate ? *o + acc[i][j] : acc[i][j];
    }
  }
}

HK_API int hk_gemm_generic(const void* a, const void* w, int dtype, float* out, int M, int N, int K,
                           long long lda, long long ldw, long long ldo, int accumulate, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((N + GG_BN - 1) / GG_BN, (M + GG_BM - 1) / GG_BM);
  if (grid.y > 65535) return HK_ERR_UNSUPPORTED;
  if (dtype == HK_F32)
    gemm_generic_kernel<float><<<grid, 256, 0, s>>>((const float*)a, (const float*)w, out, M, N, K, lda,
                                                   ldw, ldo, accumulate);
  else if (dtype == HK_BF16)
    gemm_generic_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)a, (const bf16*)w, out, M, N, K, lda, ldw,
                                                  ldo, accumulate);
  else
    return HK_ERR_UNSUPPORTED;
  return hk_launch_status();
}
