// Weight-streaming bf16 matrix product for few rows (decode): out[M, N] (fp32) = a[M, K] * w[N, K]^T,
// M <= 64.  The step is bound by reading w once from HBM, so the kernel is built around 16-byte loads of
// w that go straight from global memory into tensor-core fragments:
//
//   * a CTA owns RT*16 consecutive rows of w; its 8 warps split K among themselves;
//   * mma.sync.m16n8k16 with the roles swapped: 16 rows of w are the "M" side, 8 tokens the "N" side.
//     A lane loads 16 bytes (8 consecutive k) of w row g (and g + 8) and the same 8 k of token g; the two
//     MMAs that consume them pair slot with slot, so any k order is fine as long as both sides agree;
//   * the 8 partial sums meet in shared memory and are added in warp order (deterministic), then stored
//     or added onto `out` (the residual sum).
// The activations are tiny and come from L2; tokens beyond M and rows beyond N are clamped on load and
// skipped on store.  Needs K % 8 == 0 and 16-byte aligned a and w.
//
// Reference counterpart: `gemv_bf16` (warp per row, 16-byte loads, one token), src/cuda_device.zig:1294-1351.
#include "common.cuh"

namespace {

constexpr int SM_WARPS = 8;
constexpr int KCHUNK = 64;

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// MT: token tiles of 8 (M <= 8*MT).  RT: row tiles of 16 per CTA.
template <int MT, int RT, bool ADD>
__global__ void __launch_bounds__(SM_WARPS * 32)
gemm_smallm_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, float* __restrict__ out, int M, int N, int K,
                   long long ldo) {
  extern __shared__ float red[];   // [SM_WARPS][RT*16][MT*8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = (int)blockIdx.x * (RT * 16);

  float acc[RT][MT][4];
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;

  // this warp's share of the 64-wide chunks of K (the CTA's warps cut K evenly)
  const int chunks = (K + KCHUNK - 1) / KCHUNK;
  const int c_begin = (int)((long long)chunks * warp / SM_WARPS);
  const int c_end = (int)((long long)chunks * (warp + 1) / SM_WARPS);

  const bf16* wrow[RT][2];
#pragma unroll
  for (int r = 0; r < RT; ++r) {
    wrow[r][0] = w + (size_t)min(n0 + r * 16 + g, N - 1) * K;
    wrow[r][1] = w + (size_t)min(n0 + r * 16 + g + 8, N - 1) * K;
  }
  const bf16* arow[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) arow[j] = a + (size_t)min(j * 8 + g, M - 1) * K;

  // Two chunks of weights are always on their way while a third is multiplied.
  uint4 wf[2][RT][2][2];   // [buffer][row tile][row g / g+8][k half of the chunk]
  auto load_w = [&](int c, int b) {
    const int k0 = c * KCHUNK + t * 8;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
          const int k = k0 + kh * 32;
          wf[b][r][h][kh] = k < K ? ldg_stream(wrow[r][h] + k) : make_uint4(0, 0, 0, 0);
        }
  };
  auto multiply = [&](int c, uint4 (&cur)[RT][2][2]) {
    const int k0 = c * KCHUNK + t * 8;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int kh = 0; kh < 2; ++kh) {
        const int k = k0 + kh * 32;
        uint4 x = k < K ? *reinterpret_cast<const uint4*>(arow[j] + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < RT; ++r) {
          // first MMA: elements 0..3 of the 8 loaded k; second: elements 4..7
          uint32_t a0[4] = {cur[r][0][kh].x, cur[r][1][kh].x, cur[r][0][kh].y, cur[r][1][kh].y};
          mma_bf16_16816(acc[r][j], a0, x.x, x.y);
          uint32_t a1[4] = {cur[r][0][kh].z, cur[r][1][kh].z, cur[r][0][kh].w, cur[r][1][kh].w};
          mma_bf16_16816(acc[r][j], a1, x.z, x.w);
        }
      }
    }
  };

  // The weights do not depend on the kernel before: the first chunks are on their way before this kernel
  // waits for that kernel's output (the activations).
  if (c_begin < c_end) load_w(c_begin, 0);
  if (c_begin + 1 < c_end) load_w(c_begin + 1, 1);
  pdl_wait();
  for (int c = c_begin; c < c_end; c += 2) {
    uint4 cur[RT][2][2];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) cur[r][h][kh] = wf[0][r][h][kh];
    if (c + 2 < c_end) load_w(c + 2, 0);
    multiply(c, cur);
    if (c + 1 < c_end) {
#pragma unroll
      for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int kh = 0; kh < 2; ++kh) cur[r][h][kh] = wf[1][r][h][kh];
      if (c + 3 < c_end) load_w(c + 3, 1);
      multiply(c + 1, cur);
    }
  }

  pdl_launch_dependents();   // the weights are read: the next kernel may move in beside the reduction
  // accumulator layout: c0,c1 -> (row g, tokens 2t, 2t+1); c2,c3 -> (row g+8, tokens 2t, 2t+1)
  constexpr int ROWS = RT * 16, COLS = MT * 8;
  float* mine = red + (size_t)warp * ROWS * COLS;
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int col = j * 8 + 2 * t;
      mine[(r * 16 + g) * COLS + col] = acc[r][j][0];
      mine[(r * 16 + g) * COLS + col + 1] = acc[r][j][1];
      mine[(r * 16 + g + 8) * COLS + col] = acc[r][j][2];
      mine[(r * 16 + g + 8) * COLS + col + 1] = acc[r][j][3];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < ROWS * COLS; i += SM_WARPS * 32) {
    const int row = i % ROWS, m = i / ROWS;    // rows fastest: consecutive threads write consecutive floats
    if (m >= M || n0 + row >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < SM_WARPS; ++wv) s += red[(size_t)wv * ROWS * COLS + row * COLS + m];
    float* o = out + (size_t)m * ldo + n0 + row;
    *o = ADD ? *o + s : s;
  }
}

template <int MT, int RT>
int launch(const void* a, const void* w, float* out, int M, int N, int K, long long ldo, int add, cudaStream_t s) {
  const size_t smem = (size_t)SM_WARPS * RT * 16 * MT * 8 * sizeof(float);
  static HkSmemCache allowed_store = {}, allowed_add = {};
  if (int e = hk_allow_smem(gemm_smallm_kernel<MT, RT, false>, smem, allowed_store)) return e;
  if (int e = hk_allow_smem(gemm_smallm_kernel<MT, RT, true>, smem, allowed_add)) return e;
  const unsigned grid = (unsigned)((N + RT * 16 - 1) / (RT * 16));
  // launched so that it may start while the kernel before it drains: its first weights are on their way before it
  // waits for that kernel's output (0.8 microseconds a launch, measured over a decode step)
  if (add)
    return hk_launch_pdl(gemm_smallm_kernel<MT, RT, true>, dim3(grid), dim3(SM_WARPS * 32), smem, s, (const bf16*)a, (const bf16*)w,
                         out, M, N, K, ldo);
  return hk_launch_pdl(gemm_smallm_kernel<MT, RT, false>, dim3(grid), dim3(SM_WARPS * 32), smem, s, (const bf16*)a, (const bf16*)w,
                       out, M, N, K, ldo);
}

}  // namespace

// rt: row tiles of 16 per CTA (1, 2 or 4).  Refuses (HK_ERR_UNSUPPORTED) M > 64, K % 8 != 0, unaligned operands.
HK_API int hk_gemm_smallm(const void* a, const void* w, float* out, int M, int N, int K, long long ldo, int add, int rt,
                          void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const int mt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
#define HK_CASE(MT, RT) \
  if (mt == MT && rt == RT) return launch<MT, RT>(a, w, out, M, N, K, ldo, add, s);
  HK_CASE(1, 1) HK_CASE(1, 2) HK_CASE(1, 4)
  HK_CASE(2, 1) HK_CASE(2, 2) HK_CASE(2, 4)
  HK_CASE(4, 1) HK_CASE(4, 2)
  HK_CASE(8, 1) HK_CASE(8, 2)
#undef HK_CASE
  return HK_ERR_UNSUPPORTED;
}
