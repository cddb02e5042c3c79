// bf16 matrix product on the 5th-generation tensor cores: out[M, N] = a[M, K] * w[N, K]^T with fp32
// accumulation in tensor memory.  One persistent CTA per SM walks over 128 x BN output tiles.
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the a tile [128 x 64] and the w tile
//               [BN x 64] (128-byte swizzle) into a ring of shared-memory stages
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128 x BN x 16, both operands
//               K-major from shared memory) and commits stage releases / accumulator-ready signals
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (one row per thread), then one of
//               STORE (fp32), ADD (fp32 += : the residual sum), SWIGLU (bf16 silu(gate)*up from a
//               weight [all gate rows | all up rows]: a tile takes half its rows from each)
// BN (the tile width, 16 to 256) and the ring depth are run-time values chosen by the caller per shape.
// Two accumulator buffers (2 x 256 columns of tensor memory) let the epilogue of one tile overlap
// the main loop of the next.  Every mbarrier wait is bounded: on time-out the CTA records an
// error in `status`, all roles leave their loops, tensor memory is freed and the kernel returns.
// No cluster multicast is used anywhere: every CTA loads its own tiles.
//
// Reference counterpart: `gemm_tc_<fmt>` (mma.sync, 64 x 128 blocks), src/cuda_device.zig:348-499.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int BM = 128;

// Floats from one K slice's partial sums to the next: M * N and a pad, so that the same element of all slices
// does not lie a power of two apart (the kernel that adds the slices reads them together).
__host__ __device__ inline size_t slice_floats(int M, int N) { return (size_t)M * N + 2080; }
constexpr int BK = 64;       // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int MAX_BN = 256;             // the widest tile; also the distance of the two accumulator buffers in tensor memory
constexpr int MAX_STAGES = 12;
constexpr int A_BYTES = 128 * 64 * 2;  // the a tile of a stage
constexpr int CONTROL_BYTES = 1024;
constexpr int RING_BYTES = 227 * 1024 - 2 * 1024;   // what is left of an SM's shared memory after the control block and the alignment
constexpr uint32_t TMEM_COLS = 2 * MAX_BN;
constexpr uint32_t WAIT_LIMIT = 1u << 24;

enum Epilogue { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another one timed out).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// K-major operand tile in shared memory, rows of 128 bytes with the 128-byte swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset); the leading byte offset is unused (1); version 1 = sm_100.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
template <int W>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* r) {
  if (W == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared memory: [Control | ring of `stages` stages], a stage = the a tile (128 x 64 bf16 = 16 KB) followed by the
// w tile (bn x 64 bf16, rounded up to 1 KB).  Tile width and ring depth are run-time values: the host picks the
// width that fills whole waves of SMs and as many stages as fit.
struct Control {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Control) <= CONTROL_BYTES, "control block too large");

__host__ __device__ inline uint32_t stage_bytes_of(int bn) { return (uint32_t)A_BYTES + (((uint32_t)bn * BK * 2 + 1023u) & ~1023u); }

// W columns [c0, c0 + W) of this thread's accumulator row to fp32 out (stored or added).
template <int W, bool ADD>
__device__ __forceinline__ void store_chunk(uint32_t taddr, float* o, int c0, int n_out, bool row_ok, bool vec_ok) {
  uint32_t v[W];
  tmem_ld<W>(taddr + (uint32_t)c0, v);
  tmem_ld_wait();
  if (!row_ok) return;
  if (c0 + W <= n_out && vec_ok) {
#pragma unroll
    for (int j = 0; j < W; j += 4) {
      float4 x = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      float4* p = reinterpret_cast<float4*>(o + c0 + j);
      if (ADD) {
        float4 y = *p;
        x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
      }
      *p = x;
    }
  } else {
    for (int j = 0; j < W; ++j)
      if (c0 + j < n_out) {
        float x = __uint_as_float(v[j]);
        o[c0 + j] = ADD ? o[c0 + j] + x : x;
      }
  }
}

// The same for 32 columns added onto values of `out` that are in registers already (asked for two chunks ahead).
__device__ __forceinline__ void add_chunk_prefetched(uint32_t taddr, float* o, int c0, const float4* y) {
  uint32_t v[32];
  tmem_ld32(taddr + (uint32_t)c0, v);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    float4 x = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
    const float4 r = y[j >> 2];
    x.x += r.x; x.y += r.y; x.z += r.z; x.w += r.w;
    *reinterpret_cast<float4*>(o + c0 + j) = x;
  }
}
__device__ __forceinline__ void load_chunk(const float* o, int c0, float4* y) {
#pragma unroll
  for (int j = 0; j < 8; ++j) y[j] = *reinterpret_cast<const float4*>(o + c0 + 4 * j);
}

// W gate columns at c0 and their up columns `h` further on -> W bf16 outputs silu(gate) * up.
template <int W>
__device__ __forceinline__ void swiglu_chunk(uint32_t taddr, bf16* o, int c0, int h, int n_out, bool row_ok, bool vec_ok) {
  uint32_t g[W], u[W];
  tmem_ld<W>(taddr + (uint32_t)c0, g);
  tmem_ld<W>(taddr + (uint32_t)(h + c0), u);
  tmem_ld_wait();
  if (!row_ok) return;
  if (c0 + W <= n_out && vec_ok) {
#pragma unroll
    for (int j = 0; j < W; j += 8) {
      uint32_t packed[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float g0 = __uint_as_float(g[j + 2 * e]), g1 = __uint_as_float(g[j + 2 * e + 1]);
        float h0 = g0 / (1.0f + __expf(-g0)) * __uint_as_float(u[j + 2 * e]);
        float h1 = g1 / (1.0f + __expf(-g1)) * __uint_as_float(u[j + 2 * e + 1]);
        __nv_bfloat162 p = __floats2bfloat162_rn(h0, h1);
        packed[e] = *reinterpret_cast<uint32_t*>(&p);
      }
      *reinterpret_cast<uint4*>(o + c0 + j) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  } else {
    for (int j = 0; j < W; ++j)
      if (c0 + j < n_out) {
        float gv = __uint_as_float(g[j]);
        o[c0 + j] = __float2bfloat16_rn(gv / (1.0f + __expf(-gv)) * __uint_as_float(u[j]));
      }
  }
}

// `bn`: tile width, a multiple of 16 (32 with the SwiGLU epilogue) up to 256.  With the SwiGLU epilogue w is
// [F gate rows | F up rows] (N = 2 F) and a tile holds bn / 2 gate rows and the bn / 2 up rows that match them,
// brought by two copies; its accumulator columns are [gates | ups].
template <int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ out,
               int M, int N, int K, long long ldo, int bn, int stages, int splits, float* __restrict__ partial,
               int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Control& sm = *reinterpret_cast<Control*>(base);
  uint8_t* ring = base + CONTROL_BYTES;
  volatile int* abort_flag = &sm.abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = bn >> 1, F = N >> 1;
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = EPI == EPI_SWIGLU ? (F + h - 1) / h : (N + bn - 1) / bn;
  // With splits > 1 a work item is (output tile, slice of K); slice s of every tile comes before slice s + 1
  // of any, so the CTAs running together read different weights.  Each item stores its fp32 partial to
  // partial[s][M][N] (slices `slice_floats` apart); a second kernel adds the slices in order.
  const int mn_tiles = m_tiles * n_tiles;
  const int total_tiles = mn_tiles * splits;
  const int k_blocks_all = (K + BK - 1) / BK;
  const uint32_t stage_bytes = stage_bytes_of(bn);
  const uint32_t tx_bytes = (uint32_t)(BM + bn) * BK * 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.tmem_full[b], 1);
      mbar_init(&sm.tmem_empty[b], 4);
    }
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  pdl_wait();          // launched beside the end of the kernel before: set up, now wait for that kernel's output

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mn = tile % mn_tiles, ks = tile / mn_tiles;
        const int m0 = (mn % m_tiles) * BM, nt = mn / m_tiles;
        const int kb0 = (int)((long long)k_blocks_all * ks / splits), kb1 = (int)((long long)k_blocks_all * (ks + 1) / splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&sm.empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* st = ring + (size_t)stage * stage_bytes;
          mbar_expect_tx(&sm.full[stage], tx_bytes);
          tma_load_2d(st, &map_a, &sm.full[stage], kb * BK, m0);
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(st + A_BYTES, &map_w, &sm.full[stage], kb * BK, nt * h);
            tma_load_2d(st + A_BYTES + h * (BK * 2), &map_w, &sm.full[stage], kb * BK, F + nt * h);
          } else {
            tma_load_2d(st + A_BYTES, &map_w, &sm.full[stage], kb * BK, nt * bn);
          }
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
      pdl_launch_dependents();   // this CTA's operands are asked for: the next kernel may move in and set up
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N and M encoded
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t use = (uint32_t)(local >> 1);
        if (!mbar_wait(&sm.tmem_empty[buf], (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * MAX_BN);
        const int ks = tile / mn_tiles;
        const int kb0 = (int)((long long)k_blocks_all * ks / splits), kb1 = (int)((long long)k_blocks_all * (ks + 1) / splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&sm.full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st = smem_u32(ring + (size_t)stage * stage_bytes);
          const uint64_t da = make_smem_desc(st);
          const uint64_t db = make_smem_desc(st + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance both start addresses by 32 bytes (16 bf16) inside the swizzled row
            umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&sm.empty[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&sm.tmem_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;                     // the TMEM lanes this warp may read: 32*quarter ..
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const uint32_t use = (uint32_t)(local >> 1);
      const int mn = tile % mn_tiles, ks = tile / mn_tiles;
      const int m0 = (mn % m_tiles) * BM, nt = mn / m_tiles;
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < M;
      // Adding onto `out` (the residual sum): the values to add onto do not depend on the product, so the first two
      // chunks of this thread's row are asked for before the accumulator is waited for, and then two chunks ahead:
      // after a CTA's last tile nothing hides the epilogue, and a load per chunk in turn made it 10 us long.
      // (for a whole warp or not at all: the tensor-memory loads below are warp-wide instructions)
      const bool pre = EPI == EPI_ADD && splits == 1 && (ldo & 3) == 0 && nt * bn + bn <= N && bn >= 64 &&
                       __all_sync(0xffffffffu, row_ok);
      float4 y0[8], y1[8];
      float* o_add = reinterpret_cast<float*>(out) + (size_t)row * ldo + nt * bn;
      if (pre) {
        load_chunk(o_add, 0, y0);
        load_chunk(o_add, 32, y1);
      }
      if (!mbar_wait(&sm.tmem_full[buf], use & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * MAX_BN);
      if (splits > 1) {
        // a slice's partial sum, fp32 [M, N], a tile's columns as the accumulator has them
        const int n0 = nt * bn;
        float* o = partial + (size_t)ks * slice_floats(M, N) + (size_t)row * N + n0;
        const int n_out = N - n0;
        const bool vec_ok = (N & 3) == 0;
        int c0 = 0;
#pragma unroll 1
        for (; c0 + 32 <= bn; c0 += 32) store_chunk<32, false>(taddr, o, c0, n_out, row_ok, vec_ok);
        if (c0 < bn) store_chunk<16, false>(taddr, o, c0, n_out, row_ok, vec_ok);
      } else if (EPI == EPI_SWIGLU) {
        bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * ldo + nt * h;
        const int n_out = F - nt * h;
        const bool vec_ok = (ldo & 7) == 0 && ((nt * h) & 7) == 0;
        int c0 = 0;
#pragma unroll 1
        for (; c0 + 32 <= h; c0 += 32) swiglu_chunk<32>(taddr, o, c0, h, n_out, row_ok, vec_ok);
        if (c0 < h) swiglu_chunk<16>(taddr, o, c0, h, n_out, row_ok, vec_ok);
      } else {
        const int n0 = nt * bn;
        float* o = reinterpret_cast<float*>(out) + (size_t)row * ldo + n0;
        const int n_out = N - n0;
        const bool vec_ok = (ldo & 3) == 0;
        int c0 = 0;
        if (pre) {
#pragma unroll 1
          for (; c0 + 64 <= bn; c0 += 64) {
            add_chunk_prefetched(taddr, o, c0, y0);
            if (c0 + 96 <= bn) load_chunk(o, c0 + 64, y0);
            add_chunk_prefetched(taddr, o, c0 + 32, y1);
            if (c0 + 128 <= bn) load_chunk(o, c0 + 96, y1);
          }
          if (c0 + 32 <= bn) {
            add_chunk_prefetched(taddr, o, c0, y0);
            c0 += 32;
          }
        }
#pragma unroll 1
        for (; c0 + 32 <= bn; c0 += 32) store_chunk<32, EPI == EPI_ADD>(taddr, o, c0, n_out, row_ok, vec_ok);
        if (c0 < bn) store_chunk<16, EPI == EPI_ADD>(taddr, o, c0, n_out, row_ok, vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.tmem_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) atomicExch(status, 1);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host side: tensor maps ------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// bf16 matrix [rows, cols] with `cols` contiguous; box = 64 columns x box_rows rows, 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Adds the K slices of a split product in slice order.  mode 0: out fp32 = sum; 1: out fp32 += sum;
// 2: out bf16 [M, N/2] = silu(gate) * up, the partial sums' columns in tiles of [bn / 2 gates | their bn / 2 ups].
template <int MODE>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, int M, int N, long long ldo,
                                     int splits, int bn) {
  const long long total = MODE == 2 ? (long long)M * (N / 2) : (long long)M * N;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();          // the partial sums come from the kernel before
  if (i >= total) return;
  const size_t slice = slice_floats(M, N);
  if (MODE == 2) {
    const int F = N / 2;
    const int m = (int)(i / F), j = (int)(i % F);
    const int h = bn >> 1;
    const size_t gi = (size_t)m * N + (size_t)(j / h) * bn + (j % h);
    float gsum = 0.f, usum = 0.f;
    for (int s = 0; s < splits; ++s) {
      gsum += partial[s * slice + gi];
      usum += partial[s * slice + gi + h];
    }
    reinterpret_cast<bf16*>(out)[(size_t)m * ldo + j] = __float2bfloat16_rn(gsum / (1.0f + __expf(-gsum)) * usum);
  } else {
    const int m = (int)(i / N), n = (int)(i % N);
    float sum = 0.f;
    for (int s = 0; s < splits; ++s) sum += partial[s * slice + i];
    float* o = reinterpret_cast<float*>(out) + (size_t)m * ldo + n;
    *o = MODE == 1 ? *o + sum : sum;
  }
}

// The same sums four columns a thread (16-byte loads and stores; N and ldo multiples of 4), slices in the same order.
template <int MODE>
__global__ void splitk_reduce_vec_kernel(const float* __restrict__ partial, float* __restrict__ out, int M, int N, long long ldo,
                                         int splits) {
  const long long quads = (long long)M * (N / 4);
  const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();          // the partial sums come from the kernel before
  if (q >= quads) return;
  const int m = (int)(q / (N / 4)), n = (int)(q % (N / 4)) * 4;
  const size_t slice = slice_floats(M, N);
  const float* p = partial + (size_t)m * N + n;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int s = 0; s < splits; ++s) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(p + s * slice));
    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
  }
  float4* o = reinterpret_cast<float4*>(out + (size_t)m * ldo + n);
  if (MODE == 1) {
    const float4 r = *o;
    sum.x = r.x + sum.x; sum.y = r.y + sum.y; sum.z = r.z + sum.z; sum.w = r.w + sum.w;
  }
  *o = sum;
}

template <int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* out, int M, int N, int K, long long ldo, int bn, int splits,
           float* partial, int* status, cudaStream_t s) {
  static HkSmemCache allowed = {};
  const uint32_t stage_bytes = stage_bytes_of(bn);
  int stages = RING_BYTES / (int)stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  const size_t smem = (size_t)stages * stage_bytes + CONTROL_BYTES + 1024;
  if (int e = hk_allow_smem(gemm_tc_kernel<EPI>, smem, allowed)) return e;
  const int n_tiles = EPI == EPI_SWIGLU ? (N / 2 + bn / 2 - 1) / (bn / 2) : (N + bn - 1) / bn;
  const int tiles = ((M + BM - 1) / BM) * n_tiles * splits;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  // dependent launches (measured over decode steps of 24 and 64 rows: 1 % faster; the kernels after this one set up while it drains)
  int code = hk_launch_pdl(gemm_tc_kernel<EPI>, dim3(grid), dim3(NUM_THREADS), smem, s, ma, mw, out, M, N, K, ldo, bn, stages, splits, partial, status);
  if (code != 0 || splits <= 1) return code;
  if (EPI != EPI_SWIGLU && (N & 3) == 0 && (ldo & 3) == 0 && ((uintptr_t)out & 15) == 0) {
    const long long quads = (long long)M * (N / 4);
    return hk_launch_pdl(splitk_reduce_vec_kernel<EPI == EPI_ADD ? 1 : 0>, dim3((unsigned)((quads + 127) / 128)), dim3(128), 0, s,
                         (const float*)partial, reinterpret_cast<float*>(out), M, N, ldo, splits);
  }
  const long long total = EPI == EPI_SWIGLU ? (long long)M * (N / 2) : (long long)M * N;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  return hk_launch_pdl(splitk_reduce_kernel<EPI>, dim3(blocks), dim3(256), 0, s, (const float*)partial, out, M, N, ldo, splits, bn);
}

}  // namespace

// out = a w^T.  epilogue 0: out fp32 [M, N] stored; 1: out fp32 [M, N] += ; 2: out bf16 [M, N/2] =
// silu(gate) * up with w = [N/2 gate rows | N/2 up rows].  `bn` is the tile width: a multiple of 16 from 16 to 256
// (of 32 for epilogue 2, where a tile holds bn/2 gate rows and their up rows).  `status` is a device int
// that a timed-out wait sets to 1 (the caller reads it when it next synchronises).
// Requirements (else HK_ERR_UNSUPPORTED): K % 8 == 0, a and w 16-byte aligned, for epilogue 2 N even.
// splits > 1 cuts K into that many slices computed by different CTAs (for few output tiles: decode batches);
// `partial` must then hold hk_gemm_tc_partial_floats(M, N, splits) floats of scratch; with epilogue 2 the tiles must
// then fit N exactly ((N / 2) % (bn / 2) == 0).
HK_API int hk_gemm_tc(const void* a, const void* w, void* out, int M, int N, int K, long long ldo, int epilogue, int bn,
                      int splits, float* partial, int* status, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return HK_ERR_UNSUPPORTED;
  if (epilogue < EPI_STORE || epilogue > EPI_SWIGLU) return HK_ERR_UNSUPPORTED;
  if (bn < 16 || bn > MAX_BN || (bn & 15)) return HK_ERR_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU && ((N & 1) || (bn & 31))) return HK_ERR_UNSUPPORTED;
  if (splits < 1 || splits > (K + BK - 1) / BK || (splits > 1 && partial == nullptr)) return HK_ERR_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU && splits > 1 && (N / 2) % (bn / 2) != 0) return HK_ERR_UNSUPPORTED;
  CUtensorMap ma, mw;
  if (!make_map(&ma, a, M, K, BM) || !make_map(&mw, w, N, K, epilogue == EPI_SWIGLU ? bn / 2 : bn)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (epilogue == EPI_STORE) return launch<EPI_STORE>(ma, mw, out, M, N, K, ldo, bn, splits, partial, status, s);
  if (epilogue == EPI_ADD) return launch<EPI_ADD>(ma, mw, out, M, N, K, ldo, bn, splits, partial, status, s);
  return launch<EPI_SWIGLU>(ma, mw, out, M, N, K, ldo, bn, splits, partial, status, s);
}

// Floats of scratch that `hk_gemm_tc` needs for `splits` K slices.
HK_API long long hk_gemm_tc_partial_floats(int M, int N, int splits) { return (long long)(slice_floats(M, N) * (size_t)splits); }
