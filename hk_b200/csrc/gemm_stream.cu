// Persistent weight-streaming bf16 matrix product for decode batches: out[M, N] = a[M, K] * w[N, K]^T with
// M <= 32.  A decode step is bound by reading every weight once from HBM, so the kernel is built to keep a
// constant, large number of bytes on their way to every SM:
//
//   * one CTA per SM; a producer warp issues TMA tile copies (128-byte swizzle) of weights and activations into
//     a ring of 9-12 shared-memory stages (16 KB of weights each); the bytes in flight do not depend on how far
//     the consumers are;
//   * eight consumer warps read the stages with ldmatrix and multiply with mma.sync.m16n8k16, roles swapped:
//     16 rows of w are the "M" side, 8 tokens the "N" side (M <= 8 needs no padding to a 128-row tile).  A warp
//     loads all its fragments of a stage before it multiplies, into two accumulator sets, so that neither the
//     shared-memory latency nor the tensor-core latency is paid once per 16 k (one SM must take in well over
//     its even share of the HBM bandwidth, or a narrow product that leaves SMs idle is slow);
//   * the work is cut into units (tile of BN weight rows, K chunk of BK) and every CTA gets the same number of
//     them, so all SMs stream for the same time whatever N is: each CTA owns tiles / CTAs whole tiles, and the
//     tiles that are left over are shared stream-K fashion (numbered tile by tile, every CTA takes an equal,
//     contiguous range of their units).  A shared tile is finished by the CTA that arrives last: each writes
//     its partial sums to a workspace and counts itself in; the last one adds the partials in K order (a fixed
//     order: results do not depend on timing) and runs the epilogue.  Nobody waits for anybody.  A CTA does
//     its shared units first, so that this hand-over happens while its own tiles still stream;
//   * one TMA copy brings a whole stage of weights: w is described as a 3-D tensor [K / 64][N][64] (the K
//     columns of 64 as the outermost dimension), so a box of {64, rows, columns} lands as columns x rows x 128
//     bytes, which is the swizzled layout ldmatrix wants;
//   * epilogues: store fp32, add onto fp32 `out` (the residual sum), or silu(gate) * up -> bf16 over a weight
//     [all gate rows | all up rows] (a tile then holds BN/2 gate rows and, as its second half, their up rows).
//
// Every mbarrier wait is bounded; on a time-out the CTA records it in `status`, its warps stop touching memory
// but still meet at their barriers, and the kernel returns.
//
// `workspace` (floats) and `counters` (ints, zero before the first launch; the kernel leaves them zero) belong
// to one stream of launches: two launches that overlap in time must not share them.
//
// Reference counterpart: `gemv_bf16` (warp per row, one token), src/cuda_device.zig:1294-1351.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int CONSUMERS = 8;
constexpr int NUM_THREADS = (CONSUMERS + 1) * 32;
constexpr uint32_t WAIT_LIMIT = 1u << 20;
// Shared memory a CTA may take.  Not all of the SM's: with 200 KB nothing else fits beside a CTA of this kernel, so the
// kernels after it (norm, small-M product: launched as dependents) could not become resident and set up until it had left.
// Measured over whole decode steps of the 8B layer sizes at batch 8 (ms a step) against the budget in KB:
// 112: 4.16, 120: 4.01, 128-152: 3.93-3.95, 168-184: 3.95-3.96, 200: 4.03; batch 12 and 16 gain 0.6-0.9 % at 152.
constexpr int SMEM_BUDGET = 152 * 1024;
constexpr int SMEM_BUDGET_WIDE = 200 * 1024;     // 17 to 32 rows: a stage is 48 KB, and three must fit

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
// Bounded wait.  Returns false when the CTA is giving up (this wait or another one ran out).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory"); }

// RW: consumer warps side by side over the tile's rows (BN = 16 * RW); the other CONSUMERS / RW warps split the
// stage's K chunk (BK = 64 per such warp: one swizzled box).  MT: token tiles of 8.
template <int RW, int MT>
struct Shape {
  static constexpr int KW = CONSUMERS / RW;
  static constexpr int BN = 16 * RW;
  static constexpr int BK = 64 * KW;
  static constexpr int W_COL = (BN / 2) * 128;           // one K column (64 bf16 = 128 bytes a row) of half the tile's rows
  static constexpr int W_HALF = KW * W_COL;              // one copy: half the tile's rows, all K columns of the stage
  static constexpr int W_BYTES = 2 * W_HALF;             // = 16 KB
  static constexpr int A_COL = 8 * MT * 128;
  static constexpr int A_BYTES = KW * A_COL;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  static constexpr int COLS = 8 * MT;
  static constexpr int TILE_FLOATS = KW * BN * (COLS + 1);
  static constexpr int FIXED = TILE_FLOATS * 4 + 1024;   // tile buffer, barriers, flags
  static constexpr int BUDGET = MT <= 2 ? SMEM_BUDGET : SMEM_BUDGET_WIDE;
  static constexpr int STAGES_RAW = (BUDGET - FIXED) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static constexpr int SMEM = STAGES * STAGE_BYTES + FIXED + 1024;     // + room to align the ring to 1024 bytes
  static_assert(W_COL % 1024 == 0 && A_COL % 1024 == 0, "columns must keep the swizzle atoms aligned");
  static_assert(STAGES >= 3, "too few stages");
};

struct Control {
  uint64_t full[12];
  uint64_t empty[12];
  int abort_flag;
  int last;
};

// First row of the tile's first (second) half.  Plain product: the halves are consecutive.  SwiGLU: w is
// [F gate rows | F up rows]; the first half are gate rows, the second their up rows, F further down.
template <int BN, int EPI>
__device__ __forceinline__ int tile_row(int tile, int half, int F) {
  if (EPI == EPI_SWIGLU) return tile * (BN / 2) + half * F;
  return tile * BN + half * (BN / 2);
}

// How one product's units (tile of BN weight rows, K chunk of BK) are dealt to the CTAs: every CTA owns `own` whole
// tiles and the units of the left-over (shared) tiles are cut evenly, shared units first.
struct Sched {
  int kc, n_tiles, own, shared_tiles, ns, n_local, own_first;
  long long units, PS, u0;
};

__device__ __forceinline__ Sched make_sched(int n_tiles, int kc, long long P, long long bid) {
  Sched sc;
  sc.kc = kc;
  sc.n_tiles = n_tiles;
  sc.own = n_tiles / (int)P;                                             // whole tiles of every CTA
  sc.shared_tiles = n_tiles - sc.own * (int)P;                           // tiles 0 .. shared_tiles - 1, cut stream-K fashion
  sc.units = (long long)sc.shared_tiles * kc;                            // units of the shared tiles
  sc.PS = sc.units < P ? sc.units : P;                                   // CTAs that take part in them (each gets some)
  const bool sharing = bid < sc.PS;
  sc.u0 = sharing ? sc.units * bid / sc.PS : 0;
  const long long u1 = sharing ? sc.units * (bid + 1) / sc.PS : 0;
  sc.ns = (int)(u1 - sc.u0);                                             // this CTA's shared units come first
  sc.n_local = sc.ns + sc.own * kc;
  sc.own_first = sc.shared_tiles + (int)bid * sc.own;
  return sc;
}

// The consumer warps' side of one product: multiplies this CTA's units as their stages fill (unit i of the product
// is stage (i_base + i) % STAGES of the ring) and hands every tile, or share of a tile, over.
template <int RW, int MT, int EPI>
__device__ __forceinline__ void consume_units(const Sched& sc, uint32_t i_base, uint32_t ring, Control* ctl, float* tile_buf,
                                              void* __restrict__ out, int M, int N, long long ldo, float* __restrict__ workspace,
                                              int* __restrict__ counters) {
  using S = Shape<RW, MT>;
  constexpr int BN = S::BN, KW = S::KW, COLS = S::COLS, STAGES = S::STAGES;
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kc = sc.kc, ns = sc.ns, n_local = sc.n_local, own_first = sc.own_first;
  const long long units = sc.units, PS = sc.PS, u0 = sc.u0;
  const int rg = warp % RW, kp = warp / RW;
  const int g = lane >> 2, t = lane & 3;
  const int tid = threadIdx.x;                           // 0 .. 255
  float acc[MT][2][4];       // two sets: consecutive MMAs do not wait for each other
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][0][e] = acc[j][1][e] = 0.f;

  // ldmatrix addresses inside a box: weights: row = lane & 15, 16-byte chunk 2 * ks + (lane >> 4);
  // activations: token = lane & 7 (+ 8 per token tile), chunk 4 * kq + (lane >> 3); chunk ^= row & 7 (swizzle)
  const int wrow = rg * 16 + (lane & 15);                 // row of the tile; the stage holds the tile's halves apart
  const uint32_t w_off = (uint32_t)(wrow / (BN / 2)) * S::W_HALF + (uint32_t)kp * S::W_COL + (uint32_t)(wrow % (BN / 2)) * 128u;
  const uint32_t w_x = (uint32_t)(wrow & 7), w_hi = (uint32_t)(lane >> 4);
  const uint32_t a_off = (uint32_t)S::W_BYTES + (uint32_t)kp * S::A_COL + (uint32_t)(lane & 7) * 128u;
  const uint32_t a_x = (uint32_t)(lane & 7), a_hi = (uint32_t)(lane >> 3);

  int tile = ns > 0 ? (int)(u0 / kc) : own_first, c = ns > 0 ? (int)(u0 % kc) : 0;
  bool tile_from_start = c == 0;           // this CTA has the tile's first unit
  bool dead = false;                       // gave up: no more memory traffic, barriers only
  for (uint32_t i = 0; i < (uint32_t)n_local; ++i) {
    const uint32_t stage = (i_base + i) % STAGES, phase = ((i_base + i) / STAGES) & 1u;
    if (!dead && !mbar_wait(&ctl->full[stage], phase, abort_flag)) dead = true;
    if (!dead) {
      const uint32_t base = ring + stage * S::STAGE_BYTES;
      const uint32_t wbox = base + w_off;
      const uint32_t abox = base + a_off;
      uint32_t afrag[4][4], bfrag[MT][2][4];
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) ldmatrix_x4(wbox + (((ks * 2 + w_hi) ^ w_x) << 4), afrag[ks]);
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int kq = 0; kq < 2; ++kq) ldmatrix_x4(abox + j * 1024 + (((kq * 4 + a_hi) ^ a_x) << 4), bfrag[j][kq]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int j = 0; j < MT; ++j)
          mma_bf16_16816(acc[j][ks & 1], afrag[ks], bfrag[j][ks >> 1][2 * (ks & 1)], bfrag[j][ks >> 1][2 * (ks & 1) + 1]);
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->empty[stage]);
    }
    if ((int)i == n_local - 1) pdl_launch_dependents();   // this CTA's weights are read: the next kernel may move in
    const bool tile_ends = c == kc - 1;
    const bool share_ends = (int)i == ns - 1;          // the last of this CTA's units of the shared tiles
    if (tile_ends || share_ends) {
      // ---- the tile (or this CTA's share of it) is summed: hand it over ----
      consumer_sync();                                  // the buffer of the tile before is read
      float* mine = tile_buf + (size_t)kp * BN * (COLS + 1);
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        const int col = j * 8 + 2 * t;
        mine[(rg * 16 + g) * (COLS + 1) + col] = acc[j][0][0] + acc[j][1][0];
        mine[(rg * 16 + g) * (COLS + 1) + col + 1] = acc[j][0][1] + acc[j][1][1];
        mine[(rg * 16 + g + 8) * (COLS + 1) + col] = acc[j][0][2] + acc[j][1][2];
        mine[(rg * 16 + g + 8) * (COLS + 1) + col + 1] = acc[j][0][3] + acc[j][1][3];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][0][e] = acc[j][1][e] = 0.f;
      }
      consumer_sync();
      const bool whole = tile_from_start && tile_ends;
      const bool ok = !*abort_flag;
      // element e of a tile: token e / BN, row e % BN (rows fastest: stores to consecutive addresses)
      auto summed = [&](int e) {
        const int m = e / BN, row = e % BN;
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < KW; ++q) s += tile_buf[(size_t)q * BN * (COLS + 1) + row * (COLS + 1) + m];
        return s;
      };
      auto finish = [&](auto value) {
        if (EPI == EPI_SWIGLU) {
          const int f0 = tile * (BN / 2);
          for (int e = tid; e < (BN / 2) * COLS; e += CONSUMERS * 32) {
            const int m = e / (BN / 2), row = e % (BN / 2);
            if (m >= M) continue;
            const float gate = value(m * BN + row), up = value(m * BN + row + BN / 2);
            reinterpret_cast<bf16*>(out)[(size_t)m * ldo + f0 + row] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
          }
        } else {
          const int n0 = tile * BN;
          for (int e = tid; e < BN * COLS; e += CONSUMERS * 32) {
            const int m = e / BN, row = e % BN;
            if (m >= M || n0 + row >= N) continue;
            float* o = reinterpret_cast<float*>(out) + (size_t)m * ldo + n0 + row;
            const float v = value(e);
            *o = EPI == EPI_ADD ? *o + v : v;
          }
        }
      };
      if (whole) {
        if (ok) finish(summed);
      } else {
        // contributors of this tile, in K order: the CTAs whose unit ranges meet [tile * kc, (tile + 1) * kc)
        const long long t0 = (long long)tile * kc, t1 = t0 + kc;
        const int c_first = (int)(((t0 + 1) * PS + units - 1) / units) - 1;
        const int c_last = (int)((t1 * PS + units - 1) / units) - 1;
        constexpr int SLOT = BN * COLS;
        auto slot_of = [&](int cta) {
          const long long start = units * cta / PS;
          return workspace + ((size_t)cta * 2 + (start / kc == tile ? 0 : 1)) * SLOT;
        };
        float* my_slot = slot_of((int)blockIdx.x);
        if (ok)
          for (int e = tid; e < SLOT; e += CONSUMERS * 32) my_slot[e] = summed(e);
        __threadfence();
        consumer_sync();
        if (tid == 0) {
          int last = 0;
          if (ok) {
            const int old = atomicAdd(&counters[tile], 1);
            last = old == c_last - c_first;
            if (last) counters[tile] = 0;               // everyone has counted: ready for the next launch
          }
          ctl->last = last;
        }
        consumer_sync();
        if (ctl->last) {
          __threadfence();
          constexpr int PER = SLOT / (CONSUMERS * 32) > 0 ? SLOT / (CONSUMERS * 32) : 1;
          float sum[PER];
#pragma unroll
          for (int q = 0; q < PER; ++q) sum[q] = 0.f;
          for (int cta = c_first; cta <= c_last; ++cta) {      // K order, whoever came last
            const float* slot = slot_of(cta);
#pragma unroll
            for (int q = 0; q < PER; ++q)
              if (tid + q * CONSUMERS * 32 < SLOT) sum[q] += __ldcg(slot + tid + q * CONSUMERS * 32);
          }
          float* flat = tile_buf;                              // [SLOT], element order as in the slots
#pragma unroll
          for (int q = 0; q < PER; ++q)
            if (tid + q * CONSUMERS * 32 < SLOT) flat[tid + q * CONSUMERS * 32] = sum[q];
          consumer_sync();
          finish([&](int e) { return flat[e]; });
        }
      }
      tile_from_start = true;
    }
    if (share_ends) { tile = own_first; c = 0; }
    else if (++c == kc) { c = 0; ++tile; }
  }
}

template <int RW, int MT, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                   void* __restrict__ out, int M, int N, int K, long long ldo, float* __restrict__ workspace,
                   int* __restrict__ counters, int* __restrict__ status) {
  using S = Shape<RW, MT>;
  constexpr int BN = S::BN, BK = S::BK, KW = S::KW, STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* after = smem_raw + (ring - smem_u32(smem_raw)) + (size_t)STAGES * S::STAGE_BYTES;
  float* tile_buf = reinterpret_cast<float*>(after);                     // [KW][BN][COLS + 1]
  Control* ctl = reinterpret_cast<Control*>(after + S::TILE_FLOATS * 4);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Sched sc = make_sched(EPI == EPI_SWIGLU ? N / BN : (N + BN - 1) / BN, (K + BK - 1) / BK, gridDim.x, blockIdx.x);
  const int kc = sc.kc, ns = sc.ns, n_local = sc.n_local, own_first = sc.own_first;
  const long long u0 = sc.u0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], CONSUMERS);
    }
    ctl->abort_flag = 0;
    ctl->last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();          // launched beside the end of the kernel before: set up, now wait for that kernel's output

  if (warp == CONSUMERS) {
    // ---- producer ----
    if (lane == 0) {
      int tile = ns > 0 ? (int)(u0 / kc) : own_first, c = ns > 0 ? (int)(u0 % kc) : 0;
      uint32_t i = 0;
      for (; i < (uint32_t)n_local; ++i) {
        const uint32_t stage = i % STAGES, phase = (i / STAGES) & 1u;
        if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) break;
        mbar_expect_tx(&ctl->full[stage], S::STAGE_BYTES);
        const uint32_t base = ring + stage * S::STAGE_BYTES;
        tma_load_3d(base, &map_w, &ctl->full[stage], 0, tile_row<BN, EPI>(tile, 0, N / 2), c * KW);
        tma_load_3d(base + S::W_HALF, &map_w, &ctl->full[stage], 0, tile_row<BN, EPI>(tile, 1, N / 2), c * KW);
        tma_load_3d(base + S::W_BYTES, &map_a, &ctl->full[stage], 0, 0, c * KW);
        if ((int)i + 1 == ns) { tile = own_first; c = 0; }
        else if (++c == kc) { c = 0; ++tile; }
      }
      if (*abort_flag) {
        // giving up: let the copies that are still on their way land before the shared memory goes away
        const uint32_t pending = i < (uint32_t)STAGES ? i : (uint32_t)STAGES;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t it = i - 1 - j;
          for (uint32_t spin = 0; spin < WAIT_LIMIT; ++spin)
            if (mbar_try_wait(&ctl->full[it % STAGES], (it / STAGES) & 1u)) break;
        }
      }
    }
  } else {
    consume_units<RW, MT, EPI>(sc, 0u, ring, ctl, tile_buf, out, M, N, ldo, workspace, counters);
  }
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag) atomicExch(status, 1);
}

// ---- host side ---------------------------------------------------------------------------------------

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

// bf16 matrix [rows, cols] with `cols` contiguous and cols % 64 == 0, seen as [cols / 64][rows][64]: a box of
// {64, box_rows, box_cols} lands in shared memory as box_cols x box_rows x 128 bytes, 128-byte swizzle, zeros outside
bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows, int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_cols};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
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

template <int RW, int MT, int EPI>
int launch(const void* a, const void* w, void* out, int M, int N, int K, long long ldo, float* workspace, int* counters,
           int* status, int max_ctas, cudaStream_t s) {
  using S = Shape<RW, MT>;
  CUtensorMap ma, mw;
  if (!make_map(&ma, a, M, K, 8 * MT, S::KW) || !make_map(&mw, w, N, K, S::BN / 2, S::KW)) return HK_ERR_UNSUPPORTED;
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(gemm_stream_kernel<RW, MT, EPI>, (size_t)S::SMEM, allowed)) return e;
  const int n_tiles = EPI == EPI_SWIGLU ? N / S::BN : (N + S::BN - 1) / S::BN;
  const long long units = (long long)n_tiles * ((K + S::BK - 1) / S::BK);
  long long grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (units < grid) grid = units;
  return hk_launch_pdl(gemm_stream_kernel<RW, MT, EPI>, dim3((unsigned)grid), dim3(NUM_THREADS), (size_t)S::SMEM, s, ma, mw, out, M, N, K,
                   ldo, workspace, counters, status);
}

template <int RW, int MT>
int launch_epi(int epilogue, const void* a, const void* w, void* out, int M, int N, int K, long long ldo, float* workspace,
               int* counters, int* status, int max_ctas, cudaStream_t s) {
  if (epilogue == EPI_STORE) return launch<RW, MT, EPI_STORE>(a, w, out, M, N, K, ldo, workspace, counters, status, max_ctas, s);
  if (epilogue == EPI_ADD) return launch<RW, MT, EPI_ADD>(a, w, out, M, N, K, ldo, workspace, counters, status, max_ctas, s);
  return launch<RW, MT, EPI_SWIGLU>(a, w, out, M, N, K, ldo, workspace, counters, status, max_ctas, s);
}


}  // namespace

// out = a w^T for M <= 32.  epilogue 0: out fp32 [M, N] stored; 1: out fp32 [M, N] +=; 2: out bf16 [M, N/2] =
// silu(gate) * up with w = [N/2 gate rows | N/2 up rows] (N a multiple of the tile's rows, 16 * rw).
// rw: 8, 4, 2 or 1 consumer warps across a tile's rows (tiles of 128, 64, 32 or 16 rows; the other warps split K).
// workspace: at least hk_gemm_stream_workspace(M, rw) floats; counters: one int per tile of 16 rows of w, zero
// before the first launch (left zero); status: device int that a timed-out wait sets to 1.
// max_ctas: 0 = one CTA per SM; smaller values only for tests of the hand-over between CTAs.
// Refuses (HK_ERR_UNSUPPORTED) M > 32, K % 64 != 0, operands not 16-byte aligned, bad rw.
HK_API int hk_gemm_stream(const void* a, const void* w, void* out, int M, int N, int K, long long ldo, int epilogue, int rw,
                          float* workspace, int* counters, int* status, int max_ctas, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K <= 0 || (K & 63) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return HK_ERR_UNSUPPORTED;
  if (epilogue < 0 || epilogue > 2 || (epilogue == EPI_SWIGLU && (rw < 1 || N % (16 * rw)))) return HK_ERR_UNSUPPORTED;
  if (workspace == nullptr || counters == nullptr || status == nullptr) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const int mt = M <= 8 ? 1 : M <= 16 ? 2 : 4;
#define HK_CASE(RW, MT) \
  if (rw == RW && mt == MT) return launch_epi<RW, MT>(epilogue, a, w, out, M, N, K, ldo, workspace, counters, status, max_ctas, s);
  HK_CASE(8, 1) HK_CASE(4, 1) HK_CASE(2, 1) HK_CASE(1, 1)
  HK_CASE(8, 2) HK_CASE(4, 2) HK_CASE(2, 2) HK_CASE(1, 2)
  HK_CASE(8, 4) HK_CASE(4, 4) HK_CASE(2, 4)
#undef HK_CASE
  return HK_ERR_UNSUPPORTED;
}

// Floats of workspace a launch may touch: two partial tiles per CTA.
HK_API long long hk_gemm_stream_workspace(int M, int rw) {
  const int mt = M <= 8 ? 1 : M <= 16 ? 2 : 4;
  return (long long)sm_count() * 2 * (16 * rw) * (8 * mt);
}
