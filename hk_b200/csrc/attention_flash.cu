// Flash attention over the paged cache for bf16 serving: prompt portions, decode tokens and mixed
// batches in one kernel, grouped-query aware, with optional key splitting for long contexts.
//
// Work is cut on the host into *items*: (request slot, a run of consecutive query tokens, a key range).
// A CTA takes one item for one kv head.  Its rows are (query token, query head of the group) pairs, 16 per
// warp, so the K/V pages of a kv head are read once for all the heads that share it.  Keys come in tiles of
// 64 through cp.async (double buffered) from wherever the block table says the pages are; scores and
// weighted values run on mma.sync.m16n8k16 (bf16 in, fp32 out) with the softmax state (max, sum) in fp32
// registers, as in the reference's single-sequence kernel `attention_tc_128`
// (src/cuda_device.zig:1069-1248), which this replaces together with its split-KV decode kernels
// `attention_part_warp` + `attention_combine` (:1654-1815).  A row at position p sees keys
// [max(0, p - window + 1), p]; its own key was written earlier in the step.
//
// With splitting, each CTA writes an unnormalised partial (values, max, sum) to scratch and
// `attention_combine_kernel` merges the partials of a (token, head) exactly, in split order.
// Head sizes: multiples of 16 up to 128.  Any group size up to 16 * warps.
#include <cuda.h>
#include <math_constants.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int TILE_N = 64;

struct Item {
  int q_row0;     // row of the first query token in the batch
  int n_tokens;   // query tokens of this item
  int slot;       // request slot (row of the block table)
  int pos0;       // position of the first query token
  int kv_lo;      // first key this item may read
  int kv_hi;      // one past the last key
  int part;       // index of the partial in scratch, or -1: write the output directly
  int pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD, int NW>
__global__ void __launch_bounds__(NW * 32, 3)
attention_flash_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                       const int* __restrict__ block_table, int table_stride, const Item* __restrict__ items,
                       bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int H, int G,
                       int page_tokens, int window, float scale_log2) {
  constexpr int ROWS = NW * 16;
  constexpr int LD = HD + 8;            // padded row: (HD/8 + 1) 16-byte chunks, an odd count -> no ldmatrix conflicts
  constexpr int CPR = HD / 8;           // 16-byte chunks per row
  constexpr int KSTEPS = HD / 16;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);             // [2][TILE_N][LD]
  bf16* vs = ks + 2 * TILE_N * LD;                          // [2][TILE_N][LD]
  int* tile_pages = reinterpret_cast<int*>(vs + 2 * TILE_N * LD);   // [2][TILE_N]

  // one CTA per (item, kv head), kv heads fastest: prompt items come heaviest first, and so do the CTAs of all heads
  const Item it = items[blockIdx.x / G];
  const int g = blockIdx.x % G;
  const int group = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qr = lane >> 2, qt = lane & 3;
  const int* bt = block_table + (size_t)it.slot * table_stride;

  // the two rows this thread owns in its warp's 16: r0 and r0 + 8
  int row[2], pos[2], lo[2];
  bool valid[2];
  const bf16* qp[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    row[i] = warp * 16 + qr + 8 * i;
    int tq = row[i] / group;
    valid[i] = tq < it.n_tokens;
    if (!valid[i]) tq = 0;
    pos[i] = it.pos0 + tq;
    lo[i] = window > 0 ? max(0, pos[i] - window + 1) : 0;
    qp[i] = q + ((size_t)(it.q_row0 + tq) * H + g * group + row[i] % group) * HD;
  }

  // Q fragments (A operand): per k-step a0 = (r0, d 2t..), a1 = (r0+8, d 2t..), a2 = (r0, d 2t+8..), a3 = (r0+8, d 2t+8..)
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int s = 0; s < KSTEPS; ++s) {
    qf[s][0] = *reinterpret_cast<const uint32_t*>(qp[0] + s * 16 + 2 * qt);
    qf[s][1] = *reinterpret_cast<const uint32_t*>(qp[1] + s * 16 + 2 * qt);
    qf[s][2] = *reinterpret_cast<const uint32_t*>(qp[0] + s * 16 + 8 + 2 * qt);
    qf[s][3] = *reinterpret_cast<const uint32_t*>(qp[1] + s * 16 + 8 + 2 * qt);
  }

  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};

  const int t_begin = it.kv_lo / TILE_N;
  const int t_end = (it.kv_hi + TILE_N - 1) / TILE_N;

  // Page ids of a tile's keys are looked up once per tile (64 / page_tokens pages, or one page when pages
  // are larger) into shared memory; the copy loop then only does arithmetic.
  auto load_tile = [&](int t, int stage) {
    bf16* kd = ks + stage * TILE_N * LD;
    bf16* vd = vs + stage * TILE_N * LD;
    int* pg = tile_pages + stage * TILE_N;     // per key row: its row in the [rows, HD] view of the pages, or -1
    for (int r = threadIdx.x; r < TILE_N; r += NW * 32) {
      const int j = t * TILE_N + r;
      int row_of_key = -1;
      if (j >= it.kv_lo && j < it.kv_hi) {
        const int pi = j / page_tokens;
        const int page = bt[pi];
        if (page >= 0) row_of_key = (page * G + g) * page_tokens + (j - pi * page_tokens);
      }
      pg[r] = row_of_key;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < TILE_N * CPR; idx += NW * 32) {
      const int r = idx / CPR, c = idx % CPR;
      const int row_of_key = pg[r];
      const bool ok = row_of_key >= 0;
      const size_t off = ok ? (size_t)row_of_key * HD + c * 8 : 0;
      cp_async16(kd + r * LD + c * 8, k_pages + off, ok);
      cp_async16(vd + r * LD + c * 8, v_pages + off, ok);
    }
  };

  if (t_begin < t_end) load_tile(t_begin, 0);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    const int stage = (t - t_begin) & 1;
    if (t + 1 < t_end) load_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* kt = ks + stage * TILE_N * LD;
    const bf16* vt = vs + stage * TILE_N * LD;

    // ---- scores: 16 rows x 64 keys per warp
    float s[TILE_N / 8][4];
#pragma unroll
    for (int n = 0; n < TILE_N / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int np = 0; np < TILE_N / 16; ++np) {
        uint32_t b[4];
        const int mi = lane >> 3, r8 = lane & 7;
        ldmatrix_x4(b, kt + (np * 16 + (mi >> 1) * 8 + r8) * LD + kk * 16 + (mi & 1) * 8);
        mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
      }
    }
    // ---- mask, scale, running maximum.  A tile that every row of this thread sees whole (the common case
    // far below the diagonal) needs no per-element tests.
    float mt[2] = {-CUDART_INF_F, -CUDART_INF_F};
    const int j_first = t * TILE_N, j_last = t * TILE_N + TILE_N - 1;
    const bool whole = valid[0] && valid[1] && j_first >= max(max(lo[0], lo[1]), it.kv_lo) &&
                       j_last <= min(min(pos[0], pos[1]), it.kv_hi - 1);
    if (whole) {
#pragma unroll
      for (int n = 0; n < TILE_N / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[n][e] *= scale_log2;
          mt[e >> 1] = fmaxf(mt[e >> 1], s[n][e]);
        }
    } else {
#pragma unroll
      for (int n = 0; n < TILE_N / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int j = t * TILE_N + n * 8 + 2 * qt + (e & 1);
          const bool ok = valid[i] && j >= lo[i] && j <= pos[i] && j >= it.kv_lo && j < it.kv_hi;
          s[n][e] = ok ? s[n][e] * scale_log2 : -CUDART_INF_F;
          mt[i] = fmaxf(mt[i], s[n][e]);
        }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 1));
      mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 2));
      const float mn = fmaxf(m[i], mt[i]);
      msafe[i] = mn == -CUDART_INF_F ? 0.f : mn;
      corr[i] = exp2f(m[i] - msafe[i]);       // m = -inf -> 0
      m[i] = mn;
      l[i] *= corr[i];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
    // ---- probabilities (bf16 A fragments) and weighted values
#pragma unroll
    for (int kk = 0; kk < TILE_N / 16; ++kk) {
      uint32_t pf[4];
      float p[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[h][e] = exp2f(s[2 * kk + h][e] - msafe[e >> 1]);
          l[e >> 1] += p[h][e];
        }
      pf[0] = pack_bf16(p[0][0], p[0][1]);
      pf[1] = pack_bf16(p[0][2], p[0][3]);
      pf[2] = pack_bf16(p[1][0], p[1][1]);
      pf[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        const int mi = lane >> 3, r8 = lane & 7;
        ldmatrix_x4_trans(b, vt + (kk * 16 + (mi & 1) * 8 + r8) * LD + dp * 16 + (mi >> 1) * 8);
        mma_bf16(o[2 * dp], pf, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
      }
    }
    __syncthreads();   // the stage is free for the load after next
  }
  cp_async_wait<0>();

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  if (it.part < 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!valid[i]) continue;
      const int tq = row[i] / group;
      bf16* op = out + ((size_t)(it.q_row0 + tq) * H + g * group + row[i] % group) * HD;
      const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<uint32_t*>(op + n * 8 + 2 * qt) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
  } else {
    const size_t base = ((size_t)it.part * G + g) * ROWS;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float* po = part_o + (base + row[i]) * HD;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(po + n * 8 + 2 * qt) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      if (qt == 0) *reinterpret_cast<float2*>(part_ml + (base + row[i]) * 2) = make_float2(m[i], l[i]);
    }
  }
}

// Decode variant, built for bandwidth: few rows (the heads of one group for one or a few tokens), long key
// ranges.  The CTA's DW warps share the same 16 rows and split every DT-key tile among themselves, 16 keys
// each; tiles come through a DS-stage cp.async ring (DS - 1 tiles in flight per CTA) and several small CTAs
// share an SM, so enough bytes are in flight to keep HBM busy.  The item's page ids are read into shared
// memory once, up front, so no tile waits on a block-table load.  The warps' softmax states are merged through
// shared memory at the end, in warp order.
constexpr int DW = 2;            // warps
constexpr int DT = DW * 16;      // keys per tile
constexpr int DS = 4;            // stages

template <int HD>
__global__ void __launch_bounds__(DW * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                        const int* __restrict__ block_table, int table_stride, const Item* __restrict__ items,
                        bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int H, int G,
                        int page_tokens, int window, float scale_log2, int pages_cap) {
  constexpr int ROWS = 16;
  constexpr int LD = HD + 8, CPR = HD / 8, KSTEPS = HD / 16;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);            // [DS][DT][LD]
  bf16* vs = ks + DS * DT * LD;                            // [DS][DT][LD]
  int* pages = reinterpret_cast<int*>(vs + DS * DT * LD);  // [pages_cap]

  const Item it = items[blockIdx.x];
  const int g = blockIdx.y;
  const int group = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qr = lane >> 2, qt = lane & 3;
  const int* bt = block_table + (size_t)it.slot * table_stride;

  const int page_lo = it.kv_lo / page_tokens;
  const int n_pages = it.kv_hi > it.kv_lo ? min((it.kv_hi - 1) / page_tokens - page_lo + 1, pages_cap) : 0;
  for (int i = threadIdx.x; i < n_pages; i += DW * 32) pages[i] = bt[page_lo + i];

  int row[2], pos[2], lo[2];
  bool valid[2];
  const bf16* qp[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    row[i] = qr + 8 * i;
    int tq = row[i] / group;
    valid[i] = tq < it.n_tokens;
    if (!valid[i]) tq = 0;
    pos[i] = it.pos0 + tq;
    lo[i] = window > 0 ? max(0, pos[i] - window + 1) : 0;
    qp[i] = q + ((size_t)(it.q_row0 + tq) * H + g * group + row[i] % group) * HD;
  }
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int s = 0; s < KSTEPS; ++s) {
    qf[s][0] = *reinterpret_cast<const uint32_t*>(qp[0] + s * 16 + 2 * qt);
    qf[s][1] = *reinterpret_cast<const uint32_t*>(qp[1] + s * 16 + 2 * qt);
    qf[s][2] = *reinterpret_cast<const uint32_t*>(qp[0] + s * 16 + 8 + 2 * qt);
    qf[s][3] = *reinterpret_cast<const uint32_t*>(qp[1] + s * 16 + 8 + 2 * qt);
  }
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};

  const int t_begin = it.kv_lo / DT;
  const int t_end = (it.kv_hi + DT - 1) / DT;
  __syncthreads();   // page ids are in place

  auto load_tile = [&](int t, int stage) {
    bf16* kd = ks + stage * DT * LD;
    bf16* vd = vs + stage * DT * LD;
#pragma unroll 4
    for (int idx = threadIdx.x; idx < DT * CPR; idx += DW * 32) {
      const int r = idx / CPR, c = idx % CPR;
      const int j = t * DT + r;
      const int pi = j / page_tokens - page_lo;
      const bool ok = j >= it.kv_lo && j < it.kv_hi && pi < n_pages;
      const int page = ok ? pages[pi] : -1;
      const bool use = page >= 0;
      const size_t off = use ? (((size_t)page * G + g) * page_tokens + (j % page_tokens)) * HD + c * 8 : 0;
      cp_async16(kd + r * LD + c * 8, k_pages + off, use);
      cp_async16(vd + r * LD + c * 8, v_pages + off, use);
    }
  };

#pragma unroll
  for (int s = 0; s < DS - 1; ++s) {
    if (t_begin + s < t_end) load_tile(t_begin + s, s);
    cp_async_commit();
  }
  for (int t = t_begin; t < t_end; ++t) {
    const int stage = (t - t_begin) % DS;
    cp_async_wait<DS - 2>();
    __syncthreads();      // tile t has landed for everyone, and everyone is done with tile t - 1
    if (t + DS - 1 < t_end) load_tile(t + DS - 1, (stage + DS - 1) % DS);
    cp_async_commit();
    const bf16* kt = ks + stage * DT * LD + warp * 16 * LD;   // this warp's 16 keys of the tile
    const bf16* vt = vs + stage * DT * LD + warp * 16 * LD;
    const int mi = lane >> 3, r8 = lane & 7;

    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t b[4];
      ldmatrix_x4(b, kt + ((mi >> 1) * 8 + r8) * LD + kk * 16 + (mi & 1) * 8);
      mma_bf16(s[0], qf[kk], b[0], b[1]);
      mma_bf16(s[1], qf[kk], b[2], b[3]);
    }
    float mt[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = t * DT + warp * 16 + n * 8 + 2 * qt + (e & 1);
        const bool ok = valid[i] && j >= lo[i] && j <= pos[i] && j >= it.kv_lo && j < it.kv_hi;
        s[n][e] = ok ? s[n][e] * scale_log2 : -CUDART_INF_F;
        mt[i] = fmaxf(mt[i], s[n][e]);
      }
    float corr[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 1));
      mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 2));
      const float mn = fmaxf(m[i], mt[i]);
      msafe[i] = mn == -CUDART_INF_F ? 0.f : mn;
      corr[i] = exp2f(m[i] - msafe[i]);
      m[i] = mn;
      l[i] *= corr[i];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
    uint32_t pf[4];
    float p[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[h][e] = exp2f(s[h][e] - msafe[e >> 1]);
        l[e >> 1] += p[h][e];
      }
    pf[0] = pack_bf16(p[0][0], p[0][1]);
    pf[1] = pack_bf16(p[0][2], p[0][3]);
    pf[2] = pack_bf16(p[1][0], p[1][1]);
    pf[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vt + ((mi & 1) * 8 + r8) * LD + dp * 16 + (mi >> 1) * 8);
      mma_bf16(o[2 * dp], pf, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the warps' states (the tile buffers are free now)
  float* mo = reinterpret_cast<float*>(smem_raw);        // [DW][ROWS][HD]
  float* mm = mo + DW * ROWS * HD;                       // [DW][ROWS]
  float* ml = mm + DW * ROWS;                            // [DW][ROWS]
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    float* dst = mo + ((size_t)warp * ROWS + row[i]) * HD;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<float2*>(dst + n * 8 + 2 * qt) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
    if (qt == 0) {
      mm[warp * ROWS + row[i]] = m[i];
      ml[warp * ROWS + row[i]] = l[i];
    }
  }
  __syncthreads();
  const size_t pbase = it.part < 0 ? 0 : ((size_t)it.part * G + g) * ROWS;
  for (int idx = threadIdx.x; idx < ROWS * HD; idx += DW * 32) {
    const int r = idx / HD, d = idx % HD;
    float mx = mm[r];
#pragma unroll
    for (int w = 1; w < DW; ++w) mx = fmaxf(mx, mm[w * ROWS + r]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < DW; ++w) {
      const float mw = mm[w * ROWS + r];
      const float f = mw == -CUDART_INF_F ? 0.f : exp2f(mw - mx);
      acc += mo[((size_t)w * ROWS + r) * HD + d] * f;
      lsum += ml[w * ROWS + r] * f;
    }
    if (it.part < 0) {
      const int tq = r / group;
      if (tq < it.n_tokens)
        out[((size_t)(it.q_row0 + tq) * H + g * group + r % group) * HD + d] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    } else {
      part_o[(pbase + r) * HD + d] = acc;
      if (d == 0) *reinterpret_cast<float2*>(part_ml + (pbase + r) * 2) = make_float2(mx, lsum);
    }
  }
}

// Decode variant fed by TMA, for head sizes 64 and 128 and pages of 16 tokens or more (a power of two).
// A (page, kv head) slab of the cache is contiguous, so a tile of 64 keys is a few boxes of box_rows keys; ONE
// thread of a producer warp requests them with cp.async.bulk.tensor (a 3-d view [64 columns, rows, halves of
// the head] so that a box brings all of a key's columns and lands as [half][row][128 bytes] with the 128-byte
// swizzle), completion on a "full" mbarrier per stage.  The four consumer warps only compute: each takes 16 of
// the tile's 64 keys, reads K and V through ldmatrix with the swizzle applied to the address, and releases the
// stage on an "empty" mbarrier; there is no block-wide barrier inside the loop.  TS stages per CTA and two
// CTAs per SM keep about 128 KB in flight per SM.  Boxes outside the item's key range are not requested; what
// the stage then holds is masked (K) or finite and multiplied by zero (V: the stages are zeroed once at the
// start).  Every wait is bounded; on time-out the CTA sets `status`, writes nothing and leaves.
constexpr int TW = 4;             // consumer warps (a fifth warp produces)
constexpr int TT = 64;            // keys per tile
constexpr int TS = 3;             // stages
constexpr uint32_t T_WAIT_LIMIT = 1u << 22;

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
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// false: gave up (this wait timed out, or another warp of the CTA already did)
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < T_WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int HD>
__global__ void __launch_bounds__((TW + 1) * 32, 2)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const bf16* __restrict__ q, const int* __restrict__ block_table, int table_stride,
                            const Item* __restrict__ items, bf16* __restrict__ out, float* __restrict__ part_o,
                            float* __restrict__ part_ml, int H, int G, int page_tokens, int box_rows, int window,
                            float scale_log2, int pages_cap, int* __restrict__ status) {
  constexpr int ROWS = 16;
  constexpr int KSTEPS = HD / 16;
  constexpr int TILE_BYTES = TT * HD * 2;            // K (or V) of one stage
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint8_t* kbuf = base;                              // [TS][boxes][HALVES][box_rows][128 bytes]
  uint8_t* vbuf = base + TS * TILE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(vbuf + TS * TILE_BYTES);   // [TS]
  uint64_t* empty = full + TS;                                           // [TS]
  int* abort_flag_s = reinterpret_cast<int*>(empty + TS);
  int* pages = abort_flag_s + 2;                     // [pages_cap]
  volatile int* abort_flag = abort_flag_s;

  const Item it = items[blockIdx.x];
  const int g = blockIdx.y;
  const int group = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = block_table + (size_t)it.slot * table_stride;

  const int page_lo = it.kv_lo / page_tokens;
  const int n_pages = it.kv_hi > it.kv_lo ? min((it.kv_hi - 1) / page_tokens - page_lo + 1, pages_cap) : 0;
  for (int i = threadIdx.x; i < n_pages; i += (TW + 1) * 32) pages[i] = bt[page_lo + i];
  // zero the V stages once: a box that is never requested must not leave NaN patterns to be multiplied by 0
  for (int i = threadIdx.x; i < TS * TILE_BYTES / 16; i += (TW + 1) * 32) reinterpret_cast<uint4*>(vbuf)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < TS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], TW);
    }
    *abort_flag_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeroes are ordered before the TMA writes
  const int t_begin = it.kv_lo / TT;
  const int t_end = (it.kv_hi + TT - 1) / TT;
  // All of the above read only what the host wrote before the step (items, block table); the queries and this
  // step's keys and values come from the kernel before.
  pdl_wait();
  __syncthreads();   // page ids, zeroes and barriers are in place

  float o[HD / 8][4];
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  int row[2] = {0, 0};
  const int qr = lane >> 2, qt = lane & 3;

  if (warp == TW) {
    // ------------------------------------------------------------------ producer
    // One lane per box: lanes [0, boxes) bring the K boxes of a tile, lanes [boxes, 2 * boxes) the V boxes (with
    // 16-token pages a tile is eight copies of 4 KB: issued by one lane they were the kernel's bound).
    const int boxes = TT / box_rows;
    const uint32_t box_bytes = (uint32_t)box_rows * HD * 2;
    const bool is_v = lane >= boxes;
    const int b = is_v ? lane - boxes : lane;
    for (int t = t_begin; t < t_end; ++t) {
      const int n = t - t_begin;
      const int stage = n % TS;
      int ok = 1;
      if (n >= TS && lane == 0) ok = mbar_wait_bounded(&empty[stage], (uint32_t)((n / TS - 1) & 1), abort_flag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int j = t * TT + b * box_rows;
      const int pi = j / page_tokens - page_lo;
      const bool wanted = lane < 2 * boxes && j < it.kv_hi && j + box_rows > it.kv_lo && pi >= 0 && pi < n_pages && pages[pi] >= 0;
      const unsigned mask = __ballot_sync(0xffffffffu, wanted);
      if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)__popc(mask) * box_bytes);
      __syncwarp();
      if (wanted) {
        const int grow = (pages[pi] * G + g) * page_tokens + (j % page_tokens);    // row of the [rows, HD] view
        tma_load_3d((is_v ? vbuf : kbuf) + stage * TILE_BYTES + b * box_bytes, is_v ? &map_v : &map_k, &full[stage], 0, grow, 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    int pos[2], lo[2];
    bool valid[2];
    const bf16* qp[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      row[i] = qr + 8 * i;
      int tq = row[i] / group;
      valid[i] = tq < it.n_tokens;
      if (!valid[i]) tq = 0;
      pos[i] = it.pos0 + tq;
      lo[i] = window > 0 ? max(0, pos[i] - window + 1) : 0;
      qp[i] = q + ((size_t)(it.q_row0 + tq) * H + g * group + row[i] % group) * HD;
    }
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
      qf[s][0] = *reinterpret_cast<const uint32_t*>(qp[0] + s * 16 + 2 * qt);
      qf[s][1] = *reinterpret_cast<const uint32_t*>(qp[1] + s * 16 + 2 * qt);
      qf[s][2] = *reinterpret_cast<const uint32_t*>(qp[0] + s * 16 + 8 + 2 * qt);
      qf[s][3] = *reinterpret_cast<const uint32_t*>(qp[1] + s * 16 + 8 + 2 * qt);
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[n][e] = 0.f;

    // this warp's 16 keys of a tile sit in box (warp * 16) / box_rows at rows (warp * 16) % box_rows ..
    const int my_box = (warp * 16) / box_rows, my_row0 = (warp * 16) % box_rows;
    const uint32_t box_bytes = (uint32_t)box_rows * HD * 2;
    const uint32_t half_bytes = (uint32_t)box_rows * 128;
    const int mi = lane >> 3, r8 = lane & 7;

    for (int t = t_begin; t < t_end; ++t) {
      const int n = t - t_begin;
      const int stage = n % TS;
      if (!mbar_wait_bounded(&full[stage], (uint32_t)((n / TS) & 1), abort_flag)) break;
      const uint32_t kt = smem_u32(kbuf + stage * TILE_BYTES) + my_box * box_bytes;
      const uint32_t vt = smem_u32(vbuf + stage * TILE_BYTES) + my_box * box_bytes;

      float s[2][4];
#pragma unroll
      for (int nn = 0; nn < 2; ++nn)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nn][e] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t b[4];
        const int r = my_row0 + (mi >> 1) * 8 + r8;
        const int d0 = kk * 16 + (mi & 1) * 8;
        const uint32_t addr = kt + (d0 / 64) * half_bytes + r * 128 + ((((d0 % 64) >> 3) ^ (r & 7)) << 4);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(addr));
        mma_bf16(s[0], qf[kk], b[0], b[1]);
        mma_bf16(s[1], qf[kk], b[2], b[3]);
      }
      float mt[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int nn = 0; nn < 2; ++nn)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int j = t * TT + warp * 16 + nn * 8 + 2 * qt + (e & 1);
          const bool ok = valid[i] && j >= lo[i] && j <= pos[i] && j >= it.kv_lo && j < it.kv_hi;
          s[nn][e] = ok ? s[nn][e] * scale_log2 : -CUDART_INF_F;
          mt[i] = fmaxf(mt[i], s[nn][e]);
        }
      float corr[2], msafe[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 1));
        mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 2));
        const float mn = fmaxf(m[i], mt[i]);
        msafe[i] = mn == -CUDART_INF_F ? 0.f : mn;
        corr[i] = exp2f(m[i] - msafe[i]);
        m[i] = mn;
        l[i] *= corr[i];
      }
#pragma unroll
      for (int nn = 0; nn < HD / 8; ++nn) {
        o[nn][0] *= corr[0];
        o[nn][1] *= corr[0];
        o[nn][2] *= corr[1];
        o[nn][3] *= corr[1];
      }
      uint32_t pf[4];
      float p[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[h][e] = exp2f(s[h][e] - msafe[e >> 1]);
          l[e >> 1] += p[h][e];
        }
      pf[0] = pack_bf16(p[0][0], p[0][1]);
      pf[1] = pack_bf16(p[0][2], p[0][3]);
      pf[2] = pack_bf16(p[1][0], p[1][1]);
      pf[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        const int r = my_row0 + (mi & 1) * 8 + r8;
        const int d0 = dp * 16 + (mi >> 1) * 8;
        const uint32_t addr = vt + (d0 / 64) * half_bytes + r * 128 + ((((d0 % 64) >> 3) ^ (r & 7)) << 4);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(addr));
        mma_bf16(o[2 * dp], pf, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);   // this warp is done with the stage
    }
  }
  __syncthreads();
  pdl_launch_dependents();   // the keys are read: the next kernel may move in
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;            // nothing is written
  }

  // ---- merge the consumer warps' states through the (now idle) K stages
  float* mo = reinterpret_cast<float*>(kbuf);            // [TW][ROWS][HD]
  float* mm = mo + TW * ROWS * HD;                       // [TW][ROWS]
  float* ml = mm + TW * ROWS;                            // [TW][ROWS]
  if (warp < TW) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
      float* dst = mo + ((size_t)warp * ROWS + row[i]) * HD;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + 2 * qt) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      if (qt == 0) {
        mm[warp * ROWS + row[i]] = m[i];
        ml[warp * ROWS + row[i]] = l[i];
      }
    }
  }
  __syncthreads();
  const size_t pbase = it.part < 0 ? 0 : ((size_t)it.part * G + g) * ROWS;
  for (int idx = threadIdx.x; idx < ROWS * HD; idx += (TW + 1) * 32) {
    const int r = idx / HD, d = idx % HD;
    float mx = mm[r];
#pragma unroll
    for (int w = 1; w < TW; ++w) mx = fmaxf(mx, mm[w * ROWS + r]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < TW; ++w) {
      const float mw = mm[w * ROWS + r];
      const float f = mw == -CUDART_INF_F ? 0.f : exp2f(mw - mx);
      acc += mo[((size_t)w * ROWS + r) * HD + d] * f;
      lsum += ml[w * ROWS + r] * f;
    }
    if (it.part < 0) {
      const int tq = r / group;
      if (tq < it.n_tokens)
        out[((size_t)(it.q_row0 + tq) * H + g * group + r % group) * HD + d] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    } else {
      part_o[(pbase + r) * HD + d] = acc;
      if (d == 0) *reinterpret_cast<float2*>(part_ml + (pbase + r) * 2) = make_float2(mx, lsum);
    }
  }
}

// One warp per (token, head): merges `count[t]` partials starting at `first[t]` (row `row0[t] + head % group`).
// Tokens with count 0 were written directly by the main kernel.  The partials' (max, sum) pairs are read by
// one lane each, the weights come from a warp-wide maximum, and the value rows are then added in partial
// order with several loads in flight.
template <int HD>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int* __restrict__ first, const int* __restrict__ count,
                                         const int* __restrict__ row0, bf16* __restrict__ out, int n_tokens, int H, int G,
                                         int rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= n_tokens * H) return;
  const int t = w / H, h = w % H;
  const int n = count[t];
  if (n <= 0) return;
  const int group = H / G, g = h / group;
  const int r = row0[t] + h % group;
  const size_t base0 = ((size_t)first[t] * G + g) * rows + r;       // partial s sits at base0 + s * G * rows
  const size_t step = (size_t)G * rows;
  constexpr int PER = (HD + 31) / 32;
  float acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  float mm = -CUDART_INF_F;
  for (int s0 = 0; s0 < n; s0 += 32) {                               // the maximum over all partials
    const int s = s0 + lane;
    mm = fmaxf(mm, s < n ? part_ml[(base0 + s * step) * 2] : -CUDART_INF_F);
  }
  mm = warp_max(mm);
  float lsum = 0.f;
  for (int s0 = 0; s0 < n; s0 += 32) {
    const int s = s0 + lane;
    float f = 0.f, ls = 0.f;
    if (s < n) {
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base0 + s * step) * 2);
      f = ml.x == -CUDART_INF_F ? 0.f : exp2f(ml.x - mm);
      ls = ml.y * f;
    }
    lsum += ls;                                                      // summed over the lanes below, in a fixed order
    const int cnt = min(32, n - s0);
#pragma unroll 8
    for (int j = 0; j < cnt; ++j) {
      const float fj = __shfl_sync(0xffffffffu, f, j);
      const float* po = part_o + (base0 + (size_t)(s0 + j) * step) * HD;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < HD) acc[i] = fmaf(po[d], fj, acc[i]);
      }
    }
  }
  lsum = warp_sum(lsum);
  const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
  bf16* op = out + ((size_t)t * H + h) * HD;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = lane + 32 * i;
    if (d < HD) op[d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

template <int HD, int NW>
int launch_flash(const void* q, const void* kp, const void* vp, const int* bt, int stride, const void* items, int n_items,
                 void* out, float* part_o, float* part_ml, int H, int G, int pt, int window, float scale_log2, cudaStream_t s) {
  const size_t smem = (size_t)4 * TILE_N * (HD + 8) * sizeof(bf16) + 2 * TILE_N * sizeof(int);
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(attention_flash_kernel<HD, NW>, smem, allowed)) return e;
  dim3 grid((unsigned)n_items * (unsigned)G);
  attention_flash_kernel<HD, NW><<<grid, NW * 32, smem, s>>>((const bf16*)q, (const bf16*)kp, (const bf16*)vp, bt, stride,
                                                            (const Item*)items, (bf16*)out, part_o, part_ml, H, G, pt, window,
                                                            scale_log2);
  return hk_launch_status();
}

template <int HD>
int launch_decode(const void* q, const void* kp, const void* vp, const int* bt, int stride, const void* items, int n_items,
                  void* out, float* part_o, float* part_ml, int H, int G, int pt, int window, float scale_log2, int pages_cap,
                  cudaStream_t s) {
  const size_t tiles = (size_t)2 * DS * DT * (HD + 8) * sizeof(bf16);
  const size_t merge = (size_t)DW * 16 * (HD + 2) * sizeof(float);
  const size_t smem = (tiles > merge ? tiles : merge) + (size_t)pages_cap * sizeof(int);
  if (smem > 200 * 1024) return HK_ERR_UNSUPPORTED;
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(attention_decode_kernel<HD>, smem, allowed)) return e;
  dim3 grid((unsigned)n_items, (unsigned)G);
  attention_decode_kernel<HD><<<grid, DW * 32, smem, s>>>((const bf16*)q, (const bf16*)kp, (const bf16*)vp, bt, stride,
                                                         (const Item*)items, (bf16*)out, part_o, part_ml, H, G, pt, window,
                                                         scale_log2, pages_cap);
  return hk_launch_status();
}

template <int HD>
int launch_hd(int nw, const void* q, const void* kp, const void* vp, const int* bt, int stride, const void* items, int n_items,
              void* out, float* part_o, float* part_ml, int H, int G, int pt, int window, float scale_log2, int pages_cap,
              cudaStream_t s) {
  if (nw == 1) return launch_decode<HD>(q, kp, vp, bt, stride, items, n_items, out, part_o, part_ml, H, G, pt, window, scale_log2, pages_cap, s);
  if (nw == 4) return launch_flash<HD, 4>(q, kp, vp, bt, stride, items, n_items, out, part_o, part_ml, H, G, pt, window, scale_log2, s);
  return HK_ERR_UNSUPPORTED;
}

}  // namespace

// items: device array of n_items records of 8 ints (see `Item`).  nw = 4: 64 rows per CTA, a warp per 16 rows;
// nw = 1: the decode variant, 16 rows per CTA whose four warps split the keys.  An item holds at most
// (16 * nw) / (H / G) query tokens.  part_o [parts, G, 16*nw, hd] and part_ml [parts, G, 16*nw, 2] are
// fp32 scratch for items with part >= 0.  scale_log2 = scale * log2(e).  pages_cap: the most pages any item's key
// range spans (the decode variant keeps that many page ids in shared memory).
HK_API int hk_attention_flash(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                              int table_stride, const void* items, int n_items, int nw, void* out, float* part_o,
                              float* part_ml, int H, int G, int hd, int page_tokens, int window, float scale_log2,
                              int pages_cap, void* stream) {
  if (n_items <= 0) return 0;
  if (G < 1 || H % G != 0 || (H / G) > 16 * nw || G > 65535) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
#define HK_HD(D) \
  if (hd == D) return launch_hd<D>(nw, q, k_pages, v_pages, block_table, table_stride, items, n_items, out, part_o, part_ml, H, G, page_tokens, window, scale_log2, pages_cap, s);
  HK_HD(16) HK_HD(32) HK_HD(48) HK_HD(64) HK_HD(80) HK_HD(96) HK_HD(112) HK_HD(128)
#undef HK_HD
  return HK_ERR_UNSUPPORTED;
}

HK_API int hk_attention_combine(const float* part_o, const float* part_ml, const int* first, const int* count,
                                const int* row0, void* out, int n_tokens, int H, int G, int hd, int rows, void* stream) {
  if (n_tokens <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int warps = 4;
  const unsigned grid = (unsigned)(((long long)n_tokens * H + warps - 1) / warps);
#define HK_HD(D) \
  if (hd == D) return hk_launch(attention_combine_kernel<D>, dim3(grid), dim3(warps * 32), 0, s, part_o, part_ml, first, count, row0, (bf16*)out, n_tokens, H, G, rows);
  HK_HD(16) HK_HD(32) HK_HD(48) HK_HD(64) HK_HD(80) HK_HD(96) HK_HD(112) HK_HD(128)
#undef HK_HD
  return HK_ERR_UNSUPPORTED;
}

// ---- host side of the TMA decode variant -----------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// The cache pages of one layer, a bf16 matrix [rows, hd], seen as [64 columns, rows, hd / 64 halves]; a box
// takes 64 columns x box_rows rows x all halves and lands as [half][row][128 bytes] with the 128-byte swizzle.
bool make_page_map(CUtensorMap* map, const void* ptr, unsigned long long rows, int hd, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(hd / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)hd * 2, 128u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)(hd / 64)};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
int launch_decode_tma(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, const int* bt, int stride, const void* items,
                      int n_items, void* out, float* part_o, float* part_ml, int H, int G, int pt, int box_rows, int window,
                      float scale_log2, int pages_cap, int* status, cudaStream_t s) {
  const size_t smem = 1024 + (size_t)2 * TS * TT * HD * 2 + 2 * TS * sizeof(uint64_t) + 8 + (size_t)pages_cap * sizeof(int);
  if (smem > 110 * 1024) return HK_ERR_UNSUPPORTED;
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(attention_decode_tma_kernel<HD>, smem, allowed)) return e;
  dim3 grid((unsigned)n_items, (unsigned)G);
  return hk_launch_pdl(attention_decode_tma_kernel<HD>, grid, dim3((TW + 1) * 32), smem, s, mk, mv, (const bf16*)q, bt, stride,
                       (const Item*)items, (bf16*)out, part_o, part_ml, H, G, pt, box_rows, window, scale_log2, pages_cap, status);
}

}  // namespace

// The decode variant fed by TMA.  Same arguments as hk_attention_flash with nw = 1, plus the number of pages of
// the cache tensors and a device status word (set to 2 if a wait times out).  Refuses (HK_ERR_UNSUPPORTED) head
// sizes other than 64 and 128, pages under 16 tokens or not a power of two, groups above 16 heads.
HK_API int hk_attention_decode_tma(const void* q, const void* k_pages, const void* v_pages, long long num_pages,
                                   const int* block_table, int table_stride, const void* items, int n_items, void* out,
                                   float* part_o, float* part_ml, int H, int G, int hd, int page_tokens, int window,
                                   float scale_log2, int pages_cap, int* status, void* stream) {
  if (n_items <= 0) return 0;
  if (G < 1 || H % G != 0 || (H / G) > 16 || G > 65535) return HK_ERR_UNSUPPORTED;
  if ((hd != 64 && hd != 128) || page_tokens < 16 || (page_tokens & (page_tokens - 1))) return HK_ERR_UNSUPPORTED;
  if (((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127)) return HK_ERR_UNSUPPORTED;
  const int box_rows = page_tokens < TT ? page_tokens : TT;
  const unsigned long long rows = (unsigned long long)num_pages * G * page_tokens;
  CUtensorMap mk, mv;
  if (!make_page_map(&mk, k_pages, rows, hd, box_rows) || !make_page_map(&mv, v_pages, rows, hd, box_rows)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 64)
    return launch_decode_tma<64>(mk, mv, q, block_table, table_stride, items, n_items, out, part_o, part_ml, H, G, page_tokens,
                                 box_rows, window, scale_log2, pages_cap, status, s);
  return launch_decode_tma<128>(mk, mv, q, block_table, table_stride, items, n_items, out, part_o, part_ml, H, G, page_tokens,
                                box_rows, window, scale_log2, pages_cap, status, s);
}

// ---- the entry point that allocates nothing (see attention_noalloc.h) -------------------------------------
#include "attention_noalloc.h"

// Scratch for the partial results, part of the library image: [n_parts][G][16][hd] values, then
// [n_parts][G][16][2] (max, sum).  In host code this name is only a stand-in for the symbol; the device
// address comes from cudaGetSymbolAddress below and is what the kernels are given.
static __device__ __align__(256) float hk_noalloc_scratch[HK_NOALLOC_SCRATCH_BYTES / sizeof(float)];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;
}  // namespace

HK_API int hk_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                       int table_stride, const void* items, int n_items, int n_parts, const int* first,
                                       const int* count, const int* row0, void* out, int n_tokens, int H, int G, int hd,
                                       int page_tokens, int window, float scale_log2, int pages_cap, void* stream) {
  if (n_items <= 0 || n_tokens <= 0) return 0;
  if (n_parts < 0 || G < 1 || hd < 1) return HK_ERR_UNSUPPORTED;
  const size_t rows = 16;
  const size_t need = (size_t)n_parts * G * rows * ((size_t)hd + 2) * sizeof(float);
  if (need > HK_NOALLOC_SCRATCH_BYTES) return HK_ERR_SCRATCH_TOO_SMALL;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return HK_ERR_UNSUPPORTED;
  float* scratch;
  {
    // set-up, once per device, with that device current: the array's address on this device
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
      float* p = nullptr;
      e = cudaGetSymbolAddress((void**)&p, hk_noalloc_scratch);
      if (e != cudaSuccess) return (int)e;
      g_noalloc_ptr[dev] = p;
    }
    scratch = g_noalloc_ptr[dev];
  }
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)n_parts * G * rows * hd;
  int code = hk_attention_flash(q, k_pages, v_pages, block_table, table_stride, items, n_items, 1, out, part_o, part_ml, H, G,
                                hd, page_tokens, window, scale_log2, pages_cap, stream);
  if (code != 0 || n_parts == 0) return code;
  return hk_attention_combine(part_o, part_ml, first, count, row0, out, n_tokens, H, G, hd, (int)rows, stream);
}
