// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores, for head sizes
// 64 and 128 (bf16).  One CTA takes one work item (a run of query tokens of one request, with its key range)
// for one kv head: its 128 rows are (token, query head of the group) pairs, so the group's heads share every
// K/V tile.  Keys come in tiles of 128 (a product of 128 x 128 x 16 reads 8 KB of shared-memory operands for
// 0.5 MFLOP and is bound by the tensor pipe; at 64 keys it was bound by the operand reads, and every tile pays
// one chain of hand-offs whatever its width) through a ring of three K stages and two V stages.  Per tile:
//
//   loader warps (4)   together they cp.async the K tile and the V tile from wherever the block table says the
//                      pages are (any page size) into shared memory in the 128-byte-swizzled layout the tensor
//                      core reads ([half of the head][key][128 bytes]); Q is loaded the same way once
//   MMA warp (1 lane)  S = Q K^T   : tcgen05.mma 128 x 128 x 16, Q and K K-major from shared memory, S in
//                                     tensor memory (two S buffers, so the next tile's scores are computed
//                                     while this tile's softmax runs)
//                      O += P V    : tcgen05.mma 128 x HD x 16, P from tensor memory (two buffers of 64
//                                     columns beside S and O: it never passes through shared memory), V MN-major
//                                     (keys are its K dimension) from shared memory, O in tensor memory
//   softmax warps (8)  two threads per row (half of the tile's keys each): tcgen05.ld of the S row, mask, running
//                      max and sum in fp32, P = exp2(scale * S - max) written as bf16 to tensor memory
//                      (tcgen05.st); the O row is rescaled in tensor memory (tcgen05.ld / tcgen05.st) when the
//                      reference max has to move; at the end O / sum goes out as bf16
//
// Products into different accumulators are only ordered by their barriers here: a buffer of S, P or O is written
// again only after a commit has said that the instruction that read it is complete.
//
// All hand-offs are mbarriers; every wait is bounded and a time-out makes the CTA set `status`, free its tensor
// memory and leave without writing.  Reference counterpart: `attention_tc_128`, src/cuda_device.zig:1069-1248
// (mma.sync, single sequence, contiguous cache).
#include <cuda.h>
#include <math_constants.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int ROWS = 128;        // query rows per CTA = TMEM lanes
constexpr int TK = 128;          // keys per tile
constexpr int KSTAGES = 3;       // K tiles in shared memory (the next tile's scores are taken a tile ahead)
constexpr int VSTAGES = 2;       // V tiles
constexpr int NUM_THREADS = 416; // warps 0-7 softmax, 8 MMA, 9-12 loaders
constexpr uint32_t WAIT_LIMIT = 1u << 17;   // tries of about 100 ns each: some 13 ms, far beyond any legitimate wait

struct Item {
  int q_row0, n_tokens, slot, pos0, kv_lo, kv_hi, part, pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 4) __nanosleep(100);      // a waiting warp must not take issue slots from the working ones
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptors, 128-byte swizzle, version 1 (sm_100).
// K-major ([row][64 elements = 128 bytes], 8-row groups 1024 bytes apart): leading offset unused.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major ([k row][64 elements of the MN dimension = 128 bytes]): 8-row groups of k 1024 bytes apart (stride),
// the next 64 MN elements `lbo` bytes further (leading).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (128 lanes = rows, 8 columns of two bf16 each per 16 k).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ float ex2(float x) {      // 2^x, one instruction; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// byte offset of (row r, 16-byte chunk c along the row) in a [halves][rows][128 bytes] swizzled tile of `rows` rows
__device__ __forceinline__ uint32_t swz(int r, int c, int rows) {
  return (uint32_t)((c >> 3) * (rows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

template <int HD>
struct Smem {
  alignas(1024) uint8_t q[ROWS * HD * 2];
  alignas(1024) uint8_t k[KSTAGES][TK * HD * 2];
  alignas(1024) uint8_t v[VSTAGES][TK * HD * 2];
  alignas(8) uint64_t q_full, k_full[KSTAGES], v_full[VSTAGES], k_empty[KSTAGES], v_empty[VSTAGES], s_full[2], s_empty[2], p_full[2], pv_done[2];
  float xmax[2][2][ROWS];   // [tile parity][key half][row]: partial row maxima of the two threads of a row
  float xsum[2][ROWS];
  uint32_t tmem_base;
  int abort_flag;
  int pages[1];        // [pages_cap], the tail of the dynamic allocation: page ids of the item's key range
};

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_prefill_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                            const int* __restrict__ block_table, int table_stride, const Item* __restrict__ items,
                            bf16* __restrict__ out, int H, int G, int page_tokens, int window, float scale_log2,
                            int pages_cap, int* __restrict__ status) {
  constexpr int CPR = HD / 8;              // 16-byte chunks per row
  constexpr int KSTEPS = HD / 16;          // MMA k-steps over the head dimension
  constexpr uint32_t TMEM_COLS = 512;     // two S buffers of 128 columns, O of HD columns, two P buffers of 64
  constexpr uint32_t S_COL[2] = {0, 128};
  constexpr uint32_t O_COL = 256;
  constexpr uint32_t P_COL[2] = {384, 448};
  // instruction descriptors: fp32 accumulate, bf16 operands; N at bit 17 (>> 3), M at bit 24 (>> 4); bit 16: B is MN-major
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TK >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  Smem<HD>& sm = *reinterpret_cast<Smem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  volatile int* abort_flag = &sm.abort_flag;

  // kv heads are the fast index of the grid: the items come heaviest first, and so do the CTAs of all heads together
  const Item it = items[blockIdx.x / G];
  const int g = blockIdx.x % G;
  const int group = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = block_table + (size_t)it.slot * table_stride;
  const int t_begin = it.kv_lo / TK;
  const int t_end = (it.kv_hi + TK - 1) / TK;
  const int n_rows = it.n_tokens * group;
  int* pages = sm.pages;
  const int page_lo = it.kv_lo / page_tokens;
  const int n_pages = it.kv_hi > it.kv_lo ? min((it.kv_hi - 1) / page_tokens - page_lo + 1, pages_cap) : 0;
  for (int i = threadIdx.x; i < n_pages; i += NUM_THREADS) pages[i] = bt[page_lo + i];

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 128);
    for (int i = 0; i < KSTAGES; ++i) {
      mbar_init(&sm.k_full[i], 128);
      mbar_init(&sm.k_empty[i], 1);
    }
    for (int i = 0; i < VSTAGES; ++i) {
      mbar_init(&sm.v_full[i], 128);
      mbar_init(&sm.v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.s_full[i], 1);
      mbar_init(&sm.s_empty[i], 256);
    }
    mbar_init(&sm.p_full[0], 256);
    mbar_init(&sm.p_full[1], 256);
    mbar_init(&sm.pv_done[0], 1);
    mbar_init(&sm.pv_done[1], 1);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp >= 9) {   // the loaders send for Q at once: it needs nothing of what the others set up
    const int lt = threadIdx.x - 288;
    {   // Q once: row r = (token r / group, head r % group of this kv head's group); rows past the item are zero.
        // A thread copies chunk qc of rows qr0, qr0 + 128 / CPR, ...; token and head advance without divisions.
      const uint32_t qs = smem_u32(sm.q);
      constexpr int QSTEP = 128 / CPR;
      const int qc = lt % CPR, qr0 = lt / CPR;
      int tok = qr0 / group, head = qr0 - tok * group;
#pragma unroll 4
      for (int r = qr0; r < ROWS; r += QSTEP) {
        const bool ok = r < n_rows;
        const bf16* src = q + ((size_t)(it.q_row0 + (ok ? tok : 0)) * H + g * group + (ok ? head : 0)) * HD + qc * 8;
        cp_async16(qs + swz(r, qc, ROWS), src, ok);
        head += QSTEP;
        while (head >= group) {
          head -= group;
          ++tok;
        }
      }
      cp_async_commit();          // the oldest group of this thread; its arrival is signalled inside the tile loop
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp >= 9) {
    // ================================================================= loaders (128 threads)
    // The four warps copy every tile together: a thread copies chunk `c` of rows r0, r0 + RSTEP, ...; a row's
    // page and offset are worked out once per tile (from the page ids preloaded into shared memory) and serve
    // both K and V.  Copy groups go out in the order Q, K(0), V(0), K(1), V(1), ...; a thread tells the tensor
    // core about a tile once its own copies of it have landed: after it has sent K(n) it waits for everything
    // before that (so V(n - 1) is in), after V(n) likewise (so K(n) is in).  One tile's copies are always under
    // way while the thread waits.
    constexpr int RSTEP = 128 / CPR, NR = TK / RSTEP;
    const int lt = threadIdx.x - 288;
    const int c = lt % CPR, r0 = lt / CPR;
    bool q_signalled = false;
    bool alive = true;
    int n = 0;
    for (int t = t_begin; t < t_end; ++t, ++n) {
      const int ks_i = n % KSTAGES, vs_i = n % VSTAGES;
      size_t off[NR];
      uint32_t okbits = 0;
      // one division per tile; from there the page index and the place in the page advance by steps
      int pi = (t * TK + r0) / page_tokens, in_page = (t * TK + r0) - pi * page_tokens;
      pi -= page_lo;
#pragma unroll
      for (int k = 0; k < NR; ++k) {
        const int j = t * TK + r0 + k * RSTEP;
        const int page = (j >= it.kv_lo && j < it.kv_hi && pi >= 0 && pi < n_pages) ? pages[pi] : -1;
        if (page >= 0) okbits |= 1u << k;
        off[k] = page >= 0 ? (((size_t)page * G + g) * page_tokens + in_page) * HD + c * 8 : 0;
        in_page += RSTEP;
        while (in_page >= page_tokens) {
          in_page -= page_tokens;
          ++pi;
        }
      }
      if (!mbar_wait(&sm.k_empty[ks_i], (uint32_t)(((n / KSTAGES) & 1) ^ 1), abort_flag)) { alive = false; break; }   // a fresh barrier lets the first fill through
      const uint32_t ks = smem_u32(sm.k[ks_i]), vs = smem_u32(sm.v[vs_i]);
#pragma unroll
      for (int k = 0; k < NR; ++k) cp_async16(ks + swz(r0 + k * RSTEP, c, TK), k_pages + off[k], (okbits >> k) & 1u);
      cp_async_commit();
      cp_async_wait<1>();         // everything but K(n): Q and, from the second tile on, V(n - 1)
      fence_async_proxy();
      if (!q_signalled) {
        mbar_arrive(&sm.q_full);
        q_signalled = true;
      } else {
        mbar_arrive(&sm.v_full[(n - 1) % VSTAGES]);
      }
      if (!mbar_wait(&sm.v_empty[vs_i], (uint32_t)(((n / VSTAGES) & 1) ^ 1), abort_flag)) { alive = false; break; }
#pragma unroll
      for (int k = 0; k < NR; ++k) cp_async16(vs + swz(r0 + k * RSTEP, c, TK), v_pages + off[k], (okbits >> k) & 1u);
      cp_async_commit();
      cp_async_wait<1>();         // everything but V(n): K(n) is in
      fence_async_proxy();
      mbar_arrive(&sm.k_full[ks_i]);
    }
    cp_async_wait<0>();
    fence_async_proxy();
    if (!q_signalled) mbar_arrive(&sm.q_full);        // no tile at all: Q alone
    else if (alive && n > 0) mbar_arrive(&sm.v_full[(n - 1) % VSTAGES]);
  } else if (warp == 8) {
    // ================================================================= MMA issuer (one lane)
    if (lane == 0) {
      bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
      const uint32_t qs = smem_u32(sm.q);
      // scores of tile t into S buffer (t - t_begin) & 1
      auto issue_s = [&](int t) -> bool {
        const int n = t - t_begin, st = n % KSTAGES, sb = n & 1;
        if (!mbar_wait(&sm.k_full[st], (uint32_t)((n / KSTAGES) & 1), abort_flag)) return false;
        if (!mbar_wait(&sm.s_empty[sb], (uint32_t)(((n >> 1) & 1) ^ 1), abort_flag)) return false;
        tc_fence_after();
        const uint32_t ks = smem_u32(sm.k[st]);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          // half kk / 4 of the head (Q and K: 128 rows per half), 32 bytes per step inside the swizzled row
          umma(tmem + S_COL[sb], desc_k_major(qs + (uint32_t)((kk >> 2) * (ROWS * 128) + (kk & 3) * 32)),
               desc_k_major(ks + (uint32_t)((kk >> 2) * (TK * 128) + (kk & 3) * 32)), IDESC_S, kk ? 1u : 0u);
        }
        umma_commit(&sm.k_empty[st]);
        umma_commit(&sm.s_full[sb]);
        return true;
      };
      if (ok && t_begin < t_end) ok = issue_s(t_begin);
      for (int t = t_begin; t < t_end && ok; ++t) {
        const int n = t - t_begin, st = n % VSTAGES;
        if (t + 1 < t_end && !issue_s(t + 1)) { ok = false; break; }    // next tile's scores run under this tile's softmax
        if (!mbar_wait(&sm.p_full[n & 1], (uint32_t)((n >> 1) & 1), abort_flag)) { ok = false; break; }
        if (!mbar_wait(&sm.v_full[st], (uint32_t)((n / VSTAGES) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t vs = smem_u32(sm.v[st]);
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk) {
          // P: in tensor memory (8 columns per step).  V: MN-major, 16 keys = 16 rows of 128 bytes per step.
          umma_ts(tmem + O_COL, tmem + P_COL[n & 1] + (uint32_t)(kk * 8), desc_mn_major(vs + (uint32_t)kk * 2048u, (uint32_t)(TK * 128)), IDESC_O,
                  (n > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&sm.v_empty[st]);
        umma_commit(&sm.pv_done[n & 1]);     // tile n's product: barrier n & 1, its completion number n >> 1
      }
    }
  } else {
    // ================================================================= softmax (256 threads, two per row)
    // Warp w reads tensor-memory lanes 32 * (w & 3) .. (its rows) and takes half w >> 2 of the tile's keys and of
    // the O columns.  The two threads of a row meet through shared memory for the row's maximum and, at the
    // end, its sum.
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;               // row = TMEM lane
    const int tq = r / group;
    const bool valid = r < n_rows;
    const int pos = it.pos0 + (valid ? tq : 0);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    constexpr int HK = TK / 2, HO = HD / 2;          // keys and O columns per thread
    float m = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int t = t_begin; t < t_end; ++t) {
      const int n = t - t_begin, sb = n & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&sm.s_full[sb], (uint32_t)((n >> 1) & 1), abort_flag))) { ok = false; break; }
      tc_fence_after();
      uint32_t su[HK];
      tmem_ld32(lane_addr + S_COL[sb] + (uint32_t)(half * HK), su);
      tmem_ld32(lane_addr + S_COL[sb] + (uint32_t)(half * HK + 32), su + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&sm.s_empty[sb]);                  // the S buffer may be overwritten by the tile after next
      // Raw scores stay in `su`; the scale is folded into the exponent's multiply-add (it is positive, so the
      // maximum can be taken on raw scores).  Masked keys become -inf once, here.
      const int j0 = t * TK + half * HK;
      const bool whole = valid && j0 >= max(lo, it.kv_lo) && j0 + HK - 1 <= min(pos, it.kv_hi - 1);
      if (!whole) {
#pragma unroll
        for (int i = 0; i < HK; ++i) {
          const int j = j0 + i;
          const bool see = valid && j >= lo && j <= pos && j >= it.kv_lo && j < it.kv_hi;
          if (!see) su[i] = 0xff800000u;             // -inf
        }
      }
      float mraw = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < HK; ++i) mraw = fmaxf(mraw, __uint_as_float(su[i]));
      sm.xmax[n & 1][half][r] = mraw;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");     // the two warps of this quarter
      mraw = fmaxf(mraw, sm.xmax[n & 1][half ^ 1][r]);
      const float mt = mraw * scale_log2;
      // Lazy rescaling: the exponentials are taken against a reference maximum `m` that only moves when the row's
      // true maximum has run ahead of it by more than 2^8 (P then stays below 256, exact in bf16's range, and
      // sum and O stay consistent with it, so the result is the same).  Moving it costs a pass over the O row
      // in tensor memory, which this makes rare.
      const bool move = mt > m + 8.0f;                   // also true for the first finite maximum (m = -inf)
      const float mn = move ? mt : m;
      const float msafe = mn == -CUDART_INF_F ? 0.f : mn;
      const float corr = move ? exp2f(m - msafe) : 1.0f;  // m = -inf -> 0
      l *= corr;
      // P goes into one of two buffers in tensor memory: this tile's was last read by the P V product of the tile
      // before the last one, which has to be complete.  O may only be touched once the product of the last tile has
      // finished, which matters only when the reference moves.  (Two barriers, alternating by tile: a parity wait
      // must never be two completions behind its barrier.)
      const bool any_move = __any_sync(0xffffffffu, n > 0 && move);
      const int need = any_move ? n - 1 : n - 2;     // the P V product that has to be complete by now
      if (need >= 0 && !__all_sync(0xffffffffu, mbar_wait(&sm.pv_done[need & 1], (uint32_t)((need >> 1) & 1), abort_flag))) { ok = false; break; }
      tc_fence_after();
      uint32_t pw[HK / 2];
#pragma unroll
      for (int e = 0; e < HK / 2; ++e) {
        const float p0 = ex2(fmaf(__uint_as_float(su[2 * e]), scale_log2, -msafe));
        const float p1 = ex2(fmaf(__uint_as_float(su[2 * e + 1]), scale_log2, -msafe));
        l += p0 + p1;
        __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        pw[e] = *reinterpret_cast<uint32_t*>(&pk);
      }
      tmem_st32(lane_addr + P_COL[sb] + (uint32_t)(half * (HK / 2)), pw);
      // tensor-memory loads and stores are warp-wide: if any row of the warp moved its reference, the whole warp
      // goes through its half of the O columns (the others multiply by one)
      if (any_move) {
#pragma unroll
        for (int c0 = 0; c0 < HO; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(lane_addr + O_COL + (uint32_t)(half * HO + c0), o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st32(lane_addr + O_COL + (uint32_t)(half * HO + c0), o);
        }
      }
      tmem_st_wait();                                // P (and O) are in tensor memory before the tensor core is told
      m = mn;
      tc_fence_before();
      mbar_arrive(&sm.p_full[n & 1]);
    }
    sm.xsum[half][r] = l;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    l += sm.xsum[half ^ 1][r];
    const int last = t_end - t_begin - 1;
    if (ok && last >= 0 && __all_sync(0xffffffffu, mbar_wait(&sm.pv_done[last & 1], (uint32_t)((last >> 1) & 1), abort_flag))) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* op = out + ((size_t)(it.q_row0 + (valid ? tq : 0)) * H + g * group + (valid ? r % group : 0)) * HD + half * HO;
#pragma unroll
      for (int c0 = 0; c0 < HO; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(lane_addr + O_COL + (uint32_t)(half * HO + c0), o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * e]) * inv, __uint_as_float(o[i + 2 * e + 1]) * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(op + c0 + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) atomicExch(status, 3);
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

template <int HD>
int launch(const void* q, const void* kp, const void* vp, const int* bt, int stride, const void* items, int n_items, void* out,
           int H, int G, int pt, int window, float scale_log2, int pages_cap, int* status, cudaStream_t s) {
  const size_t smem = sizeof(Smem<HD>) + 1024 + (size_t)pages_cap * sizeof(int);
  if (smem > 225 * 1024) return HK_ERR_UNSUPPORTED;
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(attention_prefill_tc_kernel<HD>, smem, allowed)) return e;
  dim3 grid((unsigned)n_items * (unsigned)G);
  attention_prefill_tc_kernel<HD><<<grid, NUM_THREADS, smem, s>>>((const bf16*)q, (const bf16*)kp, (const bf16*)vp, bt, stride,
                                                                 (const Item*)items, (bf16*)out, H, G, pt, window, scale_log2,
                                                                 pages_cap, status);
  return hk_launch_status();
}


// =================================================================================================================
// Two query tiles per CTA.  256 rows = two tiles of 128 (token, head) rows share every K/V tile, and each tile has
// softmax warps of its own (four: one thread per row, no exchange between threads), so that one tile's chain of
// hand-offs (scores ready -> tensor-memory load -> exponentials -> tensor-memory store -> product) runs while the
// other tile's products occupy the tensor pipe.  Tensor memory (512 columns): per tile 128 columns of scores, which
// the probabilities overwrite in place (bf16, the first 64 columns), and HD columns of O.  Because P lies where S
// lay, a tile's next scores are issued after its P V product; tensor-core instructions of one thread run in the
// order they were issued, so they overwrite P only once that product has read it, and a commit after them says
// that everything before is complete (which is why the softmax may touch O once it has seen the next scores).
//
//   warps 0-3 / 4-7   softmax of tile A / B: the row's 128 scores in four chunks of 32 (two live at a time: holding the
//                     row spilled registers, and that local-memory traffic slowed every phase): mask, chunk maximum,
//                     lazy rescaling against an integer reference maximum, exponentials, P -> tensor memory; at the
//                     end O / sum -> out
//   warp 8 (1 lane)   issues S_A S_B | PV_A S_A' | PV_B S_B' | ...
//   warp 9            TMA: K and V tiles of 128 keys, page by page, one lane per box (a box of {64 columns, the page's keys, 1 half
//                     of the head}), into two K and two V stages laid out [half][key][128 bytes], 128-byte swizzle
//
// Q is loaded by the softmax threads (each its own row, cp.async).  The cache pages must be TMA-able as whole
// boxes: 128 % page_tokens == 0 with page_tokens a multiple of 8, or page_tokens a multiple of 128.
constexpr int NT2 = 320;

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

template <int HD>
struct Smem2 {
  alignas(1024) uint8_t q[2][ROWS * HD * 2];
  alignas(1024) uint8_t k[2][TK * HD * 2];
  alignas(1024) uint8_t v[2][TK * HD * 2];
  alignas(8) uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full[2], o_done[2];
  uint32_t tmem_base;
  int abort_flag;
  int pages[1];        // [pages_cap]
};

template <int HD>
__global__ void __launch_bounds__(NT2, 1)
attention_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const bf16* __restrict__ q, const int* __restrict__ block_table, int table_stride,
                             const Item* __restrict__ items, bf16* __restrict__ out, int H, int G, int page_tokens, int window,
                             float scale_log2, int pages_cap, int* __restrict__ status) {
  constexpr int CPR = HD / 8;
  constexpr int KSTEPS = HD / 16;
  constexpr int HALVES = HD / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t SP_COL[2] = {0, 128};
  constexpr uint32_t O_COL[2] = {256, 256 + HD};
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TK >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  Smem2<HD>& sm = *reinterpret_cast<Smem2<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  volatile int* abort_flag = &sm.abort_flag;

  const Item it = items[blockIdx.x / G];
  const int g = blockIdx.x % G;
  const int group = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = block_table + (size_t)it.slot * table_stride;
  const int t_begin = it.kv_lo / TK;
  const int t_end = (it.kv_hi + TK - 1) / TK;
  const int n_rows = it.n_tokens * group;
  const bool two = n_rows > ROWS;                 // the second tile has rows at all
  int* pages = sm.pages;
  const int page_lo = it.kv_lo / page_tokens;
  const int n_pages = it.kv_hi > it.kv_lo ? min((it.kv_hi - 1) / page_tokens - page_lo + 1, pages_cap) : 0;
  for (int i = threadIdx.x; i < n_pages; i += NT2) pages[i] = bt[page_lo + i];
  // The V stages start as zeros: a box that is not copied (a page outside the key range, or one that the request
  // does not hold) leaves its rows as they are, and whatever is there is multiplied by a probability of zero, which
  // must not meet a NaN pattern.  K needs none: a score of such a key is masked before it is looked at.
  {
    uint4* z = reinterpret_cast<uint4*>(sm.v[0]);
    constexpr int N16 = 2 * TK * HD * 2 / 16;
    for (int i = threadIdx.x; i < N16; i += NT2) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 256);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.k_empty[i], 1);
      mbar_init(&sm.v_empty[i], 1);
      mbar_init(&sm.s_full[i], 1);
      mbar_init(&sm.p_full[i], 128);
      mbar_init(&sm.o_done[i], 1);
    }
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp < 8) {
    // Q: every softmax thread sends for its own row (token r / group, head r % group); rows past the item are zero
    const int qt = warp >> 2, r = threadIdx.x & 127, row = qt * ROWS + r;
    const bool ok = row < n_rows;
    const int tok = ok ? row / group : 0, head = ok ? row - tok * group : 0;
    const bf16* src = q + ((size_t)(it.q_row0 + tok) * H + g * group + head) * HD;
    const uint32_t qs = smem_u32(sm.q[qt]);
#pragma unroll
    for (int c = 0; c < CPR; ++c) cp_async16(qs + swz(r, c, ROWS), src + c * 8, ok);
    cp_async_commit();
  }
  fence_async_proxy();            // the zeros above, before the TMA writes of the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const int n_tiles = t_end - t_begin;

  if (warp == 9) {
    // ================================================================= TMA producer (one warp; a lane per box)
    // With small pages a tile is many boxes (16-token pages: 8 boxes of 2 KB per half for K and as many for V), so
    // the lanes issue them side by side; lane 0 alone waits for the stage and announces the bytes.
    const int box_rows = page_tokens < TK ? page_tokens : TK;
    const int boxes = TK / box_rows;                                   // at most 16
    const uint32_t box_bytes = (uint32_t)box_rows * 128u;
    for (int n = 0; n < n_tiles; ++n) {
      const int t = t_begin + n, st = n & 1;
      const uint32_t par = (uint32_t)(((n >> 1) & 1) ^ 1);            // a fresh barrier lets the first fill through
      // this lane's box of the tile: does it hold keys of the range, and does the request hold its page?
      int row = -1;
      if (lane < boxes) {
        const int j = t * TK + lane * box_rows;
        const int pi = j / page_tokens - page_lo;
        if (j < it.kv_hi && j + box_rows > it.kv_lo && pi >= 0 && pi < n_pages && pages[pi] >= 0)
          row = (pages[pi] * G + g) * page_tokens + (j % page_tokens);
      }
      const uint32_t bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, row >= 0)) * box_bytes * HALVES;
      bool alive = true;
      for (int kv = 0; kv < 2 && alive; ++kv) {
        uint64_t* full = kv == 0 ? &sm.k_full[st] : &sm.v_full[st];
        int go = 1;
        if (lane == 0) {
          go = mbar_wait(kv == 0 ? &sm.k_empty[st] : &sm.v_empty[st], par, abort_flag) ? 1 : 0;
          if (go) {
            if (bytes == 0) mbar_arrive(full);
            else mbar_expect_tx(full, bytes);
          }
        }
        go = __shfl_sync(0xffffffffu, go, 0);
        if (!go) { alive = false; break; }
        if (row >= 0) {
          const uint32_t base = smem_u32(kv == 0 ? sm.k[st] : sm.v[st]) + (uint32_t)(lane * box_rows) * 128u;
          const CUtensorMap* map = kv == 0 ? &map_k : &map_v;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) tma_load_3d(base + (uint32_t)h * (TK * 128), map, full, 0, row, h);
        }
      }
      if (!alive) break;
    }
  } else if (warp == 8) {
    // ================================================================= MMA issuer (one lane)
    if (lane == 0) {
      bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
      const int nq = two ? 2 : 1;
      auto issue_s = [&](int qt, int n) {
        const uint32_t qs = smem_u32(sm.q[qt]), ks = smem_u32(sm.k[n & 1]);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk)
          umma(tmem + SP_COL[qt], desc_k_major(qs + (uint32_t)((kk >> 2) * (ROWS * 128) + (kk & 3) * 32)),
               desc_k_major(ks + (uint32_t)((kk >> 2) * (TK * 128) + (kk & 3) * 32)), IDESC_S, kk ? 1u : 0u);
        umma_commit(&sm.s_full[qt]);
      };
      if (ok && n_tiles > 0) {
        ok = mbar_wait(&sm.k_full[0], 0, abort_flag);
        if (ok) {
          tc_fence_after();
          for (int qt = 0; qt < nq; ++qt) issue_s(qt, 0);
          umma_commit(&sm.k_empty[0]);
        }
      }
      for (int n = 0; n < n_tiles && ok; ++n) {
        const int st = n & 1;
        const uint32_t vs = smem_u32(sm.v[st]);
        for (int qt = 0; qt < nq && ok; ++qt) {
          if (!mbar_wait(&sm.p_full[qt], (uint32_t)(n & 1), abort_flag)) { ok = false; break; }
          if (qt == 0 && !mbar_wait(&sm.v_full[st], (uint32_t)((n >> 1) & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < TK / 16; ++kk)
            umma_ts(tmem + O_COL[qt], tmem + SP_COL[qt] + (uint32_t)(kk * 8), desc_mn_major(vs + (uint32_t)kk * 2048u, (uint32_t)(TK * 128)),
                    IDESC_O, (n > 0 || kk > 0) ? 1u : 0u);
          if (qt == nq - 1) umma_commit(&sm.v_empty[st]);
          if (n + 1 < n_tiles) {
            if (qt == 0 && !mbar_wait(&sm.k_full[(n + 1) & 1], (uint32_t)(((n + 1) >> 1) & 1), abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_s(qt, n + 1);       // after this tile's P V: it overwrites the P that product reads
            if (qt == nq - 1) umma_commit(&sm.k_empty[(n + 1) & 1]);
          } else {
            umma_commit(&sm.o_done[qt]);
          }
        }
      }
    }
  } else {
    // ================================================================= softmax (two groups of 128 threads, one per row)
    const int qt = warp >> 2, quarter = warp & 3;
    const int r = quarter * 32 + lane;                 // row of the tile = TMEM lane
    const int row = qt * ROWS + r;
    const int tq = row / group;
    const bool valid = row < n_rows;
    const int pos = it.pos0 + (valid ? tq : 0);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    cp_async_wait<0>();
    fence_async_proxy();
    mbar_arrive(&sm.q_full);
    float m = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    bool ok = true;
    if (qt == 0 || two) {
      for (int n = 0; n < n_tiles; ++n) {
        const int t = t_begin + n;
        if (!__all_sync(0xffffffffu, mbar_wait(&sm.s_full[qt], (uint32_t)(n & 1), abort_flag))) { ok = false; break; }
        tc_fence_after();
        // The row's 128 scores in four chunks of 32: while one chunk's exponentials run, the next chunk is on its way
        // from tensor memory, and a thread holds two chunks, not the row.  The reference maximum m is an integer and
        // moves only when a chunk's maximum runs ahead of it by more than 8 (so a probability is at most 2^8); what was
        // summed under the old reference (l, O, this tile's earlier chunks of P) is then multiplied by a power of two,
        // which is exact.  The scores of this tile are complete, and so is every product issued before them, the last
        // P V among them: O may be touched.
        const int j0 = t * TK;
        const bool whole = valid && j0 >= max(lo, it.kv_lo) && j0 + TK - 1 <= min(pos, it.kv_hi - 1);
        uint32_t sc[2][32];
        tmem_ld32(lane_addr + SP_COL[qt], sc[0]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < TK / 32; ++c) {
          uint32_t* su = sc[c & 1];
          if (c + 1 < TK / 32) tmem_ld32(lane_addr + SP_COL[qt] + (uint32_t)(32 * (c + 1)), sc[(c + 1) & 1]);
          if (!whole) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int j = j0 + 32 * c + i;
              const bool see = valid && j >= lo && j <= pos && j >= it.kv_lo && j < it.kv_hi;
              if (!see) su[i] = 0xff800000u;             // -inf
            }
          }
          float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
#pragma unroll
            for (int e = 0; e < 4; ++e) mx[e] = fmaxf(mx[e], fmaxf(__uint_as_float(su[i + 2 * e]), __uint_as_float(su[i + 2 * e + 1])));
          }
          const float cm = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
          const bool move = cm > m + 8.0f;
          if (__any_sync(0xffffffffu, move)) {
            const float mn = move ? ceilf(cm) : m;
            const float corr = move ? exp2f(m - mn) : 1.0f;      // m = -inf: 0; nothing was summed yet
            l0 *= corr;
            l1 *= corr;
            if (n > 0) {
#pragma unroll 1
              for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(lane_addr + O_COL[qt] + (uint32_t)c0, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                tmem_st32(lane_addr + O_COL[qt] + (uint32_t)c0, o);
              }
            }
            if (c > 0) tmem_st_wait();       // this tile's earlier chunks of P are in tensor memory before they are read back
#pragma unroll 1
            for (int cp = 0; cp < c; ++cp) {
              uint32_t pp[16];
              tmem_ld16(lane_addr + SP_COL[qt] + (uint32_t)(16 * cp), pp);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&pp[i]);
                float2 f = __bfloat1622float2(v);
                v = __floats2bfloat162_rn(f.x * corr, f.y * corr);
                pp[i] = *reinterpret_cast<uint32_t*>(&v);
              }
              tmem_st16(lane_addr + SP_COL[qt] + (uint32_t)(16 * cp), pp);
            }
            m = mn;
          }
          const float msafe = m == -CUDART_INF_F ? 0.f : m;
          uint32_t pw[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = ex2(fmaf(__uint_as_float(su[2 * e]), scale_log2, -msafe));
            const float p1 = ex2(fmaf(__uint_as_float(su[2 * e + 1]), scale_log2, -msafe));
            l0 += p0;
            l1 += p1;
            __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
            pw[e] = *reinterpret_cast<uint32_t*>(&pk);
          }
          tmem_st16(lane_addr + SP_COL[qt] + (uint32_t)(16 * c), pw);
          if (c + 1 < TK / 32) tmem_ld_wait();
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&sm.p_full[qt]);
      }
      if (ok && n_tiles > 0 && __all_sync(0xffffffffu, mbar_wait(&sm.o_done[qt], 0, abort_flag))) {
        tc_fence_after();
        const float l = l0 + l1;
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        bf16* op = out + ((size_t)(it.q_row0 + (valid ? tq : 0)) * H + g * group + (valid ? row % group : 0)) * HD;
        // the whole row of O at once (the registers that held scores are free now): one wait instead of HD / 32
        uint32_t o[HD];
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) tmem_ld32(lane_addr + O_COL[qt] + (uint32_t)c0, o + c0);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < HD; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * e]) * inv, __uint_as_float(o[i + 2 * e + 1]) * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(op + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) atomicExch(status, 3);
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

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

// The cache pages of one layer, a bf16 matrix [rows, hd], seen as [64 columns, rows, hd / 64 halves]; a box takes
// 64 columns x box_rows rows of one half and lands as [row][128 bytes] with the 128-byte swizzle.  The map covers
// this GPU's own memory; the loads use no multicast.
bool make_page_map(CUtensorMap* map, const void* ptr, unsigned long long rows, int hd, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(hd / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)hd * 2, 128u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
int launch2(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, const int* bt, int stride, const void* items, int n_items,
            void* out, int H, int G, int pt, int window, float scale_log2, int pages_cap, int* status, cudaStream_t s) {
  const size_t smem = sizeof(Smem2<HD>) + 1024 + (size_t)pages_cap * sizeof(int);
  if (smem > 225 * 1024) return HK_ERR_UNSUPPORTED;
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(attention_prefill_tc2_kernel<HD>, smem, allowed)) return e;
  dim3 grid((unsigned)n_items * (unsigned)G);
  return hk_launch(attention_prefill_tc2_kernel<HD>, grid, dim3(NT2), smem, s, mk, mv, (const bf16*)q, bt, stride, (const Item*)items,
                   (bf16*)out, H, G, pt, window, scale_log2, pages_cap, status);
}

}  // namespace

// items: n_items records of 8 ints {first query row, query tokens (at most 128 / (H / G)), request slot, position
// of the first token, first key, one past the last key, -1, 0}.  pages_cap: the most pages an item's key range spans.  Writes out[token, head, :] directly (no key
// splitting).  `status` is a device int set to 3 if a wait timed out.  Refuses (HK_ERR_UNSUPPORTED) head sizes
// other than 64 and 128 and groups above 128 heads.
HK_API int hk_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                   int table_stride, const void* items, int n_items, void* out, int H, int G, int hd,
                                   int page_tokens, int window, float scale_log2, int pages_cap, int* status, void* stream) {
  if (n_items <= 0) return 0;
  if (G < 1 || H % G != 0 || (H / G) > ROWS || G > 65535 || page_tokens < 1 || !(scale_log2 > 0.f)) return HK_ERR_UNSUPPORTED;
  if ((((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) & 15) != 0) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 128) return launch<128>(q, k_pages, v_pages, block_table, table_stride, items, n_items, out, H, G, page_tokens, window, scale_log2, pages_cap, status, s);
  if (hd == 64) return launch<64>(q, k_pages, v_pages, block_table, table_stride, items, n_items, out, H, G, page_tokens, window, scale_log2, pages_cap, status, s);
  return HK_ERR_UNSUPPORTED;
}

// The same for items of up to 256 / (H / G) query tokens (two query tiles per CTA, K and V by TMA).  `num_pages`:
// pages of the cache tensors.  Refuses (HK_ERR_UNSUPPORTED) what hk_attention_prefill_tc refuses and page sizes
// whose pages are not whole TMA boxes of a 128-key tile: it takes multiples of 8 that divide 128, and multiples of 128.
HK_API int hk_attention_prefill_tc2(const void* q, const void* k_pages, const void* v_pages, long long num_pages,
                                    const int* block_table, int table_stride, const void* items, int n_items, void* out, int H,
                                    int G, int hd, int page_tokens, int window, float scale_log2, int pages_cap, int* status,
                                    void* stream) {
  if (n_items <= 0) return 0;
  if (G < 1 || H % G != 0 || (H / G) > ROWS || G > 65535 || page_tokens < 1 || !(scale_log2 > 0.f)) return HK_ERR_UNSUPPORTED;
  if (hd != 64 && hd != 128) return HK_ERR_UNSUPPORTED;
  const bool boxes_ok = (page_tokens % 8 == 0 && TK % page_tokens == 0) || page_tokens % TK == 0;
  if (!boxes_ok) return HK_ERR_UNSUPPORTED;
  if ((((uintptr_t)q | (uintptr_t)out) & 15) != 0 || (((uintptr_t)k_pages | (uintptr_t)v_pages) & 127) != 0) return HK_ERR_UNSUPPORTED;
  const int box_rows = page_tokens < TK ? page_tokens : TK;
  const unsigned long long rows = (unsigned long long)num_pages * G * page_tokens;
  CUtensorMap mk, mv;
  if (!make_page_map(&mk, k_pages, rows, hd, box_rows) || !make_page_map(&mv, v_pages, rows, hd, box_rows)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 128) return launch2<128>(mk, mv, q, block_table, table_stride, items, n_items, out, H, G, page_tokens, window, scale_log2, pages_cap, status, s);
  return launch2<64>(mk, mv, q, block_table, table_stride, items, n_items, out, H, G, page_tokens, window, scale_log2, pages_cap, status, s);
}

