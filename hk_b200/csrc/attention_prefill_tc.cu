// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores, for head sizes
// 64 and 128 (bf16).  One CTA takes one work item (a run of query tokens of one request, with its key range)
// for one kv head: its 128 rows are (token, query head of the group) pairs, so the group's heads share every
// K/V tile.  Keys come in tiles of 64 through a ring of four stages (three tiles in flight).  Per tile:
//
//   loader warps (4)   warp w owns stage w and every fourth tile: it cp.asyncs the K tile and the V tile from
//                      wherever the block table says the pages are into shared memory in the 128-byte-swizzled
//                      layout the tensor core reads ([half of the head][key][128 bytes]); Q is loaded the same
//                      way once
//   MMA warp (1 lane)  S = Q K^T   : tcgen05.mma 128 x 64 x 16, Q and K K-major from shared memory, S in
//                                     tensor memory (two S buffers, so the next tile's scores are computed
//                                     while this tile's softmax runs)
//                      O += P V    : tcgen05.mma 128 x HD x 16, P from tensor memory (two buffers of 32
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
#include <math_constants.h>

#include "common.cuh"

#ifdef HK_TRACE
// Timing probes for one CTA (the first, heaviest work item, kv head 0): role r writes clock64() at its n-th probe.
__device__ long long hk_trace_buf[4][512];
__device__ int hk_trace_n[4];
#define TRACE(role) do { if (trace_on) { if (trace_i < 512) { hk_trace_buf[role][trace_i] = clock64(); hk_trace_n[role] = ++trace_i; } } } while (0)
#else
#define TRACE(role) do { } while (0)
#endif

namespace {

constexpr int ROWS = 128;        // query rows per CTA = TMEM lanes
constexpr int TK = 64;           // keys per tile
constexpr int STAGES = 4;        // K/V stages, one per loader warp
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
  alignas(1024) uint8_t k[STAGES][TK * HD * 2];
  alignas(1024) uint8_t v[STAGES][TK * HD * 2];
  alignas(8) uint64_t q_full, k_full[STAGES], v_full[STAGES], k_empty[STAGES], v_empty[STAGES], s_full[2], s_empty[2], p_full[2], pv_done[2];
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
  constexpr uint32_t TMEM_COLS = 512;     // two S buffers of 64 columns, O of HD columns, two P buffers of 32 (a power of two is allocated)
  constexpr uint32_t S_COL[2] = {0, 64};
  constexpr uint32_t O_COL = 128;
  constexpr uint32_t P_COL[2] = {256, 288};
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
#ifdef HK_TRACE
  const bool trace_on = blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 8 || warp == 9 || warp == 10);
  int trace_i = 0;      // the probe count lives in a register: a probe is one clock read and two stores
  if (threadIdx.x == 0 && blockIdx.x == 0) { hk_trace_n[0] = hk_trace_n[1] = hk_trace_n[2] = hk_trace_n[3] = 0; }
#endif
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
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&sm.k_full[i], 32);
      mbar_init(&sm.v_full[i], 32);
      mbar_init(&sm.k_empty[i], 1);
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
    bool q_signalled = false;
    // Loader warp w owns stage w and tiles w, w + 4, ...: it can wait for its own copies to land without
    // holding up the other three, so up to four tiles are on their way.  A lane copies chunk `c` of rows r0,
    // r0 + RSTEP, ...; a row's page and offset are worked out once per tile (from the page ids preloaded into
    // shared memory) and serve both K and V.
    constexpr int RSTEP = 32 / CPR, NR = TK / RSTEP;
    const int lw = warp - 9;
    const int c = lane % CPR, r0 = lane / CPR;
    for (int t = t_begin + lw; t < t_end; t += STAGES) {
      const int n = t - t_begin, st = lw;
      const uint32_t par = (uint32_t)((((n / STAGES) & 1)) ^ 1);      // a fresh barrier lets the first fill through
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
      TRACE(2 + (lw & 1));
      if (!mbar_wait(&sm.k_empty[st], par, abort_flag)) break;
      TRACE(2 + (lw & 1));
      const uint32_t ks = smem_u32(sm.k[st]), vs = smem_u32(sm.v[st]);
#pragma unroll
      for (int k = 0; k < NR; ++k) cp_async16(ks + swz(r0 + k * RSTEP, c, TK), k_pages + off[k], (okbits >> k) & 1u);
      cp_async_commit();
      if (!mbar_wait(&sm.v_empty[st], par, abort_flag)) break;
      TRACE(2 + (lw & 1));
#pragma unroll
      for (int k = 0; k < NR; ++k) cp_async16(vs + swz(r0 + k * RSTEP, c, TK), v_pages + off[k], (okbits >> k) & 1u);
      cp_async_commit();
      if (!q_signalled) {         // Q went out first: it has landed when at most the two groups after it are pending
        cp_async_wait<2>();
        fence_async_proxy();
        mbar_arrive(&sm.q_full);
        q_signalled = true;
      }
      cp_async_wait<1>();
      fence_async_proxy();
      mbar_arrive(&sm.k_full[st]);
      cp_async_wait<0>();
      fence_async_proxy();
      mbar_arrive(&sm.v_full[st]);
      TRACE(2 + (lw & 1));
    }
    if (!q_signalled) {           // a loader warp without a tile of its own (short key ranges) still delivers its part of Q
      cp_async_wait<0>();
      fence_async_proxy();
      mbar_arrive(&sm.q_full);
    }
  } else if (warp == 8) {
    // ================================================================= MMA issuer (one lane)
    if (lane == 0) {
      bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
      const uint32_t qs = smem_u32(sm.q);
      // scores of tile t into S buffer (t - t_begin) & 1
      auto issue_s = [&](int t) -> bool {
        const int n = t - t_begin, st = n % STAGES, sb = n & 1;
        TRACE(1);
        if (!mbar_wait(&sm.k_full[st], (uint32_t)((n / STAGES) & 1), abort_flag)) return false;
        TRACE(1);
        if (!mbar_wait(&sm.s_empty[sb], (uint32_t)(((n >> 1) & 1) ^ 1), abort_flag)) return false;
        tc_fence_after();
        const uint32_t ks = smem_u32(sm.k[st]);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          // half kk / 4 of the head (Q: 128 rows per half, K: 64), 32 bytes per step inside the swizzled row
          umma(tmem + S_COL[sb], desc_k_major(qs + (uint32_t)((kk >> 2) * (ROWS * 128) + (kk & 3) * 32)),
               desc_k_major(ks + (uint32_t)((kk >> 2) * (TK * 128) + (kk & 3) * 32)), IDESC_S, kk ? 1u : 0u);
        }
        umma_commit(&sm.k_empty[st]);
        umma_commit(&sm.s_full[sb]);
        return true;
      };
      if (ok && t_begin < t_end) ok = issue_s(t_begin);
      for (int t = t_begin; t < t_end && ok; ++t) {
        const int n = t - t_begin, st = n % STAGES;
        if (t + 1 < t_end && !issue_s(t + 1)) { ok = false; break; }    // next tile's scores run under this tile's softmax
        TRACE(1);
        if (!mbar_wait(&sm.p_full[n & 1], (uint32_t)((n >> 1) & 1), abort_flag)) { ok = false; break; }
        TRACE(1);
        if (!mbar_wait(&sm.v_full[st], (uint32_t)((n / STAGES) & 1), abort_flag)) { ok = false; break; }
        TRACE(1);
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
      TRACE(0);
      if (!__all_sync(0xffffffffu, mbar_wait(&sm.s_full[sb], (uint32_t)((n >> 1) & 1), abort_flag))) { ok = false; break; }
      TRACE(0);
      tc_fence_after();
      uint32_t su[HK];
      tmem_ld32(lane_addr + S_COL[sb] + (uint32_t)(half * HK), su);
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
      TRACE(0);
      const bool any_move = __any_sync(0xffffffffu, n > 0 && move);
      const int need = any_move ? n - 1 : n - 2;     // the P V product that has to be complete by now
      if (need >= 0 && !__all_sync(0xffffffffu, mbar_wait(&sm.pv_done[need & 1], (uint32_t)((need >> 1) & 1), abort_flag))) { ok = false; break; }
      TRACE(0);
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
      tmem_st16(lane_addr + P_COL[sb] + (uint32_t)(half * (HK / 2)), pw);
      TRACE(0);
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
      TRACE(0);
      TRACE(0);
      tc_fence_before();
      mbar_arrive(&sm.p_full[n & 1]);
      TRACE(0);
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

#ifdef HK_TRACE
// Copies the probes of the last traced launch to the host: out[4][512] clocks, counts[4].
HK_API int hk_attention_prefill_tc_trace(long long* out, int* counts) {
  cudaError_t e = cudaMemcpyFromSymbol(out, hk_trace_buf, sizeof(long long) * 4 * 512);
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(counts, hk_trace_n, sizeof(int) * 4);
  return (int)e;
}
#endif
