// Sampling on the device: argmax, and the reference's chain penalties -> top-k -> top-p ->
// min-p -> temperature -> draw (src/sampler.zig:3-6,115-217), one thread block per row of
// logits.  The reference samples on the host from a copy of the logits; here the logits stay
// on the device and only the chosen token ids leave it.
//
//   * temperature <= 0: the first maximum wins (src/sampler.zig:128-135).
//   * top-k: at most min(top_k or 4096, 4096) finite candidates survive (:31,137-161); among
//     equal logits the smaller id is kept (lessCand, :62-66).  Found by a radix select over
//     order-preserving integer keys, then gathered in id order.
//   * candidates sorted by logit descending, id ascending (:162-167): bitonic sort in shared memory.
//   * probabilities at temperature 1 over the candidates; top-p keeps through the first
//     candidate at which the running sum reaches p (:169-191); min-p keeps the leading
//     candidates with probability >= p0 * min_p, at least one (:192-197).
//   * temperature on the survivors, then inverse-CDF draw with one uniform number (:199-216).
// The uniform number comes from a counter-based generator keyed by (seed, counter) per row,
// so a request's draws repeat exactly for the same seed and do not depend on the batch.
#include <math_constants.h>

#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_MAX_CAND 4096

__device__ __forceinline__ unsigned int order_key(float f) {
  // larger float -> larger unsigned key
  unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_to_float(unsigned int k) {
  unsigned int u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ bool is_finite(float f) { return fabsf(f) <= 3.402823466e38f; }

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// uniform in [0, 1) with 24 bits, from (seed, counter)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter) {
  unsigned long long h = splitmix64(splitmix64(seed) ^ (counter * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
  return (float)(h >> 40) * (1.0f / 16777216.0f);
}

// ---- block-wide helpers (blockDim.x == SMP_THREADS) -----------------------------------------

// argmax with "first maximum wins"; NaN never wins.  Returns to every thread.
__device__ int block_argmax(const float* __restrict__ row, int V, float* s_val, int* s_idx) {
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = row[i];
    if (v > best || (bi == 0x7fffffff && v == best)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    s_val[wid] = best;
    s_idx[wid] = bi;
  }
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    best = lane < nw ? s_val[lane] : -CUDART_INF_F;
    bi = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) s_idx[0] = (bi == 0x7fffffff) ? 0 : bi;
  }
  __syncthreads();
  int r = s_idx[0];
  __syncthreads();
  return r;
}

// inclusive prefix sum of one int per thread; returns the thread's inclusive value, *total = sum
__device__ int block_scan_int(int v, int* s_warp, int* total) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) s_warp[wid] = x;
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    int w = lane < nw ? s_warp[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    if (lane < nw) s_warp[lane] = w;
  }
  __syncthreads();
  int base = wid > 0 ? s_warp[wid - 1] : 0;
  *total = s_warp[(blockDim.x >> 5) - 1];
  __syncthreads();
  return base + x;
}

// inclusive prefix sum over s[0..n) floats in shared memory, n <= 4 * blockDim.x, in place
__device__ void block_scan_float4(float* s, int n, float* s_warp) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int b = threadIdx.x * 4;
  float a0 = b < n ? s[b] : 0.f, a1 = b + 1 < n ? s[b + 1] : 0.f, a2 = b + 2 < n ? s[b + 2] : 0.f,
        a3 = b + 3 < n ? s[b + 3] : 0.f;
  a1 += a0;
  a2 += a1;
  a3 += a2;
  float x = a3;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) s_warp[wid] = x;
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    float w = lane < nw ? s_warp[lane] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    if (lane < nw) s_warp[lane] = w;
  }
  __syncthreads();
  float base = (wid > 0 ? s_warp[wid - 1] : 0.f) + (x - a3);
  if (b < n) s[b] = base + a0;
  if (b + 1 < n) s[b + 1] = base + a1;
  if (b + 2 < n) s[b + 2] = base + a2;
  if (b + 3 < n) s[b + 3] = base + a3;
  __syncthreads();
}

// ---- argmax ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SMP_THREADS) argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  int r = block_argmax(logits + (size_t)blockIdx.x * V, V, s_val, s_idx);
  if (threadIdx.x == 0) out[blockIdx.x] = r;
}

HK_API int hk_argmax(const float* logits, int rows, int V, int* out, void* stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, SMP_THREADS, 0, (cudaStream_t)stream>>>(logits, V, out);
  return hk_launch_status();
}

// ---- penalties and bias -----------------------------------------------------------------------
// For row r, entries [offsets[r], offsets[r+1]) of (ids, counts, bias): a token seen `count`
// times among the recent ones gets l = l > 0 ? l / rp : l * rp, then l -= count * freq + presence
// (src/sampler.zig:82-111); every entry then adds its bias (the logit_bias list).
__global__ void adjust_logits_kernel(float* __restrict__ logits, int V, const int* __restrict__ offsets,
                                     const int* __restrict__ ids, const int* __restrict__ counts,
                                     const float* __restrict__ bias, const float* __restrict__ repeat_penalty,
                                     const float* __restrict__ freq_penalty, const float* __restrict__ presence_penalty) {
  int r = blockIdx.x;
  float rp = repeat_penalty[r], fp = freq_penalty[r], pp = presence_penalty[r];
  for (int e = offsets[r] + threadIdx.x; e < offsets[r + 1]; e += blockDim.x) {
    int id = ids[e];
    if (id < 0 || id >= V) continue;
    float* p = logits + (size_t)r * V + id;
    float l = *p;
    int c = counts[e];
    if (c > 0) {
      if (rp != 1.0f) l = l > 0.f ? l / rp : l * rp;
      l -= (float)c * fp + pp;
    }
    *p = l + bias[e];
  }
}

HK_API int hk_adjust_logits(float* logits, int rows, int V, const int* offsets, const int* ids, const int* counts,
                            const float* bias, const float* repeat_penalty, const float* freq_penalty,
                            const float* presence_penalty, void* stream) {
  if (rows <= 0) return 0;
  adjust_logits_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(logits, V, offsets, ids, counts, bias, repeat_penalty,
                                                             freq_penalty, presence_penalty);
  return hk_launch_status();
}

// ---- the sampling chain ---------------------------------------------------------------------
struct SampleShared {
  unsigned long long cand[SMP_MAX_CAND];  // (~key << 32) | id : ascending sort = logit desc, id asc
  float prob[SMP_MAX_CAND];
  unsigned int hist[256];
  float s_val[32];
  int s_idx[32];
  int s_warp[32];
  float s_warpf[32];
  unsigned int prefix;    // key bits decided so far
  int remaining;          // candidates still to find among keys equal to the prefix
  int n_finite;
  int keep;
  int chosen;
};

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
              int* __restrict__ out) {
  extern __shared__ unsigned char smem_raw[];
  SampleShared& sh = *reinterpret_cast<SampleShared*>(smem_raw);
  int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  float T = temperature[r];
  if (!(T > 0.f)) {
    int a = block_argmax(row, V, sh.s_val, sh.s_idx);
    if (threadIdx.x == 0) out[r] = a;
    return;
  }
  // how many finite logits there are
  int nf = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) nf += is_finite(row[i]) ? 1 : 0;
  int tot;
  block_scan_int(nf, sh.s_warp, &tot);
  if (tot == 0) {
    if (threadIdx.x == 0) out[r] = 0;   // src/sampler.zig:161
    return;
  }
  int want = top_k[r] <= 0 ? SMP_MAX_CAND : min(top_k[r], SMP_MAX_CAND);
  int k = min(want, tot);

  // radix select: the key of the k-th largest finite logit
  if (threadIdx.x == 0) {
    sh.prefix = 0;
    sh.remaining = k;
  }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0;
    __syncthreads();
    unsigned int prefix = sh.prefix;
    unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float v = row[i];
      if (!is_finite(v)) continue;
      unsigned int key = order_key(v);
      if ((key & mask) == (prefix & mask)) atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int rem = sh.remaining;
      int b = 255;
      for (; b > 0; --b) {
        int c = (int)sh.hist[b];
        if (c >= rem) break;
        rem -= c;
      }
      sh.prefix = prefix | ((unsigned int)b << shift);
      sh.remaining = rem;   // candidates to take among keys whose decided bits equal the prefix
    }
    __syncthreads();
  }
  unsigned int thr = sh.prefix;   // key of the k-th largest
  int ties_to_take = sh.remaining; // how many keys == thr are kept (smallest ids first)
  __syncthreads();

  // gather in id order: keys > thr, and the first `ties_to_take` keys == thr
  int n_above_so_far = 0, n_ties_so_far = 0;
  for (int base = 0; base < V; base += blockDim.x) {
    int i = base + threadIdx.x;
    float v = i < V ? row[i] : 0.f;
    bool fin = i < V && is_finite(v);
    unsigned int key = fin ? order_key(v) : 0u;
    int above = fin && key > thr;
    int tie = fin && key == thr;
    int ta, tt;
    int pa = block_scan_int(above, sh.s_warp, &ta);
    int pt = block_scan_int(tie, sh.s_warp, &tt);
    int tie_rank = n_ties_so_far + pt - tie;   // 0-based rank among ties, in id order
    bool take_tie = tie && tie_rank < ties_to_take;
    int ties_taken_before = min(n_ties_so_far, ties_to_take) + min(pt - tie, max(0, ties_to_take - n_ties_so_far));
    if (above || take_tie) {
      int slot = n_above_so_far + (pa - above) + ties_taken_before;
      sh.cand[slot] = ((unsigned long long)(~key) << 32) | (unsigned int)i;
    }
    n_above_so_far += ta;
    n_ties_so_far += tt;
    __syncthreads();
  }
  // pad to a power of two with keys that sort last
  int n2 = 1;
  while (n2 < k) n2 <<= 1;
  for (int i = k + threadIdx.x; i < n2; i += blockDim.x) sh.cand[i] = 0xffffffffffffffffull;
  __syncthreads();
  // bitonic sort ascending
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (n2 >> 1); t += blockDim.x) {
        int lo = (t / stride) * (stride << 1) + (t % stride);
        int hi = lo + stride;
        bool up = ((lo & size) == 0);
        unsigned long long a = sh.cand[lo], b = sh.cand[hi];
        if ((a > b) == up) {
          sh.cand[lo] = b;
          sh.cand[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  // probabilities at temperature 1
  float max_logit = key_to_float(~(unsigned int)(sh.cand[0] >> 32));
  for (int i = threadIdx.x; i < k; i += blockDim.x)
    sh.prob[i] = expf(key_to_float(~(unsigned int)(sh.cand[i] >> 32)) - max_logit);
  __syncthreads();
  block_scan_float4(sh.prob, k, sh.s_warpf);   // prob[i] = running sum
  float total = sh.prob[k - 1];
  float p0 = sh.prob[0] / total;
  if (threadIdx.x == 0) sh.keep = k;
  __syncthreads();
  float tp = top_p[r];
  if (tp > 0.f && tp < 1.f) {
    // first i with cum_i / total >= tp
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
      float cum = sh.prob[i] / total;
      float prev = i > 0 ? sh.prob[i - 1] / total : 0.f;
      if (cum >= tp && (i == 0 || prev < tp)) atomicMin(&sh.keep, i + 1);
    }
    __syncthreads();
  }
  int keep = sh.keep;
  float mp = min_p[r];
  __syncthreads();
  if (mp > 0.f) {
    float floor_p = p0 * mp;
    // the candidates are sorted, so those at or above the floor are a prefix
    if (threadIdx.x == 0) sh.chosen = keep;
    __syncthreads();
    for (int i = threadIdx.x; i < keep; i += blockDim.x) {
      float q = (sh.prob[i] - (i > 0 ? sh.prob[i - 1] : 0.f)) / total;
      if (!(q >= floor_p)) atomicMin(&sh.chosen, i);
    }
    __syncthreads();
    keep = max(1, sh.chosen);
    __syncthreads();
  }
  // temperature on the survivors, then the draw
  for (int i = threadIdx.x; i < keep; i += blockDim.x)
    sh.prob[i] = expf((key_to_float(~(unsigned int)(sh.cand[i] >> 32)) - max_logit) / T);
  __syncthreads();
  block_scan_float4(sh.prob, keep, sh.s_warpf);
  float norm = sh.prob[keep - 1];
  float u = uniform01(seeds[r], counters[r]) * norm;
  if (threadIdx.x == 0) sh.chosen = keep - 1;
  __syncthreads();
  for (int i = threadIdx.x; i < keep; i += blockDim.x) {
    float prev = i > 0 ? sh.prob[i - 1] : 0.f;
    if (sh.prob[i] >= u && (i == 0 || prev < u)) atomicMin(&sh.chosen, i);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = (int)(sh.cand[sh.chosen] & 0xffffffffull);
}

HK_API int hk_sample(const float* logits, int rows, int V, const float* temperature, const int* top_k,
                     const float* top_p, const float* min_p, const unsigned long long* seeds,
                     const unsigned long long* counters, int* out, void* stream) {
  if (rows <= 0) return 0;
  static HkSmemCache allowed = {};
  size_t smem = sizeof(SampleShared);
  if (int e = hk_allow_smem(sample_kernel, smem, allowed)) return e;
  sample_kernel<<<rows, SMP_THREADS, smem, (cudaStream_t)stream>>>(logits, V, temperature, top_k, top_p, min_p, seeds,
                                                                 counters, out);
  return hk_launch_status();
}
