// Row-wise kernels of the decoder: embedding gather, RMS norm, the fused per-head
// norm + rotation + paged cache write, and SwiGLU.  Each is templated on the storage
// type (float for the true 32-bit path, bf16 for serving); all arithmetic is fp32.
//
// Reference counterparts (one launch each there, none fused): `rms_norm`
// src/cuda_device.zig:1393-1403, `head_norm` :1406-1415, `rope` :1420-1441,
// `kv_write` :1453-1477, `swiglu` :1824-1829; host-side embedding
// src/cuda/engine.zig:724-737.  The fusion of norm + rotation + cache write follows
// the idea of shaders/rope_kv.comp:2-7.
#include "common.cuh"

// ----------------------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] widened to fp32 (the residual stream is fp32).
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int n, int d, int vocab) {
  int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // the host validates ids; this only keeps the read in bounds
  const T* src = table + (size_t)id * d;
  float* dst = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

// The same with 16-byte loads (8 bf16 or 4 floats per thread and step), all issued before any is used.
template <typename T, int PER>
__global__ void embedding_vec_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                     int d, int vocab) {
  constexpr int E = 16 / sizeof(T);   // elements per 16-byte load
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * d);
  float* dst = out + (size_t)t * d;
  const int chunks = d / E;
  uint4 v[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) v[k] = src[c];
  }
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    int c = threadIdx.x + k * blockDim.x;
    if (c >= chunks) continue;
    const T* e = reinterpret_cast<const T*>(&v[k]);
    float f[E];
#pragma unroll
    for (int i = 0; i < E; ++i) f[i] = to_f32<T>(e[i]);
#pragma unroll
    for (int i = 0; i < E; i += 4) *reinterpret_cast<float4*>(dst + c * E + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
  }
}

HK_API int hk_embedding(const void* table, int table_dtype, const int* ids, float* out, int n, int d,
                        int vocab, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  {
    const int e = table_dtype == HK_F32 ? 4 : 8;
    if (d % e == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0 && d / e <= 4 * 256) {
      if (table_dtype == HK_F32)
        return hk_launch(embedding_vec_kernel<float, 4>, dim3(n), dim3(256), 0, s, (const float*)table, ids, out, d, vocab);
      else if (table_dtype == HK_BF16)
        return hk_launch(embedding_vec_kernel<bf16, 4>, dim3(n), dim3(256), 0, s, (const bf16*)table, ids, out, d, vocab);
      else
        return HK_ERR_UNSUPPORTED;
      return hk_launch_status();
    }
  }
  int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == HK_F32)
    embedding_kernel<float><<<n, threads, 0, s>>>((const float*)table, ids, out, n, d, vocab);
  else if (table_dtype == HK_BF16)
    embedding_kernel<bf16><<<n, threads, 0, s>>>((const bf16*)table, ids, out, n, d, vocab);
  else
    return HK_ERR_UNSUPPORTED;
  return hk_launch_status();
}

// ----------------------------------------------------------------------------- rms norm
// out[r, :] = x[row(r), :] * rsqrt(mean(x^2) + eps) * w, with row(r) = rows ? rows[r] : r.
// The sum of squares runs in a fixed order (thread-strided partials, warp tree, then
// warps in order), so a row's result does not depend on what else is in the batch.
template <typename TO>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                const int* __restrict__ rows, TO* __restrict__ out, int d, float eps) {
  __shared__ float warp_part[32];
  __shared__ float inv_s;
  int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = src[i];
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) warp_part[wid] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += warp_part[i];
    inv_s = 1.0f / sqrtf(tot / (float)d + eps);
  }
  __syncthreads();
  float inv = inv_s;
  TO* dst = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<TO>(src[i] * inv * w[i]);
}

// The same for widths that are a multiple of 4 and at most 4 * PER * 256: the row is read once with 16-byte
// loads that are all in flight together, and stays in registers between the two passes.  The order of the
// sum depends on the width alone.
template <typename TO, int PER>
__global__ void __launch_bounds__(256)
rms_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                    TO* __restrict__ out, int d, float eps) {
  __shared__ float warp_part[8];
  __shared__ float inv_s;
  const int r = blockIdx.x;
  const float4* wv = reinterpret_cast<const float4*>(w);
  const int chunks = d >> 2;
  float4 v[PER], g[PER];
  pdl_launch_dependents();
#pragma unroll
  for (int k = 0; k < PER; ++k) {     // the norm's weight does not depend on the kernel before
    const int c = threadIdx.x + k * 256;
    if (c < chunks) g[k] = wv[c];
  }
  pdl_wait();
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    v[k] = c < chunks ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    ss = fmaf(v[k].x, v[k].x, ss);
    ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss);
    ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = warp_sum(ss);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += warp_part[i];
    inv_s = 1.0f / sqrtf(tot / (float)d + eps);
  }
  __syncthreads();
  const float inv = inv_s;
  TO* dst = out + (size_t)r * d;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c >= chunks) continue;
    const float a0 = v[k].x * inv * g[k].x, a1 = v[k].y * inv * g[k].y, a2 = v[k].z * inv * g[k].z, a3 = v[k].w * inv * g[k].w;
    if (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + 4 * c) = make_float4(a0, a1, a2, a3);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1), hi = __floats2bfloat162_rn(a2, a3);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + 4 * c) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

template <int PER>
static int rms_norm_vec(const float* x, const float* w, const int* rows, void* out, int out_dtype, int n_out, int d, float eps,
                        cudaStream_t s) {
  if (out_dtype == HK_F32)
    return hk_launch_pdl(rms_norm_vec_kernel<float, PER>, dim3(n_out), dim3(256), 0, s, x, w, rows, (float*)out, d, eps);
  if (out_dtype == HK_BF16)
    return hk_launch_pdl(rms_norm_vec_kernel<bf16, PER>, dim3(n_out), dim3(256), 0, s, x, w, rows, (bf16*)out, d, eps);
  return HK_ERR_UNSUPPORTED;
}

HK_API int hk_rms_norm(const float* x, const float* w, const int* rows, void* out, int out_dtype,
                       int n_out, int d, float eps, void* stream) {
  if (n_out <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if ((d & 3) == 0 && d >= 1024 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
    const int chunks = d >> 2;
    if (chunks <= 2 * 256) return rms_norm_vec<2>(x, w, rows, out, out_dtype, n_out, d, eps, s);
    if (chunks <= 4 * 256) return rms_norm_vec<4>(x, w, rows, out, out_dtype, n_out, d, eps, s);
    if (chunks <= 8 * 256) return rms_norm_vec<8>(x, w, rows, out, out_dtype, n_out, d, eps, s);
  }
  int threads = d >= 2048 ? 256 : 128;
  if (out_dtype == HK_F32)
    rms_norm_kernel<float><<<n_out, threads, 0, s>>>(x, w, rows, (float*)out, d, eps);
  else if (out_dtype == HK_BF16)
    rms_norm_kernel<bf16><<<n_out, threads, 0, s>>>(x, w, rows, (bf16*)out, d, eps);
  else
    return HK_ERR_UNSUPPORTED;
  return hk_launch_status();
}

// ------------------------------------------------- per-head norm + rotation + cache write
// One warp per (token, head) of the fused projection output qkv[n, (H + 2G) * hd] (fp32):
//   q heads: optional RMS norm over hd (weight shared by the heads), rotate-half rotation of
//            the first `rot` dims by the token's position, stored to q_out[n, H*hd];
//   k heads: the same with the key norm weight, stored into the token's cache page;
//   v heads: stored into the cache page unchanged.
// `bias` (or null) [(H + 2G) * hd] is added to the projection output first.  `pairing` 0 rotates dims
// (i, i + rot/2) ("rotate-half"), 1 rotates dims (2i, 2i + 1) ("adjacent"); both read angle i of the tables.
// Page of a token: block_table[slot_of_token[t]][pos / page_tokens]; the cache layout is
// [page][G][page_tokens][hd].  With write_kv == 0 only q is produced (a layer that reads
// another layer's cache).
#define QKR_MAX_HD 256
#define QKR_WARPS 4

template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(
    const float* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int rot, const int* __restrict__ positions,
    const int* __restrict__ slot_of_token, const int* __restrict__ block_table, int table_stride,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int n, int H, int G, int hd, int page_tokens,
    int write_kv, const float* __restrict__ bias, int pairing) {
  __shared__ float buf[QKR_WARPS][QKR_MAX_HD];
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int heads_total = H + (write_kv ? 2 * G : 0);
  long long item = (long long)blockIdx.x * QKR_WARPS + wid;
  if (item >= (long long)n * heads_total) return;
  int t = (int)(item / heads_total);
  int hh = (int)(item % heads_total);
  const float* src = qkv + (size_t)t * (H + 2 * G) * hd + (size_t)hh * hd;
  float* v = buf[wid];
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    float a = src[i];
    if (bias) a += bias[(size_t)hh * hd + i];
    v[i] = a;
    ss = fmaf(a, a, ss);
  }
  __syncwarp();
  int kind = hh < H ? 0 : (hh < H + G ? 1 : 2);  // q, k, v
  int pos = positions[t];
  if (kind != 2) {
    const float* w = kind == 0 ? q_w : k_w;
    if (w) {
      ss = warp_sum(ss);
      float inv = 1.0f / sqrtf(ss / (float)hd + eps);
      for (int i = lane; i < hd; i += 32) v[i] = v[i] * inv * w[i];
      __syncwarp();
    }
    if (rot > 0) {
      int half = rot >> 1;
      const float* c = cos_t + (size_t)pos * half;
      const float* s = sin_t + (size_t)pos * half;
      for (int i = lane; i < half; i += 32) {
        const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
        float a = v[ia], b = v[ib];
        float ci = c[i], si = s[i];
        v[ia] = a * ci - b * si;
        v[ib] = a * si + b * ci;
      }
      __syncwarp();
    }
  }
  T* dst;
  if (kind == 0) {
    dst = q_out + (size_t)t * H * hd + (size_t)hh * hd;
  } else {
    int g = kind == 1 ? hh - H : hh - H - G;
    int page = block_table[(size_t)slot_of_token[t] * table_stride + pos / page_tokens];
    if (page < 0) return;  // the host never schedules this; keeps a stale table from writing out of bounds
    T* base = kind == 1 ? k_pages : v_pages;
    dst = base + (((size_t)page * G + g) * page_tokens + (pos % page_tokens)) * hd;
  }
  for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(v[i]);
}

// The same for head sizes up to 128 that are a multiple of 4 (and a rotary width that is a multiple of 8):
// a lane holds 4 consecutive dims, read with one 16-byte load; the rotation partner (dim + rot/2) sits
// (rot/8) lanes away and comes by shuffle, so nothing goes through shared memory.
#define QKV_WARPS 8
template <typename T>
__global__ void __launch_bounds__(QKV_WARPS * 32)
qk_norm_rope_kv_write_vec_kernel(
    const float* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int rot, const int* __restrict__ positions,
    const int* __restrict__ slot_of_token, const int* __restrict__ block_table, int table_stride,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int n, int H, int G, int hd, int page_tokens,
    int write_kv, const float* __restrict__ bias, int pairing) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int heads_total = H + (write_kv ? 2 * G : 0);
  const long long item = (long long)blockIdx.x * QKV_WARPS + wid;
  if (item >= (long long)n * heads_total) return;
  const int t = (int)(item / heads_total);
  const int hh = (int)(item % heads_total);
  const int d0 = lane * 4;
  const bool active = d0 < hd;
  const float* src = qkv + (size_t)t * (H + 2 * G) * hd + (size_t)hh * hd;
  float4 v = active ? *reinterpret_cast<const float4*>(src + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
  if (bias && active) {
    const float4 b = *reinterpret_cast<const float4*>(bias + (size_t)hh * hd + d0);
    v = make_float4(v.x + b.x, v.y + b.y, v.z + b.z, v.w + b.w);
  }
  const int kind = hh < H ? 0 : (hh < H + G ? 1 : 2);
  const int pos = positions[t];
  if (kind != 2) {
    const float* w = kind == 0 ? q_w : k_w;
    if (w) {
      float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
      if (active) {
        const float4 g = *reinterpret_cast<const float4*>(w + d0);
        v = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
      }
    }
    if (rot > 0 && pairing) {
      // adjacent pairs: a lane's four dims are the pairs d0/2 and d0/2 + 1, both its own
      if (d0 < rot) {
        const int half = rot >> 1;
        const float2 c = *reinterpret_cast<const float2*>(cos_t + (size_t)pos * half + (d0 >> 1));
        const float2 sn = *reinterpret_cast<const float2*>(sin_t + (size_t)pos * half + (d0 >> 1));
        v = make_float4(v.x * c.x - v.y * sn.x, v.x * sn.x + v.y * c.x, v.z * c.y - v.w * sn.y, v.z * sn.y + v.w * c.y);
      }
    } else if (rot > 0) {
      const int half = rot >> 1, shift = half >> 2;        // partner lanes are `shift` apart
      const bool low = d0 < half, in_rot = d0 < rot;
      const int partner = low ? lane + shift : lane - shift;
      const int src_lane = in_rot ? partner : lane;
      float4 p;
      p.x = __shfl_sync(0xffffffffu, v.x, src_lane);
      p.y = __shfl_sync(0xffffffffu, v.y, src_lane);
      p.z = __shfl_sync(0xffffffffu, v.z, src_lane);
      p.w = __shfl_sync(0xffffffffu, v.w, src_lane);
      if (in_rot) {
        const int i0 = low ? d0 : d0 - half;                // index into the tables
        const float4 c = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i0);
        const float4 sn = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i0);
        // low half: x' = a c - b s (a = own, b = partner); high half: x' = a s + b c (a = partner, b = own)
        if (low)
          v = make_float4(v.x * c.x - p.x * sn.x, v.y * c.y - p.y * sn.y, v.z * c.z - p.z * sn.z, v.w * c.w - p.w * sn.w);
        else
          v = make_float4(p.x * sn.x + v.x * c.x, p.y * sn.y + v.y * c.y, p.z * sn.z + v.z * c.z, p.w * sn.w + v.w * c.w);
      }
    }
  }
  if (!active) return;
  T* dst;
  if (kind == 0) {
    dst = q_out + (size_t)t * H * hd + (size_t)hh * hd;
  } else {
    const int g = kind == 1 ? hh - H : hh - H - G;
    const int page = block_table[(size_t)slot_of_token[t] * table_stride + pos / page_tokens];
    if (page < 0) return;
    T* base = kind == 1 ? k_pages : v_pages;
    dst = base + (((size_t)page * G + g) * page_tokens + (pos % page_tokens)) * hd;
  }
  if (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + d0) = v;
  } else {
    __nv_bfloat162 lo2 = __floats2bfloat162_rn(v.x, v.y), hi2 = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + d0) =
        make_uint2(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2));
  }
}

HK_API int hk_qk_norm_rope_kv_write(const float* qkv, void* q_out, int dtype, const float* q_w,
                                    const float* k_w, float eps, const float* cos_t, const float* sin_t,
                                    int rot, const int* positions, const int* slot_of_token,
                                    const int* block_table, int table_stride, void* k_pages,
                                    void* v_pages, int n, int H, int G, int hd, int page_tokens,
                                    int write_kv, const float* bias, int pairing, void* stream) {
  if (n <= 0) return 0;
  if (hd > QKR_MAX_HD || hd < 2 || rot > hd || (rot & 1) || pairing < 0 || pairing > 1) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  long long items = (long long)n * (H + (write_kv ? 2 * G : 0));
  const bool aligned = ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)q_w |
                          (uintptr_t)k_w | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)bias) & 15) == 0);
  if (hd <= 128 && (hd & 3) == 0 && (rot & 7) == 0 && aligned) {
    unsigned vblocks = (unsigned)((items + QKV_WARPS - 1) / QKV_WARPS);
    if (dtype == HK_F32)
      return hk_launch_pdl(qk_norm_rope_kv_write_vec_kernel<float>, dim3(vblocks), dim3(QKV_WARPS * 32), 0, s, qkv, (float*)q_out,
                       q_w, k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (float*)k_pages,
                       (float*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing);
    if (dtype == HK_BF16)
      return hk_launch_pdl(qk_norm_rope_kv_write_vec_kernel<bf16>, dim3(vblocks), dim3(QKV_WARPS * 32), 0, s, qkv, (bf16*)q_out, q_w,
                       k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (bf16*)k_pages,
                       (bf16*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing);
    return HK_ERR_UNSUPPORTED;
  }
  unsigned blocks = (unsigned)((items + QKR_WARPS - 1) / QKR_WARPS);
  if (dtype == HK_F32)
    return hk_launch(qk_norm_rope_kv_write_kernel<float>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s, qkv, (float*)q_out, q_w,
                         k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (float*)k_pages,
                         (float*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing);
  if (dtype == HK_BF16)
    return hk_launch(qk_norm_rope_kv_write_kernel<bf16>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s, qkv, (bf16*)q_out, q_w,
                         k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (bf16*)k_pages,
                         (bf16*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- bias
// out[t, j] += bias[j] for a projection with a bias whose product kernel has no such epilogue.
__global__ void add_bias_kernel(float* __restrict__ out, const float* __restrict__ bias, long long total, int N) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] += bias[i % N];
}

HK_API int hk_add_bias(float* out, const float* bias, int n, int N, void* stream) {
  if (n <= 0 || N <= 0) return 0;
  long long total = (long long)n * N;
  return hk_launch(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, out, bias, total, N);
}

// ----------------------------------------------------------------------------- swiglu
// out[t, j] = silu(gate_j) * up_j for the fused projection gu[n, 2F], laid out in blocks of
// `block` gates followed by the matching `block` ups (block == F: all gates, then all ups).
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ out, long long total, int F, int block) {
  pdl_launch_dependents();
  pdl_wait();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  long long t = i / F;
  int j = (int)(i % F);
  long long gi = t * 2 * F + (long long)(j / block) * 2 * block + (j % block);
  float g = gu[gi];
  float u = gu[gi + block];
  out[i] = from_f32<TO>(g / (1.0f + expf(-g)) * u);
}

HK_API int hk_swiglu(const float* gu, void* out, int out_dtype, int n, int F, int block, void* stream) {
  if (n <= 0) return 0;
  if (block <= 0 || F % block) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  long long total = (long long)n * F;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == HK_F32) return hk_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, s, gu, (float*)out, total, F, block);
  if (out_dtype == HK_BF16) return hk_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, s, gu, (bf16*)out, total, F, block);
  return HK_ERR_UNSUPPORTED;
}
