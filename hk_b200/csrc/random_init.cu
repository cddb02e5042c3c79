// Seeded random weights on the device: the counter-based stream of weights/random_stream.py, bit for bit.
//
// value_i = offset + float32(z_i) * scale, z_i = sqrt(-2 ln u1) * cos(angle) from the i-th splitmix64 output of
// the tensor's key (the definition, with the fixed operation sequences that stand in for ln and cos, is in
// weights/random_stream.py).  Every double operation below is an explicitly rounded intrinsic, so the compiler
// cannot contract a multiplication and an addition into one fused operation with another rounding.
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

__device__ __forceinline__ float stream_normal(unsigned long long key, unsigned long long i) {
  const unsigned long long r = mix64(key + (i + 1ull) * 0x9E3779B97F4A7C15ull);
  const long long a = (long long)(r >> 40);
  const long long b = (long long)((r >> 16) & 0xFFFFFFull);
  // ln u1, u1 = (2a + 1) / 2^25
  const long long n = 2 * a + 1;
  int e = 63 - __clzll(n);                                  // n = m * 2^e, m in [1, 2)
  double m = __longlong_as_double(((long long)(1023) << 52) | ((n << (52 - e)) & 0x000FFFFFFFFFFFFFll));
  if (m > 1.4142135623730951) {
    m = __dmul_rn(m, 0.5);
    e += 1;
  }
  const double t = __ddiv_rn(__dsub_rn(m, 1.0), __dadd_rn(m, 1.0));
  const double s = __dmul_rn(t, t);
  double p = 1.0 / 25.0;
#pragma unroll
  for (int k = 11; k >= 0; --k) p = __dadd_rn(__dmul_rn(p, s), 1.0 / (double)(2 * k + 1));
  const double ln_u = __dadd_rn(__dmul_rn((double)(e - 25), 0.6931471805599453), __dmul_rn(2.0, __dmul_rn(t, p)));
  const double radius = __dsqrt_rn(__dmul_rn(-2.0, ln_u));
  // cos(angle), angle = 2 pi b / 2^24
  const int quadrant = (int)(b >> 22);
  const double theta = __dmul_rn((double)(b & 0x3FFFFF), 1.5707963267948966 * 0x1p-22);
  const double th2 = __dmul_rn(theta, theta);
  double c = 1.0, g = 1.0;
#pragma unroll
  for (int k = 13; k >= 1; --k) {
    c = __dsub_rn(1.0, __dmul_rn(__dmul_rn(th2, 1.0 / (double)((2 * k - 1) * (2 * k))), c));
    g = __dsub_rn(1.0, __dmul_rn(__dmul_rn(th2, 1.0 / (double)((2 * k) * (2 * k + 1))), g));
  }
  g = __dmul_rn(theta, g);
  const double cosine = quadrant == 0 ? c : quadrant == 1 ? -g : quadrant == 2 ? -c : g;
  return __double2float_rn(__dmul_rn(radius, cosine));
}

template <typename T>
__global__ void random_init_kernel(T* out, long long count, unsigned long long key, float scale, float offset, int add_offset) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    float v = __fmul_rn(stream_normal(key, (unsigned long long)i), scale);
    if (add_offset) v = __fadd_rn(v, offset);
    out[i] = from_f32<T>(v);
  }
}

}  // namespace

// out[i] = (offset +) z_i * scale for i < count, in float32 arithmetic, stored as `dtype` (HK_F32 or HK_BF16).
HK_API int hk_random_init(void* out, int dtype, long long count, unsigned long long key, float scale, float offset,
                          int add_offset, void* stream) {
  if (count <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  long long blocks = (count + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == HK_F32)
    return hk_launch(random_init_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, s, (float*)out, count, key, scale, offset, add_offset);
  if (dtype == HK_BF16)
    return hk_launch(random_init_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, s, (bf16*)out, count, key, scale, offset, add_offset);
  return HK_ERR_UNSUPPORTED;
}
