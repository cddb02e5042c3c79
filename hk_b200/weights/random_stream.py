"""The random stream of seeded random weights: counter-based, the same bits on every route.

A tensor's values depend only on (seed, tensor name, element index): neither on the device that
draws them, nor on the order of tensors, nor on which other tensors exist.  The reference seeds
its fixtures the same way, in one place (tests/support/tiny_model.zig:231,340).  Definition, all
integers unsigned 64-bit with wrap-around:

  key   = first 8 bytes, little-endian, of sha256("<seed>:<name>")
  r_i   = mix(key + (i + 1) * 0x9E3779B97F4A7C15)                  (the splitmix64 sequence from `key`)
          mix(x): x ^= x >> 30; x *= 0xBF58476D1CE4E5B9; x ^= x >> 27; x *= 0x94D049BB133111EB; x ^= x >> 31
  u1    = (2 * (r_i >> 40) + 1) / 2^25        24 bits, never 0 or 1
  angle = 2 pi * ((r_i >> 16) & 0xFFFFFF) / 2^24
  z_i   = sqrt(-2 ln u1) * cos(angle)         Box-Muller, one normal per element
  value = float32(z_i) * float32(std)         or 1 + float32(z_i) * float32(norm_std), in float32

ln and cos are not taken from a math library (their last bits differ between a GPU and a CPU): they
are fixed sequences of IEEE double additions, multiplications, one division and one square root, each
rounded once (no fused multiply-add), so that this file (numpy) and `csrc/random_init.cu` (CUDA) give
identical bits:

  ln u1:  n = 2a + 1 = m * 2^e with m in [1, 2); if m > SQRT2: m /= 2, e += 1
          t = (m - 1) / (m + 1); s = t * t; p = 1/25; for k = 11 .. 0: p = p * s + 1/(2k + 1)
          ln u1 = (e - 25) * LN2 + 2 * (t * p)
  cos:    b = 24 bits; quadrant = b >> 22; theta = (b & 0x3FFFFF) * (pi/2 * 2^-22) in [0, pi/2)
          c = 1; for k = 13 .. 1: c = 1 - (theta^2 * (1 / ((2k - 1) * 2k))) * c           (cos theta)
          g = 1; for k = 13 .. 1: g = 1 - (theta^2 * (1 / (2k * (2k + 1)))) * g; g = theta * g   (sin theta)
          cos(angle) = c, -g, -c, g for quadrant 0, 1, 2, 3
"""
from __future__ import annotations

import hashlib

import numpy as np

GOLDEN = np.uint64(0x9E3779B97F4A7C15)
M1 = np.uint64(0xBF58476D1CE4E5B9)
M2 = np.uint64(0x94D049BB133111EB)
LN2 = 0.6931471805599453
SQRT2 = 1.4142135623730951
HALF_PI_STEP = 1.5707963267948966 * 2.0 ** -22
LN_TERMS = 12
TRIG_TERMS = 13


def tensor_key(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _bits(key: int, start: int, count: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = np.uint64(key) + (np.arange(start + 1, start + count + 1, dtype=np.uint64) * GOLDEN)
        x ^= x >> np.uint64(30)
        x *= M1
        x ^= x >> np.uint64(27)
        x *= M2
        x ^= x >> np.uint64(31)
    return x


def standard_normal(key: int, start: int, count: int) -> np.ndarray:
    """Elements start .. start+count-1 of the stream `key`, as float32 standard normals."""
    r = _bits(key, start, count)
    a = (r >> np.uint64(40)).astype(np.int64)
    b = ((r >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.int64)
    # ln u1
    n = 2 * a + 1
    m, e = np.frexp(n.astype(np.float64))          # n = m * 2^e, m in [0.5, 1)
    m = m * 2.0
    e = e - 1
    big = m > SQRT2
    m = np.where(big, m * 0.5, m)
    e = np.where(big, e + 1, e)
    t = (m - 1.0) / (m + 1.0)
    s = t * t
    p = np.full(count, 1.0 / (2 * LN_TERMS + 1))
    for k in range(LN_TERMS - 1, -1, -1):
        p = p * s + 1.0 / (2 * k + 1)
    ln_u = (e - 25).astype(np.float64) * LN2 + 2.0 * (t * p)
    radius = np.sqrt(-2.0 * ln_u)
    # cos(angle)
    quadrant = b >> 22
    theta = (b & 0x3FFFFF).astype(np.float64) * HALF_PI_STEP
    th2 = theta * theta
    c = np.ones(count)
    g = np.ones(count)
    for k in range(TRIG_TERMS, 0, -1):
        c = 1.0 - (th2 * (1.0 / ((2 * k - 1) * (2 * k)))) * c
        g = 1.0 - (th2 * (1.0 / ((2 * k) * (2 * k + 1)))) * g
    g = theta * g
    cosine = np.choose(quadrant, [c, -g, -c, g])
    return (radius * cosine).astype(np.float32)


def fill(key: int, count: int, scale: float, offset: float, chunk: int = 1 << 20) -> np.ndarray:
    """float32 [count]: offset + z_i * scale in float32 arithmetic (offset 0: plain scaling)."""
    out = np.empty(count, dtype=np.float32)
    sc, off = np.float32(scale), np.float32(offset)
    for s0 in range(0, count, chunk):
        c = min(chunk, count - s0)
        z = standard_normal(key, s0, c) * sc
        out[s0:s0 + c] = z + off if offset != 0.0 else z
    return out
