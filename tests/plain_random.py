"""The random-weight stream restated element by element in plain Python (integers and floats only),
independent of the package's numpy version and of the CUDA kernel.  Definition: per-tensor key =
first 8 bytes (little-endian) of sha256("<seed>:<name>"); element i takes the i-th output of the
splitmix64 sequence started at the key; 24 of its bits give u1, 24 more the angle of a Box-Muller
draw; ln and cos are fixed sequences of singly rounded double operations (a Python float operation
is exactly that).  The reference seeds its fixtures per model in one place
(tests/support/tiny_model.zig:231,340); the stream itself is this engine's."""
import hashlib
import math
import struct

MASK = (1 << 64) - 1


def key_of(seed, name):
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def mix(x):
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & MASK
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & MASK
    x ^= x >> 31
    return x


def to_f32(x):
    return struct.unpack("<f", struct.pack("<f", x))[0]


def normal(key, i):
    r = mix((key + (i + 1) * 0x9E3779B97F4A7C15) & MASK)
    a, b = r >> 40, (r >> 16) & 0xFFFFFF
    n = 2 * a + 1
    e = n.bit_length() - 1
    m = n / (1 << e)                     # exact: a division by a power of two
    if m > 1.4142135623730951:
        m, e = m * 0.5, e + 1
    t = (m - 1.0) / (m + 1.0)
    s = t * t
    p = 1.0 / 25
    for k in range(11, -1, -1):
        p = p * s + 1.0 / (2 * k + 1)
    ln_u = (e - 25) * 0.6931471805599453 + 2.0 * (t * p)
    radius = math.sqrt(-2.0 * ln_u)
    quadrant = b >> 22
    theta = (b & 0x3FFFFF) * (1.5707963267948966 * 2.0 ** -22)
    th2 = theta * theta
    c = g = 1.0
    for k in range(13, 0, -1):
        c = 1.0 - (th2 * (1.0 / ((2 * k - 1) * (2 * k)))) * c
        g = 1.0 - (th2 * (1.0 / ((2 * k) * (2 * k + 1)))) * g
    g = theta * g
    cosine = (c, -g, -c, g)[quadrant]
    return to_f32(radius * cosine)


def value(seed, name, i, scale, offset=None):
    """Element i of tensor `name`: float32(z) * float32(scale) (+ float32(offset)), each rounded to float32."""
    v = to_f32(normal(key_of(seed, name), i) * to_f32(scale))     # the product of two float32 is exact in double
    if offset is not None:
        v = to_f32(v + to_f32(offset))
    return v
