"""Plain statement of the seeded random weights: one value at a time, in Python integers and
floats (IEEE doubles, no fused operations), sharing no code with the package.

A weight is a function of (seed, tensor name, element index):

    key   = mix(fnv1a64(name) ^ mix((seed + 1) * GOLDEN))
    h     = mix(key + (index + 1) * GOLDEN)                      (mix: the splitmix64 finalizer)
    u1    = ((h >> 32) + 1) / 2^32,  turn = (h & 0xffffffff) / 2^32
    z     = sqrt(-2 ln u1) * cos(2 pi turn)                      (Box-Muller)
    value = float32(mean + std * z), rounded once more to bfloat16 for a 16-bit tensor

with ln, cos and sin as the fixed polynomials below, so that every machine rounds the same.  The
reference makes its test fixtures from an integer hash of the index in the same spirit
(crates/engine/model/src/forward.rs:873-881); matrices ~ N(0, 0.02) and gains 1 + N(0, 0.01) are
what the benchmark configurations name.
"""
from __future__ import annotations

import math
import struct

MASK = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def mix(z: int) -> int:
    z &= MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK
    z ^= z >> 31
    return z


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & MASK
    return h


def key_of(seed: int, name: str) -> int:
    return mix(fnv1a64(name) ^ mix((seed + 1) * GOLDEN))


def ln_unit(n: int) -> float:
    """ln(n / 2^32) for 1 <= n <= 2^32."""
    e = n.bit_length() - 1
    m = float(n) / float(1 << e)          # exact: division by a power of two
    if m > 1.4142135623730951:
        m = m * 0.5
        e += 1
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    p = 1.0 / 21.0
    for k in (19.0, 17.0, 15.0, 13.0, 11.0, 9.0, 7.0, 5.0, 3.0, 1.0):
        p = p * s2
        p = p + 1.0 / k
    return float(e - 32) * 0.6931471805599453 + (2.0 * s) * p


def cos_turn(k: int) -> float:
    """cos(2 pi k / 2^32) for a 32-bit k."""
    quarter = k >> 30
    x = (float(k & 0x3FFFFFFF) * 2.0 ** -30) * 1.5707963267948966
    x2 = x * x
    if quarter % 2 == 0:
        p = -1.0 / float(math.factorial(22))
        for sign, k2 in ((1.0, 20), (-1.0, 18), (1.0, 16), (-1.0, 14), (1.0, 12), (-1.0, 10),
                         (1.0, 8), (-1.0, 6), (1.0, 4), (-1.0, 2), (1.0, 0)):
            p = p * x2
            p = p + sign / float(math.factorial(k2))
        r = p
    else:
        p = -1.0 / float(math.factorial(23))
        for sign, k2 in ((1.0, 21), (-1.0, 19), (1.0, 17), (-1.0, 15), (1.0, 13), (-1.0, 11),
                         (1.0, 9), (-1.0, 7), (1.0, 5), (-1.0, 3), (1.0, 1)):
            p = p * x2
            p = p + sign / float(math.factorial(k2))
        r = p * x
    return -r if quarter in (1, 2) else r


def standard_normal(key: int, index: int) -> float:
    h = mix(key + (index + 1) * GOLDEN)
    radius = math.sqrt(-2.0 * ln_unit((h >> 32) + 1))     # math.sqrt is correctly rounded
    return radius * cos_turn(h & 0xFFFFFFFF)


def to_f32(v: float) -> float:
    return struct.unpack("<f", struct.pack("<f", v))[0]


def to_bf16(v: float) -> float:
    """Round a float32 value to bfloat16, to nearest, ties to even."""
    bits = struct.unpack("<I", struct.pack("<f", v))[0]
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def weight(seed: int, name: str, index: int, one_dimensional: bool, bf16: bool) -> float:
    """The value of element ``index`` (row-major) of tensor ``name``."""
    mean, std = (1.0, 0.01) if one_dimensional else (0.0, 0.02)
    v = to_f32(mean + std * standard_normal(key_of(seed, name), index))
    return to_bf16(v) if bf16 else v
