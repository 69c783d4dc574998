"""Seeded normal values as a pure function of (seed, tensor name, element index).

The same arithmetic as ``csrc/random_weights.cu``, in NumPy: a splitmix64 finalizer of the index
feeds a Box-Muller transform whose logarithm, cosine and sine are written out in IEEE double
additions, multiplications, divisions and a square root, which round the same on every machine.
A model made on the device therefore equals, bit for bit, the model a host makes from the same
seed, whatever the order or the slabs in which the elements are produced.  (The reference's test
fixtures are a pure function of the index too: crates/engine/model/src/forward.rs:873-881.)
"""
from __future__ import annotations

import math

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_MASK = (1 << 64) - 1


def _mix_int(z: int) -> int:
    z &= _MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return z


def tensor_key(seed: int, name: str) -> int:
    """64-bit key of a tensor: FNV-1a of its name, mixed with the seed."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return _mix_int(h ^ _mix_int((int(seed) + 1) * 0x9E3779B97F4A7C15))


def _mix(z: np.ndarray) -> np.ndarray:
    z = z ^ (z >> np.uint64(30))
    z = z * _M1
    z = z ^ (z >> np.uint64(27))
    z = z * _M2
    return z ^ (z >> np.uint64(31))


_LN_COEF = [1.0 / k for k in (21.0, 19.0, 17.0, 15.0, 13.0, 11.0, 9.0, 7.0, 5.0, 3.0)] + [1.0]
_COS_COEF = [s / float(math.factorial(k)) for s, k in
             ((-1.0, 22), (1.0, 20), (-1.0, 18), (1.0, 16), (-1.0, 14), (1.0, 12), (-1.0, 10),
              (1.0, 8), (-1.0, 6), (1.0, 4), (-1.0, 2))] + [1.0]
_SIN_COEF = [s / float(math.factorial(k)) for s, k in
             ((-1.0, 23), (1.0, 21), (-1.0, 19), (1.0, 17), (-1.0, 15), (1.0, 13), (-1.0, 11),
              (1.0, 9), (-1.0, 7), (1.0, 5), (-1.0, 3))] + [1.0]


def _horner(coef, x2: np.ndarray) -> np.ndarray:
    p = np.full_like(x2, coef[0])
    for c in coef[1:]:
        p = p * x2 + c          # two roundings: NumPy does not fuse them
    return p


def standard_normal(key: int, first: int, n: int) -> np.ndarray:
    """float64 values z(key, first + i) for i < n."""
    with np.errstate(over="ignore"):
        idx = np.arange(first + 1, first + n + 1, dtype=np.uint64)
        h = _mix(np.uint64(key) + idx * _GOLDEN)
    hi = (h >> np.uint64(32)) + np.uint64(1)                    # 1 .. 2^32
    lo = h & np.uint64(0xFFFFFFFF)
    # ln(hi / 2^32): hi = m * 2^e, m in (1/sqrt 2, sqrt 2]
    m, e = np.frexp(hi.astype(np.float64))                      # m in [0.5, 1)
    m = m * 2.0
    e = e - 1
    big = m > 1.4142135623730951
    m = np.where(big, m * 0.5, m)
    e = np.where(big, e + 1, e)
    s = (m + -1.0) / (m + 1.0)
    p = _horner(_LN_COEF, s * s)
    ln_u = (e - 32).astype(np.float64) * 0.6931471805599453 + (2.0 * s) * p
    radius = np.sqrt(-2.0 * ln_u)
    # cos(2 pi lo / 2^32)
    quarter = (lo >> np.uint64(30)).astype(np.int64)
    x = ((lo & np.uint64(0x3FFFFFFF)).astype(np.float64) * 9.313225746154785e-10) \
        * 1.5707963267948966
    x2 = x * x
    c = _horner(_COS_COEF, x2)
    sn = _horner(_SIN_COEF, x2) * x
    r = np.where((quarter & 1) == 0, c, sn)
    r = np.where((quarter == 1) | (quarter == 2), -r, r)
    return radius * r


def normal_f32(key: int, first: int, n: int, mean: float, std: float) -> np.ndarray:
    """float32(mean + std * z): what a 32-bit tensor holds; a 16-bit tensor rounds it once more
    (to nearest, ties to even)."""
    return (mean + std * standard_normal(key, first, n)).astype(np.float32)
