"""Seeded synthetic inputs shared by the tests, the smoke check and the bench.

A counter-based generator (SplitMix64 over the element index) so that any slice of any tensor can be
regenerated anywhere — CPU oracle and GPU read the same arrays.  Normals come from Box-Muller on two
uniform draws, uniforms use the top 24 bits of a draw.  All values are produced in f32; callers round
to f16 (round-to-nearest-even) with `.astype(np.float16)`.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    """SplitMix64 finaliser applied element-wise to a uint64 array of counters."""
    with np.errstate(over="ignore"):
        z = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _draws(seed, count, lane):
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed], dtype=np.uint64) * np.uint64(2) + np.uint64(lane))[0]
        idx = np.arange(count, dtype=np.uint64)
        return _splitmix64(idx * np.uint64(0x9E3779B97F4A7C15) + base)


def uniform01(seed, shape):
    """U[0,1) with 24 bits of mantissa, f32."""
    n = int(np.prod(shape)) if len(shape) else 1
    u = (_draws(seed, n, 0) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / (1 << 24))
    return u.reshape(shape)


def uniform(seed, shape, lo, hi):
    return (np.float32(lo) + uniform01(seed, shape) * np.float32(hi - lo)).astype(np.float32)


def normal(seed, shape, std=1.0):
    """N(0, std^2), f32, Box-Muller."""
    n = int(np.prod(shape)) if len(shape) else 1
    u1 = ((_draws(seed, n, 0) >> np.uint64(40)).astype(np.float64) + 1.0) * (1.0 / (1 << 24))  # (0, 1]
    u2 = (_draws(seed, n, 1) >> np.uint64(40)).astype(np.float64) * (1.0 / (1 << 24))
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).astype(np.float32).reshape(shape)
