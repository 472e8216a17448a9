"""Shared helpers of the tests: seeded inputs, the reference tests' LCG, byte comparisons."""
from __future__ import annotations

import numpy as np


def lcg_stream(seed: int, n: int) -> np.ndarray:
    """The reference tests' generator (aiis-clef src/cuda/mod.rs:6877-6881, 8144-8148):
    seed = seed*1664525 + 1013904223 (mod 2^32); value = (seed >> 9) / 2^23 - 1, in [-1, 1).
    Returns the n successive values as float32 (before the test's own scale factor).
    Vectorised: state_k = a^k * seed + c * (a^(k-1) + ... + 1), all products wrapping in uint32."""
    with np.errstate(over="ignore"):
        apow = np.cumprod(np.full(n, 1664525, np.uint32), dtype=np.uint32)           # a^1 .. a^n
        geo = np.cumsum(np.concatenate(([np.uint32(1)], apow[:-1])), dtype=np.uint32)  # 1 + a + .. + a^(k-1)
        states = apow * np.uint32(seed & 0xFFFFFFFF) + np.uint32(1013904223) * geo
    return ((states >> np.uint32(9)).astype(np.float32) / np.float32(1 << 23)) - np.float32(1.0)


def lcg_stream_loop(seed: int, n: int) -> np.ndarray:
    """Same sequence by the plain recurrence (used to check the vectorised form)."""
    s = seed & 0xFFFFFFFF
    vals = np.empty(n, np.uint32)
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        vals[i] = s
    return (vals >> 9).astype(np.float32) / np.float32(1 << 23) - np.float32(1.0)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round-to-nearest-even (finite inputs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16(rng, shape, scale=1.0, outlier_channels=0, outlier_gain=20.0):
    """N(0, scale) rounded to bf16 bits; optionally `outlier_channels` columns multiplied by a gain."""
    x = (rng.standard_normal(shape) * scale).astype(np.float32)
    if outlier_channels:
        cols = rng.choice(shape[-1], outlier_channels, replace=False)
        x[..., cols] *= outlier_gain
    return to_bf16_bits(x)


def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in bf16 ulps between two arrays of bf16 bit patterns (monotone integer mapping)."""
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, 0x8000 - b, b)
    return np.abs(key(a_bits) - key(b_bits))


def first_diff(a: np.ndarray, b: np.ndarray):
    a = np.asarray(a).reshape(-1)
    b = np.asarray(b).reshape(-1)
    assert a.size == b.size, f"sizes differ: {a.size} vs {b.size}"
    d = np.flatnonzero(a != b)
    return None if d.size == 0 else (int(d[0]), int(d.size))


def assert_bytes_equal(got, want, what: str):
    d = first_diff(got, want)
    if d is not None:
        i, n = d
        g = np.asarray(got).reshape(-1)[i]
        w = np.asarray(want).reshape(-1)[i]
        raise AssertionError(f"{what}: {n} of {np.asarray(got).size} bytes differ, first at {i}: got {g:#04x} want {w:#04x}")
