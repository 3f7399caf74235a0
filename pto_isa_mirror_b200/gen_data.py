"""Seeded synthetic inputs for the GEMM hot path (the role of the reference kernels' scripts/gen_data.py).

The reference has no dataset: every kernel directory generates its inputs with a seeded numpy script
(kernels/manual/a2a3/gemm_performance/scripts/gen_data.py:17-46, kernels/manual/a5/matmul_mxfp8_performance/
scripts/gen_data.py:24-67). These generators are counter-based (splitmix64 of the element index), so any slice
of any matrix can be produced independently and identically on every machine.
"""
from __future__ import annotations

import numpy as np

_U64 = np.uint64


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + _U64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> _U64(30))) * _U64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> _U64(27))) * _U64(0x94D049BB133111EB)
        return z ^ (z >> _U64(31))


def _counters(count: int, seed: int, stream: int, offset: int = 0) -> np.ndarray:
    base = _splitmix64(np.array([seed * 1315423911 + stream * 2654435761 + 12345], dtype=_U64))[0]
    with np.errstate(over="ignore"):
        return np.arange(offset, offset + count, dtype=_U64) + base


def uniform01(count: int, seed: int, stream: int = 0, offset: int = 0) -> np.ndarray:
    """float64 uniform in [0, 1) with 53 random bits."""
    bits = _splitmix64(_counters(count, seed, stream, offset))
    return (bits >> _U64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def uniform(shape, lo: float, hi: float, seed: int, stream: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform01(n, seed, stream)).astype(np.float32).reshape(shape)


def normal(shape, seed: int, stream: int = 0) -> np.ndarray:
    """float32 N(0, 1) by Box-Muller on two counter streams."""
    n = int(np.prod(shape))
    u1 = 1.0 - uniform01(n, seed, 2 * stream + 100)  # (0, 1]
    u2 = uniform01(n, seed, 2 * stream + 101)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32).reshape(shape)


def randint(shape, lo: int, hi: int, seed: int, stream: int = 0) -> np.ndarray:
    """int64 uniform integers in [lo, hi] (inclusive)."""
    n = int(np.prod(shape))
    bits = _splitmix64(_counters(n, seed, stream))
    return (lo + (bits % _U64(hi - lo + 1)).astype(np.int64)).reshape(shape)


# ----------------------------------------------------------------------------- storage formats

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def clear_low13(x: np.ndarray) -> np.ndarray:
    """fp32 values with the low 13 mantissa bits cleared: the per-column dequant scales the reference's fixpipe
    actually applies (it reads a sign/8-bit exponent/10-bit mantissa float from bits [31:13] of the scale word,
    include/pto/cpu/common.hpp:116-137)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32)


def encode_e4m3fn(x: np.ndarray) -> np.ndarray:
    """Nearest e4m3fn code (ties to the even code, saturating at +-448, magnitudes rounding to zero give +0):
    the element encoding of the OCP MX quantiser, include/pto/cpu/TQuant.hpp:118-153."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    c = np.clip(x, -448.0, 448.0)
    ax = np.abs(c)
    sub = np.rint(ax * np.float32(512.0)).astype(np.uint32)
    fr, e = np.frexp(np.where(ax > 0, ax, np.float32(1.0)))
    q = np.rint((fr * np.float32(2.0) - np.float32(1.0)) * np.float32(8.0)).astype(np.int64)
    ee = e.astype(np.int64) - 1
    carry = q == 8
    q = np.where(carry, 0, q)
    ee = np.where(carry, ee + 1, ee)
    norm = np.minimum(((ee + 7) << 3) | q, 0x7E).astype(np.uint32)
    code = np.where(ax < np.float32(0.015625), sub, norm)
    sign = np.where((code != 0) & np.signbit(c), 0x80, 0).astype(np.uint32)
    out = (code | sign).astype(np.uint8)
    return np.where(np.isnan(x), np.uint8(0x7F), out)


def mx_quantize_e4m3(x: np.ndarray):
    """OCP MX quantisation along the last axis in blocks of 32 (include/pto/cpu/TQuant.hpp:178-190,226-237,461-494):
    e8m0 = max(biased_exp(absmax) - 8, 0); element = e4m3fn(x * 2^(127 - e8m0)).
    Returns (e4m3 bytes [rows, k], e8m0 bytes [rows, k // 32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    assert k % 32 == 0
    g = x.reshape(rows, k // 32, 32)
    amax = np.abs(g).max(axis=-1)
    exp = (amax.view(np.uint32) >> np.uint32(23)) & np.uint32(0xFF)
    e8m0 = np.where(exp <= 8, 0, exp.astype(np.int64) - 8).astype(np.uint8)
    scaling = ((np.uint32(254) - e8m0.astype(np.uint32)) << np.uint32(23)).view(np.float32)
    scaling = np.where(scaling == 0, np.float32(2.0 ** -127), scaling)
    y = g * scaling[..., None]
    return encode_e4m3fn(y).reshape(rows, k), e8m0


# ----------------------------------------------------------------------------- the benchmark configurations

def dense_inputs(m: int, n: int, k: int, dtype: str, seed: int, dist: str = "normal"):
    """A [m, k] and B stored column-major as [n, k] (the reference's is_btrans convention), as uint16 bit patterns.
    dist "uniform": uniform[-1, 1) (the CPU-demo style case); "normal": N(0, 1) / sqrt(k)."""
    if dist == "uniform":
        a = uniform((m, k), -1.0, 1.0, seed, 0)
        b = uniform((n, k), -1.0, 1.0, seed, 1)
    else:
        s = np.float32(1.0 / np.sqrt(k))
        a = normal((m, k), seed, 0) * s
        b = normal((n, k), seed, 1) * s
    conv = f32_to_bf16_bits if dtype == "bf16" else f32_to_f16_bits
    return conv(a), conv(b)


def s8_inputs(m: int, n: int, k: int, seed: int):
    """int8 A [m, k], B [n, k] uniform in [-127, 127]; s_row [m], s_col [n] fp32 uniform[1e-3, 1e-2], s_col with the
    low 13 mantissa bits cleared."""
    a = randint((m, k), -127, 127, seed, 0).astype(np.int8)
    b = randint((n, k), -127, 127, seed, 1).astype(np.int8)
    s_row = uniform((m,), 1e-3, 1e-2, seed, 2)
    s_col = clear_low13(uniform((n,), 1e-3, 1e-2, seed, 3))
    return a, b, s_row, s_col


def mx_inputs(m: int, n: int, k: int, seed: int):
    """MXFP8 A [m, k] / B [n, k] e4m3 bytes with e8m0 scales [m, k/32] / [n, k/32], quantised from N(0, 1)."""
    a, sfa = mx_quantize_e4m3(normal((m, k), seed, 0))
    b, sfb = mx_quantize_e4m3(normal((n, k), seed, 1))
    return a, b, sfa, sfb
