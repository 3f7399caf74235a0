"""CPU checkers of the GEMM hot path. TEST INFRASTRUCTURE ONLY.

Two shared libraries sit behind this module:

* ``libpto_oracle.so``  - the plain-C restatement of the reference CPU simulator's arithmetic
  (``pto_gemm_oracle.c``), functions ``gemm_f32acc``, ``gemm_s8``, ``gemm_mx``, ``store_cast``,
  ``dequant_bf16``, ``mx_quantize_e4m3``;
* ``_ref/libpto_ref.so`` - the reference's own simulator compiled from its headers (``ref_shim.cpp``),
  exposed as :class:`Ref`; it exists wherever ``make -C oracle`` has run with the reference tree present.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the product
(``pto_isa_mirror_b200``) never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(HERE, "libpto_oracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libpto_ref.so")
REF_LIB_1T = os.path.join(HERE, "_ref", "libpto_ref_1t.so")

F16, BF16, F32 = 0, 1, 2
B_DN, B_ND = 0, 1
E4M3, E5M2, E2M1 = 5, 6, 7

_ll = ctypes.c_longlong
_i = ctypes.c_int
_p = ctypes.c_void_p


def build(ref_root: str | None = None) -> None:
    """Compile the C restatement and, when the reference tree is present, the reference shim."""
    cmd = ["make", "-C", HERE]
    if ref_root:
        cmd.append(f"REF={ref_root}")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + proc.stdout + proc.stderr)


_oracle = None


def _lib() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_LIB):
            build()
        lib = ctypes.CDLL(ORACLE_LIB)
        lib.pto_oracle_gemm_f32acc.argtypes = [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i]
        lib.pto_oracle_gemm_f32acc_bias.argtypes = [_p, _p, _p, _i, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i]
        lib.pto_oracle_gemm_s8.argtypes = [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i]
        lib.pto_oracle_gemm_s8_bias.argtypes = [_p, _p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i]
        lib.pto_oracle_gemm_mx_bias.argtypes = [_p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _i, _i,
                                                _i]
        lib.pto_oracle_gemm_mx.argtypes = [_p, _p, _p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _i, _i, _i]
        lib.pto_oracle_store_cast.argtypes = [_p, _p, _ll, _i]
        lib.pto_oracle_dequant_bf16.argtypes = [_p, _p, _p, _p, _i, _i, _ll, _ll, _i]
        lib.pto_oracle_mx_quantize_e4m3.argtypes = [_p, _p, _p, _i, _i, _ll]
        lib.pto_oracle_mx_quantize_e4m3_alg.argtypes = [_p, _p, _p, _i, _i, _ll, _i]
        lib.pto_oracle_mx_quantize_e2m1.argtypes = [_p, _p, _p, _i, _i, _ll, _i]
        lib.pto_oracle_quant_store.argtypes = [_p, _i, _p, _i, _i, _i, _p, _i, _i, _ll, _ll]
        lib.pto_oracle_float_to_bf16.argtypes = [ctypes.c_float]
        lib.pto_oracle_float_to_bf16.restype = ctypes.c_uint16
        lib.pto_oracle_float_to_half.argtypes = [ctypes.c_float]
        lib.pto_oracle_float_to_half.restype = ctypes.c_uint16
        lib.pto_oracle_half_to_float.argtypes = [ctypes.c_uint16]
        lib.pto_oracle_half_to_float.restype = ctypes.c_float
        lib.pto_oracle_fp8_to_double.argtypes = [ctypes.c_uint8, _i]
        lib.pto_oracle_fp8_to_double.restype = ctypes.c_double
        lib.pto_oracle_e8m0_to_double.argtypes = [ctypes.c_uint8]
        lib.pto_oracle_e8m0_to_double.restype = ctypes.c_double
        _oracle = lib
    return _oracle


def _c(a: np.ndarray, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype != np.dtype(dtype):
        raise TypeError(f"expected {np.dtype(dtype)}, got {a.dtype}")
    return a


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


# ----------------------------------------------------------------------------- restatement

def gemm_f32acc(a: np.ndarray, b: np.ndarray, in_dtype: int, b_layout: int = B_DN, threads: int = 0,
                bias: np.ndarray | None = None, bias_after_k: int = 0) -> np.ndarray:
    """Sequential-k fmaf GEMM. a [m, k]; b [n, k] (B_DN) or [k, n] (B_ND). F16/BF16 arrays are uint16 bit patterns.
    ``bias`` [n] float32 joins the chain after ``bias_after_k`` values of k (TMATMUL_BIAS on the first chunk;
    0 = after the whole K)."""
    store = np.float32 if in_dtype == F32 else np.uint16
    a = _c(a, store)
    b = _c(b, store)
    m, k = a.shape
    n = b.shape[0] if b_layout == B_DN else b.shape[1]
    assert (b.shape[1] if b_layout == B_DN else b.shape[0]) == k
    c = np.empty((m, n), dtype=np.float32)
    if bias is not None:
        bias = _c(bias, np.float32)
        assert bias.shape == (n,)
        _lib().pto_oracle_gemm_f32acc_bias(_ptr(a), _ptr(b), _ptr(bias), bias_after_k, _ptr(c), m, n, k, a.shape[1],
                                           b.shape[1], n, in_dtype, b_layout, threads)
        return c
    _lib().pto_oracle_gemm_f32acc(_ptr(a), _ptr(b), _ptr(c), m, n, k, a.shape[1], b.shape[1], n, in_dtype, b_layout,
                                  threads)
    return c


def gemm_s8(a: np.ndarray, b_dn: np.ndarray, threads: int = 0, bias: np.ndarray | None = None) -> np.ndarray:
    a = _c(a, np.int8)
    b_dn = _c(b_dn, np.int8)
    m, k = a.shape
    n = b_dn.shape[0]
    assert b_dn.shape[1] == k
    c = np.empty((m, n), dtype=np.int32)
    if bias is not None:
        bias = _c(bias, np.int32)
        assert bias.shape == (n,)
        _lib().pto_oracle_gemm_s8_bias(_ptr(a), _ptr(b_dn), _ptr(bias), _ptr(c), m, n, k, k, k, n, threads)
        return c
    _lib().pto_oracle_gemm_s8(_ptr(a), _ptr(b_dn), _ptr(c), m, n, k, k, k, n, threads)
    return c


def gemm_mx(a: np.ndarray, b_dn: np.ndarray, sfa: np.ndarray, sfb: np.ndarray, a_fmt: int = E4M3, b_fmt: int = E4M3,
            threads: int = 0, bias: np.ndarray | None = None, bias_after_k: int = 0) -> np.ndarray:
    a = _c(a, np.uint8)
    b_dn = _c(b_dn, np.uint8)
    sfa = _c(sfa, np.uint8)
    sfb = _c(sfb, np.uint8)
    m = a.shape[0]
    k = a.shape[1] * (2 if a_fmt == E2M1 else 1)          # E2M1: two elements per byte
    n = b_dn.shape[0]
    assert b_dn.shape[1] * (2 if b_fmt == E2M1 else 1) == k and sfa.shape == (m, k // 32) and sfb.shape == (n, k // 32)
    c = np.empty((m, n), dtype=np.float32)
    if bias is not None:
        bias = _c(bias, np.float32)
        assert bias.shape == (n,)
        _lib().pto_oracle_gemm_mx_bias(_ptr(a), _ptr(b_dn), _ptr(sfa), _ptr(sfb), _ptr(bias), bias_after_k, _ptr(c), m,
                                       n, k, k, k, n, k // 32, k // 32, a_fmt, b_fmt, threads)
        return c
    _lib().pto_oracle_gemm_mx(_ptr(a), _ptr(b_dn), _ptr(sfa), _ptr(sfb), _ptr(c), m, n, k, k, k, n, k // 32, k // 32,
                              a_fmt, b_fmt, threads)
    return c


def store_cast(src: np.ndarray, out_dtype: int) -> np.ndarray:
    """fp32 -> bf16 / f16 bit patterns (uint16), round to nearest even."""
    src = _c(src, np.float32)
    dst = np.empty(src.shape, dtype=np.uint16)
    _lib().pto_oracle_store_cast(_ptr(src), _ptr(dst), src.size, out_dtype)
    return dst


def dequant_bf16(acc: np.ndarray, s_row: np.ndarray, s_col: np.ndarray, truncate13: bool = True) -> np.ndarray:
    acc = _c(acc, np.int32)
    s_row = _c(s_row, np.float32)
    s_col = _c(s_col, np.float32)
    m, n = acc.shape
    out = np.empty((m, n), dtype=np.uint16)
    _lib().pto_oracle_dequant_bf16(_ptr(acc), _ptr(s_row), _ptr(s_col), _ptr(out), m, n, n, n, int(truncate13))
    return out


OUT_BF16, OUT_F16, OUT_S8, OUT_U8, OUT_S16 = 0, 1, 2, 3, 4


def quant_store(acc: np.ndarray, words, vector: bool, relu: bool = False, out_f16=False) -> np.ndarray:
    """TSTORE with a pre-quant scale: int32 or float32 accumulators [m, n] -> bf16 / f16 bit patterns (uint16), or with
    ``out_f16 = OUT_S8 / OUT_U8`` the 8-bit results in the low byte of each uint16. ``words``: one 64-bit scale word
    (scalar form) or n of them (vector form, one per column)."""
    acc = np.ascontiguousarray(acc)
    if acc.dtype not in (np.dtype(np.int32), np.dtype(np.float32)):
        raise TypeError("accumulators must be int32 or float32")
    words = np.ascontiguousarray(np.atleast_1d(np.asarray(words, dtype=np.uint64)))
    m, n = acc.shape
    assert words.shape == ((n,) if vector else (1,))
    out = np.empty((m, n), dtype=np.uint16)
    _lib().pto_oracle_quant_store(_ptr(acc), int(acc.dtype == np.int32), _ptr(words), int(vector), int(relu),
                                  int(out_f16), _ptr(out), m, n, n, n)
    return out


OCP, NV = 0, 1


def mx_quantize_e2m1(src: np.ndarray, scale_alg: int = OCP):
    """MX quantisation of fp32 [rows, k] to MXFP4 -> (packed e2m1 bytes [rows, k/2], element 2i in the low nibble;
    e8m0 bytes [rows, k/32]), with the OCP or the NV scale rule."""
    src = _c(src, np.float32)
    rows, k = src.shape
    assert k % 32 == 0
    data = np.empty((rows, k // 2), dtype=np.uint8)
    scales = np.empty((rows, k // 32), dtype=np.uint8)
    _lib().pto_oracle_mx_quantize_e2m1(_ptr(src), _ptr(data), _ptr(scales), rows, k, k, scale_alg)
    return data, scales


def mx_quantize_e4m3(src: np.ndarray, scale_alg: int = OCP):
    """MX quantisation of fp32 [rows, k] along k in blocks of 32 -> (e4m3 bytes [rows, k], e8m0 bytes [rows, k/32]),
    with the OCP or the NV scale rule."""
    src = _c(src, np.float32)
    rows, k = src.shape
    assert k % 32 == 0
    data = np.empty((rows, k), dtype=np.uint8)
    scales = np.empty((rows, k // 32), dtype=np.uint8)
    _lib().pto_oracle_mx_quantize_e4m3_alg(_ptr(src), _ptr(data), _ptr(scales), rows, k, k, scale_alg)
    return data, scales


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return store_cast(np.ascontiguousarray(x, dtype=np.float32), BF16)


# ----------------------------------------------------------------------------- the reference itself

class Ref:
    """The reference simulator (oracle/_ref). ``single_thread`` picks the PTO_CPU_MAX_THREADS=1 build."""

    TILE_M, TILE_N = 128, 256

    def __init__(self, single_thread: bool = False):
        path = REF_LIB_1T if single_thread else REF_LIB
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} not built (run `make -C oracle` where the reference tree is present)")
        lib = ctypes.CDLL(path)
        lib.ref_tile_f16.argtypes = [_p, _p, _p, _i]
        lib.ref_tile_f32.argtypes = [_p, _p, _p, _i]
        lib.ref_tile_s8.argtypes = [_p, _p, _p, _i]
        lib.ref_tile_mx.argtypes = [_p, _p, _p, _p, _p, _i, _i, _i]
        if hasattr(lib, "ref_tile_f16_bias"):  # absent from a shim built before the bias entry points existed
            lib.ref_tile_f16_bias.argtypes = [_p, _p, _p, _p, _i]
            lib.ref_tile_s8_bias.argtypes = [_p, _p, _p, _p, _i]
            lib.ref_tile_mx_bias.argtypes = [_p, _p, _p, _p, _p, _p, _i]
        lib.ref_dequant_col.argtypes = [ctypes.c_int32, ctypes.c_float]
        lib.ref_dequant_col.restype = ctypes.c_float
        lib.ref_cast_bf16.argtypes = [ctypes.c_float]
        lib.ref_cast_bf16.restype = ctypes.c_uint16
        lib.ref_cast_f16.argtypes = [ctypes.c_float]
        lib.ref_cast_f16.restype = ctypes.c_uint16
        if hasattr(lib, "ref_quant_store"):
            lib.ref_quant_store.argtypes = [_i, _i, _i, _i, ctypes.c_int32, ctypes.c_float, ctypes.c_uint64]
            lib.ref_quant_store.restype = ctypes.c_uint16
        lib.ref_mx_quantize_e4m3.argtypes = [_p, _p, _p, _i, _i]
        if hasattr(lib, "ref_mx_quantize_e2m1"):
            lib.ref_mx_quantize_e2m1.argtypes = [_p, _p, _p, _i, _i, _i]
        if hasattr(lib, "ref_mx_quantize_e4m3_nv"):
            lib.ref_mx_quantize_e4m3_nv.argtypes = [_p, _p, _p, _i, _i]
        lib.ref_fp8_to_double.argtypes = [ctypes.c_uint8, _i]
        lib.ref_fp8_to_double.restype = ctypes.c_double
        lib.ref_e8m0_to_double.argtypes = [ctypes.c_uint8]
        lib.ref_e8m0_to_double.restype = ctypes.c_double
        self.lib = lib

    @staticmethod
    def available(single_thread: bool = False) -> bool:
        return os.path.exists(REF_LIB_1T if single_thread else REF_LIB)

    def has_real_bf16(self) -> bool:
        return bool(self.lib.ref_has_real_bf16())

    def _tile(self, fn, a, b_dn, store, out_dtype):
        a = _c(a, store)
        b_dn = _c(b_dn, store)
        assert a.shape[0] == self.TILE_M and b_dn.shape[0] == self.TILE_N and a.shape[1] == b_dn.shape[1]
        out = np.empty((self.TILE_M, self.TILE_N), dtype=out_dtype)
        rc = fn(_ptr(out), _ptr(a), _ptr(b_dn), a.shape[1])
        if rc != 0:
            raise ValueError(f"K={a.shape[1]} is not instantiated in ref_shim.cpp")
        return out

    def tile_f16(self, a, b_dn):
        """RunGemmE2E<float, half, half, ...> on a [128, K] x [256, K] tile (K in 256, 1024, 6144)."""
        return self._tile(self.lib.ref_tile_f16, a, b_dn, np.uint16, np.float32)

    def tile_f32(self, a, b_dn):
        return self._tile(self.lib.ref_tile_f32, a, b_dn, np.float32, np.float32)

    def tile_s8(self, a, b_dn):
        return self._tile(self.lib.ref_tile_s8, a, b_dn, np.int8, np.int32)

    def tile_f16_bias(self, a, b_dn, bias):
        """TMATMUL_BIAS on the first 64-deep chunk, TMATMUL_ACC on the rest; fp16 bit patterns, fp32 bias [256]."""
        a, b_dn, bias = _c(a, np.uint16), _c(b_dn, np.uint16), _c(bias, np.float32)
        assert a.shape[0] == self.TILE_M and b_dn.shape == (self.TILE_N, a.shape[1]) and bias.shape == (self.TILE_N,)
        out = np.empty((self.TILE_M, self.TILE_N), dtype=np.float32)
        if self.lib.ref_tile_f16_bias(_ptr(out), _ptr(a), _ptr(b_dn), _ptr(bias), a.shape[1]) != 0:
            raise ValueError("K must be a positive multiple of 64")
        return out

    def tile_s8_bias(self, a, b_dn, bias):
        a, b_dn, bias = _c(a, np.int8), _c(b_dn, np.int8), _c(bias, np.int32)
        assert a.shape[0] == self.TILE_M and b_dn.shape == (self.TILE_N, a.shape[1]) and bias.shape == (self.TILE_N,)
        out = np.empty((self.TILE_M, self.TILE_N), dtype=np.int32)
        if self.lib.ref_tile_s8_bias(_ptr(out), _ptr(a), _ptr(b_dn), _ptr(bias), a.shape[1]) != 0:
            raise ValueError("K must be a positive multiple of 64")
        return out

    def tile_mx(self, a, b_dn, sfa, sfb, a_fmt=E4M3, b_fmt=E4M3):
        a = _c(a, np.uint8)
        b_dn = _c(b_dn, np.uint8)
        sfa = _c(sfa, np.uint8)
        sfb = _c(sfb, np.uint8)
        k = a.shape[1] * (2 if a_fmt == E2M1 else 1)
        assert a.shape[0] == self.TILE_M and b_dn.shape[0] == self.TILE_N
        assert sfa.shape == (self.TILE_M, k // 32) and sfb.shape == (self.TILE_N, k // 32)
        out = np.empty((self.TILE_M, self.TILE_N), dtype=np.float32)
        rc = self.lib.ref_tile_mx(_ptr(out), _ptr(a), _ptr(b_dn), _ptr(sfa), _ptr(sfb), k, a_fmt, b_fmt)
        if rc != 0:
            raise ValueError("unsupported K or format for ref_tile_mx")
        return out

    def tile_mx_bias(self, a, b_dn, sfa, sfb, bias):
        """e4m3 x e4m3 tile, six-operand TMATMUL_MX (fp32 bias [256]) on the first 128-deep chunk."""
        a, b_dn, sfa, sfb = _c(a, np.uint8), _c(b_dn, np.uint8), _c(sfa, np.uint8), _c(sfb, np.uint8)
        bias = _c(bias, np.float32)
        k = a.shape[1]
        assert a.shape[0] == self.TILE_M and b_dn.shape == (self.TILE_N, k) and bias.shape == (self.TILE_N,)
        out = np.empty((self.TILE_M, self.TILE_N), dtype=np.float32)
        if self.lib.ref_tile_mx_bias(_ptr(out), _ptr(a), _ptr(b_dn), _ptr(sfa), _ptr(sfb), _ptr(bias), k) != 0:
            raise ValueError("K must be a positive multiple of 128")
        return out

    def quant_store(self, acc, words, vector, relu=False, out_f16=False):
        """TSTORE with a pre-quant scale through the simulator's quantize_element, element by element."""
        acc = np.ascontiguousarray(acc)
        is_int = acc.dtype == np.int32
        words = np.atleast_1d(np.asarray(words, dtype=np.uint64))
        m, n = acc.shape
        out = np.empty((m, n), dtype=np.uint16)
        fn = self.lib.ref_quant_store
        for i in range(m):
            for j in range(n):
                w = int(words[j if vector else 0])
                v = acc[i, j]
                out[i, j] = fn(int(is_int), int(out_f16), int(vector), int(relu), int(v) if is_int else 0,
                               0.0 if is_int else float(v), w)
        return out

    def mx_quantize_e2m1(self, src, scale_alg=0):
        src = _c(src, np.float32)
        rows, k = src.shape
        data = np.empty((rows, k // 2), dtype=np.uint8)
        scales = np.empty((rows, k // 32), dtype=np.uint8)
        self.lib.ref_mx_quantize_e2m1(_ptr(src), _ptr(data), _ptr(scales), rows, k, int(scale_alg))
        return data, scales

    def mx_quantize_e4m3(self, src, scale_alg=0):
        src = _c(src, np.float32)
        rows, k = src.shape
        data = np.empty((rows, k), dtype=np.uint8)
        scales = np.empty((rows, k // 32), dtype=np.uint8)
        fn = self.lib.ref_mx_quantize_e4m3_nv if scale_alg else self.lib.ref_mx_quantize_e4m3
        fn(_ptr(src), _ptr(data), _ptr(scales), rows, k)
        return data, scales
