"""Comparison helpers shared by the GPU parity tests."""
import numpy as np


def max_rel_err(out, ref):
    """max |out - ref| / max |ref|: the tolerance the benchmark specification states (1e-3 dense, 1e-2 MXFP8)."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(out - ref).max() / max(np.abs(ref).max(), 1e-300))


def max_elem_rel_err(out, ref):
    """max element-wise relative error over the elements with |ref| >= rms(ref)."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = np.sqrt(np.mean(ref * ref))
    mask = np.abs(ref) >= rms
    if not mask.any():
        return 0.0
    return float((np.abs(out - ref)[mask] / np.abs(ref)[mask]).max())


def result_cmp(exp, act, eps):
    """The reference comparator (tests/common/test_common.h:231-309): an element fails iff |d| > eps and
    |d| / |exp| > eps; the case passes iff failures <= eps * N and at most 1000 outputs are zero where the
    golden is not."""
    exp = np.asarray(exp, dtype=np.float64).ravel()
    act = np.asarray(act, dtype=np.float64).ravel()
    d = np.abs(exp - act)
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.where(exp != 0, d / np.abs(exp), np.inf)
    fails = int(((d > eps) & (rel > eps)).sum()) + int((np.isnan(exp) != np.isnan(act)).sum())
    zeros = int(((act == 0) & (exp != 0)).sum())
    return fails <= eps * exp.size and zeros <= 1000


def bf16_ulp_distance(a_bits, b_bits):
    """Largest distance, in representable bf16 values, between two uint16 bit-pattern arrays."""
    def ordinal(u):
        u = np.asarray(u, dtype=np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return int(np.abs(ordinal(a_bits) - ordinal(b_bits)).max())
