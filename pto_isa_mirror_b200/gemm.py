"""Host-side GEMM entry points over the C ABI, taking torch CUDA tensors as device buffers.

These mirror how the reference's upper layers call its GEMM: a torch op that checks dtype / shape /
contiguity and launches on the current stream (demos/baseline/gemm_basic/csrc/host/my_gemm_basic.cpp:22-48)
and ctypes launchers that pass raw device pointers (demos/torch_jit/gemm/jit_util_gemm.py:61-93).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _capi
from ._capi import B_DN, B_ND, BF16, E2M1, E4M3, E5M2, F16, F32, S8, S32

_TORCH_TO_PTO = {
    torch.float16: F16,
    torch.bfloat16: BF16,
    torch.float32: F32,
    torch.int8: S8,
    torch.int32: S32,
    torch.uint8: _capi.U8,
    torch.int16: _capi.S16,
}
_PTO_TO_TORCH = {v: k for k, v in _TORCH_TO_PTO.items()}
if hasattr(torch, "float8_e4m3fn"):
    _TORCH_TO_PTO[torch.float8_e4m3fn] = E4M3
    _TORCH_TO_PTO[torch.float8_e5m2] = E5M2


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def _require_cuda_2d(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D")
    if t.stride(1) != 1:
        raise ValueError(f"{name} must have unit stride in its last dimension")


_WORKSPACES = {}


def gemm_workspace(device: torch.device, stream_ptr: int) -> torch.Tensor:
    """The zero-initialised split-last-wave workspace of one (device, stream): launches on different streams may
    overlap on the GPU, so each stream gets its own."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(int(_capi.load().pto_b200_gemm_workspace_bytes()), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def gemm(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype = torch.float32, b_layout: int = B_DN,
         out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None,
         launch_block_count: int = 0, workspace=None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ B with fp32 (int32 for int8 inputs) accumulation over the whole K.

    ``bias``: n values of the accumulator type (float32, or int32 for int8 inputs) added per output column before the
    store cast (TMATMUL_BIAS); not combined with ``launch_block_count`` / ``workspace``.

    ``launch_block_count`` caps the thread blocks (SMs) the GEMM occupies, 0 = all of them: the knob the reference's
    launchGemmCompute has for leaving cores to the communication kernel that runs beside it.
    ``workspace``: None (default: tiles are never split), "auto" (a cached per-stream buffer that lets the last, partly
    filled wave of tiles be split along K) or a uint8 CUDA tensor of ``pto_b200_gemm_workspace_bytes()`` zeroed bytes.
    Measured on bf16 4096^3 the split does not pay yet (103.4 us with, 97.9 us without, same GPU): the two extra
    accumulator passes at the end of the kernel cost more than the half wave they save.

    a: [M, K] row-major (row stride >= K). b: [N, K] when ``b_layout == B_DN`` (column-major K x N, the
    layout of gemm_performance) or [K, N] when ``B_ND`` (the CPU demo's layout). Strided views are allowed,
    which is how a K-split rank passes its slice (A[:, k0:k1], B_dn[:, k0:k1]).
    """
    lib = _capi.load()
    _require_cuda_2d(a, "a")
    _require_cuda_2d(b, "b")
    if a.dtype != b.dtype or a.dtype not in (torch.float16, torch.bfloat16, torch.int8):
        raise ValueError("a and b must both be float16, bfloat16 or int8")
    m, k = a.shape
    if b_layout == B_DN:
        n, kb = b.shape
    else:
        kb, n = b.shape
    if kb != k:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    else:
        _require_cuda_2d(out, "out")
        if tuple(out.shape) != (m, n):
            raise ValueError("out has the wrong shape")
        out_dtype = out.dtype
    sp = _stream_ptr(stream)
    if bias is not None:
        if launch_block_count != 0 or workspace is not None:
            raise ValueError("bias cannot be combined with launch_block_count or workspace")
        want = torch.int32 if a.dtype == torch.int8 else torch.float32
        if bias.dtype != want or not bias.is_cuda or bias.numel() != n or not bias.is_contiguous():
            raise ValueError(f"bias must be a contiguous CUDA {want} tensor with {n} elements")
        rc = lib.pto_b200_gemm_bias(sp, out.data_ptr(), a.data_ptr(), b.data_ptr(), bias.data_ptr(), m, n, k,
                                    a.stride(0), b.stride(0), out.stride(0), _TORCH_TO_PTO[a.dtype],
                                    _TORCH_TO_PTO[out_dtype], b_layout)
        _capi.check(rc, "pto_b200_gemm_bias")
        return out
    if isinstance(workspace, str):
        workspace = gemm_workspace(a.device, sp)
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel()) if workspace is not None else (None, 0)
    rc = lib.pto_b200_gemm_ws(sp, out.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0), b.stride(0),
                              out.stride(0), _TORCH_TO_PTO[a.dtype], _TORCH_TO_PTO[out_dtype], b_layout,
                              launch_block_count, ws_ptr, ws_bytes)
    _capi.check(rc, "pto_b200_gemm_ws")
    return out


def gemm_s8_dequant(a: torch.Tensor, b_dn: torch.Tensor, s_row: torch.Tensor, s_col: torch.Tensor,
                    out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """bf16((float(int32 acc) * s_col[j]) * s_row[i]) for int8 a [M, K] and b_dn [N, K]."""
    lib = _capi.load()
    _require_cuda_2d(a, "a")
    _require_cuda_2d(b_dn, "b_dn")
    if a.dtype != torch.int8 or b_dn.dtype != torch.int8:
        raise ValueError("a and b_dn must be int8")
    m, k = a.shape
    n, kb = b_dn.shape
    if kb != k:
        raise ValueError("inner dimensions differ")
    for s, cnt, name in ((s_row, m, "s_row"), (s_col, n, "s_col")):
        if s.dtype != torch.float32 or not s.is_cuda or s.numel() != cnt or not s.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA float32 tensor with {cnt} elements")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    rc = lib.pto_b200_gemm_s8_dequant(_stream_ptr(stream), out.data_ptr(), a.data_ptr(), b_dn.data_ptr(),
                                      s_row.data_ptr(), s_col.data_ptr(), m, n, k, a.stride(0), b_dn.stride(0),
                                      out.stride(0))
    _capi.check(rc, "pto_b200_gemm_s8_dequant")
    return out


def gemm_quant(a: torch.Tensor, b_dn: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
               pre_quant_scalar: int = 0, fp_words: Optional[torch.Tensor] = None, relu: bool = False,
               out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """GEMM with the pre-quant store: TSTORE(dst, acc, preQuantScalar) when ``fp_words`` is None (the scale is the
    float32 value in the low 32 bits of ``pre_quant_scalar``), TSTORE(dst, acc, fpTile) / TSTORE_FP when ``fp_words`` is a
    CUDA tensor of n 64-bit words (int64 / uint64), one per column, whose bits [31:13] hold the scale. a, b_dn: int8
    (int32 accumulators) or float16 / bfloat16 (float32 accumulators); the result is bfloat16 or float16, or - the
    REQ8 / QF322B8_PRE forms - int8 / uint8: round(acc * scale + offset) with the word's offset (bits [45:37]) and sign
    flag (bit 46: clamp to -128..127, else to 0..255); or int16 for int8 inputs - the SHIFTS322S16 form:
    int16(acc >> (1 + bits [35:32] of the word))."""
    lib = _capi.load()
    _require_cuda_2d(a, "a")
    _require_cuda_2d(b_dn, "b_dn")
    if a.dtype != b_dn.dtype or a.dtype not in (torch.float16, torch.bfloat16, torch.int8):
        raise ValueError("a and b_dn must both be float16, bfloat16 or int8")
    m, k = a.shape
    n, kb = b_dn.shape
    if kb != k:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    elif tuple(out.shape) != (m, n) or out.dtype not in (torch.bfloat16, torch.float16, torch.int8, torch.uint8,
                                                         torch.int16):
        raise ValueError("out must be [m, n] bfloat16, float16, int8, uint8 or int16")
    words_ptr = None
    if fp_words is not None:
        if not fp_words.is_cuda or fp_words.element_size() != 8 or fp_words.numel() != n or not fp_words.is_contiguous():
            raise ValueError(f"fp_words must be a contiguous CUDA tensor of {n} 64-bit words")
        words_ptr = fp_words.data_ptr()
    rc = lib.pto_b200_gemm_quant(_stream_ptr(stream), out.data_ptr(), a.data_ptr(), b_dn.data_ptr(), m, n, k,
                                 a.stride(0), b_dn.stride(0), out.stride(0), _TORCH_TO_PTO[a.dtype],
                                 _TORCH_TO_PTO[out.dtype], int(pre_quant_scalar) & 0xFFFFFFFFFFFFFFFF, words_ptr,
                                 int(bool(relu)))
    _capi.check(rc, "pto_b200_gemm_quant")
    return out


def gemm_mx_workspace_bytes(m: int, n: int, k: int, split_last_wave: bool = False) -> int:
    """Bytes of the re-tiled scales; with ``split_last_wave`` also the room (``pto_b200_gemm_workspace_bytes``) that
    lets the CTA-pair kernel cut a partly filled last wave of tiles into K halves. A workspace of the larger size must
    not be shared by calls that can overlap."""
    lib = _capi.load()
    extra = int(lib.pto_b200_gemm_workspace_bytes()) if split_last_wave else 0
    return int(lib.pto_b200_gemm_mx_workspace_bytes(m, n, k)) + extra


def gemm_mx(a: torch.Tensor, b_dn: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor,
            out_dtype: torch.dtype = torch.bfloat16, a_fmt: int = E4M3, b_fmt: int = E4M3,
            workspace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            stream: Optional[torch.cuda.Stream] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """MX block-scaled GEMM (TMATMUL_MX): a [M, K] and b_dn [N, K] fp8 bytes (uint8 or torch fp8 dtypes), or with
    ``a_fmt = b_fmt = E2M1`` (MXFP4) [M, K/2] and [N, K/2] bytes holding two 4-bit values each, the even element low;
    sfa [M, K/32] and sfb [N, K/32] e8m0 bytes (uint8). ``workspace`` is a uint8 CUDA tensor of at least
    ``gemm_mx_workspace_bytes(m, n, k)`` bytes; one is allocated through torch when omitted. ``bias``: n float32
    values added per column to the finished accumulator (the six-operand TMATMUL_MX)."""
    lib = _capi.load()
    for t, name in ((a, "a"), (b_dn, "b_dn"), (sfa, "sfa"), (sfb, "sfb")):
        _require_cuda_2d(t, name)
        if t.element_size() != 1:
            raise ValueError(f"{name} must have one-byte elements")
    # MXFP4 (a_fmt = b_fmt = E2M1): two elements per byte, so the byte tensors are [M, K/2] and [N, K/2]
    per_byte = 2 if a_fmt == E2M1 else 1
    m, k = a.shape[0], a.shape[1] * per_byte
    n, kb = b_dn.shape[0], b_dn.shape[1] * (2 if b_fmt == E2M1 else 1)
    if kb != k:
        raise ValueError("inner dimensions differ")
    if k % 32 != 0 or tuple(sfa.shape) != (m, k // 32) or tuple(sfb.shape) != (n, k // 32):
        raise ValueError("scales must be [M, K/32] and [N, K/32] with K a multiple of 32")
    if workspace is None:
        workspace = torch.zeros(gemm_mx_workspace_bytes(m, n, k, split_last_wave=True), dtype=torch.uint8, device=a.device)
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if bias is not None:
        if bias.dtype != torch.float32 or not bias.is_cuda or bias.numel() != n or not bias.is_contiguous():
            raise ValueError(f"bias must be a contiguous CUDA float32 tensor with {n} elements")
        rc = lib.pto_b200_gemm_mx_bias(_stream_ptr(stream), out.data_ptr(), a.data_ptr(), b_dn.data_ptr(),
                                       sfa.data_ptr(), sfb.data_ptr(), bias.data_ptr(), workspace.data_ptr(),
                                       workspace.numel(), m, n, k, a.stride(0) * per_byte, b_dn.stride(0) * per_byte,
                                       out.stride(0), sfa.stride(0), sfb.stride(0), a_fmt, b_fmt, _TORCH_TO_PTO[out.dtype])
        _capi.check(rc, "pto_b200_gemm_mx_bias")
        return out
    rc = lib.pto_b200_gemm_mx(_stream_ptr(stream), out.data_ptr(), a.data_ptr(), b_dn.data_ptr(), sfa.data_ptr(),
                              sfb.data_ptr(), workspace.data_ptr(), workspace.numel(), m, n, k, a.stride(0) * per_byte,
                              b_dn.stride(0) * per_byte, out.stride(0), sfa.stride(0), sfb.stride(0), a_fmt, b_fmt,
                              _TORCH_TO_PTO[out.dtype])
    _capi.check(rc, "pto_b200_gemm_mx")
    return out


def mx_retile_scales(sfa: torch.Tensor, sfb: torch.Tensor, k: int, workspace: Optional[torch.Tensor] = None,
                     stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Re-tile the e8m0 scales sfa [M, K/32] and sfb [N, K/32] into the layout the block-scaled kernels read
    (``pto_b200_mx_retile_scales``) and return the workspace, for use with :func:`gemm_mx_pretiled`."""
    lib = _capi.load()
    for t, name in ((sfa, "sfa"), (sfb, "sfb")):
        _require_cuda_2d(t, name)
        if t.element_size() != 1 or t.shape[1] != k // 32:
            raise ValueError(f"{name} must be [rows, K/32] bytes")
    m, n = sfa.shape[0], sfb.shape[0]
    if workspace is None:
        workspace = torch.zeros(gemm_mx_workspace_bytes(m, n, k, split_last_wave=True), dtype=torch.uint8,
                                device=sfa.device)
    rc = lib.pto_b200_mx_retile_scales(_stream_ptr(stream), workspace.data_ptr(), workspace.numel(), sfa.data_ptr(),
                                       sfb.data_ptr(), m, n, k, sfa.stride(0), sfb.stride(0))
    _capi.check(rc, "pto_b200_mx_retile_scales")
    return workspace


def gemm_mx_pretiled(a: torch.Tensor, b_dn: torch.Tensor, tiled_scales: torch.Tensor,
                     out_dtype: torch.dtype = torch.bfloat16, a_fmt: int = E4M3, b_fmt: int = E4M3,
                     out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """:func:`gemm_mx` with scales that :func:`mx_retile_scales` already re-tiled for the same m, n, k: one kernel launch."""
    lib = _capi.load()
    _require_cuda_2d(a, "a")
    _require_cuda_2d(b_dn, "b_dn")
    m, k = a.shape
    n = b_dn.shape[0]
    if b_dn.shape[1] != k or a.element_size() != 1 or b_dn.element_size() != 1:
        raise ValueError("a [M, K] and b_dn [N, K] must be fp8 bytes with the same K")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    rc = lib.pto_b200_gemm_mx_pretiled(_stream_ptr(stream), out.data_ptr(), a.data_ptr(), b_dn.data_ptr(),
                                       tiled_scales.data_ptr(), tiled_scales.numel(), m, n, k, a.stride(0),
                                       b_dn.stride(0), out.stride(0), a_fmt, b_fmt, _TORCH_TO_PTO[out.dtype])
    _capi.check(rc, "pto_b200_gemm_mx_pretiled")
    return out


def gemv(x: torch.Tensor, b_dn: torch.Tensor, out_dtype: torch.dtype = torch.float32,
         bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """TGEMV: out[j] = sum_k x[k] * b_dn[j, k] (+ bias[j]) for one left row x [K] (or [1, K]) and column-major
    b_dn [N, K]. float16 / bfloat16 inputs give float32 / bfloat16 / float16; int8 inputs give int32. Returns [N]."""
    lib = _capi.load()
    _require_cuda_2d(b_dn, "b_dn")
    if not x.is_cuda or x.dtype != b_dn.dtype or x.numel() != b_dn.shape[1] or not x.is_contiguous():
        raise ValueError("x must be a contiguous CUDA tensor of b_dn's dtype with K elements")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.int8):
        raise ValueError("inputs must be float16, bfloat16 or int8")
    n, k = b_dn.shape
    if x.dtype == torch.int8:
        out_dtype = torch.int32
    if out is None:
        out = torch.empty((n,), dtype=out_dtype, device=x.device)
    elif out.numel() != n or not out.is_contiguous() or not out.is_cuda:
        raise ValueError("out must be a contiguous CUDA tensor with N elements")
    bias_ptr = None
    if bias is not None:
        want = torch.int32 if x.dtype == torch.int8 else torch.float32
        if bias.dtype != want or not bias.is_cuda or bias.numel() != n or not bias.is_contiguous():
            raise ValueError(f"bias must be a contiguous CUDA {want} tensor with {n} elements")
        bias_ptr = bias.data_ptr()
    rc = lib.pto_b200_gemv(_stream_ptr(stream), out.data_ptr(), x.data_ptr(), b_dn.data_ptr(), bias_ptr, n, k,
                           b_dn.stride(0), _TORCH_TO_PTO[x.dtype], _TORCH_TO_PTO[out.dtype])
    _capi.check(rc, "pto_b200_gemv")
    return out


def gemv_mx(x: torch.Tensor, b_dn: torch.Tensor, sfx: torch.Tensor, sfb: torch.Tensor,
            out_dtype: torch.dtype = torch.float32, a_fmt: int = E4M3, b_fmt: int = E4M3,
            bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """TGEMV_MX: out[j] = sum_k x[k] * b_dn[j, k] * 2^(sfx[k/32]-127) * 2^(sfb[j, k/32]-127) (+ bias[j]) for one left
    row x [K] of fp8 bytes with its K/32 e8m0 scales sfx, and column-major b_dn [N, K] with scales sfb [N, K/32]."""
    lib = _capi.load()
    _require_cuda_2d(b_dn, "b_dn")
    _require_cuda_2d(sfb, "sfb")
    n, k = b_dn.shape
    if (not x.is_cuda or x.element_size() != 1 or b_dn.element_size() != 1 or x.numel() != k or not x.is_contiguous()
            or k % 32):
        raise ValueError("x must be K contiguous fp8 bytes, b_dn [N, K] fp8 bytes, K a multiple of 32")
    if sfx.numel() != k // 32 or not sfx.is_contiguous() or tuple(sfb.shape) != (n, k // 32):
        raise ValueError("scales must be [K/32] and [N, K/32] bytes")
    if out is None:
        out = torch.empty((n,), dtype=out_dtype, device=x.device)
    bias_ptr = None
    if bias is not None:
        if bias.dtype != torch.float32 or not bias.is_cuda or bias.numel() != n or not bias.is_contiguous():
            raise ValueError(f"bias must be a contiguous CUDA float32 tensor with {n} elements")
        bias_ptr = bias.data_ptr()
    rc = lib.pto_b200_gemv_mx(_stream_ptr(stream), out.data_ptr(), x.data_ptr(), b_dn.data_ptr(), sfx.data_ptr(),
                              sfb.data_ptr(), bias_ptr, n, k, b_dn.stride(0), sfb.stride(0), a_fmt, b_fmt,
                              _TORCH_TO_PTO[out.dtype])
    _capi.check(rc, "pto_b200_gemv_mx")
    return out


def mx_quantize_e4m3(src: torch.Tensor, stream: Optional[torch.cuda.Stream] = None,
                     data: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None,
                     scale_alg: int = _capi.SCALE_OCP):
    """OCP MX quantisation (TQUANT, MXFP8): float32 src [rows, K] -> (e4m3 bytes [rows, K] uint8, e8m0 scales
    [rows, K/32] uint8), one scale per 32 elements along K. Finite input only. ``data`` / ``scales``: caller's output
    buffers of those shapes (allocated when omitted). ``scale_alg``: ``_capi.SCALE_OCP`` (default) or ``_capi.SCALE_NV``,
    the reference's QuantScaleAlg."""
    lib = _capi.load()
    _require_cuda_2d(src, "src")
    if src.dtype != torch.float32:
        raise ValueError("src must be float32")
    rows, k = src.shape
    if k % 32 != 0:
        raise ValueError("K must be a multiple of 32")
    if data is None:
        data = torch.empty((rows, k), dtype=torch.uint8, device=src.device)
    if scales is None:
        scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=src.device)
    for t, shape, name in ((data, (rows, k), "data"), (scales, (rows, k // 32), "scales")):
        _require_cuda_2d(t, name)
        if t.dtype != torch.uint8 or tuple(t.shape) != shape:
            raise ValueError(f"{name} must be a uint8 CUDA tensor of shape {shape}")
    rc = lib.pto_b200_mx_quantize_e4m3_ex(_stream_ptr(stream), data.data_ptr(), scales.data_ptr(), src.data_ptr(), rows,
                                          k, src.stride(0), data.stride(0), scales.stride(0), scale_alg)
    _capi.check(rc, "pto_b200_mx_quantize_e4m3_ex")
    return data, scales


def mx_quantize_e2m1(src: torch.Tensor, stream: Optional[torch.cuda.Stream] = None,
                     data: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None,
                     scale_alg: int = _capi.SCALE_OCP):
    """MX quantisation to MXFP4 (TQUANT, MXFP4_E2M1): float32 src [rows, K] -> (packed e2m1 bytes [rows, K/2] uint8 with
    element 2i in the low nibble of byte i, e8m0 scales [rows, K/32] uint8): the operands ``gemm_mx`` takes with
    ``a_fmt = b_fmt = E2M1``. Finite input only; ``scale_alg`` as for :func:`mx_quantize_e4m3`."""
    lib = _capi.load()
    _require_cuda_2d(src, "src")
    if src.dtype != torch.float32:
        raise ValueError("src must be float32")
    rows, k = src.shape
    if k % 32 != 0:
        raise ValueError("K must be a multiple of 32")
    if data is None:
        data = torch.empty((rows, k // 2), dtype=torch.uint8, device=src.device)
    if scales is None:
        scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=src.device)
    for t, shape, name in ((data, (rows, k // 2), "data"), (scales, (rows, k // 32), "scales")):
        _require_cuda_2d(t, name)
        if t.dtype != torch.uint8 or tuple(t.shape) != shape:
            raise ValueError(f"{name} must be a uint8 CUDA tensor of shape {shape}")
    rc = lib.pto_b200_mx_quantize_e2m1(_stream_ptr(stream), data.data_ptr(), scales.data_ptr(), src.data_ptr(), rows, k,
                                       src.stride(0), data.stride(0), scales.stride(0), scale_alg)
    _capi.check(rc, "pto_b200_mx_quantize_e2m1")
    return data, scales


def cast_f32_to_bf16(src: torch.Tensor, out: Optional[torch.Tensor] = None,
                     stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    lib = _capi.load()
    if src.dtype != torch.float32 or not src.is_cuda or not src.is_contiguous():
        raise ValueError("src must be a contiguous CUDA float32 tensor")
    if out is None:
        out = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    rc = lib.pto_b200_cast_f32_to_bf16(_stream_ptr(stream), out.data_ptr(), src.data_ptr(), src.numel())
    _capi.check(rc, "pto_b200_cast_f32_to_bf16")
    return out


def pto_gemm_basic(a: torch.Tensor, b_dn: torch.Tensor) -> torch.Tensor:
    """The torch op of demos/baseline/gemm_basic: fp16 a [M, K] x fp16 b_dn [N, K] (= b.t().contiguous())
    -> fp32 [M, N], same argument checks, any shape instead of the reference's fixed 512 x 2048 x 1536."""
    if a.dtype != torch.float16 or b_dn.dtype != torch.float16:
        raise ValueError("a and b_dn must be float16")
    if a.dim() != 2 or b_dn.dim() != 2:
        raise ValueError("a and b_dn must be 2D tensors")
    if not a.is_contiguous() or not b_dn.is_contiguous():
        raise ValueError("a and b_dn must be contiguous")
    return gemm(a, b_dn, torch.float32, B_DN)


def device_status() -> int:
    """Synchronise and return the kernels' status word (0 = no bounded wait gave up)."""
    st = ctypes.c_int(0)
    rc = _capi.load().pto_b200_device_status(ctypes.byref(st))
    if rc not in (_capi.OK, _capi.ETIMEOUT):
        _capi.check(rc, "pto_b200_device_status")
    return st.value


def launch_count() -> int:
    return int(_capi.load().pto_b200_launch_count())
