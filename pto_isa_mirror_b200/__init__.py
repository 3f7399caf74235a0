"""B200 (sm_100a) implementation of the PTO tile library's GEMM hot path.

Host-side mirror of the reference's GEMM entry points over the C ABI in ``include/pto_b200.h``:
``gemm`` (TLOAD -> TMATMUL/TMATMUL_ACC -> TSTORE), ``gemm_s8_dequant`` (int8 + fixpipe dequant), ``gemm_quant``
(TSTORE with a pre-quant scale word / TSTORE_FP),
``gemm_mx`` (TMATMUL_MX, e8m0 block scales), ``gemv`` (TGEMV), ``gemv_mx`` (TGEMV_MX), ``mx_quantize_e4m3`` / ``mx_quantize_e2m1`` (TQUANT, MXFP8 / MXFP4),
``pto_gemm_basic`` (the torch op of demos/baseline/gemm_basic)
and the K-split GEMM + allreduce (``ksplit``). PyTorch is used for device memory, streams and
torch.distributed only; all arithmetic runs in the CUDA library.
"""
from . import _capi
from ._capi import B_DN, B_ND, BF16, E2M1, E4M3, E5M2, F16, F32, S8, S32, PtoB200Error
from .gemm import (
    cast_f32_to_bf16,
    device_status,
    gemm,
    gemm_mx,
    gemm_mx_pretiled,
    gemm_mx_workspace_bytes,
    gemm_quant,
    gemm_s8_dequant,
    gemv,
    gemv_mx,
    launch_count,
    mx_quantize_e2m1,
    mx_quantize_e4m3,
    mx_retile_scales,
    pto_gemm_basic,
)

__all__ = [
    "gemm", "gemm_s8_dequant", "gemm_quant", "gemm_mx", "gemm_mx_pretiled", "mx_retile_scales", "gemm_mx_workspace_bytes", "gemv", "gemv_mx", "mx_quantize_e4m3", "mx_quantize_e2m1", "cast_f32_to_bf16",
    "pto_gemm_basic",
    "device_status", "launch_count", "PtoB200Error",
    "F16", "BF16", "F32", "S8", "S32", "E4M3", "E5M2", "E2M1", "B_DN", "B_ND",
]
