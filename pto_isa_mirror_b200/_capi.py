"""ctypes binding of ``include/pto_b200.h`` (the C ABI of the sm_100a GEMM tile loop).

The shared library is built in-tree by :mod:`pto_isa_mirror_b200.build` into ``lib/libpto_b200.so``.
There is no fallback: if the library is missing, loading raises with the build command to run.
"""
from __future__ import annotations

import ctypes
import os

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
LIB_PATH = os.path.join(_LIB_DIR, "libpto_b200.so")

# pto_b200_dtype
F16, BF16, F32, S8, S32, E4M3, E5M2, E2M1, U8, S16 = range(10)
# pto_b200_b_layout
B_DN, B_ND = 0, 1
# return codes
OK, EINVAL, EALIGN, EDTYPE, EWORKSPACE, ECUDA, EDEVICE, ETIMEOUT, ESCRATCH = range(9)
MX_STATIC_SCRATCH_BYTES = 8 * 1024 * 1024
# pto_b200_scale_alg
SCALE_OCP, SCALE_NV = 0, 1

# every symbol include/pto_b200.h declares: name -> (restype, argtypes)
_u8p = ctypes.c_void_p
_ll = ctypes.c_longlong
_i = ctypes.c_int
SYMBOLS = {
    "pto_b200_gemm": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i]),
    "pto_b200_gemm_ex": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i]),
    "pto_b200_gemm_workspace_bytes": (ctypes.c_size_t, []),
    "pto_b200_gemm_ws": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _u8p, ctypes.c_size_t],
    ),
    "pto_b200_gemm_bias": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i],
    ),
    "pto_b200_gemm_quant": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _ll, _i, _i, ctypes.c_ulonglong, ctypes.c_void_p, _i],
    ),
    "pto_b200_gemm_s8_dequant": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, ctypes.c_void_p, ctypes.c_void_p, _i, _i, _i, _ll, _ll, _ll],
    ),
    "pto_b200_gemm_mx": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, _u8p, _u8p, ctypes.c_size_t, _i, _i, _i, _ll, _ll, _ll, _ll, _ll,
         _i, _i, _i],
    ),
    "pto_b200_gemm_mx_bias": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, _u8p, _u8p, _u8p, ctypes.c_size_t, _i, _i, _i, _ll, _ll, _ll, _ll,
         _ll, _i, _i, _i],
    ),
    "pto_b200_gemm_mx_workspace_bytes": (ctypes.c_size_t, [_i, _i, _i]),
    "pto_b200_mx_retile_scales": (_i, [ctypes.c_void_p, _u8p, ctypes.c_size_t, _u8p, _u8p, _i, _i, _i, _ll, _ll]),
    "pto_b200_gemm_mx_pretiled": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, ctypes.c_size_t, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i],
    ),
    "pto_b200_gemv": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, _i, _i, _ll, _i, _i]),
    "pto_b200_gemv_mx": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, _u8p, _u8p, _i, _i, _ll, _ll, _i, _i, _i]),
    "pto_b200_mx_quantize_e4m3": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _ll, _ll, _ll]),
    "pto_b200_mx_quantize_e4m3_ex": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _ll, _ll, _ll, _i]),
    "pto_b200_mx_quantize_e2m1": (_i, [ctypes.c_void_p, _u8p, _u8p, _u8p, _i, _i, _ll, _ll, _ll, _i]),
    "pto_b200_gemm_mx_static": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _u8p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _i, _i, _i],
    ),
    "pto_b200_cast_f32_to_bf16": (_i, [ctypes.c_void_p, _u8p, _u8p, _ll]),
    "pto_b200_ksplit_signal": (_i, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), _i, _i, _i, _i]),
    "pto_b200_ksplit_reduce": (
        _i,
        [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
         ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p, _i, _i, _i, _i, _ll, _i, _i, _ll, _ll, _i,
         ctypes.c_void_p, ctypes.c_void_p],
    ),
    "pto_b200_ksplit_wait": (_i, [ctypes.c_void_p, ctypes.c_void_p, _i, _i, _i, _i]),
    "pto_b200_ksplit_gemm_allreduce": (
        _i,
        [ctypes.c_void_p, _u8p, _u8p, _i, _i, _i, _ll, _ll, _i, ctypes.POINTER(ctypes.c_void_p),
         ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
         ctypes.c_void_p, ctypes.c_void_p, _i, _i, _i, _i, _i, _ll, _ll, ctypes.c_void_p, ctypes.c_void_p, _i],
    ),
    "pto_b200_allgather_gemm": (
        _i,
        [ctypes.c_void_p, _u8p, ctypes.POINTER(ctypes.c_void_p), _u8p, _i, _i, _i, _ll, _ll, _ll, _i, _i,
         ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p, _i, _i, _i, ctypes.c_void_p, _i],
    ),
    "pto_b200_set_wait_limit": (_ll, [_ll]),
    "call_kernel": (None, [ctypes.c_uint32, ctypes.c_void_p, _u8p, _u8p, _u8p]),
    "pto_b200_device_status": (_i, [ctypes.POINTER(_i)]),
    "pto_b200_error_string": (ctypes.c_char_p, [_i]),
    "pto_b200_last_cuda_error": (ctypes.c_char_p, []),
    "pto_b200_launch_count": (ctypes.c_ulonglong, []),
}

_lib = None


class PtoB200Error(RuntimeError):
    def __init__(self, code: int, where: str):
        lib = load()
        msg = lib.pto_b200_error_string(code).decode()
        detail = lib.pto_b200_last_cuda_error().decode()
        super().__init__(f"{where}: error {code}: {msg}" + (f" [{detail}]" if detail and code == ECUDA else ""))
        self.code = code


def load() -> ctypes.CDLL:
    """Load libpto_b200.so and set the prototypes. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m pto_isa_mirror_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int, where: str) -> None:
    if code != OK:
        raise PtoB200Error(code, where)
