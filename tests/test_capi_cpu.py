"""CPU-side checks of the C ABI: the library loads, exports every symbol include/pto_b200.h declares, and
rejects bad arguments before touching a device (no compute calls here)."""
import ctypes
import os
import re

import pytest

from pto_isa_mirror_b200 import _capi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _capi.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "pto_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pto_b200_\w+|call_kernel)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_functions()
    assert "pto_b200_gemm" in names and "call_kernel" in names and len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/pto_b200.h but not exported"
    assert sorted(_capi.SYMBOLS) == names


def test_error_strings(lib):
    for code in range(9):
        assert lib.pto_b200_error_string(code)
    assert b"unknown" in lib.pto_b200_error_string(99)


def test_argument_errors_come_before_any_launch(lib):
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 15) & ~15
    F16, BF16, F32, S8, S32 = _capi.F16, _capi.BF16, _capi.F32, _capi.S8, _capi.S32
    g = lib.pto_b200_gemm
    before = lib.pto_b200_launch_count()
    assert g(None, None, p, p, 16, 16, 16, 16, 16, 16, F16, F32, 0) == _capi.EINVAL
    assert g(None, p, p, p, 0, 16, 16, 16, 16, 16, F16, F32, 0) == _capi.EINVAL          # empty M
    assert g(None, p, p, p, 16, 16, 16, 8, 16, 16, F16, F32, 0) == _capi.EINVAL          # lda < k
    assert g(None, p, p, p, 16, 16, 16, 16, 16, 8, F16, F32, 0) == _capi.EINVAL          # ldc < n
    assert g(None, p, p + 2, p, 16, 16, 16, 16, 16, 16, F16, F32, 0) == _capi.EALIGN      # A not 16-byte aligned
    assert g(None, p, p, p, 16, 16, 12, 12, 12, 16, F16, F32, 0) == _capi.EALIGN          # 24-byte row pitch
    assert g(None, p, p, p, 16, 16, 16, 16, 16, 16, F32, F32, 0) == _capi.EDTYPE          # fp32 inputs
    assert g(None, p, p, p, 16, 16, 16, 16, 16, 16, F16, S32, 0) == _capi.EDTYPE          # half -> int32
    assert g(None, p, p, p, 16, 16, 16, 16, 16, 16, S8, F32, 0) == _capi.EDTYPE           # int8 -> float
    assert g(None, p, p, p, 16, 16, 16, 16, 16, 16, S8, S32, 1) == _capi.EDTYPE           # int8 with row-major B
    assert g(None, p, p, p, 16, 16, 16, 16, 16, 16, BF16, F32, 7) == _capi.EDTYPE         # unknown layout
    d = lib.pto_b200_gemm_s8_dequant
    assert d(None, p, p, p, None, p, 16, 16, 16, 16, 16, 16) == _capi.EINVAL
    mx = lib.pto_b200_gemm_mx
    E4M3, E5M2 = _capi.E4M3, _capi.E5M2
    assert mx(None, p, p, p, p, p, p, 1 << 20, 16, 16, 48, 48, 48, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EINVAL   # k % 32
    assert mx(None, p, p, p, p, p, p, 1 << 20, 16, 16, 64, 64, 64, 16, 2, 2, S8, E4M3, BF16) == _capi.EDTYPE
    assert mx(None, p, p, p, p, p, p, 1 << 20, 16, 16, 64, 64, 64, 16, 2, 2, E4M3, E5M2, F16 + 0) == _capi.EDTYPE
    E2M1 = _capi.E2M1
    assert mx(None, p, p, p, p, p, p, 1 << 20, 16, 16, 128, 128, 128, 16, 4, 4, E2M1, E4M3, BF16) == _capi.EDTYPE   # fp4 x fp8
    assert mx(None, p, p, p, p, p, p, 1 << 20, 16, 16, 64, 64, 64, 16, 2, 2, E2M1, E2M1, BF16) == _capi.EINVAL     # fp4: k % 128
    assert mx(None, p, p, p, p, p, p, 1 << 20, 16, 16, 128, 160, 128, 16, 4, 4, E2M1, E2M1, BF16) == _capi.EALIGN  # fp4: lda % 64
    assert mx(None, p, p, p, p, p, None, 0, 16, 16, 64, 64, 64, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EWORKSPACE
    assert mx(None, p, p, p, p, p, p, 16, 16, 16, 64, 64, 64, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EWORKSPACE   # too small
    gb = lib.pto_b200_gemm_bias
    assert gb(None, p, p, p, None, 16, 16, 16, 16, 16, 16, F16, F32, 0) == _capi.EINVAL        # bias missing
    assert gb(None, p, p, p, p + 2, 16, 16, 16, 16, 16, 16, F16, F32, 0) == _capi.EALIGN       # bias not 4-byte aligned
    assert gb(None, p, p, p, p, 16, 16, 16, 16, 16, 16, S8, F32, 0) == _capi.EDTYPE
    mxb = lib.pto_b200_gemm_mx_bias
    assert mxb(None, p, p, p, p, p, None, p, 1 << 20, 16, 16, 64, 64, 64, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EINVAL
    gv = lib.pto_b200_gemv
    assert gv(None, None, p, p, None, 16, 16, 16, F16, F32) == _capi.EINVAL
    assert gv(None, p, p, p, None, 16, 16, 8, F16, F32) == _capi.EINVAL                         # ldb < k
    assert gv(None, p, p, p, None, 16, 0, 16, F16, F32) == _capi.EINVAL                         # empty K
    assert gv(None, p, p + 2, p, None, 16, 16, 16, F16, F32) == _capi.EALIGN                    # row not 16-byte aligned
    assert gv(None, p, p, p, None, 16, 12, 12, BF16, F32) == _capi.EALIGN                       # 24-byte column pitch
    assert gv(None, p, p, p, None, 16, 16, 16, S8, F32) == _capi.EDTYPE                         # int8 -> float
    assert gv(None, p, p, p, None, 16, 16, 16, F32, F32) == _capi.EDTYPE
    gvm = lib.pto_b200_gemv_mx
    assert gvm(None, p, p, p, p, p, None, 16, 48, 48, 2, E4M3, E4M3, F32) == _capi.EINVAL          # k % 32
    assert gvm(None, p, p, p, None, p, None, 16, 64, 64, 2, E4M3, E4M3, F32) == _capi.EINVAL      # row scales missing
    assert gvm(None, p, p, p, p, p, None, 16, 64, 64, 2, S8, E4M3, F32) == _capi.EDTYPE
    assert gvm(None, p, p, p, p, p, None, 16, 64, 64, 2, E4M3, E5M2, F16) == _capi.EDTYPE
    assert gvm(None, p, p + 4, p, p, p, None, 16, 64, 64, 2, E4M3, E4M3, F32) == _capi.EALIGN
    qx = lib.pto_b200_mx_quantize_e4m3_ex
    assert qx(None, p, p, p, 4, 64, 64, 64, 2, 7) == _capi.EDTYPE                                  # unknown scale rule
    q = lib.pto_b200_mx_quantize_e4m3
    assert q(None, p, p, None, 4, 64, 64, 64, 2) == _capi.EINVAL
    assert q(None, p, p, p, 4, 48, 48, 48, 2) == _capi.EINVAL                                   # k % 32
    assert q(None, p, p, p, 4, 64, 64, 64, 1) == _capi.EINVAL                                   # ld_scales < k / 32
    assert q(None, p, p, p + 4, 4, 64, 64, 64, 2) == _capi.EALIGN                               # src not 16-byte aligned
    assert q(None, p, p, p, 4, 64, 66, 64, 2) == _capi.EALIGN                                   # ld_src % 4
    q4 = lib.pto_b200_mx_quantize_e2m1
    assert q4(None, p, p, None, 4, 64, 64, 32, 2, 0) == _capi.EINVAL
    assert q4(None, p, p, p, 4, 64, 64, 16, 2, 0) == _capi.EINVAL                                 # ld_data < k / 2
    assert q4(None, p, p, p, 4, 48, 48, 24, 2, 0) == _capi.EINVAL                                 # k % 32
    assert q4(None, p, p, p, 4, 64, 64, 32, 2, 9) == _capi.EDTYPE                                 # unknown scale rule
    assert q4(None, p + 1, p, p, 4, 64, 64, 32, 2, 1) == _capi.EALIGN                             # data not 2-byte aligned
    assert q4(None, p, p, p, 4, 64, 64, 33, 2, 1) == _capi.EALIGN                                 # odd ld_data
    # the workspace-free MX entry reports argument errors like pto_b200_gemm_mx, before it needs a device
    mxs = lib.pto_b200_gemm_mx_static
    assert mxs(None, p, p, p, p, p, 16, 16, 48, 48, 48, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EINVAL           # k % 32
    assert mxs(None, p, p, p, p, p, 16, 16, 64, 64, 64, 16, 2, 2, S8, E4M3, BF16) == _capi.EDTYPE
    assert mxs(None, p, p, p, p, None, 16, 16, 64, 64, 64, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EINVAL        # no B scales
    assert mxs(None, p, p + 2, p, p, p, 16, 16, 64, 64, 64, 16, 2, 2, E4M3, E4M3, BF16) == _capi.EALIGN
    assert mxs(None, p, p, p, p, p, 32768, 8192, 8192, 8192, 8192, 8192, 256, 256, E4M3, E4M3, BF16) == _capi.ESCRATCH
    # pre-quant store forms
    gq = lib.pto_b200_gemm_quant
    assert gq(None, p, p, p, 16, 16, 16, 16, 16, 16, S8, F32, 0, None, 0) == _capi.EDTYPE         # 8- and 16-bit destinations only
    assert gq(None, p, p, p, 16, 16, 16, 16, 16, 16, F32, BF16, 0, None, 0) == _capi.EDTYPE
    assert gq(None, p, p, p, 16, 16, 16, 16, 16, 16, S8, BF16, 0, p + 4, 0) == _capi.EALIGN       # words not 8-byte aligned
    assert gq(None, None, p, p, 16, 16, 16, 16, 16, 16, S8, BF16, 0, None, 0) == _capi.EINVAL
    # one-kernel K-split step
    PA = ctypes.c_void_p * 2
    two = PA(p, p)
    ks = lib.pto_b200_ksplit_gemm_allreduce
    common = (two, two, two, two, p, p)
    assert ks(None, p, p, 256, 256, 64, 64, 64, BF16, *common, 9, 0, 0, 1, 256, 256, 256, None, None, 0) == _capi.EINVAL  # 9 ranks
    assert ks(None, p, p, 256, 256, 64, 64, 64, BF16, *common, 2, 0, 0, 0, 256, 256, 256, None, None, 0) == _capi.EINVAL  # epoch 0
    assert ks(None, p, p, 256, 256, 64, 64, 64, BF16, *common, 2, 0, 0, 1, 100, 256, 256, None, None, 0) == _capi.EINVAL  # panel rows
    assert ks(None, p, p, 256, 256, 64, 64, 64, S8, *common, 2, 0, 0, 1, 256, 256, 256, None, None, 0) == _capi.EDTYPE
    assert ks(None, p, p, 256, 256, 64, 64, 64, BF16, PA(p, None), two, two, two, p, p, 2, 0, 0, 1, 256, 256, 256, None, None,
              0) == _capi.EINVAL                                                                   # a rank's buffer missing
    assert ks(None, p, p, 256, 250, 64, 64, 64, BF16, *common, 2, 0, 0, 1, 256, 250, 250, None, None, 0) == _capi.EALIGN  # n % 4
    assert lib.pto_b200_cast_f32_to_bf16(None, None, p, 4) == _capi.EINVAL
    assert lib.pto_b200_cast_f32_to_bf16(None, p, p, 0) == _capi.OK
    assert lib.pto_b200_launch_count() == before


def test_mx_workspace_size(lib):
    ws = lib.pto_b200_gemm_mx_workspace_bytes
    assert ws(0, 16, 32) == 0
    # 512-byte atoms per 128-wide K block: two per 256-row tile of A plus two per 256-column tile of B
    assert ws(128, 256, 128) == 512 * (2 + 2)
    assert ws(129, 257, 129) == 2 * 512 * (2 + 4)
    assert ws(16384, 8192, 8192) == 64 * 512 * (128 + 64)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", str(tmp_path / "libpto_b200.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _capi.load()


def test_wait_limit_setter_round_trips(lib):
    default = lib.pto_b200_set_wait_limit(123456)
    assert default == 4_000_000_000
    assert lib.pto_b200_set_wait_limit(0) == 123456          # 0 restores the default
    assert lib.pto_b200_set_wait_limit(default) == default
