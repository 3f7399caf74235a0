"""Parity of the bias forms (TMATMUL_BIAS, six-operand TMATMUL_MX), TGEMV and the MX quantiser (TQUANT) with the
oracle and the reference-generated fixtures, through the C ABI.

Integer-valued cases (the reference tests' own style, tests/cpu/st/testcase/tmatmul/gen_data.py:40-61) must be exact;
int32 accumulators and quantised bytes are bit-exact; fp32 results are held to the dense / MX tolerances."""
import numpy as np
import pytest
import torch

import oracle
import pto_isa_mirror_b200 as pto
from conftest import golden
from parity import max_rel_err, result_cmp
from pto_isa_mirror_b200 import gen_data as gd

pytestmark = pytest.mark.gpu
DEV = "cuda"
DENSE_TOL = 1e-3
MX_TOL = 1e-2


def dev16(bits, dtype):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(DEV).view(dtype)


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def host(t):
    torch.cuda.synchronize()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def padded(x, mult):
    rows, cols = x.shape
    pitch = (cols + mult - 1) // mult * mult
    buf = torch.zeros((rows, pitch), dtype=x.dtype, device=DEV)
    buf[:, :cols] = x
    return buf[:, :cols]


@pytest.fixture(autouse=True)
def status_word_stays_clear():
    yield
    assert pto.device_status() == 0, "a kernel gave up on a bounded wait"


# ------------------------------------------------------------------ bias

def test_bias_golden_tiles():
    g = golden("f16_bias_k256")
    a, b = gd.dense_inputs(128, 256, 256, "f16", 7, "uniform")
    out = host(pto.gemm(dev16(a, torch.float16), dev16(b, torch.float16), torch.float32, bias=dev(g["bias"])))
    assert max_rel_err(out, g["out"]) <= DENSE_TOL
    assert result_cmp(g["out"], out, DENSE_TOL)
    out16 = host(pto.gemm(dev16(a, torch.float16), dev16(b, torch.float16), torch.bfloat16, bias=dev(g["bias"])))
    assert np.array_equal(out16, gd.f32_to_bf16_bits(out))      # the bias joins before the store cast

    g = golden("s8_bias_k1024")
    a8, b8, _, _ = gd.s8_inputs(128, 256, 1024, 2)
    assert np.array_equal(host(pto.gemm(dev(a8), dev(b8), torch.int32, bias=dev(g["bias"]))), g["out"])

    g = golden("mx_bias_k256")
    am, sfa = gd.mx_quantize_e4m3(gd.normal((128, 256), 3, 0))
    bm, sfb = gd.mx_quantize_e4m3(gd.normal((256, 256), 3, 1))
    outm = host(pto.gemm_mx(dev(am), dev(bm), dev(sfa), dev(sfb), torch.float32, bias=dev(g["bias"])))
    assert max_rel_err(outm, g["out"]) <= MX_TOL


# bias cases of tests/cpu/st/testcase/tmatmul/gen_data.py:108-111,118 (m, k, n there; m, n, k here)
@pytest.mark.parametrize("kind,m,n,k", [("s8", 8, 6, 7), ("f16", 16, 16, 15), ("f16", 1, 50, 110), ("bf16", 16, 16, 15),
                                        ("f16", 127, 63, 128)])
def test_reference_bias_cases_exact(kind, m, n, k):
    ai = gd.randint((m, k), 1, 5, 29, 0)
    bi = gd.randint((n, k), 1, 5, 29, 1)
    bias = gd.randint((n,), 1, 10, 29, 2)
    exact = ai @ bi.T + bias[None, :]
    if kind == "s8":
        a = padded(dev(ai.astype(np.int8)), 16)
        b = padded(dev(bi.astype(np.int8)), 16)
        out = host(pto.gemm(a, b, torch.int32, bias=dev(bias.astype(np.int32))))
        assert np.array_equal(out, exact)
        assert np.array_equal(oracle.gemm_s8(ai.astype(np.int8), bi.astype(np.int8), bias=bias.astype(np.int32)), exact)
        return
    dt = torch.float16 if kind == "f16" else torch.bfloat16
    a = padded(dev(ai.astype(np.float32)).to(dt), 8)
    b = padded(dev(bi.astype(np.float32)).to(dt), 8)
    out = host(pto.gemm(a, b, torch.float32, bias=dev(bias.astype(np.float32))))
    assert np.array_equal(out.astype(np.int64), exact)
    b_nd = padded(dev(np.ascontiguousarray(bi.T).astype(np.float32)).to(dt), 8)
    out_nd = host(pto.gemm(a, b_nd, torch.float32, pto.B_ND, bias=dev(bias.astype(np.float32))))
    assert np.array_equal(out_nd.astype(np.int64), exact)


@pytest.mark.parametrize("kind", ["f16", "s8"])
def test_bias_on_the_pair_kernel_exact(kind):
    """Enough 256 x 256 tiles for the CTA-pair kernel (9 x 9 = 81 >= 74 pairs), ragged edges, integer values."""
    m, n, k = 2200, 2290, 192
    ai = gd.randint((m, k), -4, 4, 31, 0)
    bi = gd.randint((n, k), -4, 4, 31, 1)
    bias = gd.randint((n,), -1000, 1000, 31, 2)
    exact = ai @ bi.T + bias[None, :]
    if kind == "s8":
        out = host(pto.gemm(dev(ai.astype(np.int8)), dev(bi.astype(np.int8)), torch.int32,
                            bias=dev(bias.astype(np.int32))))
        assert np.array_equal(out, exact)
        rows = slice(1000, 1064)
        assert np.array_equal(oracle.gemm_s8(ai[rows].astype(np.int8), bi.astype(np.int8), bias=bias.astype(np.int32)),
                              exact[rows])
    else:
        a = dev(ai.astype(np.float32)).to(torch.float16)
        b = dev(bi.astype(np.float32)).to(torch.float16)
        out = host(pto.gemm(a, b, torch.float32, bias=dev(bias.astype(np.float32))))
        assert np.array_equal(out.astype(np.int64), exact)
        out16 = host(pto.gemm(a, b, torch.bfloat16, bias=dev(bias.astype(np.float32))))
        assert np.array_equal(out16, oracle.store_cast(exact.astype(np.float32), oracle.BF16))


def test_mx_bias_on_the_pair_kernel():
    m, n, k = 2304, 2304, 256
    am, sfa = gd.mx_quantize_e4m3(gd.normal((m, k), 33, 0))
    bm, sfb = gd.mx_quantize_e4m3(gd.normal((n, k), 33, 1))
    bias = (gd.normal((n,), 33, 2) * np.float32(4.0)).astype(np.float32)
    out = host(pto.gemm_mx(dev(am), dev(bm), dev(sfa), dev(sfb), torch.float32, bias=dev(bias)))
    rows = slice(1200, 1264)
    ref = oracle.gemm_mx(am[rows], bm, sfa[rows], sfb, bias=bias, bias_after_k=128)
    assert max_rel_err(out[rows], ref) <= MX_TOL
    plain = host(pto.gemm_mx(dev(am), dev(bm), dev(sfa), dev(sfb), torch.float32))
    assert np.array_equal(out, plain + bias[None, :])           # one fp32 add of the same accumulator


# ------------------------------------------------------------------ TGEMV

# m = 1 cases of tests/cpu/st/testcase/tmatmul/gen_data.py:106,111 plus ragged K tails and an int8 row
@pytest.mark.parametrize("kind,n,k", [("f16", 50, 110), ("bf16", 64, 128), ("f16", 513, 1000), ("s8", 90, 89),
                                      ("s8", 300, 4112)])
def test_gemv_integer_cases_exact(kind, n, k):
    xi = gd.randint((1, k), 1, 5, 37, 0)
    bi = gd.randint((n, k), 1, 5, 37, 1)
    bias = gd.randint((n,), 1, 10, 37, 2)
    exact = (xi @ bi.T)[0]
    if kind == "s8":
        x = dev(xi[0].astype(np.int8))
        b = padded(dev(bi.astype(np.int8)), 16)
        assert np.array_equal(host(pto.gemv(x, b)), exact)
        assert np.array_equal(host(pto.gemv(x, b, bias=dev(bias.astype(np.int32)))), exact + bias)
        assert np.array_equal(oracle.gemm_s8(xi.astype(np.int8), bi.astype(np.int8))[0], exact)
        return
    dt = torch.float16 if kind == "f16" else torch.bfloat16
    x = dev(xi[0].astype(np.float32)).to(dt)
    b = padded(dev(bi.astype(np.float32)).to(dt), 8)
    assert np.array_equal(host(pto.gemv(x, b, torch.float32)).astype(np.int64), exact)
    assert np.array_equal(host(pto.gemv(x, b, torch.float32, bias=dev(bias.astype(np.float32)))).astype(np.int64),
                          exact + bias)
    got16 = host(pto.gemv(x, b, torch.bfloat16))
    assert np.array_equal(got16, oracle.store_cast(exact.astype(np.float32), oracle.BF16))
    # the tile loop with a one-row left operand computes the same thing
    assert np.array_equal(host(pto.gemm(padded(x.view(1, k), 8), b, torch.float32))[0].astype(np.int64), exact)


def test_gemv_bf16_against_the_oracle():
    n, k = 4096, 8192
    a, b = gd.dense_inputs(1, n, k, "bf16", 41)
    out = host(pto.gemv(dev16(a, torch.bfloat16).view(-1), dev16(b, torch.bfloat16), torch.float32))
    ref = oracle.gemm_f32acc(a, b, oracle.BF16)[0]
    assert max_rel_err(out, ref) <= DENSE_TOL
    assert result_cmp(ref, out, DENSE_TOL)


def test_gemv_rejects_bad_arguments():
    b = torch.zeros((8, 64), dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        pto.gemv(torch.zeros(32, dtype=torch.float16, device=DEV), b)
    with pytest.raises(ValueError):
        pto.gemv(torch.zeros(64, dtype=torch.bfloat16, device=DEV), b)
    with pytest.raises(pto.PtoB200Error):
        pto.gemv(torch.zeros(72, dtype=torch.float16, device=DEV)[8:], torch.zeros((8, 72), dtype=torch.float16,
                                                                                    device=DEV)[:, 4:68])


# ------------------------------------------------------------------ MX quantiser

def test_mx_quantiser_bit_exact():
    g = golden("mx_quantize")                                   # zeros, 1e-30 and 1e30 blocks, a lone negative tiny value
    d, s = pto.mx_quantize_e4m3(dev(g["src"]))
    assert np.array_equal(host(d), g["data"]) and np.array_equal(host(s), g["scales"])

    src = gd.normal((300, 4096), 43)
    src[5] *= np.float32(1e-20)
    src[6] *= np.float32(1e20)
    src[7, ::3] = 0
    src[8] = -np.abs(src[8]) * np.float32(1e-4)
    src[9, :64] = np.float32(2.0) ** np.arange(-32, 32, dtype=np.float32)      # exact powers of two
    src[10, :32] = np.float32(448.0) * np.float32(2.0) ** -np.arange(32, dtype=np.float32)
    # ties between neighbouring e4m3 codes: the block maximum 1.9375 gives a scaling of 2^8, so 1 + (2 i + 1) / 16
    # lands midway between two normal codes and j / 2 * 2^-17 midway between two subnormal codes (or zero)
    sub = np.array([0.5, 1.5, 2.5, 3.5, 6.5, 7.5, 8.5, -0.5, -1.5, -2.5, -7.5, 0.25, -0.25, 0.75]) * 2.0 ** -17
    src[11, :32] = np.concatenate([[1.9375], 1.0 + (2 * np.arange(7) + 1) / 16.0, sub, np.zeros(10)])
    d, s = pto.mx_quantize_e4m3(dev(src))
    rd, rs = oracle.mx_quantize_e4m3(src)
    assert np.array_equal(host(s), rs)
    assert np.array_equal(host(d), rd)

    # a strided view (row pitch larger than K)
    wide = torch.zeros((64, 512 + 64), dtype=torch.float32, device=DEV)
    wide[:, :512] = dev(src[:64, :512])
    d2, s2 = pto.mx_quantize_e4m3(wide[:, :512])
    assert np.array_equal(host(d2), rd[:64, :512]) and np.array_equal(host(s2), rs[:64, :16])


def test_quantise_then_multiply_matches_the_oracle_pipeline():
    m, n, k = 128, 256, 512
    xa, xb = gd.normal((m, k), 47, 0), gd.normal((n, k), 47, 1)
    a, sfa = pto.mx_quantize_e4m3(dev(xa))
    b, sfb = pto.mx_quantize_e4m3(dev(xb))
    out = host(pto.gemm_mx(a, b, sfa, sfb, torch.float32))
    ra, rsa = oracle.mx_quantize_e4m3(xa)
    rb, rsb = oracle.mx_quantize_e4m3(xb)
    assert np.array_equal(host(a), ra) and np.array_equal(host(sfb), rsb)
    assert max_rel_err(out, oracle.gemm_mx(ra, rb, rsa, rsb)) <= MX_TOL


# ------------------------------------------------------------------ TSTORE with a pre-quant scale word / TSTORE_FP

def words_dev(words):
    return torch.from_numpy(np.ascontiguousarray(words).view(np.int64)).to(DEV)


QUANT_GOLDEN = [("s32_scalar_bf16", False, False, torch.bfloat16), ("s32_vector_bf16", True, False, torch.bfloat16),
                ("s32_vector_bf16_relu", True, True, torch.bfloat16), ("s32_scalar_f16", False, False, torch.float16),
                ("s32_vector_f16_relu", True, True, torch.float16)]


@pytest.mark.parametrize("name,vector,relu,odt", QUANT_GOLDEN)
def test_quant_store_int8_golden_bit_exact(name, vector, relu, odt):
    """The int8 tile of configuration 3 stored through TSTORE(dst, acc, preQuantScalar) and TSTORE_FP: the simulator's
    own outputs (tests/golden/quant_store.npz), bit for bit."""
    g = golden("quant_store")
    a, b, _, _ = gd.s8_inputs(128, 256, 1024, 2)
    scalar = int(g["scalar_word"][0])
    out = pto.gemm_quant(dev(a), dev(b), odt, pre_quant_scalar=scalar,
                         fp_words=words_dev(g["vector_words"]) if vector else None, relu=relu)
    assert np.array_equal(host(out), g[name])


@pytest.mark.parametrize("kind", ["s8", "f16", "bf16"])
def test_quant_store_on_the_pair_kernel(kind):
    """Every pre-quant form on a problem that takes the CTA-pair kernel (ragged 2300 x 2328, store boxes and register
    stores), against the oracle's store applied to the GPU's own accumulators: bit-exact."""
    m, n, k = 2300, 2328, 256
    if kind == "s8":
        a, b, _, _ = gd.s8_inputs(m, n, k, 81)
        ta, tb = dev(a), dev(b)
        acc = host(pto.gemm(ta, tb, torch.int32))
        scalar = np.array([np.float32(0.0123)]).view(np.uint32).astype(np.uint64)
    else:
        a, b = gd.dense_inputs(m, n, k, kind, 82)
        dt = torch.float16 if kind == "f16" else torch.bfloat16
        ta, tb = dev16(a, dt), dev16(b, dt)
        acc = host(pto.gemm(ta, tb, torch.float32))
        scalar = np.array([np.float32(700000.0)]).view(np.uint32).astype(np.uint64)  # half outputs reach the clamp
    col = gd.uniform((n,), 0.5, 2.0, 83, 0) * (np.float32(0.01) if kind == "s8" else np.float32(600000.0))
    col[3] = -col[3]
    col[5] = 0.0
    words = col.view(np.uint32).astype(np.uint64)
    for vector in (False, True):
        for relu in (False, True):
            for odt, f16 in ((torch.bfloat16, False), (torch.float16, True)):
                out = pto.gemm_quant(ta, tb, odt, pre_quant_scalar=int(scalar[0]),
                                     fp_words=words_dev(words) if vector else None, relu=relu)
                want = oracle.quant_store(acc, words if vector else scalar, vector, relu, f16)
                assert np.array_equal(host(out), want), (kind, vector, relu, f16)


def test_quant_store_rejects_bad_arguments():
    a = torch.zeros((128, 64), dtype=torch.int8, device=DEV)
    with pytest.raises(pto.PtoB200Error) as e:
        pto.gemm_quant(a, a, torch.float32)                    # only 16-bit destinations
    assert e.value.code == 3
    with pytest.raises(ValueError):
        pto.gemm_quant(a, a, torch.bfloat16, fp_words=torch.zeros(5, dtype=torch.int64, device=DEV))


def test_mx_quantiser_nv_rule_bit_exact():
    """pto_b200_mx_quantize_e4m3_ex with QuantScaleAlg::NV against the simulator's fixture and, on a larger matrix,
    against the oracle."""
    from pto_isa_mirror_b200 import _capi

    g = golden("mx_quantize_nv")
    d, s = pto.mx_quantize_e4m3(dev(g["src"]), scale_alg=_capi.SCALE_NV)
    assert np.array_equal(host(s), g["scales"])
    assert np.array_equal(host(d), g["data"])
    x = gd.normal((777, 1056), 17) * np.float32(5.0)
    x[::7] *= np.float32(1e-6)
    d, s = pto.mx_quantize_e4m3(dev(x), scale_alg=_capi.SCALE_NV)
    rd, rs = oracle.mx_quantize_e4m3(x, oracle.NV)
    assert np.array_equal(host(s), rs) and np.array_equal(host(d), rd)
    with pytest.raises(pto.PtoB200Error):
        pto.mx_quantize_e4m3(dev(x), scale_alg=5)


# ------------------------------------------------------------------ TGEMV_MX (one left row, block-scaled)

@pytest.mark.parametrize("fa,fb", [(pto.E4M3, pto.E4M3), (pto.E4M3, pto.E5M2), (pto.E5M2, pto.E4M3),
                                   (pto.E5M2, pto.E5M2)])
def test_gemv_mx_integer_cases_exact(fa, fb):
    """Integers in [-10, 10] with scales 2^0..2^2 (tests/cpu/st/testcase/tmatmul_mx/gen_data.py:113-138): exact."""
    import ml_dtypes

    n, k = 300, 1056
    enc = {pto.E4M3: ml_dtypes.float8_e4m3fn, pto.E5M2: ml_dtypes.float8_e5m2}
    xi = gd.randint((1, k), -10, 10, 23, 0).astype(np.float32)
    bi = gd.randint((n, k), -10, 10, 23, 1).astype(np.float32)
    # (e5m2 cannot hold 9: the encoder rounds it; the expected values are computed from the encoded bytes)
    x8 = xi.astype(enc[fa]).view(np.uint8)
    b8 = bi.astype(enc[fb]).view(np.uint8)
    sfx = gd.randint((1, k // 32), 127, 129, 23, 2).astype(np.uint8)
    sfb = gd.randint((n, k // 32), 127, 129, 23, 3).astype(np.uint8)
    exact = oracle.gemm_mx(x8, b8, sfx, sfb, fa, fb)[0]
    bias = gd.normal((n,), 24).astype(np.float32).round()
    out = pto.gemv_mx(dev(x8[0]), dev(b8), dev(sfx[0]), dev(sfb), torch.float32, fa, fb)
    assert np.array_equal(host(out), exact)
    outb = pto.gemv_mx(dev(x8[0]), dev(b8), dev(sfx[0]), dev(sfb), torch.float32, fa, fb, bias=dev(bias))
    assert np.array_equal(host(outb), exact + bias)


def test_gemv_mx_against_the_oracle_and_the_tile_kernel():
    """Quantised N(0, 1) data: within the MX tolerance of the oracle's chain, and of row 0 of the block-scaled GEMM."""
    n, k = 2048, 4096
    a, b, sfa, sfb = gd.mx_inputs(128, n, k, 25)
    ref = oracle.gemm_mx(a[:1], b, sfa[:1], sfb)[0]
    out = pto.gemv_mx(dev(a[0]), dev(b), dev(sfa[0]), dev(sfb), torch.float32)
    assert max_rel_err(host(out), ref) <= MX_TOL
    full = pto.gemm_mx(dev(a), dev(b), dev(sfa), dev(sfb), torch.float32)
    assert max_rel_err(host(out), host(full)[0]) <= MX_TOL
    out16 = pto.gemv_mx(dev(a[0]), dev(b), dev(sfa[0]), dev(sfb), torch.bfloat16)
    assert np.array_equal(host(out16), gd.f32_to_bf16_bits(host(out)))
    with pytest.raises(pto.PtoB200Error):
        pto.gemv_mx(dev(a[0]), dev(b), dev(sfa[0]), dev(sfb), torch.float16)


@pytest.mark.parametrize("n,k", [(9, 8192), (4, 10240), (7, 12320), (3, 16384), (5, 16416), (5, 40960), (33, 41984),
                                 (37, 65536)])
def test_gemv_mx_long_rows_exact(n, k):
    """Left rows up to 40960 values are kept in shared memory as floats; longer ones take the kernel that multiplies
    whole scale blocks with the warp-level fp8 MMA. Integers with power-of-two scales: both are exact, odd column
    counts and K that is not a multiple of 512 included."""
    import ml_dtypes

    xi = gd.randint((1, k), -6, 6, 27, 0).astype(np.float32)
    bi = gd.randint((n, k), -6, 6, 27, 1).astype(np.float32)
    x8 = xi.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    b8 = bi.astype(ml_dtypes.float8_e5m2).view(np.uint8)
    sfx = gd.randint((1, k // 32), 126, 128, 27, 2).astype(np.uint8)
    sfb = gd.randint((n, k // 32), 126, 128, 27, 3).astype(np.uint8)
    exact = oracle.gemm_mx(x8, b8, sfx, sfb, pto.E4M3, pto.E5M2)[0]
    out = pto.gemv_mx(dev(x8[0]), dev(b8), dev(sfx[0]), dev(sfb), torch.float32, pto.E4M3, pto.E5M2)
    assert np.array_equal(host(out), exact)


# ------------------------------------------------------------------ TQUANT to MXFP4 (float4_e2m1x2_t)

@pytest.mark.parametrize("alg", ["ocp", "nv"])
def test_mxfp4_quantiser_bit_exact(alg):
    """pto_b200_mx_quantize_e2m1 against the simulator's fixture (every rounding tie, zero / tiny / huge blocks, maxima
    that the OCP rule truncates to bf16) and, on a larger matrix with a strided view, against the oracle."""
    from pto_isa_mirror_b200 import _capi

    code = _capi.SCALE_OCP if alg == "ocp" else _capi.SCALE_NV
    ocode = oracle.OCP if alg == "ocp" else oracle.NV
    g = golden("mxfp4_quantize")
    d, s = pto.mx_quantize_e2m1(dev(g["src"]), scale_alg=code)
    assert np.array_equal(host(s), g["scales_" + alg])
    assert np.array_equal(host(d), g["data_" + alg])
    x = gd.normal((777, 1056), 19) * np.float32(3.0)
    x[::7] *= np.float32(1e-6)
    x[5] *= np.float32(1e20)
    x[6, ::3] = 0
    x[9, :64] = np.float32(2.0) ** np.arange(-32, 32, dtype=np.float32)
    rd, rs = oracle.mx_quantize_e2m1(x, ocode)
    d, s = pto.mx_quantize_e2m1(dev(x), scale_alg=code)
    assert np.array_equal(host(s), rs) and np.array_equal(host(d), rd)
    wide = torch.zeros((64, 512 + 64), dtype=torch.float32, device=DEV)
    wide[:, :512] = dev(x[:64, :512])
    d2, s2 = pto.mx_quantize_e2m1(wide[:, :512], scale_alg=code)
    assert np.array_equal(host(d2), rd[:64, :256]) and np.array_equal(host(s2), rs[:64, :16])
    with pytest.raises(pto.PtoB200Error):
        pto.mx_quantize_e2m1(dev(x), scale_alg=5)


def test_mxfp4_quantise_then_multiply():
    """Both MXFP4 operands produced on the device by the quantiser and multiplied by the block-scaled kernel: equal to
    the oracle's product of the same quantised bytes, and close to the fp32 product of the unquantised matrices."""
    m, n, k = 256, 512, 1024
    a32 = gd.normal((m, k), 51)
    b32 = gd.normal((n, k), 52)
    a4, sa = pto.mx_quantize_e2m1(dev(a32))
    b4, sb = pto.mx_quantize_e2m1(dev(b32))
    out = host(pto.gemm_mx(a4, b4, sa, sb, torch.float32, pto.E2M1, pto.E2M1))
    ref = oracle.gemm_mx(host(a4)[:128], host(b4), host(sa)[:128], host(sb), oracle.E2M1, oracle.E2M1)
    assert max_rel_err(out[:128], ref) <= MX_TOL
    exact = a32.astype(np.float64) @ b32.astype(np.float64).T
    assert np.abs(out - exact).max() / np.abs(exact).max() < 0.25      # 4-bit operands: a coarse product


# ------------------------------------------------------------------ 8-bit destinations of the pre-quant store

@pytest.mark.parametrize("name,words,vector,relu,odt", [
    ("s32_scalar_s8", "w_si", False, False, torch.int8), ("s32_scalar_u8_relu", "w_ui", False, True, torch.uint8),
    ("s32_vector_s8", "vec_i", True, False, torch.int8), ("s32_vector_s8_relu", "vec_i", True, True, torch.int8)])
def test_quant_store_8_bit_golden_bit_exact(name, words, vector, relu, odt):
    """REQ8 / VREQ8 on the int8 tile of configuration 3 against the simulator's own outputs."""
    g = golden("quant_store_b8")
    a, b, _, _ = gd.s8_inputs(128, 256, 1024, 2)
    out = pto.gemm_quant(dev(a), dev(b), odt, pre_quant_scalar=int(g[words][0]),
                         fp_words=words_dev(g[words]) if vector else None, relu=relu)
    assert np.array_equal(host(out).view(np.uint8), g[name].astype(np.uint8))


@pytest.mark.parametrize("kind", ["s8", "bf16"])
def test_quant_store_8_bit_on_the_pair_kernel(kind):
    """The 8-bit forms on a ragged problem that takes the CTA-pair kernel, rows off every alignment (pitch n + 3), against
    the oracle's store applied to the GPU's own accumulators: bit-exact, padding untouched."""
    m, n, k = 2300, 2328, 256
    if kind == "s8":
        a, b, _, _ = gd.s8_inputs(m, n, k, 91)
        ta, tb = dev(a), dev(b)
        acc = host(pto.gemm(ta, tb, torch.int32))
        scale = np.float32(100.0 / np.abs(acc).max())
    else:
        a, b = gd.dense_inputs(m, n, k, "bf16", 92)
        ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
        acc = host(pto.gemm(ta, tb, torch.float32))
        scale = np.float32(100.0 / np.abs(acc).max())
    col = (gd.uniform((n,), 0.5, 1.5, 93, 0) * scale).astype(np.float32)
    offs = (np.arange(n) % 9).astype(np.uint64)
    sign = (np.arange(n) % 3 != 0).astype(np.uint64)
    vec = col.view(np.uint32).astype(np.uint64) | (offs << np.uint64(37)) | (sign << np.uint64(46))
    scalar = (np.array([scale * np.float32(1.7)]).view(np.uint32).astype(np.uint64) | (np.uint64(5) << np.uint64(37))
              | (np.uint64(1) << np.uint64(46)))
    for vector in (False, True):
        for relu in (False, True):
            for pitch in (n + 3, n + 24):
                buf = torch.full((m + 2, pitch), 77, dtype=torch.uint8, device=DEV)
                pto.gemm_quant(ta, tb, torch.uint8, pre_quant_scalar=int(scalar[0]),
                               fp_words=words_dev(vec) if vector else None, relu=relu, out=buf[1:m + 1, :n])
                got = host(buf)
                want = oracle.quant_store(acc, vec if vector else scalar, vector, relu, oracle.OUT_U8).astype(np.uint8)
                assert np.array_equal(got[1:m + 1, :n], want), (kind, vector, relu, pitch)
                assert (got[0] == 77).all() and (got[m + 1] == 77).all() and (got[:, n:] == 77).all()


@pytest.mark.parametrize("name,words,vector,relu", [("s32_scalar_s16", "w_shift", False, False),
                                                    ("s32_vector_s16", "vec_shift", True, False),
                                                    ("s32_vector_s16_relu", "vec_shift", True, True)])
def test_quant_store_int16_shift_golden_bit_exact(name, words, vector, relu):
    """SHIFTS322S16 / VSHIFTS322S16 on the int8 tile of configuration 3 against the simulator's own outputs."""
    g = golden("quant_store_s16")
    a, b, _, _ = gd.s8_inputs(128, 256, 1024, 2)
    out = pto.gemm_quant(dev(a), dev(b), torch.int16, pre_quant_scalar=int(g[words][0]),
                         fp_words=words_dev(g[words]) if vector else None, relu=relu)
    assert np.array_equal(host(out).view(np.uint16), g[name])


def test_quant_store_int16_on_the_pair_kernel():
    """The shift form on a ragged problem that takes the CTA-pair kernel (TMA store boxes for the 16-byte pitch, register
    stores for the odd one), against the oracle's store applied to the GPU's own accumulators."""
    m, n, k = 2300, 2328, 256
    a, b, _, _ = gd.s8_inputs(m, n, k, 95)
    ta, tb = dev(a), dev(b)
    acc = host(pto.gemm(ta, tb, torch.int32))
    vec = ((np.arange(n) % 7).astype(np.uint64) << np.uint64(32)) | np.uint64(0x777)
    scalar = np.array([np.uint64(2) << np.uint64(32)], dtype=np.uint64)
    for vector in (False, True):
        for relu in (False, True):
            for pitch in (n, n + 5):
                buf = torch.full((m + 2, pitch), 77, dtype=torch.int16, device=DEV)
                pto.gemm_quant(ta, tb, torch.int16, pre_quant_scalar=int(scalar[0]),
                               fp_words=words_dev(vec) if vector else None, relu=relu, out=buf[1:m + 1, :n])
                got = host(buf).view(np.uint16)
                want = oracle.quant_store(acc, vec if vector else scalar, vector, relu, oracle.OUT_S16)
                assert np.array_equal(got[1:m + 1, :n], want), (vector, relu, pitch)
                assert (got[0] == 77).all() and (got[m + 1] == 77).all() and (got[:, n:] == 77).all()
    with pytest.raises(pto.PtoB200Error):                       # float accumulators have no shift form
        pto.gemm_quant(torch.zeros((128, 64), dtype=torch.bfloat16, device=DEV),
                       torch.zeros((128, 64), dtype=torch.bfloat16, device=DEV), torch.int16)
