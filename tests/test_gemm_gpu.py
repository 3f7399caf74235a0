"""Parity of the CUDA tile loop with the oracle, through the C ABI (ctypes) with torch tensors as device buffers.

Tolerances (from the benchmark specification): int8 accumulators bit-exact; fp16/bf16 -> fp32 max relative
error <= 1e-3; MXFP8 <= 1e-2; integer-valued inputs (the reference tests' own style) exact in every precision."""
import numpy as np
import pytest
import torch

import oracle
import pto_isa_mirror_b200 as pto
from conftest import golden
from parity import bf16_ulp_distance, max_elem_rel_err, max_rel_err, result_cmp
from pto_isa_mirror_b200 import gen_data as gd

pytestmark = pytest.mark.gpu
DEV = "cuda"
DENSE_TOL = 1e-3
MX_TOL = 1e-2


def dev16(bits, dtype):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(DEV).view(dtype)


def dev8(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def host(t):
    torch.cuda.synchronize()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    if t.dtype == torch.float16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


@pytest.fixture(autouse=True)
def status_word_stays_clear():
    yield
    assert pto.device_status() == 0, "a kernel gave up on a bounded wait"


# ------------------------------------------------------------------ configuration 1 and the reference's small cases

@pytest.mark.parametrize("b_layout", [pto.B_DN, pto.B_ND])
def test_c1_fp16_128x256x256(b_layout):
    g = golden("c1_f16_k256")
    a, b = gd.dense_inputs(128, 256, 256, "f16", 0, "uniform")
    bt = dev16(b if b_layout == pto.B_DN else np.ascontiguousarray(b.T), torch.float16)
    out = host(pto.gemm(dev16(a, torch.float16), bt, torch.float32, b_layout))
    assert max_rel_err(out, g["out"]) <= DENSE_TOL
    assert max_elem_rel_err(out, g["out"]) <= DENSE_TOL
    assert result_cmp(g["out"], out, 1e-3)
    assert np.array_equal(oracle.gemm_f32acc(a, b, oracle.F16), g["out"])


def test_pto_gemm_basic_op():
    a, b = gd.dense_inputs(512, 1536, 2048, "f16", 21)   # the op's reference shape
    out = host(pto.pto_gemm_basic(dev16(a, torch.float16), dev16(b, torch.float16)))
    ref = oracle.gemm_f32acc(a[:128], b[:256], oracle.F16)
    assert max_rel_err(out[:128, :256], ref) <= DENSE_TOL
    with pytest.raises(ValueError):
        pto.pto_gemm_basic(dev16(a, torch.float16).float(), dev16(b, torch.float16))


def padded(x, mult):
    """Copy x into a buffer whose row pitch is a multiple of `mult` elements and return the [rows, cols] view."""
    rows, cols = x.shape
    pitch = (cols + mult - 1) // mult * mult
    buf = torch.zeros((rows, pitch), dtype=x.dtype, device=DEV)
    buf[:, :cols] = x
    return buf[:, :cols]


# shapes of tests/cpu/st/testcase/tmatmul/gen_data.py:102-119 and tests/npu/a2a3/src/st/testcase/tmatmul/gen_data.py:170-190
REF_SMALL = [("f16", 40, 50, 60), ("f16", 128, 128, 64), ("f16", 1, 110, 50), ("bf16", 40, 50, 60),
             ("bf16", 11, 402, 30), ("s8", 6, 7, 8), ("s8", 65, 90, 89), ("f16", 120, 110, 50), ("f16", 127, 72, 64)]


@pytest.mark.parametrize("kind,m,n,k", REF_SMALL)
def test_reference_small_integer_cases_exact(kind, m, n, k):
    ai = gd.randint((m, k), 1, 5, 19, 0)
    bi = gd.randint((n, k), 1, 5, 19, 1)
    exact = ai @ bi.T
    if kind == "s8":
        a = padded(torch.from_numpy(ai.astype(np.int8)).to(DEV), 16)
        b = padded(torch.from_numpy(bi.astype(np.int8)).to(DEV), 16)
        out = host(pto.gemm(a, b, torch.int32))
        assert np.array_equal(out, exact)
        assert np.array_equal(oracle.gemm_s8(ai.astype(np.int8), bi.astype(np.int8)), exact)
        return
    dt = torch.float16 if kind == "f16" else torch.bfloat16
    a = padded(torch.from_numpy(ai.astype(np.float32)).to(DEV).to(dt), 8)
    b = padded(torch.from_numpy(bi.astype(np.float32)).to(DEV).to(dt), 8)
    out = host(pto.gemm(a, b, torch.float32))
    assert np.array_equal(out.astype(np.int64), exact)
    # row-major B (the demo's layout) gives the same result
    b_nd = padded(torch.from_numpy(np.ascontiguousarray(bi.T).astype(np.float32)).to(DEV).to(dt), 8)
    assert np.array_equal(host(pto.gemm(a, b_nd, torch.float32, pto.B_ND)).astype(np.int64), exact)
    # 16-bit stores: values <= 25 * k are exact in half only for small k; compare against the oracle's cast
    for out_dt, code in ((torch.float16, oracle.F16), (torch.bfloat16, oracle.BF16)):
        got = host(pto.gemm(a, b, out_dt))
        assert np.array_equal(got, oracle.store_cast(exact.astype(np.float32), code))


def test_split_k_accumulation_equals_one_chain():
    """TMATMUL then TMATMUL_ACC over K chunks (tmatmul split-K case) is the same sum as one call over the whole K."""
    a, b = gd.dense_inputs(128, 128, 320, "f16", 23)
    ta, tb = dev16(a, torch.float16), dev16(b, torch.float16)
    whole = host(pto.gemm(ta, tb, torch.float32))
    ref = oracle.gemm_f32acc(a, b, oracle.F16)
    assert max_rel_err(whole, ref) <= DENSE_TOL


# ------------------------------------------------------------------ sampled tiles of the big configurations

@pytest.mark.parametrize("k", [1024, 4096, 8192, 65536])
def test_bf16_golden_tiles(k):
    g = golden(f"bf16_tile_k{k}")
    seed = 1 if k <= 4096 else 4
    a, b = gd.dense_inputs(128, 256, k, "bf16", seed)
    ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
    out32 = host(pto.gemm(ta, tb, torch.float32))
    assert max_rel_err(out32, g["out"]) <= DENSE_TOL
    assert max_elem_rel_err(out32, g["out"]) <= DENSE_TOL
    out16 = host(pto.gemm(ta, tb, torch.bfloat16))
    assert np.array_equal(out16, gd.f32_to_bf16_bits(out32))   # the store cast itself is exact RNE
    # against the reference's bf16 store: at most one bf16 step apart wherever the value is not near zero
    # (near zero an fp32 difference of 1e-6 of the matrix scale spans several tiny bf16 steps)
    big = np.abs(g["out"]) >= np.sqrt(np.mean(g["out"] ** 2)) / 16
    assert bf16_ulp_distance(out16[big], g["out_bf16"][big]) <= 1
    assert max_rel_err(gd.bf16_bits_to_f32(out16), gd.bf16_bits_to_f32(g["out_bf16"])) <= DENSE_TOL + 2.0 ** -8


@pytest.mark.parametrize("k", [1024, 8192])
def test_int8_golden_tiles_bit_exact(k):
    g = golden(f"s8_tile_k{k}")
    a, b, s_row, s_col = gd.s8_inputs(128, 256, k, 2)
    ta, tb = dev8(a), dev8(b)
    assert np.array_equal(host(pto.gemm(ta, tb, torch.int32)), g["acc"])
    deq = host(pto.gemm_s8_dequant(ta, tb, dev8(s_row), dev8(s_col)))
    assert np.array_equal(deq, g["deq_bf16"])


@pytest.mark.parametrize("k", [256, 8192])
def test_mx_golden_tiles(k):
    g = golden(f"mx_tile_k{k}")
    a, sfa = gd.mx_quantize_e4m3(gd.normal((128, k), 3, 0))
    b, sfb = gd.mx_quantize_e4m3(gd.normal((256, k), 3, 1))
    out = host(pto.gemm_mx(dev8(a), dev8(b), dev8(sfa), dev8(sfb), torch.float32))
    assert max_rel_err(out, g["out"]) <= MX_TOL
    assert max_elem_rel_err(out, g["out"]) <= MX_TOL
    out16 = host(pto.gemm_mx(dev8(a), dev8(b), dev8(sfa), dev8(sfb), torch.bfloat16))
    assert np.array_equal(out16, gd.f32_to_bf16_bits(out))


def test_mx_mixed_formats_integers_exact():
    g = golden("mx_randint_e4m3_e5m2_k256")
    out = host(pto.gemm_mx(dev8(g["a"]), dev8(g["b"]), dev8(g["sfa"]), dev8(g["sfb"]), torch.float32,
                           a_fmt=pto.E4M3, b_fmt=pto.E5M2))
    assert np.array_equal(out, g["out"])


# shapes of tests/cpu/st/testcase/tmatmul_mx/gen_data.py (K rounded up to the 32-element block)
@pytest.mark.parametrize("m,n,k,fa,fb", [(128, 64, 64, 5, 5), (127, 72, 64, 5, 6), (10, 50, 64, 6, 5),
                                          (4, 30, 128, 6, 6), (200, 136, 96, 5, 5), (1, 256, 32, 5, 5)])
def test_mx_reference_shapes_integers_exact(m, n, k, fa, fb):
    import ml_dtypes

    def enc(x, f):
        return x.astype(ml_dtypes.float8_e4m3fn if f == 5 else ml_dtypes.float8_e5m2).view(np.uint8)

    ai = gd.randint((m, k), -10, 10, 19, 2).astype(np.float32)
    bi = gd.randint((n, k), -10, 10, 19, 3).astype(np.float32)
    a8, b8 = enc(ai, fa), enc(bi, fb)
    sfa = gd.randint((m, k // 32), 127, 129, 19, 4).astype(np.uint8)
    sfb = gd.randint((n, k // 32), 127, 129, 19, 5).astype(np.uint8)
    ref = oracle.gemm_mx(a8, b8, sfa, sfb, fa, fb)
    ta, tb = padded(dev8(a8), 16), padded(dev8(b8), 16)
    tsa, tsb = dev8(sfa), dev8(sfb)
    out = host(pto.gemm_mx(ta, tb, tsa, tsb, torch.float32, a_fmt=fa, b_fmt=fb))
    assert np.array_equal(out, ref)


# ------------------------------------------------------------------ full-size configurations: sampled tiles + whole-matrix properties

def sample_tiles(m, n, count, seed):
    idx = gd.randint((count, 2), 0, 1 << 30, seed, 9)
    return [(int(i % (m // 128)) * 128, int(j % (n // 256)) * 256) for i, j in idx]


def test_c2_bf16_4096_cubed():
    m = n = k = 4096
    a, b = gd.dense_inputs(m, n, k, "bf16", 1)
    ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
    out32 = host(pto.gemm(ta, tb, torch.float32, workspace="auto"))      # with the split last wave
    out16 = host(pto.gemm(ta, tb, torch.bfloat16, workspace="auto"))
    assert np.array_equal(out16, gd.f32_to_bf16_bits(out32))
    for r0, c0 in sample_tiles(m, n, 8, 31):
        ref = oracle.gemm_f32acc(a[r0:r0 + 128], b[c0:c0 + 256], oracle.BF16)
        assert max_rel_err(out32[r0:r0 + 128, c0:c0 + 256], ref) <= DENSE_TOL
        big = np.abs(ref) >= np.sqrt(np.mean(ref ** 2)) / 16
        assert bf16_ulp_distance(out16[r0:r0 + 128, c0:c0 + 256][big], gd.f32_to_bf16_bits(ref)[big]) <= 1
    # linearity in a power of two is exact, and a row permutation of A permutes C bit for bit
    a2 = gd.f32_to_bf16_bits(gd.bf16_bits_to_f32(a) * np.float32(2.0))
    assert np.array_equal(host(pto.gemm(dev16(a2, torch.bfloat16), tb, torch.float32, workspace="auto")),
                          out32 * np.float32(2.0))
    # without the workspace no tile is split along K, and then a row permutation of A permutes C bit for bit
    plain = host(pto.gemm(ta, tb, torch.float32, workspace=None))
    perm = np.argsort(gd.uniform01(m, 77))
    assert np.array_equal(host(pto.gemm(dev16(a[perm], torch.bfloat16), tb, torch.float32, workspace=None)), plain[perm])
    # with it the 34 leftover tiles of the fourth wave are summed as two K halves: same values up to
    # the fp32 summation order, and most tiles are untouched
    assert max_rel_err(out32, plain) <= 1e-5
    assert (out32 == plain).mean() > 0.8 and (out32 != plain).any()


def test_c3_int8_8192_cubed_exact():
    m = n = k = 8192
    a, b, s_row, s_col = gd.s8_inputs(m, n, k, 2)
    ta, tb = dev8(a), dev8(b)
    acc_t = pto.gemm(ta, tb, torch.int32)
    # whole-matrix checksums, exact in int64: sum_j C[i][j] = A[i] . (sum_j B[j]) and sum_i C[i][j] = (sum_i A[i]) . B[j]
    row_sums = acc_t.sum(dim=1, dtype=torch.int64).cpu().numpy()
    col_sums = acc_t.sum(dim=0, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(row_sums, a.astype(np.int64) @ b.astype(np.int64).sum(axis=0))
    assert np.array_equal(col_sums, b.astype(np.int64) @ a.astype(np.int64).sum(axis=0))
    acc = host(acc_t)
    deq = host(pto.gemm_s8_dequant(ta, tb, dev8(s_row), dev8(s_col)))
    for r0, c0 in sample_tiles(m, n, 4, 32):
        ref = oracle.gemm_s8(a[r0:r0 + 128], b[c0:c0 + 256])
        assert np.array_equal(acc[r0:r0 + 128, c0:c0 + 256], ref)
        assert np.array_equal(deq[r0:r0 + 128, c0:c0 + 256],
                              oracle.dequant_bf16(ref, s_row[r0:r0 + 128], s_col[c0:c0 + 256], True))
    # the fused dequant store equals the oracle's store applied to the GPU's own accumulators, everywhere
    assert np.array_equal(deq[:1024], oracle.dequant_bf16(acc[:1024], s_row[:1024], s_col, True))


def test_split_last_wave_int8_exact():
    """4096 x 4096 leaves 34 tiles for the fourth wave on 74 CTA pairs; they are computed as two K halves. Integer
    accumulators must come out identical with and without the split."""
    m = n = 4096
    k = 1024
    a, b, s_row, s_col = gd.s8_inputs(m, n, k, 6)
    ta, tb = dev8(a), dev8(b)
    split = pto.gemm(ta, tb, torch.int32, workspace="auto")
    plain = pto.gemm(ta, tb, torch.int32, workspace=None)
    assert torch.equal(split, plain)
    row_sums = split.sum(dim=1, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(row_sums, a.astype(np.int64) @ b.astype(np.int64).sum(axis=0))
    # twice more on the same workspace: its counters must have been left clean
    for _ in range(2):
        assert torch.equal(pto.gemm(ta, tb, torch.int32, workspace="auto"), plain)


def test_c4_mxfp8_sampled_tiles():
    m, n, k = 16384, 8192, 8192
    # full-size inputs are quantised block by block from the counter-based generator
    xa = gd.normal((1024, k), 3, 0)
    a_blk, sfa_blk = gd.mx_quantize_e4m3(xa)
    xb = gd.normal((1024, k), 3, 1)
    b_blk, sfb_blk = gd.mx_quantize_e4m3(xb)
    ta = dev8(a_blk).repeat(m // 1024, 1)
    tsa = dev8(sfa_blk).repeat(m // 1024, 1)
    tb = dev8(b_blk).repeat(n // 1024, 1)
    tsb = dev8(sfb_blk).repeat(n // 1024, 1)
    # make the repeats differ: negate whole row blocks of A (sign bit of e4m3 bytes)
    for blk in range(1, m // 1024, 2):
        ta[blk * 1024:(blk + 1) * 1024] ^= 0x80
    out = pto.gemm_mx(ta, tb, tsa, tsb, torch.float32)
    a_h, sfa_h, b_h, sfb_h = host(ta), host(tsa), host(tb), host(tsb)
    out_h = host(out)
    for r0, c0 in sample_tiles(m, n, 4, 33):
        ref = oracle.gemm_mx(a_h[r0:r0 + 128], b_h[c0:c0 + 256], sfa_h[r0:r0 + 128], sfb_h[c0:c0 + 256])
        assert max_rel_err(out_h[r0:r0 + 128, c0:c0 + 256], ref) <= MX_TOL
        assert max_elem_rel_err(out_h[r0:r0 + 128, c0:c0 + 256], ref) <= MX_TOL
    # negating A's rows negates C's rows exactly; identical row blocks give identical results
    assert np.array_equal(out_h[0:1024], -out_h[1024:2048])
    assert np.array_equal(out_h[0:1024], out_h[2048:3072])


def test_c5_ksplit_slices_on_one_gpu():
    """K-split partials of configuration 5's shape class (strided K slices of A and B), summed in fp32."""
    m, n, k, ranks = 512, 1024, 8192, 4
    a, b = gd.dense_inputs(m, n, k, "bf16", 4)
    ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
    total = torch.zeros((m, n), dtype=torch.float32, device=DEV)
    kr = k // ranks
    for r in range(ranks):
        total += pto.gemm(ta[:, r * kr:(r + 1) * kr], tb[:, r * kr:(r + 1) * kr], torch.float32)
    out16 = host(pto.cast_f32_to_bf16(total))
    ref = oracle.gemm_f32acc(a[:128], b[:256], oracle.BF16)
    assert max_rel_err(host(total)[:128, :256], ref) <= DENSE_TOL
    assert np.array_equal(out16, gd.f32_to_bf16_bits(host(total)))
    unsplit = host(pto.gemm(ta, tb, torch.float32))
    assert max_rel_err(host(total), unsplit) <= DENSE_TOL


# ------------------------------------------------------------------ edges

@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (129, 257, 72), (128, 256, 64), (300, 40, 1000), (77, 513, 136)])
def test_ragged_edges_leave_padding_untouched(m, n, k):
    a, b = gd.dense_inputs(m, n, k, "bf16", 41)
    ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
    ref = oracle.gemm_f32acc(a, b, oracle.BF16)
    for out_dt in (torch.float32, torch.bfloat16):
        pitch = n + 5                                   # odd pitch: the scalar store path
        buf = torch.full((m + 2, pitch), -768.0, dtype=out_dt, device=DEV)
        view = buf[1:m + 1, :n]
        pto.gemm(ta, tb, out=view)
        got = buf.float().cpu().numpy()
        assert max_rel_err(got[1:m + 1, :n], ref) <= (DENSE_TOL if out_dt == torch.float32 else 8e-3)
        assert (got[0] == -768.0).all() and (got[m + 1] == -768.0).all() and (got[:, n:] == -768.0).all()


def test_wrapper_rejects_bad_arguments():
    a = torch.zeros((16, 12), dtype=torch.float16, device=DEV)     # 24-byte row pitch
    with pytest.raises(pto.PtoB200Error) as e:
        pto.gemm(a, a, torch.float32)
    assert e.value.code == 2
    with pytest.raises(ValueError):
        pto.gemm(a.float(), a.float())
    before = pto.launch_count()
    pto.gemm(torch.zeros((16, 16), dtype=torch.float16, device=DEV), torch.zeros((16, 16), dtype=torch.float16, device=DEV))
    assert pto.launch_count() == before + 1


def test_launch_is_asynchronous_on_the_given_stream():
    a, b = gd.dense_inputs(256, 256, 256, "bf16", 43)
    ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    out = pto.gemm(ta, tb, torch.float32, stream=s)
    s.synchronize()
    assert max_rel_err(out.cpu().numpy(), oracle.gemm_f32acc(a, b, oracle.BF16)) <= DENSE_TOL


def test_host_pipeline_matches_one_product_at_a_time():
    """HostGemmPipeline (copies of neighbouring products overlapped with the GEMM) returns the bits of HostGemm.run."""
    from pto_isa_mirror_b200.host_api import HostGemm, HostGemmPipeline

    m, n, k = 256, 512, 320
    pairs = []
    for i in range(7):
        a, b = gd.dense_inputs(m, n, k, "bf16", 50 + i)
        pairs.append((torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).pin_memory(),
                      torch.from_numpy(b.view(np.int16)).view(torch.bfloat16).pin_memory()))
    one = HostGemm(m, n, k, torch.bfloat16, torch.float32)
    want = [one.run(a, b).clone() for a, b in pairs]
    pipe = HostGemmPipeline(m, n, k, torch.bfloat16, torch.float32, depth=3)
    got = {}
    for i, (a, b) in enumerate(pairs):
        t = pipe.submit(a, b)
        assert t == i
        if t >= 2:
            got[t - 2] = pipe.result(t - 2).clone()
    for t in range(len(pairs) - 2, len(pairs)):
        got[t] = pipe.result(t).clone()
    for i in range(len(pairs)):
        assert torch.equal(got[i], want[i]), i
    ref = oracle.gemm_f32acc(gd.dense_inputs(m, n, k, "bf16", 50)[0], gd.dense_inputs(m, n, k, "bf16", 50)[1], oracle.BF16)
    assert max_rel_err(got[0].numpy(), ref) <= DENSE_TOL
    with pytest.raises(ValueError):
        pipe.result(0)                                              # overwritten four submissions ago


# ------------------------------------------------------------------ the CTA-pair kernel at depth, its store paths, fixed-shape launcher

def test_pair_kernel_at_k65536():
    """2304 x 2304 x 65536 bf16: 81 tiles of 256 x 256, more than the 74 CTA pairs, so the cta_group::2 kernel runs the
    depth of the K-split configuration unsplit (1024 k-blocks per tile, 170 wraps of its stage ring). The reference's
    own golden tile for K = 65536 sits at a tile position inside the matrix; two more tiles are checked against the
    oracle's sequential chain."""
    m = n = 2304
    k = 65536
    g = golden("bf16_tile_k65536")
    ga, gb = gd.dense_inputs(128, 256, k, "bf16", 4)
    gen = torch.Generator(device=DEV).manual_seed(65536)
    ta = (torch.randn((m, k), generator=gen, device=DEV) / 256.0).to(torch.bfloat16)
    tb = (torch.randn((n, k), generator=gen, device=DEV) / 256.0).to(torch.bfloat16)
    r0g, c0g = 384, 1280                 # second CTA of a pair in M, second tile half in N
    ta[r0g:r0g + 128] = dev16(ga, torch.bfloat16)
    tb[c0g:c0g + 256] = dev16(gb, torch.bfloat16)
    out32 = pto.gemm(ta, tb, torch.float32)
    out16 = pto.gemm(ta, tb, torch.bfloat16)
    o32, o16 = host(out32), host(out16)
    assert np.array_equal(o16, gd.f32_to_bf16_bits(o32))
    tile = o32[r0g:r0g + 128, c0g:c0g + 256]
    assert max_rel_err(tile, g["out"]) <= DENSE_TOL
    assert max_elem_rel_err(tile, g["out"]) <= DENSE_TOL
    a_h, b_h = host(ta), host(tb)
    for r0, c0 in ((0, 0), (2176, 2048)):
        ref = oracle.gemm_f32acc(a_h[r0:r0 + 128], b_h[c0:c0 + 256], oracle.BF16)
        assert max_rel_err(o32[r0:r0 + 128, c0:c0 + 256], ref) <= DENSE_TOL


def test_call_kernel_fixed_shape_launcher():
    """call_kernel(blockDim, stream, out, src0, src1): fp16 6144^3, B column-major, fp32 out, through the C ABI."""
    from pto_isa_mirror_b200 import _capi

    lib = _capi.load()
    dim = 6144
    gen = torch.Generator(device=DEV).manual_seed(6144)
    ta = (torch.randn((dim, dim), generator=gen, device=DEV) / dim ** 0.5).to(torch.float16)
    tb = (torch.randn((dim, dim), generator=gen, device=DEV) / dim ** 0.5).to(torch.float16)
    out = torch.full((dim, dim), float("nan"), dtype=torch.float32, device=DEV)
    before = lib.pto_b200_launch_count()
    lib.call_kernel(24, torch.cuda.current_stream().cuda_stream, out.data_ptr(), ta.data_ptr(), tb.data_ptr())
    assert lib.pto_b200_launch_count() == before + 1
    o = host(out)
    assert not np.isnan(o).any()
    a_h, b_h = host(ta), host(tb)
    for r0, c0 in sample_tiles(dim, dim, 2, 61):
        ref = oracle.gemm_f32acc(a_h[r0:r0 + 128], b_h[c0:c0 + 256], oracle.F16)
        assert max_rel_err(o[r0:r0 + 128, c0:c0 + 256], ref) <= DENSE_TOL


@pytest.mark.parametrize("kind", ["bf16", "f32", "s32", "deq", "mx"])
def test_pair_kernel_store_paths_agree(kind):
    """The CTA-pair kernel sends finished tiles through shared memory and TMA stores when C is 16-byte aligned with a
    16-byte pitch, and stores from registers otherwise. Both paths must write the same bits, ragged edges included,
    and leave everything around C untouched."""
    m, n, k = 2400, 2500, 256            # 10 x 10 tiles of 256 x 256 (ragged in both directions) on 74 pairs
    fill = -768.0
    if kind in ("bf16", "f32"):
        a, b = gd.dense_inputs(m, n, k, "bf16", 71)
        ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
        odt = torch.bfloat16 if kind == "bf16" else torch.float32
        run = lambda out: pto.gemm(ta, tb, out=out)  # noqa: E731
    elif kind in ("s32", "deq"):
        a, b, s_row, s_col = gd.s8_inputs(m, n, k, 72)
        ta, tb, sr, sc = dev8(a), dev8(b), dev8(s_row), dev8(s_col)
        odt = torch.int32 if kind == "s32" else torch.bfloat16
        fill = -768
        run = (lambda out: pto.gemm(ta, tb, out=out)) if kind == "s32" else (
            lambda out: pto.gemm_s8_dequant(ta, tb, sr, sc, out=out))
    else:
        a, b, sfa, sfb = gd.mx_inputs(m, n, k, 73)
        ta, tb, tsa, tsb = dev8(a), dev8(b), dev8(sfa), dev8(sfb)
        odt = torch.bfloat16
        run = lambda out: pto.gemm_mx(ta, tb, tsa, tsb, out=out)  # noqa: E731
    results = []
    # n + 12: 16-byte multiple for 2- and 4-byte elements (TMA); n + 5: odd pitch; n + 2 and n + 4: 16-bit rows that
    # start on 4- and 8-byte boundaries (the register path's narrower pieces)
    for pitch in (n + 12, n + 5, n + 2, n + 4):
        buf = torch.full((m + 2, pitch), fill, dtype=odt, device=DEV)
        run(buf[1:m + 1, :n])
        got = buf.cpu()
        assert (got[0] == fill).all() and (got[m + 1] == fill).all() and (got[:, n:] == fill).all()
        results.append(got[1:m + 1, :n].contiguous())
    for other in results[1:]:
        assert torch.equal(results[0].view(torch.uint8), other.view(torch.uint8))
    if kind == "s32":
        assert np.array_equal(results[0].numpy()[:128, :256], oracle.gemm_s8(a[:128], b[:256]))


def test_bounded_wait_expires_and_reports():
    """A wait that nothing satisfies gives up after the run-time limit: the kernel returns, the status word names the
    wait, reading it clears it, and the device goes on working. The wait is pto_b200_ksplit_wait on flags that nobody
    sets, with the limit lowered to about a millisecond; nothing traps and no kernel is left waiting."""
    import ctypes

    from pto_isa_mirror_b200 import _capi

    lib = _capi.load()
    flags = torch.zeros((4, 8), dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    old = lib.pto_b200_set_wait_limit(2_000_000)
    try:
        rc = lib.pto_b200_ksplit_wait(torch.cuda.current_stream().cuda_stream, flags.data_ptr(), 2, 0, 2, 1)
        assert rc == _capi.OK
        st = ctypes.c_int(0)
        assert lib.pto_b200_device_status(ctypes.byref(st)) == _capi.ETIMEOUT
        assert st.value == 17                                   # ST_KSPLIT_DONE_TIMEOUT
        assert lib.pto_b200_device_status(ctypes.byref(st)) == _capi.OK and st.value == 0
    finally:
        assert lib.pto_b200_set_wait_limit(old) == 2_000_000
    a, b = gd.dense_inputs(256, 256, 256, "bf16", 43)
    out = host(pto.gemm(dev16(a, torch.bfloat16), dev16(b, torch.bfloat16), torch.float32))
    assert max_rel_err(out, oracle.gemm_f32acc(a, b, oracle.BF16)) <= DENSE_TOL


@pytest.mark.parametrize("m,n,k", [(2560, 2560, 512), (130, 260, 160), (384, 128, 1056)])
def test_mx_pretiled_scales_match_the_one_call_form(m, n, k):
    """pto_b200_mx_retile_scales + pto_b200_gemm_mx_pretiled give the bits of pto_b200_gemm_mx, on the two-CTA kernel and
    on both tile widths of the one-CTA kernel (the re-tiled layout does not depend on the kernel that reads it)."""
    a, b, sfa, sfb = gd.mx_inputs(m, n, k, 91)
    ta, tb, tsa, tsb = dev8(a), dev8(b), dev8(sfa), dev8(sfb)
    want = pto.gemm_mx(ta, tb, tsa, tsb, torch.float32)
    tiled = pto.mx_retile_scales(tsa, tsb, k)
    before = pto.launch_count()
    got = pto.gemm_mx_pretiled(ta, tb, tiled, torch.float32)
    assert pto.launch_count() == before + 1
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    ref = oracle.gemm_mx(a[:128], b[:128], sfa[:128], sfb[:128])
    assert max_rel_err(host(got)[:128, :128], ref) <= MX_TOL


# ------------------------------------------------------------------ MXFP4 (float4_e2m1x2_t operands, e8m0 block scales)

def test_mxfp4_golden_tile_exact():
    """The reference's own outputs for a 128 x 256 x 256 fp4 tile: every sum is exact in fp32, so the bits must match."""
    g = golden("mxfp4_tile_k256")
    out = pto.gemm_mx(dev8(g["a"]), dev8(g["b"]), dev8(g["sfa"]), dev8(g["sfb"]), torch.float32, pto.E2M1, pto.E2M1)
    assert np.array_equal(host(out), g["out"])


@pytest.mark.parametrize("m,n,k", [(2560, 2560, 512), (2040, 2500, 384), (300, 520, 1152)])
def test_mxfp4_against_the_oracle(m, n, k):
    """Random 4-bit codes with scales 2^-1..2^1 on the two-CTA kernel (100 tiles; 80 ragged ones) and on a ragged one-CTA shape: exact
    against the oracle's chain on sampled rows; the bf16 store is the RNE cast of the fp32 result."""
    a = gd.randint((m, k // 2), 0, 255, 31, 0).astype(np.uint8)
    b = gd.randint((n, k // 2), 0, 255, 31, 1).astype(np.uint8)
    sfa = gd.randint((m, k // 32), 126, 128, 31, 2).astype(np.uint8)
    sfb = gd.randint((n, k // 32), 126, 128, 31, 3).astype(np.uint8)
    out = host(pto.gemm_mx(dev8(a), dev8(b), dev8(sfa), dev8(sfb), torch.float32, pto.E2M1, pto.E2M1))
    for r0 in (0, m - 128):
        ref = oracle.gemm_mx(a[r0:r0 + 128], b, sfa[r0:r0 + 128], sfb, oracle.E2M1, oracle.E2M1)
        assert np.array_equal(out[r0:r0 + 128], ref)
    out16 = host(pto.gemm_mx(dev8(a), dev8(b), dev8(sfa), dev8(sfb), torch.bfloat16, pto.E2M1, pto.E2M1))
    assert np.array_equal(out16, gd.f32_to_bf16_bits(out))


def test_mxfp4_rejects_mixed_and_misaligned_operands():
    a = torch.zeros((128, 64), dtype=torch.uint8, device=DEV)
    s = torch.full((128, 4), 127, dtype=torch.uint8, device=DEV)
    with pytest.raises(pto.PtoB200Error) as e:
        b8 = torch.zeros((128, 128), dtype=torch.uint8, device=DEV)
        pto.gemm_mx(a, b8, s, s, torch.float32, pto.E2M1, pto.E4M3)      # fp4 x fp8 is not in CheckMadMxValid's table
    assert e.value.code == 3
    with pytest.raises(pto.PtoB200Error) as e:
        pto.gemm_mx(a[:, :48], a[:, :48], s[:, :3], s[:, :3], torch.float32, pto.E2M1, pto.E2M1)   # K = 96
    assert e.value.code in (1, 2)


# ------------------------------------------------------------------ the largest index ranges

@pytest.mark.parametrize("kind", ["bf16", "s8"])
def test_output_beyond_two_to_the_31_elements(kind):
    """49152 x 49152 outputs (2.4e9 elements, 36 864 tiles): element offsets into C pass 2^31, so every offset the
    store path forms must be 64-bit. Small integers keep every sum exact; tiles at the far corners, in the middle and
    around the 2^31-th element are compared with the oracle's chain."""
    m = n = 49152
    k = 128
    if kind == "bf16":
        a = gd.f32_to_bf16_bits(gd.randint((m, k), -4, 4, 81, 0).astype(np.float32))
        b = gd.f32_to_bf16_bits(gd.randint((n, k), -4, 4, 81, 1).astype(np.float32))
        ta, tb = dev16(a, torch.bfloat16), dev16(b, torch.bfloat16)
        out = pto.gemm(ta, tb, torch.bfloat16)
        ref_tile = lambda r0, c0: gd.f32_to_bf16_bits(oracle.gemm_f32acc(a[r0:r0 + 128], b[c0:c0 + 256], oracle.BF16))  # noqa: E731
        got_tile = lambda r0, c0: host(out[r0:r0 + 128, c0:c0 + 256].contiguous())  # noqa: E731
    else:
        a, b, _, _ = gd.s8_inputs(m, n, k, 82)
        ta, tb = dev8(a), dev8(b)
        out = pto.gemm(ta, tb, torch.int32)                      # int32 accumulators
        ref_tile = lambda r0, c0: oracle.gemm_s8(a[r0:r0 + 128], b[c0:c0 + 256])  # noqa: E731
        got_tile = lambda r0, c0: host(out[r0:r0 + 128, c0:c0 + 256].contiguous())  # noqa: E731
    assert out.numel() > 2 ** 31
    row_2_31 = (2 ** 31) // n                                    # the row that holds element 2^31
    for r0, c0 in ((0, 0), (m - 128, n - 256), (m - 128, 0), (0, n - 256), (24576, 24576),
                   (row_2_31 - 64, 33792), (row_2_31 - 64, 0)):
        assert np.array_equal(got_tile(r0, c0), ref_tile(r0, c0)), (r0, c0)
    del out
    torch.cuda.empty_cache()
