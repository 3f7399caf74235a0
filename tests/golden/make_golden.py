"""Generate the golden fixtures under tests/golden/ by running the REFERENCE CPU simulator (oracle/_ref).

Run where the reference tree is mounted:  make -C oracle && python tests/golden/make_golden.py [name fragment ...]
(with fragments only the fixtures whose file name contains one of them are rewritten).
Inputs are not stored: they are regenerated from pto_isa_mirror_b200.gen_data with the seeds below, and each
fixture carries the SHA-256 of its input bytes so a drifting generator is caught. Outputs are the reference's.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from pto_isa_mirror_b200 import gen_data as gd  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


ONLY = sys.argv[1:]  # name fragments; empty = every fixture


def wanted(name) -> bool:
    return not ONLY or any(frag in name for frag in ONLY)


def save(name, **kw):
    if not wanted(name):
        return
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **kw)
    print("wrote", name, {k: getattr(v, "shape", v) for k, v in kw.items()})


def main():
    ref = oracle.Ref()
    assert ref.has_real_bf16()

    # C1: fp16 128 x 256 x 256, uniform[-1, 1), seed 0 (RunGemmE2E<float, half, half, ...>)
    a, b = gd.dense_inputs(128, 256, 256, "f16", 0, "uniform")
    save("c1_f16_k256", out=ref.tile_f16(a, b), input_sha=sha(a, b), seed=0)

    # the reference's exactness style: small integers (tests/cpu/st/testcase/tmatmul/gen_data.py:43-45)
    ai = gd.randint((128, 1024), 1, 5, 19, 0).astype(np.float16).view(np.uint16)
    bi = gd.randint((256, 1024), 1, 5, 19, 1).astype(np.float16).view(np.uint16)
    save("f16_randint_k1024", out=ref.tile_f16(ai, bi), input_sha=sha(ai, bi), seed=19)

    # C2 / C5 sampled tiles: bf16 values through the float path, full K of the configuration
    for k, seed in ((1024, 1), (4096, 1), (8192, 4), (65536, 4)):
        a, b = gd.dense_inputs(128, 256, k, "bf16", seed)
        out = ref.tile_f32(gd.bf16_bits_to_f32(a), gd.bf16_bits_to_f32(b))
        out_bf16 = np.array([ref.lib.ref_cast_bf16(float(v)) for v in out.ravel()], dtype=np.uint16).reshape(out.shape)
        save(f"bf16_tile_k{k}", out=out, out_bf16=out_bf16, input_sha=sha(a, b), seed=seed)

    # C3 sampled tile: int8, exact int32 accumulators + the dequantised bf16 store
    for k in (1024, 8192):
        a, b, s_row, s_col = gd.s8_inputs(128, 256, k, 2)
        acc = ref.tile_s8(a, b)
        deq = np.empty(acc.shape, dtype=np.uint16)
        for i in range(acc.shape[0]):
            for j in range(acc.shape[1]):
                t = np.float32(ref.lib.ref_dequant_col(int(acc[i, j]), float(s_col[j])))
                deq[i, j] = ref.lib.ref_cast_bf16(float(np.float32(t * s_row[i])))
        save(f"s8_tile_k{k}", acc=acc, deq_bf16=deq, input_sha=sha(a, b, s_row, s_col), seed=2)

    # C4 sampled tile: MXFP8 e4m3 with e8m0 block scales, inputs through the reference's OCP quantiser
    for k in (256, 8192):
        xa = gd.normal((128, k), 3, 0)
        xb = gd.normal((256, k), 3, 1)
        a, sfa = ref.mx_quantize_e4m3(xa)
        b, sfb = ref.mx_quantize_e4m3(xb)
        save(f"mx_tile_k{k}", out=ref.tile_mx(a, b, sfa, sfb), a_sha=sha(a, sfa), b_sha=sha(b, sfb), seed=3)

    # the reference's MX exactness style: integers in [-10, 10], scales 2^0..2^2, mixed e4m3 x e5m2
    ai = gd.randint((128, 256), -10, 10, 19, 2).astype(np.float32)
    bi = gd.randint((256, 256), -10, 10, 19, 3).astype(np.float32)
    a8 = gd.encode_e4m3fn(ai)
    import ml_dtypes

    b8 = bi.astype(ml_dtypes.float8_e5m2).view(np.uint8)
    sfa = gd.randint((128, 8), 127, 129, 19, 4).astype(np.uint8)
    sfb = gd.randint((256, 8), 127, 129, 19, 5).astype(np.uint8)
    save("mx_randint_e4m3_e5m2_k256", out=ref.tile_mx(a8, b8, sfa, sfb, oracle.E4M3, oracle.E5M2), a=a8, b=b8, sfa=sfa,
         sfb=sfb)

    # MXFP4: float4_e2m1x2_t operands (every 4-bit code occurs), two per byte, e8m0 scales 2^-2..2^3
    if wanted("mxfp4"):
        a4 = gd.randint((128, 128), 0, 255, 29, 0).astype(np.uint8)       # [128, K/2] bytes, K = 256
        b4 = gd.randint((256, 128), 0, 255, 29, 1).astype(np.uint8)
        sfa4 = gd.randint((128, 8), 125, 130, 29, 2).astype(np.uint8)
        sfb4 = gd.randint((256, 8), 125, 130, 29, 3).astype(np.uint8)
        save("mxfp4_tile_k256", out=ref.tile_mx(a4, b4, sfa4, sfb4, oracle.E2M1, oracle.E2M1), a=a4, b=b4, sfa=sfa4,
             sfb=sfb4)

    # bias forms: TMATMUL_BIAS on the first chunk then TMATMUL_ACC (fp16 and int8), six-operand TMATMUL_MX
    if wanted("bias"):
        a, b = gd.dense_inputs(128, 256, 256, "f16", 7, "uniform")
        bias = (gd.normal((256,), 8) * np.float32(3.0)).astype(np.float32)
        save("f16_bias_k256", out=ref.tile_f16_bias(a, b, bias), bias=bias, input_sha=sha(a, b), seed=7)
        a, b, _, _ = gd.s8_inputs(128, 256, 1024, 2)
        bias_i = gd.randint((256,), -100000, 100000, 9, 0).astype(np.int32)
        save("s8_bias_k1024", out=ref.tile_s8_bias(a, b, bias_i), bias=bias_i, input_sha=sha(a, b), seed=2)
        a, sfa = ref.mx_quantize_e4m3(gd.normal((128, 256), 3, 0))
        b, sfb = ref.mx_quantize_e4m3(gd.normal((256, 256), 3, 1))
        save("mx_bias_k256", out=ref.tile_mx_bias(a, b, sfa, sfb, bias), bias=bias, a_sha=sha(a, sfa),
             b_sha=sha(b, sfb), seed=3)

    # TSTORE with a pre-quant scale word (scalar form: fp32 in bits [31:0]; vector form: one word per column, the
    # simulator reads bits [31:13]) on the int8 tile's int32 accumulators and on configuration 1's float accumulators
    if wanted("quant_store"):
        acc_i = np.load(os.path.join(HERE, "s8_tile_k1024.npz"))["acc"]
        acc_f = np.load(os.path.join(HERE, "c1_f16_k256.npz"))["out"] * np.float32(3000.0)
        scalar_word = np.array([np.float32(0.00314159)]).view(np.uint32).astype(np.uint64)
        col = gd.uniform((256,), 1e-3, 1e-2, 12, 0)          # full-precision scales: the truncation to 19 bits shows
        col[7] = -col[7]
        vector_words = col.view(np.uint32).astype(np.uint64)
        save("quant_store",
             scalar_word=scalar_word, vector_words=vector_words,
             s32_scalar_bf16=ref.quant_store(acc_i, scalar_word, False),
             s32_vector_bf16=ref.quant_store(acc_i, vector_words, True),
             s32_vector_bf16_relu=ref.quant_store(acc_i, vector_words, True, relu=True),
             s32_scalar_f16=ref.quant_store(acc_i, scalar_word, False, out_f16=True),
             s32_vector_f16_relu=ref.quant_store(acc_i, vector_words, True, relu=True, out_f16=True),
             f32_scalar_bf16=ref.quant_store(acc_f, scalar_word, False),
             f32_vector_bf16_relu=ref.quant_store(acc_f, vector_words, True, relu=True),
             f32_vector_f16=ref.quant_store(acc_f, vector_words, True, out_f16=True),
             f32_scalar_f16_relu=ref.quant_store(acc_f, scalar_word, False, relu=True, out_f16=True))

    # the 8-bit destinations of the pre-quant store (REQ8 / VREQ8 on int32, QF322B8_PRE / VQF322B8_PRE on float
    # accumulators): offset field, signed and unsigned clamp ranges, ReLU, exact .5 ties and saturation at both ends
    if wanted("quant_store_b8"):
        acc_i = np.load(os.path.join(HERE, "s8_tile_k1024.npz"))["acc"]
        acc_f = np.load(os.path.join(HERE, "c1_f16_k256.npz"))["out"] * np.float32(3000.0)
        ramp_i = (np.arange(128 * 256, dtype=np.int32).reshape(128, 256) % 1201) - 600
        ramp_f = ramp_i.astype(np.float32) * np.float32(0.25)

        def word(scale, offset, signed):
            return (np.array([np.float32(scale)]).view(np.uint32).astype(np.uint64) | (np.uint64(offset) << np.uint64(37))
                    | (np.uint64(signed) << np.uint64(46)))

        s_i = float(100.0 / np.abs(acc_i).max())
        s_f = float(100.0 / np.abs(acc_f).max())
        col = gd.uniform((256,), 0.5, 1.5, 13, 0)
        offs = (np.arange(256) % 9).astype(np.uint64)
        sign = (np.arange(256) % 3 != 0).astype(np.uint64)
        vec_i = ((col * np.float32(s_i)).astype(np.float32).view(np.uint32).astype(np.uint64) | (offs << np.uint64(37))
                 | (sign << np.uint64(46)))
        vec_f = ((col * np.float32(s_f)).astype(np.float32).view(np.uint32).astype(np.uint64) | (offs << np.uint64(37))
                 | (sign << np.uint64(46)))
        w_si, w_ui = word(s_i, 0, 1), word(s_i, 128, 0)
        w_sf, w_uf = word(s_f, 3, 1), word(s_f, 100, 0)
        w_half_s, w_half_u = word(0.5, 0, 1), word(0.5, 7, 0)
        save("quant_store_b8", ramp_i=ramp_i, ramp_f=ramp_f, w_si=w_si, w_ui=w_ui, w_sf=w_sf, w_uf=w_uf, vec_i=vec_i,
             vec_f=vec_f, w_half_s=w_half_s, w_half_u=w_half_u,
             s32_scalar_s8=ref.quant_store(acc_i, w_si, False, out_f16=2),
             s32_scalar_u8_relu=ref.quant_store(acc_i, w_ui, False, relu=True, out_f16=3),
             s32_vector_s8=ref.quant_store(acc_i, vec_i, True, out_f16=2),
             s32_vector_s8_relu=ref.quant_store(acc_i, vec_i, True, relu=True, out_f16=2),
             f32_scalar_s8=ref.quant_store(acc_f, w_sf, False, out_f16=2),
             f32_scalar_u8=ref.quant_store(acc_f, w_uf, False, out_f16=3),
             f32_vector_u8=ref.quant_store(acc_f, vec_f, True, out_f16=3),
             ramp_i_s8=ref.quant_store(ramp_i, w_half_s, False, out_f16=2),
             ramp_i_u8=ref.quant_store(ramp_i, w_half_u, False, out_f16=3),
             ramp_f_s8=ref.quant_store(ramp_f, w_half_s, False, out_f16=2))

    # the int16 destination of the pre-quant store (SHIFTS322S16 / VSHIFTS322S16): arithmetic shift by 1 + bits [35:32],
    # the wrapping cast to int16, ReLU
    if wanted("quant_store_s16"):
        acc_i = np.load(os.path.join(HERE, "s8_tile_k1024.npz"))["acc"]
        w_shift = np.array([np.uint64(6) << np.uint64(32)], dtype=np.uint64)            # >> 7: wraps for |acc| > 2^22
        vec_shift = ((np.arange(256) % 16).astype(np.uint64) << np.uint64(32)) | np.uint64(0x12345)
        save("quant_store_s16", w_shift=w_shift, vec_shift=vec_shift,
             s32_scalar_s16=ref.quant_store(acc_i, w_shift, False, out_f16=4),
             s32_scalar_s16_relu=ref.quant_store(acc_i, w_shift, False, relu=True, out_f16=4),
             s32_vector_s16=ref.quant_store(acc_i, vec_shift, True, out_f16=4),
             s32_vector_s16_relu=ref.quant_store(acc_i, vec_shift, True, relu=True, out_f16=4))

    # scalar tables: store casts, fp8 / e8m0 decode, quantiser
    x = np.concatenate([gd.normal((4096,), 5) * np.float32(3.0),
                        np.array([0, -0.0, 65504, 65519.9, 65520, 1e-8, 5.96e-8, 2.98e-8, 3e-8, 6.1e-5, 1e38, -1e38,
                                  1.00390625, 1.01171875], dtype=np.float32)])
    save("store_casts", x=x, bf16=np.array([ref.lib.ref_cast_bf16(float(v)) for v in x], dtype=np.uint16),
         f16=np.array([ref.lib.ref_cast_f16(float(v)) for v in x], dtype=np.uint16))
    save("fp8_decode", e4m3=np.array([ref.lib.ref_fp8_to_double(i, 5) for i in range(256)]),
         e5m2=np.array([ref.lib.ref_fp8_to_double(i, 6) for i in range(256)]),
         e8m0=np.array([ref.lib.ref_e8m0_to_double(i) for i in range(256)]))
    src = gd.normal((64, 256), 6)
    src[0, :32] = 0
    src[1, :32] *= 1e-30
    src[2, :32] *= 1e30
    src[3, 5] = -1e-9
    d, s = ref.mx_quantize_e4m3(src)
    save("mx_quantize", src=src, data=d, scales=s)
    # the NV scale rule (QuantScaleAlg::NV): power-of-two maxima (no round-up), the -2^-10 tie, tiny negatives that keep
    # their sign, a range of block magnitudes
    if wanted("mx_quantize_nv"):
        src = gd.normal((64, 256), 16)
        src[0, :32] = 0
        src[1, :32] *= 1e-30
        src[2, :32] *= 1e30
        src[3, 5] = -1e-9
        src[4, :32] = np.float32(448.0) * np.float32(2.0) ** np.arange(-16, 16)
        src[5, :32] = np.float32(-(2.0 ** -10))
        src[5, 0] = np.float32(1.0)
        src[6, :32] = np.linspace(-1, 1, 32).astype(np.float32) * np.float32(2.0 ** -12)
        src[6, 31] = np.float32(448.0)
        for i in range(8, 40):
            src[i, :32] *= np.float32(2.0) ** (i - 24)
        d, s = ref.mx_quantize_e4m3(src, 1)
        save("mx_quantize_nv", src=src, data=d, scales=s)
    # TQUANT to MXFP4 (float4_e2m1x2_t) under both scale rules: zero and tiny blocks, huge values, every rounding tie
    # of the e2m1 grid in both signs, maxima just below and on a power of two (the OCP rule truncates them to bf16), a
    # range of block magnitudes
    if wanted("mxfp4_quantize"):
        src = gd.normal((64, 256), 17)
        src[0, :32] = 0
        src[1, :32] *= 1e-30
        src[2, :32] *= 1e30
        src[3, 5] = -1e-9
        ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0], dtype=np.float32)
        src[4, :32] = np.concatenate([ties, -ties, ties * np.float32(0.999), -ties * np.float32(1.001)])
        src[5, :32] = np.float32(6.0) * np.float32(2.0) ** np.arange(-16, 16)
        src[6, :32] = np.linspace(-1, 1, 32).astype(np.float32)
        src[6, 31] = np.float32(1.9999999)          # truncates to 1.9921875 in bf16: the OCP exponent stays 127
        src[7, :32] = np.linspace(-1, 1, 32).astype(np.float32)
        src[7, 0] = np.float32(-4.0)
        for i in range(8, 40):
            src[i, :32] *= np.float32(2.0) ** (i - 24)
        d0, s0 = ref.mx_quantize_e2m1(src, 0)
        d1, s1 = ref.mx_quantize_e2m1(src, 1)
        save("mxfp4_quantize", src=src, data_ocp=d0, scales_ocp=s0, data_nv=d1, scales_nv=s1)


if __name__ == "__main__":
    main()
