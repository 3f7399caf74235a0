/*
 * pto_gemm_oracle.c - plain C restatement of the PTO CPU simulator's GEMM arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY (see pto_gemm_oracle.h). Parity pinned against the reference simulator compiled
 * from its own headers (oracle/_ref) and the fixtures under tests/golden/.
 *
 * The element order of every accumulation follows the simulator exactly; only the loop nest around it is
 * rearranged (rows across threads, columns innermost) so that the independent per-element chains vectorise.
 */
#define _GNU_SOURCE
#include "pto_gemm_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------------ scalar conversions */

static inline float bits_to_float(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint32_t float_to_bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

float pto_oracle_half_to_float(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) {
            return bits_to_float(sign);
        }
        const float v = ldexpf((float)man, -24);
        return sign ? -v : v;
    }
    if (exp == 31) {
        return bits_to_float(sign | 0x7F800000u | (man << 13));
    }
    return bits_to_float(sign | ((exp + 112u) << 23) | (man << 13));
}

float pto_oracle_bf16_to_float(uint16_t h) { return bits_to_float((uint32_t)h << 16); }

/* static_cast<bfloat16_t>(float): round to nearest, ties to even (include/pto/cpu/common.hpp:187-198). */
uint16_t pto_oracle_float_to_bf16(float f)
{
    uint32_t u = float_to_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* static_cast<half>(float): round to nearest, ties to even, overflow to infinity. */
uint16_t pto_oracle_float_to_half(float f)
{
    const uint32_t u = float_to_bits(f);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t abs = u & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) {
        return (uint16_t)(sign | 0x7E00u);
    }
    if (abs >= 0x47800000u) { /* >= 65536: inf (65520 and up also round to inf below) */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (abs < 0x33000000u) { /* < 2^-25 rounds to zero */
        return sign;
    }
    const int e = (int)(abs >> 23) - 127;
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half: value = man * 2^(e-23), unit 2^-24 */
        shift = -e - 1; /* 13 + (-14 - e) */
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half_ulp = 1u << (shift - 1);
    if (rem > half_ulp || (rem == half_ulp && (q & 1u))) {
        q += 1;
    }
    return (uint16_t)(sign | (base + q)); /* a mantissa carry walks into the exponent, up to inf */
}

double pto_oracle_fp8_to_double(uint8_t raw, int fmt);

/* float4_e2m1x2_t (include/pto/cpu/MXTypes.hpp:316-332, decode :254-274): one sign, two exponent (bias 1) and one
   mantissa bit per 4-bit code: 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives. */
static double e2m1_to_double(unsigned nibble)
{
    static const double mag[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
    const double v = mag[nibble & 7u];
    return (nibble & 8u) ? -v : v;
}

/* Element kk of row `row` of an MX operand: one byte per element for fp8; for ORACLE_E2M1 two elements per byte, the
   even one in the low nibble (GetProperDataPart, include/pto/cpu/MXTypes.hpp:351-359), ld counted in elements. */
static double mx_element(const uint8_t* base, long long row, long long ld, int kk, int fmt)
{
    if (fmt == ORACLE_E2M1) {
        const uint8_t byte = base[(size_t)row * (size_t)(ld / 2) + (size_t)(kk / 2)];
        return e2m1_to_double((kk & 1) ? (unsigned)(byte >> 4) : (unsigned)(byte & 0xFu));
    }
    return pto_oracle_fp8_to_double(base[(size_t)row * (size_t)ld + (size_t)kk], fmt);
}

/* include/pto/cpu/MXTypes.hpp:232-252 */
double pto_oracle_fp8_to_double(uint8_t raw, int fmt)
{
    if (fmt == ORACLE_E2M1) {
        return e2m1_to_double(raw & 0xFu);
    }
    const int sign = raw >> 7;
    const int mag = raw & 0x7F;
    double v;
    if (fmt == ORACLE_E5M2) {
        const int exp = (mag >> 2) & 0x1F;
        const int man = mag & 3;
        if (mag > 0x7C) {
            return NAN;
        }
        if (mag == 0x7C) {
            return sign ? -INFINITY : INFINITY;
        }
        v = (exp == 0) ? ldexp((double)man, 1 - 15 - 2) : ldexp((double)(4 + man), exp - 15 - 2);
    } else {
        const int exp = (mag >> 3) & 0xF;
        const int man = mag & 7;
        if (mag == 0x7F) {
            return NAN;
        }
        v = (exp == 0) ? ldexp((double)man, 1 - 7 - 3) : ldexp((double)(8 + man), exp - 7 - 3);
    }
    return sign ? -v : v;
}

/* e8m0: 2^(raw - 127) for every raw byte (the generic decode has no NaN case; cpu/MXTypes.hpp:256-259). */
double pto_oracle_e8m0_to_double(uint8_t raw) { return ldexp(1.0, (int)raw - 127); }

/* ------------------------------------------------------------------ row-parallel driver */

typedef void (*row_fn)(void* ctx, int row_begin, int row_end);

typedef struct {
    row_fn fn;
    void* ctx;
    int begin, end;
} row_task;

static void* row_thread(void* arg)
{
    row_task* t = (row_task*)arg;
    t->fn(t->ctx, t->begin, t->end);
    return NULL;
}

static int resolve_threads(int threads, int rows)
{
    if (threads <= 0) {
        long n = sysconf(_SC_NPROCESSORS_ONLN);
        threads = n > 0 ? (int)n : 1;
    }
    if (threads > rows) {
        threads = rows;
    }
    if (threads > 256) {
        threads = 256;
    }
    return threads < 1 ? 1 : threads;
}

static void parallel_rows(row_fn fn, void* ctx, int rows, int threads)
{
    threads = resolve_threads(threads, rows);
    if (threads == 1) {
        fn(ctx, 0, rows);
        return;
    }
    pthread_t tid[256];
    row_task task[256];
    const int chunk = (rows + threads - 1) / threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        task[t].fn = fn;
        task[t].ctx = ctx;
        task[t].begin = t * chunk;
        task[t].end = (t + 1) * chunk < rows ? (t + 1) * chunk : rows;
        if (task[t].begin >= task[t].end) {
            break;
        }
        if (pthread_create(&tid[t], NULL, row_thread, &task[t]) != 0) {
            fn(ctx, task[t].begin, task[t].end);
            tid[t] = 0;
        }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t) {
        if (tid[t]) {
            pthread_join(tid[t], NULL);
        }
    }
}

/* ------------------------------------------------------------------ dense fp32-accumulate GEMM */

#define JBLOCK 256

typedef struct {
    const float* a; /* m x k, converted to float */
    const float* bt; /* k x n, converted to float, row-major */
    float* c;
    int n, k;
    long long ldc;
    const float* bias; /* per column, or NULL */
    int bias_after_k;  /* the bias joins the chain after this many k (the first TMATMUL_BIAS chunk) */
} dense_ctx;

/* acc[j] = fmaf(a, b[j], acc[j]) for one k; fused, single rounding, like std::fma in TMatmulNzZn. */
#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) static void fma_row_hw(float* acc, const float* b, float a, int n)
{
    for (int j = 0; j < n; ++j) {
        acc[j] = __builtin_fmaf(a, b[j], acc[j]);
    }
}
#endif

static void fma_row_sw(float* acc, const float* b, float a, int n)
{
    for (int j = 0; j < n; ++j) {
        acc[j] = fmaf(a, b[j], acc[j]);
    }
}

static int have_hw_fma(void)
{
#if defined(__x86_64__)
    return __builtin_cpu_supports("fma") && __builtin_cpu_supports("avx2");
#else
    return 0;
#endif
}

static void dense_rows(void* vctx, int r0, int r1)
{
    const dense_ctx* x = (const dense_ctx*)vctx;
    const int hw = have_hw_fma();
    float acc[JBLOCK];
    for (int i = r0; i < r1; ++i) {
        const float* arow = x->a + (size_t)i * x->k;
        for (int j0 = 0; j0 < x->n; j0 += JBLOCK) {
            const int jn = x->n - j0 < JBLOCK ? x->n - j0 : JBLOCK;
            for (int j = 0; j < jn; ++j) {
                acc[j] = 0.0f;
            }
            for (int kk = 0; kk < x->k; ++kk) {
                const float* brow = x->bt + (size_t)kk * x->n + j0;
#if defined(__x86_64__)
                if (hw) {
                    fma_row_hw(acc, brow, arow[kk], jn);
                } else
#endif
                {
                    fma_row_sw(acc, brow, arow[kk], jn);
                }
                if (x->bias && kk + 1 == x->bias_after_k) {
                    /* TMATMUL_BIAS: the finished first chunk, then += bias per column (cpu/TMatmul.hpp:223-229) */
                    for (int j = 0; j < jn; ++j) {
                        acc[j] += x->bias[j0 + j];
                    }
                }
            }
            memcpy(x->c + (size_t)i * x->ldc + j0, acc, (size_t)jn * sizeof(float));
        }
    }
}

static float load_as_float(const void* base, size_t idx, int dtype)
{
    switch (dtype) {
        case ORACLE_F16:
            return pto_oracle_half_to_float(((const uint16_t*)base)[idx]);
        case ORACLE_BF16:
            return pto_oracle_bf16_to_float(((const uint16_t*)base)[idx]);
        default:
            return ((const float*)base)[idx];
    }
}

void pto_oracle_gemm_f32acc(const void* a, const void* b, float* c, int m, int n, int k, long long lda,
                            long long ldb, long long ldc, int in_dtype, int b_layout, int threads)
{
    pto_oracle_gemm_f32acc_bias(a, b, NULL, 0, c, m, n, k, lda, ldb, ldc, in_dtype, b_layout, threads);
}

void pto_oracle_gemm_f32acc_bias(const void* a, const void* b, const float* bias, int bias_after_k, float* c, int m,
                                 int n, int k, long long lda, long long ldb, long long ldc, int in_dtype,
                                 int b_layout, int threads)
{
    if (m <= 0 || n <= 0 || k <= 0) {
        return;
    }
    if (bias_after_k <= 0 || bias_after_k > k) {
        bias_after_k = k;
    }
    float* af = (float*)malloc((size_t)m * k * sizeof(float));
    float* bt = (float*)malloc((size_t)k * n * sizeof(float));
    if (!af || !bt) {
        free(af);
        free(bt);
        return;
    }
    /* operands are cast to the accumulator type before the fma (cpu/TMatmul.hpp:101-102) */
    for (int i = 0; i < m; ++i) {
        for (int kk = 0; kk < k; ++kk) {
            af[(size_t)i * k + kk] = load_as_float(a, (size_t)i * lda + kk, in_dtype);
        }
    }
    if (b_layout == ORACLE_B_DN) {
        for (int j = 0; j < n; ++j) {
            for (int kk = 0; kk < k; ++kk) {
                bt[(size_t)kk * n + j] = load_as_float(b, (size_t)j * ldb + kk, in_dtype);
            }
        }
    } else {
        for (int kk = 0; kk < k; ++kk) {
            for (int j = 0; j < n; ++j) {
                bt[(size_t)kk * n + j] = load_as_float(b, (size_t)kk * ldb + j, in_dtype);
            }
        }
    }
    dense_ctx x = {af, bt, c, n, k, ldc, bias, bias_after_k};
    parallel_rows(dense_rows, &x, m, threads);
    free(af);
    free(bt);
}

/* ------------------------------------------------------------------ int8 GEMM */

typedef struct {
    const int8_t* a;
    const int32_t* bt; /* k x n widened */
    int32_t* c;
    int n, k;
    long long lda, ldc;
    const int32_t* bias; /* per column, or NULL; integer addition commutes, so its place in the chain is free */
} s8_ctx;

static void s8_rows(void* vctx, int r0, int r1)
{
    const s8_ctx* x = (const s8_ctx*)vctx;
    int32_t acc[JBLOCK];
    for (int i = r0; i < r1; ++i) {
        const int8_t* arow = x->a + (size_t)i * x->lda;
        for (int j0 = 0; j0 < x->n; j0 += JBLOCK) {
            const int jn = x->n - j0 < JBLOCK ? x->n - j0 : JBLOCK;
            memset(acc, 0, sizeof(acc));
            for (int kk = 0; kk < x->k; ++kk) {
                const int32_t av = arow[kk];
                const int32_t* brow = x->bt + (size_t)kk * x->n + j0;
                for (int j = 0; j < jn; ++j) {
                    acc[j] += av * brow[j];
                }
            }
            if (x->bias) {
                for (int j = 0; j < jn; ++j) {
                    acc[j] = (int32_t)((uint32_t)acc[j] + (uint32_t)x->bias[j0 + j]);
                }
            }
            memcpy(x->c + (size_t)i * x->ldc + j0, acc, (size_t)jn * sizeof(int32_t));
        }
    }
}

void pto_oracle_gemm_s8(const int8_t* a, const int8_t* b, int32_t* c, int m, int n, int k, long long lda,
                        long long ldb, long long ldc, int threads)
{
    pto_oracle_gemm_s8_bias(a, b, NULL, c, m, n, k, lda, ldb, ldc, threads);
}

void pto_oracle_gemm_s8_bias(const int8_t* a, const int8_t* b, const int32_t* bias, int32_t* c, int m, int n, int k,
                             long long lda, long long ldb, long long ldc, int threads)
{
    if (m <= 0 || n <= 0 || k <= 0) {
        return;
    }
    int32_t* bt = (int32_t*)malloc((size_t)k * n * sizeof(int32_t));
    if (!bt) {
        return;
    }
    for (int j = 0; j < n; ++j) {
        for (int kk = 0; kk < k; ++kk) {
            bt[(size_t)kk * n + j] = b[(size_t)j * ldb + kk];
        }
    }
    s8_ctx x = {a, bt, c, n, k, lda, ldc, bias};
    parallel_rows(s8_rows, &x, m, threads);
    free(bt);
}

/* ------------------------------------------------------------------ MX block-scaled GEMM */

typedef struct {
    const uint8_t* a;
    const uint8_t* sfa;
    const double* bt; /* k x n, element times its block scale (exact in double) */
    float* c;
    int n, k, a_fmt;
    long long lda, ldc, ld_sfa;
    const float* bias; /* per column, or NULL */
    int bias_after_k;
} mx_ctx;

static void mx_rows(void* vctx, int r0, int r1)
{
    const mx_ctx* x = (const mx_ctx*)vctx;
    float acc[JBLOCK];
    double* arow = (double*)malloc((size_t)x->k * sizeof(double));
    if (!arow) {
        return;
    }
    for (int i = r0; i < r1; ++i) {
        for (int kk = 0; kk < x->k; ++kk) {
            arow[kk] = mx_element(x->a, i, x->lda, kk, x->a_fmt) *
                       pto_oracle_e8m0_to_double(x->sfa[(size_t)i * x->ld_sfa + kk / 32]);
        }
        for (int j0 = 0; j0 < x->n; j0 += JBLOCK) {
            const int jn = x->n - j0 < JBLOCK ? x->n - j0 : JBLOCK;
            for (int j = 0; j < jn; ++j) {
                acc[j] = 0.0f;
            }
            for (int kk = 0; kk < x->k; ++kk) {
                const double av = arow[kk];
                const double* brow = x->bt + (size_t)kk * x->n + j0;
                for (int j = 0; j < jn; ++j) {
                    /* mul_acc += a * b * scaleFactor with a double right-hand side and a float accumulator:
                       the sum is formed in double and rounded to float once per k. The product is exact in
                       double (8-bit significands times powers of two), so the grouping of its factors is free. */
                    acc[j] = (float)((double)acc[j] + av * brow[j]);
                }
                if (x->bias && kk + 1 == x->bias_after_k) {
                    /* six-operand TMATMUL_MX: the finished first chunk, then += bias (cpu/TMatmul.hpp:285-291) */
                    for (int j = 0; j < jn; ++j) {
                        acc[j] += x->bias[j0 + j];
                    }
                }
            }
            memcpy(x->c + (size_t)i * x->ldc + j0, acc, (size_t)jn * sizeof(float));
        }
    }
    free(arow);
}

void pto_oracle_gemm_mx(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, float* c, int m,
                        int n, int k, long long lda, long long ldb, long long ldc, long long ld_sfa,
                        long long ld_sfb, int a_fmt, int b_fmt, int threads)
{
    pto_oracle_gemm_mx_bias(a, b, sfa, sfb, NULL, 0, c, m, n, k, lda, ldb, ldc, ld_sfa, ld_sfb, a_fmt, b_fmt, threads);
}

void pto_oracle_gemm_mx_bias(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                             const float* bias, int bias_after_k, float* c, int m, int n, int k, long long lda,
                             long long ldb, long long ldc, long long ld_sfa, long long ld_sfb, int a_fmt, int b_fmt,
                             int threads)
{
    if (m <= 0 || n <= 0 || k <= 0) {
        return;
    }
    if (bias_after_k <= 0 || bias_after_k > k) {
        bias_after_k = k;
    }
    double* bt = (double*)malloc((size_t)k * n * sizeof(double));
    if (!bt) {
        return;
    }
    for (int j = 0; j < n; ++j) {
        for (int kk = 0; kk < k; ++kk) {
            bt[(size_t)kk * n + j] = mx_element(b, j, ldb, kk, b_fmt) *
                                     pto_oracle_e8m0_to_double(sfb[(size_t)j * ld_sfb + kk / 32]);
        }
    }
    mx_ctx x = {a, sfa, bt, c, n, k, a_fmt, lda, ldc, ld_sfa, bias, bias_after_k};
    parallel_rows(mx_rows, &x, m, threads);
    free(bt);
}

/* ------------------------------------------------------------------ stores */

void pto_oracle_store_cast(const float* src, uint16_t* dst, long long count, int out_dtype)
{
    for (long long i = 0; i < count; ++i) {
        dst[i] = (out_dtype == ORACLE_F16) ? pto_oracle_float_to_half(src[i]) : pto_oracle_float_to_bf16(src[i]);
    }
}

/* extract_m1_from_quant<true>: sign(1) exponent(8) mantissa(10) taken from bits [31:13] of the scale word. */
static float scale_from_19_bits(float s)
{
    const uint32_t m1 = (float_to_bits(s) >> 13) & 0x7FFFFu;
    const uint32_t sign = (m1 >> 18) & 1u;
    const uint32_t exponent = (m1 >> 10) & 0xFFu;
    const uint32_t mantissa = m1 & 0x3FFu;
    if (exponent == 0 && mantissa == 0) {
        return 0.0f;
    }
    const float sign_val = sign ? -1.0f : 1.0f;
    const float mantissa_val = 1.0f + ((float)mantissa / 1024.0f);
    const float exponent_val = powf(2.0f, (float)exponent - 127.0f);
    return sign_val * mantissa_val * exponent_val;
}

void pto_oracle_dequant_bf16(const int32_t* acc, const float* s_row, const float* s_col, uint16_t* out, int m, int n,
                             long long ld_acc, long long ld_out, int truncate13)
{
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            const float sc = truncate13 ? scale_from_19_bits(s_col[j]) : s_col[j];
            volatile float t = (float)acc[(size_t)i * ld_acc + j] * sc;
            float tf = t;
            if (isfinite(tf)) { /* clamp to the finite fp32 range: a no-op kept for fidelity (common.hpp:166-171) */
                tf = fminf(fmaxf(tf, -3.402823466e38f), 3.402823466e38f);
            }
            volatile float u = tf * s_row[i];
            out[(size_t)i * ld_out + j] = pto_oracle_float_to_bf16(u);
        }
    }
}

/* TSTORE with a pre-quant scale word (cpu/TStore.hpp:154-181 -> quantize_element, cpu/common.hpp:139-185), modes as
   the overloads select them (common.hpp:58-108): int32 / float accumulators to bf16 / half, scalar form (fp32 scale in
   bits [31:0] of the word, one word for the whole tile) or vector form (one word per column, scale = the 19-bit float
   in bits [31:13]), optional ReLU after the scaling. Saturation control of the task cookie is off (its default).
   out_f16: 0 bfloat16, 1 half, 2 int8, 3 uint8, 4 int16 (int32 accumulators only) destinations. */
void pto_oracle_quant_store(const void* acc, int acc_is_int, const uint64_t* words, int vector, int relu, int out_f16,
                            uint16_t* out, int m, int n, long long ld_acc, long long ld_out)
{
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            const uint64_t w = words[vector ? j : 0];
            const float lo = bits_to_float((uint32_t)(w & 0xFFFFFFFFu));
            const float scale = vector ? scale_from_19_bits(lo) : lo;
            const float src = acc_is_int ? (float)((const int32_t*)acc)[(size_t)i * ld_acc + j]
                                         : ((const float*)acc)[(size_t)i * ld_acc + j];
            if (out_f16 == 4) {
                /* SHIFTS322S16 / VSHIFTS322S16 (common.hpp:172-178): the int32 accumulator shifted right (arithmetic)
                   by 1 + bits [35:32] of the word, then narrowed to int16 by the cast (it wraps; the clamp after it
                   has nothing left to do); ReLU on the result. */
                const int shift = (int)((w >> 32) & 0xFu) + 1;
                const int32_t shifted = ((const int32_t*)acc)[(size_t)i * ld_acc + j] >> shift;
                int16_t v16 = (int16_t)shifted;
                if (relu && v16 < 0) {
                    v16 = 0;
                }
                out[(size_t)i * ld_out + j] = (uint16_t)v16;
                continue;
            }
            volatile float t = src * scale;
            float r = t;
            if (out_f16 >= 2) {
                /* REQ8 / VREQ8 / QF322B8_PRE / VQF322B8_PRE (common.hpp:151-156): add the 9-bit offset of bits [45:37],
                   round to nearest even, clamp to the signed range when bit 46 is set, else to 0..255; ReLU; the
                   destination's integer cast. The result sits in the low byte of the 16-bit slot. */
                const float offset = (float)((w >> 37) & 0x1FFu);
                const int is_signed = (int)((w >> 46) & 1u);
                volatile float shifted = r + offset;
                float q = rintf(shifted);
                q = fminf(fmaxf(q, is_signed ? -128.0f : 0.0f), is_signed ? 127.0f : 255.0f);
                if (relu) {
                    q = (q > 0.0f) ? q : 0.0f;
                }
                out[(size_t)i * ld_out + j] = (uint16_t)((uint32_t)(int32_t)q & 0xFFu);
                continue;
            }
            if (out_f16) {
                /* DEQF16 / VDEQF16 clamp always; QF322F16_PRE / VQF322F16_PRE clamp finite values (common.hpp:157-164) */
                if (acc_is_int || isfinite(r)) {
                    r = fminf(fmaxf(r, -65504.0f), 65504.0f);
                }
            } else if (isfinite(r)) {
                r = fminf(fmaxf(r, -3.402823466e38f), 3.402823466e38f);
            }
            if (relu) {
                r = (r > 0.0f) ? r : 0.0f;
            }
            out[(size_t)i * ld_out + j] = out_f16 ? pto_oracle_float_to_half(r) : pto_oracle_float_to_bf16(r);
        }
    }
}

/* ------------------------------------------------------------------ MX quantiser (data preparation) */

/* Nearest e4m3fn code, ties to the even code; magnitudes that round to zero give +0 (code 0x00), as the
   simulator's search over all codes does (cpu/TQuant.hpp:118-153). Input already clamped to +-448. */
static uint8_t encode_e4m3fn(float v)
{
    if (isnan(v)) {
        return 0x7Fu;
    }
    float c = v;
    if (c > 448.0f) {
        c = 448.0f;
    }
    if (c < -448.0f) {
        c = -448.0f;
    }
    const float ax = fabsf(c);
    uint32_t code;
    if (ax < 0.015625f) { /* below the smallest normal 2^-6: subnormal grid of 2^-9 */
        code = (uint32_t)rintf(ax * 512.0f); /* 0..8; 8 is the code of 2^-6 */
    } else {
        int e;
        const float fr = frexpf(ax, &e); /* ax = fr * 2^e, fr in [0.5, 1) */
        uint32_t q = (uint32_t)rintf((fr * 2.0f - 1.0f) * 8.0f); /* 0..8 */
        int ee = e - 1;
        if (q == 8) {
            q = 0;
            ee += 1;
        }
        code = ((uint32_t)(ee + 7) << 3) | q;
        if (code > 0x7Eu) {
            code = 0x7Eu;
        }
    }
    if (code == 0) {
        return 0;
    }
    return (uint8_t)(code | (signbit(c) ? 0x80u : 0u));
}

/* scale_alg 0: OCP rule (ComputeSharedExponent, cpu/TQuant.hpp:178-190); 1: NV rule (ComputeNvSharedExponent with the
   e4m3 spec, :33-37,:194-211: e8m0 = ceil(log2(amax / 448)) as a biased exponent; scaling :239-248; the NV form of the
   element encoder keeps the sign of values below 2^-10, :118-131). */
void pto_oracle_mx_quantize_e4m3_alg(const float* src, uint8_t* data, uint8_t* scales, int rows, int k, long long ld,
                                     int scale_alg)
{
    const int groups = k / 32;
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < groups; ++g) {
            const float* x = src + (size_t)r * ld + (size_t)g * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) {
                const float ax = fabsf(x[i]);
                if (ax > amax) {
                    amax = ax;
                }
            }
            uint8_t e8m0;
            float scaling;
            if (scale_alg == 0) {
                /* ComputeSharedExponent: biased exponent of the block maximum minus 8, floored at 0 */
                const uint32_t bits = float_to_bits(amax);
                const uint32_t exponent = (bits & 0x7F800000u) >> 23;
                e8m0 = (exponent <= 8u) ? 0u : (uint8_t)(exponent - 8u);
                /* ComputeMxScalingFromExponent: 2^(127 - e8m0), with the zero bit pattern replaced by 2^-127 */
                scaling = bits_to_float((254u - (uint32_t)e8m0) << 23);
                if (scaling == 0.0f) {
                    scaling = ldexpf(1.0f, -127);
                }
            } else {
                e8m0 = 0;
                if (amax != 0.0f) {
                    volatile float descale = amax * (1.0f / 448.0f);
                    const uint32_t bits = float_to_bits(descale);
                    const uint32_t exponent = (bits & 0x7F800000u) >> 23;
                    const uint32_t mantissa = bits & 0x007FFFFFu;
                    if (exponent == 0xFFu) {
                        e8m0 = mantissa == 0u ? 0xFEu : 0xFFu;
                    } else {
                        const int round_up = mantissa > 0u && exponent != 0xFEu && !(exponent == 0u && mantissa <= 0x00400000u);
                        e8m0 = (uint8_t)(exponent + (round_up ? 1u : 0u));
                    }
                }
                if (e8m0 == 0xFFu) {
                    scaling = amax; /* NaN block */
                } else if (e8m0 == 0xFEu) {
                    scaling = ldexpf(1.0f, -127);
                } else {
                    scaling = bits_to_float((254u - (uint32_t)e8m0) << 23);
                    if (scaling == 0.0f) {
                        scaling = ldexpf(1.0f, -127);
                    }
                }
            }
            scales[(size_t)r * groups + g] = e8m0;
            for (int i = 0; i < 32; ++i) {
                volatile float y = x[i] * scaling;
                const float yv = y;
                if (scale_alg != 0 && !isnan(yv) && fabsf(yv) < 0.0009765625f) {
                    data[(size_t)r * k + (size_t)g * 32 + i] = signbit(yv) ? 0x80u : 0x00u;
                } else {
                    data[(size_t)r * k + (size_t)g * 32 + i] = encode_e4m3fn(yv);
                }
            }
        }
    }
}

/* TQUANT to MXFP4 (float4_e2m1x2_t, two codes per byte, element 2i in the low nibble) with e8m0 block scales.
   OCP rule (cpu/TQuant.hpp:280-305,210-221): the block maximum is taken over the values TRUNCATED to bf16, e8m0 =
   max(biased exponent - 2, 0). NV rule (:194-208 with the e2m1 spec :39-45): e8m0 = biased exponent of amax / 6,
   rounded up. Scaling 2^(127 - e8m0) (:226-248). Element code (EncodeE2M1Magic, :155-176): the magnitude is rounded to
   nearest even on the grid of its binade - steps of 0.5 below 2, 1 below 4, 2 above - by adding a power of two, and
   saturates at 6; the sign bit is kept, also on a zero. Inputs finite. */
static uint8_t encode_e2m1_magic(float value)
{
    const uint32_t value_bits = float_to_bits(value);
    const uint8_t sign = (uint8_t)((value_bits >> 28) & 0x8u);
    const float abs_value = fabsf(value);
    const uint32_t abs_bits = float_to_bits(abs_value);
    uint32_t biased = (abs_bits & 0x7F800000u) >> 23;
    biased = biased < 127u ? 127u : (biased > 129u ? 129u : biased);
    const uint32_t magic_bits = (biased + 22u) << 23;
    volatile float sum = abs_value + bits_to_float(magic_bits);
    const uint32_t q = float_to_bits(sum) - magic_bits;
    const uint32_t base = (biased - 127u) << 1;
    const uint32_t mag = (q + base) > 7u ? 7u : (q + base);
    return (uint8_t)(sign | mag);
}

void pto_oracle_mx_quantize_e2m1(const float* src, uint8_t* data, uint8_t* scales, int rows, int k, long long ld,
                                 int scale_alg)
{
    const int groups = k / 32;
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < groups; ++g) {
            const float* x = src + (size_t)r * ld + (size_t)g * 32;
            float amax = 0.0f;
            uint32_t amax_bf16 = 0;
            for (int i = 0; i < 32; ++i) {
                const float ax = fabsf(x[i]);
                const uint32_t top = (float_to_bits(x[i]) >> 16) & 0x7FFFu;
                if (ax > amax) {
                    amax = ax;
                }
                if (top > amax_bf16) {
                    amax_bf16 = top;
                }
            }
            uint8_t e8m0 = 0;
            float scaling;
            if (scale_alg == 0) {
                const uint32_t exponent = (amax_bf16 >> 7) & 0xFFu; /* of the truncated maximum */
                e8m0 = (exponent <= 2u) ? 0u : (uint8_t)(exponent - 2u);
            } else if (amax != 0.0f) {
                volatile float descale = amax * (1.0f / 6.0f);
                const uint32_t bits = float_to_bits(descale);
                const uint32_t exponent = (bits & 0x7F800000u) >> 23;
                const uint32_t mantissa = bits & 0x007FFFFFu;
                const int round_up = mantissa > 0u && exponent != 0xFEu && !(exponent == 0u && mantissa <= 0x00400000u);
                e8m0 = (uint8_t)(exponent + (round_up ? 1u : 0u));
            }
            scaling = (e8m0 >= 0xFEu) ? ldexpf(1.0f, -127) : bits_to_float((254u - (uint32_t)e8m0) << 23);
            scales[(size_t)r * groups + g] = e8m0;
            for (int i = 0; i < 32; i += 2) {
                volatile float y0 = x[i] * scaling;
                volatile float y1 = x[i + 1] * scaling;
                data[(size_t)r * (k / 2) + (size_t)g * 16 + i / 2] =
                    (uint8_t)(encode_e2m1_magic(y0) | (encode_e2m1_magic(y1) << 4));
            }
        }
    }
}

void pto_oracle_mx_quantize_e4m3(const float* src, uint8_t* data, uint8_t* scales, int rows, int k, long long ld)
{
    pto_oracle_mx_quantize_e4m3_alg(src, data, scales, rows, k, ld, 0);
}
