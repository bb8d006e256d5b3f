/*
 * CPU oracle for the MXFP8 quantise + AllGather-Matmul path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker the CUDA path is compared with (tests, the smoke check and the CPU
 * baseline leg of the benchmark).  Nothing in the shipped library links or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference's CPU golden path and of its
 * device kernel for this path:
 *   - examples/utils/gen_mx_quant_allgather_data.py:168-189  (_e8m0_exp: block exponent,
 *     epsilon rule for tiny blocks)
 *   - examples/utils/gen_mx_quant_allgather_data.py:255-313  (_quantize_axis_last_fp8:
 *     amax per 32, divide by 2^exp, clamp to +-448, cast RNE)   -> mode MXO_MODE_GOLDEN
 *   - include/catccos/comm/block/comm_block_mx_quant.hpp:413-523,569-664 (ComputeMxQuant,
 *     FP8 branch: exponent-field max, shared exponent, reciprocal scale, clamp, CAST_RINT)
 *                                                               -> mode MXO_MODE_DEVICE
 *   - examples/utils/gen_mx_quant_allgather_data.py:48-52 and comm_block_mx_quant.hpp:75-76,410 (the E5M2
 *     output type: emax 15, max 57344)                          -> mxo_quantize_rows_e5m2
 *   - examples/utils/gen_data_fp8_mx_allgather_matmul.py:643-658 (golden GEMM: rank-order
 *     concat of dequantised A times dequantised B, fp32) and :650-656 (B scale file layout
 *     [K/64, N, 2]).
 *
 * Parity is pinned: tests/golden/ holds outputs of the reference generator itself
 * (backend "native"), produced by tests/golden/make_golden.py, and the oracle is checked
 * against them bit for bit.
 *
 * The two modes differ only for blocks whose amax is below 1e-12 (see mxo_block_scale).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define MXO_BLOCK 32
#define MXO_MODE_GOLDEN 0
#define MXO_MODE_DEVICE 1

static inline float bf16_to_f32(uint16_t b)
{
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline float pow2i(int e) /* 2^e for e in [-149, 127]; below -126 the result is a subnormal */
{
    if (e < -126) {
        return ldexpf(1.0f, e); /* reached by E1M2 (emax 0): a block maximum of 2^127 is divided by 2^127 */
    }
    uint32_t u = (uint32_t)(e + 127) << 23;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* fp32 -> E4M3FN, round to nearest even, finite inputs with |v| <= 448 (callers clamp).
 * NaN -> 0x7F.  Follows torch's float8_e4m3fn cast used by the golden's "native" backend
 * (gen_mx_quant_allgather_data.py:286-287) and the device CAST_RINT/SAT cast
 * (comm_block_mx_quant.hpp:592-603). */
uint8_t mxo_e4m3_from_f32(float v)
{
    uint32_t u;
    memcpy(&u, &v, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) {
        return 0x7F;
    }
    float av;
    memcpy(&av, &a, 4);
    if (av > 448.0f) {
        av = 448.0f;
        memcpy(&a, &av, 4);
    }
    if (av < 0.015625f) { /* below the smallest normal 2^-6: subnormal grid of 2^-9 */
        float q = rintf(av * 512.0f); /* default rounding mode: nearest even */
        return (uint8_t)(sign | (uint8_t)q);
    }
    int e = (int)(a >> 23) - 127; /* -6 .. 8 */
    uint32_t man = a & 0x7FFFFFu;
    uint32_t keep = man >> 20;
    uint32_t rem = man & 0xFFFFFu;
    uint32_t code = ((uint32_t)(e + 7) << 3) | keep;
    if (rem > 0x80000u || (rem == 0x80000u && (keep & 1u))) {
        code += 1; /* the carry runs into the exponent field, which is what RNE needs */
    }
    return (uint8_t)(sign | (uint8_t)code);
}

/* E4M3FN code -> fp32 (0x7F/0xFF are NaN). */
float mxo_e4m3_to_f32(uint8_t c)
{
    uint32_t mag = c & 0x7F;
    float v;
    if (mag == 0x7F) {
        v = NAN;
    } else if ((mag >> 3) == 0) {
        v = (float)(mag & 7) * 0.001953125f; /* 2^-9 */
    } else {
        v = (1.0f + (float)(mag & 7) * 0.125f) * pow2i((int)(mag >> 3) - 7);
    }
    return (c & 0x80) ? -v : v;
}

/* fp32 -> E5M2, round to nearest even, finite inputs with |v| <= 57344 (callers clamp); NaN -> 0x7F.
 * E5M2 is the top byte of IEEE half: torch's float8_e5m2 cast used by the golden's "native" backend
 * (gen_mx_quant_allgather_data.py:48-52,286-287); device cast as for E4M3 (comm_block_mx_quant.hpp:592-603). */
uint8_t mxo_e5m2_from_f32(float v)
{
    uint32_t u;
    memcpy(&u, &v, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) {
        return 0x7F;
    }
    float av;
    memcpy(&av, &a, 4);
    if (av > 57344.0f) {
        av = 57344.0f;
        memcpy(&a, &av, 4);
    }
    if (av < 6.103515625e-05f) { /* below the smallest normal 2^-14: subnormal grid of 2^-16 */
        float q = rintf(av * 65536.0f);
        return (uint8_t)(sign | (uint8_t)q);
    }
    int e = (int)(a >> 23) - 127; /* -14 .. 15 */
    uint32_t man = a & 0x7FFFFFu;
    uint32_t keep = man >> 21;
    uint32_t rem = man & 0x1FFFFFu;
    uint32_t code = ((uint32_t)(e + 15) << 2) | keep;
    if (rem > 0x100000u || (rem == 0x100000u && (keep & 1u))) {
        code += 1;
    }
    return (uint8_t)(sign | (uint8_t)code);
}

/* E5M2 code -> fp32 (0x7C/0xFC are infinities, 0x7D..0x7F NaN). */
float mxo_e5m2_to_f32(uint8_t c)
{
    uint32_t mag = c & 0x7F;
    float v;
    if (mag > 0x7C) {
        v = NAN;
    } else if (mag == 0x7C) {
        v = INFINITY;
    } else if ((mag >> 2) == 0) {
        v = (float)(mag & 3) * 1.52587890625e-05f; /* 2^-16 */
    } else {
        int e = (int)(mag >> 2) - 15;
        v = (1.0f + (float)(mag & 3) * 0.25f) * (e >= -126 ? pow2i(e) : 0.0f);
    }
    return (c & 0x80) ? -v : v;
}

/* E8M0 byte -> fp32 scale 2^(byte-127); 0xFF is NaN.  byte 0 is 2^-127 (a subnormal). */
float mxo_e8m0_to_f32(uint8_t b)
{
    if (b == 0xFF) {
        return NAN;
    }
    if (b == 0) {
        return 5.877471754111438e-39f;
    }
    return pow2i((int)b - 127);
}

/* One block of 32 bf16 values -> scale byte, and what to multiply by.
 * returns 0 = normal block (multiply by *mul), 1 = all codes are signed zeros,
 *         2 = block holds Inf/NaN (scale 0xFF, codes 0x7F; device rule,
 *             comm_block_mx_quant.hpp:496,503,513 - no reference test pins this case). */
static int mxo_block_scale_fmt(const uint16_t* x, size_t stride, int mode, int emax, uint8_t* scale, float* mul)
{
    uint16_t amax = 0;
    for (int i = 0; i < MXO_BLOCK; ++i) {
        uint16_t a = x[(size_t)i * stride] & 0x7FFF;
        if (a > amax) {
            amax = a;
        }
    }
    int E = amax >> 7; /* biased exponent of the block maximum = floor(log2(amax)) + 127 */
    if (E == 0xFF) {
        *scale = 0xFF;
        return 2;
    }
    if (mode == MXO_MODE_GOLDEN) {
        /* gen_mx_quant_allgather_data.py:181-189: amax < 1e-12 -> exponent 0 (scale 1.0,
         * byte 0x7F).  For bf16 inputs "< 1e-12f" is "bits <= 0x2B8C". */
        if (amax <= 0x2B8C) {
            *scale = 0x7F;
            return 1;
        }
        *scale = (uint8_t)(E - emax);
        *mul = pow2i(127 - (E - emax));
        return 0;
    }
    /* device: shared = max(E,emax) - emax; byte = shared; recip scale 0 when shared == 0
     * (comm_block_mx_quant.hpp:498-517; emax 8 for E4M3, 15 for E5M2, :409-410). */
    int byte = E > emax ? E - emax : 0;
    *scale = (uint8_t)byte;
    if (byte == 0) {
        return 1;
    }
    *mul = pow2i(127 - byte);
    return 0;
}

static int mxo_block_scale(const uint16_t* x, size_t stride, int mode, uint8_t* scale, float* mul)
{
    return mxo_block_scale_fmt(x, stride, mode, 8, scale, mul);
}

/* fmt 0 = E4M3 (max 448), 1 = E5M2 (max 57344) */
static inline uint8_t mxo_encode_fmt(uint16_t xb, int kind, float mul, int fmt)
{
    if (kind == 2) {
        return 0x7F;
    }
    if (kind == 1) {
        return (uint8_t)((xb >> 8) & 0x80);
    }
    const float lim = fmt == 1 ? 57344.0f : 448.0f;
    float y = bf16_to_f32(xb) * mul;
    if (y > lim) {
        y = lim;
    }
    if (y < -lim) {
        y = -lim;
    }
    return fmt == 1 ? mxo_e5m2_from_f32(y) : mxo_e4m3_from_f32(y);
}

static inline uint8_t mxo_encode(uint16_t xb, int kind, float mul)
{
    return mxo_encode_fmt(xb, kind, mul, 0);
}

/* The E5M2 form of mxo_quantize_rows (MX_QUANT_DTYPE = 1 in the reference: emax 15,
 * gen_mx_quant_allgather_data.py:48-52; comm_block_mx_quant.hpp:75-76,410). */
int mxo_quantize_rows_e5m2(const uint16_t* x, size_t rows, size_t K, uint8_t* codes, uint8_t* scales, int mode)
{
    if (K % MXO_BLOCK != 0) {
        return -1;
    }
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t b = 0; b < nb; ++b) {
            const uint16_t* xb = x + (size_t)r * K + b * MXO_BLOCK;
            uint8_t s;
            float mul = 0.0f;
            int kind = mxo_block_scale_fmt(xb, 1, mode, 15, &s, &mul);
            scales[(size_t)r * nb + b] = s;
            for (int i = 0; i < MXO_BLOCK; ++i) {
                codes[(size_t)r * K + b * MXO_BLOCK + i] = mxo_encode_fmt(xb[i], kind, mul, 1);
            }
        }
    }
    return 0;
}

/* Dequantise row-quantised E5M2 codes: out fp32 [rows, K]. */
void mxo_dequant_rows_e5m2(const uint8_t* codes, const uint8_t* scales, size_t rows, size_t K, float* out)
{
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t k = 0; k < K; ++k) {
            out[(size_t)r * K + k] =
                mxo_e5m2_to_f32(codes[(size_t)r * K + k]) * mxo_e8m0_to_f32(scales[(size_t)r * nb + k / MXO_BLOCK]);
        }
    }
}

/* ---- FP4 E2M1 (the reference's fp4 variant of the same operators: emax 2, max 6;
 * gen_mx_quant_allgather_data.py:55-62,349-397,413-452; comm_block_mx_quant.hpp:69-70,525-568).  Oracle and
 * fixtures only: no CUDA kernel reads these yet. ------------------------------------------------------- */

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
/* E1M2 (one exponent bit, two mantissa bits, bias 1; emax 0, max 1.75; gen_mx_quant_allgather_data.py:63-70) */
static const float kE1M2[8] = {0.0f, 0.25f, 0.5f, 0.75f, 1.0f, 1.25f, 1.5f, 1.75f};

static uint8_t mxo_fp4_from_f32(const float* table, float v, int ties_to_zero)
{
    float a = fabsf(v);
    if (a > table[7]) {
        a = table[7];
    }
    int best = 0;
    for (int i = 1; i < 8; ++i) {
        float d = fabsf(a - table[i]), db = fabsf(a - table[best]);
        if (d < db) {
            best = i;
        } else if (d == db && !ties_to_zero && (i & 1) == 0) {
            best = i; /* a tie between neighbours: the even code wins under round-to-nearest-even */
        }
    }
    if (ties_to_zero) {
        return (uint8_t)((v < 0.0f && best != 0) ? (best | 8) : best);
    }
    return (uint8_t)(signbit(v) ? (best | 8) : best);
}

/* E2M1 code (4 bits: sign, two exponent bits, one mantissa bit) -> fp32. */
float mxo_e2m1_to_f32(uint8_t c)
{
    float v = kE2M1[c & 7];
    return (c & 8) ? -v : v;
}

/* fp32 (finite, callers clamp to +-6) -> E2M1 code.
 * ties_to_zero = 1: the golden's rule, nearest table entry with the smaller index winning a tie
 *                   (gen_mx_quant_allgather_data.py:383-397): ties go toward zero and every zero is +0.
 * ties_to_zero = 0: round to nearest even with the sign kept (CAST_RINT on the device,
 *                   comm_block_mx_quant.hpp:538-555; cvt.rn.satfinite.e2m1x2.f32 on a GPU). */
uint8_t mxo_e2m1_from_f32(float v, int ties_to_zero)
{
    return mxo_fp4_from_f32(kE2M1, v, ties_to_zero);
}

float mxo_e1m2_to_f32(uint8_t c)
{
    float v = kE1M2[c & 7];
    return (c & 8) ? -v : v;
}

uint8_t mxo_e1m2_from_f32(float v, int ties_to_zero)
{
    return mxo_fp4_from_f32(kE1M2, v, ties_to_zero);
}

/* x bf16 [rows, K] -> packed codes [rows, K/2] (low nibble = even column, _pack_fp4_nibbles :400-411) and
 * scales [rows, K/32].  mode MXO_MODE_GOLDEN: golden rounding and tiny-block rule; MXO_MODE_DEVICE: RNE,
 * byte = max(E - 2, 0).  K % 32 == 0. */
static int mxo_quantize_rows_fp4(const float* table, int emax, const uint16_t* x, size_t rows, size_t K, uint8_t* packed,
                                 uint8_t* scales, int mode)
{
    if (K % MXO_BLOCK != 0) {
        return -1;
    }
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t b = 0; b < nb; ++b) {
            const uint16_t* xb = x + (size_t)r * K + b * MXO_BLOCK;
            uint8_t s;
            float mul = 0.0f;
            int kind = mxo_block_scale_fmt(xb, 1, mode, emax, &s, &mul);
            scales[(size_t)r * nb + b] = s;
            for (int i = 0; i < MXO_BLOCK; i += 2) {
                uint8_t c[2];
                for (int j = 0; j < 2; ++j) {
                    if (kind == 2) {
                        c[j] = 0x7; /* no NaN in E2M1: the largest magnitude stands in (no reference test pins it) */
                    } else if (kind == 1) {
                        c[j] = (uint8_t)((mode == MXO_MODE_GOLDEN) ? 0 : ((xb[i + j] >> 12) & 8));
                    } else {
                        c[j] = mxo_fp4_from_f32(table, bf16_to_f32(xb[i + j]) * mul, mode == MXO_MODE_GOLDEN);
                    }
                }
                packed[(size_t)r * (K / 2) + (b * MXO_BLOCK + i) / 2] = (uint8_t)(c[0] | (c[1] << 4));
            }
        }
    }
    return 0;
}

int mxo_quantize_rows_e2m1(const uint16_t* x, size_t rows, size_t K, uint8_t* packed, uint8_t* scales, int mode)
{
    return mxo_quantize_rows_fp4(kE2M1, 2, x, rows, K, packed, scales, mode);
}

/* The E1M2 form (emax 0, max 1.75): oracle only. */
int mxo_quantize_rows_e1m2(const uint16_t* x, size_t rows, size_t K, uint8_t* packed, uint8_t* scales, int mode)
{
    return mxo_quantize_rows_fp4(kE1M2, 0, x, rows, K, packed, scales, mode);
}

static void mxo_dequant_rows_fp4(const float* table, const uint8_t* packed, const uint8_t* scales, size_t rows, size_t K,
                                 float* out)
{
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t k = 0; k < K; ++k) {
            uint8_t byte = packed[(size_t)r * (K / 2) + k / 2];
            uint8_t c = (k & 1) ? (byte >> 4) : (byte & 15);
            float v = table[c & 7];
            out[(size_t)r * K + k] = ((c & 8) ? -v : v) * mxo_e8m0_to_f32(scales[(size_t)r * nb + k / MXO_BLOCK]);
        }
    }
}

/* packed E2M1 / E1M2 codes [rows, K/2] + scales [rows, K/32] -> fp32 [rows, K]. */
void mxo_dequant_rows_e2m1(const uint8_t* packed, const uint8_t* scales, size_t rows, size_t K, float* out)
{
    mxo_dequant_rows_fp4(kE2M1, packed, scales, rows, K, out);
}

void mxo_dequant_rows_e1m2(const uint8_t* packed, const uint8_t* scales, size_t rows, size_t K, float* out)
{
    mxo_dequant_rows_fp4(kE1M2, packed, scales, rows, K, out);
}

/* Quantise along the last axis: x bf16 [rows, K] -> codes [rows, K], scales [rows, K/32]
 * (row-major).  K % 32 == 0 (mx_quant_allgather_host.h:21-25).  Returns 0, or -1 on a bad shape. */
int mxo_quantize_rows(const uint16_t* x, size_t rows, size_t K, uint8_t* codes, uint8_t* scales, int mode)
{
    if (K % MXO_BLOCK != 0) {
        return -1;
    }
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t b = 0; b < nb; ++b) {
            const uint16_t* xb = x + (size_t)r * K + b * MXO_BLOCK;
            uint8_t s;
            float mul = 0.0f;
            int kind = mxo_block_scale(xb, 1, mode, &s, &mul);
            scales[(size_t)r * nb + b] = s;
            for (int i = 0; i < MXO_BLOCK; ++i) {
                codes[(size_t)r * K + b * MXO_BLOCK + i] = mxo_encode(xb[i], kind, mul);
            }
        }
    }
    return 0;
}

/* Quantise a weight B bf16 [K, N] along axis 0 (blocks of 32 along K for every column n):
 * codes [K, N]; scales in the reference file layout [K/64, N, 2]
 * (gen_mx_quant_allgather_data.py:316-324, gen_data_fp8_mx_allgather_matmul.py:650-656).
 * K % 64 == 0. */
int mxo_quantize_weight(const uint16_t* b, size_t K, size_t N, uint8_t* codes, uint8_t* scales, int mode)
{
    if (K % 64 != 0) {
        return -1;
    }
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t kb = 0; kb < (ptrdiff_t)nb; ++kb) {
        for (size_t n = 0; n < N; ++n) {
            const uint16_t* xb = b + (size_t)kb * MXO_BLOCK * N + n;
            uint8_t s;
            float mul = 0.0f;
            int kind = mxo_block_scale(xb, N, mode, &s, &mul);
            scales[((size_t)(kb / 2) * N + n) * 2 + (kb & 1)] = s;
            for (int i = 0; i < MXO_BLOCK; ++i) {
                codes[((size_t)kb * MXO_BLOCK + i) * N + n] = mxo_encode(xb[(size_t)i * N], kind, mul);
            }
        }
    }
    return 0;
}

/* Dequantise row-quantised codes: out fp32 [rows, K]. */
void mxo_dequant_rows(const uint8_t* codes, const uint8_t* scales, size_t rows, size_t K, float* out)
{
    size_t nb = K / MXO_BLOCK;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t k = 0; k < K; ++k) {
            out[(size_t)r * K + k] =
                mxo_e4m3_to_f32(codes[(size_t)r * K + k]) * mxo_e8m0_to_f32(scales[(size_t)r * nb + k / MXO_BLOCK]);
        }
    }
}

/* Dequantise a weight: codes [K, N], scales [K/64, N, 2] -> out fp32 [K, N]. */
void mxo_dequant_weight(const uint8_t* codes, const uint8_t* scales, size_t K, size_t N, float* out)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t k = 0; k < (ptrdiff_t)K; ++k) {
        size_t kb = (size_t)k / MXO_BLOCK;
        for (size_t n = 0; n < N; ++n) {
            out[(size_t)k * N + n] = mxo_e4m3_to_f32(codes[(size_t)k * N + n]) *
                                     mxo_e8m0_to_f32(scales[((kb / 2) * N + n) * 2 + (kb & 1)]);
        }
    }
}

/* Golden GEMM: C fp32 [M, N] = A fp32 [M, K] @ B fp32 [K, N], fp32 accumulate
 * (gen_data_fp8_mx_allgather_matmul.py:643).  Plain ikj loops, threads over rows. */
void mxo_gemm_f32(const float* A, const float* B, float* C, size_t M, size_t N, size_t K)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t m = 0; m < (ptrdiff_t)M; ++m) {
        float* c = C + (size_t)m * N;
        for (size_t n = 0; n < N; ++n) {
            c[n] = 0.0f;
        }
        for (size_t k = 0; k < K; ++k) {
            float a = A[(size_t)m * K + k];
            const float* b = B + k * N;
            for (size_t n = 0; n < N; ++n) {
                c[n] += a * b[n];
            }
        }
    }
}
