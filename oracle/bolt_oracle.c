/*
 * bolt_oracle.c -- TEST INFRASTRUCTURE ONLY (see bolt_oracle.h).
 *
 * Scalar restatement of Bolt's quantized inference arithmetic.  Build:
 *   gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared bolt_oracle.c -o libbolt_oracle.so -lm
 */
#include "bolt_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------ */
/* helpers                                                                        */
/* ------------------------------------------------------------------------------ */

/* vcvtps2dq as used in blas_common_int8.h:1195-1209 and avx512/quantize.cpp:153:
 * RNE under the default MXCSR; the "integer indefinite" 0x80000000 for NaN and for
 * |f| >= 2^31. */
int32_t oracle_cvt_rne(float f)
{
    if (!(f > -2147483904.0f && f < 2147483648.0f)) {
        return INT32_MIN;
    }
    return (int32_t)lrintf(f); /* default rounding mode = nearest-even */
}

/* vpmovusdb (mmm_avx512_vnni.cpp:1457, avx512/quantize.cpp:156,385): unsigned
 * saturation of a dword that is interpreted as unsigned. */
uint8_t oracle_usat8(int32_t v)
{
    uint32_t u = (uint32_t)v;
    return (uint8_t)(u > 255u ? 255u : u);
}

/* vpmovsdb (avx512/quantize.cpp:211,339). */
int8_t oracle_ssat8(int32_t v)
{
    return (int8_t)(v > 127 ? 127 : (v < -128 ? -128 : v));
}

/* ------------------------------------------------------------------------------ */
/* GEMM / GEMV                                                                    */
/* ------------------------------------------------------------------------------ */

/* mmm_avx512_vnni.cpp:81-87 (rhsN) and :112-118 (rhsT); mvm_avx512_vnni.cpp:72-78,118-124. */
void oracle_offsetc(const int8_t *B, uint32_t K, uint32_t N, int b_transposed, int32_t *offsetC)
{
    for (uint32_t n = 0; n < N; ++n) {
        int32_t s = 0;
        for (uint32_t k = 0; k < K; ++k) {
            s += b_transposed ? B[(size_t)n * K + k] : B[(size_t)k * N + n];
        }
        offsetC[n] = s * (-128);
    }
}

/* Epilogue of mmm_avx512_vnni.cpp:1446-1461 with blas_common_int8.h:922-932
 * (vcvtdq2ps, vmulps) and :1195-1209 (vcvtps2dq, vpaddd 128) + vpmovusdb. */
static inline float acc_to_f32(int32_t acc, float factor)
{
    return (float)acc * factor;
}
static inline uint8_t acc_to_u8(int32_t acc, float factor)
{
    int32_t r = oracle_cvt_rne((float)acc * factor);
    return oracle_usat8((int32_t)((uint32_t)r + 128u));
}

/* mmm_avx512_vnni.cpp:1760-1891: acc initial value = offsetC (loadOffset, :1391),
 * C added as int32 (addC, :1449), factor = 1/scale[0] (:1805) or scale[1] (:1799);
 * in the u8 mode the int32 partials live in a zeroed tmp buffer (:1800-1801), so the
 * incoming C never contributes. */
void oracle_gemm_u8s8(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, int a_transposed,
    const int8_t *B, int b_transposed, const int32_t *offsetC, void *C, const float *scale)
{
    int mode = 0; /* 0 s32, 1 f32, 2 u8 */
    float factor = 0;
    if (scale != NULL) {
        if (scale[0] < 0) {
            mode = 2;
            factor = scale[1];
        } else {
            mode = 1;
            factor = 1 / scale[0];
        }
    }
    for (uint32_t m = 0; m < M; ++m) {
        for (uint32_t n = 0; n < N; ++n) {
            int32_t acc = offsetC ? offsetC[n] : 0;
            for (uint32_t k = 0; k < K; ++k) {
                int32_t a = a_transposed ? A[(size_t)k * M + m] : A[(size_t)m * K + k];
                int32_t b = b_transposed ? B[(size_t)n * K + k] : B[(size_t)k * N + n];
                acc += a * b;
            }
            size_t o = (size_t)m * N + n;
            if (mode == 2) {
                ((uint8_t *)C)[o] = acc_to_u8(acc, factor);
            } else {
                acc = (int32_t)((uint32_t)acc + ((uint32_t *)C)[o]);
                if (mode == 1) {
                    ((float *)C)[o] = acc_to_f32(acc, factor);
                } else {
                    ((int32_t *)C)[o] = acc;
                }
            }
        }
    }
}

/* mvm_avx512_vnni.cpp:703-759 (driver), :566-640 (vector rows), :667-701 (scalar
 * tail rows: offsetC only, `(I32)(f + 128)` truncation, upper clamp only). */
void oracle_gemv_s8u8(uint32_t N, uint32_t K, const int8_t *W, int w_transposed,
    const uint8_t *x, const int32_t *offsetC, void *y, const float *scale)
{
    int mode = 0;
    float factor = 0;
    if (scale != NULL) {
        if (scale[0] < 0) {
            mode = 2;
            factor = scale[1];
        } else {
            mode = 1;
            factor = 1 / scale[0];
        }
    }
    uint32_t tail_begin = N - (N % 8);
    for (uint32_t n = 0; n < N; ++n) {
        int32_t acc = offsetC ? offsetC[n] : 0;
        for (uint32_t k = 0; k < K; ++k) {
            int32_t w = w_transposed ? W[(size_t)k * N + n] : W[(size_t)n * K + k];
            acc += w * (int32_t)x[k];
        }
        int tail = (n >= tail_begin);
        if (mode == 2) {
            if (tail) {
                float f = (float)acc * factor;
                int32_t t = (int32_t)(f + 128);
                ((uint8_t *)y)[n] = (uint8_t)((t > 255) ? 255 : t);
            } else {
                ((uint8_t *)y)[n] = acc_to_u8(acc, factor);
            }
        } else {
            if (!tail) {
                acc = (int32_t)((uint32_t)acc + ((uint32_t *)y)[n]);
            }
            if (mode == 1) {
                ((float *)y)[n] = (float)acc * factor;
            } else {
                ((int32_t *)y)[n] = acc;
            }
        }
    }
}

/* ------------------------------------------------------------------------------ */
/* quantize / dequantize                                                          */
/* ------------------------------------------------------------------------------ */

/* avx512/quantize.cpp:21-68: sign-bit mask + vmaxps, then 127/max (fp32 divide). */
float oracle_scale_f32(const float *x, uint64_t n)
{
    float mx = 0;
    for (uint64_t i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        if (a > mx) {
            mx = a;
        }
    }
    return (mx == 0) ? 1.0f : 127 / mx;
}

/* avx512/quantize.cpp:70-119: vpabsd + vpmaxsd, then 127.0f / (float)max. */
float oracle_scale_i32(const int32_t *x, uint64_t n)
{
    int32_t mx = 0;
    for (uint64_t i = 0; i < n; ++i) {
        int32_t a = (x[i] < 0) ? (int32_t)(0u - (uint32_t)x[i]) : x[i];
        if (a > mx) {
            mx = a;
        }
    }
    return (mx == 0) ? 1.0f : 127.0f / (float)mx;
}

/* avx512/quantize.cpp:121-179: vmulps, vaddps 128.0f, vcvtps2dq{rn}, max 1, min 255. */
void oracle_quantize_f32_u8(const float *x, uint64_t n, uint8_t *q, float *scale, int mode)
{
    if (!mode || *scale <= 0) {
        float min_scale = *scale;
        float s = oracle_scale_f32(x, n);
        *scale = (min_scale > s) ? min_scale : s;
    }
    float s = *scale;
    for (uint64_t i = 0; i < n; ++i) {
        float t = x[i] * s;
        t = t + 128.0f;
        int32_t r = oracle_cvt_rne(t);
        r = r < 1 ? 1 : r;
        r = r > 255 ? 255 : r;
        q[i] = (uint8_t)r;
    }
}

/* avx512/quantize.cpp:181-234: vmulps, vcvtps2dq, max -127, min 127. */
void oracle_quantize_f32_i8(const float *x, uint64_t n, int8_t *q, float *scale, int mode)
{
    if (!mode || *scale <= 0) {
        float min_scale = *scale;
        float s = oracle_scale_f32(x, n);
        *scale = (min_scale > s) ? min_scale : s;
    }
    float s = *scale;
    for (uint64_t i = 0; i < n; ++i) {
        int32_t r = oracle_cvt_rne(x[i] * s);
        r = r < -127 ? -127 : r;
        r = r > 127 ? 127 : r;
        q[i] = (int8_t)r;
    }
}

/* avx512/quantize.cpp:315-326,364-375: choice of the raw requantization factor. */
static float requant_factor_i32(const int32_t *x, uint64_t n, float *scale)
{
    float raw = 0;
    if (scale[0] < 0 && scale[1] > 0) {
        raw = oracle_scale_i32(x, n);
        scale[0] = scale[1] * raw;
    } else if (scale[0] > 0 && scale[1] > 0) {
        raw = scale[0] / scale[1];
    }
    return raw;
}

/* avx512/quantize.cpp:364-416: vcvtdq2ps, vmulps, vaddps 128.0f, vcvtps2dq, vpmovusdb. */
void oracle_quantize_i32_u8(const int32_t *x, uint64_t n, uint8_t *q, float *scale)
{
    float raw = requant_factor_i32(x, n, scale);
    for (uint64_t i = 0; i < n; ++i) {
        float t = (float)x[i] * raw;
        t = t + 128.0f;
        q[i] = oracle_usat8(oracle_cvt_rne(t));
    }
}

/* avx512/quantize.cpp:315-361: vcvtdq2ps, vmulps, vcvtps2dq, vpmovsdb. */
void oracle_quantize_i32_i8(const int32_t *x, uint64_t n, int8_t *q, float *scale)
{
    float raw = requant_factor_i32(x, n, scale);
    for (uint64_t i = 0; i < n; ++i) {
        q[i] = oracle_ssat8(oracle_cvt_rne((float)x[i] * raw));
    }
}

/* avx512/quantize.cpp:271-313: vpaddb 0x80 (wraps). */
void oracle_u8_to_i8(const uint8_t *x, uint64_t n, int8_t *q)
{
    for (uint64_t i = 0; i < n; ++i) {
        q[i] = (int8_t)(uint8_t)(x[i] + 0x80u);
    }
}

/* avx512/quantize.cpp:236-269: round() is C round (half away from zero) of the fp32
 * product; bias == NULL copies offsetC, offsetC == NULL leaves the rounded bias. */
void oracle_bias_offsetc(const float *bias, const int32_t *offsetC, uint32_t n, float scaleO,
    int32_t *out)
{
    for (uint32_t i = 0; i < n; ++i) {
        int32_t b = 0;
        if (bias != NULL) {
            float p = bias[i] * scaleO;
            b = (int32_t)roundf(p);
        }
        out[i] = b + (offsetC ? offsetC[i] : 0);
    }
}

/* avx512/dequantize.cpp:18-52: factor = 1/scale; vcvtdq2ps; vmulps. */
void oracle_dequantize_i32_f32(const int32_t *q, uint64_t n, float scale, float *out)
{
    float factor = 1 / scale;
    for (uint64_t i = 0; i < n; ++i) {
        out[i] = (float)q[i] * factor;
    }
}

/* avx512/dequantize.cpp:54-101: (int)q - 128, vcvtdq2ps, vmulps by 1.0f/scale. */
void oracle_dequantize_u8_f32(const uint8_t *q, uint64_t n, float scale, float *out)
{
    float factor = 1.0f / scale;
    for (uint64_t i = 0; i < n; ++i) {
        out[i] = (float)((int32_t)q[i] - 128) * factor;
    }
}
