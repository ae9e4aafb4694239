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

/* mvm_avx512_vnni_row.cpp:931-1028 (driver: offset = -128 * sum of the vector, :940-983; rows in
 * groups of 16 / 8 / 4, the rest one by one, :1012-1024), :384-406, :632-640, :786-791 (vpmovusdb
 * in the multi-row kernels) and :884-900 (single-row kernel: add 128, signed compare with 255,
 * low byte stored).  The result buffer is only written, never read. */
void oracle_gemv_u8s8_row(uint32_t N, uint32_t K, const uint8_t *Mx, int m_transposed, const int8_t *v,
    void *y, const float *scale)
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
    int32_t off = 0;
    for (uint32_t k = 0; k < K; ++k) {
        off += v[k];
    }
    off *= -128;
    uint32_t single_begin = N - (N % 4);
    for (uint32_t n = 0; n < N; ++n) {
        int32_t acc = off;
        for (uint32_t k = 0; k < K; ++k) {
            int32_t m = m_transposed ? Mx[(size_t)k * N + n] : Mx[(size_t)n * K + k];
            acc += m * (int32_t)v[k];
        }
        if (mode == 0) {
            ((int32_t *)y)[n] = acc;
        } else if (mode == 1) {
            ((float *)y)[n] = (float)acc * factor;
        } else if (n >= single_begin) {
            int32_t t = (int32_t)((uint32_t)oracle_cvt_rne((float)acc * factor) + 128u);
            ((uint8_t *)y)[n] = (t < 255) ? (uint8_t)t : 255;
        } else {
            ((uint8_t *)y)[n] = acc_to_u8(acc, factor);
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

/* ------------------------------------------------------------------------------ */
/* u8 pooling on NCHWc16 (compute/tensor/src/cpu/x86/int8/avx512/pooling_int8.cpp)  */
/* ------------------------------------------------------------------------------ */

/* pooling_uint8, :317-429.  mode 0 = max (vpmaxub over the clipped window), 1 = mean: the sum of the window
 * minus 128 per element, times poolSize = 65536 / (KH*KW) -- or 65536 / (clipped size) when padding is not
 * counted -- as a 32-bit product (vpmulld), LOGICAL shift right by 16 (vpsrld: a negative sum becomes a large
 * word), plus 128, stored with unsigned saturation (vpmovusdb): :277-314.  scale[1] receives the output scale
 * (:362-366).  Returns 0, or 51 (NOT_SUPPORTED) / 2 (NOT_MATCH) where the reference refuses. */
int oracle_pooling_u8(uint32_t n, uint32_t c, uint32_t ih, uint32_t iw, uint32_t oh, uint32_t ow, uint32_t kh_, uint32_t kw_,
    uint32_t sh, uint32_t sw, uint32_t pt, uint32_t pl, int mode, int count_include_pad, const uint8_t *in, uint8_t *out,
    float *scale)
{
    if (pt >= kh_ || pl >= kw_) {
        return 51;
    }
    if (c % 16 != 0) {
        return 2;
    }
    const int32_t shift = 65536;
    const int32_t factor = shift / (int32_t)(kh_ * kw_);
    if (factor < 1 || (mode != 0 && mode != 1)) {
        return 51;
    }
    if (scale != NULL) {
        scale[1] = (mode == 0) ? scale[0] : scale[0] * factor * (kw_ * kh_) / (float)shift;
    }
    const uint32_t cb = c / 16;
    for (uint32_t img = 0; img < n * cb; ++img) {
        const uint8_t *src = in + (size_t)img * ih * iw * 16;
        uint8_t *dst = out + (size_t)img * oh * ow * 16;
        for (uint32_t h = 0; h < oh; ++h) {
            for (uint32_t w = 0; w < ow; ++w) {
                int hs = (int)(h * sh) - (int)pt, ws = (int)(w * sw) - (int)pl;
                int he = hs + (int)kh_ < (int)ih ? hs + (int)kh_ : (int)ih;
                int we = ws + (int)kw_ < (int)iw ? ws + (int)kw_ : (int)iw;
                hs = hs > 0 ? hs : 0;
                ws = ws > 0 ? ws : 0;
                const int kh = he - hs, kw = we - ws;
                const int32_t pool = count_include_pad ? factor : shift / (kh * kw);
                for (int ch = 0; ch < 16; ++ch) {
                    if (mode == 0) {
                        uint8_t m = src[((size_t)hs * iw + ws) * 16 + ch];
                        for (int y = hs; y < he; ++y) {
                            for (int x = ws; x < we; ++x) {
                                const uint8_t v = src[((size_t)y * iw + x) * 16 + ch];
                                m = v > m ? v : m;
                            }
                        }
                        dst[((size_t)h * ow + w) * 16 + ch] = m;
                    } else {
                        int32_t acc = -128 * kh * kw;
                        for (int y = hs; y < he; ++y) {
                            for (int x = ws; x < we; ++x) {
                                acc += src[((size_t)y * iw + x) * 16 + ch];
                            }
                        }
                        const uint32_t prod = (uint32_t)acc * (uint32_t)pool;   /* vpmulld: low 32 bits */
                        const uint32_t v = (prod >> 16) + 128u;
                        dst[((size_t)h * ow + w) * 16 + ch] = (uint8_t)(v > 255u ? 255u : v);
                    }
                }
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------ */
/* int8 convolution                                                               */
/* ------------------------------------------------------------------------------ */

/* compute/tensor/src/convolution.cpp:28-145 (convolution_infer_output_size) */
void oracle_conv_out_hw(const oracle_conv_shape *s, uint32_t *oh, uint32_t *ow)
{
    uint32_t fhd = (s->fh - 1) * s->dil_h + 1, fwd = (s->fw - 1) * s->dil_w + 1;
    *oh = (s->ih + s->pad_t + s->pad_b - fhd) / s->stride_h + 1;
    *ow = (s->iw + s->pad_l + s->pad_r - fwd) / s->stride_w + 1;
}

/* element offset of channel c, pixel (h, w) of image n in a channel-blocked tensor whose blocks
 * are `blk` channels wide with one narrower tail block (avx512/convolution_direct.cpp:2766,
 * simdOc = min(16, ocSize)); blk == 0 is plain NCHW */
static size_t blocked_off(uint32_t n, uint32_t C, uint32_t H, uint32_t W, uint32_t blk, uint32_t c,
    uint32_t h, uint32_t w)
{
    if (blk == 0) {
        return (((size_t)n * C + c) * H + h) * W + w;
    }
    uint32_t b = c / blk;
    uint32_t width = (C - b * blk < blk) ? (C - b * blk) : blk; /* tail block */
    return ((size_t)n * C + (size_t)b * blk) * H * W + ((size_t)h * W + w) * width + (c - b * blk);
}

/* avx512/convolution_direct.cpp:2584-2809 and convolution_1x1_direct.cpp:2073-2327:
 * scaleO = scaleI * scaleF (:2687); offsetC + round(bias * scaleO) (:2703-2707, quantize.cpp:259-266);
 * padding value 128 (transform_functions_int8.h:41,67-79), i.e. padded taps cancel exactly;
 * fp32 output: (float)acc * (1/scaleO), + eltwise, max(0) (:2133-2165);
 * u8 output: ReLU on int32, then quantizeI32ToU8 with a dynamic scale over the whole tensor,
 * scale[1] = scaleO * raw written back (:2798-2806); u8 output with an eltwise input: the fp32 result
 * is staged and quantized F32 -> U8_Q with its own dynamic scale (:2693-2695,2798-2806).
 * `relu` carries the activation mode number: the kernels apply ReLU when mode & 3 != 0
 * (flags = mode << 2 tested with `and $0xC`, :2143-2146,2747). */
void oracle_conv_int8(const oracle_conv_shape *s, const uint8_t *in, const int8_t *filter,
    const float *bias, const float *eltwise, void *out, float *scale, int32_t *acc32)
{
    uint32_t oh, ow;
    oracle_conv_out_hw(s, &oh, &ow);
    float scaleO = scale[0] * scale[2];
    float factor = 1 / scaleO;
    size_t total = (size_t)s->n * s->oc * oh * ow;
    int32_t *acc = acc32 ? acc32 : (int32_t *)malloc(total * sizeof(int32_t));
    const int relu = (s->relu & 3u) != 0;
    const int staged_f32 = s->out_u8 && eltwise != NULL;
    float *fout = staged_f32 ? (float *)malloc(total * sizeof(float)) : (float *)out;
    for (uint32_t n = 0; n < s->n; ++n) {
        for (uint32_t o = 0; o < s->oc; ++o) {
            int32_t b = 0;
            if (bias != NULL) {
                float p = bias[o] * scaleO;
                b = (int32_t)roundf(p);
            }
            for (uint32_t y = 0; y < oh; ++y) {
                for (uint32_t x = 0; x < ow; ++x) {
                    int32_t a = b;
                    for (uint32_t c = 0; c < s->ic; ++c) {
                        for (uint32_t kh = 0; kh < s->fh; ++kh) {
                            int32_t iy = (int32_t)(y * s->stride_h + kh * s->dil_h) - (int32_t)s->pad_t;
                            if (iy < 0 || iy >= (int32_t)s->ih) {
                                continue; /* pad: (128 - 128) * w */
                            }
                            for (uint32_t kw = 0; kw < s->fw; ++kw) {
                                int32_t ix = (int32_t)(x * s->stride_w + kw * s->dil_w) - (int32_t)s->pad_l;
                                if (ix < 0 || ix >= (int32_t)s->iw) {
                                    continue;
                                }
                                int32_t xv = in[blocked_off(n, s->ic, s->ih, s->iw, s->cin_block, c,
                                    (uint32_t)iy, (uint32_t)ix)];
                                int32_t wv = filter[(((size_t)o * s->ic + c) * s->fh + kh) * s->fw + kw];
                                a += (xv - 128) * wv;
                            }
                        }
                    }
                    size_t off = blocked_off(n, s->oc, oh, ow, s->cout_block, o, y, x);
                    if (!s->out_u8 || staged_f32) {
                        float f = (float)a * factor;
                        if (eltwise != NULL) {
                            f = f + eltwise[off];
                        }
                        if (relu) {
                            f = (f > 0) ? f : 0.0f; /* vmaxps(f, 0) */
                        }
                        fout[off] = f;
                        if (acc32) {
                            acc[off] = a;
                        }
                    } else {
                        if (relu && a < 0) {
                            a = 0; /* vpmaxsd(acc, 0) */
                        }
                        acc[off] = a;
                    }
                }
            }
        }
    }
    if (staged_f32) {
        float sc = -1;
        oracle_quantize_f32_u8(fout, total, (uint8_t *)out, &sc, 0);
        scale[1] = sc;
        free(fout);
    } else if (s->out_u8) {
        float sc[2] = {-1, scaleO};
        oracle_quantize_i32_u8(acc, total, (uint8_t *)out, sc);
        scale[1] = sc[0];
    } else {
        scale[1] = scaleO;
    }
    if (!acc32) {
        free(acc);
    }
}

/* ------------------------------------------------------------------------------ */
/* 1-bit convolution (ARMv8.2 semantics; no x86 build exists, so this part of the  */
/* oracle is pinned only by hand-checkable cases: "parity unpinned")              */
/* ------------------------------------------------------------------------------ */

float oracle_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* exact value v = mant * 2^e2 (mant may be any signed 128-bit integer) -> binary16, RNE */
static uint16_t round_to_f16(__int128 mant, int e2)
{
    if (mant == 0) {
        return 0;
    }
    uint16_t sign = 0;
    if (mant < 0) {
        sign = 0x8000u;
        mant = -mant;
    }
    unsigned __int128 m = (unsigned __int128)mant;
    int msb = 127;
    while (!((m >> msb) & 1)) {
        --msb;
    }
    int e = msb + e2; /* value in [2^e, 2^(e+1)) */
    /* number of fraction bits kept: 10 for normals; subnormals keep down to 2^-24 */
    int lsb_exp = (e < -14) ? -24 : e - 10; /* weight of the last kept bit */
    int shift = lsb_exp - e2;               /* drop `shift` low bits of m */
    unsigned __int128 q;
    if (shift <= 0) {
        q = m << (-shift);
    } else if (shift > 127) {
        q = 0;
    } else {
        unsigned __int128 rem = m & ((((unsigned __int128)1) << shift) - 1);
        unsigned __int128 half = ((unsigned __int128)1) << (shift - 1);
        q = m >> shift;
        if (rem > half || (rem == half && (q & 1))) {
            ++q;
        }
    }
    /* q * 2^lsb_exp; renormalise if rounding carried */
    if (e >= -14) {
        if (q >> 11) {
            q >>= 1;
            ++e;
        }
        if (e > 15) {
            return sign | 0x7C00u; /* overflow -> inf */
        }
        return sign | (uint16_t)((e + 15) << 10) | (uint16_t)(q & 0x3FFu);
    }
    /* subnormal (q may round up to the smallest normal, which this encoding handles) */
    return sign | (uint16_t)q;
}

uint16_t oracle_f32_to_f16(float f)
{
    uint32_t b;
    memcpy(&b, &f, 4);
    uint32_t exp = (b >> 23) & 0xFF, man = b & 0x7FFFFFu;
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    if (exp == 255) {
        return sign | 0x7C00u | (man ? 0x200u : 0);
    }
    if (exp == 0 && man == 0) {
        return sign;
    }
    __int128 m = (exp == 0) ? man : (man | 0x800000u);
    int e2 = (exp == 0 ? 1 : (int)exp) - 127 - 23;
    if (e2 < -200) {
        return sign;
    }
    uint16_t r = round_to_f16(m, e2);
    return (uint16_t)(r | sign);
}

/* scvtf / ucvtf to half precision: RNE (convolution_xnor_A76.cpp:300-312) */
uint16_t oracle_i32_to_f16(int32_t v)
{
    return round_to_f16((__int128)v, 0);
}

/* finite binary16 -> integer multiple of 2^-24 */
static int64_t f16_units(uint16_t h)
{
    int64_t man = h & 0x3FF;
    int exp = (h >> 10) & 0x1F;
    int64_t v = (exp == 0) ? man : ((man | 0x400) << (exp - 1));
    return (h & 0x8000u) ? -v : v;
}

/* fmla in half precision: a * b + c with one rounding (convolution_xnor_A76.cpp:322-374).
 * Finite inputs only (the convolution never produces anything else from finite scale/bias). */
uint16_t oracle_f16_fma(uint16_t a, uint16_t b, uint16_t c)
{
    __int128 prod = (__int128)f16_units(a) * f16_units(b); /* units of 2^-48 */
    __int128 sum = prod + ((__int128)f16_units(c) << 24);
    if (sum == 0) {
        /* exact zero: sign of +0 unless both addends are negative zeros */
        int pneg = ((a ^ b) & 0x8000u) != 0, cneg = (c & 0x8000u) != 0;
        return (pneg && cneg) ? 0x8000u : 0;
    }
    return round_to_f16(sum, -48);
}

/* B3 (common/uni/include/data_type.h:197-233): bit = (x >= 0) for DT_BIN11, (x >= 0.5) for DT_BIN01.
 * B4 (cpu/arm/bnn/convolution_xnor_A76.cpp:67-79,300-374): zero-bit padding (= -1),
 *    sum = fh*fw*ic - 2*popcount(x XOR w) in int16, out = fma_f16((f16)sum, scale, bias).
 * B5 (cpu/arm/bnn/convolution_dorefa_A76.cpp:167-199,290-306): zero padding, sum = popcount(x AND w).
 * Filter bits: NCHW, MSB first (cpu/general/convolution.cpp:161-179). Input / output: fp16 NCHWc8. */
void oracle_bnn_conv(const oracle_bnn_shape *s, const uint16_t *in, const uint8_t *filter_bits,
    const uint16_t *scale, const uint16_t *bias, uint16_t *out, int32_t *sum32)
{
    uint32_t oh = (s->ih + s->pad_t + s->pad_b - s->fh) / s->stride_h + 1;
    uint32_t ow = (s->iw + s->pad_l + s->pad_r - s->fw) / s->stride_w + 1;
    size_t npix = (size_t)s->n * s->ic * s->ih * s->iw;
    uint8_t *xb = (uint8_t *)malloc(npix);
    float thr = s->xnor ? 0.0f : 0.5f;
    for (size_t i = 0; i < npix; ++i) {
        xb[i] = oracle_f16_to_f32(in[i]) >= thr;
    }
    for (uint32_t n = 0; n < s->n; ++n) {
        for (uint32_t o = 0; o < s->oc; ++o) {
            for (uint32_t y = 0; y < oh; ++y) {
                for (uint32_t x = 0; x < ow; ++x) {
                    int32_t sum = 0;
                    for (uint32_t c = 0; c < s->ic; ++c) {
                        for (uint32_t kh = 0; kh < s->fh; ++kh) {
                            for (uint32_t kw = 0; kw < s->fw; ++kw) {
                                size_t fp = (((size_t)o * s->ic + c) * s->fh + kh) * s->fw + kw;
                                int wbit = (filter_bits[fp / 8] >> (7 - fp % 8)) & 1;
                                int32_t iy = (int32_t)(y * s->stride_h + kh) - (int32_t)s->pad_t;
                                int32_t ix = (int32_t)(x * s->stride_w + kw) - (int32_t)s->pad_l;
                                int xbit = 0; /* padding is a zero bit in both modes */
                                if (iy >= 0 && iy < (int32_t)s->ih && ix >= 0 && ix < (int32_t)s->iw) {
                                    xbit = xb[blocked_off(n, s->ic, s->ih, s->iw, 8, c, (uint32_t)iy, (uint32_t)ix)];
                                }
                                if (s->xnor) {
                                    sum += (xbit == wbit) ? 1 : -1;
                                } else {
                                    sum += xbit & wbit;
                                }
                            }
                        }
                    }
                    size_t off = blocked_off(n, s->oc, oh, ow, 8, o, y, x);
                    if (sum32) {
                        sum32[off] = sum;
                    }
                    out[off] = oracle_f16_fma(oracle_i32_to_f16((int16_t)sum), scale[o], bias[o]);
                }
            }
        }
    }
    free(xb);
}
