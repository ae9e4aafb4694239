/*
 * bolt_oracle.h -- TEST INFRASTRUCTURE ONLY.
 *
 * Scalar CPU restatement of the arithmetic of Bolt's x86 AVX512-VNNI quantized
 * inference path (and of the ARMv8.2 1-bit convolution, which has no x86 build).
 * It is the checker for the CUDA library: only the test-suite, the smoke check and
 * the CPU-baseline leg of the benchmark may call it.  Nothing in the product path
 * links, loads or imports it.
 *
 * Every function cites the reference file:line (paths inside huawei-noah/bolt) whose
 * arithmetic it restates.  Plain C, single thread, no intrinsics: float operations
 * are IEEE binary32 with one rounding per operation (build with -ffp-contract=off).
 */
#ifndef BOLT_ORACLE_H
#define BOLT_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- shared scalar helpers -------------------------------------------------- */
/* vcvtps2dq semantics: round-to-nearest-even, out-of-range / NaN -> INT32_MIN. */
int32_t oracle_cvt_rne(float f);
/* vpmovusdb on a dword: the dword is read as UNSIGNED, so negatives become 255. */
uint8_t oracle_usat8(int32_t v);
/* vpmovsdb: signed saturation to [-128,127]. */
int8_t oracle_ssat8(int32_t v);

/* ---- GEMM / GEMV (compute/blas_enhance) ---------------------------------------- */
/* offsetC[n] = -128 * sum_k B[k,n].  b_transposed: B stored [N,K] instead of [K,N]. */
void oracle_offsetc(const int8_t *B, uint32_t K, uint32_t N, int b_transposed, int32_t *offsetC);

/* C = epilogue( C_in + offsetC[n] + sum_k A_u8[m,k] * B_s8[k,n] ).
 * a_transposed: A stored [K,M].  b_transposed: B stored [N,K].
 * scale == NULL       : C is int32 [M,N], accumulated into.
 * scale[0] >= 0       : C is fp32 [M,N]; its incoming BITS are added as int32 first.
 * scale[0] <  0       : C is u8  [M,N]; C_in ignored; factor = scale[1]. */
void oracle_gemm_u8s8(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, int a_transposed,
    const int8_t *B, int b_transposed, const int32_t *offsetC, void *C, const float *scale);

/* y = epilogue( y_in + offsetC[n] + sum_k W_s8[n,k] * x_u8[k] ), W stored [N,K]
 * (w_transposed: [K,N]).  Same scale protocol.  Rows n >= N - N%8 follow the
 * reference's scalar tail: y_in ignored, u8 conversion truncates. */
void oracle_gemv_s8u8(uint32_t N, uint32_t K, const int8_t *W, int w_transposed,
    const uint8_t *x, const int32_t *offsetC, void *y, const float *scale);

/* y = epilogue( -128 * sum_k v[k] + sum_k M_u8[n,k] * v_s8[k] ), M stored [N,K] (m_transposed: [K,N]).
 * The incoming y is never added.  Same scale protocol; the last N%4 rows follow the reference's
 * single-row kernel, whose u8 store keeps the low byte of (rne + 128) unless that sum is >= 255. */
void oracle_gemv_u8s8_row(uint32_t N, uint32_t K, const uint8_t *Mx, int m_transposed, const int8_t *v,
    void *y, const float *scale);

/* ---- quantize / dequantize (compute/tensor) -------------------------------------- */
float oracle_scale_f32(const float *x, uint64_t n);      /* 127/absmax, 1 if absmax==0 */
float oracle_scale_i32(const int32_t *x, uint64_t n);    /* 127.0f/(float)max|x| */
/* mode / *scale handling as quantizeF32ToU8: dynamic unless (mode && *scale > 0). */
void oracle_quantize_f32_u8(const float *x, uint64_t n, uint8_t *q, float *scale, int mode);
void oracle_quantize_f32_i8(const float *x, uint64_t n, int8_t *q, float *scale, int mode);
void oracle_quantize_i32_u8(const int32_t *x, uint64_t n, uint8_t *q, float *scale /*[2]*/);
void oracle_quantize_i32_i8(const int32_t *x, uint64_t n, int8_t *q, float *scale /*[2]*/);
void oracle_u8_to_i8(const uint8_t *x, uint64_t n, int8_t *q);
void oracle_bias_offsetc(const float *bias, const int32_t *offsetC, uint32_t n, float scaleO,
    int32_t *out);
void oracle_dequantize_i32_f32(const int32_t *q, uint64_t n, float scale, float *out);
void oracle_dequantize_u8_f32(const uint8_t *q, uint64_t n, float scale, float *out);
int oracle_pooling_u8(uint32_t n, uint32_t c, uint32_t ih, uint32_t iw, uint32_t oh, uint32_t ow, uint32_t kh, uint32_t kw,
    uint32_t sh, uint32_t sw, uint32_t pt, uint32_t pl, int mode, int count_include_pad, const uint8_t *in, uint8_t *out,
    float *scale);

/* ---- int8 convolution ------------------------------------------------------------ */
typedef struct {
    uint32_t n, ic, ih, iw;       /* input  u8, channel-blocked NCHWc{cin_block}      */
    uint32_t oc, fh, fw;          /* filter s8, plain NCHW [oc, ic, fh, fw]           */
    uint32_t stride_h, stride_w, pad_t, pad_b, pad_l, pad_r, dil_h, dil_w;
    uint32_t cin_block;           /* 8 or 16 (0 = plain NCHW)                         */
    uint32_t cout_block;          /* 8 or 16: output is NCHWc{cout_block}             */
    uint32_t relu;                /* 0 / 1                                            */
    uint32_t out_u8;              /* 0: fp32 output; 1: u8 output, dynamic requantize */
} oracle_conv_shape;

void oracle_conv_out_hw(const oracle_conv_shape *s, uint32_t *oh, uint32_t *ow);
/* scale[0]=input scale, scale[1]=output scale (written when out_u8), scale[2]=filter scale.
 * acc32 (optional, may be NULL) receives the int32 accumulators in output layout. */
void oracle_conv_int8(const oracle_conv_shape *s, const uint8_t *in, const int8_t *filter,
    const float *bias, const float *eltwise, void *out, float *scale, int32_t *acc32);

/* ---- 1-bit convolution --------------------------------------------------------------- */
uint16_t oracle_f32_to_f16(float f);
float oracle_f16_to_f32(uint16_t h);
uint16_t oracle_f16_fma(uint16_t a, uint16_t b, uint16_t c);   /* one rounding */
uint16_t oracle_i32_to_f16(int32_t v);                         /* scvtf/ucvtf, RNE */

typedef struct {
    uint32_t n, ic, ih, iw, oc, fh, fw;
    uint32_t stride_h, stride_w, pad_t, pad_b, pad_l, pad_r;
    uint32_t xnor;                /* 1: DT_BIN11 (bits are +-1, pad = -1); 0: DT_BIN01 */
} oracle_bnn_shape;
/* in: fp16 NCHWc8 activations; filter_bits: NCHW bit-packed MSB-first along the
 * flattened [oc][ic][fh][fw] index; scale/bias: fp16 [oc]; out: fp16 NCHWc8. */
void oracle_bnn_conv(const oracle_bnn_shape *s, const uint16_t *in, const uint8_t *filter_bits,
    const uint16_t *scale, const uint16_t *bias, uint16_t *out, int32_t *sum32);

#ifdef __cplusplus
}
#endif
#endif
