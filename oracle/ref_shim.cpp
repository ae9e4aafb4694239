// ref_shim.cpp -- TEST INFRASTRUCTURE ONLY.
//
// Thin extern "C" harness around the UNMODIFIED reference (huawei-noah/bolt) x86
// AVX512-VNNI int8 path.  It is compiled together with the reference's own source
// files, taken from where they lie in the mounted reference tree, into
// oracle/_ref/libbolt_ref.so (see oracle/Makefile).  The harness only sequences the
// reference's public calls the way its own tests do
// (compute/blas_enhance/tests/test_mmm.cpp:69-91, test_mvm.cpp:60-100,
// compute/tensor/tests/test_convolution_int8.cpp:60-140); it holds no arithmetic.
//
// Used to (1) validate the scalar restatement in bolt_oracle.c, (2) generate the
// golden fixtures under tests/golden/, (3) time the reference's CPU path
// (cpu_baseline.kind = "reference").  Needs a host CPU with avx512_vnni.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "uni.h"
#include "blas_enhance.h"
#include "cpu/x86/tensor_computing_x86.h"
#include "cpu/x86/int8/tensor_computing_int8.h"
#include "affinity_policy.h"

namespace {
struct Buf {
    void *p = nullptr;
    explicit Buf(size_t n)
    {
        if (posix_memalign(&p, 64, n + 256) != 0) {
            p = nullptr;
        }
        if (p) {
            memset(p, 0, n + 256);
        }
    }
    ~Buf()
    {
        free(p);
    }
};
DataType c_dtype(int out_kind)
{
    return out_kind == 0 ? DT_I32 : (out_kind == 1 ? DT_F32 : DT_U8_Q);
}
}  // namespace

extern "C" {

void ref_set_threads(int n)
{
    OMP_NUM_THREADS = n;
}

int ref_get_threads()
{
    return OMP_NUM_THREADS;
}

// ---- pre-packed weight handle: pack once, multiply many (timed path) -------------
struct RefGemmPlan {
    uint32_t M, N, K;
    int transA;
    TensorDesc aDesc, bPacked, cDesc;
    Buf *packed;
    Buf *tmp;
    uint32_t tmpBytes, rhsBytes;
};

// out_kind: 0 = int32, 1 = fp32, 2 = u8.  B is s8 [K,N] (transB=0) or [N,K] (transB=1).
RefGemmPlan *ref_gemm_plan(uint32_t M, uint32_t N, uint32_t K, int transA, int transB,
    const int8_t *B, int out_kind)
{
    RefGemmPlan *pl = new RefGemmPlan();
    pl->M = M;
    pl->N = N;
    pl->K = K;
    pl->transA = transA;
    pl->aDesc = transA ? tensor2df(DT_U8_Q, DF_TRANSPOSE, K, M) : tensor2df(DT_U8_Q, DF_NORMAL, M, K);
    TensorDesc bDesc = transB ? tensor2df(DT_I8, DF_TRANSPOSE, N, K) : tensor2df(DT_I8, DF_NORMAL, K, N);
    pl->cDesc = tensor2df(c_dtype(out_kind), DF_NORMAL, M, N);
    U32 bytes = 0, rhsBytes = 0;
    if (matrix_matrix_multiply_transform_rhs_bytes(bDesc, &bytes, &rhsBytes, X86_AVX512) != SUCCESS) {
        delete pl;
        return nullptr;
    }
    pl->rhsBytes = rhsBytes;
    pl->packed = new Buf(bytes);
    if (matrix_matrix_multiply_transform_rhs(bDesc, B, &pl->bPacked, pl->packed->p, X86_AVX512) !=
        SUCCESS) {
        delete pl->packed;
        delete pl;
        return nullptr;
    }
    U32 tmpBytes = 0;
    matrix_matrix_multiply_tmp_bytes(pl->aDesc, pl->bPacked, &tmpBytes, X86_AVX512);
    if (out_kind == 2) {
        tmpBytes += M * N * 4;  // callers add the int32 staging for u8 output (compute/tensor/src/fully_connected.cpp:154-155)
    }
    pl->tmpBytes = tmpBytes;
    pl->tmp = new Buf(tmpBytes);
    return pl;
}

// offsetC_override: if non-null, N int32 values used instead of the packed colsum offset
// (the bias-folded offset a fully-connected caller builds, fully_connected.cpp:400-407).
int ref_gemm_run(RefGemmPlan *pl, const uint8_t *A, void *C, const float *scale,
    const int32_t *offsetC_override)
{
    const void *off = offsetC_override ? (const void *)offsetC_override
                                       : (const void *)((const char *)pl->packed->p + pl->rhsBytes);
    memcpy(pl->tmp->p, off, pl->N * sizeof(int32_t));
    return (int)matrix_matrix_multiply(pl->aDesc, A, pl->bPacked, pl->packed->p, pl->tmpBytes,
        pl->tmp->p, pl->cDesc, C, scale, X86_AVX512);
}

void ref_gemm_offsetc(RefGemmPlan *pl, int32_t *out)
{
    memcpy(out, (const char *)pl->packed->p + pl->rhsBytes, pl->N * sizeof(int32_t));
}

void ref_gemm_free(RefGemmPlan *pl)
{
    if (pl) {
        delete pl->packed;
        delete pl->tmp;
        delete pl;
    }
}

// One-shot GEMM without pre-packing: B is packed inside matrix_matrix_multiply (mmm.cpp:207-219).
int ref_gemm_unpacked(uint32_t M, uint32_t N, uint32_t K, int transA, int transB,
    const uint8_t *A, const int8_t *B, void *C, int out_kind, const float *scale)
{
    TensorDesc aDesc = transA ? tensor2df(DT_U8_Q, DF_TRANSPOSE, K, M) : tensor2df(DT_U8_Q, DF_NORMAL, M, K);
    TensorDesc bDesc = transB ? tensor2df(DT_I8, DF_TRANSPOSE, N, K) : tensor2df(DT_I8, DF_NORMAL, K, N);
    TensorDesc cDesc = tensor2df(c_dtype(out_kind), DF_NORMAL, M, N);
    U32 bytes = 0;
    matrix_matrix_multiply_tmp_bytes(aDesc, bDesc, &bytes, X86_AVX512);
    if (out_kind == 2) {
        bytes += M * N * 4;
    }
    Buf tmp(bytes);
    return (int)matrix_matrix_multiply(aDesc, A, bDesc, B, bytes, tmp.p, cDesc, C, scale, X86_AVX512);
}

// ---- GEMV ------------------------------------------------------------------------
struct RefGemvPlan {
    uint32_t N, K;
    TensorDesc wPacked, xDesc, yDesc;
    Buf *packed;
    Buf *tmp;
    uint32_t tmpBytes;
};

RefGemvPlan *ref_gemv_plan(uint32_t N, uint32_t K, int transW, const int8_t *W, int out_kind)
{
    RefGemvPlan *pl = new RefGemvPlan();
    pl->N = N;
    pl->K = K;
    TensorDesc wDesc = transW ? tensor2df(DT_I8, DF_TRANSPOSE, K, N) : tensor2df(DT_I8, DF_NORMAL, N, K);
    pl->xDesc = tensor1d(DT_U8_Q, K);
    pl->yDesc = tensor1d(c_dtype(out_kind), N);
    U32 bytes = 0;
    matrix_vector_multiply_transform_weight_bytes(wDesc, &bytes, X86_AVX512);
    pl->packed = new Buf(bytes);
    if (matrix_vector_multiply_transform_weight(wDesc, W, &pl->wPacked, pl->packed->p, X86_AVX512) !=
        SUCCESS) {
        delete pl->packed;
        delete pl;
        return nullptr;
    }
    U32 tmpBytes = 0;
    matrix_vector_multiply_tmp_bytes(pl->wPacked, pl->xDesc, &tmpBytes, X86_AVX512);
    tmpBytes += N * 8 + 64;  // offsetC copy + int32 staging used by the u8 mode (mvm_avx512_vnni.cpp:727)
    pl->tmpBytes = tmpBytes;
    pl->tmp = new Buf(tmpBytes);
    return pl;
}

int ref_gemv_run(RefGemvPlan *pl, const uint8_t *x, void *y, const float *scale,
    const int32_t *offsetC_override)
{
    // offsetC sits behind the packed matrix (test_mvm.cpp:85, fully_connected.cpp:404).
    const char *off = (const char *)pl->packed->p + UNI_ALIGN(pl->N, 16) * UNI_ALIGN(pl->K, 8);
    memcpy(pl->tmp->p, offsetC_override ? (const void *)offsetC_override : (const void *)off,
        pl->N * sizeof(int32_t));
    return (int)matrix_vector_multiply(pl->wPacked, pl->packed->p, pl->xDesc, x, pl->tmpBytes,
        pl->tmp->p, pl->yDesc, y, scale, X86_AVX512);
}

void ref_gemv_free(RefGemvPlan *pl)
{
    if (pl) {
        delete pl->packed;
        delete pl->tmp;
        delete pl;
    }
}

// u8 matrix x s8 vector (the GEMV Bolt's matmul uses when the output is a vector, matmul.cpp:376-379).
// Mx: u8 [N,K] (transM=0) or [K,N] (transM=1).
int ref_gemv_row(uint32_t N, uint32_t K, int transM, const uint8_t *Mx, const int8_t *v, void *y, int out_kind,
    const float *scale)
{
    TensorDesc mDesc = transM ? tensor2df(DT_U8_Q, DF_TRANSPOSE, K, N) : tensor2df(DT_U8_Q, DF_NORMAL, N, K);
    TensorDesc vDesc = tensor1d(DT_I8, K);
    TensorDesc yDesc = tensor1d(c_dtype(out_kind), N);
    U32 bytes = 0;
    matrix_vector_multiply_tmp_bytes(mDesc, vDesc, &bytes, X86_AVX512);
    Buf tmp((size_t)bytes + (size_t)N * K + (size_t)N * 8 + 256);
    Buf mcopy((size_t)N * K + 256);  // the kernels read whole 64-byte vectors: keep slack behind the matrix
    memcpy(mcopy.p, Mx, (size_t)N * K);
    Buf vcopy((size_t)K + 256);
    memcpy(vcopy.p, v, K);
    return (int)matrix_vector_multiply(mDesc, mcopy.p, vDesc, vcopy.p, bytes + N * K + N * 8, tmp.p, yDesc, y, scale,
        X86_AVX512);
}

// ---- quantize / dequantize ---------------------------------------------------------
// src_kind / dst_kind use Bolt DataType numbers (DT_F32=6, DT_I32=3, DT_U8_Q=10, DT_I8=1).
int ref_quantize(uint32_t n, int src_dt, const void *src, int dst_dt, void *dst, float *scale, int mode)
{
    TensorDesc d = tensor1d((DataType)src_dt, n);
    TensorDesc q = tensor1d((DataType)dst_dt, n);
    return (int)quantize_x86(d, src, &q, dst, scale, mode);
}

int ref_dequantize(uint32_t n, int src_dt, void *src, const float *scale, float *dst)
{
    TensorDesc q = tensor1d((DataType)src_dt, n);
    TensorDesc d = tensor1d(DT_F32, n);
    TensorDesc b = tensor1d(DT_F32, 0);
    return (int)dequantize_x86(q, src, scale, b, nullptr, d, dst);
}

// filter_has_offset: offsetC points at N int32 (the packed-weight offset) or null.
int ref_bias_offsetc(uint32_t n, const float *bias, const int32_t *offsetC, float scaleO, int32_t *out)
{
    TensorDesc biasDesc = tensor1d(DT_F32, bias ? n : 0);
    // any non-native format makes the reference read offsetC from `filter`
    TensorDesc fDesc = tensor2df(DT_I8, offsetC ? DF_NKNxKx : DF_NORMAL, n, n);
    return (int)quantize_bias_offsetC(bias, biasDesc, DT_I32, offsetC, fDesc, &scaleO, out);
}

// ---- int8 convolution ----------------------------------------------------------------
struct RefConvPlan {
    TensorDesc inDesc, fDesc, ftmDesc, biasDesc, outDesc;
    ConvolutionParamSpec p;
    ConvolutionForwardAlgorithm alg;
    ActivationParamSpec act;
    Buf *ftm;
    Buf *tmp;
    uint32_t tmpBytes;
};

// in_df: 0 = NCHW, 8 = NCHWc8, 16 = NCHWc16.  out_u8: 0 fp32 output, 1 u8 output.
// The output layout is c16 blocks whenever oc % 16 == 0 (convolution_direct.cpp:2663) --
// out_df reports what the caller asked the desc to say; the kernels decide themselves.
RefConvPlan *ref_conv_plan(uint32_t n, uint32_t ic, uint32_t ih, uint32_t iw, uint32_t oc, uint32_t fh,
    uint32_t fw, uint32_t stride, uint32_t pad, int in_df, int out_df, int out_u8, int relu,
    const int8_t *filter /* NCHW s8 */)
{
    RefConvPlan *pl = new RefConvPlan();
    memset(&pl->p, 0, sizeof(pl->p));
    pl->p.num_outputs = oc;
    pl->p.num_outputs_origin = oc;
    pl->p.kernel_t = 1;
    pl->p.kernel_h = fh;
    pl->p.kernel_w = fw;
    pl->p.stride_t = 1;
    pl->p.stride_h = stride;
    pl->p.stride_w = stride;
    pl->p.pad_top = pl->p.pad_bottom = pl->p.pad_left = pl->p.pad_right = pad;
    pl->p.group = 1;
    pl->p.dilatedRate_t = pl->p.dilatedRate_h = pl->p.dilatedRate_w = 1;
    pl->p.convolution_type = CONVOLUTION_POINTWISE;
    pl->p.dw_activation_type = ACTIVATION_NULL;
    // `relu` is the activation mode number (0 none, 1 ReLU, others as the caller's model would carry them)
    pl->p.pw_activation_type = (ActivationMode)relu;
    pl->act.mode = (ActivationMode)relu;
    uint32_t oh = (ih + 2 * pad - fh) / stride + 1;
    uint32_t ow = (iw + 2 * pad - fw) / stride + 1;
    DataFormat idf = in_df == 16 ? DF_NCHWC16 : (in_df == 8 ? DF_NCHWC8 : DF_NCHW);
    DataFormat odf = out_df == 16 ? DF_NCHWC16 : DF_NCHWC8;
    pl->inDesc = tensor4df(DT_U8_Q, idf, n, ic, ih, iw);
    pl->fDesc = tensor4df(DT_I8, DF_NCHW, oc, ic, fh, fw);
    pl->biasDesc = tensor1d(DT_F32, oc);
    pl->outDesc = tensor4df(out_u8 ? DT_U8_Q : DT_F32, odf, n, oc, oh, ow);
    pl->alg = (fh == 1 && fw == 1) ? CONVOLUTION_ALGORITHM_POINTWISE : CONVOLUTION_ALGORITHM_DIRECT;
    // bytes as convolution_transform_filter_bytes_x86 (cpu/x86/convolution.cpp:141-166):
    // ALIGN(fn,8) * ALIGN(fc,16) * fh * fw + 4 * fn + 32
    U32 fbytes = UNI_ALIGN(oc, 8) * UNI_ALIGN(ic, 16) * fh * fw + 4 * oc + 32;
    pl->ftm = new Buf(fbytes);
    if (convolution_transform_filter_int8(pl->fDesc, filter, pl->p, pl->alg, &pl->ftmDesc,
            (INT8 *)pl->ftm->p) != SUCCESS) {
        delete pl->ftm;
        delete pl;
        return nullptr;
    }
    U32 tmpBytes = 0;
    convolution_infer_forward_tmp_bytes_int8(pl->inDesc, pl->ftmDesc, pl->outDesc, pl->p, pl->alg, &tmpBytes);
    pl->tmpBytes = tmpBytes;
    pl->tmp = new Buf(tmpBytes);
    return pl;
}

// scale[3] = {input scale, output scale (in: -1 for dynamic; out: written), filter scale}
int ref_conv_run(RefConvPlan *pl, uint8_t *in, float *eltwise, const float *bias, void *out, float *scale)
{
    return (int)convolution_int8(pl->inDesc, in, eltwise, pl->ftmDesc, (const INT8 *)pl->ftm->p, pl->p,
        pl->alg, pl->biasDesc, bias, pl->tmpBytes, pl->tmp->p, pl->outDesc, out, scale, pl->act,
        X86_AVX512);
}

void ref_conv_free(RefConvPlan *pl)
{
    if (pl) {
        delete pl->ftm;
        delete pl->tmp;
        delete pl;
    }
}


// ---- u8 pooling (cpu/x86/int8/avx512/pooling_int8.cpp: pooling_uint8) --------------------------
int ref_pooling_u8(uint32_t n, uint32_t c, uint32_t ih, uint32_t iw, uint32_t oh, uint32_t ow, uint32_t kh, uint32_t kw,
    uint32_t sh, uint32_t sw, uint32_t pt, uint32_t pl, int mode, int count_include_pad, const uint8_t *in, uint8_t *out,
    float *scale)
{
    PoolingParamSpec p;
    memset(&p, 0, sizeof(p));
    p.kernel_t = 1;
    p.kernel_h = kh;
    p.kernel_w = kw;
    p.stride_t = 1;
    p.stride_h = sh;
    p.stride_w = sw;
    p.pad_top = pt;
    p.pad_bottom = pt;
    p.pad_left = pl;
    p.pad_right = pl;
    p.round_mode = ROUND_CEIL;
    p.mode = mode == 0 ? POOLING_MAX : POOLING_MEAN;
    p.count_include_pad = count_include_pad != 0;
    TensorDesc inDesc = tensor4df(DT_U8_Q, DF_NCHWC16, n, c, ih, iw);
    TensorDesc outDesc = tensor4df(DT_U8_Q, DF_NCHWC16, n, c, oh, ow);
    return (int)pooling_uint8(inDesc, in, p, outDesc, out, scale);
}
}  // extern "C"
