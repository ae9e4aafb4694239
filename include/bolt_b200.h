/*
 * bolt_b200.h -- C ABI of libbolt_b200.so: Bolt's quantized-inference hot path on NVIDIA B200.
 *
 * Three groups of entry points, all `extern "C"`, plain pointers and sizes:
 *
 *   1. runtime      bolt_b200_*           device, stream, memory, status
 *   2. kernels      *_cuda_b200           one-to-one with the per-architecture functions that
 *                                         Bolt's dispatchers call for x86 (`*_x86`); these are the
 *                                         symbols a `CUDA_B200` branch in Bolt's dispatchers binds
 *   3. operators    b200_*                Bolt's public blas_enhance / tensor signatures
 *                                         (TensorDesc by value, Arch last) for users that do not
 *                                         link Bolt itself; they check arguments like Bolt's
 *                                         dispatchers and forward to group 2
 *
 * Every comment "replaces <file>:<line>" names the function of huawei-noah/bolt whose contract the
 * entry point follows (paths relative to the Bolt source tree).
 *
 * Pointers may be device pointers (used in place, work is enqueued on the current stream and the
 * call returns without waiting) or host pointers (staged through an internal device workspace;
 * the call returns after the result is back in host memory).  `scale` arguments and `U32 *bytes`
 * outputs are always host pointers, as in Bolt.
 *
 * Errors are returned as EE codes; the library never prints and never exits.
 */
#ifndef BOLT_B200_H
#define BOLT_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef BOLT_B200_WITH_BOLT_HEADERS
/* Building inside Bolt: take the real definitions. */
#include "sys.h"
#include "error.h"
#include "tensor_desc.h"
#include "parameter_spec.h"
#else
/* Stand-alone: ABI-identical mirrors of the few Bolt types the path uses. */
typedef int8_t INT8;
typedef uint8_t UINT8;
typedef int32_t I32;
typedef uint32_t U32;
typedef float F32;
typedef uint16_t F16; /* raw IEEE binary16 bits, as Bolt's non-ARM builds (data_type.h:30) */

/* common/uni/include/error.h:159-170 */
typedef enum {
    SUCCESS = 0,
    NULL_POINTER = 1,
    NOT_MATCH = 2,
    NOT_FOUND = 3,
    ALLOC_FAILED = 4,
    NOT_IMPLEMENTED = 50,
    NOT_SUPPORTED = 51,
    GCL_ERROR = 52,
    FILE_ERROR = 53,
    UNKNOWN = 99
} EE;

/* common/uni/include/sys.h:44-55; CUDA_B200 is the one added value. */
typedef enum {
    CPU_GENERAL = 1,
    MALI = 2,
    ARM_V7 = 3,
    ARM_V8 = 4,
    ARM_A55 = 5,
    ARM_A76 = 6,
    QUALCOMM = 7,
    X86_AVX2 = 8,
    X86_AVX512 = 9,
    X86_AVXVNNI = 10,
    CUDA_B200 = 11
} Arch;

typedef struct {
    Arch arch;
    void *archPara; /* for CUDA_B200: NULL or a bolt_b200_para* */
} ArchInfo;
typedef ArchInfo *ArchInfo_t;

/* common/uni/include/data_type.h:67-85 (32-bit enums in Bolt's non-LITE build) */
typedef uint32_t DataType;
enum {
    DT_U8 = 0,
    DT_I8 = 1,
    DT_U32 = 2,
    DT_I32 = 3,
    DT_F16 = 4,
    DT_F16_8Q = 5,
    DT_F32 = 6,
    DT_BIN01 = 7,
    DT_BIN11 = 8,
    DT_F32_8Q = 9,
    DT_U8_Q = 10
};

/* common/uni/include/tensor_desc.h:33-78 -- only the values the path touches */
typedef uint32_t DataFormat;
enum {
    DF_NCHW = 0,
    DF_NCHWC8 = 2,
    DF_NCHWN16C8 = 9,
    DF_TRANSPOSE = 13,
    DF_NORMAL = 14,
    DF_NK = 17,
    DF_NKN32K4 = 21,
    DF_NKNxKx = 39,
    DF_NCHWC16 = 41,
    DF_NCHWC2NxC4 = 42
};

/* common/uni/include/tensor_desc.h:93-100: dims[0] is the innermost extent. */
#pragma pack(push, 8)
typedef struct TensorDesc {
    DataType dt;
    DataFormat df;
    U32 nDims;
    U32 dims[20];
} TensorDesc;
#pragma pack(pop)

/* common/uni/include/parameter_spec.h:60-87 (values used), :150-169, :256-283 */
typedef uint32_t ActivationMode;
enum { ACTIVATION_NULL = 0, ACTIVATION_RELU = 1 };
typedef uint32_t ConvolutionForwardAlgorithm;
enum {
    CONVOLUTION_ALGORITHM_POINTWISE = 0,
    CONVOLUTION_ALGORITHM_DIRECT = 1,
    CONVOLUTION_ALGORITHM_BNN = 6,
    CONVOLUTION_ALGORITHM_NULL = 9
};
typedef uint32_t ConvolutionPolicy;
#pragma pack(push, 8)
typedef struct ActivationParamSpec {
    ActivationMode mode;
    float value[4];
} ActivationParamSpec;
typedef struct {
    U32 num_outputs;
    U32 kernel_t, kernel_h, kernel_w;
    U32 stride_t, stride_h, stride_w;
    U32 pad_before, pad_after, pad_top, pad_bottom, pad_left, pad_right;
    U32 group;
    U32 dilatedRate_t, dilatedRate_h, dilatedRate_w;
    U32 num_outputs_origin;
    uint32_t convolution_type;
    ActivationMode dw_activation_type;
    ActivationMode pw_activation_type;
    float activation_spec[2]; /* ActivationSpec union (parameter_spec.h:244-247), 8 bytes */
    uint32_t round_mode;
    U32 output_pad_t, output_pad_h, output_pad_w;
} ConvolutionParamSpec;
typedef uint32_t PoolingMode;
enum { POOLING_MAX = 0, POOLING_MEAN = 1 };
typedef struct {
    U32 kernel_t, kernel_h, kernel_w;
    U32 stride_t, stride_h, stride_w;
    U32 pad_before, pad_after, pad_top, pad_bottom, pad_left, pad_right;
    uint32_t round_mode;
    PoolingMode mode;
    bool count_include_pad;
} PoolingParamSpec; /* parameter_spec.h:285-301 */
#pragma pack(pop)
#endif /* BOLT_B200_WITH_BOLT_HEADERS */

#ifdef __cplusplus
extern "C" {
#endif

/* ============================== 1. runtime =============================================== */

/* What ArchInfo.archPara points at for CUDA_B200 (the slot Bolt's Mali backend uses for its
 * handle, compute/tensor/src/convolution.cpp:181-183). */
typedef struct {
    int device;
    void *stream; /* cudaStream_t */
} bolt_b200_para;
/* What a dispatcher's CUDA_B200 branch calls first with ArchInfo.archPara: selects the device and stream of
 * the calling thread's later calls.  NULL: the thread's current CUDA device and the default stream. */
EE bolt_b200_use_para(const bolt_b200_para *para);

/* Select the CUDA device used by the calling thread's later calls.  Without it the library follows the
 * CUDA device that is current in the calling thread (cudaGetDevice).  GEMM / GEMV calls return NOT_MATCH for
 * a data pointer that lives on another GPU. */
EE bolt_b200_set_device(int device);
/* Stream used by the calling thread's later calls (default: the legacy default stream). */
EE bolt_b200_set_stream(void *cuda_stream);
/* Wait for the current stream; returns UNKNOWN if a kernel recorded a device-side error
 * (a bounded wait that ran out) since the last call. */
EE bolt_b200_synchronize(void);
/* Device-side error word of the current device (0 = none); reading it clears it. */
int bolt_b200_device_status(void);
/* 0 (default): classify every pointer with cudaPointerGetAttributes.
 * 1: the caller promises that all data pointers are device pointers (skips the query). */
EE bolt_b200_set_pointer_mode(int device_only);
/* Device memory for callers without a CUDA runtime of their own. */
void *bolt_b200_malloc(size_t bytes);
void bolt_b200_free(void *p);
EE bolt_b200_memcpy_h2d(void *dst, const void *src, size_t bytes);
EE bolt_b200_memcpy_d2h(void *dst, const void *src, size_t bytes);
/* A packed weight written into HOST memory by a transform call keeps a device-resident twin,
 * found again by the host address.  Drop it before the host buffer is freed or reused. */
EE bolt_b200_release_weight(const void *host_packed);
/* Measurement aid, no counterpart in Bolt: the rate at which the GPU retires tcgen05.mma.kind::i8 when
 * nothing else limits it -- every SM issues mma_per_sm MMAs of 128 x 256 x 32 back to back on operands
 * resident in shared memory (no loads, no stores).  The ceiling the int8 GEMM and convolution kernels are
 * compared with.  Blocks until the run is over; a short run (a millisecond) gives the burst figure, one of
 * seconds the figure under the board's power limit. */
EE bolt_b200_i8_mma_rate(U32 mma_per_sm, F32 *milliseconds, F32 *tops);
/* Self-test of the bounded waits every kernel of this library uses on its barriers: launches one block
 * that waits, with a limit of `limit_cycles` SM cycles (1 .. 2e9), on a barrier nobody arrives on.  The
 * wait gives up, the kernel stores 21 in the device status word and returns; the next
 * bolt_b200_synchronize() therefore returns UNKNOWN (and clears the word), and later calls work as
 * before.  No counterpart in the reference. */
EE bolt_b200_selftest_wait_limit(U32 limit_cycles);
/* Number of kernels this library has launched in this process (all threads). */
uint64_t bolt_b200_launch_count(void);
/* 1 if the u8 x s8 tensor-core (tcgen05) GEMM was used by the last GEMM call of this thread. */
int bolt_b200_last_gemm_used_tensor_cores(void);

/* ============================== 2. kernels ================================================ */

/* ---- GEMM: C[M,N] (+)= A_u8[M,K] * B_s8[K,N] ------------------------------------------ */

/* replaces compute/blas_enhance/src/cpu/x86/mmm.cpp:54-76
 * (matrix_matrix_multiply_transform_rhs_bytes_x86 -> mmm_avx512_vnni.cpp:22-40).
 * rhsBytes = ALIGN(N,16)*ALIGN(K,8); bytes = rhsBytes + 4N + 64; both 0 for a packed format.
 * The int32 offsetC[N] = -128*colsum(B) sits at packed + rhsBytes, where Bolt's callers read it
 * (blas_enhance/tests/test_mmm.cpp:84, tensor/src/fully_connected.cpp:404). */
EE matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(
    U32 N, U32 K, DataType bdt, DataFormat bdf, U32 *bytes, U32 *rhsBytes);

/* replaces cpu/x86/mmm.cpp:129-152 (matrix_matrix_multiply_transform_rhs_x86).
 * src: s8 [K,N] (DF_NORMAL) or [N,K] (DF_TRANSPOSE).  dst layout (opaque to callers):
 * ALIGN(N,16) rows of ALIGN(K,8) bytes, K contiguous, zero padded -- the K-major operand
 * layout the tensor-core kernel loads with TMA -- then offsetC.  descTran->df = DF_NKNxKx. */
EE matrix_matrix_multiply_transform_rhs_cuda_b200(
    const TensorDesc *desc, const void *src, TensorDesc *descTran, void *dst);

/* replaces cpu/x86/mmm.cpp:22-52 (matrix_matrix_multiply_tmp_bytes_x86):
 * packed-B bytes if B is not packed yet, plus 4N + 64 for offsetC. */
EE matrix_matrix_multiply_tmp_bytes_cuda_b200(U32 N, U32 M, U32 K, DataType adt, DataFormat adf,
    DataType bdt, DataFormat bdf, U32 *bytes);

/* replaces cpu/x86/mmm.cpp:154-186 (mmm_x86 -> mmm_avx512_vnni_int8, mmm_avx512_vnni.cpp:1760-1891).
 * A: u8 [M,K] (adf = DF_NORMAL) or [K,M] (DF_TRANSPOSE); B: packed by transform_rhs;
 * tmp: first 4N bytes = int32 offsetC[N];
 * acc[m,n] = offsetC[n] + sum_k A[m,k]*B[k,n], then
 *   scale == NULL   : C int32,  C += acc
 *   scale[0] >= 0   : C fp32 whose incoming bits are int32 partial sums (callers zero it):
 *                     C = (float)(C_bits + acc) * (1/scale[0])
 *   scale[0] <  0   : C u8 = usat8( rne((float)acc * scale[1]) + 128 ), where usat8 reads the
 *                     sum as UNSIGNED (a negative sum stores 255, as vpmovusdb does).
 * Rows of the u8 output are N bytes apart.  (The AVX512 kernel advances u8 rows by 4N bytes
 * inside a register tile, mmm_avx512_vnni.cpp:1468,1473, which overruns C for M > 1; the
 * per-element values are the same and are what this function stores.) */
EE mmm_cuda_b200(U32 N, U32 M, U32 K, DataType dt, DataFormat adf, const void *A, const void *B,
    void *tmp, void *C, const F32 *scale);

/* Extension without a counterpart in Bolt (its weight scale is per tensor,
 * common/model_spec/src/model_deserialize.cpp:277): per-output-channel weight scales and
 * per-row (per-token) activation scales in the epilogue, and an overwrite mode that does not
 * read C.  The accumulators are those of mmm_cuda_b200; the conversion factor becomes
 * num / (sA * sB) with the reference's operation order (fp32 multiply, fp32 divide, then the
 * multiply with the accumulator; cf. fully_connected.cpp:396,409 and mmm_avx512_vnni.cpp:1805):
 *   out_dt DT_I32 : C (+)= acc                                 (scales unused)
 *   out_dt DT_F32 : C = (float)acc * (1.0f / (sA[m] * sB[n]))
 *   out_dt DT_U8_Q: C = usat8( rne((float)acc * (out_scale / (sA[m] * sB[n]))) + 128 )
 * With all scale pointers NULL and the same scalars this is bit-identical to mmm_cuda_b200 called
 * with scale = {sA*sB} (fp32 output) or {-1, out_scale/(sA*sB)} (u8 output). */
typedef struct {
    DataType out_dt;      /* DT_I32, DT_F32 or DT_U8_Q */
    int accumulate;       /* != 0: add the incoming int32 bits of C (DT_I32 / DT_F32 only) */
    F32 out_scale;        /* scale of the u8 output; ignored otherwise */
    F32 sA, sB;           /* per-tensor activation / weight scale */
    const F32 *d_sA;      /* device scalar overriding sA (e.g. from bolt_b200_absmax_scale_f32) */
    const F32 *row_scale; /* device [M], overrides sA / d_sA */
    const F32 *col_scale; /* device [N], overrides sB */
    const F32 *col_factor; /* device [N]: ready-made conversion factors (bolt_b200_col_factor); when set,
                              out_scale, sA, sB, d_sA and col_scale are not used (row_scale must be NULL) */
    const void *prefetch;  /* device memory that a later call on this stream will read -- typically the next
                              layer's packed weight -- or NULL.  The kernel asks for it to be brought into L2
                              while it computes, so that the next GEMM does not start on cold DRAM reads.  Only a
                              hint: nothing is written, results do not depend on it. */
    size_t prefetch_bytes; /* bytes at `prefetch` (tensor-core path only; ignored elsewhere) */
} bolt_b200_gemm_epilogue;
EE bolt_b200_gemm_u8s8_ex(U32 N, U32 M, U32 K, const void *A, const void *packedB,
    const I32 *offsetC, void *C, const bolt_b200_gemm_epilogue *ep);
/* factor[n] = num / (sA * sB[n]) in the reference's operation order (fp32 multiply, fp32 divide;
 * fully_connected.cpp:396,409): num = 1 for fp32 output, the output scale for u8 output.  d_sA (device
 * scalar) overrides sA, col_scale (device [N]) overrides sB.  factor: device [N]. */
/* The same GEMM with a u8 result that is stored, tile by tile from the epilogue, into n_dest copies of a wider
 * matrix [M][ld] at columns col0 .. col0 + N - 1: this GPU's copy and its peers' (pointers obtained with
 * bolt_b200_ipc_import, or peer-enabled allocations of one process).  It is the N-split of a GEMM over the
 * GPUs of one box with the all-gather fused into the kernel: every rank computes its N columns and leaves them
 * in everybody's [M][ld] result over NVLink while it computes the next tile.  The caller synchronises the
 * ranks afterwards (a barrier); until then other ranks' columns of a destination are not complete.
 * Device pointers only; N % 32 == 0, ld % 16 == 0, col0 % 32 == 0, at most 8 destinations, K % 16 == 0.
 * No counterpart in the reference (which is a single-process CPU library). */
typedef struct {
    U32 n_dest;
    void *dest[8];
    U32 ld;
    U32 col0;
} bolt_b200_scatter;
EE bolt_b200_gemm_u8s8_scatter(U32 N, U32 M, U32 K, const void *A, const void *packedB, const I32 *offsetC,
    const bolt_b200_gemm_epilogue *ep, const bolt_b200_scatter *sc);
/* Buffers shared between the processes of one box: a 64-byte handle for memory from bolt_b200_malloc, the
 * peer's mapping of it, and the unmapping. */
EE bolt_b200_ipc_export(void *p, void *handle64);
EE bolt_b200_ipc_import(const void *handle64, void **p);
EE bolt_b200_ipc_close(void *p);

EE bolt_b200_col_factor(F32 num, F32 sA, const F32 *d_sA, F32 sB, const F32 *col_scale, U32 N, F32 *factor);
/* Extension: F32 -> U8_Q quantization with the scale read from device memory. */
EE bolt_b200_quantize_f32_u8_dev(const F32 *data, uint64_t n, UINT8 *q, const F32 *d_scale);

/* ---- GEMV: y[N] (+)= W_s8[N,K] * x_u8[K] --------------------------------------------------- */

/* replaces cpu/x86/mvm.cpp:23-41: 4N (offsetC) + ALIGN(N,16)*ALIGN(K,8) + 32 when not packed. */
EE matrix_vector_multiply_transform_weight_bytes_cuda_b200(
    U32 row, U32 col, DataType dt, DataFormat df, U32 *bytes);
/* replaces cpu/x86/mvm.cpp:43-75 (-> mvm_avx512_vnni.cpp:28-131).  src s8 [N,K] (DF_NORMAL) or
 * [K,N] (DF_TRANSPOSE); dst = ALIGN(N,16) rows of ALIGN(K,8) bytes; offsetC[N] = -128*rowsum goes
 * to offsetCBias, or behind the matrix at dst + ALIGN(N,16)*ALIGN(K,8) when offsetCBias is NULL.
 * descTran->df = DF_NKN32K4. */
EE matrix_vector_multiply_transform_weight_cuda_b200(const TensorDesc *desc, const void *src,
    TensorDesc *descTran, void *dst, void *offsetCBias);
/* replaces cpu/x86/mvm.cpp:77-100 */
EE matrix_vector_multiply_tmp_bytes_cuda_b200(U32 row, U32 col, DataType dt, DataFormat df, U32 *bytes);
/* replaces cpu/x86/mvm.cpp:102-138 (mvm_x86 -> mvm_avx512_int8, mvm_avx512_vnni.cpp:703-759).
 * Same three output modes as mmm_cuda_b200.  The last N%8 rows follow the reference's scalar
 * tail (mvm_avx512_vnni.cpp:667-701): incoming y ignored, u8 = min(255, trunc(f + 128)).
 * dt == DT_U8_Q selects the other operand order, a u8 matrix ([N,K] DF_NORMAL or [K,N]
 * DF_TRANSPOSE, not packed) times an s8 vector -- mvm_avx512_int8_row_i8u8,
 * mvm_avx512_vnni_row.cpp:931-1028, what Bolt's matmul uses for vector outputs (matmul.cpp:376-379):
 * y = -128*sum(vector) + M*v, y is only written; the last N%4 rows use the single-row kernel's u8
 * store (low byte of rne + 128 unless that is >= 255).  offsetCBias must be non-NULL, it is not read. */
EE mvm_cuda_b200(U32 row, U32 col, DataType dt, DataFormat df, const void *matrix,
    const void *vector, void *result, void *offsetCBias, const F32 *scale);

/* ---- quantize / dequantize ------------------------------------------------------------------ */

/* replaces compute/tensor/src/cpu/x86/quantize.cpp:19-62 (quantize_x86) and
 * cpu/x86/int8/avx512/quantize.cpp:21-416.  F32->U8_Q, F32->I8, U8_Q->I8, I32->U8_Q, I32->I8.
 * `scale` is a host pointer, read and written as in the reference ([2] for I32 sources). */
EE quantize_cuda_b200(const TensorDesc *dDesc, const void *data, TensorDesc *qDesc, void *qData,
    F32 *scale, int mode);
/* replaces cpu/x86/quantize.cpp:64-121 (quantize_bias_offsetC): out = round(bias*scale) + offsetC */
EE quantize_bias_offsetC_cuda_b200(const void *bias, const TensorDesc *biasDesc, DataType qType,
    const void *filter, const TensorDesc *filterDesc, const F32 *scale, void *offsetCBias);
/* replaces cpu/x86/dequantize.cpp:19-48 (dequantize_x86): I32->F32, U8_Q->F32; bias ignored. */
EE dequantize_cuda_b200(const TensorDesc *qDesc, const void *qData, const F32 *scale,
    const TensorDesc *bDesc, const void *bData, const TensorDesc *dDesc, void *dData);
/* Extension: scale finding that leaves 127/absmax in DEVICE memory (no host round trip), for
 * pipelines that stay on the stream.  d_scale: one float on the device. */
EE bolt_b200_absmax_scale_f32(const F32 *data, uint64_t n, F32 *d_scale);

/* No counterpart in Bolt.  F32 -> U8_Q with a dynamic per-tensor scale (the arithmetic of
 * quantize_cuda_b200) for callers that must not allocate device memory when they call: servers
 * whose own pool owns the whole GPU, hosts that forbid allocation on the serving path, fixed
 * memory budgets.  It makes no cudaMalloc / cudaFree call and does not create the library's
 * per-device context; its reduction scratch is a fixed 16.5 KiB array inside the library's device
 * image (held by every GPU that loads the library until the process exits), which limits one call
 * to BOLT_B200_NOALLOC_MAX_ELEMENTS elements -- more returns NOT_SUPPORTED, as does n == 0.
 * data, q and d_scale (one float, receives 127/absmax) are device pointers; the work is enqueued
 * on the thread's current stream (bolt_b200_set_stream) of the current CUDA device.  The first
 * call on a device looks up the scratch address; make that call before any stream capture.  All
 * calls share the one array: two calls that overlap on the GPU (different streams or threads)
 * race and may both produce wrong scales -- serialise them. */
#define BOLT_B200_NOALLOC_MAX_ELEMENTS 67108864ull
EE bolt_b200_quantize_f32_u8_noalloc(const F32 *data, uint64_t n, UINT8 *q, F32 *d_scale);

/* ---- int8 and 1-bit convolution --------------------------------------------------------------- */

/* replaces convolution_infer_output_size_cpu (compute/tensor/src/convolution.cpp:28-108) for 4-D tensors:
 * oh = (ih + pad_top + pad_bottom - ((fh-1)*dilation + 1)) / stride + 1 (or the SAME round modes), fn % 8 == 0
 * required, output format DF_NCHWC16 for a U8_Q target with fn != 8 and DF_NCHWC8 otherwise -- the rule of
 * the AVX512 int8 build (:98-103).  Note that, as in the reference, the int8 kernels always write 16-channel
 * blocks (plus one 8-channel tail block), also under a DF_NCHWC8 descriptor. */
EE convolution_infer_output_size_cuda_b200(const TensorDesc *inputDesc, const TensorDesc *filterDesc,
    const ConvolutionParamSpec *convParamSpec, TensorDesc *outputDesc, DataType targetDataType);
/* replaces compute/tensor/src/cpu/x86/convolution.cpp:23-103 */
EE convolution_infer_forward_algorithm_cuda_b200(const TensorDesc *inputDesc,
    const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *convParamSpec, ConvolutionPolicy policy,
    ConvolutionForwardAlgorithm *algorithm, DataType targetDataType);
/* replaces cpu/x86/convolution.cpp:105-170.  int8: the reference's count plus 4*fn*fh*fw bytes, the
 * per-tap weight sums kept behind the packed filter (they stand in for the padded copy of the input). */
EE convolution_transform_filter_bytes_cuda_b200(const TensorDesc *filterDesc,
    const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm, U32 *bytes);
/* replaces cpu/x86/convolution.cpp:172-231 (-> int8/convolution_transform.cpp:18-238) and, for
 * 1-bit filters, cpu/arm/bnn/convolution_transform_bnn.h:32-86. */
EE convolution_transform_filter_cuda_b200(const TensorDesc *filterDesc, const void *filter,
    const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm,
    TensorDesc *ftmDesc, void *filterTransformed);
/* replaces cpu/x86/int8/convolution.cpp:17-95 */
EE convolution_infer_forward_tmp_bytes_cuda_b200(const TensorDesc *inputDesc,
    const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm, U32 *bytes);
/* replaces cpu/x86/convolution.cpp:233-363 (convolution_x86 -> convolution_int8,
 * int8/convolution.cpp:97-150) and cpu/arm/bnn/convolution.cpp:16-72 (convolution_bnn).
 * int8: input U8_Q (NCHWc16 / NCHWc8 / NCHW) or F32 (quantized first, scale[0] read and written like
 * quantize_x86); scale = {scaleI, scaleO, scaleF}; scaleO = scaleI * scaleF is written to scale[1] for an
 * fp32 output; a U8_Q output is requantized with the dynamic scale 127 / max|acc| of the whole output and
 * scale[1] = scaleO * that -- whatever scale[1] held on entry (convolution_direct.cpp:2687,2798-2806); with
 * an eltwise input the U8_Q output is the dynamic quantization of the fp32 result (:2693-2695).  ReLU is
 * applied when activation mode & 3 != 0, as the AVX512 kernels test it (:2143-2146). */
EE convolution_cuda_b200(const TensorDesc *inputDesc, void *input, void *eltwiseInput,
    const TensorDesc *filterDesc, const void *filter, const ConvolutionParamSpec *convParamSpec,
    ConvolutionForwardAlgorithm algorithm, const TensorDesc *scaleDesc, void *scale,
    const TensorDesc *biasDesc, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *activationDesc);

/* Extension without a counterpart in Bolt (its convolution has one weight scale per tensor and always
 * requantizes a u8 output dynamically, convolution_direct.cpp:2687,2798-2806): convolution_cuda_b200 with
 *   output_scale > 0  : a U8_Q output is requantized in the epilogue with this known scale,
 *                       u8 = usat8(rne(relu(acc) * (output_scale / scaleO) + 128)) -- the arithmetic of
 *                       quantizeI32ToU8 with both scales given (avx512/quantize.cpp:372-414); scale[1] returns it;
 *   filter_scales     : device or host [OC], one weight scale per output channel instead of scale[2]:
 *                       scaleO[oc] = scaleI * filter_scales[oc] in the bias term and in the conversion factor.
 *                       A U8_Q output without output_scale is then the dynamic quantization of the fp32 result.
 * With ext == NULL, or output_scale <= 0 and filter_scales == NULL, this is convolution_cuda_b200. */
typedef struct {
    F32 output_scale;
    const F32 *filter_scales;
} bolt_b200_conv_ext;
EE bolt_b200_convolution_ex(const TensorDesc *inputDesc, void *input, void *eltwiseInput,
    const TensorDesc *filterDesc, const void *filter, const ConvolutionParamSpec *convParamSpec,
    ConvolutionForwardAlgorithm algorithm, const TensorDesc *scaleDesc, void *scale,
    const TensorDesc *biasDesc, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *activationDesc,
    const bolt_b200_conv_ext *ext);

/* ---- pooling: the u8 branch of Bolt's operator (cpu/x86/pooling.cpp:50-55 -> int8/avx512/pooling_int8.cpp:317-429)
 * U8_Q NCHWc16 in and out, maximum or mean over kernel_h x kernel_w windows clipped to the image.  scale, if not
 * NULL, points at {input scale, output scale}: the output scale is written (pooling_int8.cpp:362-371).  The
 * mean uses the reference's integer arithmetic, including its logical shift (a window below the zero point
 * stores 255).  Replaces pooling_x86 for DT_U8_Q. */
EE pooling_cuda_b200(const TensorDesc *inputDesc, const void *input, const PoolingParamSpec *poolingParamSpec,
    void *scale, const TensorDesc *outputDesc, void *output);

/* ---- matmul: the int8 branch of Bolt's operator (compute/tensor/src/matmul.cpp:303-557) ------------------
 * Both operands are activations: fp32 ones are quantized per call (A to U8_Q and B to I8; when the result
 * is a row or a column, A to I8 and B to U8_Q: matmul.cpp:373-398), B is packed on the fly for every batch
 * (mmm.cpp:208-219), leading dimensions broadcast (matmul.cpp:489-517).  aScale / bScale / *cScale stand for
 * Tensor::get_scale() of the three tensors: a scale <= 0 asks for 127 / absmax; for an operand that is
 * already quantized it is the scale its bytes carry.  The output is DT_F32 (the int8 path is taken when
 * (I32)*cScale != 0 or an operand is quantized) or DT_U8_Q (requantized inside the product when *cScale > 0,
 * else quantized dynamically from the fp32 product, *cScale receiving the scale: matmul.cpp:535-547).
 * `bias`, if given, is repeated over the product's bytes before the multiplication, which accumulates on
 * top of them as the reference does (matmul.cpp:453-466).  Replaces matmul_infer_output_size_cpu,
 * matmul_infer_forward_tmp_bytes and matmul for Arch CUDA_B200. */
EE matmul_infer_output_size_cuda_b200(const TensorDesc *matrixADesc, int transposeA,
    const TensorDesc *matrixBDesc, int transposeB, TensorDesc *matrixCDesc);
EE matmul_infer_forward_tmp_bytes_cuda_b200(const TensorDesc *matrixADesc, int transposeA,
    const TensorDesc *matrixBDesc, int transposeB, const TensorDesc *matrixCDesc, F32 cScale, U32 *bytes);
EE matmul_cuda_b200(const TensorDesc *matrixADesc, int transposeA, const void *matrixA, F32 aScale,
    const TensorDesc *matrixBDesc, int transposeB, const void *matrixB, F32 bScale,
    const TensorDesc *biasDesc, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *matrixCDesc, void *matrixC, F32 *cScale);

/* ============================== 3. operators ================================================= */
/* Bolt's public signatures (compute/blas_enhance/include/blas_enhance.h:21-88); arch must be
 * CUDA_B200, anything else returns NOT_SUPPORTED.  Argument checks follow mmm.cpp:161-197 and
 * mvm.cpp:143-160. */
EE b200_matrix_matrix_multiply_tmp_bytes(TensorDesc matrixADesc, TensorDesc matrixBDesc, U32 *bytes, Arch arch);
EE b200_matrix_matrix_multiply(TensorDesc matrixADesc, const void *matrixA, TensorDesc matrixBDesc,
    const void *matrixB, U32 bytes, void *tmp, TensorDesc matrixCDesc, void *matrixC,
    const F32 *scale, Arch arch);
DataFormat b200_matrix_matrix_multiply_rhs_format(DataType dt);
EE b200_matrix_matrix_multiply_transform_rhs_bytes(TensorDesc desc, U32 *bytes, U32 *rhsBytes, Arch arch);
EE b200_matrix_matrix_multiply_transform_rhs(TensorDesc desc, const void *src, TensorDesc *descTran, void *dst, Arch arch);
EE b200_matrix_vector_multiply_tmp_bytes(TensorDesc matrixDesc, TensorDesc vectorDesc, U32 *bytes, Arch arch);
EE b200_matrix_vector_multiply(TensorDesc matrixDesc, const void *matrix, TensorDesc vectorDesc,
    const void *vector, U32 bytes, void *tmp, TensorDesc resultDesc, void *result, const F32 *scale,
    Arch arch);
DataFormat b200_matrix_vector_multiply_weight_format(DataType dt);
EE b200_matrix_vector_multiply_transform_weight_bytes(TensorDesc desc, U32 *bytes, Arch arch);
EE b200_matrix_vector_multiply_transform_weight(TensorDesc desc, const void *src, TensorDesc *descTran, void *dst, Arch arch);

#ifdef __cplusplus
}
#endif
#endif /* BOLT_B200_H */
