// matmul.cu -- the int8 branch of Bolt's `matmul` operator (compute/tensor/src/matmul.cpp:303-557) for
// CUDA_B200: both operands may arrive as fp32 and are quantized per call (dynamic scale 127 / absmax, or the
// scale the tensor carries), B is an activation and is therefore packed on the fly for every batch, the
// product runs on the tensor-core GEMM (or on a GEMV kernel when the result is a row or a column), and the
// result is written as fp32 (accumulator / (scaleA * scaleB)) or requantized to u8.
//
// The x86 convention applies (matmul.cpp:373-398): u8 activations with zero point 128 times s8, except
// when the result is a vector, where A becomes s8 and B u8.  Leading (batch) dimensions broadcast as in
// matmul.cpp:489-517.  All work is enqueued on the thread's stream; scales come back to the host, which is
// what the operator's interface (Tensor::get_scale) requires.
#include "common.cuh"

namespace b200 {
namespace {

inline size_t bytes_of(DataType dt)
{
    return (dt == DT_F32 || dt == DT_I32 || dt == DT_U32 || dt == DT_F32_8Q) ? 4 : (dt == DT_F16 ? 2 : 1);
}
inline uint64_t elems(const TensorDesc &d)
{
    uint64_t n = d.nDims ? 1 : 0;
    for (U32 i = 0; i < d.nDims; ++i) {
        n *= d.dims[i];
    }
    return n;
}
inline bool use_int8(DataType a, DataType b, DataType c, F32 cScale)
{
    // matmul.cpp:205-209; the scale is read through an I32 parameter, so |scale| < 1 does not count
    return a == DT_I8 || b == DT_I8 || a == DT_U8_Q || b == DT_U8_Q || c == DT_U8_Q || c == DT_I8 || (I32)cScale != 0;
}
void align_descs(TensorDesc *a, TensorDesc *b)
{
    while (a->nDims < b->nDims) {
        a->dims[a->nDims++] = 1;
    }
    while (b->nDims < a->nDims) {
        b->dims[b->nDims++] = 1;
    }
}
TensorDesc desc2d(DataType dt, DataFormat df, U32 rows, U32 cols)
{
    TensorDesc d;
    d.dt = dt;
    d.df = df;
    d.nDims = 2;
    d.dims[0] = cols;
    d.dims[1] = rows;
    return d;
}
TensorDesc desc1d(DataType dt, U32 len)
{
    TensorDesc d;
    d.dt = dt;
    d.df = DF_NORMAL;
    d.nDims = 1;
    d.dims[0] = len;
    return d;
}

// what the operator decides before touching data
struct Plan {
    TensorDesc a, b, c;          // a and b aligned to the same rank; c as the caller gave it
    bool is_mvm;
    DataType qa, qb, qc;         // operand types of the product, type the product writes
    bool quantA, quantB, stageC;
    bool static_u8;              // u8 output requantized inside the product with the caller's scale
    U32 kDimA, kDimB;
    DataFormat dfA, dfB;
    U32 mmm_bytes;
    uint64_t loopsA, loopsB, loopsC;
};

EE inner_tmp_bytes(const Plan &p, U32 *bytes)
{
    // matmul.cpp:211-243
    const TensorDesc &A = p.a, &B = p.b;
    if (A.dims[1 - p.kDimA] == 1) {
        return b200_matrix_vector_multiply_tmp_bytes(
            desc2d(p.qb, p.dfB == DF_TRANSPOSE ? DF_NORMAL : DF_TRANSPOSE, B.dims[1], B.dims[0]),
            desc1d(p.qa, A.dims[p.kDimA]), bytes, CUDA_B200);
    }
    if (B.dims[1 - p.kDimB] == 1) {
        return b200_matrix_vector_multiply_tmp_bytes(
            desc2d(p.qa, p.dfA, A.dims[1], A.dims[0]), desc1d(p.qb, B.dims[p.kDimB]), bytes, CUDA_B200);
    }
    return b200_matrix_matrix_multiply_tmp_bytes(
        desc2d(p.qa, p.dfA, A.dims[1], A.dims[0]), desc2d(p.qb, p.dfB, B.dims[1], B.dims[0]), bytes, CUDA_B200);
}

EE make_plan(const TensorDesc *aDesc, int tA, const TensorDesc *bDesc, int tB, const TensorDesc *cDesc, F32 cScale, Plan *p)
{
    if (aDesc == nullptr || bDesc == nullptr || cDesc == nullptr) {
        return NULL_POINTER;
    }
    p->a = *aDesc;
    p->b = *bDesc;
    p->c = *cDesc;
    if (p->a.nDims < 1 || p->b.nDims < 2 || p->a.nDims > 6 || p->b.nDims > 6 || p->c.nDims > 6) {
        return NOT_SUPPORTED;
    }
    if (!use_int8(p->a.dt, p->b.dt, p->c.dt, cScale)) {
        return NOT_SUPPORTED;  // the floating-point matmul is not part of this library
    }
    if (p->c.dt != DT_F32 && p->c.dt != DT_U8_Q) {
        return NOT_SUPPORTED;
    }
    if (p->a.nDims == 1) {  // matmul.cpp:360-365
        p->a.nDims = 2;
        p->a.dims[1] = 1;
        p->c.nDims = 2;
        p->c.dims[1] = 1;
    }
    p->is_mvm = (p->c.dims[0] == 1) || (p->c.dims[1] == 1);
    p->qa = p->is_mvm ? DT_I8 : DT_U8_Q;
    p->qb = p->is_mvm ? DT_U8_Q : DT_I8;
    p->qc = DT_F32;
    p->static_u8 = false;
    if (p->c.dt == DT_U8_Q && cScale > 0) {
        p->qc = DT_U8_Q;
        p->static_u8 = true;
    }
    p->quantA = p->a.dt != p->qa;
    p->quantB = p->b.dt != p->qb;
    p->stageC = p->c.dt != p->qc;
    // an operand is either fp32 (quantized here) or already of the type the product wants
    if ((p->quantA && p->a.dt != DT_F32) || (p->quantB && p->b.dt != DT_F32)) {
        return NOT_SUPPORTED;
    }
    p->kDimA = tA ? 1 : 0;
    p->dfA = tA ? DF_TRANSPOSE : DF_NORMAL;
    p->kDimB = tB ? 0 : 1;
    p->dfB = tB ? DF_TRANSPOSE : DF_NORMAL;
    align_descs(&p->a, &p->b);
    if (p->a.dims[p->kDimA] != p->b.dims[p->kDimB]) {
        return NOT_MATCH;
    }
    if (p->c.dims[0] != p->b.dims[1 - p->kDimB] || p->c.dims[1] != p->a.dims[1 - p->kDimA]) {
        return NOT_MATCH;
    }
    const uint64_t a2 = (uint64_t)p->a.dims[0] * p->a.dims[1], b2 = (uint64_t)p->b.dims[0] * p->b.dims[1];
    const uint64_t c2 = (uint64_t)p->c.dims[0] * p->c.dims[1];
    if (a2 == 0 || b2 == 0 || c2 == 0) {
        return NOT_MATCH;
    }
    p->loopsA = elems(p->a) / a2;
    p->loopsB = elems(p->b) / b2;
    p->loopsC = elems(p->c) / c2;
    return inner_tmp_bytes(*p, &p->mmm_bytes);
}

__global__ void fill_rows_kernel(uint8_t *dst, uint64_t total, const uint8_t *row, uint32_t row_bytes)
{
    // dst = the bias bytes repeated (matmul.cpp:457-466); a zero fill when row == nullptr
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        dst[i] = row ? row[i % row_bytes] : (uint8_t)0;
    }
}

U32 global_index(uint64_t ic, const TensorDesc &c, const TensorDesc &x)
{
    // matmul.cpp:494-517: the batch coordinates of C, each folded to 0 where the operand's extent is smaller
    U32 idx[8];
    for (U32 i = 2; i < c.nDims; ++i) {
        idx[i] = (U32)(ic % c.dims[i]);
        ic /= c.dims[i];
    }
    U32 g = 0;
    for (int i = (int)x.nDims - 1; i >= 2; --i) {
        U32 v = (U32)i < c.nDims ? idx[i] : 0;
        if (v >= x.dims[i]) {
            v = 0;
        }
        g = g * x.dims[i] + v;
    }
    return g;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

// matmul.cpp:42-99
EE matmul_infer_output_size_cuda_b200(const TensorDesc *aDesc, int transposeA, const TensorDesc *bDesc, int transposeB,
    TensorDesc *cDesc)
{
    if (aDesc == nullptr || bDesc == nullptr || cDesc == nullptr) {
        return NULL_POINTER;
    }
    TensorDesc a = *aDesc, b = *bDesc;
    if (a.nDims < 2 || b.nDims < 2 || a.nDims > 6 || b.nDims > 6) {
        return NOT_SUPPORTED;
    }
    if (transposeA) {
        std::swap(a.dims[0], a.dims[1]);
    }
    if (transposeB) {
        std::swap(b.dims[0], b.dims[1]);
    }
    if (a.dims[0] != b.dims[1]) {
        return NOT_MATCH;
    }
    align_descs(&a, &b);
    *cDesc = a;
    cDesc->dims[0] = b.dims[0];
    for (U32 i = 2; i < a.nDims; ++i) {
        const U32 x = a.dims[i], y = b.dims[i];
        if (x != y && x != 1 && y != 1) {
            return NOT_MATCH;
        }
        cDesc->dims[i] = x > y ? x : y;
    }
    return SUCCESS;
}

// matmul.cpp:245-301
EE matmul_infer_forward_tmp_bytes_cuda_b200(const TensorDesc *aDesc, int transposeA, const TensorDesc *bDesc,
    int transposeB, const TensorDesc *cDesc, F32 cScale, U32 *bytes)
{
    if (bytes == nullptr) {
        return NULL_POINTER;
    }
    Plan p;
    B200_EE(make_plan(aDesc, transposeA, bDesc, transposeB, cDesc, cScale, &p));
    uint64_t total = B200_ALIGN((uint64_t)p.mmm_bytes, 256) + 1024;
    if (p.quantA) {
        total += B200_ALIGN(elems(p.a), 256);
    }
    if (p.quantB) {
        total += B200_ALIGN(elems(p.b), 256);
    }
    if (p.stageC) {
        total += B200_ALIGN(elems(p.c) * 4, 256);
    }
    if (total > 0xffffffffull) {
        return NOT_SUPPORTED;
    }
    *bytes = (U32)total;
    return SUCCESS;
}

EE matmul_cuda_b200(const TensorDesc *aDesc, int transposeA, const void *A, F32 aScale, const TensorDesc *bDesc,
    int transposeB, const void *B, F32 bScale, const TensorDesc *biasDesc, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *cDesc, void *C, F32 *cScale)
{
    if (A == nullptr || B == nullptr || C == nullptr || cScale == nullptr) {
        return NULL_POINTER;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    Plan p;
    B200_EE(make_plan(aDesc, transposeA, bDesc, transposeB, cDesc, *cScale, &p));
    U32 need = 0;
    B200_EE(matmul_infer_forward_tmp_bytes_cuda_b200(aDesc, transposeA, bDesc, transposeB, cDesc, *cScale, &need));
    if (tmp == nullptr || tmpBytes < need) {
        return NOT_MATCH;
    }
    const uint64_t nA = elems(p.a), nB = elems(p.b), nC = elems(p.c);
    const size_t bias_bytes = (bias != nullptr && biasDesc != nullptr) ? (size_t)elems(*biasDesc) * bytes_of(biasDesc->dt) : 0;
    cudaStream_t st = tls().stream;

    // host pointers: the whole operator runs on device copies made for this call
    const bool host = !is_device_ptr(A) || !is_device_ptr(B) || !is_device_ptr(C) || !is_device_ptr(tmp) ||
        (bias_bytes && !is_device_ptr(bias));
    std::vector<void *> owned;
    struct Free {
        std::vector<void *> &v;
        ~Free()
        {
            for (void *q : v) {
                cudaFree(q);
            }
        }
    } guard{owned};
    const size_t c_bytes = (size_t)nC * bytes_of(p.c.dt);
    void *hostC = nullptr;
    if (host) {
        if (tls().device_only) {
            return NOT_MATCH;
        }
        auto dev_copy = [&](const void *src, size_t bytes, bool copy) -> void * {
            if (is_device_ptr(src)) {
                return const_cast<void *>(src);
            }
            void *d = nullptr;
            if (cudaMalloc(&d, bytes ? bytes : 16) != cudaSuccess) {
                cudaGetLastError();
                return nullptr;
            }
            owned.push_back(d);
            if (copy && cudaMemcpyAsync(d, src, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) {
                return nullptr;
            }
            return d;
        };
        A = dev_copy(A, (size_t)nA * bytes_of(p.a.dt), true);
        B = dev_copy(B, (size_t)nB * bytes_of(p.b.dt), true);
        if (bias_bytes) {
            bias = dev_copy(bias, bias_bytes, true);
        }
        tmp = dev_copy(tmp, tmpBytes, false);
        if (!is_device_ptr(C)) {
            hostC = C;
        }
        C = dev_copy(C, c_bytes, false);
        if (A == nullptr || B == nullptr || tmp == nullptr || C == nullptr || (bias_bytes && bias == nullptr)) {
            return ALLOC_FAILED;
        }
    }
    if (on_other_device(A) || on_other_device(B) || on_other_device(C) || on_other_device(tmp)) {
        return NOT_MATCH;
    }

    char *t = reinterpret_cast<char *>(tmp);
    F32 scaleO = 1;
    // operands: quantize into tmp, or take the caller's quantized bytes and scale (matmul.cpp:401-421)
    if (p.quantA) {
        F32 s = aScale;
        TensorDesc q = p.a;
        q.dt = p.qa;
        B200_EE(quantize_cuda_b200(&p.a, A, &q, t, &s, 0));
        scaleO *= s;
        A = t;
        t += B200_ALIGN(nA, 256);
    } else {
        scaleO *= aScale;
    }
    if (p.quantB) {
        F32 s = bScale;
        TensorDesc q = p.b;
        q.dt = p.qb;
        B200_EE(quantize_cuda_b200(&p.b, B, &q, t, &s, 0));
        scaleO *= s;
        B = t;
        t += B200_ALIGN(nB, 256);
    } else {
        scaleO *= bScale;
    }
    void *prod = C;
    if (p.stageC) {
        prod = t;
        t += B200_ALIGN(nC * 4, 256);
    }
    F32 scaleArray[2] = {-1, -1};
    const F32 *scalePtr = &scaleO;
    if (p.static_u8) {
        scaleArray[1] = *cScale / scaleO;  // matmul.cpp:383-386,429-431
        scalePtr = scaleArray;
    }
    // the product accumulates on top of C: zero, or the bias bytes repeated (matmul.cpp:453-476)
    const size_t prod_bytes = (size_t)nC * bytes_of(p.qc);
    if (bias_bytes) {
        if (prod_bytes % bias_bytes != 0) {
            return NOT_MATCH;
        }
        const uint32_t grid = (uint32_t)std::min<uint64_t>((prod_bytes + 255) / 256, (uint64_t)c->sm_count * 8);
        fill_rows_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<uint8_t *>(prod), prod_bytes,
            reinterpret_cast<const uint8_t *>(bias), (uint32_t)bias_bytes);
        count_launch();
    } else {
        B200_CUDA(cudaMemsetAsync(prod, 0, prod_bytes, st));
    }

    const size_t a2 = (size_t)p.a.dims[0] * p.a.dims[1], b2 = (size_t)p.b.dims[0] * p.b.dims[1];
    const size_t c2 = (size_t)p.c.dims[0] * p.c.dims[1] * bytes_of(p.qc);
    for (uint64_t ic = 0; ic < p.loopsC; ++ic) {
        const uint64_t ia = p.loopsA == p.loopsC ? ic : global_index(ic, p.c, p.a);
        const uint64_t ib = p.loopsB == p.loopsC ? ic : global_index(ic, p.c, p.b);
        const char *pa = reinterpret_cast<const char *>(A) + ia * a2;
        const char *pb = reinterpret_cast<const char *>(B) + ib * b2;
        char *pc = reinterpret_cast<char *>(prod) + ic * c2;
        EE ret;
        if (p.a.dims[1 - p.kDimA] == 1) {
            ret = b200_matrix_vector_multiply(
                desc2d(p.qb, p.dfB == DF_TRANSPOSE ? DF_NORMAL : DF_TRANSPOSE, p.b.dims[1], p.b.dims[0]), pb,
                desc1d(p.qa, p.a.dims[p.kDimA]), pa, p.mmm_bytes, t, desc1d(p.qc, p.c.dims[0]), pc, scalePtr, CUDA_B200);
        } else if (p.b.dims[1 - p.kDimB] == 1) {
            ret = b200_matrix_vector_multiply(desc2d(p.qa, p.dfA, p.a.dims[1], p.a.dims[0]), pa,
                desc1d(p.qb, p.b.dims[p.kDimB]), pb, p.mmm_bytes, t, desc1d(p.qc, p.c.dims[1]), pc, scalePtr, CUDA_B200);
        } else {
            ret = b200_matrix_matrix_multiply(desc2d(p.qa, p.dfA, p.a.dims[1], p.a.dims[0]), pa,
                desc2d(p.qb, p.dfB, p.b.dims[1], p.b.dims[0]), pb, p.mmm_bytes, t,
                desc2d(p.qc, DF_NORMAL, p.c.dims[1], p.c.dims[0]), pc, scalePtr, CUDA_B200);
        }
        B200_EE(ret);
    }
    // matmul.cpp:535-554: a u8 output without a given scale is quantized from the fp32 product
    if (p.stageC) {
        F32 scales[2] = {*cScale, scaleO};
        TensorDesc src = p.c;
        src.dt = p.qc;
        B200_EE(quantize_cuda_b200(&src, prod, &p.c, C, scales, 0));
        *cScale = scales[0];
    }
    if (hostC != nullptr) {
        B200_CUDA(cudaMemcpyAsync(hostC, C, c_bytes, cudaMemcpyDeviceToHost, st));
    }
    if (host) {
        B200_CUDA(cudaStreamSynchronize(st));
    }
    return SUCCESS;
}

}  // extern "C"
