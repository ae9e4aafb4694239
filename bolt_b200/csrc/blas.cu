// blas.cu -- GEMM / GEMV entry points: the per-architecture functions (`*_cuda_b200`) and the
// mirrors of Bolt's public blas_enhance functions (`b200_*`).
//
// Host logic only: argument checks, the tmp / packed-weight protocol of Bolt's callers, pointer
// staging, kernel selection.  The arithmetic lives in gemm_i8_tcgen05.cu, gemm_i8_simt.cu, gemv_i8.cu.
#include <cstring>
#include <utility>

#include "common.cuh"

using namespace b200;

namespace {

// tensor2dGet (common/uni/include/tensor_desc.h:195-212): dims[0] = columns, dims[1] = rows
EE get2d(const TensorDesc &d, DataType *dt, DataFormat *df, U32 *rows, U32 *cols)
{
    if (d.nDims != 2) {
        return NOT_MATCH;
    }
    *dt = d.dt;
    *df = d.df;
    *cols = d.dims[0];
    *rows = d.dims[1];
    return SUCCESS;
}
EE get1d(const TensorDesc &d, DataType *dt, DataFormat *df, U32 *len)
{
    if (d.nDims != 1) {
        return NOT_MATCH;
    }
    *dt = d.dt;
    *df = d.df;
    *len = d.dims[0];
    return SUCCESS;
}
uint64_t num_elems(const TensorDesc &d)
{
    if (d.nDims == 0) {
        return 0;
    }
    uint64_t n = 1;
    for (U32 i = 0; i < d.nDims && i < 20; ++i) {
        n *= d.dims[i];
    }
    return n;
}

// Device address of a packed weight: the pointer itself when it is device memory, else its
// registered device twin, else a staged copy.
const void *resolve_weight(const void *w, size_t bytes, Stage &sg)
{
    if (is_device_ptr(w)) {
        return w;
    }
    DeviceCtx *c = ctx();
    {
        std::lock_guard<std::mutex> g(c->twin_mu);
        auto it = c->twins.find(w);
        if (it != c->twins.end() && it->second.bytes >= bytes) {
            return it->second.dev;
        }
    }
    return sg.in(w, bytes);
}

// Packs `src` into `dst` (matrix, then offsetC at off_bytes or into `off_dst`).  A host `dst`
// gets the packed bytes copied back and keeps a device twin.
EE pack_weight(const void *src, bool src_is_nk, U32 N, U32 K, void *dst, size_t mat_bytes, void *off_dst)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    cudaStream_t st = tls().stream;
    const U32 Np = B200_ALIGN(N, 16), Kp = B200_ALIGN(K, 8);
    Stage sg;
    const int8_t *d_src = reinterpret_cast<const int8_t *>(sg.in(src, (size_t)N * K));
    if (d_src == nullptr) {
        return ALLOC_FAILED;
    }
    const bool dst_dev = is_device_ptr(dst);
    // offsetC placement: separate buffer, or right behind the matrix
    const bool off_separate = off_dst != nullptr;
    const size_t total = mat_bytes + (off_separate ? 0 : (size_t)N * 4);
    char *d_dst = reinterpret_cast<char *>(dst);
    if (!dst_dev) {
        void *twin = nullptr;
        B200_CUDA(cudaMalloc(&twin, B200_ALIGN(mat_bytes + (size_t)N * 4, 256)));
        d_dst = reinterpret_cast<char *>(twin);
    }
    int32_t *d_off = reinterpret_cast<int32_t *>(d_dst + mat_bytes);
    int32_t *d_off_user = nullptr;
    if (off_separate) {
        d_off_user = reinterpret_cast<int32_t *>(sg.out(off_dst, (size_t)N * 4));
        if (d_off_user == nullptr) {
            return ALLOC_FAILED;
        }
        if (dst_dev) {
            d_off = d_off_user;  // nothing is written behind a caller's device matrix
        }
    }
    EE ret = launch_pack_rhs(d_src, src_is_nk, N, K, reinterpret_cast<int8_t *>(d_dst), Kp, Np, d_off, st);
    if (ret == SUCCESS && off_separate && d_off != d_off_user) {
        ret = cuda_ee(cudaMemcpyAsync(d_off_user, d_off, (size_t)N * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (ret == SUCCESS && !dst_dev) {
        ret = cuda_ee(cudaMemcpyAsync(dst, d_dst, total, cudaMemcpyDeviceToHost, st));
    }
    if (ret == SUCCESS) {
        ret = sg.finish();
    }
    if (!dst_dev) {
        if (ret == SUCCESS) {
            ret = cuda_ee(cudaStreamSynchronize(st));
        }
        if (ret != SUCCESS) {
            cudaFree(d_dst);
            return ret;
        }
        std::lock_guard<std::mutex> g(c->twin_mu);
        auto it = c->twins.find(dst);
        if (it != c->twins.end()) {
            cudaFree(it->second.dev);
        }
        c->twins[dst] = WeightTwin{d_dst, mat_bytes + (size_t)N * 4};
    }
    return ret;
}

EE run_gemm(U32 N, U32 M, U32 K, bool a_t, const void *A, const void *B, const void *offsetC, void *C,
    GemmEpilogue ep)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (M == 0 || N == 0) {
        return SUCCESS;
    }
    if (A == nullptr || B == nullptr || C == nullptr) {
        return NULL_POINTER;
    }
    if (on_other_device(A) || on_other_device(B) || on_other_device(C)) {
        return NOT_MATCH;  // device memory of a GPU other than the one this thread's calls run on
    }
    const U32 Np = B200_ALIGN(N, 16), Kp = B200_ALIGN(K, 8);
    const size_t esz = ep.out_kind == 2 ? 1 : 4;
    Stage sg;
    const uint8_t *dA = reinterpret_cast<const uint8_t *>(sg.in(A, (size_t)M * K));
    const int8_t *dB = reinterpret_cast<const int8_t *>(resolve_weight(B, (size_t)Np * Kp, sg));
    const int32_t *dOff = offsetC ? reinterpret_cast<const int32_t *>(sg.in(offsetC, (size_t)N * 4)) : nullptr;
    void *dC = sg.out(C, (size_t)M * N * esz, ep.out_kind != 2 && ep.accumulate);
    if (dA == nullptr || dB == nullptr || dC == nullptr || (offsetC && dOff == nullptr)) {
        return ALLOC_FAILED;
    }
    ep.offsetC = dOff;
    cudaStream_t st = tls().stream;
    EE ret;
    if (gemm_tcgen05_eligible(M, N, K, dA, dB, Kp, a_t)) {
        ret = launch_gemm_tcgen05(M, N, K, dA, dB, Kp, dC, ep, st);
        tls().last_gemm_tc = 1;
    } else if (ep.scatter_n > 0) {
        return NOT_SUPPORTED;  // the scatter epilogue exists on the tensor-core path only
    } else {
        ret = launch_gemm_simt(M, N, K, dA, a_t, dB, Kp, dC, ep, st);
        tls().last_gemm_tc = 0;
    }
    B200_EE(ret);
    return sg.finish();
}

// scale protocol of mmm_avx512_vnni_int8 / mvm_avx512_int8 (mmm_avx512_vnni.cpp:1796-1808)
void scale_to_epilogue(const F32 *scale, GemmEpilogue *ep)
{
    std::memset(ep, 0, sizeof(*ep));
    if (scale == nullptr) {
        ep->out_kind = 0;
        ep->accumulate = 1;
    } else if (scale[0] < 0) {
        ep->out_kind = 2;
        ep->factor = scale[1];
    } else {
        ep->out_kind = 1;
        ep->accumulate = 1;
        ep->factor = 1 / scale[0];
    }
}

}  // namespace

extern "C" {

// =============================== GEMM ========================================================
EE matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(
    U32 N, U32 K, DataType bdt, DataFormat bdf, U32 *bytes, U32 *rhsBytes)
{
    if (bdt != DT_I8 && bdt != DT_U8_Q) {
        return NOT_SUPPORTED;
    }
    U32 matrix = 0, total = 0;
    if (bdf != DF_NKNxKx) {
        total += N * 4;
        matrix = B200_ALIGN(N, 16) * B200_ALIGN(K, 8);
        total += matrix + 64;
    }
    if (rhsBytes != nullptr) {
        *rhsBytes = matrix;
    }
    if (bytes != nullptr) {
        *bytes = total;
    }
    return SUCCESS;
}

EE matrix_matrix_multiply_transform_rhs_cuda_b200(
    const TensorDesc *desc, const void *src, TensorDesc *descTran, void *dst)
{
    if (desc == nullptr || descTran == nullptr) {
        return NULL_POINTER;
    }
    if (desc->df == DF_NKNxKx) {
        return SUCCESS;  // already packed (cpu/x86/mmm.cpp:132-134)
    }
    if (desc->dt != DT_I8 || (desc->df != DF_NORMAL && desc->df != DF_TRANSPOSE)) {
        return NOT_SUPPORTED;
    }
    if (src == nullptr || dst == nullptr) {
        return NULL_POINTER;
    }
    DataType dt;
    DataFormat df;
    U32 rows, cols;
    B200_EE(get2d(*desc, &dt, &df, &rows, &cols));
    const bool is_nk = (df == DF_TRANSPOSE);
    const U32 N = is_nk ? rows : cols;
    const U32 K = is_nk ? cols : rows;
    const size_t mat = (size_t)B200_ALIGN(N, 16) * B200_ALIGN(K, 8);
    B200_EE(pack_weight(src, is_nk, N, K, dst, mat, nullptr));
    *descTran = *desc;
    descTran->df = DF_NKNxKx;
    if (is_nk) {
        std::swap(descTran->dims[0], descTran->dims[1]);
    }
    return SUCCESS;
}

EE matrix_matrix_multiply_tmp_bytes_cuda_b200(
    U32 N, U32 M, U32 K, DataType adt, DataFormat adf, DataType bdt, DataFormat bdf, U32 *bytes)
{
    (void)M;
    if (bytes == nullptr) {
        return NULL_POINTER;
    }
    if (adt != DT_U8_Q && adt != DT_I8) {
        return NOT_SUPPORTED;
    }
    if (adf != DF_NORMAL && adf != DF_TRANSPOSE) {
        return NOT_SUPPORTED;
    }
    B200_EE(matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(N, K, bdt, bdf, bytes, nullptr));
    *bytes += N * 4 + 64;
    return SUCCESS;
}

EE mmm_cuda_b200(U32 N, U32 M, U32 K, DataType dt, DataFormat adf, const void *A, const void *B, void *tmp,
    void *C, const F32 *scale)
{
    if (dt != DT_I8) {
        return NOT_SUPPORTED;
    }
    if (adf != DF_NORMAL && adf != DF_TRANSPOSE) {
        return NOT_SUPPORTED;
    }
    if (tmp == nullptr) {
        return NULL_POINTER;
    }
    GemmEpilogue ep;
    scale_to_epilogue(scale, &ep);
    return run_gemm(N, M, K, adf == DF_TRANSPOSE, A, B, tmp, C, ep);
}

EE bolt_b200_gemm_u8s8_ex(U32 N, U32 M, U32 K, const void *A, const void *packedB, const I32 *offsetC,
    void *C, const bolt_b200_gemm_epilogue *e)
{
    if (e == nullptr) {
        return NULL_POINTER;
    }
    GemmEpilogue ep;
    std::memset(&ep, 0, sizeof(ep));
    if (e->out_dt == DT_I32) {
        ep.out_kind = 0;
    } else if (e->out_dt == DT_F32) {
        ep.out_kind = 1;
        ep.num = 1.0f;
    } else if (e->out_dt == DT_U8_Q) {
        ep.out_kind = 2;
        ep.num = e->out_scale;
    } else {
        return NOT_SUPPORTED;
    }
    ep.accumulate = (e->accumulate != 0 && ep.out_kind != 2) ? 1 : 0;
    ep.per_channel = ep.out_kind != 0;
    ep.sA = e->sA;
    ep.sB = e->sB;
    ep.sA_dev = e->d_sA;
    ep.row_scale = e->row_scale;
    ep.col_scale = e->col_scale;
    ep.col_factor = e->col_factor;
    ep.prefetch = e->prefetch;
    ep.prefetch_bytes = e->prefetch_bytes;
    if (e->col_factor != nullptr && e->row_scale != nullptr) {
        return NOT_SUPPORTED;
    }
    return run_gemm(N, M, K, false, A, packedB, offsetC, C, ep);
}

EE bolt_b200_gemm_u8s8_scatter(U32 N, U32 M, U32 K, const void *A, const void *packedB, const I32 *offsetC,
    const bolt_b200_gemm_epilogue *e, const bolt_b200_scatter *sc)
{
    if (e == nullptr || sc == nullptr) {
        return NULL_POINTER;
    }
    if (e->out_dt != DT_U8_Q || sc->n_dest == 0 || sc->n_dest > 8 || e->col_factor != nullptr) {
        return NOT_SUPPORTED;
    }
    if (!is_device_ptr(A) || !is_device_ptr(packedB) || (offsetC != nullptr && !is_device_ptr(offsetC))) {
        return NOT_MATCH;  // device memory only: the destinations are peers' buffers
    }
    GemmEpilogue ep;
    std::memset(&ep, 0, sizeof(ep));
    ep.out_kind = 2;
    ep.num = e->out_scale;
    ep.per_channel = 1;
    ep.sA = e->sA;
    ep.sB = e->sB;
    ep.sA_dev = e->d_sA;
    ep.row_scale = e->row_scale;
    ep.col_scale = e->col_scale;
    ep.prefetch = e->prefetch;
    ep.prefetch_bytes = e->prefetch_bytes;
    for (U32 q = 0; q < sc->n_dest; ++q) {
        if (sc->dest[q] == nullptr) {
            return NULL_POINTER;
        }
        ep.scatter_dst[q] = sc->dest[q];
    }
    ep.scatter_n = sc->n_dest;
    ep.scatter_ld = sc->ld;
    ep.scatter_col0 = sc->col0;
    // C of the common path: the first destination (used only for the argument checks)
    return run_gemm(N, M, K, false, A, packedB, offsetC, sc->dest[0], ep);
}

// =============================== GEMV ========================================================
EE matrix_vector_multiply_transform_weight_bytes_cuda_b200(U32 row, U32 col, DataType dt, DataFormat df, U32 *bytes)
{
    if (bytes == nullptr) {
        return NULL_POINTER;
    }
    if (dt == DT_U8_Q) {
        // the u8 matrix x s8 vector form needs no packing here; the reference's counts are kept so that
        // callers size tmp the same way (cpu/x86/mvm.cpp:30-40)
        *bytes = (col % 32 != 0) ? 32 * (row + 1) : 0;
        if (df != DF_NK) {
            *bytes += B200_ALIGN(row, 16) * B200_ALIGN(col, 8) + 32;
        }
        return SUCCESS;
    }
    if (dt != DT_I8) {
        return NOT_SUPPORTED;
    }
    *bytes = row * 4;
    if (df != DF_NKN32K4) {
        *bytes += B200_ALIGN(row, 16) * B200_ALIGN(col, 8) + 32;
    }
    return SUCCESS;
}

EE matrix_vector_multiply_transform_weight_cuda_b200(
    const TensorDesc *desc, const void *src, TensorDesc *descTran, void *dst, void *offsetCBias)
{
    if (desc == nullptr || descTran == nullptr) {
        return NULL_POINTER;
    }
    if (desc->df == DF_NKN32K4) {
        return SUCCESS;
    }
    if (desc->dt != DT_I8 || (desc->df != DF_NORMAL && desc->df != DF_TRANSPOSE)) {
        return NOT_SUPPORTED;
    }
    if (src == nullptr || dst == nullptr) {
        return NULL_POINTER;
    }
    DataType dt;
    DataFormat df;
    U32 rows, cols;
    B200_EE(get2d(*desc, &dt, &df, &rows, &cols));
    const bool is_nk = (df == DF_NORMAL);  // matrix [N,K]; DF_TRANSPOSE stores [K,N]
    const U32 N = is_nk ? rows : cols;
    const U32 K = is_nk ? cols : rows;
    const size_t mat = (size_t)B200_ALIGN(N, 16) * B200_ALIGN(K, 8);
    B200_EE(pack_weight(src, is_nk, N, K, dst, mat, offsetCBias));
    *descTran = *desc;
    if (df == DF_TRANSPOSE) {
        std::swap(descTran->dims[0], descTran->dims[1]);
    }
    descTran->df = DF_NKN32K4;
    return SUCCESS;
}

EE matrix_vector_multiply_tmp_bytes_cuda_b200(U32 row, U32 col, DataType dt, DataFormat df, U32 *bytes)
{
    return matrix_vector_multiply_transform_weight_bytes_cuda_b200(row, col, dt, df, bytes);
}

EE mvm_cuda_b200(U32 row, U32 col, DataType dt, DataFormat df, const void *matrix, const void *vector,
    void *result, void *offsetCBias, const F32 *scale)
{
    if (dt != DT_I8 && dt != DT_U8_Q) {
        return NOT_SUPPORTED;
    }
    if (offsetCBias == nullptr) {
        return NULL_POINTER;  // CHECK_REQUIREMENT(offsetCBias != nullptr), cpu/x86/mvm.cpp:119,126
    }
    if (dt == DT_U8_Q) {
        // u8 matrix x s8 vector (mvm_avx512_int8_row_i8u8): the offset is -128 * sum(vector), found per call
        if (df != DF_NORMAL && df != DF_TRANSPOSE) {
            return NOT_SUPPORTED;
        }
        if (ctx() == nullptr) {
            return UNKNOWN;
        }
        if (row == 0) {
            return SUCCESS;
        }
        if (matrix == nullptr || vector == nullptr || result == nullptr) {
            return NULL_POINTER;
        }
        GemmEpilogue ep;
        scale_to_epilogue(scale, &ep);
        Stage sg;
        const uint8_t *dM = reinterpret_cast<const uint8_t *>(sg.in(matrix, (size_t)row * col));
        const int8_t *dv = reinterpret_cast<const int8_t *>(sg.in(vector, col));
        void *dy = sg.out(result, (size_t)row * (ep.out_kind == 2 ? 1 : 4));
        if (dM == nullptr || dv == nullptr || dy == nullptr) {
            return ALLOC_FAILED;
        }
        B200_EE(launch_gemv_row(row, col, dM, df == DF_TRANSPOSE, dv, dy, ep.out_kind, ep.factor, tls().stream));
        return sg.finish();
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (row == 0) {
        return SUCCESS;
    }
    if (matrix == nullptr || vector == nullptr || result == nullptr) {
        return NULL_POINTER;
    }
    const U32 N = row, K = col;
    const U32 Np = B200_ALIGN(N, 16), Kp = B200_ALIGN(K, 8);
    // packed on the fly into tmp: offsetC first, matrix behind it (mvm_avx512_vnni.cpp:724-726)
    const char *mat = reinterpret_cast<const char *>(matrix);
    if (matrix == offsetCBias) {
        mat += (size_t)N * 4;
    }
    GemmEpilogue ep;
    scale_to_epilogue(scale, &ep);
    const size_t esz = ep.out_kind == 2 ? 1 : 4;
    Stage sg;
    const int8_t *dW = reinterpret_cast<const int8_t *>(resolve_weight(mat, (size_t)Np * Kp, sg));
    const uint8_t *dx = reinterpret_cast<const uint8_t *>(sg.in(vector, K));
    const int32_t *dOff = reinterpret_cast<const int32_t *>(sg.in(offsetCBias, (size_t)N * 4));
    void *dy = sg.out(result, (size_t)N * esz, ep.out_kind != 2);
    if (dW == nullptr || dx == nullptr || dOff == nullptr || dy == nullptr) {
        return ALLOC_FAILED;
    }
    B200_EE(launch_gemv(N, K, dW, Kp, dx, dOff, dy, ep.out_kind, ep.factor, tls().stream));
    return sg.finish();
}

// =============================== operator-level mirrors ========================================
EE b200_matrix_matrix_multiply_tmp_bytes(TensorDesc aDesc, TensorDesc bDesc, U32 *bytes, Arch arch)
{
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    DataType adt, bdt;
    DataFormat adf, bdf;
    U32 aM, aK, bK, bN;
    B200_EE(get2d(aDesc, &adt, &adf, &aM, &aK));
    B200_EE(get2d(bDesc, &bdt, &bdf, &bK, &bN));
    if (adf == DF_TRANSPOSE) {
        std::swap(aM, aK);
    }
    if (bdf == DF_TRANSPOSE) {
        std::swap(bK, bN);
    }
    return matrix_matrix_multiply_tmp_bytes_cuda_b200(bN, aM, bK, adt, adf, bdt, bdf, bytes);
}

DataFormat b200_matrix_matrix_multiply_rhs_format(DataType dt)
{
    (void)dt;
    return DF_NKNxKx;  // mmm.cpp:85-88 for DT_I8
}

EE b200_matrix_matrix_multiply_transform_rhs_bytes(TensorDesc desc, U32 *bytes, U32 *rhsBytes, Arch arch)
{
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    DataType dt;
    DataFormat df;
    U32 K, N;
    B200_EE(get2d(desc, &dt, &df, &K, &N));
    if (df == DF_TRANSPOSE) {
        std::swap(K, N);
    }
    return matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(N, K, dt, df, bytes, rhsBytes);
}

EE b200_matrix_matrix_multiply_transform_rhs(TensorDesc desc, const void *src, TensorDesc *descTran, void *dst, Arch arch)
{
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    return matrix_matrix_multiply_transform_rhs_cuda_b200(&desc, src, descTran, dst);
}

// mmm.cpp:150-238
EE b200_matrix_matrix_multiply(TensorDesc aDesc, const void *A, TensorDesc bDesc, const void *B, U32 bytes,
    void *tmp, TensorDesc cDesc, void *C, const F32 *scale, Arch arch)
{
    if (bytes != 0 && tmp == nullptr) {
        return NULL_POINTER;
    }
    if (A == nullptr || B == nullptr || C == nullptr) {
        return NULL_POINTER;
    }
    if (num_elems(cDesc) == 0) {
        return SUCCESS;
    }
    DataType adt, bdt, cdt;
    DataFormat adf, bdf, cdf;
    U32 aM, aK, bK, bN, cM, cN;
    B200_EE(get2d(aDesc, &adt, &adf, &aM, &aK));
    B200_EE(get2d(bDesc, &bdt, &bdf, &bK, &bN));
    B200_EE(get2d(cDesc, &cdt, &cdf, &cM, &cN));
    if (adt != bdt && !(adt == DT_U8_Q && bdt == DT_I8)) {
        return NOT_MATCH;
    }
    if (adf == DF_TRANSPOSE) {
        std::swap(aM, aK);
    }
    if (bdf == DF_TRANSPOSE) {
        std::swap(bK, bN);
    }
    if (aM != cM || bN != cN || aK != bK) {
        return NOT_MATCH;
    }
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    if (!(adt == DT_U8_Q && bdt == DT_I8)) {
        return NOT_SUPPORTED;
    }
    const void *packed = B;
    bool packed_here = false;
    if (bdf != DF_NKNxKx) {
        U32 rhsBytes = 0;
        B200_EE(matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(bN, bK, bdt, bdf, nullptr, &rhsBytes));
        if (bytes < rhsBytes + bN * 4) {
            return NOT_MATCH;  // CHECK_REQUIREMENT(bytes >= transBBytes), mmm.cpp:211-212
        }
        TensorDesc packedDesc;
        B200_EE(matrix_matrix_multiply_transform_rhs_cuda_b200(&bDesc, B, &packedDesc, tmp));
        packed = tmp;
        packed_here = true;
        tmp = reinterpret_cast<char *>(tmp) + rhsBytes;  // offsetC sits there (mmm.cpp:217-218)
    }
    if (cdt == DT_I32) {
        scale = nullptr;  // mmm.cpp:222-224
    }
    const EE ret = mmm_cuda_b200(cN, cM, aK, bdt, adf, A, packed, tmp, C, scale);
    if (packed_here && !is_device_ptr(packed)) {
        // the caller's scratch is not a weight: its device copy served this call only (a later call may
        // put other bytes at the same host address)
        bolt_b200_release_weight(packed);
    }
    return ret;
}

EE b200_matrix_vector_multiply_tmp_bytes(TensorDesc mDesc, TensorDesc vDesc, U32 *bytes, Arch arch)
{
    (void)vDesc;
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    DataType dt;
    DataFormat df;
    U32 row, col;
    B200_EE(get2d(mDesc, &dt, &df, &row, &col));
    if (df == DF_TRANSPOSE) {
        std::swap(row, col);
    }
    return matrix_vector_multiply_tmp_bytes_cuda_b200(row, col, dt, df, bytes);
}

DataFormat b200_matrix_vector_multiply_weight_format(DataType dt)
{
    return dt == DT_U8_Q ? DF_NK : DF_NKN32K4;  // mvm.cpp:55-70
}

EE b200_matrix_vector_multiply_transform_weight_bytes(TensorDesc desc, U32 *bytes, Arch arch)
{
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    DataType dt;
    DataFormat df;
    U32 row, col;
    B200_EE(get2d(desc, &dt, &df, &row, &col));
    if (df == DF_TRANSPOSE) {
        std::swap(row, col);
    }
    return matrix_vector_multiply_transform_weight_bytes_cuda_b200(row, col, dt, df, bytes);
}

EE b200_matrix_vector_multiply_transform_weight(TensorDesc desc, const void *src, TensorDesc *descTran, void *dst, Arch arch)
{
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    return matrix_vector_multiply_transform_weight_cuda_b200(&desc, src, descTran, dst, nullptr);
}

// mvm.cpp:132-194
EE b200_matrix_vector_multiply(TensorDesc mDesc, const void *matrix, TensorDesc vDesc, const void *vector, U32 bytes,
    void *tmp, TensorDesc rDesc, void *result, const F32 *scale, Arch arch)
{
    if ((bytes != 0 && tmp == nullptr) || matrix == nullptr || vector == nullptr || result == nullptr) {
        return NULL_POINTER;
    }
    DataType mdt, vdt, rdt;
    DataFormat mdf, vdf, rdf;
    U32 row, col, vlen, rlen;
    B200_EE(get2d(mDesc, &mdt, &mdf, &row, &col));
    B200_EE(get1d(vDesc, &vdt, &vdf, &vlen));
    B200_EE(get1d(rDesc, &rdt, &rdf, &rlen));
    if (mdf == DF_TRANSPOSE) {
        std::swap(row, col);
    }
    if (row != rlen || col != vlen) {
        return NOT_MATCH;
    }
    if (arch != CUDA_B200) {
        return NOT_SUPPORTED;
    }
    if (!((mdt == DT_I8 && vdt == DT_U8_Q) || (mdt == DT_U8_Q && vdt == DT_I8))) {
        return NOT_SUPPORTED;
    }
    if (tmp == nullptr) {
        return NULL_POINTER;
    }
    if (rdt == DT_I32) {
        scale = nullptr;
    }
    if (mdt == DT_U8_Q) {
        if (mdf == DF_NK) {
            return NOT_SUPPORTED;  // mvm.cpp:170-173
        }
        return mvm_cuda_b200(row, col, mdt, mdf, matrix, vector, result, tmp, scale);
    }
    const void *dataB = matrix;
    if (mdf != DF_NKN32K4) {
        // pack into tmp: offsetC first, matrix behind it (mvm.cpp:175-181)
        if (bytes < rlen * 4 + B200_ALIGN(row, 16) * B200_ALIGN(col, 8)) {
            return NOT_MATCH;
        }
        TensorDesc packedDesc;
        B200_EE(matrix_vector_multiply_transform_weight_cuda_b200(
            &mDesc, matrix, &packedDesc, reinterpret_cast<char *>(tmp) + (size_t)rlen * 4, tmp));
        dataB = tmp;
    }
    const EE ret = mvm_cuda_b200(row, col, mdt, mdf, dataB, vector, result, tmp, scale);
    if (dataB == tmp && !is_device_ptr(tmp)) {
        // the caller's scratch is not a weight: drop the device copy made while packing into it
        bolt_b200_release_weight(reinterpret_cast<char *>(tmp) + (size_t)rlen * 4);
    }
    return ret;
}

}  // extern "C"
