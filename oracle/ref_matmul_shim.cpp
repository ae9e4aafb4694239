// ref_matmul_shim.cpp -- TEST INFRASTRUCTURE ONLY.
//
// extern "C" harness around the UNMODIFIED reference's `matmul` (compute/tensor/src/matmul.cpp) on its
// x86 AVX512-VNNI int8 branch: Tensors are made over the caller's buffers, the call sequence is the one of
// compute/tensor/tests/test_matmul_int8.cpp (infer output size, query tmp bytes, run).  Compiled into
// oracle/_ref/libbolt_ref.so together with the reference's own sources (see oracle/Makefile).
//
// `quantize_cpu` is what matmul.cpp calls for its operands.  In the reference's x86 int8 build that function is a
// plain forward to quantize_x86 (compute/tensor/src/cpu/quantize.cpp:62-72); its translation unit also pulls in
// fp32 array helpers that this reduced build does not carry, so the forward is restated here.
#include <cstring>
#include <memory>
#include <vector>

#include "tensor_computing.h"
#include "cpu/tensor_computing_cpu.h"
#include "cpu/x86/tensor_computing_x86.h"

EE quantize_cpu(TensorDesc dDesc, const void *data, TensorDesc *qDesc, void *qData, F32 *scale, Arch arch, int mode)
{
    if (nullptr == data || nullptr == qDesc || nullptr == qData || nullptr == scale) {
        return NULL_POINTER;
    }
    return quantize_x86(dDesc, data, qDesc, qData, scale, mode);
}

namespace {
Tensor over(const TensorDesc &desc, void *ptr, float scale)
{
    Tensor t;
    t.resize(desc);
    if (ptr != nullptr) {
        ((CpuMemory *)t.get_memory())->set_shared_ptr(std::shared_ptr<U8>((U8 *)ptr, [](U8 *) {}));
    }
    t.set_scale(scale);
    return t;
}
TensorDesc make_desc(int dt, uint32_t nd, const uint32_t *dims_outer_first)
{
    TensorDesc d;
    d.dt = (DataType)dt;
    d.df = nd == 2 ? DF_NORMAL : (nd == 3 ? DF_MTK : DF_NCHW);
    d.nDims = nd;
    for (uint32_t i = 0; i < nd; ++i) {
        d.dims[nd - 1 - i] = dims_outer_first[i];
    }
    return d;
}
}  // namespace

extern "C" {

// dims are given outermost first (numpy order).  c_dt / c_scale describe the output tensor the caller
// allocated (DT_F32 with a non-zero scale flag, or DT_U8_Q with a positive or non-positive scale).
// Returns the reference's status; writes the output dims (outermost first) and the output tensor's scale.
int ref_matmul(int a_dt, uint32_t a_nd, const uint32_t *a_dims, float a_scale, int transA, void *A,
    int b_dt, uint32_t b_nd, const uint32_t *b_dims, float b_scale, int transB, void *B,
    uint32_t bias_n, void *bias, int c_dt, float c_scale, void *C, uint64_t c_capacity_bytes,
    uint32_t *c_nd, uint32_t *c_dims, float *c_scale_out)
{
    ArchInfo arch;
    arch.arch = X86_AVX512;
    arch.archPara = nullptr;
    Tensor a = over(make_desc(a_dt, a_nd, a_dims), A, a_scale);
    Tensor b = over(make_desc(b_dt, b_nd, b_dims), B, b_scale);
    Tensor c;
    EE ret = matmul_infer_output_size(&a, transA != 0, &b, transB != 0, &c, &arch);
    if (ret != SUCCESS) {
        return (int)ret;
    }
    TensorDesc cd = c.get_desc();
    cd.dt = (DataType)c_dt;
    if (tensorNumBytes(cd) > c_capacity_bytes) {
        return (int)NOT_MATCH;
    }
    c = over(cd, C, c_scale);
    U32 bytes = 0;
    ret = matmul_infer_forward_tmp_bytes(a, transA != 0, b, transB != 0, c, &bytes, &arch);
    if (ret != SUCCESS) {
        return (int)ret;
    }
    std::vector<U8> tmp_store((size_t)bytes + 4096, 0);
    std::vector<Tensor> tmps = {over(tensor1d(DT_U8, bytes + 2048), tmp_store.data(), 1.0f)};
    Tensor biasT;
    if (bias_n > 0) {
        biasT = over(tensor1d(DT_F32, bias_n), bias, 1.0f);
    }
    ret = matmul(a, transA != 0, b, transB != 0, biasT, tmps, c, &arch);
    *c_nd = cd.nDims;
    for (uint32_t i = 0; i < cd.nDims; ++i) {
        c_dims[i] = cd.dims[cd.nDims - 1 - i];
    }
    *c_scale_out = c.get_scale();
    return (int)ret;
}
}
