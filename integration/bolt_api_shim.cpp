// C-callable wrappers around Bolt's C++ (Tensor-based) entry points, for tests written in Python.
//
// Everything here is Bolt's own API used as an application would use it: a Tensor is made over a
// caller's buffer, an ArchInfo with arch = CUDA_B200 is passed, and Bolt's dispatcher -- built with
// the CUDA_B200 branch by build_dispatch.py -- does the rest.  No function of libbolt_b200.so is
// called from this file.
#include <memory>
#include <vector>

#include "tensor_computing.h"
#include "blas_enhance.h"

namespace {
Tensor over(const TensorDesc &desc, void *ptr)
{
    Tensor t;
    t.resize(desc);
    if (ptr != nullptr) {
        ((CpuMemory *)t.get_memory())->set_shared_ptr(std::shared_ptr<U8>((U8 *)ptr, [](U8 *) {}));
    }
    return t;
}

ArchInfo b200()
{
    ArchInfo a;
    a.arch = CUDA_B200;
    a.archPara = nullptr;
    return a;
}
}  // namespace

extern "C" {

int shim_arch_cuda_b200()
{
    return (int)CUDA_B200;
}

const char *shim_arch_name()
{
    return ArchName()[CUDA_B200];
}

EE shim_quantize(const TensorDesc *dDesc, void *data, TensorDesc *qDesc, void *qData, F32 *scale)
{
    ArchInfo a = b200();
    Tensor in = over(*dDesc, data), out = over(*qDesc, qData);
    EE ret = quantize(in, &out, scale, &a);
    *qDesc = out.get_desc();
    return ret;
}

EE shim_dequantize(const TensorDesc *qDesc, void *qData, const F32 *scale, const TensorDesc *bDesc,
    void *bData, const TensorDesc *dDesc, void *data)
{
    ArchInfo a = b200();
    Tensor in = over(*qDesc, qData), out = over(*dDesc, data);
    Tensor bias = bData ? over(*bDesc, bData) : Tensor();
    if (!bData) {
        TensorDesc none = *bDesc;
        bias.resize(none);
    }
    return dequantize(in, scale, bias, out, &a);
}

EE shim_conv_output_size(const TensorDesc *inDesc, const TensorDesc *fDesc,
    const ConvolutionParamSpec *p, TensorDesc *outDesc, DataType target)
{
    ArchInfo a = b200();
    Tensor in = over(*inDesc, nullptr), f = over(*fDesc, nullptr), out;
    EE ret = convolution_infer_output_size(&in, f, *p, &out, target, &a);
    *outDesc = out.get_desc();
    return ret;
}

// matmul as inference/engine/include/cpu/matmul_cpu.hpp drives it: output size, tmp bytes, run; scales in the tensors
EE shim_matmul(const TensorDesc *aDesc, void *A, F32 aScale, int transposeA, const TensorDesc *bDesc, void *B,
    F32 bScale, int transposeB, U32 biasLen, void *bias, DataType cType, F32 *cScale, void *C, TensorDesc *cDesc,
    void *tmp, U32 tmpCapacity)
{
    ArchInfo a = b200();
    Tensor ta = over(*aDesc, A), tb = over(*bDesc, B), tc;
    ta.set_scale(aScale);
    tb.set_scale(bScale);
    EE ret = matmul_infer_output_size(&ta, transposeA != 0, &tb, transposeB != 0, &tc, &a);
    if (ret != SUCCESS) {
        return ret;
    }
    TensorDesc cd = tc.get_desc();
    cd.dt = cType;
    tc = over(cd, C);
    tc.set_scale(*cScale);
    U32 bytes = 0;
    ret = matmul_infer_forward_tmp_bytes(ta, transposeA != 0, tb, transposeB != 0, tc, &bytes, &a);
    if (ret != SUCCESS) {
        return ret;
    }
    if (bytes > tmpCapacity) {
        return NOT_MATCH;
    }
    std::vector<Tensor> tmps = {over(tensor1d(DT_U8, bytes), tmp)};
    Tensor tbias;
    if (biasLen > 0) {
        tbias = over(tensor1d(DT_F32, biasLen), bias);
    }
    ret = matmul(ta, transposeA != 0, tb, transposeB != 0, tbias, tmps, tc, &a);
    *cScale = tc.get_scale();
    *cDesc = cd;
    return ret;
}

// the sequence an operator runs once (algorithm, packed-filter size, packing) ...
EE shim_conv_prepare(const TensorDesc *inDesc, const TensorDesc *fDesc, void *filter,
    const TensorDesc *outDesc, const ConvolutionParamSpec *p, const ActivationParamSpec *act,
    DataType target, int *algorithm, U32 *ftmBytes, void *ftm, TensorDesc *ftmDesc, U32 *tmpBytes)
{
    ArchInfo a = b200();
    Tensor in = over(*inDesc, nullptr), f = over(*fDesc, filter), out = over(*outDesc, nullptr);
    ConvolutionForwardAlgorithm alg = CONVOLUTION_ALGORITHM_NULL;
    EE ret = convolution_infer_forward_algorithm(
        in, f, out, *p, CONVOLUTION_FASTEST, &alg, target, *act, &a);
    if (ret != SUCCESS) {
        return ret;
    }
    *algorithm = (int)alg;
    U32 bytes = 0;
    ret = convolution_transform_filter_bytes(f, *p, alg, &bytes, &a);
    if (ret != SUCCESS) {
        return ret;
    }
    *ftmBytes = bytes;
    ret = convolution_infer_forward_tmp_bytes(in, f, out, *p, alg, tmpBytes, &a);
    if (ret != SUCCESS || ftm == nullptr) {
        return ret;
    }
    TensorDesc flat = tensor1d(DT_U8, bytes);
    Tensor packed = over(flat, ftm), none;
    ret = convolution_transform_filter(f, *p, alg, none, &packed, &a);
    *ftmDesc = packed.get_desc();
    return ret;
}

// ... and the call it makes per inference
EE shim_convolution(const TensorDesc *inDesc, void *input, const TensorDesc *eltDesc, void *eltwise,
    const TensorDesc *ftmDesc, void *ftm, const ConvolutionParamSpec *p, int algorithm, F32 *scale,
    const TensorDesc *bDesc, void *bias, U32 tmpBytes, void *tmp, const TensorDesc *outDesc,
    void *output, const ActivationParamSpec *act)
{
    ArchInfo a = b200();
    std::vector<Tensor> ins = {over(*inDesc, input)};
    if (eltwise != nullptr) {
        ins.push_back(over(*eltDesc, eltwise));
    }
    std::vector<Tensor> tmps = {over(tensor1d(DT_U8, tmpBytes), tmp)};
    Tensor f = over(*ftmDesc, ftm), b = over(*bDesc, bias), out = over(*outDesc, output);
    return convolution(ins, f, *p, (ConvolutionForwardAlgorithm)algorithm, scale, b, tmps, out, *act, &a);
}
}
