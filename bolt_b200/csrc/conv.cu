// conv.cu -- convolution entry points: dispatch on the filter type to the int8 implicit-GEMM path
// (conv_i8.cu) or the 1-bit path (bnn.cu), as Bolt's convolution dispatchers do
// (compute/tensor/src/convolution.cpp:367-470, cpu/x86/convolution.cpp:233-363,
//  cpu/arm/convolution.cpp:492-494).
#include <cstring>

#include "common.cuh"

namespace b200 {
EE conv_i8_transform_filter_bytes(const TensorDesc *filterDesc, U32 *bytes);
EE conv_i8_transform_filter(const TensorDesc *filterDesc, const void *filter, TensorDesc *ftmDesc, void *dst);
EE conv_i8_tmp_bytes(const TensorDesc *inputDesc, const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *cp, U32 *bytes);
EE conv_i8_run(const TensorDesc *inputDesc, void *input, void *eltwiseInput, const TensorDesc *filterDesc,
    const void *filter, const ConvolutionParamSpec *cp, void *scale, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *act, const bolt_b200_conv_ext *ext);
EE bnn_transform_filter_bytes(const TensorDesc *filterDesc, U32 *bytes);
EE bnn_transform_filter(const TensorDesc *filterDesc, const void *filter, TensorDesc *ftmDesc, void *dst);
EE bnn_tmp_bytes(const TensorDesc *inputDesc, const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *cp, U32 *bytes);
EE bnn_run(const TensorDesc *inputDesc, const void *input, const TensorDesc *filterDesc, const void *filter,
    const ConvolutionParamSpec *cp, const void *scale, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output);
}  // namespace b200

using namespace b200;

namespace {
bool is_bnn(DataType dt)
{
    return dt == DT_BIN01 || dt == DT_BIN11;
}
}  // namespace

extern "C" {

EE convolution_infer_output_size_cuda_b200(const TensorDesc *inputDesc, const TensorDesc *filterDesc,
    const ConvolutionParamSpec *p, TensorDesc *outputDesc, DataType targetDataType)
{
    if (inputDesc == nullptr || filterDesc == nullptr || p == nullptr || outputDesc == nullptr) {
        return NULL_POINTER;
    }
    if (inputDesc->nDims != 4 || filterDesc->nDims != 4) {
        return NOT_SUPPORTED;  // the 3-D (t, h, w) form of convolution.cpp:47-49 is not on this path
    }
    const U32 iw = inputDesc->dims[0], ih = inputDesc->dims[1], in = inputDesc->dims[3];
    const U32 fw = filterDesc->dims[0], fh = filterDesc->dims[1], fn = filterDesc->dims[3];
    EE ret = SUCCESS;
    if (fh < 1 || fw < 1) {
        ret = NOT_SUPPORTED;
    }
    const U32 fhd = (fh - 1) * p->dilatedRate_h + 1, fwd = (fw - 1) * p->dilatedRate_w + 1;
    const U32 sh = p->stride_h ? p->stride_h : 1, sw = p->stride_w ? p->stride_w : 1;
    long oh, ow;
    if (p->round_mode == 6 /* ROUND_SAME_UPPER, parameter_spec.h:24-33 */) {
        oh = (ih + sh - 1) / sh;
        ow = (iw + sw - 1) / sw;
    } else if (p->round_mode == 7 /* ROUND_SAME_LOWER */) {
        oh = ih / sh;
        ow = iw / sw;
    } else {
        oh = ((long)ih + p->pad_top + p->pad_bottom - (long)fhd) / (long)sh + 1;
        ow = ((long)iw + p->pad_left + p->pad_right - (long)fwd) / (long)sw + 1;
    }
    if (oh < 0 || ow < 0) {
        ret = NOT_MATCH;
    }
    if (fn % 8 != 0) {
        return NOT_SUPPORTED;  // convolution.cpp:95-97
    }
    // the rule of the AVX512 int8 build (convolution.cpp:98-103), whose layouts this backend writes
    const DataFormat odf = (targetDataType == DT_U8_Q && fn != 8) ? DF_NCHWC16 : DF_NCHWC8;
    std::memset(outputDesc, 0, sizeof(*outputDesc));
    outputDesc->dt = targetDataType;
    outputDesc->df = odf;
    outputDesc->nDims = 4;
    outputDesc->dims[0] = (U32)(ow < 0 ? 0 : ow);
    outputDesc->dims[1] = (U32)(oh < 0 ? 0 : oh);
    outputDesc->dims[2] = fn;
    outputDesc->dims[3] = in;
    return ret;
}

EE convolution_infer_forward_algorithm_cuda_b200(const TensorDesc *inputDesc, const TensorDesc *filterDesc,
    const TensorDesc *outputDesc, const ConvolutionParamSpec *convParamSpec, ConvolutionPolicy policy,
    ConvolutionForwardAlgorithm *algorithm, DataType targetDataType)
{
    (void)inputDesc;
    (void)outputDesc;
    (void)policy;
    (void)targetDataType;
    if (filterDesc == nullptr || convParamSpec == nullptr || algorithm == nullptr) {
        return NULL_POINTER;
    }
    if (*algorithm != CONVOLUTION_ALGORITHM_NULL) {
        return SUCCESS;  // a preset algorithm is honoured (convolution.cpp:158-160)
    }
    if (filterDesc->nDims != 4) {
        return NOT_SUPPORTED;
    }
    if (is_bnn(filterDesc->dt)) {
        *algorithm = CONVOLUTION_ALGORITHM_BNN;
    } else if (filterDesc->dims[0] == 1 && filterDesc->dims[1] == 1) {
        *algorithm = CONVOLUTION_ALGORITHM_POINTWISE;  // cpu/x86/convolution.cpp:60-62
    } else {
        *algorithm = CONVOLUTION_ALGORITHM_DIRECT;
    }
    return SUCCESS;
}

EE convolution_transform_filter_bytes_cuda_b200(const TensorDesc *filterDesc, const ConvolutionParamSpec *convParamSpec,
    ConvolutionForwardAlgorithm algorithm, U32 *bytes)
{
    (void)convParamSpec;
    (void)algorithm;
    if (filterDesc == nullptr || bytes == nullptr) {
        return NULL_POINTER;
    }
    if (is_bnn(filterDesc->dt)) {
        return bnn_transform_filter_bytes(filterDesc, bytes);
    }
    if (filterDesc->dt != DT_I8) {
        return NOT_SUPPORTED;
    }
    return conv_i8_transform_filter_bytes(filterDesc, bytes);
}

EE convolution_transform_filter_cuda_b200(const TensorDesc *filterDesc, const void *filter,
    const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm, TensorDesc *ftmDesc,
    void *filterTransformed)
{
    (void)algorithm;
    if (filterDesc == nullptr || ftmDesc == nullptr) {
        return NULL_POINTER;
    }
    if (convParamSpec != nullptr && convParamSpec->group > 1) {
        return NOT_SUPPORTED;
    }
    if (is_bnn(filterDesc->dt)) {
        return bnn_transform_filter(filterDesc, filter, ftmDesc, filterTransformed);
    }
    if (filterDesc->dt != DT_I8) {
        return NOT_SUPPORTED;
    }
    return conv_i8_transform_filter(filterDesc, filter, ftmDesc, filterTransformed);
}

EE convolution_infer_forward_tmp_bytes_cuda_b200(const TensorDesc *inputDesc, const TensorDesc *filterDesc,
    const TensorDesc *outputDesc, const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm,
    U32 *bytes)
{
    (void)algorithm;
    if (inputDesc == nullptr || filterDesc == nullptr || outputDesc == nullptr || convParamSpec == nullptr) {
        return NULL_POINTER;
    }
    if (is_bnn(filterDesc->dt)) {
        return bnn_tmp_bytes(inputDesc, filterDesc, outputDesc, convParamSpec, bytes);
    }
    return conv_i8_tmp_bytes(inputDesc, filterDesc, outputDesc, convParamSpec, bytes);
}

EE convolution_cuda_b200(const TensorDesc *inputDesc, void *input, void *eltwiseInput, const TensorDesc *filterDesc,
    const void *filter, const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm,
    const TensorDesc *scaleDesc, void *scale, const TensorDesc *biasDesc, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *activationDesc)
{
    (void)algorithm;
    (void)scaleDesc;
    (void)biasDesc;
    if (inputDesc == nullptr || filterDesc == nullptr || outputDesc == nullptr || convParamSpec == nullptr) {
        return NULL_POINTER;
    }
    if (is_bnn(filterDesc->dt)) {
        // `scale` and `bias`: fp16 per-output-channel arrays (convolution.cpp:413-423 splits them)
        return bnn_run(inputDesc, input, filterDesc, filter, convParamSpec, scale, bias, tmpBytes, tmp, outputDesc,
            output);
    }
    return conv_i8_run(inputDesc, input, eltwiseInput, filterDesc, filter, convParamSpec, scale, bias, tmpBytes, tmp,
        outputDesc, output, activationDesc, nullptr);
}

EE bolt_b200_convolution_ex(const TensorDesc *inputDesc, void *input, void *eltwiseInput, const TensorDesc *filterDesc,
    const void *filter, const ConvolutionParamSpec *convParamSpec, ConvolutionForwardAlgorithm algorithm,
    const TensorDesc *scaleDesc, void *scale, const TensorDesc *biasDesc, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *activationDesc, const bolt_b200_conv_ext *ext)
{
    if (filterDesc == nullptr || ext == nullptr || is_bnn(filterDesc->dt)) {
        return convolution_cuda_b200(inputDesc, input, eltwiseInput, filterDesc, filter, convParamSpec, algorithm, scaleDesc,
            scale, biasDesc, bias, tmpBytes, tmp, outputDesc, output, activationDesc);
    }
    if (inputDesc == nullptr || outputDesc == nullptr || convParamSpec == nullptr) {
        return NULL_POINTER;
    }
    return conv_i8_run(inputDesc, input, eltwiseInput, filterDesc, filter, convParamSpec, scale, bias, tmpBytes, tmp,
        outputDesc, output, activationDesc, ext);
}

}  // extern "C"
