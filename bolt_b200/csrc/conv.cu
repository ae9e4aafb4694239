// conv.cu -- int8 and 1-bit convolution entry points.
#include "common.cuh"

extern "C" {

EE convolution_infer_forward_algorithm_cuda_b200(const TensorDesc *, const TensorDesc *, const TensorDesc *,
    const ConvolutionParamSpec *, ConvolutionPolicy, ConvolutionForwardAlgorithm *, DataType)
{
    return NOT_IMPLEMENTED;
}
EE convolution_transform_filter_bytes_cuda_b200(
    const TensorDesc *, const ConvolutionParamSpec *, ConvolutionForwardAlgorithm, U32 *)
{
    return NOT_IMPLEMENTED;
}
EE convolution_transform_filter_cuda_b200(const TensorDesc *, const void *, const ConvolutionParamSpec *,
    ConvolutionForwardAlgorithm, TensorDesc *, void *)
{
    return NOT_IMPLEMENTED;
}
EE convolution_infer_forward_tmp_bytes_cuda_b200(const TensorDesc *, const TensorDesc *, const TensorDesc *,
    const ConvolutionParamSpec *, ConvolutionForwardAlgorithm, U32 *)
{
    return NOT_IMPLEMENTED;
}
EE convolution_cuda_b200(const TensorDesc *, void *, void *, const TensorDesc *, const void *,
    const ConvolutionParamSpec *, ConvolutionForwardAlgorithm, const TensorDesc *, void *, const TensorDesc *,
    const void *, U32, void *, const TensorDesc *, void *, const ActivationParamSpec *)
{
    return NOT_IMPLEMENTED;
}
}
