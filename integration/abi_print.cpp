// Prints the size, field offsets and enumerator values of every type that crosses the C ABI.
// Compiled twice -- with the stand-in typedefs of bolt_b200.h, and with -DBOLT_B200_WITH_BOLT_HEADERS
// against Bolt's own headers -- the two outputs must be identical; the second is kept as
// tests/golden/abi_values.txt.
#include <cstddef>
#include <cstdio>

#include "bolt_b200.h"

#define V(expr) std::printf("%s = %lld\n", #expr, (long long)(expr))

int main()
{
    V(sizeof(EE));
    V(SUCCESS);
    V(NULL_POINTER);
    V(NOT_MATCH);
    V(NOT_FOUND);
    V(ALLOC_FAILED);
    V(NOT_IMPLEMENTED);
    V(NOT_SUPPORTED);
    V(UNKNOWN);
    V(sizeof(Arch));
    V(CPU_GENERAL);
    V(X86_AVX512);
    V(X86_AVXVNNI);
    V(sizeof(ArchInfo));
    V(offsetof(ArchInfo, arch));
    V(offsetof(ArchInfo, archPara));
    V(sizeof(DataType));
    V(DT_U8);
    V(DT_I8);
    V(DT_U32);
    V(DT_I32);
    V(DT_F16);
    V(DT_F32);
    V(DT_BIN01);
    V(DT_BIN11);
    V(DT_U8_Q);
    V(sizeof(DataFormat));
    V(DF_NCHW);
    V(DF_NCHWC8);
    V(DF_NCHWN16C8);
    V(DF_TRANSPOSE);
    V(DF_NORMAL);
    V(DF_NK);
    V(DF_NKN32K4);
    V(DF_NKNxKx);
    V(DF_NCHWC16);
    V(DF_NCHWC2NxC4);
    V(sizeof(TensorDesc));
    V(offsetof(TensorDesc, dt));
    V(offsetof(TensorDesc, df));
    V(offsetof(TensorDesc, nDims));
    V(offsetof(TensorDesc, dims));
    V(sizeof(ActivationMode));
    V(ACTIVATION_NULL);
    V(ACTIVATION_RELU);
    V(sizeof(ActivationParamSpec));
    V(offsetof(ActivationParamSpec, mode));
    V(offsetof(ActivationParamSpec, value));
    V(sizeof(ConvolutionForwardAlgorithm));
    V(CONVOLUTION_ALGORITHM_POINTWISE);
    V(CONVOLUTION_ALGORITHM_DIRECT);
    V(CONVOLUTION_ALGORITHM_BNN);
    V(CONVOLUTION_ALGORITHM_NULL);
    V(sizeof(ConvolutionPolicy));
    V(sizeof(ConvolutionParamSpec));
    V(offsetof(ConvolutionParamSpec, num_outputs));
    V(offsetof(ConvolutionParamSpec, kernel_t));
    V(offsetof(ConvolutionParamSpec, kernel_h));
    V(offsetof(ConvolutionParamSpec, kernel_w));
    V(offsetof(ConvolutionParamSpec, stride_t));
    V(offsetof(ConvolutionParamSpec, stride_h));
    V(offsetof(ConvolutionParamSpec, stride_w));
    V(offsetof(ConvolutionParamSpec, pad_before));
    V(offsetof(ConvolutionParamSpec, pad_after));
    V(offsetof(ConvolutionParamSpec, pad_top));
    V(offsetof(ConvolutionParamSpec, pad_bottom));
    V(offsetof(ConvolutionParamSpec, pad_left));
    V(offsetof(ConvolutionParamSpec, pad_right));
    V(offsetof(ConvolutionParamSpec, group));
    V(offsetof(ConvolutionParamSpec, dilatedRate_t));
    V(offsetof(ConvolutionParamSpec, dilatedRate_h));
    V(offsetof(ConvolutionParamSpec, dilatedRate_w));
    V(offsetof(ConvolutionParamSpec, num_outputs_origin));
    V(offsetof(ConvolutionParamSpec, convolution_type));
    V(offsetof(ConvolutionParamSpec, dw_activation_type));
    V(offsetof(ConvolutionParamSpec, pw_activation_type));
    V(offsetof(ConvolutionParamSpec, activation_spec));
    V(offsetof(ConvolutionParamSpec, round_mode));
    V(offsetof(ConvolutionParamSpec, output_pad_t));
    V(offsetof(ConvolutionParamSpec, output_pad_h));
    V(offsetof(ConvolutionParamSpec, output_pad_w));
    V(sizeof(PoolingMode));
    V(POOLING_MAX);
    V(POOLING_MEAN);
    V(sizeof(PoolingParamSpec));
    V(offsetof(PoolingParamSpec, kernel_t));
    V(offsetof(PoolingParamSpec, kernel_h));
    V(offsetof(PoolingParamSpec, kernel_w));
    V(offsetof(PoolingParamSpec, stride_h));
    V(offsetof(PoolingParamSpec, stride_w));
    V(offsetof(PoolingParamSpec, pad_top));
    V(offsetof(PoolingParamSpec, pad_left));
    V(offsetof(PoolingParamSpec, pad_right));
    V(offsetof(PoolingParamSpec, round_mode));
    V(offsetof(PoolingParamSpec, mode));
    V(offsetof(PoolingParamSpec, count_include_pad));
    return 0;
}
