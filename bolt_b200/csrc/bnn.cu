// bnn.cu -- 1-bit (XNOR / DoReFa) convolution.  Placeholder bodies until the kernels land.
#include "common.cuh"

namespace b200 {
EE bnn_transform_filter_bytes(const TensorDesc *, U32 *) { return NOT_IMPLEMENTED; }
EE bnn_transform_filter(const TensorDesc *, const void *, TensorDesc *, void *) { return NOT_IMPLEMENTED; }
EE bnn_tmp_bytes(const TensorDesc *, const TensorDesc *, const TensorDesc *, const ConvolutionParamSpec *, U32 *) { return NOT_IMPLEMENTED; }
EE bnn_run(const TensorDesc *, const void *, const TensorDesc *, const void *, const ConvolutionParamSpec *, const void *,
    const void *, U32, void *, const TensorDesc *, void *) { return NOT_IMPLEMENTED; }
}  // namespace b200
