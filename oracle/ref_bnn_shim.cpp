// TEST INFRASTRUCTURE ONLY -- never linked into, or loaded by, the product library.
//
// Compiles the reference's scalar 1-bit convolution (compute/tensor/src/cpu/general/convolution.cpp:
// bnn_input_process :141-159, bnn_filter_process :161-179, the DT_BIN01 / DT_BIN11 cases of
// convolution_general :264-285 and the loop nest :18-138) on x86, where the reference itself cannot
// build it: that code sits behind _USE_FP16, and without NEON data_type.h makes F16 an unsigned short.
// Here F16 is supplied as the compiler's _Float16 instead; the reference sources are included where
// they lie and are not modified.  _Float16 arithmetic is carried out in binary32 and rounded to
// binary16 on assignment, like __fp16 on the ARM targets the reference builds this code for.
//
// What this pins: the binarisation thresholds (>= 0, >= 0.5), the filter bit order (MSB first), the
// padding values (-1 for DT_BIN11, 0 for DT_BIN01), the tap sums -- exact while |sum| <= 2048, the
// range in which binary16 holds every integer -- and scale * sum + bias in binary32 rounded once.
#include <cstdint>
#include <cstring>
#include <vector>

#define _USE_FP16
#define _USE_GENERAL
#define F16 bolt_f16_bits_unused
#include "data_type.h"
#undef F16
typedef _Float16 F16;

#include "cpu/general/convolution.cpp"

extern "C" {

// in / out: binary16 bit patterns, NCHWc8; filter_bits: NCHW, 8 weights per byte, MSB first;
// scale / bias: binary16 [oc].  xnor != 0: DT_BIN11, else DT_BIN01.  Returns the reference's EE code.
int ref_bnn_conv(uint32_t n, uint32_t ic, uint32_t ih, uint32_t iw, uint32_t oc, uint32_t fh, uint32_t fw,
    uint32_t stride_h, uint32_t stride_w, uint32_t pad_t, uint32_t pad_b, uint32_t pad_l, uint32_t pad_r, int xnor,
    const uint16_t *in, const uint8_t *filter_bits, const uint16_t *scale, const uint16_t *bias, uint16_t *out)
{
    const uint32_t oh = (ih + pad_t + pad_b - fh) / stride_h + 1;
    const uint32_t ow = (iw + pad_l + pad_r - fw) / stride_w + 1;
    TensorDesc inputDesc = tensor4df(DT_F16, DF_NCHWC8, n, ic, ih, iw);
    TensorDesc filterDesc = tensor4df(xnor ? DT_BIN11 : DT_BIN01, DF_NCHW, oc, ic, fh, fw);
    TensorDesc outputDesc = tensor4df(DT_F16, DF_NCHWC8, n, oc, oh, ow);
    TensorDesc vecDesc = tensor1d(DT_F16, oc);
    ConvolutionParamSpec p;
    std::memset(&p, 0, sizeof(p));
    p.num_outputs = oc;
    p.kernel_t = 1;
    p.kernel_h = fh;
    p.kernel_w = fw;
    p.stride_t = 1;
    p.stride_h = stride_h;
    p.stride_w = stride_w;
    p.pad_top = pad_t;
    p.pad_bottom = pad_b;
    p.pad_left = pad_l;
    p.pad_right = pad_r;
    p.group = 1;
    p.dilatedRate_t = 1;
    p.dilatedRate_h = 1;
    p.dilatedRate_w = 1;
    ActivationParamSpec act;
    std::memset(&act, 0, sizeof(act));
    act.mode = ACTIVATION_NULL;
    return (int)convolution_general(inputDesc, (void *)in, nullptr, filterDesc, (const void *)filter_bits, p, vecDesc,
        (const void *)scale, vecDesc, (const void *)bias, 0, nullptr, outputDesc, (void *)out, act);
}

}  // extern "C"
