// bnn.cu -- 1-bit convolution (XNOR-Net: DT_BIN11, DoReFa: DT_BIN01) on packed 32-bit words.
//
// Replaces Bolt's ARMv8.2 kernels (compute/tensor/src/cpu/arm/bnn/convolution_xnor_A76.cpp:17-724,
// convolution_dorefa_A76.cpp:17-715), the filter bit repack (convolution_transform_bnn.h:32-86) and
// the input binarisation (common/uni/include/data_type.h:197-233):
//   bit(x)  = x >= 0 (BIN11) or x >= 0.5 (BIN01); padding is a zero bit in both modes
//   XNOR    : sum = fh*fw*ic - 2 * popcount(x XOR w)       (zero bit = -1)
//   DoReFa  : sum = popcount(x AND w)
//   output  = fma_fp16( (fp16)(int16)sum, scale[oc], bias[oc] ), fp16 NCHWc8
//
// Three kernels: binarise + zero-pad the fp16 NCHWc8 input into [N][Hp][Wp][C/32] words (one
// streaming pass, 16x smaller than the input), repack the filter bits into [OC][tap][C/32] words
// (once), and the convolution: a CTA owns 128 output pixels x 64 output channels, keeps its weight
// slice in shared memory (read as 128-bit broadcasts), each thread one pixel with 64 integer
// accumulators in registers; XOR/AND + __popc on 32 channels at a time; fp16 fused multiply-add
// epilogue, 16-byte stores.  The work is bound by the popcount rate (16 per clock per SM), not by
// HBM: 3x3, C = 256 needs 72 word-operations per output, the bytes are 50x less than that.
#include <cuda_fp16.h>

#include <cstring>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int PIX_TILE = 128;
constexpr int OC_TILE = 64;

struct B4d {
    DataType dt;
    DataFormat df;
    uint32_t n, c, h, w;
};
bool get4(const TensorDesc *d, B4d *o)
{
    if (d == nullptr || d->nDims != 4) {
        return false;
    }
    o->dt = d->dt;
    o->df = d->df;
    o->w = d->dims[0];
    o->h = d->dims[1];
    o->c = d->dims[2];
    o->n = d->dims[3];
    return true;
}

// filter bits NCHW, MSB first in each byte (cpu/general/convolution.cpp:161-179) -> words [OC][tap][Cw],
// bit (c % 32) of word c / 32
__global__ void bnn_pack_filter_kernel(const uint8_t *__restrict__ src, uint32_t OC, uint32_t IC, uint32_t taps,
    uint32_t Cw, uint32_t *__restrict__ dst)
{
    const size_t total = (size_t)OC * taps * Cw;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t cw = (uint32_t)(i % Cw);
        const uint32_t tap = (uint32_t)((i / Cw) % taps);
        const uint32_t oc = (uint32_t)(i / ((size_t)Cw * taps));
        uint32_t word = 0;
        for (uint32_t b = 0; b < 32; ++b) {
            const uint32_t c = cw * 32 + b;
            if (c < IC) {
                const size_t pos = ((size_t)oc * IC + c) * taps + tap;
                word |= (uint32_t)((src[pos >> 3] >> (7 - (pos & 7))) & 1u) << b;
            }
        }
        dst[i] = word;
    }
}

// fp16 NCHWc8 -> bit words [N][Hp][Wp][Cw], zero words in the padding ring
__global__ void bnn_binarize_pad_kernel(const __half *__restrict__ in, uint32_t N, uint32_t IC, uint32_t IH, uint32_t IW,
    uint32_t Hp, uint32_t Wp, uint32_t pt, uint32_t pl, uint32_t Cw, float threshold, uint32_t *__restrict__ out)
{
    const size_t total = (size_t)N * Hp * Wp * Cw;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t cw = (uint32_t)(i % Cw);
        const uint32_t x = (uint32_t)((i / Cw) % Wp);
        const uint32_t y = (uint32_t)((i / ((size_t)Cw * Wp)) % Hp);
        const uint32_t n = (uint32_t)(i / ((size_t)Cw * Wp * Hp));
        uint32_t word = 0;
        const int iy = (int)y - (int)pt, ix = (int)x - (int)pl;
        if (iy >= 0 && iy < (int)IH && ix >= 0 && ix < (int)IW) {
            const size_t pix = (size_t)iy * IW + ix;
#pragma unroll
            for (uint32_t blk = 0; blk < 4; ++blk) {
                const uint32_t c0 = cw * 32 + blk * 8;
                if (c0 < IC) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(
                        in + ((size_t)n * IC + c0) * IH * IW + pix * 8);
                    const uint32_t h[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float lo = __half2float(__ushort_as_half((unsigned short)(h[j] & 0xFFFFu)));
                        const float hi = __half2float(__ushort_as_half((unsigned short)(h[j] >> 16)));
                        word |= (lo >= threshold ? 1u : 0u) << (blk * 8 + 2 * j);
                        word |= (hi >= threshold ? 1u : 0u) << (blk * 8 + 2 * j + 1);
                    }
                }
            }
        }
        out[i] = word;
    }
}

struct BnnParams {
    uint32_t N, OH, OW, OC, Hp, Wp, Cw, FH, FW, sH, sW;
    uint32_t kbits;  // fh * fw * ic
    int xnor;
    const uint32_t *xb;
    const uint32_t *wb;
    const __half *scale;
    const __half *bias;
    __half *out;
};

template <bool XNOR>
__global__ void __launch_bounds__(PIX_TILE)
bnn_conv_kernel(const BnnParams p)
{
    extern __shared__ __align__(16) uint32_t sw[];  // [OC_TILE][taps * Cw] padded to a multiple of 4 words
    const uint32_t taps = p.FH * p.FW;
    const uint32_t kw_words = taps * p.Cw;
    const uint32_t kw_pad = (kw_words + 3) & ~3u;
    const uint32_t oc0 = blockIdx.y * OC_TILE;
    for (uint32_t i = threadIdx.x; i < OC_TILE * kw_pad; i += blockDim.x) {
        const uint32_t o = i / kw_pad, k = i - o * kw_pad;
        sw[i] = (oc0 + o < p.OC && k < kw_words) ? p.wb[(size_t)(oc0 + o) * kw_words + k] : 0u;
    }
    __syncthreads();
    const size_t npix = (size_t)p.N * p.OH * p.OW;
    const size_t pidx = (size_t)blockIdx.x * PIX_TILE + threadIdx.x;
    if (pidx >= npix) {
        return;
    }
    const uint32_t ow = (uint32_t)(pidx % p.OW);
    const uint32_t oh = (uint32_t)((pidx / p.OW) % p.OH);
    const uint32_t n = (uint32_t)(pidx / ((size_t)p.OW * p.OH));
    int acc[OC_TILE];
#pragma unroll
    for (int o = 0; o < OC_TILE; ++o) {
        acc[o] = 0;
    }
    // walk K four words at a time: one 128-bit broadcast read of the weights per output channel
    for (uint32_t k4 = 0; k4 < kw_pad; k4 += 4) {
        uint32_t x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t k = k4 + j;
            uint32_t v = 0;
            if (k < kw_words) {
                const uint32_t tap = k / p.Cw, cw = k - tap * p.Cw;
                const uint32_t kh = tap / p.FW, kw = tap - kh * p.FW;
                v = __ldg(p.xb + (((size_t)n * p.Hp + oh * p.sH + kh) * p.Wp + ow * p.sW + kw) * p.Cw + cw);
            }
            x[j] = v;
        }
#pragma unroll
        for (int o = 0; o < OC_TILE; ++o) {
            const uint4 w = *reinterpret_cast<const uint4 *>(sw + o * kw_pad + k4);
            if (XNOR) {
                acc[o] += __popc(x[0] ^ w.x) + __popc(x[1] ^ w.y) + __popc(x[2] ^ w.z) + __popc(x[3] ^ w.w);
            } else {
                acc[o] += __popc(x[0] & w.x) + __popc(x[1] & w.y) + __popc(x[2] & w.z) + __popc(x[3] & w.w);
            }
        }
    }
    // epilogue: int16 sum -> fp16 (round to nearest even), one fused multiply-add, 8 channels = 16 bytes
    const size_t plane = (size_t)p.OH * p.OW;
    const size_t pix = (size_t)oh * p.OW + ow;
#pragma unroll
    for (int ob = 0; ob < OC_TILE; ob += 8) {
        const uint32_t oc = oc0 + ob;
        if (oc >= p.OC) {
            break;
        }
        unsigned short h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int s = XNOR ? ((int)p.kbits - 2 * acc[ob + j]) : acc[ob + j];
            const __half hs = __short2half_rn((short)s);
            __half r = hs;
            if (oc + j < p.OC) {
                r = __hfma(hs, p.scale[oc + j], p.bias[oc + j]);
            }
            h[j] = __half_as_ushort(r);
        }
        const uint32_t width = min(8u, p.OC - oc);
        __half *dst = p.out + ((size_t)n * p.OC + oc) * plane + pix * width;
        if (width == 8) {
            *reinterpret_cast<uint4 *>(dst) = make_uint4(h[0] | ((uint32_t)h[1] << 16), h[2] | ((uint32_t)h[3] << 16),
                h[4] | ((uint32_t)h[5] << 16), h[6] | ((uint32_t)h[7] << 16));
        } else {
            for (uint32_t j = 0; j < width; ++j) {
                dst[j] = __ushort_as_half(h[j]);
            }
        }
    }
}

struct BnnGeom {
    B4d in, f, out;
    uint32_t sH, sW, pt, pb, pl, pr, Hp, Wp, Cw, taps;
    size_t xb_bytes;
};

EE bnn_geometry(const TensorDesc *inputDesc, const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *cp, BnnGeom *g)
{
    if (!get4(inputDesc, &g->in) || !get4(filterDesc, &g->f) || !get4(outputDesc, &g->out) || cp == nullptr) {
        return NOT_MATCH;
    }
    if (cp->group > 1 || cp->dilatedRate_h > 1 || cp->dilatedRate_w > 1) {
        return NOT_SUPPORTED;
    }
    g->sH = cp->stride_h ? cp->stride_h : 1;
    g->sW = cp->stride_w ? cp->stride_w : 1;
    g->pt = cp->pad_top;
    g->pb = cp->pad_bottom;
    g->pl = cp->pad_left;
    g->pr = cp->pad_right;
    g->Hp = g->in.h + g->pt + g->pb;
    g->Wp = g->in.w + g->pl + g->pr;
    g->Cw = (g->f.c + 31) / 32;
    g->taps = g->f.h * g->f.w;
    g->xb_bytes = (size_t)g->in.n * g->Hp * g->Wp * g->Cw * 4;
    // the output geometry must be the one the input, filter and padding give: the kernel reads the padded
    // bit tensor at (oh * stride + kh, ow * stride + kw) without further checks
    if (g->f.h == 0 || g->f.w == 0 || g->Hp < g->f.h || g->Wp < g->f.w || g->out.n != g->in.n ||
        g->out.h != (g->Hp - g->f.h) / g->sH + 1 || g->out.w != (g->Wp - g->f.w) / g->sW + 1) {
        return NOT_MATCH;
    }
    return SUCCESS;
}

}  // namespace

EE bnn_transform_filter_bytes(const TensorDesc *filterDesc, U32 *bytes)
{
    B4d f;
    if (!get4(filterDesc, &f) || bytes == nullptr) {
        return NOT_MATCH;
    }
    *bytes = f.n * f.h * f.w * ((f.c + 31) / 32) * 4 + 32;
    return SUCCESS;
}

EE bnn_transform_filter(const TensorDesc *filterDesc, const void *filter, TensorDesc *ftmDesc, void *dst)
{
    B4d f;
    if (!get4(filterDesc, &f) || ftmDesc == nullptr) {
        return NOT_MATCH;
    }
    if (f.df == DF_NCHWN16C8) {
        *ftmDesc = *filterDesc;  // already transformed (convolution_transform_bnn.h:47-50)
        return SUCCESS;
    }
    if (f.df != DF_NCHW) {
        return NOT_MATCH;
    }
    if (filter == nullptr || dst == nullptr) {
        return NULL_POINTER;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    cudaStream_t st = tls().stream;
    const uint32_t Cw = (f.c + 31) / 32, taps = f.h * f.w;
    const size_t words = (size_t)f.n * taps * Cw;
    Stage sg;
    const uint8_t *d_src = reinterpret_cast<const uint8_t *>(sg.in(filter, ((size_t)f.n * f.c * taps + 7) / 8));
    uint32_t *d_dst = reinterpret_cast<uint32_t *>(sg.out(dst, words * 4));
    if (d_src == nullptr || d_dst == nullptr) {
        return ALLOC_FAILED;
    }
    bnn_pack_filter_kernel<<<(uint32_t)((words + 255) / 256), 256, 0, st>>>(d_src, f.n, f.c, taps, Cw, d_dst);
    count_launch();
    B200_CUDA(cudaGetLastError());
    *ftmDesc = *filterDesc;
    ftmDesc->df = DF_NCHWN16C8;
    return sg.finish();
}

EE bnn_tmp_bytes(const TensorDesc *inputDesc, const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *cp, U32 *bytes)
{
    if (bytes == nullptr) {
        return NULL_POINTER;
    }
    BnnGeom g;
    B200_EE(bnn_geometry(inputDesc, filterDesc, outputDesc, cp, &g));
    const size_t b = g.xb_bytes + 512;
    if (b > 0xFFFFFFFFull) {
        return NOT_SUPPORTED;
    }
    *bytes = (U32)b;
    return SUCCESS;
}

EE bnn_run(const TensorDesc *inputDesc, const void *input, const TensorDesc *filterDesc, const void *filter,
    const ConvolutionParamSpec *cp, const void *scale, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output)
{
    BnnGeom g;
    B200_EE(bnn_geometry(inputDesc, filterDesc, outputDesc, cp, &g));
    if (input == nullptr || filter == nullptr || output == nullptr || scale == nullptr || bias == nullptr ||
        tmp == nullptr) {
        return NULL_POINTER;  // cpu/arm/bnn/convolution.cpp:32-35
    }
    if (g.in.dt != DT_F16 || g.out.dt != DT_F16) {
        return NOT_MATCH;  // :46-51
    }
    if (g.in.df != DF_NCHWC8 || g.out.df != DF_NCHWC8 || g.f.df != DF_NCHWN16C8) {
        return NOT_MATCH;  // :52-54, convolution_xnor_A76.cpp:53-55
    }
    if (g.in.c != g.f.c || g.out.c != g.f.n || (g.in.c % 8) != 0 || (g.out.c % 8) != 0) {
        return NOT_MATCH;
    }
    U32 need = 0;
    B200_EE(bnn_tmp_bytes(inputDesc, filterDesc, outputDesc, cp, &need));
    if (tmpBytes < need) {
        return NOT_MATCH;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    cudaStream_t st = tls().stream;
    const bool xnor = g.f.dt == DT_BIN11;
    const size_t in_elems = (size_t)g.in.n * g.in.c * g.in.h * g.in.w;
    const size_t out_elems = (size_t)g.out.n * g.out.c * g.out.h * g.out.w;
    const size_t w_words = (size_t)g.f.n * g.taps * g.Cw;
    Stage sg;
    const __half *d_in = reinterpret_cast<const __half *>(sg.in(input, in_elems * 2));
    const uint32_t *d_w = reinterpret_cast<const uint32_t *>(sg.in(filter, w_words * 4));
    const __half *d_scale = reinterpret_cast<const __half *>(sg.in(scale, (size_t)g.out.c * 2));
    const __half *d_bias = reinterpret_cast<const __half *>(sg.in(bias, (size_t)g.out.c * 2));
    __half *d_out = reinterpret_cast<__half *>(sg.out(output, out_elems * 2));
    char *d_tmp = is_device_ptr(tmp) ? reinterpret_cast<char *>(tmp) : reinterpret_cast<char *>(sg.scratch(need));
    if (d_in == nullptr || d_w == nullptr || d_scale == nullptr || d_bias == nullptr || d_out == nullptr ||
        d_tmp == nullptr) {
        return ALLOC_FAILED;
    }
    uint32_t *d_xb = reinterpret_cast<uint32_t *>(B200_ALIGN(reinterpret_cast<uintptr_t>(d_tmp), 256));
    {
        const size_t words = g.xb_bytes / 4;
        size_t blocks = (words + 255) / 256;
        if (blocks > (size_t)c->sm_count * 16) {
            blocks = (size_t)c->sm_count * 16;
        }
        bnn_binarize_pad_kernel<<<(uint32_t)blocks, 256, 0, st>>>(d_in, g.in.n, g.in.c, g.in.h, g.in.w, g.Hp, g.Wp, g.pt,
            g.pl, g.Cw, xnor ? 0.0f : 0.5f, d_xb);
        count_launch();
    }
    BnnParams p;
    p.N = g.in.n;
    p.OH = g.out.h;
    p.OW = g.out.w;
    p.OC = g.out.c;
    p.Hp = g.Hp;
    p.Wp = g.Wp;
    p.Cw = g.Cw;
    p.FH = g.f.h;
    p.FW = g.f.w;
    p.sH = g.sH;
    p.sW = g.sW;
    p.kbits = g.f.h * g.f.w * g.f.c;
    p.xnor = xnor ? 1 : 0;
    p.xb = d_xb;
    p.wb = d_w;
    p.scale = d_scale;
    p.bias = d_bias;
    p.out = d_out;
    const uint32_t kw_pad = (g.taps * g.Cw + 3) & ~3u;
    const size_t smem = (size_t)OC_TILE * kw_pad * 4;
    if (smem > 200 * 1024) {
        return NOT_SUPPORTED;
    }
    {
        const void *ks[2] = {(const void *)bnn_conv_kernel<true>, (const void *)bnn_conv_kernel<false>};
        B200_EE(raise_smem_limit(c, KF_BNN, ks, 2, 200 * 1024));
    }
    const size_t npix = (size_t)g.out.n * g.out.h * g.out.w;
    dim3 grid((uint32_t)((npix + PIX_TILE - 1) / PIX_TILE), (g.out.c + OC_TILE - 1) / OC_TILE);
    if (xnor) {
        bnn_conv_kernel<true><<<grid, PIX_TILE, smem, st>>>(p);
    } else {
        bnn_conv_kernel<false><<<grid, PIX_TILE, smem, st>>>(p);
    }
    count_launch();
    B200_CUDA(cudaGetLastError());
    return sg.finish();
}

}  // namespace b200
