// pooling.cu -- u8 pooling on channels-of-16 tensors, the int8 branch of Bolt's pooling operator
// (compute/tensor/src/cpu/x86/int8/avx512/pooling_int8.cpp:317-429, reached from cpu/x86/pooling.cpp:50-55).
//
// HBM bound: every input byte is read once (overlapping windows hit L1/L2), every output byte written once.
// One thread per output pixel and 16-channel block: 16-byte loads, byte-wise maximum with vmaxu4, or four
// 32-bit sums per word for the mean.  The mean keeps the reference's integer arithmetic: the window sum minus
// 128 per element, times 65536 / (window size) as a 32-bit product, LOGICAL shift right by 16, plus 128,
// unsigned saturation -- so a window whose values lie below the zero point stores 255, as the reference does.
#include "common.cuh"

namespace b200 {
namespace {

struct PoolGeom {
    uint32_t planes;   // N * C/16
    uint32_t ih, iw, oh, ow, kh, kw, sh, sw, pt, pl;
    int mean, count_include_pad;
    int32_t factor;    // 65536 / (KH * KW)
};

__device__ __forceinline__ uint32_t mean_byte(int32_t acc, int32_t pool)
{
    const uint32_t v = (((uint32_t)acc * (uint32_t)pool) >> 16) + 128u;
    return v > 255u ? 255u : v;
}

// Windows of at most K x K taps (K = 2, 3): every tap is loaded before the first is used, so a thread has up
// to nine 16-byte requests in flight; taps outside the clipped window repeat the first tap (maximum) or count
// zero (mean).
template <int K>
__global__ void __launch_bounds__(256) pooling_u8_c16_small_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, PoolGeom g)
{
    const uint64_t total = (uint64_t)g.planes * g.oh * g.ow;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t w = (uint32_t)(i % g.ow);
        const uint64_t r = i / g.ow;
        const uint32_t h = (uint32_t)(r % g.oh);
        const uint64_t plane = r / g.oh;
        int hs = (int)(h * g.sh) - (int)g.pt, ws = (int)(w * g.sw) - (int)g.pl;
        const int he = min(hs + (int)g.kh, (int)g.ih), we = min(ws + (int)g.kw, (int)g.iw);
        hs = max(hs, 0);
        ws = max(ws, 0);
        const uint4 *src = reinterpret_cast<const uint4 *>(in + plane * g.ih * g.iw * 16);
        uint4 v[K * K];
#pragma unroll
        for (int dy = 0; dy < K; ++dy) {
#pragma unroll
            for (int dx = 0; dx < K; ++dx) {
                const bool inside = hs + dy < he && ws + dx < we;
                const int y = inside ? hs + dy : hs, x = inside ? ws + dx : ws;
                v[dy * K + dx] = __ldg(src + (size_t)y * g.iw + x);
                if (g.mean && !inside) {
                    v[dy * K + dx] = make_uint4(0, 0, 0, 0);
                }
            }
        }
        uint4 res;
        if (!g.mean) {
            uint4 m = v[0];
#pragma unroll
            for (int t = 1; t < K * K; ++t) {
                m.x = __vmaxu4(m.x, v[t].x);
                m.y = __vmaxu4(m.y, v[t].y);
                m.z = __vmaxu4(m.z, v[t].z);
                m.w = __vmaxu4(m.w, v[t].w);
            }
            res = m;
        } else {
            const int n = (he - hs) * (we - ws);
            const int32_t pool = g.count_include_pad ? g.factor : 65536 / n;
            uint32_t q[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int32_t acc[4] = {-128 * n, -128 * n, -128 * n, -128 * n};
#pragma unroll
                for (int t = 0; t < K * K; ++t) {
                    const uint32_t word = k == 0 ? v[t].x : (k == 1 ? v[t].y : (k == 2 ? v[t].z : v[t].w));
                    acc[0] += (int32_t)(word & 0xFFu);
                    acc[1] += (int32_t)((word >> 8) & 0xFFu);
                    acc[2] += (int32_t)((word >> 16) & 0xFFu);
                    acc[3] += (int32_t)(word >> 24);
                }
                q[k] = mean_byte(acc[0], pool) | (mean_byte(acc[1], pool) << 8) | (mean_byte(acc[2], pool) << 16) |
                    (mean_byte(acc[3], pool) << 24);
            }
            res = make_uint4(q[0], q[1], q[2], q[3]);
        }
        reinterpret_cast<uint4 *>(out)[i] = res;
    }
}

__global__ void __launch_bounds__(256) pooling_u8_c16_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, PoolGeom g)
{
    const uint64_t total = (uint64_t)g.planes * g.oh * g.ow;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t w = (uint32_t)(i % g.ow);
        const uint64_t r = i / g.ow;
        const uint32_t h = (uint32_t)(r % g.oh);
        const uint64_t plane = r / g.oh;
        int hs = (int)(h * g.sh) - (int)g.pt, ws = (int)(w * g.sw) - (int)g.pl;
        const int he = min(hs + (int)g.kh, (int)g.ih), we = min(ws + (int)g.kw, (int)g.iw);
        hs = max(hs, 0);
        ws = max(ws, 0);
        const uint4 *src = reinterpret_cast<const uint4 *>(in + plane * g.ih * g.iw * 16);
        uint4 res;
        if (!g.mean) {
            uint4 m = __ldg(src + (size_t)hs * g.iw + ws);
            for (int y = hs; y < he; ++y) {
                for (int x = ws; x < we; ++x) {
                    const uint4 v = __ldg(src + (size_t)y * g.iw + x);
                    m.x = __vmaxu4(m.x, v.x);
                    m.y = __vmaxu4(m.y, v.y);
                    m.z = __vmaxu4(m.z, v.z);
                    m.w = __vmaxu4(m.w, v.w);
                }
            }
            res = m;
        } else {
            const int n = (he - hs) * (we - ws);
            int32_t acc[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                acc[c] = -128 * n;
            }
            for (int y = hs; y < he; ++y) {
                for (int x = ws; x < we; ++x) {
                    const uint4 v = __ldg(src + (size_t)y * g.iw + x);
                    const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        acc[c] += (int32_t)((q[c >> 2] >> (8 * (c & 3))) & 0xFFu);
                    }
                }
            }
            const int32_t pool = g.count_include_pad ? g.factor : 65536 / n;
            uint32_t q[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                q[k] = mean_byte(acc[4 * k], pool) | (mean_byte(acc[4 * k + 1], pool) << 8) |
                    (mean_byte(acc[4 * k + 2], pool) << 16) | (mean_byte(acc[4 * k + 3], pool) << 24);
            }
            res = make_uint4(q[0], q[1], q[2], q[3]);
        }
        reinterpret_cast<uint4 *>(out)[i] = res;
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" EE pooling_cuda_b200(const TensorDesc *inputDesc, const void *input, const PoolingParamSpec *p, void *scale,
    const TensorDesc *outputDesc, void *output)
{
    if (inputDesc == nullptr || outputDesc == nullptr || p == nullptr) {
        return NULL_POINTER;
    }
    if (input == nullptr || output == nullptr) {
        return NULL_POINTER;  // pooling_int8.cpp:324-326
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (inputDesc->nDims != 4 || outputDesc->nDims != 4) {
        return NOT_MATCH;
    }
    const uint32_t iw = inputDesc->dims[0], ih = inputDesc->dims[1], ic = inputDesc->dims[2], in = inputDesc->dims[3];
    const uint32_t ow = outputDesc->dims[0], oh = outputDesc->dims[1], oc = outputDesc->dims[2], on = outputDesc->dims[3];
    if (inputDesc->dt != DT_U8_Q || outputDesc->dt != DT_U8_Q || in != on || ic != oc || inputDesc->df != DF_NCHWC16 ||
        outputDesc->df != DF_NCHWC16 || ic % 16 != 0) {
        return NOT_MATCH;  // :333-341,357-359
    }
    if (p->pad_top >= p->kernel_h || p->pad_left >= p->kernel_w) {
        return NOT_SUPPORTED;  // :352-354
    }
    if (p->kernel_h == 0 || p->kernel_w == 0 || p->stride_h == 0 || p->stride_w == 0) {
        return NOT_MATCH;
    }
    const int32_t factor = 65536 / (int32_t)(p->kernel_h * p->kernel_w);
    if (factor < 1 || (p->mode != POOLING_MAX && p->mode != POOLING_MEAN)) {
        return NOT_SUPPORTED;  // :364-366,417-418
    }
    const uint64_t total = (uint64_t)in * (ic / 16) * oh * ow;
    if (total == 0) {
        return SUCCESS;
    }
    // every output window has to start inside the image (the reference divides by the clipped window size)
    if ((uint64_t)(oh - 1) * p->stride_h >= (uint64_t)ih + p->pad_top || (uint64_t)(ow - 1) * p->stride_w >= (uint64_t)iw + p->pad_left) {
        return NOT_MATCH;
    }
    if (scale != nullptr) {
        F32 *s = reinterpret_cast<F32 *>(scale);
        s[1] = (p->mode == POOLING_MAX) ? s[0] : s[0] * factor * (p->kernel_w * p->kernel_h) / (F32)65536;  // :367-371
    }
    PoolGeom g;
    g.planes = in * (ic / 16);
    g.ih = ih;
    g.iw = iw;
    g.oh = oh;
    g.ow = ow;
    g.kh = p->kernel_h;
    g.kw = p->kernel_w;
    g.sh = p->stride_h;
    g.sw = p->stride_w;
    g.pt = p->pad_top;
    g.pl = p->pad_left;
    g.mean = p->mode == POOLING_MEAN;
    g.count_include_pad = p->count_include_pad ? 1 : 0;
    g.factor = factor;
    Stage sg;
    const uint8_t *d_in = reinterpret_cast<const uint8_t *>(sg.in(input, (size_t)in * ic * ih * iw));
    uint8_t *d_out = reinterpret_cast<uint8_t *>(sg.out(output, (size_t)total * 16));
    if (d_in == nullptr || d_out == nullptr) {
        return ALLOC_FAILED;
    }
    if (on_other_device(d_in) || on_other_device(d_out)) {
        return NOT_MATCH;
    }
    const uint64_t blocks = (total + 255) / 256;
    const uint32_t grid = (uint32_t)(blocks < (uint64_t)c->sm_count * 32 ? blocks : (uint64_t)c->sm_count * 32);
    if (g.kh <= 2 && g.kw <= 2) {
        pooling_u8_c16_small_kernel<2><<<grid, 256, 0, tls().stream>>>(d_in, d_out, g);
    } else if (g.kh <= 3 && g.kw <= 3) {
        pooling_u8_c16_small_kernel<3><<<grid, 256, 0, tls().stream>>>(d_in, d_out, g);
    } else {
        pooling_u8_c16_kernel<<<grid, 256, 0, tls().stream>>>(d_in, d_out, g);
    }
    count_launch();
    B200_CUDA(cudaGetLastError());
    return sg.finish();
}
