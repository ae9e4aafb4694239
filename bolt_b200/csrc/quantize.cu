// quantize.cu -- dynamic-range scale finding, quantize, requantize, dequantize.
//
// Replaces compute/tensor/src/cpu/x86/int8/avx512/quantize.cpp:21-416 and dequantize.cpp:18-101.
// All kernels are one or two streaming passes: 128-bit loads and stores, grid sized to the SM
// count, warp-shuffle + one atomic per warp for the absmax reduction.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int TPB = 256;

inline uint32_t grid_for(uint64_t n_vec, int sms)
{
    uint64_t blocks = (n_vec + TPB - 1) / TPB;
    const uint64_t cap = (uint64_t)sms * 16;
    if (blocks > cap) {
        blocks = cap;
    }
    return (uint32_t)(blocks ? blocks : 1);
}

// max |x| as raw float bits (non-negative floats order like unsigned integers)
__global__ void absmax_f32_kernel(const float *__restrict__ x, uint64_t n, unsigned *out_bits)
{
    unsigned m = 0;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    uint64_t n4 = aligned ? n / 4 : 0;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    uint64_t i = tid;
    for (; i + 3 * stride < n4; i += 4 * stride) {  // four independent 128-bit loads in flight per thread
        const float4 a = x4[i], b = x4[i + stride], c = x4[i + 2 * stride], d = x4[i + 3 * stride];
        const unsigned ma = max(max(__float_as_uint(a.x) & 0x7FFFFFFFu, __float_as_uint(a.y) & 0x7FFFFFFFu),
            max(__float_as_uint(a.z) & 0x7FFFFFFFu, __float_as_uint(a.w) & 0x7FFFFFFFu));
        const unsigned mb = max(max(__float_as_uint(b.x) & 0x7FFFFFFFu, __float_as_uint(b.y) & 0x7FFFFFFFu),
            max(__float_as_uint(b.z) & 0x7FFFFFFFu, __float_as_uint(b.w) & 0x7FFFFFFFu));
        const unsigned mc = max(max(__float_as_uint(c.x) & 0x7FFFFFFFu, __float_as_uint(c.y) & 0x7FFFFFFFu),
            max(__float_as_uint(c.z) & 0x7FFFFFFFu, __float_as_uint(c.w) & 0x7FFFFFFFu));
        const unsigned md = max(max(__float_as_uint(d.x) & 0x7FFFFFFFu, __float_as_uint(d.y) & 0x7FFFFFFFu),
            max(__float_as_uint(d.z) & 0x7FFFFFFFu, __float_as_uint(d.w) & 0x7FFFFFFFu));
        m = max(m, max(max(ma, mb), max(mc, md)));
    }
    for (; i < n4; i += stride) {
        const float4 v = x4[i];
        m = max(m, __float_as_uint(v.x) & 0x7FFFFFFFu);
        m = max(m, __float_as_uint(v.y) & 0x7FFFFFFFu);
        m = max(m, __float_as_uint(v.z) & 0x7FFFFFFFu);
        m = max(m, __float_as_uint(v.w) & 0x7FFFFFFFu);
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) {
        m = max(m, __float_as_uint(x[i]) & 0x7FFFFFFFu);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    // one atomic per CTA: thousands of warps hitting one address serialise in L2
    __shared__ unsigned warp_max[TPB / 32];
    if ((threadIdx.x & 31) == 0) {
        warp_max[threadIdx.x >> 5] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < TPB / 32; ++w) {
            m = max(m, warp_max[w]);
        }
        if (m != 0) {
            atomicMax(out_bits, m);
        }
    }
}

// vpabsd + vpmaxsd (quantize.cpp:70-108): |INT_MIN| stays negative and never wins
__global__ void absmax_i32_kernel(const int32_t *__restrict__ x, uint64_t n, int *out)
{
    int m = 0;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    uint64_t n4 = aligned ? n / 4 : 0;
    const int4 *x4 = reinterpret_cast<const int4 *>(x);
    for (uint64_t i = tid; i < n4; i += stride) {
        const int4 v = x4[i];
        m = max(m, (int)(v.x < 0 ? 0u - (unsigned)v.x : (unsigned)v.x));
        m = max(m, (int)(v.y < 0 ? 0u - (unsigned)v.y : (unsigned)v.y));
        m = max(m, (int)(v.z < 0 ? 0u - (unsigned)v.z : (unsigned)v.z));
        m = max(m, (int)(v.w < 0 ? 0u - (unsigned)v.w : (unsigned)v.w));
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) {
        const int v = x[i];
        m = max(m, (int)(v < 0 ? 0u - (unsigned)v : (unsigned)v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    __shared__ int warp_max[TPB / 32];
    if ((threadIdx.x & 31) == 0) {
        warp_max[threadIdx.x >> 5] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < TPB / 32; ++w) {
            m = max(m, warp_max[w]);
        }
        if (m != 0) {
            atomicMax(out, m);
        }
    }
}

// 127 / absmax on the device (quantize.cpp:63-67), for pipelines that never leave the stream
__global__ void finalize_scale_kernel(const unsigned *bits, float *scale)
{
    const float mx = __uint_as_float(*bits);
    *scale = (mx == 0.f) ? 1.0f : __fdiv_rn(127.0f, mx);
}

// ---- element functions ------------------------------------------------------------------------
struct F32ToU8 {  // quantize.cpp:135-178: vmulps, vaddps 128, vcvtps2dq{rn}, max 1, min 255
    float s;
    __device__ uint32_t operator()(float x) const
    {
        const int r = cvt_rne_x86(__fadd_rn(__fmul_rn(x, s), 128.0f));
        return (uint32_t)min(255, max(1, r));
    }
};
struct F32ToI8 {  // quantize.cpp:195-233: vmulps, vcvtps2dq, max -127, min 127
    float s;
    __device__ uint32_t operator()(float x) const
    {
        const int r = cvt_rne_x86(__fmul_rn(x, s));
        return (uint32_t)(min(127, max(-127, r)) & 0xFF);
    }
};
struct I32ToU8 {  // quantize.cpp:377-414: vcvtdq2ps, vmulps, vaddps 128, vcvtps2dq, vpmovusdb
    float s;
    __device__ uint32_t operator()(int x) const
    {
        return usat8_x86(cvt_rne_x86(__fadd_rn(__fmul_rn(__int2float_rn(x), s), 128.0f)));
    }
};
struct I32ToI8 {  // quantize.cpp:328-359: vcvtdq2ps, vmulps, vcvtps2dq, vpmovsdb
    float s;
    __device__ uint32_t operator()(int x) const
    {
        return (uint32_t)(ssat8_x86(cvt_rne_x86(__fmul_rn(__int2float_rn(x), s))) & 0xFF);
    }
};

struct F32ToU8Dev {  // same arithmetic, scale read from device memory
    const float *s;
    __device__ uint32_t operator()(float x) const
    {
        const int r = cvt_rne_x86(__fadd_rn(__fmul_rn(x, *s), 128.0f));
        return (uint32_t)min(255, max(1, r));
    }
};

// 32-bit source -> 8-bit destination, 16 elements per thread step
template <typename SrcT, typename Op>
__global__ void to8_kernel(const SrcT *__restrict__ x, uint64_t n, uint8_t *__restrict__ q, Op op)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) == 0;
    const uint64_t n16 = aligned ? n / 16 : 0;
    struct alignas(16) V4 {
        SrcT a, b, c, d;
    };
    const V4 *xv = reinterpret_cast<const V4 *>(x);
    for (uint64_t i = tid; i < n16; i += stride) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const V4 v = xv[i * 4 + j];
            w[j] = op(v.a) | (op(v.b) << 8) | (op(v.c) << 16) | (op(v.d) << 24);
        }
        reinterpret_cast<uint4 *>(q)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (uint64_t i = n16 * 16 + tid; i < n; i += stride) {
        q[i] = (uint8_t)op(x[i]);
    }
}

// quantize.cpp:271-313: byte-wise + 0x80
__global__ void u8_to_i8_kernel(const uint8_t *__restrict__ x, uint64_t n, uint8_t *__restrict__ q)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) == 0;
    const uint64_t n16 = aligned ? n / 16 : 0;
    for (uint64_t i = tid; i < n16; i += stride) {
        uint4 v = reinterpret_cast<const uint4 *>(x)[i];
        v.x ^= 0x80808080u;
        v.y ^= 0x80808080u;
        v.z ^= 0x80808080u;
        v.w ^= 0x80808080u;
        reinterpret_cast<uint4 *>(q)[i] = v;
    }
    for (uint64_t i = n16 * 16 + tid; i < n; i += stride) {
        q[i] = x[i] ^ 0x80u;
    }
}

// dequantize.cpp:18-52: (float)q * (1/scale)
__global__ void dequant_i32_kernel(const int32_t *__restrict__ q, uint64_t n, float factor, float *__restrict__ out)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const uint64_t n4 = aligned ? n / 4 : 0;
    for (uint64_t i = tid; i < n4; i += stride) {
        const int4 v = reinterpret_cast<const int4 *>(q)[i];
        reinterpret_cast<float4 *>(out)[i] = make_float4(acc_to_f32(v.x, factor), acc_to_f32(v.y, factor),
            acc_to_f32(v.z, factor), acc_to_f32(v.w, factor));
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) {
        out[i] = acc_to_f32(q[i], factor);
    }
}

// dequantize.cpp:54-101: (float)((int)q - 128) * (1.0f/scale)
__global__ void dequant_u8_kernel(const uint8_t *__restrict__ q, uint64_t n, float factor, float *__restrict__ out)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const uint64_t n16 = aligned ? n / 16 : 0;
    for (uint64_t i = tid; i < n16; i += stride) {
        const uint4 v = reinterpret_cast<const uint4 *>(q)[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            reinterpret_cast<float4 *>(out)[i * 4 + j] =
                make_float4(acc_to_f32((int)(w[j] & 0xFF) - 128, factor), acc_to_f32((int)((w[j] >> 8) & 0xFF) - 128, factor),
                    acc_to_f32((int)((w[j] >> 16) & 0xFF) - 128, factor), acc_to_f32((int)(w[j] >> 24) - 128, factor));
        }
    }
    for (uint64_t i = n16 * 16 + tid; i < n; i += stride) {
        out[i] = acc_to_f32((int)q[i] - 128, factor);
    }
}

// quantize.cpp:236-269: round() = half away from zero on the fp32 product
__global__ void bias_offsetc_kernel(const float *bias, const int32_t *offsetC, uint32_t n, float scale, int32_t *out)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        int b = 0;
        if (bias != nullptr) {
            b = (int)roundf(__fmul_rn(bias[i], scale));
        }
        out[i] = b + (offsetC ? offsetC[i] : 0);
    }
}
__global__ void bias_i32_offsetc_kernel(const int32_t *bias, const int32_t *offsetC, uint32_t n, int32_t *out)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = bias[i] + (offsetC ? offsetC[i] : 0);
    }
}

uint64_t desc_elems(const TensorDesc *d)
{
    if (d->nDims == 0) {
        return 0;
    }
    uint64_t n = 1;
    for (uint32_t i = 0; i < d->nDims && i < 20; ++i) {
        n *= d->dims[i];
    }
    return n;
}

// absmax of device data, result to host
EE absmax_f32_host(const float *d_x, uint64_t n, float *mx)
{
    DeviceCtx *c = ctx();
    cudaStream_t st = tls().stream;
    std::lock_guard<std::mutex> g(c->scratch_mu);
    B200_CUDA(cudaMemsetAsync(c->d_scratch_u, 0, 4, st));
    if (n > 0) {
        absmax_f32_kernel<<<grid_for((n + 3) / 4, c->sm_count), TPB, 0, st>>>(d_x, n, c->d_scratch_u);
        count_launch();
    }
    B200_CUDA(cudaMemcpyAsync(mx, c->d_scratch_u, 4, cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    return SUCCESS;
}
EE absmax_i32_host(const int32_t *d_x, uint64_t n, int *mx)
{
    DeviceCtx *c = ctx();
    cudaStream_t st = tls().stream;
    std::lock_guard<std::mutex> g(c->scratch_mu);
    B200_CUDA(cudaMemsetAsync(c->d_scratch_u + 1, 0, 4, st));
    if (n > 0) {
        absmax_i32_kernel<<<grid_for((n + 3) / 4, c->sm_count), TPB, 0, st>>>(
            d_x, n, reinterpret_cast<int *>(c->d_scratch_u + 1));
        count_launch();
    }
    B200_CUDA(cudaMemcpyAsync(mx, c->d_scratch_u + 1, 4, cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    return SUCCESS;
}

// factor[n] = num / (sA * sB[n]): fp32 multiply, fp32 divide -- the order in which Bolt forms the
// factor of a layer (fully_connected.cpp:396,409; mmm_avx512_vnni.cpp:1805)
__global__ void col_factor_kernel(float num, float sA, const float *d_sA, float sB, const float *col_scale, uint32_t N,
    float *out)
{
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n < N) {
        const float sa = d_sA ? *d_sA : sA;
        const float sb = col_scale ? col_scale[n] : sB;
        out[n] = __fdiv_rn(num, __fmul_rn(sa, sb));
    }
}

}  // namespace

// int32 (device) -> u8 (device) with the reference's scale protocol; used by the convolution's
// u8 output (convolution_direct.cpp:2798-2806).  scale2 is a host array of two floats.
EE quantize_i32_u8_device(const int32_t *d_src, uint64_t n, uint8_t *d_q, F32 *scale2)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    float raw = 0;
    if (scale2[0] < 0 && scale2[1] > 0) {
        int mx = 0;
        B200_EE(absmax_i32_host(d_src, n, &mx));
        raw = (mx == 0) ? 1.0f : 127.0f / (float)mx;
        scale2[0] = scale2[1] * raw;
    } else if (scale2[0] > 0 && scale2[1] > 0) {
        raw = scale2[0] / scale2[1];
    }
    if (n == 0) {
        return SUCCESS;
    }
    to8_kernel<int32_t, I32ToU8><<<grid_for((n + 15) / 16, c->sm_count), TPB, 0, tls().stream>>>(d_src, n, d_q, I32ToU8{raw});
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

// F32 -> U8_Q on device pointers, scale handling of quantize_x86 (cpu/x86/quantize.cpp:33-41,
// avx512/quantize.cpp:129-133): the dynamic scale 127 / max|x| unless mode != 0 and a positive scale is given
EE quantize_f32_u8_device(const float *d_src, uint64_t n, uint8_t *d_q, F32 *scale, int mode)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (!mode || *scale <= 0) {
        float mx = 0;
        B200_EE(absmax_f32_host(d_src, n, &mx));
        const float s = (mx == 0) ? 1.0f : 127 / mx;
        *scale = (*scale > s) ? *scale : s;
    }
    if (n == 0) {
        return SUCCESS;
    }
    to8_kernel<float, F32ToU8><<<grid_for((n + 15) / 16, c->sm_count), TPB, 0, tls().stream>>>(d_src, n, d_q, F32ToU8{*scale});
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

}  // namespace b200

using namespace b200;

extern "C" {

EE quantize_cuda_b200(const TensorDesc *dDesc, const void *data, TensorDesc *qDesc, void *qData, F32 *scale,
    int mode)
{
    if (dDesc == nullptr || qDesc == nullptr) {
        return NULL_POINTER;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    const uint64_t n = desc_elems(dDesc);
    const DataType sdt = dDesc->dt, qdt = qDesc->dt;
    const bool f32 = (sdt == DT_F32 || sdt == DT_F32_8Q);
    const bool known = (f32 && (qdt == DT_I8 || qdt == DT_U8_Q)) || (sdt == DT_U8_Q && qdt == DT_I8) ||
        (sdt == DT_I32 && (qdt == DT_I8 || qdt == DT_U8_Q));
    if (!known) {
        return NOT_SUPPORTED;
    }
    if (sdt != DT_U8_Q && scale == nullptr) {
        return NOT_MATCH;  // quantize.cpp:123-125
    }
    if (n == 0) {
        return SUCCESS;
    }
    if (data == nullptr || qData == nullptr) {
        return NULL_POINTER;
    }
    cudaStream_t st = tls().stream;
    Stage sg;
    const size_t src_bytes = n * (sdt == DT_U8_Q ? 1 : 4);
    const void *d_src = sg.in(data, src_bytes);
    uint8_t *d_q = reinterpret_cast<uint8_t *>(sg.out(qData, n));
    if (d_src == nullptr || d_q == nullptr) {
        return ALLOC_FAILED;
    }
    const uint32_t grid = grid_for((n + 15) / 16, c->sm_count);
    if (f32) {
        if (!mode || *scale <= 0) {  // quantize.cpp:129-133
            float mx = 0;
            B200_EE(absmax_f32_host(reinterpret_cast<const float *>(d_src), n, &mx));
            const float s = (mx == 0) ? 1.0f : 127 / mx;
            *scale = (*scale > s) ? *scale : s;
        }
        if (qdt == DT_U8_Q) {
            to8_kernel<float, F32ToU8><<<grid, TPB, 0, st>>>(reinterpret_cast<const float *>(d_src), n, d_q, F32ToU8{*scale});
        } else {
            to8_kernel<float, F32ToI8><<<grid, TPB, 0, st>>>(reinterpret_cast<const float *>(d_src), n, d_q, F32ToI8{*scale});
        }
        count_launch();
    } else if (sdt == DT_U8_Q) {
        u8_to_i8_kernel<<<grid, TPB, 0, st>>>(reinterpret_cast<const uint8_t *>(d_src), n, d_q);
        count_launch();
    } else {
        float raw = 0;  // quantize.cpp:320-326 / 369-375
        if (scale[0] < 0 && scale[1] > 0) {
            int mx = 0;
            B200_EE(absmax_i32_host(reinterpret_cast<const int32_t *>(d_src), n, &mx));
            raw = (mx == 0) ? 1.0f : 127.0f / (float)mx;
            scale[0] = scale[1] * raw;
        } else if (scale[0] > 0 && scale[1] > 0) {
            raw = scale[0] / scale[1];
        }
        if (qdt == DT_U8_Q) {
            to8_kernel<int32_t, I32ToU8><<<grid, TPB, 0, st>>>(reinterpret_cast<const int32_t *>(d_src), n, d_q, I32ToU8{raw});
        } else {
            to8_kernel<int32_t, I32ToI8><<<grid, TPB, 0, st>>>(reinterpret_cast<const int32_t *>(d_src), n, d_q, I32ToI8{raw});
        }
        count_launch();
    }
    B200_CUDA(cudaGetLastError());
    return sg.finish();
}

EE bolt_b200_absmax_scale_f32(const F32 *data, uint64_t n, F32 *d_scale)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (data == nullptr || d_scale == nullptr) {
        return NULL_POINTER;
    }
    cudaStream_t st = tls().stream;
    unsigned *bits = c->d_scratch_u + 2;
    B200_CUDA(cudaMemsetAsync(bits, 0, 4, st));
    if (n > 0) {
        absmax_f32_kernel<<<grid_for((n + 3) / 4, c->sm_count), TPB, 0, st>>>(data, n, bits);
        count_launch();
    }
    finalize_scale_kernel<<<1, 1, 0, st>>>(bits, d_scale);
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

EE bolt_b200_col_factor(F32 num, F32 sA, const F32 *d_sA, F32 sB, const F32 *col_scale, U32 N, F32 *factor)
{
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    if (factor == nullptr) {
        return NULL_POINTER;
    }
    if (N == 0) {
        return SUCCESS;
    }
    col_factor_kernel<<<(N + 255) / 256, 256, 0, tls().stream>>>(num, sA, d_sA, sB, col_scale, N, factor);
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

EE bolt_b200_quantize_f32_u8_dev(const F32 *data, uint64_t n, UINT8 *q, const F32 *d_scale)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (data == nullptr || q == nullptr || d_scale == nullptr) {
        return NULL_POINTER;
    }
    if (n == 0) {
        return SUCCESS;
    }
    to8_kernel<float, F32ToU8Dev><<<grid_for((n + 15) / 16, c->sm_count), TPB, 0, tls().stream>>>(data, n, q,
        F32ToU8Dev{d_scale});
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

EE quantize_bias_offsetC_cuda_b200(const void *bias, const TensorDesc *biasDesc, DataType qType,
    const void *filter, const TensorDesc *filterDesc, const F32 *scale, void *offsetCBias)
{
    if (biasDesc == nullptr || filterDesc == nullptr) {
        return NULL_POINTER;
    }
    if (qType != DT_I32) {
        return NOT_SUPPORTED;
    }
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    if (bias == nullptr && filter == nullptr) {
        return SUCCESS;
    }
    // "native" formats carry no packed offset (quantize.cpp:244-259)
    const DataFormat fdf = filterDesc->df;
    const bool native = fdf == DF_NCHW || fdf == 24 /*DF_NHWC*/ || fdf == 15 /*DF_MTK*/ || fdf == DF_NORMAL ||
        fdf == DF_TRANSPOSE;
    uint32_t n = (uint32_t)desc_elems(biasDesc);
    const bool no_bias = (bias == nullptr) || n == 0;
    if (no_bias) {
        n = filterDesc->dims[0] > filterDesc->dims[1] ? filterDesc->dims[0] : filterDesc->dims[1];
    } else if (biasDesc->dt != DT_F32 && biasDesc->dt != DT_I32) {
        return NOT_SUPPORTED;
    }
    if (n == 0) {
        return SUCCESS;
    }
    if (offsetCBias == nullptr) {
        return NULL_POINTER;
    }
    cudaStream_t st = tls().stream;
    Stage sg;
    const bool i32_bias = !no_bias && biasDesc->dt == DT_I32;
    // fp32 bias (or none): the packed offset is read only from non-native filter formats;
    // int32 bias: `filter` is an offset array whenever it is given (quantize.cpp:100-111)
    const bool use_off = (filter != nullptr) && (i32_bias || !native);
    const int32_t *d_off = use_off ? reinterpret_cast<const int32_t *>(sg.in(filter, (size_t)n * 4)) : nullptr;
    const void *d_bias = no_bias ? nullptr : sg.in(bias, (size_t)n * 4);
    int32_t *d_out = reinterpret_cast<int32_t *>(sg.out(offsetCBias, (size_t)n * 4));
    if (d_out == nullptr || (use_off && d_off == nullptr) || (!no_bias && d_bias == nullptr)) {
        return ALLOC_FAILED;
    }
    if (i32_bias) {
        bias_i32_offsetc_kernel<<<(n + 255) / 256, 256, 0, st>>>(reinterpret_cast<const int32_t *>(d_bias), d_off, n,
            d_out);
    } else {
        if (!no_bias && scale == nullptr) {
            return NULL_POINTER;
        }
        bias_offsetc_kernel<<<(n + 255) / 256, 256, 0, st>>>(reinterpret_cast<const float *>(d_bias), d_off, n,
            no_bias ? 0.f : scale[0], d_out);
    }
    count_launch();
    B200_CUDA(cudaGetLastError());
    return sg.finish();
}

EE dequantize_cuda_b200(const TensorDesc *qDesc, const void *qData, const F32 *scale, const TensorDesc *bDesc,
    const void *bData, const TensorDesc *dDesc, void *dData)
{
    (void)bDesc;
    (void)bData;  // ignored, as on x86 (cpu/x86/dequantize.cpp:19-48)
    if (qDesc == nullptr || dDesc == nullptr || scale == nullptr) {
        return NULL_POINTER;
    }
    if (dDesc->dt != DT_F32 || (qDesc->dt != DT_I32 && qDesc->dt != DT_U8_Q)) {
        return NOT_SUPPORTED;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    const uint64_t n = desc_elems(dDesc);
    if (n == 0) {
        return SUCCESS;
    }
    if (qData == nullptr || dData == nullptr) {
        return NULL_POINTER;
    }
    cudaStream_t st = tls().stream;
    Stage sg;
    const bool i32 = qDesc->dt == DT_I32;
    const void *d_q = sg.in(qData, n * (i32 ? 4 : 1));
    float *d_out = reinterpret_cast<float *>(sg.out(dData, n * 4));
    if (d_q == nullptr || d_out == nullptr) {
        return ALLOC_FAILED;
    }
    const float factor = i32 ? (1 / *scale) : (1.0f / scale[0]);
    if (i32) {
        dequant_i32_kernel<<<grid_for((n + 3) / 4, c->sm_count), TPB, 0, st>>>(
            reinterpret_cast<const int32_t *>(d_q), n, factor, d_out);
    } else {
        dequant_u8_kernel<<<grid_for((n + 15) / 16, c->sm_count), TPB, 0, st>>>(
            reinterpret_cast<const uint8_t *>(d_q), n, factor, d_out);
    }
    count_launch();
    B200_CUDA(cudaGetLastError());
    return sg.finish();
}

}  // extern "C"
