// gemv_i8.cu -- y[N] = epilogue( offsetC[n] + sum_k W_s8[n,k] * x_u8[k] ), the M = 1 case.
//
// Replaces Bolt's packed-weight GEMV kernels (compute/blas_enhance/src/cpu/x86/int8/avx512/
// mvm_avx512_vnni.cpp:133-759).  The work is one pass over the weight matrix, so the kernel is
// built for HBM bandwidth: one warp per weight row, 128-bit streaming loads (four in flight per
// lane), the activation vector staged once per CTA in shared memory, dp4a (s8 x u8) accumulation
// and a warp-shuffle reduction.
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ int dp4a_s8u8(uint32_t w, uint32_t x, int acc)
{
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(x), "r"(acc));
    return d;
}
__device__ __forceinline__ uint4 ld_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ int dot16(uint4 w, uint4 x, int acc)
{
    acc = dp4a_s8u8(w.x, x.x, acc);
    acc = dp4a_s8u8(w.y, x.y, acc);
    acc = dp4a_s8u8(w.z, x.z, acc);
    acc = dp4a_s8u8(w.w, x.w, acc);
    return acc;
}

constexpr int WARPS = 8;

// out_kind 0 int32 / 1 fp32 / 2 u8.  Rows n >= N - N % 8 follow the reference's scalar tail
// (mvm_avx512_vnni.cpp:667-701): the incoming y is not added and the u8 conversion truncates.
__global__ void __launch_bounds__(WARPS * 32)
gemv_s8u8_kernel(uint32_t N, uint32_t K, const int8_t *__restrict__ W, uint32_t Kp,
    const uint8_t *__restrict__ x, const int32_t *__restrict__ offsetC, void *y, int out_kind, float factor,
    int vec_ok)
{
    extern __shared__ __align__(16) uint8_t sx[];
    // stage x, zero padded to Kp (the packed weight is zero there, any value would do)
    if ((K & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        for (uint32_t k = threadIdx.x * 16; k < Kp; k += blockDim.x * 16) {
            *reinterpret_cast<uint4 *>(sx + k) =
                (k < K) ? *reinterpret_cast<const uint4 *>(x + k) : make_uint4(0, 0, 0, 0);
        }
    } else {
        for (uint32_t k = threadIdx.x; k < Kp; k += blockDim.x) {
            sx[k] = (k < K) ? x[k] : (uint8_t)0;
        }
    }
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t tail_begin = N - (N % 8);
    for (uint32_t n = blockIdx.x * WARPS + warp; n < N; n += gridDim.x * WARPS) {
        const int8_t *row = W + (size_t)n * Kp;
        int acc = 0;
        if (vec_ok) {
            const uint4 *row4 = reinterpret_cast<const uint4 *>(row);
            const uint4 *x4 = reinterpret_cast<const uint4 *>(sx);
            const uint32_t nv = Kp >> 4;
            uint32_t i = lane;
            for (; i + 96 < nv; i += 128) {
                const uint4 w0 = ld_stream(row4 + i);
                const uint4 w1 = ld_stream(row4 + i + 32);
                const uint4 w2 = ld_stream(row4 + i + 64);
                const uint4 w3 = ld_stream(row4 + i + 96);
                acc = dot16(w0, x4[i], acc);
                acc = dot16(w1, x4[i + 32], acc);
                acc = dot16(w2, x4[i + 64], acc);
                acc = dot16(w3, x4[i + 96], acc);
            }
            for (; i < nv; i += 32) {
                acc = dot16(ld_stream(row4 + i), x4[i], acc);
            }
            for (uint32_t k = (nv << 4) + lane; k < Kp; k += 32) {
                acc += (int)row[k] * (int)sx[k];
            }
        } else {
            for (uint32_t k = lane; k < Kp; k += 32) {
                acc += (int)row[k] * (int)sx[k];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
        }
        if (lane == 0) {
            if (offsetC != nullptr) {
                acc += offsetC[n];
            }
            const bool tail = n >= tail_begin;
            if (out_kind == 2) {
                uint8_t *out = reinterpret_cast<uint8_t *>(y);
                if (tail) {
                    const float f = __fmul_rn(__int2float_rn(acc), factor);
                    // (I32)(f + 128): C++ truncation; out of range is undefined there, the
                    // x86 cvttss2si answer (0x80000000) is reproduced
                    const float g = __fadd_rn(f, 128.0f);
                    int t = (g >= -2147483648.0f && g < 2147483648.0f) ? __float2int_rz(g) : (int)0x80000000;
                    out[n] = (uint8_t)((t > 255) ? 255 : t);
                } else {
                    out[n] = (uint8_t)acc_to_u8(acc, factor);
                }
            } else {
                int32_t *yi = reinterpret_cast<int32_t *>(y);
                if (!tail) {
                    acc += yi[n];
                }
                if (out_kind == 1) {
                    reinterpret_cast<float *>(y)[n] = acc_to_f32(acc, factor);
                } else {
                    yi[n] = acc;
                }
            }
        }
    }
}

}  // namespace

EE launch_gemv(uint32_t N, uint32_t K, const int8_t *W, uint32_t Kp, const uint8_t *x, const int32_t *offsetC,
    void *y, int out_kind, float factor, cudaStream_t st)
{
    if (N == 0) {
        return SUCCESS;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    const size_t smem = B200_ALIGN((size_t)Kp, 16);
    if (smem > 200 * 1024) {
        return NOT_SUPPORTED;
    }
    static std::once_flag once;
    static cudaError_t err = cudaSuccess;
    std::call_once(once, [] {
        err = cudaFuncSetAttribute(gemv_s8u8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    });
    B200_CUDA(err);
    const int vec_ok = (Kp % 16 == 0) && (reinterpret_cast<uintptr_t>(W) % 16 == 0);
    uint32_t blocks = (N + WARPS - 1) / WARPS;
    // persistent-style grid: every CTA stages x once and then streams many rows (a short-lived CTA
    // spends as long staging x as reading its rows)
    const uint32_t cap = (uint32_t)c->sm_count * 4;
    if (blocks > cap) {
        blocks = cap;
    }
    gemv_s8u8_kernel<<<blocks, WARPS * 32, smem, st>>>(N, K, W, Kp, x, offsetC, y, out_kind, factor, vec_ok);
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

}  // namespace b200
