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

__device__ __forceinline__ int dp4a_u8s8(uint32_t m, uint32_t v, int acc)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(m), "r"(v), "r"(acc));
    return d;
}

// u8 epilogue of the reference's row GEMV: multi-row kernels use vpmovusdb, the single-row kernel
// (the last N % 4 rows) adds 128, compares signed with 255 and stores the low byte
// (mvm_avx512_vnni_row.cpp:384-406, 884-900)
__device__ __forceinline__ void row_epilogue(int acc, uint32_t n, uint32_t N, void *y, int out_kind, float factor)
{
    if (out_kind == 0) {
        reinterpret_cast<int32_t *>(y)[n] = acc;
    } else if (out_kind == 1) {
        reinterpret_cast<float *>(y)[n] = acc_to_f32(acc, factor);
    } else if (n >= N - (N % 4)) {
        const int t = (int)((uint32_t)cvt_rne_x86(__fmul_rn(__int2float_rn(acc), factor)) + 128u);
        reinterpret_cast<uint8_t *>(y)[n] = (t < 255) ? (uint8_t)t : (uint8_t)255;
    } else {
        reinterpret_cast<uint8_t *>(y)[n] = (uint8_t)acc_to_u8(acc, factor);
    }
}

// y[n] = -128 * sum(v) + sum_k M_u8[n,k] * v_s8[k]: the activation x activation GEMV of Bolt's matmul
// (mvm_avx512_int8_row_i8u8, mvm_avx512_vnni_row.cpp:931-1028).  transposed == 0: M is [N][K], one warp
// per row, 128-bit loads; transposed == 1: M is [K][N], one thread per column (coalesced along n).
__global__ void __launch_bounds__(WARPS * 32)
gemv_row_u8s8_kernel(uint32_t N, uint32_t K, const uint8_t *__restrict__ Mx, int transposed, const int8_t *__restrict__ v,
    void *y, int out_kind, float factor)
{
    extern __shared__ __align__(16) uint8_t sv[];  // the vector, zero padded to a multiple of 16
    __shared__ int warp_sum[WARPS];
    const uint32_t Kp = (K + 15) & ~15u;
    int part = 0;
    for (uint32_t k = threadIdx.x; k < Kp; k += blockDim.x) {
        const int8_t e = (k < K) ? v[k] : (int8_t)0;
        sv[k] = (uint8_t)e;
        part += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        part += __shfl_xor_sync(0xffffffffu, part, o);
    }
    if ((threadIdx.x & 31) == 0) {
        warp_sum[threadIdx.x >> 5] = part;
    }
    __syncthreads();
    int offset = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        offset += warp_sum[w];
    }
    offset *= -128;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (!transposed) {
        const bool vec = (K % 16 == 0) && (reinterpret_cast<uintptr_t>(Mx) % 16 == 0);
        for (uint32_t n = blockIdx.x * WARPS + warp; n < N; n += gridDim.x * WARPS) {
            const uint8_t *row = Mx + (size_t)n * K;
            int acc = 0;
            if (vec) {
                const uint4 *row4 = reinterpret_cast<const uint4 *>(row);
                const uint4 *v4 = reinterpret_cast<const uint4 *>(sv);
                for (uint32_t i = lane; i < (K >> 4); i += 32) {
                    const uint4 m = ld_stream(row4 + i), x = v4[i];
                    acc = dp4a_u8s8(m.x, x.x, acc);
                    acc = dp4a_u8s8(m.y, x.y, acc);
                    acc = dp4a_u8s8(m.z, x.z, acc);
                    acc = dp4a_u8s8(m.w, x.w, acc);
                }
            } else {
                for (uint32_t k = lane; k < K; k += 32) {
                    acc += (int)row[k] * (int)(int8_t)sv[k];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                acc += __shfl_xor_sync(0xffffffffu, acc, o);
            }
            if (lane == 0) {
                row_epilogue(acc + offset, n, N, y, out_kind, factor);
            }
        }
    } else {
        for (uint32_t n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x) {
            int acc = 0;
            for (uint32_t k = 0; k < K; ++k) {
                acc += (int)Mx[(size_t)k * N + n] * (int)(int8_t)sv[k];
            }
            row_epilogue(acc + offset, n, N, y, out_kind, factor);
        }
    }
}

}  // namespace

EE launch_gemv_row(uint32_t N, uint32_t K, const uint8_t *Mx, bool transposed, const int8_t *v, void *y, int out_kind,
    float factor, cudaStream_t st)
{
    if (N == 0) {
        return SUCCESS;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    const size_t smem = B200_ALIGN((size_t)K, 16) + 16;
    if (smem > 200 * 1024) {
        return NOT_SUPPORTED;
    }
    {
        const void *ks[1] = {(const void *)gemv_row_u8s8_kernel};
        B200_EE(raise_smem_limit(c, KF_GEMV_ROW, ks, 1, 200 * 1024));
    }
    uint32_t blocks = transposed ? (N + WARPS * 32 - 1) / (WARPS * 32) : (N + WARPS - 1) / WARPS;
    const uint32_t cap = (uint32_t)c->sm_count * 4;
    if (blocks > cap) {
        blocks = cap;
    }
    gemv_row_u8s8_kernel<<<blocks, WARPS * 32, smem, st>>>(N, K, Mx, transposed ? 1 : 0, v, y, out_kind, factor);
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

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
    {
        const void *ks[1] = {(const void *)gemv_s8u8_kernel};
        B200_EE(raise_smem_limit(c, KF_GEMV, ks, 1, 200 * 1024));
    }
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
