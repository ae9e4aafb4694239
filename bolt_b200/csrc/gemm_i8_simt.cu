// gemm_i8_simt.cu -- weight packing (+ colsum offset) and the any-shape CUDA-core GEMM.
//
// The tensor-core kernel needs 16-byte aligned rows (K % 16 == 0, A row-major).  Everything
// else -- ragged K, transposed A, the 1..33 shapes of Bolt's own cover test
// (compute/blas_enhance/tests/test_mmm.cpp:165-171) -- runs here on dp4a-free integer math.
// Same arithmetic, same epilogue.
#include "common.cuh"

namespace b200 {
namespace {

// ---- packing: s8 [K,N] or [N,K] -> [Np][Kp] K-major, zero padded; offsetC = -128 * sum_k ------
// replaces matrix_matrix_multiply_transform_rhsN/T_int8 (mmm_avx512_vnni.cpp:60-121) and the
// GEMV packer (mvm_avx512_vnni.cpp:28-131).  One warp per output row n.
__global__ void pack_rhs_kernel(const int8_t *__restrict__ src, int src_is_nk, uint32_t N, uint32_t K,
    int8_t *__restrict__ dst, uint32_t Kp, uint32_t Np, int32_t *__restrict__ offsetC)
{
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (n >= Np) {
        return;
    }
    int32_t sum = 0;
    for (uint32_t k = lane; k < Kp; k += 32) {
        int8_t v = 0;
        if (n < N && k < K) {
            v = src_is_nk ? src[(size_t)n * K + k] : src[(size_t)k * N + n];
        }
        dst[(size_t)n * Kp + k] = v;
        sum += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    if (lane == 0 && n < N && offsetC != nullptr) {
        offsetC[n] = sum * (-128);
    }
}

// [K,N] source: the warp-per-row kernel above reads with stride N.  This tiled variant transposes
// through shared memory so both sides are coalesced; colsums are accumulated with atomics.
constexpr int TP = 32;
__global__ void pack_rhs_kn_kernel(const int8_t *__restrict__ src, uint32_t N, uint32_t K,
    int8_t *__restrict__ dst, uint32_t Kp, uint32_t Np, int32_t *__restrict__ colsum)
{
    __shared__ int8_t tile[TP][TP + 4];
    const uint32_t n0 = blockIdx.x * TP, k0 = blockIdx.y * TP;
    for (uint32_t r = threadIdx.y; r < TP; r += blockDim.y) {
        const uint32_t k = k0 + r, n = n0 + threadIdx.x;
        tile[r][threadIdx.x] = (k < K && n < N) ? src[(size_t)k * N + n] : (int8_t)0;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.y; r < TP; r += blockDim.y) {
        const uint32_t n = n0 + r, k = k0 + threadIdx.x;
        int32_t v = tile[threadIdx.x][r];
        if (n < Np && k < Kp) {
            dst[(size_t)n * Kp + k] = (int8_t)v;
        }
        // row-sum over this tile's 32 k values
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            v += __shfl_xor_sync(0xffffffffu, v, o);
        }
        if (threadIdx.x == 0 && n < N && colsum != nullptr) {
            atomicAdd(&colsum[n], v);
        }
    }
}
__global__ void scale_offset_kernel(int32_t *offsetC, uint32_t N)
{
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n < N) {
        offsetC[n] *= -128;
    }
}

// ---- any-shape GEMM: one thread per output element, 16 x 16 tiles through shared memory ----------
constexpr int TS = 16;
__global__ void gemm_simt_kernel(uint32_t M, uint32_t N, uint32_t K, const uint8_t *__restrict__ A, int a_t,
    const int8_t *__restrict__ B, uint32_t Kp, void *C, GemmEpilogue ep)
{
    __shared__ uint8_t sa[TS][TS + 1];
    __shared__ int8_t sb[TS][TS + 1];
    const uint32_t m = blockIdx.y * TS + threadIdx.y;
    const uint32_t n = blockIdx.x * TS + threadIdx.x;
    int acc = 0;
    for (uint32_t k0 = 0; k0 < K; k0 += TS) {
        {
            // A tile: sa[row m][k]
            const uint32_t k = k0 + threadIdx.x;
            uint8_t v = 0;
            if (m < M && k < K) {
                v = a_t ? A[(size_t)k * M + m] : A[(size_t)m * K + k];
            }
            sa[threadIdx.y][threadIdx.x] = v;
            // B tile: sb[col n][k], B is [Np][Kp]
            const uint32_t nn = blockIdx.x * TS + threadIdx.y;
            int8_t w = 0;
            if (nn < N && k < K) {
                w = B[(size_t)nn * Kp + k];
            }
            sb[threadIdx.y][threadIdx.x] = w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TS; ++k) {
            acc += (int)sa[threadIdx.y][k] * (int)sb[threadIdx.x][k];
        }
        __syncthreads();
    }
    if (m >= M || n >= N) {
        return;
    }
    if (ep.offsetC != nullptr) {
        acc += ep.offsetC[n];
    }
    const size_t o = (size_t)m * N + n;
    if (ep.out_kind != 2 && ep.accumulate) {
        acc += reinterpret_cast<const int32_t *>(C)[o];
    }
    if (ep.out_kind == 0) {
        reinterpret_cast<int32_t *>(C)[o] = acc;
        return;
    }
    float fac = ep.factor;
    if (ep.col_factor != nullptr) {
        fac = ep.col_factor[n];
    } else if (ep.per_channel) {
        const float sa_ = ep.row_scale ? ep.row_scale[m] : (ep.sA_dev ? *ep.sA_dev : ep.sA);
        const float sb_ = ep.col_scale ? ep.col_scale[n] : ep.sB;
        fac = __fdiv_rn(ep.num, __fmul_rn(sa_, sb_));
    }
    if (ep.out_kind == 1) {
        reinterpret_cast<float *>(C)[o] = acc_to_f32(acc, fac);
    } else {
        reinterpret_cast<uint8_t *>(C)[o] = (uint8_t)acc_to_u8(acc, fac);
    }
}

}  // namespace

EE launch_pack_rhs(const int8_t *src, bool src_is_nk, uint32_t N, uint32_t K, int8_t *dst, uint32_t Kp,
    uint32_t Np, int32_t *offsetC, cudaStream_t st)
{
    if (N == 0 || K == 0) {
        return SUCCESS;
    }
    if (src_is_nk || N < 64) {
        const int warps = 8;
        pack_rhs_kernel<<<(Np + warps - 1) / warps, warps * 32, 0, st>>>(src, src_is_nk ? 1 : 0, N, K, dst, Kp, Np,
            offsetC);
        count_launch();
    } else {
        if (offsetC != nullptr) {
            B200_CUDA(cudaMemsetAsync(offsetC, 0, (size_t)N * 4, st));
        }
        dim3 grid((Np + TP - 1) / TP, (Kp + TP - 1) / TP);
        pack_rhs_kn_kernel<<<grid, dim3(TP, 8), 0, st>>>(src, N, K, dst, Kp, Np, offsetC);
        count_launch();
        if (offsetC != nullptr) {
            scale_offset_kernel<<<(N + 255) / 256, 256, 0, st>>>(offsetC, N);
            count_launch();
        }
    }
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

EE launch_gemm_simt(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, bool a_transposed, const int8_t *B,
    uint32_t Kp, void *C, const GemmEpilogue &ep, cudaStream_t st)
{
    if (M == 0 || N == 0) {
        return SUCCESS;
    }
    dim3 grid((N + TS - 1) / TS, (M + TS - 1) / TS);
    if (grid.y > 65535) {
        return NOT_SUPPORTED;
    }
    gemm_simt_kernel<<<grid, dim3(TS, TS), 0, st>>>(M, N, K, A, a_transposed ? 1 : 0, B, Kp, C, ep);
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

}  // namespace b200
