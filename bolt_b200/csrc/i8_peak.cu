// i8_peak.cu -- measures the rate at which this GPU's tensor cores retire tcgen05.mma.kind::i8, the
// ceiling the u8 x s8 GEMM and convolution kernels are judged against.
//
// One CTA per SM.  One thread issues `iters` MMAs of 128 x 256 x 32 (A unsigned, B signed, int32
// accumulators in tensor memory) back to back on operand tiles that sit in shared memory for the whole
// run -- nothing is loaded, nothing is stored, there is no epilogue -- and commits every 32 of them to an
// mbarrier so that at most 64 are in flight.  ops = SMs x iters x 2 x 128 x 256 x 32.
// Every wait is bounded; tensor memory is always released.
#include "common.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr uint32_t PROBE_N = 256;
constexpr uint32_t PROBE_BATCH = 32;  // MMAs per commit

__global__ void __launch_bounds__(128, 1) i8_mma_rate_kernel(uint32_t iters, int *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;                                  // 128 rows x 128 B
    uint8_t *smem_b = smem + BLOCK_M * BLOCK_K;              // 256 rows x 128 B
    __shared__ uint64_t bar[2];
    __shared__ uint32_t tmem_base_s;
    // operands: any bytes will do; fill them so that the run does not depend on what was there
    for (uint32_t i = threadIdx.x; i < (BLOCK_M + PROBE_N) * BLOCK_K / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t *>(smem)[i] = 0x01010101u * (i & 3);
    }
    if (threadIdx.x == 0) {
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if ((threadIdx.x >> 5) == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_proxy_async_smem();  // the generic-proxy fill above is read by the tensor cores
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc_i8(PROBE_N);
        const uint64_t da = make_desc_sw128(smem_u32(smem_a));
        const uint64_t db = make_desc_sw128(smem_u32(smem_b));
        uint32_t phase[2] = {0, 0};
        uint32_t committed = 0;
        bool ok = true;
        for (uint32_t i = 0; i < iters && ok; i += PROBE_BATCH) {
            const uint32_t slot = committed & 1;
            if (committed >= 2) {
                // the batch that used this barrier two commits ago must have retired
                ok = mbar_wait(&bar[slot], phase[slot]);
                phase[slot] ^= 1;
            }
            const uint32_t n = min(PROBE_BATCH, iters - i);
            for (uint32_t j = 0; j < n; ++j) {
                // alternate between the two accumulators, rotate through the four K slices of the tiles
                umma_i8(tmem_base + ((i + j) & 1) * PROBE_N, da + 2 * (j & 3), db + 2 * (j & 3), idesc, 1u);
            }
            tcgen05_commit(&bar[slot]);
            ++committed;
        }
        // drain
        for (uint32_t d = 0; d < 2 && ok; ++d) {
            const uint32_t slot = (committed + d) & 1;
            if (committed + d >= 2) {
                ok = mbar_wait(&bar[slot], phase[slot]);
                phase[slot] ^= 1;
            }
        }
        if (!ok) {
            atomicExch(status, 31);
        }
    }
    __syncthreads();
    if ((threadIdx.x >> 5) == 0) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// One CTA, one barrier that expects an arrival nobody makes: the bounded wait has to give up after
// `limit_cycles`, record it in the status word and return, leaving the context usable.
__global__ void wait_runs_out_kernel(long long limit_cycles, int *status)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait_limit(&bar, 0, limit_cycles)) {
            atomicExch(status, 21);
        }
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" EE bolt_b200_i8_mma_rate(U32 mma_per_sm, F32 *milliseconds, F32 *tops)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (milliseconds == nullptr || tops == nullptr) {
        return NULL_POINTER;
    }
    if (mma_per_sm == 0) {
        return NOT_MATCH;
    }
    const size_t smem = 1024 + (size_t)(tc::BLOCK_M + PROBE_N) * tc::BLOCK_K;
    {
        const void *ks[1] = {(const void *)i8_mma_rate_kernel};
        B200_EE(raise_smem_limit(c, KF_PROBE, ks, 1, smem));
    }
    cudaStream_t st = tls().stream;
    cudaEvent_t e0, e1;
    B200_CUDA(cudaEventCreate(&e0));
    B200_CUDA(cudaEventCreate(&e1));
    i8_mma_rate_kernel<<<c->sm_count, 128, smem, st>>>(mma_per_sm < 4096 ? mma_per_sm : 4096, c->d_status);  // warm-up
    cudaEventRecord(e0, st);
    i8_mma_rate_kernel<<<c->sm_count, 128, smem, st>>>(mma_per_sm, c->d_status);
    cudaEventRecord(e1, st);
    count_launch(2);
    cudaError_t err = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (err == cudaSuccess) {
        err = cudaEventElapsedTime(&ms, e0, e1);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    B200_CUDA(err);
    *milliseconds = ms;
    *tops = (float)((double)c->sm_count * mma_per_sm * 2.0 * tc::BLOCK_M * PROBE_N * tc::UMMA_K / (ms * 1e-3) / 1e12);
    return SUCCESS;
}

extern "C" EE bolt_b200_selftest_wait_limit(U32 limit_cycles)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (limit_cycles == 0 || limit_cycles > 2000000000u) {
        return NOT_MATCH;  // at most about a second
    }
    wait_runs_out_kernel<<<1, 32, 0, tls().stream>>>((long long)limit_cycles, c->d_status);
    count_launch(1);
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}
