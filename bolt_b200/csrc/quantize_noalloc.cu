// quantize_noalloc.cu -- dynamic per-tensor F32 -> U8_Q quantization that allocates nothing.
//
// Some hosts cannot allocate device memory when they call in: an inference server that hands the
// whole GPU to its own pool allocator at start-up (cudaMalloc then simply fails), a plug-in whose
// host forbids allocation on the serving path for latency reasons, a process running under a fixed
// memory budget.  The regular entry points create a per-device context with cudaMalloc on first
// use; this one does not.  Its scratch -- the per-block partial maxima of the absmax reduction, a
// completion counter and the resulting scale -- lives in a fixed array in the library's own device
// image, so every GPU that loads the library holds these 16.5 KiB until the process exits.
//
// Same arithmetic as quantize_cuda_b200 (F32 -> U8_Q, scale = 127 / absmax): scale finding, then
// q = clamp(rne(x * scale + 128), 1, 255).
#include <mutex>

#include "common.cuh"

namespace b200 {
namespace {

constexpr uint32_t kChunk = 16384;   // elements reduced by one block
constexpr uint32_t kSlots = 4096;    // partial maxima the scratch can hold
constexpr uint64_t kMaxElements = (uint64_t)kChunk * kSlots;  // 67,108,864
static_assert(kMaxElements == BOLT_B200_NOALLOC_MAX_ELEMENTS, "header and kernel disagree on the limit");

// [0, kSlots): partial maxima (float bits); [kSlots]: blocks finished; [kSlots + 1]: scale (float bits)
static __device__ __align__(256) unsigned g_noalloc_scratch[kSlots + 64];

// In host code the array's name is only a stand-in; the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.
std::mutex g_setup_mu;
unsigned *g_scratch_addr[16] = {nullptr};

EE scratch_for_current_device(unsigned **out)
{
    int dev = -1;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) {
        return NOT_SUPPORTED;
    }
    std::lock_guard<std::mutex> g(g_setup_mu);
    if (g_scratch_addr[dev] == nullptr) {
        void *p = nullptr;
        B200_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_scratch_addr[dev] = reinterpret_cast<unsigned *>(p);
    }
    *out = g_scratch_addr[dev];
    return SUCCESS;
}

// One block per chunk: block maximum of |x| -> its slot; the block that finishes last folds all
// slots into the scale and rewinds the counter.
__global__ void __launch_bounds__(256)
absmax_chunks_kernel(const float *__restrict__ x, uint64_t n, unsigned *scratch, float *scale_out)
{
    __shared__ unsigned warp_max[8];
    __shared__ bool is_last;
    const uint64_t begin = (uint64_t)blockIdx.x * kChunk;
    const uint64_t end = min(begin + kChunk, n);
    unsigned m = 0;
    for (uint64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
        m = max(m, __float_as_uint(x[i]) & 0x7FFFFFFFu);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    if ((threadIdx.x & 31) == 0) {
        warp_max[threadIdx.x >> 5] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            m = max(m, warp_max[w]);
        }
        scratch[blockIdx.x] = m;
        __threadfence();
        is_last = atomicAdd(&scratch[kSlots], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) {
        return;
    }
    __threadfence();
    unsigned t = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += blockDim.x) {
        t = max(t, reinterpret_cast<volatile unsigned *>(scratch)[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        t = max(t, __shfl_xor_sync(0xffffffffu, t, o));
    }
    if ((threadIdx.x & 31) == 0) {
        warp_max[threadIdx.x >> 5] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            t = max(t, warp_max[w]);
        }
        const float mx = __uint_as_float(t);
        const float s = (mx == 0.f) ? 1.0f : __fdiv_rn(127.0f, mx);  // avx512/quantize.cpp:63-67
        scratch[kSlots + 1] = __float_as_uint(s);
        *scale_out = s;
        scratch[kSlots] = 0;  // rewind for the next call
    }
}

__global__ void __launch_bounds__(256)
quantize_u8_from_scratch_kernel(const float *__restrict__ x, uint64_t n, uint8_t *__restrict__ q, const unsigned *scratch)
{
    const float s = __uint_as_float(scratch[kSlots + 1]);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        // avx512/quantize.cpp:135-178: vmulps, vaddps 128, vcvtps2dq{rn}, max 1, min 255
        const int r = cvt_rne_x86(__fadd_rn(__fmul_rn(x[i], s), 128.0f));
        q[i] = (uint8_t)min(255, max(1, r));
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" EE bolt_b200_quantize_f32_u8_noalloc(const F32 *data, uint64_t n, UINT8 *q, F32 *d_scale)
{
    if (data == nullptr || q == nullptr || d_scale == nullptr) {
        return NULL_POINTER;
    }
    if (n == 0 || n > kMaxElements) {
        return NOT_SUPPORTED;  // beyond what the fixed scratch can reduce (or nothing to do)
    }
    unsigned *scratch = nullptr;
    B200_EE(scratch_for_current_device(&scratch));
    cudaStream_t st = tls().stream;
    // the array keeps whatever the previous call left: the completion counter must start at zero
    B200_CUDA(cudaMemsetAsync(scratch + kSlots, 0, sizeof(unsigned), st));
    const uint32_t blocks = (uint32_t)((n + kChunk - 1) / kChunk);
    absmax_chunks_kernel<<<blocks, 256, 0, st>>>(data, n, scratch, d_scale);
    const uint64_t qblocks = (n + 255) / 256;
    quantize_u8_from_scratch_kernel<<<(uint32_t)(qblocks < 2368 ? qblocks : 2368), 256, 0, st>>>(data, n, q, scratch);
    count_launch(2);
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}
