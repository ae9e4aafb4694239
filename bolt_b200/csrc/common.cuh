// common.cuh -- internal declarations shared by the .cu files of libbolt_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <map>
#include <mutex>
#include <vector>

#include "bolt_b200.h"

namespace b200 {

#define B200_ALIGN(x, a) ((((x) + (a)-1) / (a)) * (a))

// ---- device-side exact arithmetic ----------------------------------------------------------
// The reference computes every float step as a separate IEEE binary32 instruction (vcvtdq2ps,
// vmulps, vaddps, vcvtps2dq); the helpers below use the _rn intrinsics so that nvcc cannot
// contract a multiply and an add into one fused operation.

// vcvtps2dq: round to nearest even; NaN and |f| >= 2^31 give 0x80000000.
__device__ __forceinline__ int cvt_rne_x86(float f)
{
    return (f >= -2147483648.0f && f < 2147483648.0f) ? __float2int_rn(f) : (int)0x80000000;
}
// vpmovusdb: the dword is read as unsigned, then clamped to 255.
__device__ __forceinline__ uint32_t usat8_x86(int v)
{
    return min((uint32_t)v, 255u);
}
// vpmovsdb
__device__ __forceinline__ int ssat8_x86(int v)
{
    return max(-128, min(127, v));
}
// GEMM / GEMV / conv u8 epilogue: vcvtdq2ps, vmulps, vcvtps2dq, vpaddd 128, vpmovusdb.
__device__ __forceinline__ uint32_t acc_to_u8(int acc, float factor)
{
    float f = __fmul_rn(__int2float_rn(acc), factor);
    // __float2int_rn saturates where vcvtps2dq returns 0x80000000; after +128 both land above
    // 255 as unsigned, except NaN (0 here), which is mapped by hand.
    int r = (f != f) ? (int)0x80000000 : __float2int_rn(f);
    return usat8_x86((int)((uint32_t)r + 128u));
}
__device__ __forceinline__ float acc_to_f32(int acc, float factor)
{
    return __fmul_rn(__int2float_rn(acc), factor);
}

// ---- per-device state ------------------------------------------------------------------------
struct WeightTwin {
    void *dev;
    size_t bytes;
};

// kernel families whose dynamic shared-memory limit has to be raised above 48 KiB; the attribute
// belongs to the device that is current when it is set, so it is remembered per device context
enum KernelFamily { KF_GEMM = 0, KF_CONV, KF_CONV_HALF, KF_GEMV, KF_GEMV_ROW, KF_BNN, KF_PROBE, KF_COUNT };

struct DeviceCtx {
    int device = 0;
    bool smem_raised[KF_COUNT] = {};
    std::mutex attr_mu;
    int max_pairs = -1;  // co-resident 2-CTA clusters of the tensor-core GEMM (-1: not queried yet)
    int sm_count = 148;
    int *d_status = nullptr;      // device-side error word
    void *d_scatter_maps = nullptr;  // 8 tensor maps of a scatter GEMM (allocated on first use)
    float *d_scratch = nullptr;   // small device scratch for reductions (absmax etc.)
    unsigned *d_scratch_u = nullptr;
    std::mutex mu;       // guards the staging workspace (one staged call at a time)
    std::mutex twin_mu;  // guards twins
    std::mutex scratch_mu;  // guards d_scratch between a reduction and its read-back
    std::map<const void *, WeightTwin> twins;  // host packed weight -> device copy
    // growable staging workspace for host-pointer calls
    char *ws = nullptr;
    size_t ws_bytes = 0;
    size_t ws_used = 0;
};

struct ThreadState {
    int device = -1;  // -1: not chosen through bolt_b200_set_device -- follow the thread's current CUDA device
    cudaStream_t stream = nullptr;
    bool device_only = false;
    int last_gemm_tc = 0;
};

DeviceCtx *ctx();          // context of the calling thread's device (created on first use)
ThreadState &tls();
extern std::atomic<uint64_t> g_launches;
inline void count_launch(int n = 1)
{
    g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed);
}

// cudaFuncAttributeMaxDynamicSharedMemorySize for every kernel of a family, once per device
// (the calling thread's device must be current, which ctx() guarantees)
EE raise_smem_limit(DeviceCtx *c, KernelFamily f, const void *const *kernels, int n, size_t bytes);

// true if p is memory the GPU can dereference (device or managed)
bool is_device_ptr(const void *p);
// true if p is plain device memory of a GPU other than the one this thread's calls run on
bool on_other_device(const void *p);

// Staging helper for one call: maps caller pointers to device pointers.  Host inputs are
// copied into the workspace; host outputs get a workspace buffer that finish() copies back.
class Stage {
public:
    Stage();
    ~Stage();
    // input: returns a device pointer holding `bytes` bytes of p
    const void *in(const void *p, size_t bytes);
    // output (optionally preloaded with the host content when `also_in`)
    void *out(void *p, size_t bytes, bool also_in = false);
    // device scratch that lives until finish()
    void *scratch(size_t bytes);
    // copy outputs back; synchronises the stream if anything was staged
    EE finish();
    bool any_host() const
    {
        return any_host_;
    }

private:
    struct Out {
        void *host;
        void *dev;
        size_t bytes;
    };
    std::vector<Out> outs_;
    std::vector<void *> big_;  // direct allocations that did not fit the workspace
    bool any_host_ = false;
    bool locked_ = false;
    void *alloc(size_t bytes);
};

EE cuda_ee(cudaError_t e);
#define B200_CUDA(call)                    \
    do {                                   \
        cudaError_t _e = (call);           \
        if (_e != cudaSuccess) {           \
            return ::b200::cuda_ee(_e);    \
        }                                  \
    } while (0)
#define B200_EE(call)          \
    do {                       \
        EE _s = (call);        \
        if (_s != SUCCESS) {   \
            return _s;         \
        }                      \
    } while (0)

// cuTensorMapEncodeTiled (found through the runtime's driver entry point) for byte tensors of
// rank <= 5; zero fill out of range.  `map` points at a CUtensorMap.
bool tensor_map_encoder_available();
bool encode_tiled_u8(void *map, uint32_t rank, const void *base, const uint64_t *dims, const uint64_t *strides,
    const uint32_t *box, const uint32_t *elem_strides, int swizzle_bytes /* 0, 32, 64 or 128 */);

// ---- kernel launchers (device pointers only) ----------------------------------------------
struct GemmEpilogue {
    int out_kind;              // 0 int32, 1 fp32, 2 u8
    int accumulate;            // add incoming int32 bits of C (kinds 0, 1)
    const int32_t *offsetC;    // [N] or null
    float factor;              // used when per_channel == 0
    int per_channel;           // 1: factor = num / (sA[m] * sB[n])
    float num, sA, sB;
    const float *sA_dev;       // device scalar overriding sA, or null
    const float *row_scale;    // [M] or null
    const float *col_scale;    // [N] or null
    const float *col_factor;   // [N] or null: ready-made per-column factors (then nothing is divided in the kernel)
    const void *prefetch;      // device memory a later call will read (the next layer's weight), or null:
    size_t prefetch_bytes;     // brought into L2 while this GEMM runs
    // u8 output stored into scatter_n matrices [M][scatter_ld] (this GPU's and its peers') at column scatter_col0
    void *scatter_dst[8];
    uint32_t scatter_n, scatter_ld, scatter_col0;
};

// B: ALIGN(N,16) rows, pitch Kp = ALIGN(K,8) bytes, K contiguous, zero padded.
EE launch_gemm_tcgen05(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, const int8_t *B,
    uint32_t Kp, void *C, const GemmEpilogue &ep, cudaStream_t st);
bool gemm_tcgen05_eligible(uint32_t M, uint32_t N, uint32_t K, const void *A, const void *B,
    uint32_t Kp, bool a_transposed);
EE launch_gemm_simt(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, bool a_transposed,
    const int8_t *B, uint32_t Kp, void *C, const GemmEpilogue &ep, cudaStream_t st);
EE launch_pack_rhs(const int8_t *src, bool src_is_nk, uint32_t N, uint32_t K, int8_t *dst,
    uint32_t Kp, uint32_t Np, int32_t *offsetC, cudaStream_t st);
EE launch_gemv_row(uint32_t N, uint32_t K, const uint8_t *Mx, bool transposed, const int8_t *v, void *y, int out_kind,
    float factor, cudaStream_t st);
EE launch_gemv(uint32_t N, uint32_t K, const int8_t *W, uint32_t Kp, const uint8_t *x,
    const int32_t *offsetC, void *y, int out_kind, float factor, cudaStream_t st);

}  // namespace b200
