// conv_i8.cu -- int8 convolution as an implicit GEMM on the sm_100a tensor cores.
//
//   acc[n,oc,oh,ow] = offsetC[oc] + round(bias[oc]*scaleO) + sum_{ic,kh,kw} W_s8 * X_u8(pad = 128)
//
// Replaces Bolt's AVX512 direct and 1x1 convolution kernels and their drivers
// (compute/tensor/src/cpu/x86/int8/avx512/convolution_direct.cpp:2584-2809,
//  convolution_1x1_direct.cpp:2073-2327), the filter transform
// (cpu/x86/int8/convolution_transform.cpp:18-238), the bias / offset fold
// (cpu/x86/quantize.cpp:64-121) and the input pad / relayout (cpu/x86/int8/transform_functions_int8.h:19-224).
//
// GEMM view: M = output pixels, N = output channels, K = (kh, kw, input-channel block of 16).  A tile is a
// TW x TH patch of TN images (at most 128 pixels).  On a channels-of-16 tensor [N][IC/16][H][W][16] a
// 16-byte K chunk of such a tile is one TMA box -- element strides carry the convolution stride, the start
// coordinates carry (kh, kw) and the padding -- and lands in shared memory as 8-row x 16-byte core
// matrices, the un-swizzled K-major operand layout of tcgen05.mma.  No im2col buffer ever exists.
//
// Padding without a padded copy: taps outside the image are filled with 0 by TMA where the reference
// fills 128, so   offsetC + sum_all W*X(pad 128)  =  sum_valid W*X - 128 * sum_valid W.   The filter
// transform leaves per-tap weight sums behind the packed filter; the pixels of a tile fall into a few
// border classes (which kh, which kw are inside), and the epilogue adds the offset of its pixel's class.
// Integer arithmetic, so the result is the reference's bit for bit.  Inputs that are not NCHWc16 with
// a multiple of 16 channels are first brought to that layout (pad value 128, one streaming pass).
//
// 1x1 / stride 1 / unpadded layers are run as images of one row of H*W pixels: tiles of 16 pixels x 8
// images fill all 128 rows and move 256 contiguous bytes per TMA row.
//
// The bias / offset fold (round(bias*scaleO) + offsetC) and the conversion factors (one per tensor, or
// one per output channel) are computed by the epilogue warps when they stage a column block's
// constants; one launch per call.  Weights are pre-packed [OC][K] and loaded like the GEMM's B operand
// (128-byte swizzle).  Warp roles, the tensor-memory double buffering and the bounded waits are those of
// gemm_i8_tcgen05.cu.
#include <cstring>

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int MAX_BLOCK_N = 256;
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int NUM_THREADS = 64 + EPI_THREADS;
constexpr int SMEM_A_STAGE = BLOCK_M * BLOCK_K;      // 8 K-chunks x 128 pixels x 16 B
constexpr int MAX_CLASSES = 16;                      // border classes of a layer (3 x 3 pad 1: 9)
constexpr int MAX_AXIS_CLASSES = 8;

// Two configurations of the kernel.  NB = 256: column blocks of up to 256 channels, four pipeline stages, all of
// tensor memory and shared memory -- one CTA per SM.  NB = 128: column blocks of up to 128 channels, three
// stages, half of tensor memory and less than half of shared memory, so that two CTAs share an SM: the layers
// with few input channels or few pixels spend their time in latencies (first load, tensor-memory read, stores)
// that a second resident CTA covers.
template <int NB>
struct Cfg {
    static constexpr int MAX_N = NB;
    static constexpr int STAGES = NB == 256 ? 4 : 3;
    static constexpr uint32_t TMEM_COLS = 2 * NB;        // two accumulators
    static constexpr int SMEM_B_STAGE = NB * BLOCK_K;
    static constexpr int CLASS_PITCH = NB + 4;           // int32 per class row; +4 staggers the banks of different classes
    static constexpr int CTAS_PER_SM = NB == 256 ? 1 : 2;
};

template <int NB>
struct __align__(16) SmemCtl {
    uint64_t full[Cfg<NB>::STAGES];
    uint64_t empty[Cfg<NB>::STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    // constants of the column block being worked on: per border class the offset of every channel
    // (offsetC-like term + round(bias * scaleO)), and the conversion factor of every channel
    __align__(16) int32_t offs[MAX_CLASSES * Cfg<NB>::CLASS_PITCH];
    __align__(16) float colf[NB];
};

template <int NB>
constexpr size_t smem_bytes()
{
    return 1024 + (size_t)Cfg<NB>::STAGES * (SMEM_A_STAGE + Cfg<NB>::SMEM_B_STAGE) + sizeof(SmemCtl<NB>);
}

struct ConvParams {
    uint32_t N, OH, OW, OC;
    uint32_t TW, TH, TN, tiles_w, tiles_h, tiles_n_img;   // tile = TW x TH pixels of TN images
    uint32_t rows;          // TW * TH * TN <= 128: pixels of a tile = rows of the A operand
    uint32_t ICb, FW, FH;
    uint32_t sH, sW, dH, dW;
    int32_t pt, pl;         // padding folded into the TMA start coordinates (0 when the input was copied padded)
    uint32_t G;             // K chunks per TMA load: divides both ICb and 8
    uint32_t merged_w;      // 1: stride-1 rows, (c16, w) merged into one byte dimension
    uint32_t total_chunks;  // taps * ICb
    uint32_t num_kb;        // ceil(total_chunks / 8)
    uint32_t block_n, tiles_n, tiles_m;
    void *out;
    const float *eltwise;
    const int32_t *offsetC; // [OC]: -128 * sum of the filter
    const int32_t *tapsum;  // [OC][taps]: sum over input channels of every tap (border classes), or null
    const float *bias;      // [OC] or null
    const float *fscale;    // [OC] per-output-channel filter scales, or null (then sF)
    float sI, sF, num;      // scaleO = sI * sF; factor = num / scaleO (num 1: fp32 out; output scale: fused u8)
    int relu;
    int *status;
    // border classes: class = row_class * n_cc + col_class; class 0 has every tap inside
    uint32_t n_rc, n_cc;
    uint8_t rc_lo[MAX_AXIS_CLASSES], rc_hi[MAX_AXIS_CLASSES];   // valid kh range [lo, hi] of a row class
    uint8_t cc_lo[MAX_AXIS_CLASSES], cc_hi[MAX_AXIS_CLASSES];
    uint8_t row_class[256], col_class[256];                      // per output row / column
};

// KIND 1: fp32 output (dequantize, + eltwise, ReLU).  KIND 0: int32 output after ReLU, the staging
// buffer of the dynamic u8 path (convolution_direct.cpp:2689-2693).  KIND 2: u8 output with a known
// output scale, the arithmetic of quantizeI32ToU8 with both scales given (avx512/quantize.cpp:372-414:
// vcvtdq2ps, vmulps, vaddps 128, vcvtps2dq, vpmovusdb) fused behind the ReLU.
template <int KIND>
__device__ __forceinline__ void store_block16(const ConvParams &p, const int32_t *offs, const float *colf, size_t base,
    uint32_t width, const uint32_t *r /*16 accumulators*/)
{
    if (KIND == 2) {
        uint8_t *out = reinterpret_cast<uint8_t *>(p.out) + base;
        uint32_t w[4];
        // Adding 1.5 * 2^23 rounds f to an integer (nearest even) in the low mantissa bits: the word is
        // 0x4B400000 + rne(f), and while 0 <= rne(f) <= 255 its low byte is the result.  `seen` collects the
        // other bits of all 16 words; anything left there (rare: the output scale does not fit the data)
        // sends the block through the clamp -- negatives wrap above 255 like vpmovusdb reads them.
        const int floor_v = p.relu ? 0 : (int)0x80000000;
        uint32_t bits[16];
        uint32_t seen = 0;
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            const int4 o = *reinterpret_cast<const int4 *>(offs + j);
            const float4 c4 = *reinterpret_cast<const float4 *>(colf + j);
            const float cf[4] = {c4.x, c4.y, c4.z, c4.w};
            const int v[4] = {(int)r[j] + o.x, (int)r[j + 1] + o.y, (int)r[j + 2] + o.z, (int)r[j + 3] + o.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float f = __fadd_rn(__fmul_rn(__int2float_rn(max(v[t], floor_v)), cf[t]), 128.0f);
                bits[j + t] = __float_as_uint(__fadd_rn(f, 12582912.0f));
                seen |= bits[j + t] ^ 0x4B400000u;
            }
            w[j >> 2] = __byte_perm(__byte_perm(bits[j], bits[j + 1], 0x0040), __byte_perm(bits[j + 2], bits[j + 3], 0x0040), 0x5410);
        }
        if (seen > 255u) {
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
                uint32_t b[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    b[t] = min(bits[j + t] - 0x4B400000u, 255u);
                }
                w[j >> 2] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
            }
        }
        if (width == 16) {
            *reinterpret_cast<uint4 *>(out) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            *reinterpret_cast<uint2 *>(out) = make_uint2(w[0], w[1]);
        }
    } else if (KIND == 1) {
        float *out = reinterpret_cast<float *>(p.out) + base;
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            if ((uint32_t)j < width) {
                const int4 o = *reinterpret_cast<const int4 *>(offs + j);
                const float4 c4 = *reinterpret_cast<const float4 *>(colf + j);
                float4 v = make_float4(acc_to_f32((int)r[j] + o.x, c4.x), acc_to_f32((int)r[j + 1] + o.y, c4.y),
                    acc_to_f32((int)r[j + 2] + o.z, c4.z), acc_to_f32((int)r[j + 3] + o.w, c4.w));
                if (p.eltwise != nullptr) {
                    const float4 e = *reinterpret_cast<const float4 *>(p.eltwise + base + j);
                    v.x = __fadd_rn(v.x, e.x);
                    v.y = __fadd_rn(v.y, e.y);
                    v.z = __fadd_rn(v.z, e.z);
                    v.w = __fadd_rn(v.w, e.w);
                }
                if (p.relu) {
                    v.x = v.x > 0.f ? v.x : 0.f;
                    v.y = v.y > 0.f ? v.y : 0.f;
                    v.z = v.z > 0.f ? v.z : 0.f;
                    v.w = v.w > 0.f ? v.w : 0.f;
                }
                *reinterpret_cast<float4 *>(out + j) = v;
            }
        }
    } else {
        int32_t *out = reinterpret_cast<int32_t *>(p.out) + base;
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            if ((uint32_t)j < width) {
                const int4 o = *reinterpret_cast<const int4 *>(offs + j);
                int4 v = make_int4((int)r[j] + o.x, (int)r[j + 1] + o.y, (int)r[j + 2] + o.z, (int)r[j + 3] + o.w);
                if (p.relu) {
                    v.x = max(v.x, 0);
                    v.y = max(v.y, 0);
                    v.z = max(v.z, 0);
                    v.w = max(v.w, 0);
                }
                *reinterpret_cast<int4 *>(out + j) = v;
            }
        }
    }
}

template <int KIND, int NB>
__global__ void __launch_bounds__(NUM_THREADS, Cfg<NB>::CTAS_PER_SM)
conv_u8s8_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    const __grid_constant__ ConvParams p)
{
    using CF = Cfg<NB>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + CF::STAGES * SMEM_A_STAGE;
    SmemCtl<NB> *ctl = reinterpret_cast<SmemCtl<NB> *>(smem + CF::STAGES * (SMEM_A_STAGE + CF::SMEM_B_STAGE));

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t chunk_bytes = p.rows * 16;   // one 16-byte K chunk of all the tile's pixels
    // distance between K chunks in shared memory: TMA destinations are 128-byte aligned, so a tile whose pixel
    // count is not a multiple of 8 gets one load per chunk (G = 1) at a rounded-up distance
    const uint32_t chunk_stride = ((p.rows + 7u) & ~7u) * 16;

    // programmatic dependent launch: the next kernel of the stream may begin its own set-up while this one runs;
    // this kernel touches no global memory before griddepcontrol.wait (the previous kernel has then completed)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
        for (int s = 0; s < CF::STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&ctl->tmem_full[a], 1);
            mbar_init(&ctl->tmem_empty[a], EPI_WARPS);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctl->tmem_base)),
                     "r"(CF::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // tile -> (first image, patch origin, first output channel)
    auto decode = [&](uint32_t tile, uint32_t &n, uint32_t &oh0, uint32_t &ow0, uint32_t &n0) {
        const uint32_t mt = tile % p.tiles_m;
        n0 = (tile / p.tiles_m) * p.block_n;
        const uint32_t per_grp = p.tiles_w * p.tiles_h;
        const uint32_t g = mt / per_grp;
        n = g * p.TN;
        const uint32_t r = mt - g * per_grp;
        oh0 = (r / p.tiles_w) * p.TH;
        ow0 = (r % p.tiles_w) * p.TW;
    };

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                uint32_t n, oh0, ow0, n0;
                decode(tile, n, oh0, ow0, n0);
                for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t q0 = kb * 8;
                    const uint32_t nq = min(8u, p.total_chunks - q0);
                    mbar_expect_tx(&ctl->full[stage], nq * chunk_bytes + p.block_n * BLOCK_K);
                    for (uint32_t j = 0; j < nq; j += p.G) {
                        const uint32_t q = q0 + j;
                        const uint32_t tap = q / p.ICb;
                        const uint32_t cb = q - tap * p.ICb;
                        const uint32_t kh = tap / p.FW, kw = tap - kh * p.FW;
                        uint8_t *dst = smem_a + stage * SMEM_A_STAGE + j * chunk_stride;
                        // taps outside the image start at negative or too large coordinates and read zeros
                        const int x = (int)(ow0 * p.sW + kw * p.dW) - p.pl;
                        const int y = (int)(oh0 * p.sH + kh * p.dH) - p.pt;
                        if (p.merged_w) {
                            // a row of TW pixels is TW * 16 contiguous bytes: one wide request per row
                            tma_load_4d(&map_x, &ctl->full[stage], dst, x * 16, y, (int)n, (int)cb);
                        } else {
                            tma_load_5d(&map_x, &ctl->full[stage], dst, 0, x, y, (int)n, (int)cb);
                        }
                    }
                    tma_load_2d(&map_w, &ctl->full[stage], smem_b + stage * CF::SMEM_B_STAGE, (int)(kb * BLOCK_K), (int)n0);
                    if (++stage == CF::STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                atomicExch(p.status, 11);
                atomicExch(&ctl->abort_flag, 1u);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_i8(p.block_n);
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * CF::MAX_N;
                for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->full[stage], phase)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t nq = min(8u, p.total_chunks - kb * 8);
                    const uint32_t a_addr = smem_u32(smem_a + stage * SMEM_A_STAGE);
                    const uint64_t db = make_desc_sw128(smem_u32(smem_b + stage * CF::SMEM_B_STAGE));
                    for (uint32_t k = 0; 2 * k < nq; ++k) {
                        // A: two 16-byte K chunks per MMA, chunk_stride apart; 8-pixel groups 128 B apart.  Rows
                        // beyond the tile's pixels read the next chunk's bytes: their accumulators are never
                        // stored.  An odd last chunk pairs with stale bytes, which meet zero weights.
                        const uint64_t da = make_desc_noswizzle(a_addr + k * 2 * chunk_stride, chunk_stride, 128);
                        umma_i8(tmem_d, da, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(&ctl->empty[stage]);
                    if (++stage == CF::STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    break;
                }
                tcgen05_commit(&ctl->tmem_full[acc]);
            }
            if (!ok) {
                atomicExch(p.status, 12);
                atomicExch(&ctl->abort_flag, 1u);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------- epilogue warps 2..9 ------------------------------------
        const uint32_t quad = warp & 3;
        const uint32_t half = (warp - 2) >> 2;
        const uint32_t et = threadIdx.x - 64;
        const uint32_t nch = p.block_n >> 5;
        const uint32_t n_classes = p.n_rc * p.n_cc;
        const uint32_t taps = p.FH * p.FW;
        const uint32_t c_begin = half ? ((nch + 1) >> 1) : 0u;
        const uint32_t c_end = half ? nch : ((nch + 1) >> 1);
        uint32_t staged_n0 = 0xFFFFFFFFu;
        uint32_t it = 0;
        // this lane's pixel inside a tile (the same for every tile): image, row and column offsets
        const uint32_t px_r = quad * 32 + lane;
        const uint32_t px_per_img = p.TH * p.TW;
        const uint32_t px_nl = px_r / px_per_img;
        const uint32_t px_rem = px_r - px_nl * px_per_img;
        const uint32_t px_th = px_rem / p.TW;
        const uint32_t px_tw = px_rem - px_th * p.TW;
        // After a bounded wait ran out somewhere the warp keeps walking the tiles without touching them:
        // the named barriers below have to be reached by every epilogue warp the same number of times.
        bool dead = false;
        for (uint32_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            uint32_t n_first, oh0, ow0, n0;
            decode(tile, n_first, oh0, ow0, n0);
            if (*reinterpret_cast<volatile uint32_t *>(&ctl->abort_flag) != 0) {
                dead = true;
            }
            if (n0 != staged_n0) {
                // Constants of this column block (tiles run row-block fastest, so this happens tiles_n times
                // per CTA): conversion factor and, per border class, the integer offset of every channel.
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");  // everyone is done with the old ones
                for (uint32_t j = et; !dead && j < p.block_n; j += EPI_THREADS) {
                    const uint32_t oc = n0 + j;
                    float factor = 0.f;
                    int boff = 0;
                    if (oc < p.OC) {
                        // scaleO = scaleI * scaleF (convolution_direct.cpp:2687), factor = 1 / scaleO (:2699)
                        const float so = __fmul_rn(p.sI, p.fscale ? p.fscale[oc] : p.sF);
                        factor = __fdiv_rn(p.num, so);
                        if (p.bias != nullptr) {
                            boff = (int)roundf(__fmul_rn(p.bias[oc], so));  // avx512/quantize.cpp:259-266
                        }
                    }
                    ctl->colf[j] = factor;
                    for (uint32_t cls = 0; cls < n_classes; ++cls) {
                        int v = 0;
                        if (oc < p.OC) {
                            if (cls == 0) {
                                v = p.offsetC[oc];
                            } else {
                                const uint32_t rc = cls / p.n_cc, cc = cls - rc * p.n_cc;
                                int sum = 0;
                                for (uint32_t kh = p.rc_lo[rc]; kh <= p.rc_hi[rc] && kh < p.FH; ++kh) {
                                    for (uint32_t kw = p.cc_lo[cc]; kw <= p.cc_hi[cc] && kw < p.FW; ++kw) {
                                        sum += p.tapsum[(size_t)oc * taps + kh * p.FW + kw];
                                    }
                                }
                                v = -128 * sum;
                            }
                        }
                        ctl->offs[cls * CF::CLASS_PITCH + j] = v + boff;
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                staged_n0 = n0;
            }
            dead = __any_sync(0xffffffffu, dead);
            if (dead) {
                continue;
            }
            bool ok = mbar_wait(&ctl->tmem_full[acc], acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) {
                    atomicExch(p.status, 13);
                    atomicExch(&ctl->abort_flag, 1u);
                }
                dead = true;
                continue;
            }
            tcgen05_fence_after();
            // this lane's pixel
            const uint32_t oh = oh0 + px_th;
            const uint32_t ow = ow0 + px_tw;
            const uint32_t n = n_first + px_nl;
            const bool row_ok = px_r < p.rows && n < p.N && oh < p.OH && ow < p.OW;
            const size_t pix = (size_t)oh * p.OW + ow;
            const size_t plane = (size_t)p.OH * p.OW;
            uint32_t cls = 0;
            if (row_ok && n_classes > 1) {
                cls = (uint32_t)p.row_class[oh] * p.n_cc + p.col_class[ow];
            }
            const int32_t *offs_px = ctl->offs + cls * CF::CLASS_PITCH;
            const uint32_t tbase = tmem_base + ((quad * 32u) << 16) + acc * CF::MAX_N;
            auto release = [&]() {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&ctl->tmem_empty[acc]);
                }
            };
            auto emit = [&](uint32_t c, const uint32_t *rr) {
                if (row_ok) {
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        const uint32_t col = c * 32 + hb * 16;
                        const uint32_t ocb = n0 + col;
                        if (ocb < p.OC) {
                            const uint32_t width = min(16u, p.OC - ocb);
                            const size_t base = ((size_t)n * p.OC + ocb) * plane + pix * width;
                            store_block16<KIND>(p, offs_px + col, ctl->colf + col, base, width, rr + hb * 16);
                        }
                    }
                }
            };
            // two register buffers: the next chunk is on its way from tensor memory while this one is
            // converted and stored; the accumulator is released as soon as its last chunk has arrived
            if (NB != 256) {
                // two CTAs per SM: the other CTA's warps cover the read latency, and the register budget of
                // a half SM leaves room for one buffer only
                uint32_t ra[32];
                for (uint32_t c = c_begin; c < c_end; ++c) {
                    tmem_ld32(tbase + c * 32, ra);
                    tmem_ld_wait(ra);
                    if (c + 1 == c_end) {
                        release();
                    }
                    emit(c, ra);
                }
                if (c_begin >= c_end) {
                    release();
                }
                continue;
            }
            uint32_t ra[32], rb[32];
            if (c_begin < c_end) {
                tmem_ld32(tbase + c_begin * 32, ra);
            }
            for (uint32_t c = c_begin; c < c_end; c += 2) {
                tmem_ld_wait(ra);
                const bool has1 = c + 1 < c_end;
                if (has1) {
                    tmem_ld32(tbase + (c + 1) * 32, rb);
                } else {
                    release();
                }
                emit(c, ra);
                if (has1) {
                    tmem_ld_wait(rb);
                    if (c + 2 < c_end) {
                        tmem_ld32(tbase + (c + 2) * 32, ra);
                    } else {
                        release();
                    }
                    emit(c + 1, rb);
                }
            }
            if (c_begin >= c_end) {
                release();
            }
        }
    }

    __syncthreads();
    if (ctl->abort_flag != 0) {
        for (int i = 0; i < 64; ++i) {
            __nanosleep(2000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(CF::TMEM_COLS)
                     : "memory");
    }
}

// ---- filter packing: s8 NCHW [OC][IC][FH][FW] -> [OCr][K], k = ((kh*FW + kw)*ICb + cb)*16 + c ------------
// offsetC[oc] = -128 * sum of the filter (convolution_transform.cpp: offsetC first, then the weights);
// tapsum[oc][tap] = sum over the input channels of one tap (what the border classes are built from).
__global__ void pack_conv_filter_kernel(const int8_t *__restrict__ src, uint32_t OC, uint32_t IC, uint32_t taps,
    uint32_t ICb, uint32_t OCr, int8_t *__restrict__ dst, int32_t *__restrict__ offsetC, int32_t *__restrict__ tapsum)
{
    const uint32_t oc = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (oc >= OCr) {
        return;
    }
    const uint32_t per_tap = ICb * 16;
    int32_t total = 0;
    for (uint32_t tap = 0; tap < taps; ++tap) {
        int32_t sum = 0;
        for (uint32_t i = lane; i < per_tap; i += 32) {
            int8_t v = 0;
            if (oc < OC && i < IC) {
                v = src[((size_t)oc * IC + i) * taps + tap];
            }
            dst[(size_t)oc * taps * per_tap + (size_t)tap * per_tap + i] = v;
            sum += v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (lane == 0 && oc < OC) {
            tapsum[(size_t)oc * taps + tap] = sum;
        }
        total += sum;
    }
    if (lane == 0 && oc < OC) {
        offsetC[oc] = total * (-128);
    }
}

// ---- input pad + relayout to [N][ICb][Hp][Wp][16], pad value 128 ------------------------------------------
// in_block: 16, 8 (channel-blocked) or 0 (plain NCHW).  One thread per 16-byte output chunk.
__global__ void pad_relayout_kernel(const uint8_t *__restrict__ in, uint32_t N, uint32_t IC, uint32_t IH, uint32_t IW,
    uint32_t in_block, uint32_t ICb, uint32_t Hp, uint32_t Wp, uint32_t pt, uint32_t pl, uint8_t *__restrict__ out)
{
    const size_t total = (size_t)N * ICb * Hp * Wp;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t x = (uint32_t)(i % Wp);
        const uint32_t y = (uint32_t)((i / Wp) % Hp);
        const uint32_t cb = (uint32_t)((i / ((size_t)Wp * Hp)) % ICb);
        const uint32_t n = (uint32_t)(i / ((size_t)Wp * Hp * ICb));
        uint4 v = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
        const int iy = (int)y - (int)pt, ix = (int)x - (int)pl;
        if (iy >= 0 && iy < (int)IH && ix >= 0 && ix < (int)IW) {
            const size_t pix = (size_t)iy * IW + ix;
            const size_t img = (size_t)n * IC * IH * IW;
            if (in_block == 16 && cb * 16 + 16 <= IC) {
                v = *reinterpret_cast<const uint4 *>(in + img + ((size_t)cb * 16) * IH * IW + pix * 16);
            } else if (in_block == 8 && (IC % 8) == 0) {
                const uint32_t c0 = cb * 16;
                const uint2 lo = *reinterpret_cast<const uint2 *>(in + img + (size_t)c0 * IH * IW + pix * 8);
                v.x = lo.x;
                v.y = lo.y;
                if (c0 + 8 < IC) {
                    const uint2 hi = *reinterpret_cast<const uint2 *>(in + img + (size_t)(c0 + 8) * IH * IW + pix * 8);
                    v.z = hi.x;
                    v.w = hi.y;
                }
            } else {
                // generic: channel-blocked with a narrower tail block, or plain NCHW
                uint32_t w[4] = {0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u};
                for (uint32_t c = 0; c < 16; ++c) {
                    const uint32_t ic = cb * 16 + c;
                    if (ic < IC) {
                        size_t off;
                        if (in_block == 0) {
                            off = img + (size_t)ic * IH * IW + pix;
                        } else {
                            const uint32_t b = ic / in_block;
                            const uint32_t width = min(in_block, IC - b * in_block);
                            off = img + (size_t)b * in_block * IH * IW + pix * width + (ic - b * in_block);
                        }
                        w[c >> 2] = (w[c >> 2] & ~(0xFFu << (8 * (c & 3)))) | ((uint32_t)in[off] << (8 * (c & 3)));
                    }
                }
                v = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        reinterpret_cast<uint4 *>(out)[i] = v;
    }
}

struct Conv4d {
    DataType dt;
    DataFormat df;
    uint32_t n, c, h, w;
};
bool get4d(const TensorDesc *d, Conv4d *o)
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

uint32_t pick_conv_block_n(uint32_t tiles_m, uint32_t OC, int sms, uint32_t max_bn = 256)
{
    uint32_t best = 32;
    double best_cost = 1e30;
    for (uint32_t bn = max_bn; bn >= 32; bn -= 32) {
        if (bn > B200_ALIGN(OC, 32) && bn != 32) {
            continue;
        }
        const uint64_t tiles = (uint64_t)tiles_m * ((OC + bn - 1) / bn);
        const uint64_t waves = (tiles + sms - 1) / sms;
        const double cost = (double)waves * (bn + 48.0);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

// Two CTAs per SM pay where a tile is short and narrow: at most 64 output channels, or at most 128 behind a K
// of one or two blocks.  Measured on the 22 ResNet-50-shaped layers at batch 64 (u8 output): 3x3 64->64 @56
// 38.9 -> 28.3 us, 1x1 256->128 @56 28.7 -> 25.0 us, 1x1 64->64 and 256->64 @56 22.5 -> 20.5 us; wider or longer
// layers lose (3x3 512->512 @14 s2 32.8 -> 51.2 us), the 256-wide tile reads the activations half as often.
bool conv_prefers_half(uint32_t tiles_m, uint32_t OC, uint32_t num_kb, int sms)
{
    (void)tiles_m;
    (void)sms;
    return OC <= 64 || (OC <= 128 && num_kb <= 2);
}

struct ConvGeom {
    Conv4d in, f, out;
    uint32_t sH, sW, dH, dW, pt, pb, pl, pr;
    uint32_t ICb, Hp, Wp, taps, K, OCr;
    bool needs_copy;     // the input has to be brought to the padded channels-of-16 layout first
    size_t xp_bytes;
};

// Border classes along one axis: output positions grouped by the range of filter taps that fall inside
// the image.  Returns the number of classes (class 0 = every tap inside), 0 if there are too many or
// some position has no tap inside at all.
uint32_t axis_classes(uint32_t out_len, uint32_t in_len, uint32_t f, uint32_t stride, uint32_t dil, uint32_t pad,
    uint8_t *lo, uint8_t *hi, uint8_t *cls_of)
{
    if (out_len > 256 || f > 255) {
        return 0;
    }
    uint32_t n = 1;
    lo[0] = 0;
    hi[0] = (uint8_t)(f - 1);
    for (uint32_t o = 0; o < out_len; ++o) {
        int first = -1, last = -1;
        for (uint32_t k = 0; k < f; ++k) {
            const long pos = (long)o * stride + (long)k * dil - (long)pad;
            if (pos >= 0 && pos < (long)in_len) {
                if (first < 0) {
                    first = (int)k;
                }
                last = (int)k;
            }
        }
        if (first < 0) {
            return 0;
        }
        // the taps inside must be one contiguous range (they are: positions grow with k)
        uint32_t c = 0;
        for (; c < n; ++c) {
            if (lo[c] == first && hi[c] == last) {
                break;
            }
        }
        if (c == n) {
            if (n == MAX_AXIS_CLASSES) {
                return 0;
            }
            lo[n] = (uint8_t)first;
            hi[n] = (uint8_t)last;
            ++n;
        }
        cls_of[o] = (uint8_t)c;
    }
    return n;
}

EE conv_geometry(const TensorDesc *inputDesc, const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *cp, ConvGeom *g)
{
    if (!get4d(inputDesc, &g->in) || !get4d(filterDesc, &g->f) || !get4d(outputDesc, &g->out) || cp == nullptr) {
        return NOT_MATCH;
    }
    if (cp->group != 1) {
        return NOT_SUPPORTED;
    }
    g->sH = cp->stride_h ? cp->stride_h : 1;
    g->sW = cp->stride_w ? cp->stride_w : 1;
    g->dH = cp->dilatedRate_h ? cp->dilatedRate_h : 1;
    g->dW = cp->dilatedRate_w ? cp->dilatedRate_w : 1;
    g->pt = cp->pad_top;
    g->pb = cp->pad_bottom;
    g->pl = cp->pad_left;
    g->pr = cp->pad_right;
    g->ICb = (g->f.c + 15) / 16;
    g->Hp = g->in.h + g->pt + g->pb;
    g->Wp = g->in.w + g->pl + g->pr;
    g->taps = g->f.h * g->f.w;
    g->K = g->taps * g->ICb * 16;
    g->OCr = B200_ALIGN(g->f.n, 8);
    // the output geometry must be the one the input, filter and padding give (convolution.cpp:60-66)
    const uint32_t eh = (g->f.h - 1) * g->dH + 1, ew = (g->f.w - 1) * g->dW + 1;
    if (g->Hp < eh || g->Wp < ew || g->out.n != g->in.n || g->out.h != (g->Hp - eh) / g->sH + 1 ||
        g->out.w != (g->Wp - ew) / g->sW + 1) {
        return NOT_MATCH;
    }
    g->needs_copy = !(g->in.df == DF_NCHWC16 && (g->in.c % 16) == 0);
    g->xp_bytes = (size_t)g->in.n * g->ICb * g->Hp * g->Wp * 16;
    return SUCCESS;
}

struct ConvLaunch {
    const uint8_t *x;        // [N][ICb][H][W][16]
    uint32_t H, W;           // extents of x (padded extents after a padded copy)
    int32_t pt, pl;          // padding still to be applied through the TMA coordinates
    const int8_t *w;         // [OCr][K]
    const int32_t *offsetC, *tapsum;
    const float *bias, *fscale, *eltwise;
    float sI, sF, num;
    void *out;
    int out_kind, relu;
};

// Launch with programmatic stream serialization (the kernel's set-up overlaps the tail of the previous kernel);
// if the attribute is refused outside a stream capture, launch without it from then on.
std::atomic<int> g_conv_pdl{-1};
template <int KIND, int NB>
cudaError_t launch_conv_kernel(uint32_t grid, cudaStream_t st, const CUtensorMap &mx, const CUtensorMap &mw, const ConvParams &p)
{
    int pdl = g_conv_pdl.load(std::memory_order_relaxed);
    if (pdl < 0) {
        const char *e = getenv("BOLT_B200_NO_PDL");
        pdl = (e != nullptr && e[0] != '\0' && e[0] != '0') ? 0 : 1;
        g_conv_pdl.store(pdl, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem_bytes<NB>();
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, conv_u8s8_tcgen05_kernel<KIND, NB>, mx, mw, p);
    if (e != cudaSuccess && pdl) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(st, &cap);
        if (cap == cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            g_conv_pdl.store(0, std::memory_order_relaxed);
            cfg.numAttrs = 0;
            e = cudaLaunchKernelEx(&cfg, conv_u8s8_tcgen05_kernel<KIND, NB>, mx, mw, p);
        }
    }
    return e;
}

// run the implicit-GEMM kernel (all pointers device)
EE launch_conv_tcgen05(const ConvGeom &g, const ConvLaunch &a, cudaStream_t st)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    {
        const void *ks[3] = {(const void *)conv_u8s8_tcgen05_kernel<0, 256>, (const void *)conv_u8s8_tcgen05_kernel<1, 256>,
            (const void *)conv_u8s8_tcgen05_kernel<2, 256>};
        B200_EE(raise_smem_limit(c, KF_CONV, ks, 3, smem_bytes<256>()));
        const void *kh[3] = {(const void *)conv_u8s8_tcgen05_kernel<0, 128>, (const void *)conv_u8s8_tcgen05_kernel<1, 128>,
            (const void *)conv_u8s8_tcgen05_kernel<2, 128>};
        B200_EE(raise_smem_limit(c, KF_CONV_HALF, kh, 3, smem_bytes<128>()));
    }
    if (!tensor_map_encoder_available()) {
        return NOT_SUPPORTED;
    }
    ConvParams p;
    std::memset(&p, 0, sizeof(p));
    uint32_t N = g.in.n, OH = g.out.h, OW = g.out.w, H = a.H, W = a.W;
    const uint32_t OC = g.out.c, FH = g.f.h, FW = g.f.w;
    const uint32_t sH = g.sH, sW = g.sW;
    // border classes (only when padding is applied through the coordinates)
    p.n_rc = 1;
    p.n_cc = 1;
    p.rc_hi[0] = (uint8_t)(FH - 1);
    p.cc_hi[0] = (uint8_t)(FW - 1);
    if (a.pt != 0 || a.pl != 0 || g.pb != 0 || g.pr != 0) {
        if (a.pt != 0 || a.pl != 0 || H == g.in.h) {   // not a padded copy
            p.n_rc = axis_classes(OH, H, FH, sH, g.dH, (uint32_t)a.pt, p.rc_lo, p.rc_hi, p.row_class);
            p.n_cc = axis_classes(OW, W, FW, sW, g.dW, (uint32_t)a.pl, p.cc_lo, p.cc_hi, p.col_class);
            if (p.n_rc == 0 || p.n_cc == 0 || p.n_rc * p.n_cc > (uint32_t)MAX_CLASSES) {
                return NOT_SUPPORTED;  // the caller falls back to a padded copy
            }
        }
    }
    // 1x1, stride 1, nothing padded: every image is one row of H*W pixels
    if (FH == 1 && FW == 1 && sH == 1 && sW == 1 && p.n_rc == 1 && p.n_cc == 1 && a.pt == 0 && a.pl == 0 && OH == H &&
        OW == W) {
        // ... or, when the pixel count allows, rows of 16 pixels (256 contiguous bytes): a tile of 8 such rows is
        // 128 consecutive pixels of ONE image, 2 KiB contiguous per channel group, instead of 16 pixels of each
        // of 8 images -- longer runs per DRAM page when the input streams from HBM
        if ((H * W) % 16 == 0) {
            H = OH = H * W / 16;
            W = OW = 16;
        } else {
            W = OW = H * W;
            H = OH = 1;
        }
    }
    p.N = N;
    p.OH = OH;
    p.OW = OW;
    p.OC = OC;
    // Tile: TW x TH pixels of TN images, at most 128 in all; the shape that needs the fewest tiles, wider rows
    // first among equals.  With stride 1 along W a row of TW pixels is TW*16 contiguous bytes; the (c16, w)
    // dimensions are then merged so that TMA moves one 16*TW-byte run per row instead of TW 16-byte ones (a
    // TMA box is at most 256 elements wide, hence TW <= 16 on that path).
    // A tile whose pixel count is a multiple of 8 lets one TMA request bring all 8 channel groups of a
    // 128-byte K block (the groups then lie 128-byte aligned behind one another in shared memory); any other
    // count needs a request per group, eight times as many.  So such shapes are preferred even when they
    // overhang the image (TW may exceed OW by up to 7 columns: the overhang reads zeros and is not stored).
    const bool merged_w = (sW == 1);
    uint64_t best_tiles = ~0ull;
    uint32_t btw = 0, bth = 0, btn = 0;
    const uint32_t tw_max = merged_w ? 16u : 128u;
    const uint32_t ow8 = (uint32_t)B200_ALIGN(OW, 8);
    for (uint32_t tw = (ow8 < tw_max ? ow8 : tw_max); tw >= 1; --tw) {
        if (tw * sW > 256) {
            continue;
        }
        for (uint32_t th = (OH < 128 / tw ? OH : 128 / tw); th >= 1; --th) {
            if (th * sH > 256) {
                continue;
            }
            uint32_t tn = 128 / (tw * th);
            tn = tn < N ? tn : N;
            if (tn == 0) {
                continue;
            }
            uint64_t tiles = (uint64_t)((OW + tw - 1) / tw) * ((OH + th - 1) / th) * ((N + tn - 1) / tn);
            if ((tw * th * tn) % 8 != 0) {
                tiles *= 4;  // weight of the eightfold request count
            }
            if (tiles < best_tiles) {
                best_tiles = tiles;
                btw = tw;
                bth = th;
                btn = tn;
            }
        }
    }
    if (btw == 0) {
        return NOT_SUPPORTED;
    }
    p.TW = btw;
    p.TH = bth;
    p.TN = btn;
    p.rows = btw * bth * btn;
    p.tiles_w = (OW + p.TW - 1) / p.TW;
    p.tiles_h = (OH + p.TH - 1) / p.TH;
    p.tiles_n_img = (N + p.TN - 1) / p.TN;
    p.ICb = g.ICb;
    p.FW = FW;
    p.FH = FH;
    p.sH = sH;
    p.sW = sW;
    p.dH = g.dH;
    p.dW = g.dW;
    p.pt = a.pt;
    p.pl = a.pl;
    p.merged_w = merged_w ? 1 : 0;
    p.G = 8;
    while (g.ICb % p.G != 0) {
        p.G >>= 1;
    }
    if (p.rows % 8 != 0) {
        p.G = 1;  // chunks of a box follow each other without gaps; only whole 128-byte units may be merged
    }
    p.total_chunks = FH * FW * g.ICb;
    p.num_kb = (p.total_chunks + 7) / 8;
    p.tiles_m = p.tiles_n_img * p.tiles_w * p.tiles_h;
    // which configuration: two CTAs per SM with column blocks of at most 128 channels, or one with up to 256
    static const int force_half = [] {
        const char *e = getenv("BOLT_B200_CONV_HALF");
        return (e == nullptr || e[0] == '\0') ? -1 : atoi(e);
    }();
    const bool half_cfg = force_half >= 0 ? force_half != 0 : conv_prefers_half(p.tiles_m, OC, p.num_kb, c->sm_count);
    p.block_n = half_cfg ? pick_conv_block_n(p.tiles_m, OC, 2 * c->sm_count, 128) : pick_conv_block_n(p.tiles_m, OC, c->sm_count);
    p.tiles_n = (OC + p.block_n - 1) / p.block_n;
    p.out = a.out;
    p.eltwise = a.eltwise;
    p.offsetC = a.offsetC;
    p.tapsum = a.tapsum;
    p.bias = a.bias;
    p.fscale = a.fscale;
    p.sI = a.sI;
    p.sF = a.sF;
    p.num = a.num;
    p.relu = a.relu;
    p.status = c->d_status;

    // x as (c16, W, H, N, ICb): a box {.., TN, G} lands as [chunk][image][row][pixel][16 B]
    CUtensorMap map_x, map_w;
    const uint64_t img = (uint64_t)g.ICb * H * W * 16, plane = (uint64_t)H * W * 16;
    if (merged_w) {
        const uint64_t dims[4] = {(uint64_t)W * 16, H, N, g.ICb};
        const uint64_t strides[3] = {(uint64_t)W * 16, img, plane};
        const uint32_t box[4] = {p.TW * 16, p.TH * sH, p.TN, p.G};
        const uint32_t es[4] = {1, sH, 1, 1};
        if (!encode_tiled_u8(&map_x, 4, a.x, dims, strides, box, es, 0)) {
            return NOT_SUPPORTED;
        }
    } else {
        const uint64_t dims[5] = {16, W, H, N, g.ICb};
        const uint64_t strides[4] = {16, (uint64_t)W * 16, img, plane};
        const uint32_t box[5] = {16, p.TW * sW, p.TH * sH, p.TN, p.G};
        const uint32_t es[5] = {1, sW, sH, 1, 1};
        if (!encode_tiled_u8(&map_x, 5, a.x, dims, strides, box, es, 0)) {
            return NOT_SUPPORTED;
        }
    }
    {
        const uint64_t K = (uint64_t)p.total_chunks * 16;
        const uint64_t dims[2] = {K, g.OCr};
        const uint64_t strides[1] = {K};
        const uint32_t box[2] = {(uint32_t)BLOCK_K, p.block_n};
        const uint32_t es[2] = {1, 1};
        if (!encode_tiled_u8(&map_w, 2, a.w, dims, strides, box, es, 128)) {
            return NOT_SUPPORTED;
        }
    }
    const uint64_t tiles = (uint64_t)p.tiles_m * p.tiles_n;
    const uint64_t slots = (uint64_t)c->sm_count * (half_cfg ? 2 : 1);
    const uint32_t grid = (uint32_t)(tiles < slots ? tiles : slots);
    cudaError_t le;
    if (half_cfg) {
        le = a.out_kind == 2 ? launch_conv_kernel<2, 128>(grid, st, map_x, map_w, p)
                             : (a.out_kind == 1 ? launch_conv_kernel<1, 128>(grid, st, map_x, map_w, p)
                                                : launch_conv_kernel<0, 128>(grid, st, map_x, map_w, p));
    } else {
        le = a.out_kind == 2 ? launch_conv_kernel<2, 256>(grid, st, map_x, map_w, p)
                             : (a.out_kind == 1 ? launch_conv_kernel<1, 256>(grid, st, map_x, map_w, p)
                                                : launch_conv_kernel<0, 256>(grid, st, map_x, map_w, p));
    }
    count_launch();
    B200_CUDA(le);
    return SUCCESS;
}

// bytes of the packed filter: offsetC, weights, per-tap sums
size_t filter_weights_off(uint32_t fn)
{
    return 4 * (size_t)fn;
}
size_t filter_tapsum_off(uint32_t fn, uint32_t OCr, uint32_t K)
{
    return B200_ALIGN(4 * (size_t)fn + (size_t)OCr * K, 16);
}

}  // namespace

// ---- entry-point bodies for the int8 branch (called from conv.cu) ----------------------------------------
EE conv_i8_transform_filter_bytes(const TensorDesc *filterDesc, U32 *bytes)
{
    Conv4d f;
    if (!get4d(filterDesc, &f) || bytes == nullptr) {
        return NOT_MATCH;
    }
    // cpu/x86/convolution.cpp:141-166 counts ALIGN(fn,8) * ALIGN(fc,16) * fh * fw + 4*fn + 32; here the int32
    // sums of every (output channel, tap) follow the weights (4 * fn * fh * fw more bytes)
    const size_t b = filter_tapsum_off(f.n, B200_ALIGN(f.n, 8), B200_ALIGN(f.c, 16) * f.h * f.w) + 4 * (size_t)f.n * f.h * f.w + 32;
    if (b > 0xFFFFFFFFull) {
        return NOT_SUPPORTED;
    }
    *bytes = (U32)b;
    return SUCCESS;
}

EE conv_i8_transform_filter(const TensorDesc *filterDesc, const void *filter, TensorDesc *ftmDesc, void *dst)
{
    Conv4d f;
    if (!get4d(filterDesc, &f) || ftmDesc == nullptr) {
        return NOT_MATCH;
    }
    if (f.df == DF_NCHWC2NxC4) {
        *ftmDesc = *filterDesc;
        return SUCCESS;
    }
    if (f.df != DF_NCHW) {
        return NOT_SUPPORTED;
    }
    if (filter == nullptr || dst == nullptr) {
        return NULL_POINTER;
    }
    if ((f.n % 4) != 0) {
        return NOT_SUPPORTED;  // the weight matrix must start 16-byte aligned behind 4*fn bytes of offsetC
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    cudaStream_t st = tls().stream;
    const uint32_t ICb = (f.c + 15) / 16, taps = f.h * f.w, OCr = B200_ALIGN(f.n, 8);
    const uint32_t K = taps * ICb * 16;
    const size_t ts_off = filter_tapsum_off(f.n, OCr, K);
    const size_t total = ts_off + 4 * (size_t)f.n * taps;
    Stage sg;
    const int8_t *d_src = reinterpret_cast<const int8_t *>(sg.in(filter, (size_t)f.n * f.c * taps));
    if (d_src == nullptr) {
        return ALLOC_FAILED;
    }
    const bool dst_dev = is_device_ptr(dst);
    char *d_dst = reinterpret_cast<char *>(dst);
    if (!dst_dev) {
        void *twin = nullptr;
        B200_CUDA(cudaMalloc(&twin, B200_ALIGN(total, 256)));
        d_dst = reinterpret_cast<char *>(twin);
    }
    const int warps = 8;
    pack_conv_filter_kernel<<<(OCr + warps - 1) / warps, warps * 32, 0, st>>>(d_src, f.n, f.c, taps, ICb, OCr,
        reinterpret_cast<int8_t *>(d_dst + filter_weights_off(f.n)), reinterpret_cast<int32_t *>(d_dst),
        reinterpret_cast<int32_t *>(d_dst + ts_off));
    count_launch();
    EE ret = cuda_ee(cudaGetLastError());
    if (ret == SUCCESS && !dst_dev) {
        ret = cuda_ee(cudaMemcpyAsync(dst, d_dst, total, cudaMemcpyDeviceToHost, st));
    }
    if (ret == SUCCESS) {
        ret = sg.finish();
    }
    if (!dst_dev) {
        if (ret == SUCCESS) {
            ret = cuda_ee(cudaStreamSynchronize(st));
        }
        if (ret != SUCCESS) {
            cudaFree(d_dst);
            return ret;
        }
        std::lock_guard<std::mutex> g(c->twin_mu);
        auto it = c->twins.find(dst);
        if (it != c->twins.end()) {
            cudaFree(it->second.dev);
        }
        c->twins[dst] = WeightTwin{d_dst, total};
    }
    // cpu/x86/int8/convolution_transform.cpp:176-185: fc is reported padded to 16
    *ftmDesc = *filterDesc;
    ftmDesc->df = DF_NCHWC2NxC4;
    ftmDesc->dims[2] = B200_ALIGN(B200_ALIGN(f.c, 4), 16);
    return ret;
}

EE conv_i8_tmp_bytes(const TensorDesc *inputDesc, const TensorDesc *filterDesc, const TensorDesc *outputDesc,
    const ConvolutionParamSpec *cp, U32 *bytes)
{
    if (bytes == nullptr) {
        return NULL_POINTER;
    }
    ConvGeom g;
    B200_EE(conv_geometry(inputDesc, filterDesc, outputDesc, cp, &g));
    // room for: an fp32 input quantized first, the padded channels-of-16 copy (needed for other layouts, and
    // kept available for paddings the border classes cannot express), and the int32 / fp32 staging of a
    // dynamically requantized u8 output
    size_t b = 512;
    if (g.in.dt == DT_F32) {
        b += B200_ALIGN((size_t)g.in.n * g.in.c * g.in.h * g.in.w, 256);
    }
    if (g.needs_copy || g.pt || g.pb || g.pl || g.pr) {
        b += B200_ALIGN(g.xp_bytes, 256);
    }
    if (g.out.dt == DT_U8_Q) {
        b += (size_t)g.out.n * g.out.c * g.out.h * g.out.w * 4;
    }
    if (b > 0xFFFFFFFFull) {
        return NOT_SUPPORTED;
    }
    *bytes = (U32)b;
    return SUCCESS;
}

EE quantize_i32_u8_device(const int32_t *d_src, uint64_t n, uint8_t *d_q, F32 *scale2);
EE quantize_f32_u8_device(const float *d_src, uint64_t n, uint8_t *d_q, F32 *scale, int mode);

// ext: NULL for Bolt's semantics; otherwise the extension of bolt_b200_convolution_ex
EE conv_i8_run(const TensorDesc *inputDesc, void *input, void *eltwiseInput, const TensorDesc *filterDesc,
    const void *filter, const ConvolutionParamSpec *cp, void *scale, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *act, const bolt_b200_conv_ext *ext)
{
    ConvGeom g;
    B200_EE(conv_geometry(inputDesc, filterDesc, outputDesc, cp, &g));
    if (input == nullptr || filter == nullptr || output == nullptr || tmp == nullptr || scale == nullptr) {
        return NULL_POINTER;
    }
    if ((g.in.dt != DT_U8_Q && g.in.dt != DT_F32) || g.f.dt != DT_I8 || (g.out.dt != DT_F32 && g.out.dt != DT_U8_Q)) {
        return NOT_SUPPORTED;
    }
    if (g.f.df != DF_NCHWC2NxC4) {
        return NOT_MATCH;  // convolution_direct.cpp:2613-2615
    }
    if (g.in.df != DF_NCHWC16 && g.in.df != DF_NCHWC8 && g.in.df != DF_NCHW) {
        return NOT_MATCH;
    }
    if (g.out.df != DF_NCHWC16 && g.out.df != DF_NCHWC8) {
        return NOT_MATCH;  // cpu/x86/int8/convolution.cpp:127-129
    }
    // the packed filter reports fc padded to 16; the input carries the real channel count
    if (B200_ALIGN(g.in.c, 16) != B200_ALIGN(g.f.c, 16) || g.out.c != g.f.n || (g.out.c % 8) != 0) {
        return NOT_MATCH;
    }
    // The AVX512 kernels test two bits of the activation mode (flags = mode << 2, `and $0xC`,
    // convolution_direct.cpp:2143-2146,2747; convolution_1x1_direct.cpp:366-369): ReLU is applied when
    // mode & 3 is not zero, whatever the mode's name.
    const bool relu = act != nullptr && ((unsigned)act->mode & 3u) != 0;
    const bool out_u8 = g.out.dt == DT_U8_Q;
    const float ext_out_scale = (ext != nullptr && out_u8) ? ext->output_scale : 0.f;
    const void *ext_fscale = ext != nullptr ? ext->filter_scales : nullptr;
    U32 need = 0;
    B200_EE(conv_i8_tmp_bytes(inputDesc, filterDesc, outputDesc, cp, &need));
    if (tmpBytes < need) {
        return NOT_MATCH;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    cudaStream_t st = tls().stream;
    F32 *sc = reinterpret_cast<F32 *>(scale);
    const size_t out_elems = (size_t)g.out.n * g.out.c * g.out.h * g.out.w;
    const size_t in_elems = (size_t)g.in.n * g.in.c * g.in.h * g.in.w;
    const size_t ts_off = filter_tapsum_off(g.f.n, g.OCr, g.K);
    const size_t w_bytes = ts_off + 4 * (size_t)g.f.n * g.taps;

    Stage sg;
    const void *d_in_any = sg.in(input, in_elems * (g.in.dt == DT_F32 ? 4 : 1));
    const char *d_w = nullptr;
    if (is_device_ptr(filter)) {
        d_w = reinterpret_cast<const char *>(filter);
    } else {
        std::lock_guard<std::mutex> lk(c->twin_mu);
        auto it = c->twins.find(filter);
        if (it != c->twins.end() && it->second.bytes >= w_bytes) {
            d_w = reinterpret_cast<const char *>(it->second.dev);
        }
    }
    if (d_w == nullptr) {
        d_w = reinterpret_cast<const char *>(sg.in(filter, w_bytes));
    }
    const float *d_bias = bias ? reinterpret_cast<const float *>(sg.in(bias, 4 * (size_t)g.out.c)) : nullptr;
    const float *d_elt = eltwiseInput ? reinterpret_cast<const float *>(sg.in(eltwiseInput, 4 * out_elems)) : nullptr;
    const float *d_fscale = ext_fscale ? reinterpret_cast<const float *>(sg.in(ext_fscale, 4 * (size_t)g.out.c)) : nullptr;
    void *d_out = sg.out(output, out_elems * (out_u8 ? 1 : 4));
    // a host `tmp` cannot be used by the device: take device scratch of the same size instead
    char *d_tmp = is_device_ptr(tmp) ? reinterpret_cast<char *>(tmp) : reinterpret_cast<char *>(sg.scratch(need));
    if (d_in_any == nullptr || d_w == nullptr || d_out == nullptr || d_tmp == nullptr || (bias && d_bias == nullptr) ||
        (eltwiseInput && d_elt == nullptr) || (ext_fscale && d_fscale == nullptr)) {
        return ALLOC_FAILED;
    }
    d_tmp = reinterpret_cast<char *>(B200_ALIGN(reinterpret_cast<uintptr_t>(d_tmp), 256));
    // an fp32 input is quantized first (convolution_direct.cpp:2679-2686); scale[0] is read and written as
    // quantize_x86 does it
    const uint8_t *d_in = reinterpret_cast<const uint8_t *>(d_in_any);
    if (g.in.dt == DT_F32) {
        uint8_t *q = reinterpret_cast<uint8_t *>(d_tmp);
        d_tmp += B200_ALIGN(in_elems, 256);
        B200_EE(quantize_f32_u8_device(reinterpret_cast<const float *>(d_in_any), in_elems, q, &sc[0], 0));
        d_in = q;
    }
    const float scaleO = sc[0] * sc[2];  // convolution_direct.cpp:2687

    ConvLaunch a;
    std::memset(&a, 0, sizeof(a));
    a.w = reinterpret_cast<const int8_t *>(d_w + filter_weights_off(g.f.n));
    a.offsetC = reinterpret_cast<const int32_t *>(d_w);
    a.tapsum = reinterpret_cast<const int32_t *>(d_w + ts_off);
    a.bias = d_bias;
    a.fscale = d_fscale;
    a.eltwise = d_elt;
    a.sI = sc[0];
    a.sF = sc[2];
    a.relu = relu ? 1 : 0;
    // Output modes.  Bolt (ext == NULL): fp32, or u8 requantized with the dynamic scale 127 / max|acc| over the
    // whole output, scale[1] written back (convolution_direct.cpp:2798-2806); with an eltwise input the u8
    // result is the dynamic F32 -> U8_Q quantization of the fp32 result (:2693-2695).  Extension: a known
    // output scale is applied in the epilogue; per-channel filter scales turn the dynamic u8 case into the
    // fp32-staged one (accumulators of different channels are not comparable).
    const bool fused_u8 = out_u8 && ext_out_scale > 0.f && d_elt == nullptr;
    const bool f32_staged = out_u8 && !fused_u8 && (d_elt != nullptr || d_fscale != nullptr);
    a.out_kind = fused_u8 ? 2 : ((out_u8 && !f32_staged) ? 0 : 1);
    a.num = fused_u8 ? ext_out_scale : 1.0f;
    char *staging = d_tmp + ((g.needs_copy || g.pt || g.pb || g.pl || g.pr) ? B200_ALIGN(g.xp_bytes, 256) : 0);
    a.out = (out_u8 && !fused_u8) ? reinterpret_cast<void *>(staging) : d_out;

    // input: in place with the padding folded into the coordinates, or through a padded copy
    EE ret = NOT_SUPPORTED;
    if (!g.needs_copy) {
        a.x = d_in;
        a.H = g.in.h;
        a.W = g.in.w;
        a.pt = (int32_t)g.pt;
        a.pl = (int32_t)g.pl;
        ret = launch_conv_tcgen05(g, a, st);
    }
    if (ret == NOT_SUPPORTED) {
        uint8_t *buf = reinterpret_cast<uint8_t *>(d_tmp);
        const size_t chunks = g.xp_bytes / 16;
        size_t blocks = (chunks + 255) / 256;
        if (blocks > (size_t)c->sm_count * 16) {
            blocks = (size_t)c->sm_count * 16;
        }
        const uint32_t in_block = g.in.df == DF_NCHWC16 ? 16u : (g.in.df == DF_NCHWC8 ? 8u : 0u);
        pad_relayout_kernel<<<(uint32_t)blocks, 256, 0, st>>>(d_in, g.in.n, g.in.c, g.in.h, g.in.w, in_block, g.ICb, g.Hp,
            g.Wp, g.pt, g.pl, buf);
        count_launch();
        a.x = buf;
        a.H = g.Hp;
        a.W = g.Wp;
        a.pt = 0;
        a.pl = 0;
        ret = launch_conv_tcgen05(g, a, st);
    }
    B200_EE(ret);
    if (fused_u8) {
        sc[1] = ext_out_scale;
    } else if (f32_staged) {
        F32 s = -1;
        B200_EE(quantize_f32_u8_device(reinterpret_cast<const float *>(a.out), out_elems, reinterpret_cast<uint8_t *>(d_out), &s, 0));
        sc[1] = s;
    } else if (out_u8) {
        F32 scales[2] = {-1, scaleO};
        B200_EE(quantize_i32_u8_device(reinterpret_cast<const int32_t *>(a.out), out_elems,
            reinterpret_cast<uint8_t *>(d_out), scales));
        sc[1] = scales[0];
    } else {
        sc[1] = scaleO;
    }
    return sg.finish();
}

}  // namespace b200
