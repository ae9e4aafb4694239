// conv_i8.cu -- int8 convolution as an implicit GEMM on the sm_100a tensor cores.
//
//   acc[n,oc,oh,ow] = offsetC[oc] + round(bias[oc]*scaleO) + sum_{ic,kh,kw} W_s8 * X_u8(pad = 128)
//
// Replaces Bolt's AVX512 direct and 1x1 convolution kernels and their drivers
// (compute/tensor/src/cpu/x86/int8/avx512/convolution_direct.cpp:2584-2809,
//  convolution_1x1_direct.cpp:2073-2327), the filter transform
// (cpu/x86/int8/convolution_transform.cpp:18-238) and the input pad / relayout
// (cpu/x86/int8/transform_functions_int8.h:19-224).
//
// GEMM view: M = output pixels (a TH x TW patch of one image = 128 rows per tile), N = output
// channels, K = (kh, kw, input-channel block of 16).  The input is brought to a padded
// channels-of-16 layout [N][IC/16][Hp][Wp][16] (pad value 128, one streaming pass; skipped when
// the caller's tensor already has it).  There a 16-byte K chunk of 128 pixels is exactly a 5-D TMA
// box {16 B, TW, TH, chunks, 1} -- element strides carry the convolution stride, the start
// coordinates carry (kh, kw) -- and lands in shared memory as 8-row x 16-byte core matrices, the
// un-swizzled K-major operand layout of tcgen05.mma.  No im2col buffer ever exists.  Weights are
// pre-packed [OC][K] and loaded like the GEMM's B operand (128-byte swizzle).  Warp roles, the
// tensor-memory double buffering and the bounded waits are those of gemm_i8_tcgen05.cu.
#include <cstring>

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int MAX_BLOCK_N = 256;
constexpr int STAGES = 4;
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int NUM_THREADS = 64 + EPI_THREADS;
constexpr uint32_t TMEM_COLS = 512;
constexpr int SMEM_A_STAGE = BLOCK_M * BLOCK_K;      // 8 K-chunks x 128 pixels x 16 B
constexpr int SMEM_B_STAGE = MAX_BLOCK_N * BLOCK_K;
constexpr int CHUNK_BYTES = BLOCK_M * 16;            // one 16-byte K chunk of all 128 pixels

struct __align__(16) SmemCtl {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    __align__(16) int32_t offs[2048];  // offsetC + bias of every output channel (layers with OC <= 2048)
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * (SMEM_A_STAGE + SMEM_B_STAGE) + sizeof(SmemCtl);

struct ConvParams {
    uint32_t N, OH, OW, OC;
    uint32_t TW, TH, tw_shift, tiles_w, tiles_h;
    uint32_t ICb, FW;
    uint32_t sH, sW, dH, dW;
    uint32_t G;             // K chunks per TMA load: divides both ICb and 8
    uint32_t merged_w;      // 1: stride-1 rows, map_x is 4-D with (c16, w) merged into one byte dimension
    uint32_t total_chunks;  // taps * ICb
    uint32_t num_kb;        // ceil(total_chunks / 8)
    uint32_t block_n, tiles_n, tiles_m;
    void *out;
    const float *eltwise;
    const int32_t *offs;    // [OC]: offsetC + round(bias * scaleO)
    float factor;           // 1 / scaleO (fp32 output) or outScale / scaleO (fused u8 output)
    int relu;
    int *status;
};

// KIND 1: fp32 output (dequantize, + eltwise, ReLU).  KIND 0: int32 output after ReLU, the staging
// buffer of the dynamic u8 path (convolution_direct.cpp:2689-2693).  KIND 2: u8 output with a known
// output scale, the arithmetic of quantizeI32ToU8 with both scales given (avx512/quantize.cpp:372-414:
// vcvtdq2ps, vmulps, vaddps 128, vcvtps2dq, vpmovusdb) fused behind the ReLU.
template <int KIND>
__device__ __forceinline__ void store_block16(const ConvParams &p, const int32_t *offs, size_t base, uint32_t width,
    const uint32_t *r /*16 accumulators*/)
{
    if (KIND == 2) {
        uint8_t *out = reinterpret_cast<uint8_t *>(p.out) + base;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            const int4 o = *reinterpret_cast<const int4 *>(offs + j);
            int v[4] = {(int)r[j] + o.x, (int)r[j + 1] + o.y, (int)r[j + 2] + o.z, (int)r[j + 3] + o.w};
            uint32_t b[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int a = p.relu ? max(v[t], 0) : v[t];
                const float f = __fadd_rn(__fmul_rn(__int2float_rn(a), p.factor), 128.0f);
                // rne(f) as unsigned, clamped at 255: negatives wrap above 255 like vpmovusdb reads them
                b[t] = min(__float_as_uint(__fadd_rn(f, 12582912.0f)) - 0x4B400000u, 255u);
            }
            w[j >> 2] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
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
                float4 v = make_float4(acc_to_f32((int)r[j] + o.x, p.factor), acc_to_f32((int)r[j + 1] + o.y, p.factor),
                    acc_to_f32((int)r[j + 2] + o.z, p.factor), acc_to_f32((int)r[j + 3] + o.w, p.factor));
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

template <int KIND>
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_u8s8_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    const ConvParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * SMEM_A_STAGE;
    SmemCtl *ctl = reinterpret_cast<SmemCtl *>(smem + STAGES * (SMEM_A_STAGE + SMEM_B_STAGE));

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&ctl->tmem_full[a], 1);
            mbar_init(&ctl->tmem_empty[a], EPI_THREADS);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctl->tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    // tile -> (image, patch origin, first output channel)
    auto decode = [&](uint32_t tile, uint32_t &n, uint32_t &oh0, uint32_t &ow0, uint32_t &n0) {
        const uint32_t mt = tile % p.tiles_m;
        n0 = (tile / p.tiles_m) * p.block_n;
        const uint32_t per_img = p.tiles_w * p.tiles_h;
        n = mt / per_img;
        const uint32_t r = mt - n * per_img;
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
                    mbar_expect_tx(&ctl->full[stage], nq * CHUNK_BYTES + p.block_n * BLOCK_K);
                    for (uint32_t j = 0; j < nq; j += p.G) {
                        const uint32_t q = q0 + j;
                        const uint32_t tap = q / p.ICb;
                        const uint32_t cb = q - tap * p.ICb;
                        const uint32_t kh = tap / p.FW, kw = tap - kh * p.FW;
                        uint8_t *dst = smem_a + stage * SMEM_A_STAGE + j * CHUNK_BYTES;
                        if (p.merged_w) {
                            // a row of TW pixels is TW * 16 contiguous bytes: one wide request per row
                            tma_load_4d(&map_x, &ctl->full[stage], dst, (int)((ow0 + kw * p.dW) * 16),
                                (int)(oh0 * p.sH + kh * p.dH), (int)cb, (int)n);
                        } else {
                            tma_load_5d(&map_x, &ctl->full[stage], dst, 0, (int)(ow0 * p.sW + kw * p.dW),
                                (int)(oh0 * p.sH + kh * p.dH), (int)cb, (int)n);
                        }
                    }
                    tma_load_2d(&map_w, &ctl->full[stage], smem_b + stage * SMEM_B_STAGE, (int)(kb * BLOCK_K), (int)n0);
                    if (++stage == STAGES) {
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
                const uint32_t tmem_d = tmem_base + acc * MAX_BLOCK_N;
                for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->full[stage], phase)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t nq = min(8u, p.total_chunks - kb * 8);
                    const uint32_t a_addr = smem_u32(smem_a + stage * SMEM_A_STAGE);
                    const uint64_t db = make_desc_sw128(smem_u32(smem_b + stage * SMEM_B_STAGE));
                    for (uint32_t k = 0; 2 * k < nq; ++k) {
                        // A: two 16-byte K chunks per MMA, CHUNK_BYTES apart; 8-pixel groups 128 B apart.
                        // An odd last chunk pairs with stale bytes, which meet zero weights.
                        const uint64_t da = make_desc_noswizzle(a_addr + k * 2 * CHUNK_BYTES, CHUNK_BYTES, 128);
                        umma_i8(tmem_d, da, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(&ctl->empty[stage]);
                    if (++stage == STAGES) {
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
        // Per-channel offsets: staged once per CTA when they fit, so that no tile waits on a global
        // load or a CTA-wide barrier; wider layers read them through L1.
        const int32_t *offs_all = p.offs;
        if (p.OC <= 2048) {
            for (uint32_t i = et; i < 2048; i += EPI_THREADS) {
                ctl->offs[i] = (i < p.OC) ? p.offs[i] : 0;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            offs_all = ctl->offs;
        }
        const uint32_t c_begin = half ? ((nch + 1) >> 1) : 0u;
        const uint32_t c_end = half ? nch : ((nch + 1) >> 1);
        uint32_t it = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            uint32_t n, oh0, ow0, n0;
            decode(tile, n, oh0, ow0, n0);
            if (*reinterpret_cast<volatile uint32_t *>(&ctl->abort_flag) != 0) {
                break;  // some role's bounded wait ran out
            }
            bool ok = mbar_wait(&ctl->tmem_full[acc], acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) {
                    atomicExch(p.status, 13);
                    atomicExch(&ctl->abort_flag, 1u);
                }
                break;
            }
            tcgen05_fence_after();
            const uint32_t r = quad * 32 + lane;
            const uint32_t oh = oh0 + (r >> p.tw_shift);
            const uint32_t ow = ow0 + (r & (p.TW - 1));
            const bool row_ok = oh < p.OH && ow < p.OW;
            const size_t pix = (size_t)oh * p.OW + ow;
            const size_t plane = (size_t)p.OH * p.OW;
            const uint32_t tbase = tmem_base + ((quad * 32u) << 16) + acc * MAX_BLOCK_N;
            auto emit = [&](uint32_t c, const uint32_t *rr) {
                if (row_ok) {
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        const uint32_t ocb = n0 + c * 32 + hb * 16;
                        if (ocb < p.OC) {
                            const uint32_t width = min(16u, p.OC - ocb);
                            const size_t base = ((size_t)n * p.OC + ocb) * plane + pix * width;
                            store_block16<KIND>(p, offs_all + ocb, base, width, rr + hb * 16);
                        }
                    }
                }
            };
            // two register buffers: the next chunk is on its way from tensor memory while this one is
            // converted and stored; the accumulator is released as soon as its last chunk has arrived
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
                    tcgen05_fence_before();
                    mbar_arrive(&ctl->tmem_empty[acc]);
                }
                emit(c, ra);
                if (has1) {
                    tmem_ld_wait(rb);
                    if (c + 2 < c_end) {
                        tmem_ld32(tbase + (c + 2) * 32, ra);
                    } else {
                        tcgen05_fence_before();
                        mbar_arrive(&ctl->tmem_empty[acc]);
                    }
                    emit(c + 1, rb);
                }
            }
            if (c_begin >= c_end) {
                tcgen05_fence_before();
                mbar_arrive(&ctl->tmem_empty[acc]);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

// ---- filter packing: s8 NCHW [OC][IC][FH][FW] -> [OCr][K], k = ((kh*FW + kw)*ICb + cb)*16 + c ------------
// offsetC[oc] = -128 * sum of the filter (convolution_transform.cpp: offsetC first, then the weights).
__global__ void pack_conv_filter_kernel(const int8_t *__restrict__ src, uint32_t OC, uint32_t IC, uint32_t taps,
    uint32_t ICb, uint32_t OCr, int8_t *__restrict__ dst, int32_t *__restrict__ offsetC)
{
    const uint32_t oc = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (oc >= OCr) {
        return;
    }
    const uint32_t K = taps * ICb * 16;
    int32_t sum = 0;
    for (uint32_t k = lane; k < K; k += 32) {
        const uint32_t c = k & 15, q = k >> 4;
        const uint32_t tap = q / ICb, cb = q - tap * ICb;
        const uint32_t ic = cb * 16 + c;
        int8_t v = 0;
        if (oc < OC && ic < IC) {
            v = src[((size_t)oc * IC + ic) * taps + tap];
        }
        dst[(size_t)oc * K + k] = v;
        sum += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    if (lane == 0 && oc < OC) {
        offsetC[oc] = sum * (-128);
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

// offs[oc] = round(bias[oc] * scaleO) + offsetC[oc]   (cpu/x86/int8/avx512/quantize.cpp:259-266)
__global__ void conv_bias_offset_kernel(const float *bias, const int32_t *offsetC, uint32_t n, float scaleO, int32_t *out)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        int b = 0;
        if (bias != nullptr) {
            b = (int)roundf(__fmul_rn(bias[i], scaleO));
        }
        out[i] = b + offsetC[i];
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

uint32_t pick_conv_block_n(uint32_t tiles_m, uint32_t OC, int sms)
{
    uint32_t best = 32;
    double best_cost = 1e30;
    for (uint32_t bn = 256; bn >= 32; bn -= 32) {
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

struct ConvGeom {
    Conv4d in, f, out;
    uint32_t sH, sW, dH, dW, pt, pb, pl, pr;
    uint32_t ICb, Hp, Wp, taps, K, OCr;
    bool needs_copy;
    size_t xp_bytes;
};

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
    g->needs_copy = !(g->in.df == DF_NCHWC16 && (g->in.c % 16) == 0 && g->pt == 0 && g->pb == 0 && g->pl == 0 && g->pr == 0);
    g->xp_bytes = (size_t)g->in.n * g->ICb * g->Hp * g->Wp * 16;
    return SUCCESS;
}

}  // namespace

// run the implicit-GEMM kernel; xp: [N][ICb][Hp][Wp][16] u8, w: [OCr][K] s8, offs: [OC] int32 (all device)
EE launch_conv_tcgen05(const uint8_t *xp, const int8_t *w, const int32_t *offs, void *out, int out_kind,
    const float *eltwise, float factor, int relu, uint32_t N, uint32_t ICb, uint32_t Hp, uint32_t Wp, uint32_t OC,
    uint32_t OCr, uint32_t OH, uint32_t OW, uint32_t FH, uint32_t FW, uint32_t sH, uint32_t sW, uint32_t dH,
    uint32_t dW, cudaStream_t st)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    {
        const void *ks[3] = {(const void *)conv_u8s8_tcgen05_kernel<0>, (const void *)conv_u8s8_tcgen05_kernel<1>,
            (const void *)conv_u8s8_tcgen05_kernel<2>};
        B200_EE(raise_smem_limit(c, KF_CONV, ks, 3, SMEM_BYTES));
    }
    if (!tensor_map_encoder_available()) {
        return NOT_SUPPORTED;
    }
    ConvParams p;
    std::memset(&p, 0, sizeof(p));
    p.N = N;
    p.OH = OH;
    p.OW = OW;
    p.OC = OC;
    // output patch of 128 pixels: the shape that wastes the fewest rows
    // With stride 1 along W a row of TW pixels is TW*16 contiguous bytes; the (c16, w) dimensions are
    // then merged so that TMA moves one 16*TW-byte run per row instead of TW 16-byte ones (a TMA box
    // is at most 256 elements wide, hence TW <= 16 on that path).
    const bool merged_w = (sW == 1);
    uint32_t best_tw = 128, best_tiles = 0xFFFFFFFFu;
    for (uint32_t tw = merged_w ? 16 : 128; tw >= 1; tw >>= 1) {
        const uint32_t th = 128 / tw;
        if (tw * sW > 256 || th * sH > 256) {
            continue;
        }
        const uint32_t tiles = ((OW + tw - 1) / tw) * ((OH + th - 1) / th);
        if (tiles < best_tiles) {
            best_tiles = tiles;
            best_tw = tw;
        }
    }
    if (best_tiles == 0xFFFFFFFFu) {
        return NOT_SUPPORTED;
    }
    p.TW = best_tw;
    p.TH = 128 / best_tw;
    p.tw_shift = 0;
    while ((1u << p.tw_shift) < p.TW) {
        ++p.tw_shift;
    }
    p.tiles_w = (OW + p.TW - 1) / p.TW;
    p.tiles_h = (OH + p.TH - 1) / p.TH;
    p.ICb = ICb;
    p.FW = FW;
    p.sH = sH;
    p.sW = sW;
    p.dH = dH;
    p.dW = dW;
    p.merged_w = merged_w ? 1 : 0;
    p.G = 8;
    while (ICb % p.G != 0) {
        p.G >>= 1;
    }
    p.total_chunks = FH * FW * ICb;
    p.num_kb = (p.total_chunks + 7) / 8;
    p.tiles_m = N * p.tiles_w * p.tiles_h;
    p.block_n = pick_conv_block_n(p.tiles_m, OC, c->sm_count);
    p.tiles_n = (OC + p.block_n - 1) / p.block_n;
    p.out = out;
    p.eltwise = eltwise;
    p.offs = offs;
    p.factor = factor;
    p.relu = relu;
    p.status = c->d_status;

    CUtensorMap map_x, map_w;
    if (merged_w) {
        const uint64_t dims[4] = {(uint64_t)Wp * 16, Hp, ICb, N};
        const uint64_t strides[3] = {(uint64_t)Wp * 16, (uint64_t)Hp * Wp * 16, (uint64_t)ICb * Hp * Wp * 16};
        const uint32_t box[4] = {p.TW * 16, p.TH * sH, p.G, 1};
        const uint32_t es[4] = {1, sH, 1, 1};
        if (!encode_tiled_u8(&map_x, 4, xp, dims, strides, box, es, 0)) {
            return NOT_SUPPORTED;
        }
    } else {
        const uint64_t dims[5] = {16, Wp, Hp, ICb, N};
        const uint64_t strides[4] = {16, (uint64_t)Wp * 16, (uint64_t)Hp * Wp * 16, (uint64_t)ICb * Hp * Wp * 16};
        const uint32_t box[5] = {16, p.TW * sW, p.TH * sH, p.G, 1};
        const uint32_t es[5] = {1, sW, sH, 1, 1};
        if (!encode_tiled_u8(&map_x, 5, xp, dims, strides, box, es, 0)) {
            return NOT_SUPPORTED;
        }
    }
    {
        const uint64_t K = (uint64_t)p.total_chunks * 16;
        const uint64_t dims[2] = {K, OCr};
        const uint64_t strides[1] = {K};
        const uint32_t box[2] = {(uint32_t)BLOCK_K, p.block_n};
        const uint32_t es[2] = {1, 1};
        if (!encode_tiled_u8(&map_w, 2, w, dims, strides, box, es, 128)) {
            return NOT_SUPPORTED;
        }
    }
    const uint64_t tiles = (uint64_t)p.tiles_m * p.tiles_n;
    const uint32_t grid = (uint32_t)(tiles < (uint64_t)c->sm_count ? tiles : (uint64_t)c->sm_count);
    if (out_kind == 2) {
        conv_u8s8_tcgen05_kernel<2><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_x, map_w, p);
    } else if (out_kind == 1) {
        conv_u8s8_tcgen05_kernel<1><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_x, map_w, p);
    } else {
        conv_u8s8_tcgen05_kernel<0><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_x, map_w, p);
    }
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

// ---- entry-point bodies for the int8 branch (called from conv.cu) ----------------------------------------
EE conv_i8_transform_filter_bytes(const TensorDesc *filterDesc, U32 *bytes)
{
    Conv4d f;
    if (!get4d(filterDesc, &f) || bytes == nullptr) {
        return NOT_MATCH;
    }
    // cpu/x86/convolution.cpp:141-166: ALIGN(fn,8) * ALIGN(fc,16) * fh * fw + 4*fn + 32
    *bytes = B200_ALIGN(f.n, 8) * B200_ALIGN(f.c, 16) * f.h * f.w + 4 * f.n + 32;
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
    const size_t mat = (size_t)OCr * taps * ICb * 16;
    const size_t total = 4 * (size_t)f.n + mat;
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
        reinterpret_cast<int8_t *>(d_dst + 4 * (size_t)f.n), reinterpret_cast<int32_t *>(d_dst));
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
    size_t b = 256;
    if (g.needs_copy) {
        b += B200_ALIGN(g.xp_bytes, 256);
    }
    b += B200_ALIGN(4 * (size_t)g.out.c, 256);
    if (g.out.dt == DT_U8_Q) {
        b += (size_t)g.out.n * g.out.c * g.out.h * g.out.w * 4;  // int32 results before quantization
    }
    if (b > 0xFFFFFFFFull) {
        return NOT_SUPPORTED;
    }
    *bytes = (U32)b;
    return SUCCESS;
}

EE quantize_i32_u8_device(const int32_t *d_src, uint64_t n, uint8_t *d_q, F32 *scale2);

EE conv_i8_run(const TensorDesc *inputDesc, void *input, void *eltwiseInput, const TensorDesc *filterDesc,
    const void *filter, const ConvolutionParamSpec *cp, void *scale, const void *bias, U32 tmpBytes, void *tmp,
    const TensorDesc *outputDesc, void *output, const ActivationParamSpec *act)
{
    ConvGeom g;
    B200_EE(conv_geometry(inputDesc, filterDesc, outputDesc, cp, &g));
    if (input == nullptr || filter == nullptr || output == nullptr || tmp == nullptr || scale == nullptr) {
        return NULL_POINTER;
    }
    if (g.in.dt != DT_U8_Q || g.f.dt != DT_I8 || (g.out.dt != DT_F32 && g.out.dt != DT_U8_Q)) {
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
    const bool relu = act != nullptr && act->mode != ACTIVATION_NULL;
    if (act != nullptr && act->mode != ACTIVATION_NULL && act->mode != ACTIVATION_RELU) {
        return NOT_SUPPORTED;
    }
    const bool out_u8 = g.out.dt == DT_U8_Q;
    if (out_u8 && eltwiseInput != nullptr) {
        return NOT_SUPPORTED;  // the reference switches to an fp32 staging + F32->U8 quantize there
    }
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
    const float scaleO = sc[0] * sc[2];  // convolution_direct.cpp:2687
    const float factor = 1 / scaleO;
    const size_t out_elems = (size_t)g.out.n * g.out.c * g.out.h * g.out.w;
    const size_t in_bytes = (size_t)g.in.n * g.in.c * g.in.h * g.in.w;
    const size_t w_bytes = 4 * (size_t)g.f.n + (size_t)g.OCr * g.K;

    Stage sg;
    const uint8_t *d_in = reinterpret_cast<const uint8_t *>(sg.in(input, in_bytes));
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
    void *d_out = sg.out(output, out_elems * (out_u8 ? 1 : 4));
    // a host `tmp` cannot be used by the device: take device scratch of the same size instead
    char *d_tmp = is_device_ptr(tmp) ? reinterpret_cast<char *>(tmp) : reinterpret_cast<char *>(sg.scratch(need));
    if (d_in == nullptr || d_w == nullptr || d_out == nullptr || d_tmp == nullptr || (bias && d_bias == nullptr) ||
        (eltwiseInput && d_elt == nullptr)) {
        return ALLOC_FAILED;
    }
    d_tmp = reinterpret_cast<char *>(B200_ALIGN(reinterpret_cast<uintptr_t>(d_tmp), 256));
    const uint8_t *xp = d_in;
    if (g.needs_copy) {
        uint8_t *buf = reinterpret_cast<uint8_t *>(d_tmp);
        d_tmp += B200_ALIGN(g.xp_bytes, 256);
        const size_t chunks = g.xp_bytes / 16;
        size_t blocks = (chunks + 255) / 256;
        if (blocks > (size_t)c->sm_count * 16) {
            blocks = (size_t)c->sm_count * 16;
        }
        const uint32_t in_block = g.in.df == DF_NCHWC16 ? 16u : (g.in.df == DF_NCHWC8 ? 8u : 0u);
        pad_relayout_kernel<<<(uint32_t)blocks, 256, 0, st>>>(d_in, g.in.n, g.in.c, g.in.h, g.in.w, in_block, g.ICb, g.Hp,
            g.Wp, g.pt, g.pl, buf);
        count_launch();
        xp = buf;
    }
    int32_t *d_offs = reinterpret_cast<int32_t *>(d_tmp);
    d_tmp += B200_ALIGN(4 * (size_t)g.out.c, 256);
    conv_bias_offset_kernel<<<(g.out.c + 255) / 256, 256, 0, st>>>(d_bias, reinterpret_cast<const int32_t *>(d_w), g.out.c,
        scaleO, d_offs);
    count_launch();
    // Extension without a counterpart in the reference's convolution (it always requantizes
    // dynamically): a positive output scale on entry fuses the requantization into the epilogue,
    // with the arithmetic Bolt uses when an output scale is known (fully_connected.cpp:479-487 ->
    // quantizeI32ToU8 with scales {out, scaleO}).
    const bool fused_u8 = out_u8 && sc[1] > 0;
    void *kernel_out = (out_u8 && !fused_u8) ? reinterpret_cast<void *>(d_tmp) : d_out;
    B200_EE(launch_conv_tcgen05(xp, reinterpret_cast<const int8_t *>(d_w + 4 * (size_t)g.f.n), d_offs, kernel_out,
        fused_u8 ? 2 : (out_u8 ? 0 : 1), d_elt, fused_u8 ? sc[1] / scaleO : factor, relu ? 1 : 0, g.in.n, g.ICb, g.Hp, g.Wp, g.out.c, g.OCr, g.out.h, g.out.w, g.f.h,
        g.f.w, g.sH, g.sW, g.dH, g.dW, st));
    if (fused_u8) {
        // sc[1] stays the caller's output scale
    } else if (out_u8) {
        // convolution_direct.cpp:2798-2806: dynamic scale over the whole output, scale[1] = scaleO * 127/max
        F32 scales[2] = {-1, scaleO};
        B200_EE(quantize_i32_u8_device(reinterpret_cast<const int32_t *>(kernel_out), out_elems,
            reinterpret_cast<uint8_t *>(d_out), scales));
        sc[1] = scales[0];
    } else {
        sc[1] = scaleO;
    }
    return sg.finish();
}

}  // namespace b200
