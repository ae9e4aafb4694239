// gemm_i8_tcgen05.cu -- u8 x s8 -> s32 GEMM on the 5th-generation tensor cores of sm_100a.
//
//   C[M,N] = epilogue( offsetC[n] + sum_k A_u8[m,k] * B_s8[n,k] )        (both operands K-major)
//
// Replaces the AVX512-VNNI micro-kernels and their driver in Bolt
// (compute/blas_enhance/src/cpu/x86/int8/avx512/mmm_avx512_vnni.cpp:383-1891).
//
// One persistent CTA per SM, 320 threads, three roles:
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D loads of a 128 x 128-byte A tile and a
//               BLOCK_N x 128-byte B tile per pipeline stage, 128-byte swizzle, mbarrier complete_tx
//   warp 1      MMA issuer: one thread issues tcgen05.mma.cta_group::1.kind::i8 (M=128, N=BLOCK_N,
//               K=32 per instruction, A unsigned / B signed, int32 accumulate, no saturation) with
//               shared-memory matrix descriptors; accumulators live in tensor memory (2 x 256 columns,
//               so the epilogue of tile i overlaps the main loop of tile i+1)
//   warps 2..9  epilogue, two warps per scheduler: the pair that shares a tensor-memory lane quadrant
//               splits the tile's columns; tcgen05.ld of 32 lanes x 32 columns, software pipelined
//               (the next chunk is in flight while this one is converted), fused offsetC / C_in add and
//               the reference's s32 -> f32 / u8 conversions, 16-byte global stores
// Every mbarrier wait is bounded; a wait that runs out sets the device status word and the CTA
// drains and exits (tensor memory is always released).
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int MAX_BLOCK_N = 256;
constexpr int MAX_STAGES = 8;        // the ring is as deep as shared memory allows for the tile width
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int NUM_THREADS = 64 + EPI_THREADS;
constexpr uint32_t TMEM_COLS = 512;  // 2 accumulators x 256 columns

constexpr int SMEM_A_STAGE = BLOCK_M * BLOCK_K;        // 16 KiB

struct __align__(16) SmemCtl {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    // per epilogue warp: offsetC and conversion factor of the (at most 128) columns it owns
    __align__(16) int32_t offs[EPI_WARPS][128];
    __align__(16) float colf[EPI_WARPS][128];
};

// 227 KiB per CTA: alignment slack + control block + as many (A tile, B tile) stages as fit
constexpr size_t SMEM_BYTES = 232448;
// u8 tiles leave through TMA stores: each epilogue warp stages 32 rows x 64 bytes (64-byte swizzle)
constexpr int STAGING_PER_WARP = 32 * 64;
constexpr size_t SMEM_STAGING_BYTES = (size_t)EPI_WARPS * STAGING_PER_WARP;  // 16 KiB
constexpr size_t SMEM_RING_BYTES = (SMEM_BYTES - 1024 - sizeof(SmemCtl) - SMEM_STAGING_BYTES) & ~(size_t)1023;

struct Params {
    uint32_t M, N, K;
    uint32_t block_n;       // multiple of 32, <= 256
    uint32_t stages;        // pipeline depth, <= MAX_STAGES
    uint32_t tiles_m, tiles_n, num_kb;
    void *C;
    GemmEpilogue ep;
    int *status;
    int vec_ok;             // rows of C are 16-byte aligned -> vector stores allowed
};

// ---- epilogue for 32 consecutive columns of one row: the common case ---------------------------
// Full, 16-byte aligned chunk, C overwritten, one conversion factor per column.  Kept free of
// branches and small, because each epilogue warp runs it 4 to 8 times per tile back to back and
// the instruction stream has to stay resident.  Per element: add offsetC, s32 -> f32 (vcvtdq2ps),
// multiply (vmulps), then for u8 the bias-add rounding of f32_to_u8_zp128.
// 32 accumulators of one row -> 32 bytes (8 words): +offsetC, s32 -> f32, * factor, round, +128, clamp
__device__ __forceinline__ void chunk_to_u8(const int32_t *offs, const float *colf, uint32_t cl, const uint32_t (&r)[32],
    uint32_t (&w)[8])
{
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
        const float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
        const uint32_t b0 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j] + o.x), c4.x));
        const uint32_t b1 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j + 1] + o.y), c4.y));
        const uint32_t b2 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j + 2] + o.z), c4.z));
        const uint32_t b3 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j + 3] + o.w), c4.w));
        w[j >> 2] = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
    }
}
// 32 bytes of row `lane` into the warp's staging box [32 rows][64 B], 64-byte swizzle: the 16-byte
// chunk index is XORed with bits 1..2 of the row, the pattern the TMA store undoes
__device__ __forceinline__ void stage_u8(uint8_t *stg, uint32_t lane, uint32_t which, const uint32_t (&w)[8])
{
    const uint32_t sw = (lane >> 1) & 3;
    uint8_t *row = stg + lane * 64;
    *reinterpret_cast<uint4 *>(row + (((which * 2) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4 *>(row + (((which * 2 + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}

template <int KIND>
__device__ __forceinline__ void store_chunk_fast(void *C, uint32_t N, const int32_t *offs, const float *colf,
    uint32_t m, uint32_t n0, uint32_t cl, const uint32_t (&r)[32])
{
    const size_t row_off = (size_t)m * N + n0;
    if (KIND == 2) {
        uint32_t w[8];
        chunk_to_u8(offs, colf, cl, r, w);
        uint8_t *out = reinterpret_cast<uint8_t *>(C) + row_off;
        *reinterpret_cast<uint4 *>(out) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4 *>(out + 16) = make_uint4(w[4], w[5], w[6], w[7]);
    } else if (KIND == 1) {
        float *out = reinterpret_cast<float *>(C) + row_off;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
            const float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
            *reinterpret_cast<float4 *>(out + j) = make_float4(acc_to_f32((int)r[j] + o.x, c4.x),
                acc_to_f32((int)r[j + 1] + o.y, c4.y), acc_to_f32((int)r[j + 2] + o.z, c4.z),
                acc_to_f32((int)r[j + 3] + o.w, c4.w));
        }
    } else {
        int32_t *out = reinterpret_cast<int32_t *>(C) + row_off;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
            *reinterpret_cast<int4 *>(out + j) =
                make_int4((int)r[j] + o.x, (int)r[j + 1] + o.y, (int)r[j + 2] + o.z, (int)r[j + 3] + o.w);
        }
    }
}

// ---- epilogue for 32 consecutive columns of one row: every other case ---------------------------
// (ragged or unaligned N, accumulate into C, per-row scales)
__device__ __forceinline__ void store_chunk(const Params &p, const int32_t *offs, const float *colf, uint32_t m,
    uint32_t n0 /*global col of r[0]*/, uint32_t cl /*tile-local col of r[0]*/, const uint32_t (&r)[32])
{
    const GemmEpilogue &ep = p.ep;
    const uint32_t ncols = min(32u, p.N - n0);
    const size_t row_off = (size_t)m * p.N + n0;
    const bool full_vec = p.vec_ok && ncols == 32;
    int acc[32];
    float cf[32];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
        const float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
        acc[j] = (int)r[j] + o.x;
        acc[j + 1] = (int)r[j + 1] + o.y;
        acc[j + 2] = (int)r[j + 2] + o.z;
        acc[j + 3] = (int)r[j + 3] + o.w;
        cf[j] = c4.x;
        cf[j + 1] = c4.y;
        cf[j + 2] = c4.z;
        cf[j + 3] = c4.w;
    }
    if (ep.out_kind != 2 && ep.accumulate) {
        const int32_t *cin = reinterpret_cast<const int32_t *>(p.C) + row_off;
        if (full_vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                int4 v = *reinterpret_cast<const int4 *>(cin + j);
                acc[j] += v.x;
                acc[j + 1] += v.y;
                acc[j + 2] += v.z;
                acc[j + 3] += v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if ((uint32_t)j < ncols) {
                    acc[j] += cin[j];
                }
            }
        }
    }
    if (ep.out_kind == 0) {
        int32_t *out = reinterpret_cast<int32_t *>(p.C) + row_off;
        if (full_vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                *reinterpret_cast<int4 *>(out + j) = make_int4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if ((uint32_t)j < ncols) {
                    out[j] = acc[j];
                }
            }
        }
        return;
    }
    // conversion factor per element
    float rs = 0.f;
    const bool per_elem = ep.per_channel && ep.row_scale != nullptr;
    if (per_elem) {
        rs = ep.row_scale[m];
    }
    if (ep.out_kind == 1) {
        float *out = reinterpret_cast<float *>(p.C) + row_off;
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float fac = cf[j];
            if (per_elem) {
                fac = __fdiv_rn(ep.num, __fmul_rn(rs, fac));
            }
            f[j] = acc_to_f32(acc[j], fac);
        }
        if (full_vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                *reinterpret_cast<float4 *>(out + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if ((uint32_t)j < ncols) {
                    out[j] = f[j];
                }
            }
        }
        return;
    }
    uint8_t *out = reinterpret_cast<uint8_t *>(p.C) + row_off;
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        uint32_t b[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            float fac = cf[j + t];
            if (per_elem) {
                fac = __fdiv_rn(ep.num, __fmul_rn(rs, fac));
            }
            b[t] = f32_to_u8_zp128(__fmul_rn(__int2float_rn(acc[j + t]), fac));
        }
        w[j >> 2] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    }
    if (full_vec) {
        *reinterpret_cast<uint4 *>(out) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4 *>(out + 16) = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if ((uint32_t)j < ncols) {
                out[j] = (uint8_t)(w[j >> 2] >> (8 * (j & 3)));
            }
        }
    }
}

// KIND >= 0: the fast epilogue for that output kind (0 s32, 1 f32, 2 u8 with direct stores, 3 u8 through
// swizzled staging + TMA stores described by map_c); KIND < 0: the general one.
template <int KIND>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_u8s8_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
    const __grid_constant__ CUtensorMap map_c, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte aligned bases
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    const uint32_t b_stage = p.block_n * BLOCK_K;  // multiple of 4 KiB: every stage stays 1024-byte aligned
    uint8_t *smem_b = smem + p.stages * SMEM_A_STAGE;
    uint8_t *smem_staging = smem + SMEM_RING_BYTES;  // 1024-byte aligned
    SmemCtl *ctl = reinterpret_cast<SmemCtl *>(smem + SMEM_RING_BYTES + SMEM_STAGING_BYTES);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t stage_bytes = (uint32_t)(BLOCK_M + p.block_n) * BLOCK_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
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

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int m0 = (int)((tile % p.tiles_m) * BLOCK_M);
                const int n0 = (int)((tile / p.tiles_m) * p.block_n);
                for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&ctl->full[stage], stage_bytes);
                    tma_load_2d(&map_a, &ctl->full[stage], smem_a + stage * SMEM_A_STAGE, (int)(kb * BLOCK_K), m0);
                    tma_load_2d(&map_b, &ctl->full[stage], smem_b + stage * b_stage, (int)(kb * BLOCK_K), n0);
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                atomicExch(p.status, 1);
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
                    const uint64_t da = make_desc_sw128(smem_u32(smem_a + stage * SMEM_A_STAGE));
                    const uint64_t db = make_desc_sw128(smem_u32(smem_b + stage * b_stage));
#pragma unroll
                    for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        // advancing K inside the 128-byte swizzle row: +32 bytes = +2 in the
                        // 16-byte units of the descriptor's start-address field
                        umma_i8(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(&ctl->empty[stage]);  // frees the stage once these MMAs retire
                    if (++stage == p.stages) {
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
                atomicExch(p.status, 2);
                atomicExch(&ctl->abort_flag, 1u);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------- epilogue warps 2..9 ------------------------------------
        const uint32_t quad = warp & 3;         // tensor-memory lane quadrant this warp may read
        const uint32_t half = (warp - 2) >> 2;  // which half of the tile's columns
        uint8_t *stg = smem_staging + (warp - 2) * STAGING_PER_WARP;
        const GemmEpilogue &ep = p.ep;
        const uint32_t nch = p.block_n >> 5;
        const uint32_t c_begin = half ? ((nch + 1) >> 1) : 0u;
        const uint32_t c_end = half ? nch : ((nch + 1) >> 1);
        // Column constants (offsetC and the conversion factor): every warp keeps those of its own
        // columns in its own slice of shared memory, lane l owning columns l, l+32, l+64, l+96 of the
        // warp's range.  The next tile's values are fetched into registers before the current
        // accumulator is awaited and written after the tile's chunks, so neither the global-load
        // latency nor any CTA-wide barrier sits between two tiles; warps drift freely.
        // The loads are volatile asm so that they stay where they are written (early); everything
        // that depends on them is written after the tile's chunks (late).
        int32_t *offs = ctl->offs[warp - 2];
        float *colf = ctl->colf[warp - 2];
        const uint32_t my_cols = (c_end - c_begin) * 32;
        auto fetch_raw = [&](uint32_t tile_n0, int32_t (&o)[4], float (&sb)[4]) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                o[q] = 0;
                sb[q] = ep.sB;
                const uint32_t j = lane + 32 * q;
                const uint32_t n = tile_n0 + c_begin * 32 + j;
                if (j < my_cols && n < p.N) {
                    if (ep.offsetC != nullptr) {
                        asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(o[q]) : "l"(ep.offsetC + n));
                    }
                    if (ep.col_factor != nullptr) {
                        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(sb[q]) : "l"(ep.col_factor + n));
                    } else if (ep.per_channel && ep.col_scale != nullptr) {
                        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(sb[q]) : "l"(ep.col_scale + n));
                    }
                }
            }
        };
        float sa_dev = ep.sA;
        if (ep.per_channel && ep.sA_dev != nullptr) {
            asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(sa_dev) : "l"(ep.sA_dev));
        }
        auto factor_of = [&](float sb) {
            if (ep.col_factor != nullptr) {
                return sb;  // already the factor
            }
            if (!ep.per_channel) {
                return ep.factor;
            }
            // with per-row scales the division is done per element; keep sB here
            return ep.row_scale ? sb : __fdiv_rn(ep.num, __fmul_rn(sa_dev, sb));
        };
        auto park = [&](const int32_t (&o)[4], const float (&sb)[4]) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                offs[lane + 32 * q] = o[q];
                colf[lane + 32 * q] = factor_of(sb[q]);
            }
            __syncwarp();
        };
        if (blockIdx.x < num_tiles) {
            int32_t o[4];
            float sb[4];
            fetch_raw((blockIdx.x / p.tiles_m) * p.block_n, o, sb);
            park(o, sb);
        }
        uint32_t it = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const uint32_t m0 = (tile % p.tiles_m) * BLOCK_M;
            const uint32_t n0 = (tile / p.tiles_m) * p.block_n;
            if (*reinterpret_cast<volatile uint32_t *>(&ctl->abort_flag) != 0) {
                break;  // some role's bounded wait ran out
            }
            const uint32_t next_tile = tile + gridDim.x;
            int32_t o_next[4];
            float sb_next[4];
            if (next_tile < num_tiles) {
                fetch_raw((next_tile / p.tiles_m) * p.block_n, o_next, sb_next);
            }
            bool ok = mbar_wait(&ctl->tmem_full[acc], acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) {
                    atomicExch(p.status, 3);
                    atomicExch(&ctl->abort_flag, 1u);
                }
                break;
            }
            tcgen05_fence_after();
            const uint32_t m = m0 + quad * 32 + lane;
            const uint32_t tbase = tmem_base + ((quad * 32u) << 16) + acc * MAX_BLOCK_N;
            const bool row_ok = m < p.M;
            uint32_t ra[32], rb[32];
            if (c_begin < c_end) {
                tmem_ld32(tbase + c_begin * 32, ra);
            }
            bool released = false;
            for (uint32_t c = c_begin; c < c_end; c += 2) {
                tmem_ld_wait(ra);
                const bool has1 = c + 1 < c_end;
                if (has1) {
                    tmem_ld32(tbase + (c + 1) * 32, rb);
                } else {
                    tcgen05_fence_before();
                    mbar_arrive(&ctl->tmem_empty[acc]);  // accumulator fully read: the MMA may reuse it
                    released = true;
                }
                if (KIND == 3) {
                    if (has1) {
                        // first half of a 64-column box: the previous box must have left the staging buffer
                        if (lane == 0) {
                            tma_store_wait_read();
                        }
                        __syncwarp();
                        uint32_t w[8];
                        chunk_to_u8(offs, colf, (c - c_begin) * 32, ra, w);
                        stage_u8(stg, lane, 0, w);
                    } else if (row_ok && n0 + c * 32 < p.N) {
                        store_chunk_fast<2>(p.C, p.N, offs, colf, m, n0 + c * 32, (c - c_begin) * 32, ra);  // odd chunk out
                    }
                } else if (row_ok && n0 + c * 32 < p.N) {
                    if (KIND >= 0) {
                        store_chunk_fast<KIND>(p.C, p.N, offs, colf, m, n0 + c * 32, (c - c_begin) * 32, ra);
                    } else {
                        store_chunk(p, offs, colf, m, n0 + c * 32, (c - c_begin) * 32, ra);
                    }
                }
                if (has1) {
                    tmem_ld_wait(rb);
                    if (c + 2 < c_end) {
                        tmem_ld32(tbase + (c + 2) * 32, ra);
                    } else {
                        tcgen05_fence_before();
                        mbar_arrive(&ctl->tmem_empty[acc]);
                        released = true;
                    }
                    if (KIND == 3) {
                        uint32_t w[8];
                        chunk_to_u8(offs, colf, (c + 1 - c_begin) * 32, rb, w);
                        stage_u8(stg, lane, 1, w);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && n0 + c * 32 < p.N) {
                            // rows beyond M and columns beyond N are clipped by the tensor map
                            tma_store_2d(&map_c, stg, (int)(n0 + c * 32), (int)(m0 + quad * 32));
                        }
                    } else if (row_ok && n0 + (c + 1) * 32 < p.N) {
                        if (KIND >= 0) {
                            store_chunk_fast<KIND>(p.C, p.N, offs, colf, m, n0 + (c + 1) * 32, (c + 1 - c_begin) * 32, rb);
                        } else {
                            store_chunk(p, offs, colf, m, n0 + (c + 1) * 32, (c + 1 - c_begin) * 32, rb);
                        }
                    }
                }
            }
            if (!released) {
                tcgen05_fence_before();
                mbar_arrive(&ctl->tmem_empty[acc]);
            }
            if (next_tile < num_tiles) {
                __syncwarp();  // every lane is done reading this tile's constants
                park(o_next, sb_next);
            }
        }
        if (KIND == 3 && lane == 0) {
            tma_store_wait_all();  // shared memory and the output must be settled before the CTA leaves
        }
        __syncwarp();
    }

    __syncthreads();
    if (ctl->abort_flag != 0) {
        // give copies that may still be in flight time to land before shared memory is released
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

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    });
    return fn;
}

// 2-D byte tensor [rows][inner] with row pitch `pitch`, box = 128 bytes x box_rows, 128B swizzle,
// out-of-range elements read as zero.
bool make_map(CUtensorMap *map, const void *base, uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_rows)
{
    const uint64_t dims[2] = {inner, rows};
    const uint64_t strides[1] = {pitch};
    const uint32_t box[2] = {(uint32_t)BLOCK_K, box_rows};
    const uint32_t estr[2] = {1, 1};
    return encode_tiled_u8(map, 2, base, dims, strides, box, estr, 128);
}

// Tile width: the widest of 256 / 192 / 128 / 64 / 32 columns that still gives every SM a tile,
// preferring the one that wastes the least of the last wave.
uint32_t pick_block_n(uint32_t M, uint32_t N, int sms)
{
    const uint32_t tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
    const uint32_t cand[] = {256, 224, 192, 160, 128, 96, 64, 32};
    uint32_t best = 32;
    double best_cost = 1e30;
    for (uint32_t bn : cand) {
        if (bn > B200_ALIGN(N, 32) && bn != 32) {
            continue;
        }
        const uint32_t tiles = tiles_m * ((N + bn - 1) / bn);
        const uint32_t waves = (tiles + sms - 1) / sms;
        // time ~ waves x (tile cost); narrow tiles pay more shared-memory traffic per MAC
        const double cost = (double)waves * (bn + 48.0);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

}  // namespace

bool tensor_map_encoder_available()
{
    return encode_fn() != nullptr;
}

bool encode_tiled_u8(void *map, uint32_t rank, const void *base, const uint64_t *dims, const uint64_t *strides,
    const uint32_t *box, const uint32_t *elem_strides, int swizzle_bytes)
{
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) {
        return false;
    }
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], es[5];
    for (uint32_t i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        es[i] = elem_strides[i];
        if (i + 1 < rank) {
            st[i] = strides[i];
        }
    }
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(map), CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void *>(base), d,
        st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
            : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool gemm_tcgen05_eligible(uint32_t M, uint32_t N, uint32_t K, const void *A, const void *B, uint32_t Kp,
    bool a_transposed)
{
    if (a_transposed || M == 0 || N == 0 || K == 0) {
        return false;
    }
    // TMA: 16-byte aligned bases and row pitches
    if ((K % 16) != 0 || (Kp % 16) != 0) {
        return false;
    }
    if ((reinterpret_cast<uintptr_t>(A) % 16) != 0 || (reinterpret_cast<uintptr_t>(B) % 16) != 0) {
        return false;
    }
    return encode_fn() != nullptr;
}

EE launch_gemm_tcgen05(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, const int8_t *B, uint32_t Kp,
    void *C, const GemmEpilogue &ep, cudaStream_t st)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, [] {
        const void *kernels[5] = {(const void *)gemm_u8s8_tcgen05_kernel<-1>, (const void *)gemm_u8s8_tcgen05_kernel<0>,
            (const void *)gemm_u8s8_tcgen05_kernel<1>, (const void *)gemm_u8s8_tcgen05_kernel<2>,
            (const void *)gemm_u8s8_tcgen05_kernel<3>};
        for (const void *k : kernels) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
            if (e != cudaSuccess) {
                attr_err = e;
            }
        }
    });
    B200_CUDA(attr_err);

    Params p;
    p.M = M;
    p.N = N;
    p.K = K;
    p.block_n = pick_block_n(M, N, c->sm_count);
    p.stages = (uint32_t)(SMEM_RING_BYTES / (SMEM_A_STAGE + (size_t)p.block_n * BLOCK_K));
    if (p.stages > (uint32_t)MAX_STAGES) {
        p.stages = MAX_STAGES;
    }
    p.tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
    p.tiles_n = (N + p.block_n - 1) / p.block_n;
    p.num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    p.C = C;
    p.ep = ep;
    p.status = c->d_status;
    const size_t esz = ep.out_kind == 2 ? 1 : 4;
    p.vec_ok = ((N * esz) % 16 == 0) && (reinterpret_cast<uintptr_t>(C) % 16 == 0);

    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, A, K, M, K, BLOCK_M) ||
        !make_map(&map_b, B, K, B200_ALIGN(N, 16), Kp, p.block_n)) {
        return NOT_SUPPORTED;
    }
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    const uint32_t grid = tiles < (uint32_t)c->sm_count ? tiles : (uint32_t)c->sm_count;
    // the fast epilogue needs whole, 16-byte aligned 32-column chunks, no read of C and one
    // conversion factor per column
    const bool fast = p.vec_ok && (N % 32 == 0) && !(ep.out_kind != 2 && ep.accumulate) &&
        !(ep.per_channel && ep.row_scale != nullptr);
    // u8 output: 32-row x 64-byte boxes, 64-byte swizzle, stored by TMA from the epilogue's staging
    CUtensorMap map_c = map_a;  // placeholder for the kinds that never touch it
    bool tma_c = false;
    if (fast && ep.out_kind == 2) {
        const uint64_t dims[2] = {N, M};
        const uint64_t strides[1] = {N};
        const uint32_t box[2] = {64, 32};
        const uint32_t estr[2] = {1, 1};
        tma_c = encode_tiled_u8(&map_c, 2, C, dims, strides, box, estr, 64);
    }
    if (!fast) {
        gemm_u8s8_tcgen05_kernel<-1><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
    } else if (ep.out_kind == 0) {
        gemm_u8s8_tcgen05_kernel<0><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
    } else if (ep.out_kind == 1) {
        gemm_u8s8_tcgen05_kernel<1><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
    } else if (tma_c) {
        gemm_u8s8_tcgen05_kernel<3><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
    } else {
        gemm_u8s8_tcgen05_kernel<2><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
    }
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

}  // namespace b200
