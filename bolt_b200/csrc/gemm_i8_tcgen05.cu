// gemm_i8_tcgen05.cu -- u8 x s8 -> s32 GEMM on the 5th-generation tensor cores of sm_100a.
//
//   C[M,N] = epilogue( offsetC[n] + sum_k A_u8[m,k] * B_s8[n,k] )        (both operands K-major)
//
// Replaces the AVX512-VNNI micro-kernels and their driver in Bolt
// (compute/blas_enhance/src/cpu/x86/int8/avx512/mmm_avx512_vnni.cpp:383-1891).
//
// One persistent CTA per SM, three roles:
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D loads of a 128 x 128-byte A tile and a
//               BLOCK_N x 128-byte B tile per pipeline stage, 128-byte swizzle, mbarrier complete_tx
//   warp 1      MMA issuer: one thread issues tcgen05.mma.cta_group::1.kind::i8 (M=128, N=BLOCK_N,
//               K=32 per instruction, A unsigned / B signed, int32 accumulate, no saturation) with
//               shared-memory matrix descriptors; accumulators live in tensor memory (2 x 256 columns,
//               so the epilogue of tile i overlaps the main loop of tile i+1)
//   warps 2..   epilogue.  The fast instantiations run 16 epilogue warps, four per scheduler: the four
//               warps that share a tensor-memory lane quadrant split the tile's columns (at most 64
//               each), read their whole share with tcgen05.ld, hand the accumulator back to the MMA
//               warp at once and only then convert: +offsetC, s32 -> f32, * factor as packed f32x2
//               operations, and for u8 the rounding by a biased add whose low byte is the result
//               (out-of-range values are detected by one OR per element and redone exactly).  u8 tiles
//               leave through swizzled staging and TMA stores.  The general instantiation (ragged N,
//               accumulate into C) keeps 8 epilogue warps and plain stores.
// Tiles are visited in groups of 16 row blocks x all column blocks, so that the CTAs of one wave
// share a few A and B panels in L2.  The kernel is launched with programmatic stream serialization:
// its set-up (barriers, tensor-memory allocation, descriptor prefetch) overlaps the tail of the
// previous kernel of the stream; nothing is read or written before griddepcontrol.wait.
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
#ifndef B200_EPI_WARPS_FAST
#define B200_EPI_WARPS_FAST 16
#endif
constexpr int EPI_WARPS_FAST = B200_EPI_WARPS_FAST;
constexpr int EPI_WARPS_GENERAL = 8;
constexpr uint32_t TMEM_COLS = 512;  // 2 accumulators x 256 columns
constexpr uint32_t GROUP_M = 16;     // row blocks per raster group

constexpr int SMEM_A_STAGE = BLOCK_M * BLOCK_K;        // 16 KiB
constexpr int CONST_SLOTS = 1024;    // per-warp column constants: EPI_WARPS x (256 / column groups)

struct __align__(16) SmemCtl {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    // per epilogue warp: offsetC and conversion factor of the columns it owns
    __align__(16) int32_t offs[CONST_SLOTS];
    __align__(16) float colf[CONST_SLOTS];
};

// 227 KiB per CTA: alignment slack + control block + staging + as many (A tile, B tile) stages as fit
constexpr size_t SMEM_BYTES = 232448;
// u8 tiles leave through TMA stores: each epilogue warp stages 32 rows x 32 bytes (32-byte swizzle)
constexpr int STAGING_PER_WARP = 32 * 32;
constexpr size_t SMEM_STAGING_BYTES = (size_t)EPI_WARPS_FAST * STAGING_PER_WARP;  // 16 KiB
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
    uint32_t prefetch_slice;  // bytes of ep.prefetch each CTA asks for (0: none)
    // scatter (u8 output through TMA stores only): every tile is stored into n_scatter destinations -- this GPU's
    // and its peers' copies of a wider [M][ld] matrix -- at column scatter_col0 + n; the tensor maps lie in
    // device memory
    const CUtensorMap *scatter_maps;
    uint32_t n_scatter, scatter_col0;
    // 1: the four warps of a lane quadrant assemble [32 rows][128 B] boxes (half the tile's width) so that the peers
    // receive 128-byte rows; needs 256-column tiles
    uint32_t scatter_wide;
};

// Raster: groups of GROUP_M row blocks, inside a group the row block runs fastest.
__device__ __forceinline__ void tile_coords(const Params &p, uint32_t tile, uint32_t &mb, uint32_t &nb)
{
    const uint32_t per_group = GROUP_M * p.tiles_n;
    const uint32_t g = tile / per_group;
    const uint32_t first = g * GROUP_M;
    const uint32_t gm = min(GROUP_M, p.tiles_m - first);
    const uint32_t r = tile - g * per_group;
    nb = r / gm;
    mb = first + (r - nb * gm);
}

// One tile of work: row block, first column, width in 32-column units (at most 8).
struct Tile {
    uint32_t mb, n0, units;
};
// The tiles of one worker (a CTA, or a CTA pair), in the order in which all its roles visit them: tile
// index = worker, worker + workers, ... in the grouped raster.
// (Cutting the columns into equal spans per SM instead of whole tiles -- no partly empty last wave -- was
// measured slower on the 4096 x 3072 x 768 shape: 13.5 us against 11.7 us per launch.)
struct TileWalk {
    uint32_t cur, end, step;
    uint32_t first, r;   // first row block of the current raster group, position inside the group
    __device__ __forceinline__ void init(const Params &p, uint32_t worker, uint32_t workers)
    {
        cur = worker;
        end = p.tiles_m * p.tiles_n;
        step = workers;
        const uint32_t per_group = GROUP_M * p.tiles_n;
        const uint32_t g = worker / per_group;
        first = g * GROUP_M;
        r = worker - g * per_group;
    }
    // every role of a CTA calls this once per tile; after the first call it costs no division (the roles
    // of a warp wait on one another through it, so it sits on the epilogue's critical path)
    __device__ __forceinline__ bool next(const Params &p, Tile &t)
    {
        if (cur >= end) {
            return false;
        }
        uint32_t gm = min(GROUP_M, p.tiles_m - first);
        while (r >= gm * p.tiles_n) {   // into the next raster group(s)
            r -= gm * p.tiles_n;
            first += gm;
            gm = min(GROUP_M, p.tiles_m - first);
        }
        uint32_t nb;
        if (gm == GROUP_M) {
            nb = r / GROUP_M;           // a shift
            t.mb = first + (r & (GROUP_M - 1));
        } else {
            nb = r / gm;
            t.mb = first + (r - nb * gm);
        }
        t.n0 = nb * p.block_n;
        t.units = p.block_n >> 5;
        cur += step;
        r += step;
        return true;
    }
};

// ---- epilogue for 32 consecutive columns of one row: the common case ---------------------------
// Full, 16-byte aligned chunk, C overwritten.  Per element: add offsetC, s32 -> f32 (vcvtdq2ps),
// multiply (vmulps), then for u8 the rounding of vcvtps2dq + vpaddd 128 + vpmovusdb.
//
// 32 accumulators of one row -> 32 bytes (8 words).  Per element: +offsetC, s32 -> f32 (vcvtdq2ps), * factor
// (vmulps), then vcvtps2dq + vpaddd 128 + vpmovusdb in one biased add: f + (1.5 * 2^23 + 128) has the bits
// 0x4B400000 + (rne(f) + 128) whenever -128 <= rne(f) <= 127 (the sum lies in [2^23, 2^24), where one ulp
// is 1 and ties go to the even sum, i.e. to even rne(f)), so the low byte is the result; every other
// input -- too large, too negative, NaN, infinity -- leaves other upper bits.  Returns the OR of
// (bits ^ 0x4B400000) over the chunk: above 255 means that some element needs the exact clamp.
// Written stage by stage over the whole chunk, in place and without a branch, so that the 32 elements
// overlap: an epilogue warp works through its tiles one after the other and the latency of this routine
// is what paces the kernel when K is short.
template <bool ROWS>
__device__ __forceinline__ uint32_t chunk_to_u8_quick(const int32_t *offs, const float *colf, uint32_t cl, float num, float rs,
    uint32_t (&r)[32], uint32_t (&w)[8])
{
    constexpr uint32_t BIAS_BITS = 0x4B400000u;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
        r[j] += (uint32_t)o.x;
        r[j + 1] += (uint32_t)o.y;
        r[j + 2] += (uint32_t)o.z;
        r[j + 3] += (uint32_t)o.w;
    }
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
        if (ROWS) {
            c4.x = __fdiv_rn(num, __fmul_rn(rs, c4.x));
            c4.y = __fdiv_rn(num, __fmul_rn(rs, c4.y));
            c4.z = __fdiv_rn(num, __fmul_rn(rs, c4.z));
            c4.w = __fdiv_rn(num, __fmul_rn(rs, c4.w));
        }
        r[j] = __float_as_uint(__fadd_rn(__fmul_rn(__int2float_rn((int)r[j]), c4.x), 12583040.0f));
        r[j + 1] = __float_as_uint(__fadd_rn(__fmul_rn(__int2float_rn((int)r[j + 1]), c4.y), 12583040.0f));
        r[j + 2] = __float_as_uint(__fadd_rn(__fmul_rn(__int2float_rn((int)r[j + 2]), c4.z), 12583040.0f));
        r[j + 3] = __float_as_uint(__fadd_rn(__fmul_rn(__int2float_rn((int)r[j + 3]), c4.w), 12583040.0f));
    }
    uint32_t s8[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        s8[q] = (r[4 * q] ^ BIAS_BITS) | (r[4 * q + 1] ^ BIAS_BITS) | (r[4 * q + 2] ^ BIAS_BITS) | (r[4 * q + 3] ^ BIAS_BITS);
        w[q] = __byte_perm(__byte_perm(r[4 * q], r[4 * q + 1], 0x0040), __byte_perm(r[4 * q + 2], r[4 * q + 3], 0x0040), 0x5410);
    }
    return ((s8[0] | s8[1]) | (s8[2] | s8[3])) | ((s8[4] | s8[5]) | (s8[6] | s8[7]));
}
// The same chunk with the exact clamp (any input).  Rare -- an element beyond the u8 range means that the
// output scale does not fit the data -- so it is kept out of line and fetches the accumulators again from
// tensor memory (the caller has not handed the accumulator back yet).  Called by whole warps.
struct Words8 {
    uint32_t w[8];
};
template <bool ROWS>
__device__ __noinline__ Words8 chunk_to_u8_exact(uint32_t taddr, const int32_t *offs, const float *colf, uint32_t cl,
    float num, float rs)
{
    uint32_t r[32];
    tmem_ld32(taddr, r);
    tmem_ld_wait(r);
    Words8 out;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
        float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
        if (ROWS) {
            c4.x = __fdiv_rn(num, __fmul_rn(rs, c4.x));
            c4.y = __fdiv_rn(num, __fmul_rn(rs, c4.y));
            c4.z = __fdiv_rn(num, __fmul_rn(rs, c4.z));
            c4.w = __fdiv_rn(num, __fmul_rn(rs, c4.w));
        }
        const uint32_t b0 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j] + o.x), c4.x));
        const uint32_t b1 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j + 1] + o.y), c4.y));
        const uint32_t b2 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j + 2] + o.z), c4.z));
        const uint32_t b3 = f32_to_u8_zp128(__fmul_rn(__int2float_rn((int)r[j + 3] + o.w), c4.w));
        out.w[j >> 2] = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
    }
    return out;
}
// 32 bytes of row `lane` into the warp's staging box [32 rows][32 B], 32-byte swizzle: the 16-byte
// chunk index is XORed with bit 2 of the row (address bit 7 into bit 4), the pattern the TMA store undoes
__device__ __forceinline__ void stage_u8(uint8_t *stg, uint32_t lane, const uint32_t (&w)[8])
{
    const uint32_t sw = (lane >> 2) & 1;
    uint8_t *row = stg + lane * 32;
    *reinterpret_cast<uint4 *>(row + ((0 ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4 *>(row + ((1 ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}

// KIND 0 s32, 1 f32, 2 u8: direct 16-byte stores of one row's 32 columns
template <int KIND, bool ROWS>
__device__ __forceinline__ void store_chunk_fast(void *C, uint32_t N, const int32_t *offs, const float *colf, float num,
    float rs, uint32_t m, uint32_t n0, uint32_t cl, const uint32_t (&r)[32])
{
    const size_t row_off = (size_t)m * N + n0;
    if (KIND == 1) {
        float *out = reinterpret_cast<float *>(C) + row_off;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
            float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
            if (ROWS) {
                c4.x = __fdiv_rn(num, __fmul_rn(rs, c4.x));
                c4.y = __fdiv_rn(num, __fmul_rn(rs, c4.y));
                c4.z = __fdiv_rn(num, __fmul_rn(rs, c4.z));
                c4.w = __fdiv_rn(num, __fmul_rn(rs, c4.w));
            }
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
// (ragged or unaligned N, accumulate into C)
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
// swizzled staging + TMA stores described by map_c), ROWS: one activation scale per row; KIND < 0: the
// general epilogue.  EW = number of epilogue warps (a multiple of 4).
//
// PAIR: the grid is launched as clusters of two CTAs that share one tcgen05.mma.cta_group::2 of 256 rows:
// CTA r of the pair loads its own 128 rows of A and half of the B tile's rows, so every SM fetches
// (128 + BLOCK_N / 2) x 128 bytes per stage instead of (128 + BLOCK_N) x 128 -- the main loop is bound by
// the operand bytes an SM can take in per clock, and this is a third less of them.  The CTA of cluster
// rank 0 issues the MMAs for both and signals both through tcgen05.commit to the two CTAs' barriers;
// every load completes on the leader's barrier; each CTA reads its own 128 accumulator rows.
template <int KIND, bool ROWS, int EW, bool PAIR>
__global__ void __launch_bounds__(64 + EW * 32, 1)
gemm_u8s8_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
    const __grid_constant__ CUtensorMap map_c, const Params p)
{
    constexpr uint32_t GROUPS = EW / 4;                 // column groups per lane quadrant
    constexpr uint32_t SLOTS = CONST_SLOTS / EW;        // constants per warp: 64 (16 warps) or 128 (8 warps)
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte aligned bases
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    const uint32_t b_rows = PAIR ? (p.block_n >> 1) : p.block_n;  // rows of a full B tile this CTA holds
    const uint32_t b_stage = (b_rows * BLOCK_K + 1023u) & ~1023u;  // every stage stays 1024-byte aligned
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const uint32_t worker = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
    const uint32_t workers = PAIR ? (gridDim.x >> 1) : gridDim.x;
    uint8_t *smem_b = smem + p.stages * SMEM_A_STAGE;
    uint8_t *smem_staging = smem + SMEM_RING_BYTES;  // 1024-byte aligned
    SmemCtl *ctl = reinterpret_cast<SmemCtl *>(smem + SMEM_RING_BYTES + SMEM_STAGING_BYTES);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (KIND == 3) {
            prefetch_tensormap(&map_c);
        }
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&ctl->tmem_full[a], 1);
            // one arrival per epilogue warp (of both CTAs in pair mode), whether or not it owns columns
            mbar_init(&ctl->tmem_empty[a], (PAIR ? 2 : 1) * EW);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            // the same warp of both CTAs of the pair allocates
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&ctl->tmem_base)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&ctl->tmem_base)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    // the next kernel of the stream may start its own set-up now; it reads nothing before its wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) {
        cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    }
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    // everything the previous kernels of the stream wrote is visible after this
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // this CTA's slice of the memory a later kernel will read, requested once the pipeline is filled
            uint32_t issued = 0;
            const uint32_t fill = min(p.stages, p.num_kb);
            TileWalk walk;
            walk.init(p, worker, workers);
            Tile t;
            while (ok && walk.next(p, t)) {
                const int m0 = (int)((PAIR ? 2 * t.mb + rank : t.mb) * BLOCK_M);
                const uint32_t my_rows = PAIR ? (t.units * 16) : (t.units * 32);  // B rows this CTA loads
                const int n0 = (int)(t.n0 + rank * my_rows);
                const uint32_t tile_bytes = (PAIR ? 2u : 1u) * (BLOCK_M + my_rows) * BLOCK_K;
                for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem_a + stage * SMEM_A_STAGE;
                    uint8_t *sb = smem_b + stage * b_stage;
                    if (PAIR) {
                        // both CTAs' bytes are expected by, and complete on, the leader's barrier
                        const uint32_t bar = mapa_shared(smem_u32(&ctl->full[stage]), 0);
                        if (rank == 0) {
                            mbar_expect_tx(&ctl->full[stage], tile_bytes);
                        }
                        tma_load_2d_pair(&map_a, bar, sa, (int)(kb * BLOCK_K), m0);
                        tma_load_2d_pair(&map_b, bar, sb, (int)(kb * BLOCK_K), n0);
                    } else {
                        mbar_expect_tx(&ctl->full[stage], tile_bytes);
                        tma_load_2d(&map_a, &ctl->full[stage], sa, (int)(kb * BLOCK_K), m0);
                        tma_load_2d(&map_b, &ctl->full[stage], sb, (int)(kb * BLOCK_K), n0);
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                    if (++issued == fill && p.prefetch_slice != 0) {
                        const size_t off = (size_t)blockIdx.x * p.prefetch_slice;
                        if (off < p.ep.prefetch_bytes) {
                            const size_t n = min((size_t)p.prefetch_slice, p.ep.prefetch_bytes - off) & ~(size_t)15;
                            if (n != 0) {
                                prefetch_l2_bulk(reinterpret_cast<const uint8_t *>(p.ep.prefetch) + off, (uint32_t)n);
                            }
                        }
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
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;
            bool ok = true;
            TileWalk walk;
            walk.init(p, worker, workers);
            Tile t;
            for (; ok && walk.next(p, t); ++it) {
                const uint32_t idesc = make_idesc_i8(t.units * 32, PAIR ? 2 * BLOCK_M : BLOCK_M);
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
                        if (PAIR) {
                            umma_i8_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        } else {
                            umma_i8(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    // frees the stage (in both CTAs) once these MMAs retire
                    if (PAIR) {
                        tcgen05_commit_pair(&ctl->empty[stage]);
                    } else {
                        tcgen05_commit(&ctl->empty[stage]);
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    break;
                }
                if (PAIR) {
                    tcgen05_commit_pair(&ctl->tmem_full[acc]);
                } else {
                    tcgen05_commit(&ctl->tmem_full[acc]);
                }
            }
            if (!ok) {
                atomicExch(p.status, 2);
                atomicExch(&ctl->abort_flag, 1u);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------- epilogue warps -----------------------------------------
        const uint32_t ew = warp - 2;
        const uint32_t quad = warp & 3;   // tensor-memory lane quadrant this warp may read
        const uint32_t grp = ew >> 2;     // which share of the tile's columns
        uint8_t *stg = smem_staging + ew * STAGING_PER_WARP;
        const GemmEpilogue &ep = p.ep;
        // Column constants (offsetC and the conversion factor): every warp keeps those of its own
        // columns in its own slice of shared memory, lane l owning columns l, l+32, ... of the warp's
        // range.  The next tile's values are fetched into registers before the current accumulator
        // is awaited and written after the tile's chunks, so neither the global-load latency nor any
        // CTA-wide barrier sits between two tiles; warps drift freely.  The loads are volatile asm
        // so that they stay where they are written (early); everything that depends on them is
        // written after the tile's chunks (late).
        int32_t *offs = ctl->offs + ew * SLOTS;
        float *colf = ctl->colf + ew * SLOTS;
        constexpr int NQ = SLOTS / 32;
        // this warp's 32-column chunks [c_begin, c_end) of a tile that is `units` chunks wide
        auto my_chunks = [&](uint32_t units, uint32_t &c_begin, uint32_t &c_end) {
            const uint32_t cpg = (units + GROUPS - 1) / GROUPS;
            c_begin = min(units, grp * cpg);
            c_end = min(units, c_begin + cpg);
        };
        constexpr bool wide = KIND == 4;  // scatter with 128-byte rows (its own instantiation: the common u8 path stays lean)
        bool dead = false;  // wide scatter only: after a failed wait the warp still meets its quadrant's barriers
        auto fetch_raw = [&](uint32_t tile_n0, uint32_t n_first, uint32_t cols, int32_t (&o)[NQ], float (&sb)[NQ]) {
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                o[q] = 0;
                sb[q] = ep.sB;
                const uint32_t j = lane + 32 * q;
                // wide scatter: slots 0-31 belong to chunk grp, slots 32-63 to chunk 4 + grp of the tile
                const uint32_t n = wide ? tile_n0 + (((q == 0 ? grp : 4u + grp)) << 5) + lane : n_first + j;
                if (j < cols && n < p.N) {
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
        auto park = [&](const int32_t (&o)[NQ], const float (&sb)[NQ]) {
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                offs[lane + 32 * q] = o[q];
                colf[lane + 32 * q] = factor_of(sb[q]);
            }
            __syncwarp();
        };
        // where this warp reports an accumulator as read: the leader's barrier
        const uint32_t empty_bar[2] = {PAIR ? mapa_shared(smem_u32(&ctl->tmem_empty[0]), 0) : smem_u32(&ctl->tmem_empty[0]),
            PAIR ? mapa_shared(smem_u32(&ctl->tmem_empty[1]), 0) : smem_u32(&ctl->tmem_empty[1])};
        auto release = [&](uint32_t acc) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) {
                    mbar_arrive_cluster(empty_bar[acc]);
                } else {
                    mbar_arrive(&ctl->tmem_empty[acc]);
                }
            }
        };
        TileWalk walk;
        walk.init(p, worker, workers);
        Tile t, t_next;
        bool have = walk.next(p, t);
        if (have) {
            int32_t o[NQ];
            float sb[NQ];
            uint32_t cb, ce;
            my_chunks(t.units, cb, ce);
            fetch_raw(t.n0, t.n0 + cb * 32, wide ? 64u : (ce - cb) * 32, o, sb);
            park(o, sb);
        }
        for (uint32_t it = 0; have; ++it) {
            const uint32_t acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const uint32_t m0 = (PAIR ? 2 * t.mb + rank : t.mb) * BLOCK_M;
            const uint32_t n0 = t.n0;
            uint32_t c_begin, c_end;
            my_chunks(t.units, c_begin, c_end);
            if (*reinterpret_cast<volatile uint32_t *>(&ctl->abort_flag) != 0) {
                if (!wide) {
                    break;  // some role's bounded wait ran out
                }
                dead = true;
            }
            const bool have_next = walk.next(p, t_next);
            int32_t o_next[NQ];
            float sb_next[NQ];
            const bool new_cols = have_next && (t_next.n0 != t.n0 || t_next.units != t.units);
            if (new_cols) {
                uint32_t cb, ce;
                my_chunks(t_next.units, cb, ce);
                fetch_raw(t_next.n0, t_next.n0 + cb * 32, wide ? 64u : (ce - cb) * 32, o_next, sb_next);
            }
            const uint32_t m = m0 + quad * 32 + lane;
            const bool row_ok = m < p.M;
            // rows beyond M get a harmless scale: a zero would turn their factors into infinities and send every
            // chunk of a partly filled row block through the exact conversion (their bytes are never stored)
            float rs = 1.f;
            if (ROWS && row_ok) {
                rs = ep.row_scale[m];
            }
            bool ok = dead ? true : mbar_wait(&ctl->tmem_full[acc], acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) {
                    atomicExch(p.status, 3);
                    atomicExch(&ctl->abort_flag, 1u);
                }
                if (!wide) {
                    break;
                }
                dead = true;
            }
            tcgen05_fence_after();
            const uint32_t tbase = tmem_base + ((quad * 32u) << 16) + acc * MAX_BLOCK_N;
            if (wide) {
                // Scatter with 128-byte rows: in pass 0 the warps of this lane quadrant convert chunks 0-3 (chunk
                // = column group), in pass 1 chunks 4-7; each pass fills the quadrant's [32 rows][128 B] box
                // (128-byte swizzle) and one thread stores it to every destination.
                uint8_t *box = smem_staging + quad * 4096;
                const uint32_t bar_id = 1 + quad;
                uint32_t ra[32], w[8];
#pragma unroll 1
                for (uint32_t pass = 0; pass < 2; ++pass) {
                    if (!dead) {
                        const uint32_t c = pass * 4 + grp;
                        const uint32_t cl = pass * 32;
                        tmem_ld32(tbase + c * 32, ra);
                        tmem_ld_wait(ra);
                        const uint32_t seen = chunk_to_u8_quick<ROWS>(offs, colf, cl, ep.num, rs, ra, w);
                        if (__any_sync(0xffffffffu, seen > 255u)) {
                            const Words8 e = chunk_to_u8_exact<ROWS>(tbase + c * 32, offs, colf, cl, ep.num, rs);
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                w[q] = e.w[q];
                            }
                        }
                        if (pass == 1) {
                            release(acc);
                        }
                        if (grp == 0 && lane == 0) {
                            tma_store_wait_read();  // the stores of the previous box have read it
                        }
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                    if (!dead) {
                        uint8_t *row = box + lane * 128;
                        const uint32_t sw = lane & 7;
                        *reinterpret_cast<uint4 *>(row + (((2 * grp) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4 *>(row + (((2 * grp + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
                        fence_proxy_async_smem();
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                    if (!dead && grp == 0 && lane == 0) {
                        for (uint32_t q = 0; q < p.n_scatter; ++q) {
                            tma_store_2d(p.scatter_maps + q, box, (int)(p.scatter_col0 + n0 + pass * 128), (int)(m0 + quad * 32));
                        }
                    }
                }
            } else if (c_begin >= c_end) {
                release(acc);  // no columns of this tile: only the hand-back
            } else if (KIND >= 2) {
                // u8 output, one 32-column chunk at a time (at most two per warp; the other warps of the scheduler
                // cover the tensor-memory read latency, and 32 live accumulators keep the warp within its register
                // share).  The accumulator goes back to the MMA warp after the last chunk's range check (the rare
                // exact conversion reads it again).
                uint32_t ra[32], w[8];
                for (uint32_t c = c_begin; c < c_end; ++c) {
                    const uint32_t cl = (c - c_begin) * 32;
                    tmem_ld32(tbase + c * 32, ra);
                    tmem_ld_wait(ra);
                    const uint32_t seen = chunk_to_u8_quick<ROWS>(offs, colf, cl, ep.num, rs, ra, w);
                    if (__any_sync(0xffffffffu, seen > 255u)) {
                        const Words8 e = chunk_to_u8_exact<ROWS>(tbase + c * 32, offs, colf, cl, ep.num, rs);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            w[q] = e.w[q];
                        }
                    }
                    if (c + 1 == c_end) {
                        release(acc);  // accumulator fully read: the MMA may reuse it
                    }
                    if (KIND == 3) {
                        // the previous box must have left the staging buffer
                        if (lane == 0) {
                            tma_store_wait_read();
                        }
                        __syncwarp();
                        stage_u8(stg, lane, w);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            // rows beyond M are clipped by the tensor map
                            if (p.n_scatter == 0) {
                                tma_store_2d(&map_c, stg, (int)(n0 + c * 32), (int)(m0 + quad * 32));
                            } else {
                                // the same box to every destination (plain stores over NVLink for the peers')
                                for (uint32_t q = 0; q < p.n_scatter; ++q) {
                                    tma_store_2d(p.scatter_maps + q, stg, (int)(p.scatter_col0 + n0 + c * 32), (int)(m0 + quad * 32));
                                }
                            }
                        }
                    } else if (row_ok) {
                        uint8_t *out = reinterpret_cast<uint8_t *>(p.C) + (size_t)m * p.N + n0 + c * 32;
                        *reinterpret_cast<uint4 *>(out) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4 *>(out + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                }
            } else if (KIND >= 0) {
                // s32 / f32 output: one 32-column chunk at a time
                uint32_t ra[32];
                for (uint32_t c = c_begin; c < c_end; ++c) {
                    const uint32_t cl = (c - c_begin) * 32;
                    tmem_ld32(tbase + c * 32, ra);
                    tmem_ld_wait(ra);
                    if (c + 1 == c_end) {
                        release(acc);  // accumulator fully read: the MMA may reuse it
                    }
                    if (row_ok) {
                        store_chunk_fast<KIND, ROWS>(p.C, p.N, offs, colf, ep.num, rs, m, n0 + c * 32, cl, ra);
                    }
                }
            } else {
                uint32_t ra[32];
                for (uint32_t c = c_begin; c < c_end; ++c) {
                    tmem_ld32(tbase + c * 32, ra);
                    tmem_ld_wait(ra);
                    if (row_ok && n0 + c * 32 < p.N) {
                        store_chunk(p, offs, colf, m, n0 + c * 32, (c - c_begin) * 32, ra);
                    }
                }
                release(acc);
            }
            if (new_cols) {
                __syncwarp();  // every lane is done reading this tile's constants
                park(o_next, sb_next);
            }
            t = t_next;
            have = have_next;
        }
        if (KIND >= 3 && lane == 0) {
            // the staging buffer must have been read before the CTA's shared memory goes away; the
            // stores themselves complete before the grid does
            tma_store_wait_read();
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
    if (PAIR) {
        // neither CTA may leave (or free tensor memory) while its peer can still read its shared
        // memory through the MMA or arrive on its barriers
        tcgen05_fence_before();
        cluster_sync_all();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        if (PAIR) {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                         : "memory");
        } else {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                         : "memory");
        }
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
uint32_t pick_block_n(uint32_t tiles_m, uint32_t N, int sms)
{
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
            : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                  : (swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE)),
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

namespace {

// One launch, with programmatic stream serialization unless BOLT_B200_NO_PDL is set in the environment
// (or the runtime refuses the attribute, in which case the plain launch is used from then on).
// PAIR launches clusters of two CTAs.
std::atomic<int> g_pdl{-1};

template <int KIND, bool ROWS, int EW, bool PAIR>
cudaError_t launch_one(uint32_t grid, cudaStream_t st, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc,
    const Params &p)
{
    int pdl = g_pdl.load(std::memory_order_relaxed);
    if (pdl < 0) {
        const char *e = getenv("BOLT_B200_NO_PDL");
        pdl = (e != nullptr && e[0] != '\0' && e[0] != '0') ? 0 : 1;
        g_pdl.store(pdl, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(64 + EW * 32);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    int n = 0;
    if (PAIR) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = 2;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    const int base = n;
    if (pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_u8s8_tcgen05_kernel<KIND, ROWS, EW, PAIR>, ma, mb, mc, p);
    if (e != cudaSuccess && pdl) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(st, &cap);
        if (cap == cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            g_pdl.store(0, std::memory_order_relaxed);
            cfg.numAttrs = base;
            e = cudaLaunchKernelEx(&cfg, gemm_u8s8_tcgen05_kernel<KIND, ROWS, EW, PAIR>, ma, mb, mc, p);
        }
    }
    return e;
}

template <bool PAIR>
cudaError_t launch_kind(int kind, bool rows, uint32_t grid, cudaStream_t st, const CUtensorMap &ma, const CUtensorMap &mb,
    const CUtensorMap &mc, const Params &p)
{
    constexpr int F = EPI_WARPS_FAST;
    switch (kind) {
        case 0:
            return launch_one<0, false, F, PAIR>(grid, st, ma, mb, mc, p);
        case 1:
            return rows ? launch_one<1, true, F, PAIR>(grid, st, ma, mb, mc, p) : launch_one<1, false, F, PAIR>(grid, st, ma, mb, mc, p);
        case 2:
            return rows ? launch_one<2, true, F, PAIR>(grid, st, ma, mb, mc, p) : launch_one<2, false, F, PAIR>(grid, st, ma, mb, mc, p);
        case 4:
            return rows ? launch_one<4, true, F, PAIR>(grid, st, ma, mb, mc, p) : launch_one<4, false, F, PAIR>(grid, st, ma, mb, mc, p);
        default:
            return rows ? launch_one<3, true, F, PAIR>(grid, st, ma, mb, mc, p) : launch_one<3, false, F, PAIR>(grid, st, ma, mb, mc, p);
    }
}

// How many CTA pairs of the tensor-core kernel the device runs at once (each CTA fills an SM).
int max_resident_pairs(DeviceCtx *c)
{
    std::lock_guard<std::mutex> g(c->attr_mu);
    if (c->max_pairs < 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)c->sm_count);
        cfg.blockDim = dim3(64 + EPI_WARPS_FAST * 32);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_u8s8_tcgen05_kernel<3, false, EPI_WARPS_FAST, true>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        c->max_pairs = n;
    }
    return c->max_pairs;
}

}  // namespace

EE launch_gemm_tcgen05(uint32_t M, uint32_t N, uint32_t K, const uint8_t *A, const int8_t *B, uint32_t Kp,
    void *C, const GemmEpilogue &ep, cudaStream_t st)
{
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    {
        constexpr int F = EPI_WARPS_FAST, G = EPI_WARPS_GENERAL;
        const void *kernels[] = {(const void *)gemm_u8s8_tcgen05_kernel<-1, false, G, false>,
            (const void *)gemm_u8s8_tcgen05_kernel<0, false, F, false>, (const void *)gemm_u8s8_tcgen05_kernel<1, false, F, false>,
            (const void *)gemm_u8s8_tcgen05_kernel<2, false, F, false>, (const void *)gemm_u8s8_tcgen05_kernel<3, false, F, false>,
            (const void *)gemm_u8s8_tcgen05_kernel<1, true, F, false>, (const void *)gemm_u8s8_tcgen05_kernel<2, true, F, false>,
            (const void *)gemm_u8s8_tcgen05_kernel<3, true, F, false>,
            (const void *)gemm_u8s8_tcgen05_kernel<0, false, F, true>, (const void *)gemm_u8s8_tcgen05_kernel<1, false, F, true>,
            (const void *)gemm_u8s8_tcgen05_kernel<2, false, F, true>, (const void *)gemm_u8s8_tcgen05_kernel<3, false, F, true>,
            (const void *)gemm_u8s8_tcgen05_kernel<1, true, F, true>, (const void *)gemm_u8s8_tcgen05_kernel<2, true, F, true>,
            (const void *)gemm_u8s8_tcgen05_kernel<3, true, F, true>,
            (const void *)gemm_u8s8_tcgen05_kernel<4, false, F, false>, (const void *)gemm_u8s8_tcgen05_kernel<4, true, F, false>,
            (const void *)gemm_u8s8_tcgen05_kernel<4, false, F, true>, (const void *)gemm_u8s8_tcgen05_kernel<4, true, F, true>};
        B200_EE(raise_smem_limit(c, KF_GEMM, kernels, (int)(sizeof(kernels) / sizeof(kernels[0])), SMEM_BYTES));
    }

    Params p;
    p.M = M;
    p.N = N;
    p.K = K;
    p.C = C;
    p.ep = ep;
    p.status = c->d_status;
    const size_t esz = ep.out_kind == 2 ? 1 : 4;
    p.vec_ok = ((N * esz) % 16 == 0) && (reinterpret_cast<uintptr_t>(C) % 16 == 0);
    // the fast epilogue needs whole, 16-byte aligned 32-column chunks and no read of C
    const bool rows = ep.per_channel && ep.row_scale != nullptr;
    const bool fast = p.vec_ok && (N % 32 == 0) && !(ep.out_kind != 2 && ep.accumulate) && !(rows && ep.out_kind == 0);
    // CTA pairs: at least two 128-row blocks, a long K (the pair's cluster set-up and its joint first
    // load cost about a microsecond, which only a main loop of many stages pays back), and a device
    // that can co-schedule pairs
    static const bool no_pair = [] {
        const char *e = getenv("BOLT_B200_NO_PAIR");
        return e != nullptr && e[0] != '\0' && e[0] != '0';
    }();
    const int pairs = (fast && M >= 256 && K >= 4096 && !no_pair) ? max_resident_pairs(c) : 0;
    const bool pair = pairs > 0;
    const uint32_t block_m = pair ? 2 * BLOCK_M : BLOCK_M;
    p.tiles_m = (M + block_m - 1) / block_m;
    p.block_n = pick_block_n(p.tiles_m, N, pair ? pairs : c->sm_count);
    // scatter with 128-byte rows needs whole 256-column tiles
    static const bool no_wide = [] {
        const char *e = getenv("BOLT_B200_NO_WIDE_SCATTER");
        return e != nullptr && e[0] != '\0' && e[0] != '0';
    }();
    const bool wide_scatter = ep.scatter_n > 0 && fast && ep.out_kind == 2 && N % 256 == 0 && !no_wide;
    if (wide_scatter) {
        p.block_n = 256;
    }
    const uint32_t b_rows = pair ? p.block_n / 2 : p.block_n;
    p.stages = (uint32_t)(SMEM_RING_BYTES / (SMEM_A_STAGE + B200_ALIGN((size_t)b_rows * BLOCK_K, 1024)));
    if (p.stages > (uint32_t)MAX_STAGES) {
        p.stages = MAX_STAGES;
    }
    p.tiles_n = (N + p.block_n - 1) / p.block_n;
    p.num_kb = (K + BLOCK_K - 1) / BLOCK_K;

    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, A, K, M, K, BLOCK_M) ||
        !make_map(&map_b, B, K, B200_ALIGN(N, 16), Kp, b_rows)) {
        return NOT_SUPPORTED;
    }
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    const uint32_t workers = pair ? (uint32_t)pairs : (uint32_t)c->sm_count;
    const uint32_t grid = (tiles < workers ? tiles : workers) * (pair ? 2u : 1u);
    // u8 output: 32-row x 32-byte boxes, 32-byte swizzle, stored by TMA from the epilogue's staging
    CUtensorMap map_c = map_a;  // placeholder for the kinds that never touch it
    bool tma_c = false;
    if (fast && ep.out_kind == 2) {
        const uint64_t dims[2] = {N, M};
        const uint64_t strides[1] = {N};
        const uint32_t box[2] = {32, 32};
        const uint32_t estr[2] = {1, 1};
        tma_c = encode_tiled_u8(&map_c, 2, C, dims, strides, box, estr, 32);
    }
    p.scatter_maps = nullptr;
    p.n_scatter = 0;
    p.scatter_col0 = 0;
    p.scatter_wide = 0;
    if (ep.scatter_n > 0) {
        // one tensor map per destination over its [M][ld] matrix, kept in a small per-device array
        if (!fast || ep.out_kind != 2 || ep.scatter_n > 8 || ep.scatter_ld % 16 != 0 || ep.scatter_col0 % 32 != 0 ||
            ep.scatter_col0 + N > ep.scatter_ld) {
            return NOT_SUPPORTED;
        }
        CUtensorMap maps[8];
        for (uint32_t q = 0; q < ep.scatter_n; ++q) {
            const uint64_t dims[2] = {ep.scatter_ld, M};
            const uint64_t strides[1] = {ep.scatter_ld};
            const uint32_t box[2] = {wide_scatter ? 128u : 32u, 32};
            const uint32_t estr[2] = {1, 1};
            if (ep.scatter_dst[q] == nullptr || (reinterpret_cast<uintptr_t>(ep.scatter_dst[q]) % 16) != 0 ||
                !encode_tiled_u8(&maps[q], 2, ep.scatter_dst[q], dims, strides, box, estr, wide_scatter ? 128 : 32)) {
                return NOT_SUPPORTED;
            }
        }
        if (c->d_scatter_maps == nullptr) {
            B200_CUDA(cudaMalloc(&c->d_scatter_maps, 8 * sizeof(CUtensorMap)));
        }
        // (the source is pageable host memory: the call returns once it has been staged)
        B200_CUDA(cudaMemcpyAsync(c->d_scatter_maps, maps, ep.scatter_n * sizeof(CUtensorMap), cudaMemcpyHostToDevice, st));
        p.scatter_maps = reinterpret_cast<const CUtensorMap *>(c->d_scatter_maps);
        p.n_scatter = ep.scatter_n;
        p.scatter_col0 = ep.scatter_col0;
        p.scatter_wide = wide_scatter ? 1u : 0u;
        tma_c = true;  // the scatter maps replace map_c
    }
    p.prefetch_slice = 0;
    if (ep.prefetch != nullptr && ep.prefetch_bytes >= 16 && (reinterpret_cast<uintptr_t>(ep.prefetch) % 16) == 0) {
        // at most 64 MiB (half of L2), split evenly over the CTAs in 16-byte units
        const size_t bytes = ep.prefetch_bytes < ((size_t)64 << 20) ? ep.prefetch_bytes : ((size_t)64 << 20);
        p.ep.prefetch_bytes = bytes;
        p.prefetch_slice = (uint32_t)B200_ALIGN((bytes + grid - 1) / grid, 16);
    }
    cudaError_t e;
    if (!fast) {
        e = launch_one<-1, false, EPI_WARPS_GENERAL, false>(grid, st, map_a, map_b, map_c, p);
    } else {
        const int kind = ep.out_kind == 2 ? (p.scatter_wide ? 4 : (tma_c ? 3 : 2)) : ep.out_kind;
        e = pair ? launch_kind<true>(kind, rows, grid, st, map_a, map_b, map_c, p)
                 : launch_kind<false>(kind, rows, grid, st, map_a, map_b, map_c, p);
    }
    count_launch();
    B200_CUDA(e);
    return SUCCESS;
}

}  // namespace b200
