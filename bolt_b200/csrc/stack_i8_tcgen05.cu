// stack_i8_tcgen05.cu -- a whole stack of quantized linear layers as ONE persistent kernel.
//
// Layer l:  C_l[M, N_l] = requant( offsetC_l[n] + sum_k C_{l-1}[m,k] * W_l[n,k] ),  C_{-1} = A0 (u8)
//
// What it replaces: one matrix_matrix_multiply per layer (Bolt runs a network operator by operator,
// inference/engine/src/cnn.cpp:611-675).  On this GPU a 4096 x 3072 x 768 layer is ~7 us of tensor-core
// work; a kernel launch per layer costs a pipeline fill and a drain each (a quarter of the layer)
// and leaves a partial last wave on 148 SMs.  Here 148 CTAs (cooperative launch, one per SM) walk
// the tiles of all layers in one fixed order -- layer-major, and inside a layer row-block-major --
// so the tensor pipe never drains between layers.  The only coupling between layers is by row block:
// a tile of layer l may load its A rows once every tile of layer l-1 in the same 128-row block has
// stored its output.  Each epilogue warp adds 1 to a per-(layer, row-block) counter when its stores
// are complete; the TMA producer of a dependent tile spins (bounded) on that counter.  Because every
// tile only depends on tiles that come earlier in the common order and all CTAs are resident, the
// walk cannot deadlock.
//
// Tile pipeline, warp roles, tensor-memory double buffering and the epilogue arithmetic are those
// of gemm_i8_tcgen05.cu (u8 output: swizzled staging + TMA stores; fp32 output: direct stores).
#include <cuda.h>

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
constexpr int MAX_LAYERS = 32;
constexpr int SMEM_A_STAGE = BLOCK_M * BLOCK_K;
constexpr int SMEM_B_STAGE = MAX_BLOCK_N * BLOCK_K;
constexpr int STAGING_PER_WARP = 32 * 64;

struct LayerDev {
    uint32_t N, K;
    uint32_t block_n, tiles_n, num_kb;
    uint32_t out_kind;    // 1 fp32, 2 u8
    uint32_t tile_begin;  // index of the layer's first tile in the common order
    uint32_t dep_target;  // counter value of a finished row block: tiles_n * EPI_WARPS
    const int32_t *offs;  // [N]
    const float *colf;    // [N]
    void *C;
};

struct __align__(16) SmemCtl {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    __align__(16) int32_t offs[EPI_WARPS][128];
    __align__(16) float colf[EPI_WARPS][128];
    LayerDev layers[MAX_LAYERS];
};

constexpr size_t SMEM_RING = (size_t)STAGES * (SMEM_A_STAGE + SMEM_B_STAGE);
constexpr size_t SMEM_STAGING = (size_t)EPI_WARPS * STAGING_PER_WARP;
constexpr size_t SMEM_BYTES = 1024 + SMEM_RING + SMEM_STAGING + sizeof(SmemCtl);
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

struct StackParams {
    uint32_t M, tiles_m, total_tiles, n_layers;
    const CUtensorMap *maps;  // device memory: {A, B, C} per layer
    const LayerDev *layers;   // device memory
    unsigned *done;           // [n_layers][tiles_m], zero at launch
    int *status;
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned *p, unsigned v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin on a progress counter written by other CTAs of this (cooperative) grid
__device__ __forceinline__ bool wait_counter(const unsigned *p, unsigned target)
{
    if (ld_acquire(p) >= target) {
        return true;
    }
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (ld_acquire(p) >= target) {
                return true;
            }
            __nanosleep(64);
        }
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            return false;
        }
    }
}

// 32 accumulators of one row -> 32 bytes: +offsetC, s32 -> f32, * factor, round, +128, clamp (see
// chunk_to_u8 in gemm_i8_tcgen05.cu; same arithmetic, same bits)
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
__device__ __forceinline__ void stage_u8(uint8_t *stg, uint32_t lane, uint32_t which, const uint32_t (&w)[8])
{
    const uint32_t sw = (lane >> 1) & 3;
    uint8_t *row = stg + lane * 64;
    *reinterpret_cast<uint4 *>(row + (((which * 2) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4 *>(row + (((which * 2 + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}
// direct stores of one 32-column chunk of one row (whole, 16-byte aligned chunks only)
__device__ __forceinline__ void store_chunk_direct(uint32_t kind, void *C, uint32_t N, const int32_t *offs, const float *colf,
    uint32_t m, uint32_t n0, uint32_t cl, const uint32_t (&r)[32])
{
    const size_t row_off = (size_t)m * N + n0;
    if (kind == 2) {
        uint32_t w[8];
        chunk_to_u8(offs, colf, cl, r, w);
        uint8_t *out = reinterpret_cast<uint8_t *>(C) + row_off;
        *reinterpret_cast<uint4 *>(out) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4 *>(out + 16) = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
        float *out = reinterpret_cast<float *>(C) + row_off;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int4 o = *reinterpret_cast<const int4 *>(offs + cl + j);
            const float4 c4 = *reinterpret_cast<const float4 *>(colf + cl + j);
            *reinterpret_cast<float4 *>(out + j) = make_float4(acc_to_f32((int)r[j] + o.x, c4.x),
                acc_to_f32((int)r[j + 1] + o.y, c4.y), acc_to_f32((int)r[j + 2] + o.z, c4.z),
                acc_to_f32((int)r[j + 3] + o.w, c4.w));
        }
    }
}

// position of tile g in the common order: layer (advanced monotonically), row block, column block
struct TilePos {
    uint32_t l, m_idx, n_idx;
};
__device__ __forceinline__ void locate(const SmemCtl *ctl, uint32_t n_layers, uint32_t g, uint32_t &l, TilePos &t)
{
    while (l + 1 < n_layers && g >= ctl->layers[l + 1].tile_begin) {
        ++l;
    }
    const uint32_t local = g - ctl->layers[l].tile_begin;
    const uint32_t tn = ctl->layers[l].tiles_n;
    t.l = l;
    t.m_idx = local / tn;
    t.n_idx = local - t.m_idx * tn;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
stack_u8s8_tcgen05_kernel(const StackParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * SMEM_A_STAGE;
    uint8_t *smem_staging = smem + SMEM_RING;
    SmemCtl *ctl = reinterpret_cast<SmemCtl *>(smem + SMEM_RING + SMEM_STAGING);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    for (uint32_t i = threadIdx.x; i < p.n_layers * (sizeof(LayerDev) / 4); i += blockDim.x) {
        reinterpret_cast<uint32_t *>(ctl->layers)[i] = reinterpret_cast<const uint32_t *>(p.layers)[i];
    }
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
    volatile uint32_t *abort_flag = &ctl->abort_flag;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, l = 0;
            bool ok = true;
            for (uint32_t g = blockIdx.x; ok && g < p.total_tiles; g += gridDim.x) {
                if (*abort_flag != 0) {
                    break;
                }
                TilePos t;
                locate(ctl, p.n_layers, g, l, t);
                const LayerDev &L = ctl->layers[t.l];
                const CUtensorMap *map_a = p.maps + 3 * t.l;
                const CUtensorMap *map_b = map_a + 1;
                const int m0 = (int)(t.m_idx * BLOCK_M);
                const int n0 = (int)(t.n_idx * L.block_n);
                if (t.l > 0) {
                    // A rows of this block are the previous layer's output: wait until all of its
                    // column tiles have been stored, then order the TMA reads behind that observation
                    if (!wait_counter(p.done + (size_t)(t.l - 1) * p.tiles_m + t.m_idx, ctl->layers[t.l - 1].dep_target)) {
                        ok = false;
                        break;
                    }
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                const uint32_t stage_bytes = (uint32_t)(BLOCK_M + L.block_n) * BLOCK_K;
                for (uint32_t kb = 0; kb < L.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&ctl->full[stage], stage_bytes);
                    tma_load_2d(map_a, &ctl->full[stage], smem_a + stage * SMEM_A_STAGE, (int)(kb * BLOCK_K), m0);
                    tma_load_2d(map_b, &ctl->full[stage], smem_b + stage * SMEM_B_STAGE, (int)(kb * BLOCK_K), n0);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                atomicExch(p.status, 21);
                atomicExch(&ctl->abort_flag, 1u);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, it = 0, l = 0;
            bool ok = true;
            for (uint32_t g = blockIdx.x; ok && g < p.total_tiles; g += gridDim.x, ++it) {
                if (*abort_flag != 0) {
                    break;
                }
                TilePos t;
                locate(ctl, p.n_layers, g, l, t);
                const LayerDev &L = ctl->layers[t.l];
                const uint32_t idesc = make_idesc_i8(L.block_n);
                const uint32_t acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * MAX_BLOCK_N;
                for (uint32_t kb = 0; kb < L.num_kb; ++kb) {
                    if (!mbar_wait(&ctl->full[stage], phase)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint64_t da = make_desc_sw128(smem_u32(smem_a + stage * SMEM_A_STAGE));
                    const uint64_t db = make_desc_sw128(smem_u32(smem_b + stage * SMEM_B_STAGE));
#pragma unroll
                    for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        umma_i8(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
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
                atomicExch(p.status, 22);
                atomicExch(&ctl->abort_flag, 1u);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------- epilogue warps 2..9 ------------------------------------
        const uint32_t quad = warp & 3;
        const uint32_t half = (warp - 2) >> 2;
        uint8_t *stg = smem_staging + (warp - 2) * STAGING_PER_WARP;
        int32_t *offs = ctl->offs[warp - 2];
        float *colf = ctl->colf[warp - 2];
        // this warp's chunk range inside a tile of layer L
        auto chunk_range = [&](const LayerDev &L, uint32_t &c_begin, uint32_t &c_end) {
            const uint32_t nch = L.block_n >> 5;
            c_begin = half ? ((nch + 1) >> 1) : 0u;
            c_end = half ? nch : ((nch + 1) >> 1);
        };
        // column constants of the warp's own columns: lane l owns columns l, l+32, l+64, l+96
        auto fetch = [&](const TilePos &t, int32_t (&o)[4], float (&f)[4]) {
            const LayerDev &L = ctl->layers[t.l];
            uint32_t cb, ce;
            chunk_range(L, cb, ce);
            const uint32_t cols = (ce - cb) * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                o[q] = 0;
                f[q] = 0.f;
                const uint32_t j = lane + 32 * q;
                const uint32_t n = t.n_idx * L.block_n + cb * 32 + j;
                if (j < cols && n < L.N) {
                    asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(o[q]) : "l"(L.offs + n));
                    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(f[q]) : "l"(L.colf + n));
                }
            }
        };
        auto park = [&](const int32_t (&o)[4], const float (&f)[4]) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                offs[lane + 32 * q] = o[q];
                colf[lane + 32 * q] = f[q];
            }
            __syncwarp();
        };
        // Completion of a tile is published one tile late: by then its bulk stores have had a whole
        // tile's time to finish, so the wait for them costs nothing.
        unsigned *pending = nullptr;
        auto publish = [&]() {
            if (pending != nullptr) {
                if (lane == 0) {
                    tma_store_wait_all();
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // bulk (async-proxy) stores before the release
                    red_release_add(pending, 1u);
                }
                pending = nullptr;
            }
        };
        uint32_t it = 0, l = 0, l_next = 0;
        if (blockIdx.x < p.total_tiles) {
            TilePos t0;
            locate(ctl, p.n_layers, blockIdx.x, l_next, t0);
            int32_t o[4];
            float f[4];
            fetch(t0, o, f);
            park(o, f);
        }
        for (uint32_t g = blockIdx.x; g < p.total_tiles; g += gridDim.x, ++it) {
            if (*abort_flag != 0) {
                break;
            }
            TilePos t;
            locate(ctl, p.n_layers, g, l, t);
            const LayerDev &L = ctl->layers[t.l];
            const CUtensorMap *map_c = p.maps + 3 * t.l + 2;
            uint32_t c_begin, c_end;
            chunk_range(L, c_begin, c_end);
            const uint32_t acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const uint32_t m0 = t.m_idx * BLOCK_M;
            const uint32_t n0 = t.n_idx * L.block_n;
            const uint32_t g_next = g + gridDim.x;
            TilePos tn;
            int32_t o_next[4];
            float f_next[4];
            if (g_next < p.total_tiles) {
                locate(ctl, p.n_layers, g_next, l_next, tn);
                fetch(tn, o_next, f_next);
            }
            bool ok = mbar_wait(&ctl->tmem_full[acc], acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) {
                    atomicExch(p.status, 23);
                    atomicExch(&ctl->abort_flag, 1u);
                }
                break;
            }
            tcgen05_fence_after();
            publish();  // the previous tile of this warp
            const uint32_t m = m0 + quad * 32 + lane;
            const uint32_t tbase = tmem_base + ((quad * 32u) << 16) + acc * MAX_BLOCK_N;
            const bool row_ok = m < p.M;
            const bool via_tma = L.out_kind == 2;
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
                    mbar_arrive(&ctl->tmem_empty[acc]);
                    released = true;
                }
                if (via_tma && has1) {
                    if (lane == 0) {
                        tma_store_wait_read();
                    }
                    __syncwarp();
                    uint32_t w[8];
                    chunk_to_u8(offs, colf, (c - c_begin) * 32, ra, w);
                    stage_u8(stg, lane, 0, w);
                } else if (row_ok && n0 + c * 32 < L.N) {
                    store_chunk_direct(L.out_kind, L.C, L.N, offs, colf, m, n0 + c * 32, (c - c_begin) * 32, ra);
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
                    if (via_tma) {
                        uint32_t w[8];
                        chunk_to_u8(offs, colf, (c + 1 - c_begin) * 32, rb, w);
                        stage_u8(stg, lane, 1, w);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && n0 + c * 32 < L.N) {
                            tma_store_2d(map_c, stg, (int)(n0 + c * 32), (int)(m0 + quad * 32));
                        }
                    } else if (row_ok && n0 + (c + 1) * 32 < L.N) {
                        store_chunk_direct(L.out_kind, L.C, L.N, offs, colf, m, n0 + (c + 1) * 32, (c + 1 - c_begin) * 32, rb);
                    }
                }
            }
            if (!released) {
                tcgen05_fence_before();
                mbar_arrive(&ctl->tmem_empty[acc]);
            }
            if (t.l + 1 < p.n_layers) {
                pending = p.done + (size_t)t.l * p.tiles_m + t.m_idx;
                // Late publication is only safe while this CTA stays inside the layer: its next tile
                // then depends on earlier layers only.  At a layer boundary the next tile may need
                // this very row block, so publish before waiting for anything else.
                if (!(g_next < p.total_tiles && tn.l == t.l)) {
                    publish();
                }
            }
            if (g_next < p.total_tiles) {
                __syncwarp();
                park(o_next, f_next);
            }
        }
        publish();
        if (lane == 0) {
            tma_store_wait_all();
        }
        __syncwarp();
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

// factor[n] = num / (sA * sB[n]): fp32 multiply, fp32 divide -- the order in which Bolt forms the
// factor of a layer (fully_connected.cpp:396,409; mmm_avx512_vnni.cpp:1805)
__global__ void col_factor_kernel(float num, float sA, const float *d_sA, float sB, const float *col_scale, uint32_t N,
    float *out)
{
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n < N) {
        const float sa = d_sA ? *d_sA : sA;
        const float sb = col_scale ? col_scale[n] : sB;
        out[n] = __fdiv_rn(num, __fmul_rn(sa, sb));
    }
}

struct StackPlan {
    StackParams p;
    CUtensorMap *d_maps = nullptr;
    LayerDev *d_layers = nullptr;
    unsigned *d_done = nullptr;
    size_t done_bytes = 0;
    int device = 0;
};

// Tile width of a layer: the widest tile whose last column tile is not mostly padding.  Narrower
// tiles were measured slower on B200 (each tile pays fixed hand-off latencies between the producer,
// the MMA issuer and the epilogue): 12 x (768 -> 3072 -> 768) at M = 4096 took 310 us with 256-wide
// tiles and 366 us with 192 / 128-wide ones.
uint32_t pick_stack_block_n(uint32_t N, uint32_t num_kb, int sms)
{
    (void)num_kb;
    (void)sms;
    uint32_t best = 32;
    double best_cost = 1e30;
    for (uint32_t bn = 256; bn >= 32; bn -= 32) {
        const uint32_t tiles = (N + bn - 1) / bn;
        const double cost = (double)tiles * (bn + 40.0);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

EE bolt_b200_col_factor(F32 num, F32 sA, const F32 *d_sA, F32 sB, const F32 *col_scale, U32 N, F32 *factor)
{
    if (ctx() == nullptr) {
        return UNKNOWN;
    }
    if (factor == nullptr) {
        return NULL_POINTER;
    }
    if (N == 0) {
        return SUCCESS;
    }
    col_factor_kernel<<<(N + 255) / 256, 256, 0, tls().stream>>>(num, sA, d_sA, sB, col_scale, N, factor);
    count_launch();
    B200_CUDA(cudaGetLastError());
    return SUCCESS;
}

EE bolt_b200_linear_stack_plan(U32 M, const void *A0, const bolt_b200_stack_layer *layers, U32 n_layers, void **plan_out)
{
    if (layers == nullptr || plan_out == nullptr || A0 == nullptr) {
        return NULL_POINTER;
    }
    *plan_out = nullptr;
    if (M == 0 || n_layers == 0 || n_layers > (U32)MAX_LAYERS) {
        return NOT_SUPPORTED;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    if (!tensor_map_encoder_available()) {
        return NOT_SUPPORTED;
    }
    std::vector<LayerDev> L(n_layers);
    std::vector<CUtensorMap> maps(3 * (size_t)n_layers);
    const uint32_t tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
    uint32_t tile_begin = 0;
    const void *A = A0;
    for (U32 l = 0; l < n_layers; ++l) {
        const bolt_b200_stack_layer &in = layers[l];
        const bool last = (l + 1 == n_layers);
        if (in.packedB == nullptr || in.C == nullptr || in.col_factor == nullptr) {
            return NULL_POINTER;
        }
        if ((in.N % 32) != 0 || (in.K % 16) != 0 || in.N == 0 || in.K == 0) {
            return NOT_SUPPORTED;
        }
        if (in.out_dt != DT_U8_Q && !(last && in.out_dt == DT_F32)) {
            return NOT_SUPPORTED;  // inner layers feed the next layer's u8 operand
        }
        if (l > 0 && in.K != layers[l - 1].N) {
            return NOT_MATCH;
        }
        if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(in.packedB) | reinterpret_cast<uintptr_t>(in.C)) & 15) {
            return NOT_SUPPORTED;
        }
        LayerDev &d = L[l];
        d.N = in.N;
        d.K = in.K;
        d.num_kb = (in.K + BLOCK_K - 1) / BLOCK_K;
        d.block_n = pick_stack_block_n(in.N, d.num_kb, c->sm_count);
        d.tiles_n = (in.N + d.block_n - 1) / d.block_n;
        d.out_kind = in.out_dt == DT_F32 ? 1u : 2u;
        d.tile_begin = tile_begin;
        d.dep_target = d.tiles_n * EPI_WARPS;
        d.offs = in.offsetC;
        d.colf = in.col_factor;
        d.C = in.C;
        tile_begin += tiles_m * d.tiles_n;
        const uint32_t Kp = B200_ALIGN(in.K, 8);
        const uint32_t es[2] = {1, 1};
        {
            const uint64_t dims[2] = {in.K, M};
            const uint64_t st[1] = {in.K};
            const uint32_t box[2] = {(uint32_t)BLOCK_K, (uint32_t)BLOCK_M};
            if (!encode_tiled_u8(&maps[3 * l], 2, A, dims, st, box, es, 128)) {
                return NOT_SUPPORTED;
            }
        }
        {
            const uint64_t dims[2] = {in.K, B200_ALIGN(in.N, 16)};
            const uint64_t st[1] = {Kp};
            const uint32_t box[2] = {(uint32_t)BLOCK_K, d.block_n};
            if (!encode_tiled_u8(&maps[3 * l + 1], 2, in.packedB, dims, st, box, es, 128)) {
                return NOT_SUPPORTED;
            }
        }
        if (d.out_kind == 2) {
            const uint64_t dims[2] = {in.N, M};
            const uint64_t st[1] = {in.N};
            const uint32_t box[2] = {64, 32};
            if (!encode_tiled_u8(&maps[3 * l + 2], 2, in.C, dims, st, box, es, 64)) {
                return NOT_SUPPORTED;
            }
        } else {
            maps[3 * l + 2] = maps[3 * l];
        }
        A = in.C;
    }
    StackPlan *pl = new StackPlan();
    pl->device = c->device;
    pl->done_bytes = (size_t)n_layers * tiles_m * sizeof(unsigned);
    if (cudaMalloc(&pl->d_maps, maps.size() * sizeof(CUtensorMap)) != cudaSuccess ||
        cudaMalloc(&pl->d_layers, L.size() * sizeof(LayerDev)) != cudaSuccess ||
        cudaMalloc(&pl->d_done, pl->done_bytes) != cudaSuccess ||
        cudaMemcpy(pl->d_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(pl->d_layers, L.data(), L.size() * sizeof(LayerDev), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(pl->d_maps);
        cudaFree(pl->d_layers);
        cudaFree(pl->d_done);
        delete pl;
        return ALLOC_FAILED;
    }
    pl->p.M = M;
    pl->p.tiles_m = tiles_m;
    pl->p.total_tiles = tile_begin;
    pl->p.n_layers = n_layers;
    pl->p.maps = pl->d_maps;
    pl->p.layers = pl->d_layers;
    pl->p.done = pl->d_done;
    pl->p.status = c->d_status;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(stack_u8s8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) {
        bolt_b200_linear_stack_free(pl);
        return cuda_ee(attr_err);
    }
    *plan_out = pl;
    return SUCCESS;
}

EE bolt_b200_linear_stack_run(void *plan)
{
    StackPlan *pl = reinterpret_cast<StackPlan *>(plan);
    if (pl == nullptr) {
        return NULL_POINTER;
    }
    DeviceCtx *c = ctx();
    if (c == nullptr) {
        return UNKNOWN;
    }
    cudaStream_t st = tls().stream;
    B200_CUDA(cudaMemsetAsync(pl->d_done, 0, pl->done_bytes, st));
    const uint32_t grid = pl->p.total_tiles < (uint32_t)c->sm_count ? pl->p.total_tiles : (uint32_t)c->sm_count;
    void *args[1] = {&pl->p};
    // cooperative: all CTAs must be resident, they wait on one another's progress counters
    B200_CUDA(cudaLaunchCooperativeKernel((const void *)stack_u8s8_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS), args,
        SMEM_BYTES, st));
    count_launch();
    return SUCCESS;
}

EE bolt_b200_linear_stack_free(void *plan)
{
    StackPlan *pl = reinterpret_cast<StackPlan *>(plan);
    if (pl != nullptr) {
        cudaFree(pl->d_maps);
        cudaFree(pl->d_layers);
        cudaFree(pl->d_done);
        delete pl;
    }
    return SUCCESS;
}

}  // extern "C"
