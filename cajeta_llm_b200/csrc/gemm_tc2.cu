// Matrix products on pairs of SMs (tcgen05 cta_group::2) for steps with many rows:
//
//     out[token, feature] (+)= sum_k X[token, k] * W[feature, k]   (+ bias[feature])
//
// Why pairs: a product tile is fed from shared memory, and shared memory is filled from L2
// at a rate that, not the tensor cores, bounds a one-SM tile of 128 x 256 (48 KB a K block
// of 64).  Two SMs working on one 256 x 256 tile each load their own 128 weight rows and only
// HALF of the token rows (32 KB a K block each); the tensor cores of both read both halves.
//
// A cluster of two blocks takes tiles cluster, cluster + clusters, ...; weights are on the
// product's 256 rows (block r holds rows 128 r .. 128 r + 127), tokens on its N (up to 256,
// block r holds the r-th half).  In each block: warp 0 loads with TMA into a ring of stages
// (the peer's loads count on the issuing block's barrier), warp 1 of block 0 issues the
// products for both, warps 2..5 of each block read that block's half of the accumulator
// (its 128 features) from its tensor memory and run the epilogue, while the next tile fills
// the second accumulator.  Epilogues: float32 store (+ bias), float32 accumulate, bf16
// store.
//
// SwiGLU (silu(x Wg^T) * (x Wu^T) to bf16) has a kernel of its own with the TOKENS on the
// product's 256 rows (block r holds tokens 128 r .. 128 r + 127 of the tile) and 128
// features of the gate matrix (loaded by block 0) beside the same 128 features of the up
// matrix (loaded by block 1) on its N = 256: every block's accumulator then holds, for its
// 128 tokens, gate in columns 0..127 and up in columns 128..255 - ONE accumulator of 256
// columns, so two fit tensor memory - and a thread (a token) finds both values of a feature
// in its own lane and stores 16 consecutive features at a time.
// Grouped form as in the one-SM kernel: token rows sorted by group, a prefix table of token
// tiles, rows past a group's end masked at the store.
//
// No load uses cluster multicast.  Every wait on a barrier is bounded (tc_common.cuh); the
// two blocks meet at a cluster barrier before tensor memory is freed.
//
// reference counterpart: the same per-expert and dense projection GEMMs as the one-SM kernel
// (io/WmmaKernel.cajeta, model/Linear.cajeta).
#include "common.cuh"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 224;          // warps 0 and 6: loads; warp 1: products; warps 2-5: epilogue
constexpr int LOADERS = 2;          // one thread keeps only so many bulk loads under way: the ring's stages are dealt to two
constexpr int FEAT_TILE = 256;      // feature rows a pair of blocks covers
constexpr int MAX_GROUPS = 1024;
constexpr int MAX_ACC_STAGES = 2;

enum Epilogue { EPI_STORE_F32 = 0, EPI_ACC_F32 = 1, EPI_SWIGLU_BF16 = 2, EPI_STORE_BF16 = 3 };

struct Args {
    int tokens, features, K;
    void* out;
    long long ldo;
    const float* bias;
    const int* group_offsets;
    int groups;
};

template <int N_TOK, int STAGES>
struct Smem {
    static constexpr int W_BYTES = 128 * BK * 2;                 // this block's 128 weight rows
    static constexpr int X_BYTES = (N_TOK / 2) * BK * 2;         // this block's half of the token rows
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = TILE_BYTES + 1024 + 256;
};

struct TileCoord {
    int tok0, tok_end, feat0, w_row0;
};

// tiles ordered (group, feature pair, token tile), the token tile fastest: clusters working
// side by side share a weight tile, so a slab is streamed from memory once
template <int N_TOK, int FEAT = FEAT_TILE>
__device__ __forceinline__ TileCoord decode_tile(const Args& p, int tile, int feat_tiles, int tok_tiles, const int* tiles_before) {
    TileCoord c;
    int group = 0, f, tt;
    if (p.group_offsets) {
        int lo = 0, hi = p.groups;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (tiles_before[mid] * feat_tiles <= tile) lo = mid; else hi = mid;
        }
        group = lo;
        int n_tt = tiles_before[group + 1] - tiles_before[group];
        int local = tile - tiles_before[group] * feat_tiles;
        f = local / n_tt;
        tt = local - f * n_tt;
        int g_lo = p.group_offsets[group], g_hi = p.group_offsets[group + 1];
        c.tok0 = g_lo + tt * N_TOK;
        c.tok_end = min(g_hi, c.tok0 + N_TOK);
    } else {
        tt = tile % tok_tiles;
        f = tile / tok_tiles;
        c.tok0 = tt * N_TOK;
        c.tok_end = min(p.tokens, c.tok0 + N_TOK);
    }
    c.feat0 = f * FEAT;
    c.w_row0 = group * p.features + c.feat0;
    return c;
}

// the product's N for a tile: its tokens rounded up to 32 (each block supplies half, in 16s)
__device__ __forceinline__ int tile_n(const TileCoord& c, int n_tok) { return min(n_tok, ((c.tok_end - c.tok0 + 31) >> 5) << 5); }

template <int N_TOK, int EPI, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_w2, Args p, int feat_tiles, int tok_tiles, int total_tiles) {
    using S = Smem<N_TOK, STAGES>;
    constexpr uint32_t STAGE_COLS = N_TOK;
    constexpr int ACC_STAGES = MAX_ACC_STAGES;
    constexpr uint32_t TMEM_COLS = 512;
    static_assert(STAGE_COLS * ACC_STAGES <= 512, "accumulators do not fit tensor memory");
    static_assert(EPI != EPI_SWIGLU_BF16, "SwiGLU has its own kernel");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + S::TILE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;
    uint64_t* acc_empty = acc_full + MAX_ACC_STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + MAX_ACC_STAGES);
    __shared__ int tiles_before[MAX_GROUPS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);           // used in block 0: its own arrive.expect_tx for the bytes of both blocks
            mbar_init(&empty_bar[s], 1);          // in both: the issuing block's commit
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(&acc_full[s], 1);           // in both: the issuing block's commit
            mbar_init(&acc_empty[s], 8);          // used in block 0: one arrival per epilogue warp of both blocks
        }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    cj::after_predecessor();          // from here on the kernel reads what earlier kernels wrote
    if (p.group_offsets && warp == 2) {
        int carry = 0;
        for (int g0 = 0; g0 < p.groups; g0 += 32) {
            int g = g0 + lane;
            int n = g < p.groups ? (p.group_offsets[g + 1] - p.group_offsets[g] + N_TOK - 1) / N_TOK : 0;
            int inc = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            if (g < p.groups) tiles_before[g] = carry + inc - n;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) tiles_before[p.groups] = carry;
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                           // both blocks' barriers are initialised before either is signalled
    cj::release_successor();                      // tensor memory is held: a following kernel may be scheduled beside
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.group_offsets) total_tiles = tiles_before[p.groups] * feat_tiles;

    if (warp == 0 || warp == 6) {
        // ---- TMA producers (in both blocks): one warp the even iterations, one the odd -------
        static_assert(LOADERS < STAGES, "a loader must stay within one round of the ring");
        const int mine = warp == 0 ? 0 : 1;
        if (elect_one()) {
            tma_prefetch_descriptor(&map_x);
            tma_prefetch_descriptor(&map_w);
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster; tile < total_tiles && ok; tile += clusters) {
                TileCoord c = decode_tile<N_TOK>(p, tile, feat_tiles, tok_tiles, tiles_before);
                const int half = tile_n(c, N_TOK) >> 1;
                const int k_blocks = (p.K + BK - 1) / BK;
                const int w_row = c.w_row0 + rank * 128;
                for (int i = 0; i < k_blocks; ++i, ++it) {
                    if ((int)(it % LOADERS) != mine) continue;
                    int s = it % STAGES;
                    ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    uint8_t* st = tiles + (size_t)s * S::STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
                    const uint32_t bar = cluster_map(&full_bar[s], 0);
                    int k0 = i * BK;
                    tma_load_2d_pair(st, &map_w, bar, k0, w_row);
                    tma_load_2d_pair(st + S::W_BYTES, &map_x, bar, k0, c.tok0 + rank * half);
                }
            }
        }
    } else if (warp == 1) {
        // ---- product issue: block 0 for the pair ---------------------------------------------
        if (rank == 0 && elect_one()) {
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int tile = cluster; tile < total_tiles && ok; tile += clusters) {
                TileCoord c = decode_tile<N_TOK>(p, tile, feat_tiles, tok_tiles, tiles_before);
                const int as = acc_it % ACC_STAGES;
                ok = mbar_wait(&acc_empty[as], ((acc_it / ACC_STAGES) & 1) ^ 1, 4);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t acc_addr = tmem_base + as * STAGE_COLS;
                const uint32_t idesc = umma_idesc_bf16(256, tile_n(c, N_TOK));
                const int k_blocks = (p.K + BK - 1) / BK;
                for (int i = 0; i < k_blocks; ++i, ++it) {
                    int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, 2);
                    if (!ok) break;
                    tcgen05_fence_after();
                    uint8_t* st = tiles + (size_t)s * S::STAGE_BYTES;
                    uint64_t dw = umma_desc_sw128(st);
                    uint64_t dx = umma_desc_sw128(st + S::W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                        umma_bf16_pair(acc_addr, dw + step, dx + step, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty_bar[s]);
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[as]);
                ++acc_it;
            }
        }
    } else if (warp < 6) {
        // ---- epilogue: warps 2..5 of both blocks, each its quarter of the block's 128 lanes -----
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        uint32_t acc_it = 0;
        bool ok = true;
        for (int tile = cluster; tile < total_tiles && ok; tile += clusters) {
            TileCoord c = decode_tile<N_TOK>(p, tile, feat_tiles, tok_tiles, tiles_before);
            const int as = acc_it % ACC_STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[as], (acc_it / ACC_STAGES) & 1, 3));
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t lane_base = tmem_base + as * STAGE_COLS + ((uint32_t)(quarter * 32) << 16);
            const int n_cols = c.tok_end - c.tok0;
            {
                const int feat = c.feat0 + (int)rank * 128 + r;
                const bool live = feat < p.features;
                const float b = (p.bias != nullptr && live) ? p.bias[feat] : 0.0f;
#pragma unroll 1
                for (int c0 = 0; c0 < N_TOK; c0 += 32) {
                    if (c0 >= n_cols) break;
                    uint32_t v[32];
                    tmem_ld16(lane_base + c0, *(uint32_t(*)[16])&v[0]);
                    tmem_ld16(lane_base + c0 + 16, *(uint32_t(*)[16])&v[16]);
                    tmem_ld_wait();
                    if (!live) continue;
                    // column j is token tok0 + c0 + j: a warp writes 32 consecutive features of a token
                    const long long o0 = (long long)(c.tok0 + c0) * p.ldo + feat;
                    if (EPI == EPI_ACC_F32) {
                        float old[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) old[j] = c0 + j < n_cols ? ((const float*)p.out)[o0 + j * p.ldo] : 0.0f;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c0 + j < n_cols) ((float*)p.out)[o0 + j * p.ldo] = old[j] + __uint_as_float(v[j]) + b;
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (c0 + j >= n_cols) break;
                            float val = __uint_as_float(v[j]) + b;
                            if (EPI == EPI_STORE_F32) ((float*)p.out)[o0 + j * p.ldo] = val;
                            else ((__nv_bfloat16*)p.out)[o0 + j * p.ldo] = __float2bfloat16_rn(val);
                        }
                    }
                }
            }
            // this warp has read its quarter: hand the stage back to the issuing block
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_map(&acc_empty[as], 0));
            ++acc_it;
        }
    }
    // nobody leaves while the peer may still read this block's shared memory or signal its barriers
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---- SwiGLU on pairs: tokens on the rows, gate | up features on N ---------------------------------
constexpr int SW_TOK = 256;          // tokens a pair's tile covers (128 a block)
constexpr int SW_FEAT = 128;         // features a tile covers (gate and up of each)

template <int STAGES>
struct SwigluSmem {
    static constexpr int X_BYTES = 128 * BK * 2;                 // this block's 128 token rows
    static constexpr int W_BYTES = SW_FEAT * BK * 2;             // block 0: gate rows, block 1: up rows
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = TILE_BYTES + 1024 + 256;
};

template <int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
swiglu_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                   const __grid_constant__ CUtensorMap map_wu, Args p, int feat_tiles, int tok_tiles, int total_tiles) {
    using S = SwigluSmem<STAGES>;
    constexpr uint32_t STAGE_COLS = 2 * SW_FEAT;       // gate | up
    constexpr int ACC_STAGES = 2;
    constexpr uint32_t TMEM_COLS = 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + S::TILE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;
    uint64_t* acc_empty = acc_full + ACC_STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + ACC_STAGES);
    __shared__ int tiles_before[MAX_GROUPS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 8);
        }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    cj::after_predecessor();          // from here on the kernel reads what earlier kernels wrote
    if (p.group_offsets && warp == 2) {
        int carry = 0;
        for (int g0 = 0; g0 < p.groups; g0 += 32) {
            int g = g0 + lane;
            int n = g < p.groups ? (p.group_offsets[g + 1] - p.group_offsets[g] + SW_TOK - 1) / SW_TOK : 0;
            int inc = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            if (g < p.groups) tiles_before[g] = carry + inc - n;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) tiles_before[p.groups] = carry;
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    cj::release_successor();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.group_offsets) total_tiles = tiles_before[p.groups] * feat_tiles;
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0 || warp == 6) {
        static_assert(LOADERS < STAGES, "a loader must stay within one round of the ring");
        const int mine = warp == 0 ? 0 : 1;
        if (elect_one()) {
            tma_prefetch_descriptor(&map_x);
            tma_prefetch_descriptor(rank == 0 ? &map_wg : &map_wu);
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster; tile < total_tiles && ok; tile += clusters) {
                TileCoord c = decode_tile<SW_TOK, SW_FEAT>(p, tile, feat_tiles, tok_tiles, tiles_before);
                for (int i = 0; i < k_blocks; ++i, ++it) {
                    if ((int)(it % LOADERS) != mine) continue;
                    int s = it % STAGES;
                    ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    uint8_t* st = tiles + (size_t)s * S::STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
                    const uint32_t bar = cluster_map(&full_bar[s], 0);
                    tma_load_2d_pair(st, &map_x, bar, i * BK, c.tok0 + (int)rank * 128);
                    tma_load_2d_pair(st + S::X_BYTES, rank == 0 ? &map_wg : &map_wu, bar, i * BK, c.w_row0);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            const uint32_t idesc = umma_idesc_bf16(256, 2 * SW_FEAT);
            for (int tile = cluster; tile < total_tiles && ok; tile += clusters) {
                const int as = acc_it % ACC_STAGES;
                ok = mbar_wait(&acc_empty[as], ((acc_it / ACC_STAGES) & 1) ^ 1, 4);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t acc_addr = tmem_base + as * STAGE_COLS;
                for (int i = 0; i < k_blocks; ++i, ++it) {
                    int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, 2);
                    if (!ok) break;
                    tcgen05_fence_after();
                    uint8_t* st = tiles + (size_t)s * S::STAGE_BYTES;
                    uint64_t dx = umma_desc_sw128(st);
                    uint64_t dw = umma_desc_sw128(st + S::X_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                        umma_bf16_pair(acc_addr, dx + step, dw + step, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty_bar[s]);
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[as]);
                ++acc_it;
            }
        }
    } else if (warp < 6) {
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        uint32_t acc_it = 0;
        bool ok = true;
        for (int tile = cluster; tile < total_tiles && ok; tile += clusters) {
            TileCoord c = decode_tile<SW_TOK, SW_FEAT>(p, tile, feat_tiles, tok_tiles, tiles_before);
            const int as = acc_it % ACC_STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[as], (acc_it / ACC_STAGES) & 1, 3));
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t lane_base = tmem_base + as * STAGE_COLS + ((uint32_t)(quarter * 32) << 16);
            const int token = c.tok0 + (int)rank * 128 + r;
            const bool live = token < c.tok_end;
            // a warp none of whose tokens exist has nothing to read
            if (__any_sync(0xffffffffu, live)) {
                __nv_bfloat16* dst_row = (__nv_bfloat16*)p.out + (long long)token * p.ldo + c.feat0;
#pragma unroll 1
                for (int c0 = 0; c0 < SW_FEAT; c0 += 16) {
                    if (c.feat0 + c0 >= p.features) break;
                    uint32_t g[16], u[16];
                    tmem_ld16(lane_base + c0, g);
                    tmem_ld16(lane_base + SW_FEAT + c0, u);
                    tmem_ld_wait();
                    if (!live) continue;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float gv = __uint_as_float(g[j]);
                        v[j] = gv * __frcp_rn(1.0f + __expf(-gv)) * __uint_as_float(u[j]);
                    }
                    __nv_bfloat16* dst = dst_row + c0;
                    if (c.feat0 + c0 + 16 <= p.features && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            uint4 w4;
                            __nv_bfloat162* b2 = (__nv_bfloat162*)&w4;
#pragma unroll
                            for (int q = 0; q < 4; ++q) b2[q] = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                            *(uint4*)(dst + j) = w4;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c.feat0 + c0 + j < p.features) dst[j] = __float2bfloat16_rn(v[j]);
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_map(&acc_empty[as], 0));
            ++acc_it;
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

inline int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <typename Kern>
int launch_pairs(Kern kern, int smem, long long total, cudaStream_t stream, const CUtensorMap& mx, const CUtensorMap& mw,
                 const CUtensorMap& mw2, const Args& a, int feat_tiles, int tok_tiles) {
    if (total > 0x7fffffffLL) return CJ_ERR_SIZE;
    int clusters = sm_count() / 2;
    if (total < clusters) clusters = (int)total;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cj::overlap_launches() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mx, mw, mw2, a, feat_tiles, tok_tiles, (int)total);
    if (e != cudaSuccess) return (int)e;
    return cj::launch_status();
}

template <int N_TOK, int EPI>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const Args& a, cudaStream_t stream) {
    constexpr int stage = Smem<N_TOK, 1>::STAGE_BYTES;
    constexpr int STAGES = (200 * 1024 / stage) > 8 ? 8 : (200 * 1024 / stage);
    using S = Smem<N_TOK, STAGES>;
    auto kern = gemm_tc2_kernel<N_TOK, EPI, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int feat_tiles = (a.features + FEAT_TILE - 1) / FEAT_TILE;
    int tok_tiles = (a.tokens + N_TOK - 1) / N_TOK + (a.group_offsets ? a.groups : 0);
    return launch_pairs(kern, S::TOTAL, (long long)feat_tiles * tok_tiles, stream, mx, mw, mw, a, feat_tiles, tok_tiles);
}

int launch_swiglu(const CUtensorMap& mx, const CUtensorMap& mwg, const CUtensorMap& mwu, const Args& a, cudaStream_t stream) {
    constexpr int STAGES = 6;
    using S = SwigluSmem<STAGES>;
    auto kern = swiglu_pair_kernel<STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int feat_tiles = (a.features + SW_FEAT - 1) / SW_FEAT;
    int tok_tiles = (a.tokens + SW_TOK - 1) / SW_TOK + (a.group_offsets ? a.groups : 0);
    return launch_pairs(kern, S::TOTAL, (long long)feat_tiles * tok_tiles, stream, mx, mwg, mwu, a, feat_tiles, tok_tiles);
}

}  // namespace

// x: [tokens, K] bf16 with row stride ldx; w (and w2 for SwiGLU): [groups * features, K] bf16,
// contiguous.  n_tok: tokens a tile covers, 128 or 256 (SwiGLU: always 256).  epilogue: 0 float32
// store, 1 float32 accumulate, 2 SwiGLU to bf16 (needs w2), 3 bf16 store.
// Refuses (negative code) what it cannot run; never a wrong result.
CJ_EXPORT int cj_gemm_tc2(const void* x, long long ldx, const void* w, const void* w2, const float* bias, void* out,
                          long long ldo, int tokens, int features, int K, int epilogue, int n_tok,
                          const int* group_offsets, int groups, cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (!x || !w || !out || K <= 0) return CJ_ERR_ARG;
    if (K % 8 != 0 || ldx % 8 != 0) return CJ_ERR_ALIGN;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)w2) & 15) return CJ_ERR_ALIGN;
    if ((epilogue == EPI_SWIGLU_BF16) != (w2 != nullptr)) return CJ_ERR_ARG;
    if (epilogue == EPI_SWIGLU_BF16 && bias) return CJ_ERR_ARG;
    if (group_offsets && groups <= 0) return CJ_ERR_ARG;
    if (n_tok != 128 && n_tok != 256) return CJ_ERR_SIZE;
    if (group_offsets && groups > MAX_GROUPS) return CJ_ERR_SIZE;
    int total_w_rows = (group_offsets ? groups : 1) * features;
    CUtensorMap mx, mw, mw2;
    if (!make_map_bf16(&mw, w, total_w_rows, K, K, 128)) return CJ_ERR_ARG;
    Args a{tokens, features, K, out, ldo, bias, group_offsets, groups};
    if (epilogue == EPI_SWIGLU_BF16) {
        // tokens on the rows: a block's box is 128 token rows whatever n_tok says
        if (!make_map_bf16(&mx, x, tokens, K, ldx, 128)) return CJ_ERR_ARG;
        if (!make_map_bf16(&mw2, w2, total_w_rows, K, K, 128)) return CJ_ERR_ARG;
        return launch_swiglu(mx, mw, mw2, a, stream);
    }
    if (!make_map_bf16(&mx, x, tokens, K, ldx, n_tok / 2)) return CJ_ERR_ARG;
#define CASE(EPI)                                                   \
    if (n_tok == 256) return launch<256, EPI>(mx, mw, a, stream);   \
    else return launch<128, EPI>(mx, mw, a, stream);
    switch (epilogue) {
        case EPI_STORE_F32: CASE(EPI_STORE_F32)
        case EPI_ACC_F32: CASE(EPI_ACC_F32)
        case EPI_STORE_BF16: CASE(EPI_STORE_BF16)
    }
#undef CASE
    return CJ_ERR_ARG;
}

CJ_EXPORT int cj_gemm_tc2_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_error_flag, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
