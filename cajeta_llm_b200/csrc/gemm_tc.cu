// Matrix products on the 5th-generation tensor cores (tcgen05) for the bfloat16 path:
//
//     out[token, feature] (+)= sum_k X[token, k] * W[feature, k]   (+ bias[feature])
//
// X: activations [tokens, K] bf16, W: weights [features, K] bf16 (torch's [out, in]), both
// K-major, so both feed tcgen05.mma straight from the 128-byte-swizzled tiles that TMA
// lays into shared memory; accumulators are float32 in tensor memory.
//
// Persistent blocks, one per SM, each taking tiles blockIdx.x, blockIdx.x + gridDim.x, ...:
// warp 0 issues the TMA loads into a ring of stages and runs ahead across tile boundaries,
// so the weight stream never stops; warp 1 (one elected thread) issues the products and
// owns the tensor-memory allocation; warps 2..5 read an accumulator back (each warp its
// own 32-lane quarter) and run the epilogue while the products of the next tile fill the
// second accumulator.  Two orientations share the code:
//   * tokens on the 128 rows of the product (SWAP = false): a step with many rows
//     (prompt portions);
//   * weights on the 128 rows, tokens on the product's N (SWAP = true, TOK = 16..128): a
//     step with few rows (decode), so that a tile of 128 x 64 weights costs 16 KB of
//     shared-memory traffic and the tokens only 2 KB.
// Epilogues: float32 store (+ bias) [optionally one of several split-K partials], float32
// accumulate (the residual add of an output projection), SwiGLU of two products to bf16
// (two weight tiles, two accumulators), bf16 store.
// Grouped form (mixture of experts): token rows are sorted by expert, offsets[g] is the
// first row of group g, the weights of group g start at row g * features of W; a block
// finds the (group, tile) of a tile index in a prefix table built at its start and masks
// rows past the group's end.
//
// reference counterpart: the indirected per-expert GEMMs over (expert, row range) chunk
// maps, io/WmmaKernel.cajeta (q4kWmmaIdMwKernel), and the dense projection GEMMs of
// model/Linear.cajeta; both wmma-class there.
#include "common.cuh"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int BK = 64;             // K elements per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;         // K of one tcgen05.mma of kind::f16
constexpr int THREADS = 224;          // warps 0 and 6: loads; warp 1: products; warps 2-5: epilogue
constexpr int LOADERS = 2;

enum Epilogue { EPI_STORE_F32 = 0, EPI_ACC_F32 = 1, EPI_SWIGLU_BF16 = 2, EPI_STORE_BF16 = 3 };

struct Args {
    int tokens;                 // rows of X
    int features;               // rows of W per group
    int K;
    void* out;
    long long ldo;              // elements between output rows (tokens)
    const float* bias;          // [features] or null
    const int* group_offsets;   // [groups + 1] or null
    int groups;
    int k_splits;               // > 1: each split stores its partial at out + split * split_stride
    long long split_stride;
    int offsets_settled;        // the groups' offsets were complete before the kernel before this one began
    int choose_height;          // grouped, weights on the rows: the tile's height is chosen in the kernel (see LowTiles)
};

// Grouped products of a decode step: how many groups hold rows is known only on the device, and with it
// the number of tiles.  352 tiles of 128 weight rows on 148 SMs are two full rounds and a third in which
// 56 SMs stream alone; tiles of 112 or 96 rows can make the rounds come out even.  So such a launch
// carries tensor maps for boxes of 112 and 96 rows too, and every block - from the same sum of the
// groups' token tiles - picks the height whose last round wastes least.  A product still spans 128
// rows: the rows past the tile's height are whatever the stage held before, and nobody reads their sums.
constexpr int LOW_HEIGHTS = 2;
__host__ __device__ constexpr int low_height(int i) { return i == 0 ? 112 : 96; }
struct LowTiles {
    CUtensorMap w[LOW_HEIGHTS], w2[LOW_HEIGHTS];
};

template <int N_MMA, bool SWAP, bool DUAL, int STAGES>
struct Smem {
    static constexpr int X_ROWS = SWAP ? N_MMA : 128;
    static constexpr int W_ROWS = SWAP ? 128 : N_MMA;
    static constexpr int X_BYTES = X_ROWS * BK * 2;
    static constexpr int W_BYTES = W_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = X_BYTES + (DUAL ? 2 : 1) * W_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = TILE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

constexpr int MAX_ACC_STAGES = 2;   // accumulators in tensor memory: one is drained while the next is filled
constexpr int MAX_GROUPS = 1024;

// Work of one block, in the order it takes its tiles: tile = blockIdx.x + i * gridDim.x.
// A tile index splits into (feature tile, token tile, K split), the feature tile running
// fastest so that neighbouring blocks stream different weights.
struct TileCoord {
    int tok0, tok_end, feat0, w_row0, kb_begin, n_kb, split;
    bool valid;
};

template <int TOK_TILE>
__device__ __forceinline__ TileCoord decode_tile(const Args& p, int tile, int feat_tiles, int tok_tiles, const int* tiles_before,
                                                 const int FEAT_TILE) {
    TileCoord c;
    c.valid = true;
    int group = 0, f, tt;
    if (p.group_offsets) {
        // grouped: tiles are ordered (split, group, feature tile, token tile), the token tile
        // running fastest, so that the blocks working side by side share a weight tile and
        // a slab is streamed from memory once.  tiles_before[g] = token tiles of the groups
        // before g.
        int per_split = tiles_before[p.groups] * feat_tiles;
        c.split = tile / per_split;
        int local = tile - c.split * per_split;
        int lo = 0, hi = p.groups;                 // invariant: tiles_before[lo] * feat_tiles <= local
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (tiles_before[mid] * feat_tiles <= local) lo = mid; else hi = mid;
        }
        group = lo;
        int n_tt = tiles_before[group + 1] - tiles_before[group];
        local -= tiles_before[group] * feat_tiles;
        f = local / n_tt;
        tt = local - f * n_tt;
        int g_lo = __ldcg(p.group_offsets + group), g_hi = __ldcg(p.group_offsets + group + 1);
        c.tok0 = g_lo + tt * TOK_TILE;
        c.tok_end = min(g_hi, c.tok0 + TOK_TILE);
    } else {
        // dense: the feature tile runs fastest, so that neighbouring blocks stream different weights
        f = tile % feat_tiles;
        int rest = tile / feat_tiles;
        tt = rest % tok_tiles;
        c.split = rest / tok_tiles;
        c.tok0 = tt * TOK_TILE;
        c.tok_end = min(p.tokens, c.tok0 + TOK_TILE);
    }
    c.feat0 = f * FEAT_TILE;
    c.w_row0 = group * p.features + c.feat0;
    int k_blocks_total = (p.K + BK - 1) / BK;
    int per_split = (k_blocks_total + p.k_splits - 1) / p.k_splits;
    c.kb_begin = c.split * per_split;
    c.n_kb = max(0, min(k_blocks_total, c.kb_begin + per_split) - c.kb_begin);
    return c;
}

template <int N_MMA, bool SWAP, bool DUAL, int EPI, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ LowTiles low, Args p, int feat_tiles,
               int tok_tiles, int total_tiles) {
    using S = Smem<N_MMA, SWAP, DUAL, STAGES>;
    constexpr int TOK_TILE = S::X_ROWS;          // token rows a tile covers
    int feat_tile = S::W_ROWS;                   // weight rows a tile covers (a grouped decode launch may choose fewer)
    int height = -1;                             // which of the lower heights, or -1
    constexpr uint32_t ACC_COLS = N_MMA;         // tensor-memory columns of one accumulator
    constexpr uint32_t STAGE_COLS = ACC_COLS * (DUAL ? 2 : 1);
    // two accumulator stages when they fit the 512 columns of tensor memory, else one (the
    // products of the next tile then wait for the epilogue; the loads still run ahead)
    constexpr int ACC_STAGES = STAGE_COLS * MAX_ACC_STAGES <= 512 ? MAX_ACC_STAGES : 1;
    constexpr uint32_t TMEM_COLS_NEEDED = STAGE_COLS * ACC_STAGES;
    constexpr uint32_t TMEM_COLS = TMEM_COLS_NEEDED <= 32 ? 32 : TMEM_COLS_NEEDED <= 64 ? 64 : TMEM_COLS_NEEDED <= 128 ? 128
                                   : TMEM_COLS_NEEDED <= 256 ? 256 : 512;
    static_assert(TMEM_COLS_NEEDED <= 512, "accumulators do not fit tensor memory");

    // ---- shared memory -----------------------------------------------------------------
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + S::TILE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;
    uint64_t* acc_empty = acc_full + MAX_ACC_STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + MAX_ACC_STAGES);
    __shared__ int tiles_before[MAX_GROUPS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);          // one arrival per epilogue warp
        }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    // Everything above touched only this block's own shared and tensor memory.  What follows
    // reads the groups' offsets (grouped launches) and then, per role, weights and activations.
    // Weights are written by no kernel, so the first ring of weight tiles leaves before the wait
    // for the kernel before, while that kernel is still draining.  The offsets may be read that
    // early only if the caller says that they were complete before the kernel before this one
    // began (they are read past L1, which may hold an older step's values); else the block
    // waits first.
    const bool dense = p.group_offsets == nullptr;
    const bool early_ok = dense || p.offsets_settled != 0;
    if (!early_ok) cj::after_predecessor();
    if (p.group_offsets && warp == 2) {
        // token tiles before each group (a warp scan over the groups, 32 at a time)
        int carry = 0;
        for (int g0 = 0; g0 < p.groups; g0 += 32) {
            int g = g0 + lane;
            int n = g < p.groups ? (__ldcg(p.group_offsets + g + 1) - __ldcg(p.group_offsets + g) + TOK_TILE - 1) / TOK_TILE : 0;
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
    tcgen05_fence_after();
    // tensor memory is held: a following kernel's blocks may now be scheduled beside this one
    // (one that took tensor memory first and then waited for this kernel would starve it)
    cj::release_successor();
    const uint32_t tmem_base = *tmem_slot;
    // a grouped launch knows its number of tiles only now (it depends on the routing)
    if (p.group_offsets) {
        if (SWAP && p.choose_height) {
            // rounds of the persistent blocks times the bytes of a tile, for each height
            const long long tt = (long long)tiles_before[p.groups] * p.k_splits, blocks = gridDim.x;
            long long best = (tt * feat_tiles + blocks - 1) / blocks * S::W_ROWS;
            // (a launch of one round is as long as one tile's chain of products, whatever the tile's height)
#pragma unroll
            for (int i = 0; i < LOW_HEIGHTS && tt * feat_tiles > blocks; ++i) {
                const int h = low_height(i), ft = (p.features + h - 1) / h;
                const long long cost = (tt * ft + blocks - 1) / blocks * h;
                if (cost < best) { best = cost; height = i; feat_tile = h; feat_tiles = ft; }
            }
        }
        total_tiles = tiles_before[p.groups] * feat_tiles * p.k_splits;
    }
    const CUtensorMap* mw = height < 0 ? &map_w : &low.w[height];
    const CUtensorMap* mw2 = height < 0 ? &map_w2 : &low.w2[height];
    const uint32_t stage_tx = S::X_BYTES + (DUAL ? 2 : 1) * (uint32_t)feat_tile * BK * 2;      // bytes a stage's loads bring

    if (warp == 0 || warp == 6) {
        // ---- TMA producers: stream stage after stage, straight across tile boundaries ----------
        // Two warps, one taking the even iterations and one the odd: what ONE thread can have
        // under way in bulk loads is bounded (measured: a thread streams 36 GB/s of cold 16 KB
        // tiles however deep its ring, two threads twice that), and with every SM streaming, one
        // issuing thread an SM stops at 5.4 TB/s.  A loader is never a whole round of the ring
        // ahead of the products (LOADERS < STAGES), which is what a wait by phase parity needs.
        static_assert(LOADERS < STAGES, "a loader must stay within one round of the ring");
        const int mine = warp == 0 ? 0 : 1;
        if (elect_one()) {
            if (mine == 0) {
                tma_prefetch_descriptor(&map_x);
                tma_prefetch_descriptor(mw);
                if (DUAL) tma_prefetch_descriptor(mw2);
            }
            uint32_t early = 0;               // stages whose weight tiles left before the wait
            if (early_ok) {
                for (int tile = blockIdx.x; tile < total_tiles && early < STAGES; tile += gridDim.x) {
                    TileCoord c = decode_tile<TOK_TILE>(p, tile, feat_tiles, tok_tiles, tiles_before, feat_tile);
                    if (!c.valid) continue;
                    for (int i = 0; i < c.n_kb && early < STAGES; ++i, ++early) {
                        if ((int)(early % LOADERS) != mine) continue;
                        uint8_t* st = tiles + (size_t)early * S::STAGE_BYTES;
                        mbar_expect_tx(&full_bar[early], stage_tx);
                        int k0 = (c.kb_begin + i) * BK;
                        tma_load_2d(st + S::X_BYTES, mw, &full_bar[early], k0, c.w_row0);
                        if (DUAL) tma_load_2d(st + S::X_BYTES + S::W_BYTES, mw2, &full_bar[early], k0, c.w_row0);
                    }
                }
                cj::after_predecessor();
            }
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                TileCoord c = decode_tile<TOK_TILE>(p, tile, feat_tiles, tok_tiles, tiles_before, feat_tile);
                if (!c.valid) continue;
                for (int i = 0; i < c.n_kb; ++i, ++it) {
                    if ((int)(it % LOADERS) != mine) continue;
                    int s = it % STAGES;
                    uint8_t* st = tiles + (size_t)s * S::STAGE_BYTES;
                    int k0 = (c.kb_begin + i) * BK;
                    if (it < early) {
                        // the stage's weights are under way and its bytes announced: only the activations are missing
                        tma_load_2d(st, &map_x, &full_bar[s], k0, c.tok0);
                        continue;
                    }
                    ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    mbar_expect_tx(&full_bar[s], stage_tx);
                    tma_load_2d(st, &map_x, &full_bar[s], k0, c.tok0);
                    tma_load_2d(st + S::X_BYTES, mw, &full_bar[s], k0, c.w_row0);
                    if (DUAL) tma_load_2d(st + S::X_BYTES + S::W_BYTES, mw2, &full_bar[s], k0, c.w_row0);
                }
            }
        }
    } else if (warp == 1) {
        // ---- product issue -----------------------------------------------------------------
        if (early_ok) cj::after_predecessor();
        if (elect_one()) {
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                TileCoord c = decode_tile<TOK_TILE>(p, tile, feat_tiles, tok_tiles, tiles_before, feat_tile);
                if (!c.valid) continue;
                const int as = acc_it % ACC_STAGES;
                ok = mbar_wait(&acc_empty[as], ((acc_it / ACC_STAGES) & 1) ^ 1, 4);      // the epilogue has drained it
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t acc_addr = tmem_base + as * STAGE_COLS;
                // weights on the rows: the product is only as wide as the tile has tokens (in 16s)
                const int n_mma = SWAP ? min(N_MMA, ((c.tok_end - c.tok0 + 15) >> 4) << 4) : N_MMA;
                const uint32_t idesc = umma_idesc_bf16(128, n_mma);
                for (int i = 0; i < c.n_kb; ++i, ++it) {
                    int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, 2);
                    if (!ok) break;
                    tcgen05_fence_after();
                    uint8_t* st = tiles + (size_t)s * S::STAGE_BYTES;
                    uint64_t dx = umma_desc_sw128(st);
                    uint64_t dw = umma_desc_sw128(st + S::X_BYTES);
                    uint64_t dw2 = DUAL ? umma_desc_sw128(st + S::X_BYTES + S::W_BYTES) : 0;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);       // 32 bytes along K inside the swizzle row
                        uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                        if (SWAP) {
                            umma_bf16(acc_addr, dw + step, dx + step, idesc, acc);
                            if (DUAL) umma_bf16(acc_addr + ACC_COLS, dw2 + step, dx + step, idesc, acc);
                        } else {
                            umma_bf16(acc_addr, dx + step, dw + step, idesc, acc);
                            if (DUAL) umma_bf16(acc_addr + ACC_COLS, dx + step, dw2 + step, idesc, acc);
                        }
                    }
                    umma_commit(&empty_bar[s]);          // the stage is free once these products have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[as]);              // this tile's accumulator is complete
                ++acc_it;
            }
        }
    } else if (warp < 6) {
        // ---- epilogue: warps 2..5, each its own quarter of the 128 lanes --------------------
        if (early_ok) cj::after_predecessor();
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;           // accumulator row of this thread
        uint32_t acc_it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            TileCoord c = decode_tile<TOK_TILE>(p, tile, feat_tiles, tok_tiles, tiles_before, feat_tile);
            if (!c.valid) continue;
            const int as = acc_it % ACC_STAGES;
            ok = mbar_wait(&acc_full[as], (acc_it / ACC_STAGES) & 1, 3);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t lane_base = tmem_base + as * STAGE_COLS + ((uint32_t)(quarter * 32) << 16);
            const long long split_off = (long long)c.split * p.split_stride;
            const bool add_bias = p.bias != nullptr && c.split == 0;
#pragma unroll 1
            for (int c0 = 0; c0 < N_MMA; c0 += 16) {
                if (SWAP && c.tok0 + c0 >= c.tok_end) break;           // no token left in these columns
                uint32_t v0[16], v1[16];
                if (c.n_kb > 0) {
                    tmem_ld16(lane_base + c0, v0);
                    if (DUAL) tmem_ld16(lane_base + ACC_COLS + c0, v1);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v0[j] = v1[j] = 0;
                }
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    v[j] = __uint_as_float(v0[j]);
                    // the result is rounded to bfloat16 (8 bits): the fast exponential and division (2 ulp of float32) do not show
                    if (EPI == EPI_SWIGLU_BF16) v[j] = __fdividef(v[j], 1.0f + __expf(-v[j])) * __uint_as_float(v1[j]);
                }
                if (!SWAP) {
                    // this thread owns one token row and 16 consecutive features of it
                    const int token = c.tok0 + r, feat = c.feat0 + c0;
                    if (token >= c.tok_end || feat >= p.features) continue;
                    const long long o = (long long)token * p.ldo + feat;
                    const bool whole = feat + 16 <= p.features;
                    if (add_bias) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (whole || feat + j < p.features) v[j] += p.bias[feat + j];
                    }
                    if (EPI == EPI_STORE_F32 || EPI == EPI_ACC_F32) {
                        float* dst = (float*)p.out + o + (EPI == EPI_STORE_F32 ? split_off : 0);
                        if (whole && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                float4 w4 = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                if (EPI == EPI_ACC_F32) {
                                    float4 old = *(float4*)(dst + j);
                                    w4.x += old.x; w4.y += old.y; w4.z += old.z; w4.w += old.w;
                                }
                                *(float4*)(dst + j) = w4;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (feat + j < p.features) dst[j] = EPI == EPI_ACC_F32 ? dst[j] + v[j] : v[j];
                        }
                    } else {
                        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + o;
                        if (whole && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 16; j += 8) {
                                uint4 u;
                                __nv_bfloat162* b2 = (__nv_bfloat162*)&u;
#pragma unroll
                                for (int q = 0; q < 4; ++q) b2[q] = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                                *(uint4*)(dst + j) = u;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (feat + j < p.features) dst[j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                } else {
                    // this thread owns one feature; column j is token tok0 + c0 + j, so a warp
                    // writes 32 consecutive features of a token at a time
                    const int feat = c.feat0 + r;
                    if (r >= feat_tile || feat >= p.features) continue;
                    const float b = add_bias ? p.bias[feat] : 0.0f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        int token = c.tok0 + c0 + j;
                        if (token >= c.tok_end) break;
                        long long o = (long long)token * p.ldo + feat;
                        float val = v[j] + b;
                        if (EPI == EPI_STORE_F32) ((float*)p.out)[o + split_off] = val;
                        else if (EPI == EPI_ACC_F32) ((float*)p.out)[o] += val;
                        else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(val);
                    }
                }
            }
            // this warp has read its quarter of the accumulator: hand the stage back
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
            ++acc_it;
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
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

// CAJETA_B200_TILE_HEIGHTS=0 keeps tiles of 128 weight rows in every launch
inline bool tile_heights() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("CAJETA_B200_TILE_HEIGHTS");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

template <int N_MMA, bool SWAP, bool DUAL, int EPI, int STAGES>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mw2, const LowTiles& low, const Args& a, cudaStream_t stream) {
    using S = Smem<N_MMA, SWAP, DUAL, STAGES>;
    auto kern = gemm_tc_kernel<N_MMA, SWAP, DUAL, EPI, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (a.group_offsets && a.groups > MAX_GROUPS) return CJ_ERR_SIZE;
    int feat_tiles = (a.features + S::W_ROWS - 1) / S::W_ROWS;
    int tok_tiles = (a.tokens + S::X_ROWS - 1) / S::X_ROWS + (a.group_offsets ? a.groups : 0);
    // (with lower tiles there are more of them: the bound covers the lowest)
    const int most_feat_tiles = a.choose_height ? (a.features + low_height(LOW_HEIGHTS - 1) - 1) / low_height(LOW_HEIGHTS - 1) : feat_tiles;
    long long total = (long long)most_feat_tiles * tok_tiles * a.k_splits;
    if (total > 0x7fffffffLL) return CJ_ERR_SIZE;
    int grid = (int)(total < sm_count() ? total : sm_count());
    cj::launch(kern, dim3(grid), dim3(THREADS), S::TOTAL, stream, mx, mw, mw2, low, a, feat_tiles, tok_tiles, (int)((long long)feat_tiles * tok_tiles * a.k_splits));
    return cj::launch_status();
}

// stages chosen so that a block stays within ~200 KB of shared memory; products of few rows
// (weights on the rows, up to 32 tokens) take all the shared memory there is: they are bound by
// HBM, and what an SM has in flight is its ring (six stages of 34 KB instead of five: +2 %
// decode tokens a second at batch 8; three stages, so that two kernels' blocks fit an SM
// side by side: -7 %)
template <int N_MMA, bool SWAP, bool DUAL, int EPI>
int launch_auto(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mw2, const LowTiles& low, const Args& a, cudaStream_t stream) {
    constexpr int stage = Smem<N_MMA, SWAP, DUAL, 1>::STAGE_BYTES;
    constexpr int budget = (SWAP && N_MMA <= 32 ? 222 : 200) * 1024;
    constexpr int cap = SWAP && N_MMA <= 32 ? 12 : 8;
    constexpr int STAGES = (budget / stage) > cap ? cap : (budget / stage);
    return launch<N_MMA, SWAP, DUAL, EPI, STAGES>(mx, mw, mw2, low, a, stream);
}

template <bool SWAP, bool DUAL, int EPI>
int dispatch_n(int n_mma, const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mw2, const LowTiles& low, const Args& a, cudaStream_t s) {
    if constexpr (SWAP) {
        switch (n_mma) {
            case 16: return launch_auto<16, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 32: return launch_auto<32, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 64: return launch_auto<64, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 96: return launch_auto<96, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 128: return launch_auto<128, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 160: return launch_auto<160, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 192: return launch_auto<192, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 256: return launch_auto<256, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
        }
    } else {
        switch (n_mma) {
            case 128: return launch_auto<128, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
            case 256: if constexpr (!DUAL) return launch_auto<256, SWAP, DUAL, EPI>(mx, mw, mw2, low, a, s);
        }
    }
    return CJ_ERR_SIZE;
}

}  // namespace

// x: [tokens, K] bf16 with row stride ldx; w (and w2 for SwiGLU): [groups * features, K] bf16,
// contiguous.  swap: 0 = tokens on the product's rows (tile 128 tokens x n_mma features),
// 1 = weights on the rows (tile 128 features x n_mma tokens).  epilogue: 0 float32 store,
// 1 float32 accumulate, 2 SwiGLU to bf16 (needs w2), 3 bf16 store.  k_splits > 1 only with
// epilogue 0: split s stores its partial sum at out + s * split_stride (the bias goes to
// split 0).  offsets_settled: non-zero if group_offsets were complete before the kernel
// before this launch began (not merely before this launch): the kernel then reads them, and
// sends for its first weight tiles, while that kernel is still draining.  Refuses (negative
// code) what it cannot run; never a wrong result.
CJ_EXPORT int cj_gemm_tc(const void* x, long long ldx, const void* w, const void* w2, const float* bias, void* out,
                         long long ldo, int tokens, int features, int K, int epilogue, int swap, int n_mma,
                         const int* group_offsets, int groups, int k_splits, long long split_stride,
                         int offsets_settled, cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (!x || !w || !out || K <= 0) return CJ_ERR_ARG;
    if (K % 8 != 0 || ldx % 8 != 0) return CJ_ERR_ALIGN;               // TMA: 16-byte strides
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)w2) & 15) return CJ_ERR_ALIGN;
    if ((epilogue == EPI_SWIGLU_BF16) != (w2 != nullptr)) return CJ_ERR_ARG;
    if (k_splits < 1 || (k_splits > 1 && epilogue != EPI_STORE_F32)) return CJ_ERR_ARG;
    if (group_offsets && groups <= 0) return CJ_ERR_ARG;
    int total_w_rows = (group_offsets ? groups : 1) * features;
    int x_box = swap ? n_mma : 128, w_box = swap ? 128 : n_mma;
    CUtensorMap mx, mw, mw2;
    if (!make_map_bf16(&mx, x, tokens, K, ldx, x_box)) return CJ_ERR_ARG;
    if (!make_map_bf16(&mw, w, total_w_rows, K, K, w_box)) return CJ_ERR_ARG;
    if (w2) { if (!make_map_bf16(&mw2, w2, total_w_rows, K, K, w_box)) return CJ_ERR_ARG; }
    else mw2 = mw;
    // a decode step's grouped products (weights on the rows, a handful of tokens): the kernel chooses the tile's height
    const int choose_height = (swap && group_offsets && n_mma <= 32 && features > 128 && tile_heights()) ? 1 : 0;
    LowTiles low;
    for (int i = 0; i < LOW_HEIGHTS; ++i) {
        low.w[i] = mw;
        low.w2[i] = mw2;
        if (choose_height) {
            if (!make_map_bf16(&low.w[i], w, total_w_rows, K, K, low_height(i))) return CJ_ERR_ARG;
            if (w2 && !make_map_bf16(&low.w2[i], w2, total_w_rows, K, K, low_height(i))) return CJ_ERR_ARG;
        }
    }
    Args a{tokens, features, K, out, ldo, bias, group_offsets, groups, k_splits, split_stride, offsets_settled, choose_height};
#define CASE(EPI, DUAL)                                                                              \
    if (swap) return dispatch_n<true, DUAL, EPI>(n_mma, mx, mw, mw2, low, a, stream);                 \
    else return dispatch_n<false, DUAL, EPI>(n_mma, mx, mw, mw2, low, a, stream);
    switch (epilogue) {
        case EPI_STORE_F32: CASE(EPI_STORE_F32, false)
        case EPI_ACC_F32: CASE(EPI_ACC_F32, false)
        case EPI_SWIGLU_BF16: CASE(EPI_SWIGLU_BF16, true)
        case EPI_STORE_BF16: CASE(EPI_STORE_BF16, false)
    }
#undef CASE
    return CJ_ERR_ARG;
}

// 0, or the code of the first bounded wait that ran out (1 producer, 2 product issue,
// 3 epilogue); reading it synchronises the device.
CJ_EXPORT int cj_gemm_tc_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_error_flag, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
