// Attention for prompt portions on the 5th-generation tensor cores (tcgen05), head size 128.
//
// A block takes 256 query rows of one request and one query head, as two tiles of 128 rows
// that share every tile of 128 keys and values the block loads.  Per key tile and query tile:
//     S = Q . K^T        tcgen05.mma, Q and K tiles in 128-byte-swizzled shared memory (TMA),
//                        the score tile [128 x 128] float32 in tensor memory
//     P = exp2(S - m)    four warps a query tile, one row per thread: the row comes out of
//                        tensor memory with tcgen05.ld, mask / running max / sum in float32
//                        registers, P goes back as bf16 into the columns its scores came from
//     O += P . V         tcgen05.mma with P read from tensor memory and V as an MN-major
//                        operand from shared memory (V rows are keys, the head's dims are
//                        contiguous), O [128 x 128] float32 in tensor memory
// The two query tiles take turns: while the four warps of one compute exponentials (16 a clock
// on an SM, as long as both products of a tile take on the tensor core), the tensor core runs
// the other tile's products.  A key tile is worked on as two halves of 64 keys, each a step of
// the running softmax of its own, so that the output product over the first half runs while the
// second half's exponentials are computed.  A half is one pass over the scores in registers
// with the reference maximum the row has so far; its own maximum is found in the same pass, on
// units the exponentials leave idle, and only if it moves the reference is the pass repeated.
// The running maximum is only moved (and O rescaled, through tcgen05.ld / st) when a tile
// raises it by more than 2^8; otherwise the old reference stays, which keeps P <= 256 and
// the rescale rare.  Keys and values come from the cache pages by TMA, one box of
// [16 keys x 64 dims] per page and half; a page that does not exist (a stretch before the
// window, or past the end) is fetched at an out-of-range coordinate, which TMA fills with
// zeros.  Roles: warp 0 TMA, warp 1 products and tensor-memory allocation, warps 2..5 the
// first query tile's softmax, rescale and final normalisation, warps 6..9 the second's.
//
// Formula: model/PagedKvCache.cajeta:374-470 (keys [from, p], from = p + 1 - w under a
// window; softmax with the maximum subtracted; o = sum e v / sum e).  The reference's
// counterpart is its query-tiled f16-WMMA flash prefill, model/AttnKernel.cajeta:2903.
// Every wait is bounded (tc_common.cuh).
#include "common.cuh"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int HD = 128;            // head size this kernel is written for
constexpr int BM = 128;            // query rows a tile
constexpr int QT = 2;              // query tiles a block
constexpr int BN = 128;            // keys a tile
constexpr int KV_STAGES = 2;
constexpr int THREADS = 320;       // TMA warp, product warp, four softmax warps for each query tile
constexpr int HALF_BYTES = 128 * 64 * 2;          // a [128 x 64] bf16 swizzled half tile: 16 KB
constexpr int TILE_BYTES = 2 * HALF_BYTES;        // a [128 x 128] bf16 tile: 32 KB
constexpr float RESCALE_THRESHOLD = 8.0f;         // in log2 units

// shared memory: Q (two tiles) | K ring | V ring | barriers
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + QT * TILE_BYTES;
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_V + KV_STAGES * TILE_BYTES;
constexpr int SMEM_TOTAL = SMEM_BAR + 256 + 1024;

// tensor memory columns: scores of the two query tiles (P over the first 64 columns of its
// scores: 128 bf16 a row), then their outputs
constexpr uint32_t TM_S = 0, TM_O = 256, TM_COLS = 512;

// instruction descriptors (kind::f16, bf16 x bf16 -> f32, M = 128, N = 128): both operands
// K-major for S = Q K^T; B MN-major (bit 16) for O = P V
constexpr uint32_t IDESC_QK = umma_idesc_bf16(128, 128);
constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, 128) | (1u << 16);

// MN-major operand, 128-byte swizzle: 64 contiguous dims (128 bytes) per key row, 8 key rows
// per 1024-byte group (stride byte offset), the next 64 dims one half tile further (leading
// byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(const void* smem_tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(smem_tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)(HALF_BYTES >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's lane from v[OFF .. OFF + 31]
template <int OFF, int N>
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[N]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[OFF + 0]), "r"(v[OFF + 1]), "r"(v[OFF + 2]), "r"(v[OFF + 3]), "r"(v[OFF + 4]), "r"(v[OFF + 5]),
          "r"(v[OFF + 6]), "r"(v[OFF + 7]), "r"(v[OFF + 8]), "r"(v[OFF + 9]), "r"(v[OFF + 10]), "r"(v[OFF + 11]),
          "r"(v[OFF + 12]), "r"(v[OFF + 13]), "r"(v[OFF + 14]), "r"(v[OFF + 15]), "r"(v[OFF + 16]), "r"(v[OFF + 17]),
          "r"(v[OFF + 18]), "r"(v[OFF + 19]), "r"(v[OFF + 20]), "r"(v[OFF + 21]), "r"(v[OFF + 22]), "r"(v[OFF + 23]),
          "r"(v[OFF + 24]), "r"(v[OFF + 25]), "r"(v[OFF + 26]), "r"(v[OFF + 27]), "r"(v[OFF + 28]), "r"(v[OFF + 29]),
          "r"(v[OFF + 30]), "r"(v[OFF + 31])
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A's rows are the lanes, two bf16 of consecutive k per column
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// two float32 operations in one instruction (sm_100 f32x2), and the maximum of three
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float2 unpack2(f32x2 v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float ex2(float x) {       // 2^x, 0 for -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 32 consecutive 32-bit columns of this thread's lane into v[OFF .. OFF + 31]
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[N]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[OFF + 0]), "=r"(v[OFF + 1]), "=r"(v[OFF + 2]), "=r"(v[OFF + 3]), "=r"(v[OFF + 4]), "=r"(v[OFF + 5]),
          "=r"(v[OFF + 6]), "=r"(v[OFF + 7]), "=r"(v[OFF + 8]), "=r"(v[OFF + 9]), "=r"(v[OFF + 10]), "=r"(v[OFF + 11]),
          "=r"(v[OFF + 12]), "=r"(v[OFF + 13]), "=r"(v[OFF + 14]), "=r"(v[OFF + 15]), "=r"(v[OFF + 16]), "=r"(v[OFF + 17]),
          "=r"(v[OFF + 18]), "=r"(v[OFF + 19]), "=r"(v[OFF + 20]), "=r"(v[OFF + 21]), "=r"(v[OFF + 22]), "=r"(v[OFF + 23]),
          "=r"(v[OFF + 24]), "=r"(v[OFF + 25]), "=r"(v[OFF + 26]), "=r"(v[OFF + 27]), "=r"(v[OFF + 28]), "=r"(v[OFF + 29]),
          "=r"(v[OFF + 30]), "=r"(v[OFF + 31])
        : "r"(taddr)
        : "memory");
}

struct Args {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* req_start;
    const int* req_prior;
    const int* table;
    int n_requests, table_stride, page_tokens, n_heads, n_kv, window;
    float scale_log2;
    int plane_rows;            // rows of the [pages * n_kv * page_tokens, 128] view of a cache plane
    int block_rows;            // query rows a block takes: 256 (both tiles) or 128 (the second tile stays empty)
};

// What a query tile of the block covers: its rows, positions and the key tiles it needs.
struct QueryTile {
    int rows;          // rows of the step in this tile (0: the tile is empty)
    int p0;            // position of its first row in the request
    int begin, end;    // key tiles [begin, end] it needs, counted from the block's first key tile (begin > end: none)
};

__global__ void __launch_bounds__(THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, Args p) {
    // A step's arrays are laid out for more requests than it may have (the shape of a captured step
    // covers the most it can hold), and the grid for the most row blocks those could make: most
    // blocks of such a launch have nothing to do.  Each finds that out from the sum of the
    // requests' row blocks - a few loads a lane, before anything else (the step's layout was
    // written before the step's first kernel) - and leaves at once; an idle block that walked the
    // whole list first kept an SM for as long as a short row block takes.
    {
        int tiles = 0;
        for (int r = threadIdx.x & 31; r < p.n_requests; r += 32)
            tiles += (__ldcg(p.req_start + r + 1) - __ldcg(p.req_start + r) + p.block_rows - 1) / p.block_rows;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tiles += __shfl_xor_sync(0xffffffffu, tiles, o);
        if ((int)blockIdx.y >= tiles) {
            cj::after_predecessor();
            return;
        }
    }
    cj::after_predecessor();
    // ---- which request and which 256 rows of it -----------------------------------------------
    // Blocks start in the order of blockIdx.y; the last rows of a request see the most keys, so
    // the last 256 rows of every request come first, then the 256 before them, and so on: the
    // longest blocks start first and the short ones fill the gaps at the end.
    // A block takes 256 rows (two tiles taking turns between the exponential unit and the tensor
    // core: by far the better rate a key tile) or, when a launch is so small that most SMs would
    // have no block, 128 (twice as many blocks, half as long).
    const int BLOCK_ROWS = p.block_rows;
    int req = -1, row0 = 0, rows = 0;
    {
        int b = (int)blockIdx.y;
        for (int level = 0; req < 0; ++level) {
            bool any = false;
            for (int r = 0; r < p.n_requests; ++r) {
                const int lo = p.req_start[r], n = p.req_start[r + 1] - lo;
                const int tiles = (n + BLOCK_ROWS - 1) / BLOCK_ROWS;
                if (tiles <= level) continue;
                any = true;
                if (b-- == 0) {
                    req = r;
                    row0 = lo + (tiles - 1 - level) * BLOCK_ROWS;
                    rows = min(BLOCK_ROWS, lo + n - row0);
                    break;
                }
            }
            if (!any) return;            // the grid has a few blocks more than there are tiles
        }
    }
    const int h = blockIdx.x, kvh = h / (p.n_heads / p.n_kv);
    const int p0 = p.req_prior[req] + (row0 - p.req_start[req]);
    const int p_last = p0 + rows - 1;
    const int key_from = (p.window > 0 && p0 + 1 > p.window) ? p0 + 1 - p.window : 0;
    const int kt_begin = key_from / BN;
    QueryTile qt[QT];
#pragma unroll
    for (int g = 0; g < QT; ++g) {
        qt[g].rows = max(0, min(BM, rows - g * BM));
        qt[g].p0 = p0 + g * BM;
        const int from = (p.window > 0 && qt[g].p0 + 1 > p.window) ? qt[g].p0 + 1 - p.window : 0;
        qt[g].begin = from / BN - kt_begin;
        qt[g].end = qt[g].rows > 0 ? (qt[g].p0 + qt[g].rows - 1) / BN - kt_begin : qt[g].begin - 1;
    }
    const int n_tiles = max(qt[0].end, qt[1].end) + 1;        // the first tile is never empty
    const int* tab = p.table + (size_t)req * p.table_stride;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + SMEM_BAR);
    uint64_t* q_full = bars;                      // both Q tiles landed
    uint64_t* k_full = bars + 1;                  // [KV_STAGES] K of a tile landed
    uint64_t* k_empty = k_full + KV_STAGES;       // [KV_STAGES] the score products have read it
    uint64_t* v_full = k_empty + KV_STAGES;       // [KV_STAGES] V of a tile landed
    uint64_t* v_empty = v_full + KV_STAGES;       // [KV_STAGES] the output products have read it
    uint64_t* s_full = v_empty + KV_STAGES;       // [QT] a query tile's scores are complete (and every product before them)
    uint64_t* p_full = s_full + QT;               // [QT][2] P of the tile's first / last 64 keys is written (and O rescaled): that half of the output product may go
    uint64_t* half_done = p_full + 2 * QT;        // [QT] the output product over a tile's first 64 keys is done
    uint64_t* o_done = half_done + QT;            // [QT] its last output product is done
    uint32_t* tmem_slot = (uint32_t*)(o_done + QT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1), mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1), mbar_init(&v_empty[s], 1);
        }
        for (int g = 0; g < QT; ++g) {
            mbar_init(&s_full[g], 1), mbar_init(&half_done[g], 1), mbar_init(&o_done[g], 1);
            mbar_init(&p_full[2 * g], BM), mbar_init(&p_full[2 * g + 1], BM);
        }
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TM_COLS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    // only now may a following kernel's blocks be scheduled beside this one: a block that took
    // tensor memory first and then waited for this kernel to end would starve this block's own
    // allocation
    cj::release_successor();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer -------------------------------------------------------------------
        if (elect_one()) {
            tma_prefetch_descriptor(&map_q);
            tma_prefetch_descriptor(&map_k);
            tma_prefetch_descriptor(&map_v);
            // Q: rows [row0, row0 + 256) of the [T, heads * 128] view, columns of this head; rows
            // past the step's end read as zero
            const int q_tiles = qt[1].rows > 0 ? 2 : 1;
            mbar_expect_tx(q_full, q_tiles * TILE_BYTES);
            for (int g = 0; g < q_tiles; ++g) {
                tma_load_2d(smem + SMEM_Q + g * TILE_BYTES, &map_q, q_full, h * HD, row0 + g * BM);
                tma_load_2d(smem + SMEM_Q + g * TILE_BYTES + HALF_BYTES, &map_q, q_full, h * HD + 64, row0 + g * BM);
            }
            // K runs ahead of V, in the order the products want them: K0, K1, V0, K2, V1, ...
            auto load_tile = [&](int i, bool values) -> bool {
                const int s = i % KV_STAGES;
                uint64_t* full = values ? &v_full[s] : &k_full[s];
                if (!mbar_wait(values ? &v_empty[s] : &k_empty[s], ((i / KV_STAGES) & 1) ^ 1, 11)) return false;
                mbar_expect_tx(full, TILE_BYTES);
                const int key0 = (kt_begin + i) * BN;
                uint8_t* dst = smem + (values ? SMEM_V : SMEM_K) + s * TILE_BYTES;
                const CUtensorMap* map = values ? &map_v : &map_k;
                for (int pg = 0; pg < BN / 16; ++pg) {
                    // one cache page (16 keys) at a time; page_tokens is 16 here
                    const int key = key0 + pg * 16;
                    int page = (key <= p_last && key + 15 >= key_from) ? tab[key / 16] : -1;
                    // a page that is not there is read past the end of the plane: zeros
                    const int row = page >= 0 ? (page * p.n_kv + kvh) * 16 : p.plane_rows;
                    tma_load_2d(dst + pg * 16 * 128, map, full, 0, row);
                    tma_load_2d(dst + HALF_BYTES + pg * 16 * 128, map, full, 64, row);
                }
                return true;
            };
            bool ok = load_tile(0, false);
            for (int i = 0; i < n_tiles && ok; ++i) {
                if (i + 1 < n_tiles) ok = load_tile(i + 1, false);
                if (ok) ok = load_tile(i, true);
            }
        }
    } else if (warp == 1) {
        // ---- products ------------------------------------------------------------------------
        // In the order issued: S_a(0) S_b(0), then per key tile i: PV_a(i) S_a(i + 1) PV_b(i) S_b(i + 1),
        // each PV in two halves of 64 keys.  S_g(i + 1) overwrites the columns PV_g(i) reads P from;
        // the tensor core runs one thread's products in the order they were issued.
        if (elect_one()) {
            bool ok = mbar_wait(q_full, 0, 12);
            int p_seen[QT] = {0, 0};                  // phases of p_full consumed
            auto uses = [&](int g, int i) { return i >= qt[g].begin && i <= qt[g].end; };
            auto scores = [&](int g, int i) {
                const int s = i % KV_STAGES;
                const uint64_t dq0 = umma_desc_sw128(smem + SMEM_Q + g * TILE_BYTES);
                const uint64_t dq1 = umma_desc_sw128(smem + SMEM_Q + g * TILE_BYTES + HALF_BYTES);
                const uint64_t dk0 = umma_desc_sw128(smem + SMEM_K + s * TILE_BYTES);
                const uint64_t dk1 = umma_desc_sw128(smem + SMEM_K + s * TILE_BYTES + HALF_BYTES);
                const uint32_t acc = tmem_base + TM_S + g * BN;
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(acc, dq0 + 2 * k, dk0 + 2 * k, IDESC_QK, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(acc, dq1 + 2 * k, dk1 + 2 * k, IDESC_QK, 1);
                umma_commit(&s_full[g]);
            };
            if (ok) ok = mbar_wait(&k_full[0], 0, 13);
            if (ok) {
                tcgen05_fence_after();
#pragma unroll
                for (int g = 0; g < QT; ++g)
                    if (uses(g, 0)) scores(g, 0);
                umma_commit(&k_empty[0]);
            }
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i % KV_STAGES;
                const bool next = i + 1 < n_tiles;
                ok = mbar_wait(&v_full[s], (i / KV_STAGES) & 1, 19);
                if (!ok) break;
                const uint64_t dv = umma_desc_mn_sw128(smem + SMEM_V + s * TILE_BYTES);
                bool k_there = false;
#pragma unroll
                for (int g = 0; g < QT; ++g) {
                    if (!ok) break;
                    if (uses(g, i)) {
                        const uint32_t acc = tmem_base + TM_O + g * HD, pa = tmem_base + TM_S + g * BN;
                        // the tile's first 64 keys go while the softmax works on its last 64
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            ok = mbar_wait(&p_full[2 * g + half], p_seen[g] & 1, 15);
                            if (!ok) break;
                            tcgen05_fence_after();
                            // K of this product = keys: 16 keys = 8 columns of P = two 8-row groups of V = 2048 bytes
#pragma unroll
                            for (int k = 4 * half; k < 4 * half + 4; ++k)
                                umma_bf16_a_tmem(acc, pa + 8 * k, dv + (uint64_t)(k * 2048 >> 4), IDESC_PV, (i > qt[g].begin || k > 0) ? 1u : 0u);
                            if (half == 0) umma_commit(&half_done[g]);
                        }
                        if (!ok) break;
                        ++p_seen[g];
                        if (i == qt[g].end) umma_commit(&o_done[g]);
                    }
                    if (g == QT - 1) umma_commit(&v_empty[s]);        // V of this tile is free
                    if (next && (uses(g, i + 1) || g == QT - 1)) {
                        if (!k_there) {
                            ok = mbar_wait(&k_full[(i + 1) % KV_STAGES], ((i + 1) / KV_STAGES) & 1, 13);
                            if (!ok) break;
                            tcgen05_fence_after();
                            k_there = true;
                        }
                        if (uses(g, i + 1)) scores(g, i + 1);
                        if (g == QT - 1) umma_commit(&k_empty[(i + 1) % KV_STAGES]);   // K of the next tile is free
                    }
                }
            }
        }
    } else {
        // ---- softmax of one query tile, one row per thread ------------------------------------------
        const int g = (warp - 2) >> 2;
        const int quarter = warp & 3;                      // the quarter of the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        const QueryTile mine = g == 0 ? qt[0] : qt[1];
        const int pos = mine.p0 + r;
        const int from = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + TM_S + g * BN + lane_off;
        const uint32_t o_addr = tmem_base + TM_O + g * HD + lane_off;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        const int n_mine = mine.end - mine.begin + 1;
        for (int j = 0; j < n_mine && ok; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[g], j & 1, 16));
            if (!ok) break;
            tcgen05_fence_after();
            // columns [lo, lo + span] of this tile are keys this row may see (span < 0: none)
            const int kbase = (kt_begin + mine.begin + j) * BN;
            const int lo = max(from - kbase, 0);
            const int span = min(pos - kbase, BN - 1) - lo;
            // The tile in two halves of 64 keys, each a step of the running softmax of its own: the
            // output product over the first half runs while the second is worked on.
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                constexpr int HC = BN / 2;
                uint32_t v[HC];
                tmem_ld32<0>(s_addr + half * HC, v);
                tmem_ld32<32>(s_addr + half * HC + 32, v);
                tmem_ld_wait();
                if (lo != 0 || span != BN - 1) {
#pragma unroll
                    for (int c = 0; c < HC; ++c)
                        if (!((unsigned)(half * HC + c - lo) <= (unsigned)span && span >= 0)) v[c] = 0xff800000u;       // -inf
                }
                // One pass gives P = exp2(S * scale - m) as bf16 (two keys a column), the sum and the
                // maximum of these 64 scores.  It runs with the reference maximum the row has so far;
                // only when these keys raise that by more than the threshold (or the row had none yet)
                // is the pass repeated with the new one, which is rare after a row's first keys.  The
                // maximum costs no time of its own this way: it is found on other units while the
                // exponential unit, which bounds the pass, works.
                float m_use = m_ref, factor = 1.0f, sum;
                bool rescale = false;
                uint32_t packed[HC];                   // only [0, 32) is used
#pragma unroll 1
                for (int attempt = 0;; ++attempt) {
                    const float neg_sub = m_use == -INFINITY ? 0.0f : -m_use;
                    const f32x2 scale2 = pack2(p.scale_log2, p.scale_log2), sub2 = pack2(neg_sub, neg_sub);
                    f32x2 sum2a = pack2(0.0f, 0.0f), sum2b = sum2a;
                    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                    for (int c = 0; c < HC; c += 4) {
                        const float2 t0 = unpack2(fma2(pack2(__uint_as_float(v[c]), __uint_as_float(v[c + 1])), scale2, sub2));
                        const float2 t1 = unpack2(fma2(pack2(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3])), scale2, sub2));
                        const float e0 = ex2(t0.x), e1 = ex2(t0.y), e2 = ex2(t1.x), e3 = ex2(t1.y);
                        sum2a = add2(sum2a, pack2(e0, e1));
                        sum2b = add2(sum2b, pack2(e2, e3));
                        __nv_bfloat162 b0 = __floats2bfloat162_rn(e0, e1), b1 = __floats2bfloat162_rn(e2, e3);
                        packed[c >> 1] = *(uint32_t*)&b0;
                        packed[(c >> 1) + 1] = *(uint32_t*)&b1;
                        mx0 = max3(mx0, __uint_as_float(v[c]), __uint_as_float(v[c + 1]));
                        mx1 = max3(mx1, __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
                    }
                    const float2 sa = unpack2(sum2a), sb = unpack2(sum2b);
                    sum = (sa.x + sa.y) + (sb.x + sb.y);
                    if (attempt == 1) break;
                    const float mx = fmaxf(mx0, mx1) * p.scale_log2;                         // scale > 0
                    float m_new = m_ref;
                    if (mx > m_ref + RESCALE_THRESHOLD || m_ref == -INFINITY) m_new = fmaxf(m_ref, mx);
                    if (!__any_sync(0xffffffffu, m_new != m_ref)) break;
                    rescale = m_new != m_ref && m_ref != -INFINITY;
                    factor = rescale ? exp2f(m_ref - m_new) : 1.0f;
                    m_use = m_new;
                }
                // the first half over columns [0, 32) of the scores, the second over [32, 64) (whose
                // scores the first half took)
                tmem_st32<0>(s_addr + half * (HC / 2), packed);
                l = l * factor + sum;
                m_ref = m_use;
                // O may be rescaled once the product before is done: the one over the last tile's second
                // half was done before this tile's scores were; the one over this tile's first half is
                // waited for here (every phase in turn, as a rule long complete)
                if (half == 1) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&half_done[g], j & 1, 17));
                    if (!ok) break;
                    tcgen05_fence_after();
                }
                if (__any_sync(0xffffffffu, rescale)) {        // rare
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 16) {
                        uint32_t o[16];
                        tmem_ld16(o_addr + c0, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 16; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * factor);
                        tmem_st16(o_addr + c0, o);
                    }
                }
                tmem_st_wait();
                tcgen05_fence_before();
                mbar_arrive(&p_full[2 * g + half]);
            }
        }
        // ---- the rows' results: O / l ----------------------------------------------------------------
        if (ok && n_mine > 0) ok = __all_sync(0xffffffffu, mbar_wait(&o_done[g], 0, 18));
        if (ok && n_mine > 0) {
            tcgen05_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + g * BM + r) * p.n_heads + h) * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 16) {
                uint32_t o[16];
                tmem_ld16(o_addr + c0, o);
                tmem_ld_wait();
                if (r < mine.rows) {
                    uint4 u0, u1;
                    __nv_bfloat162* b0 = (__nv_bfloat162*)&u0;
                    __nv_bfloat162* b1 = (__nv_bfloat162*)&u1;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        b0[q] = __floats2bfloat162_rn(__uint_as_float(o[2 * q]) * inv, __uint_as_float(o[2 * q + 1]) * inv);
                        b1[q] = __floats2bfloat162_rn(__uint_as_float(o[8 + 2 * q]) * inv, __uint_as_float(o[8 + 2 * q + 1]) * inv);
                    }
                    *(uint4*)(dst + c0) = u0;
                    *(uint4*)(dst + c0 + 8) = u1;
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// a [rows, cols] bf16 matrix cut into boxes of [box_rows, 64] with the 128-byte swizzle
bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    return make_map_bf16(map, base, rows, cols, ld, box_rows);
}

}  // namespace

// q, out: [T, n_heads, 128] bf16; planes [pages, n_kv, 16, 128] bf16; req_start [n_requests + 1],
// req_prior [n_requests].  Head size 128 and 16-token pages only; refuses anything else.  force_block_rows: 128 or 256
// query rows a block, or 0 to let the launch's size decide.
CJ_EXPORT int cj_prefill_attention_tc(const void* q, void* out, const void* kplane, const void* vplane, int n_pages,
                                      const int* req_start, const int* req_prior, int n_requests, int total_rows,
                                      const int* table, int table_stride, int page_tokens, int n_heads, int n_kv,
                                      int hd, int window, float scale, int force_block_rows, cudaStream_t stream) {
    if (total_rows <= 0 || n_requests <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !req_start || !req_prior || !table) return CJ_ERR_ARG;
    if (hd != HD || page_tokens != 16) return CJ_ERR_SIZE;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || n_pages <= 0) return CJ_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)kplane | (uintptr_t)vplane) & 15) return CJ_ERR_ALIGN;
    const long long plane_rows = (long long)n_pages * n_kv * 16;
    if (plane_rows > 0x7fffffffLL) return CJ_ERR_SIZE;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, q, total_rows, (long long)n_heads * HD, (long long)n_heads * HD, 128)) return CJ_ERR_ARG;
    if (!make_map(&mk, kplane, plane_rows, HD, HD, 16)) return CJ_ERR_ARG;
    if (!make_map(&mv, vplane, plane_rows, HD, HD, 16)) return CJ_ERR_ARG;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // 256 rows a block (two tiles taking turns: measured 1.9 times the rate of one tile a block)
    // unless that leaves more than half of the SMs without a block: then 128 (measured: one prompt
    // of 1,024 tokens 22.2 -> 19.5 us, of 512 tokens 14.9 -> 12.5 us; of 2,048 tokens 38.1 -> 40.1 us,
    // so that one stays at 256)
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sm_count = 1;
    }
    int block_rows = force_block_rows;
    if (block_rows != 128 && block_rows != 256) {
        const long long blocks_256 = ((total_rows + 255) / 256 + n_requests - 1) * n_heads;      // at most
        block_rows = 2 * blocks_256 <= sm_count ? 128 : 256;
    }
    Args a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, req_start, req_prior, table, n_requests, table_stride, page_tokens,
           n_heads, n_kv, window, scale * 1.4426950408889634f, (int)plane_rows, block_rows};
    // heads run fastest, so that blocks start in the order of their length (the last rows of a
    // request see the most keys) and the heads of one group read the same keys one after another
    const long long row_blocks = (total_rows + block_rows - 1) / block_rows + n_requests;
    if (row_blocks > 65535) return CJ_ERR_SIZE;
    dim3 grid(n_heads, (unsigned)row_blocks);
    cj::launch(prefill_attention_tc_kernel, dim3(grid), dim3(THREADS), SMEM_TOTAL, stream, mq, mk, mv, a);
    return cj::launch_status();
}

CJ_EXPORT int cj_prefill_attention_tc_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_error_flag, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
