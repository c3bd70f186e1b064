// Attention for prompt portions on the 5th-generation tensor cores (tcgen05), head size 128.
//
// A block takes 128 query rows of one request and one query head.  Per tile of 128 keys:
//     S = Q . K^T        tcgen05.mma, Q and K tiles in 128-byte-swizzled shared memory (TMA),
//                        the score tile [128 x 128] float32 in tensor memory (two of them,
//                        so that the next tile's scores are computed while this one's
//                        softmax runs)
//     P = exp2(S - m)    four warps, one query row per thread: the row comes out of tensor
//                        memory with tcgen05.ld, mask / running max / sum in float32
//                        registers, P goes to shared memory as bf16 in the K-major
//                        swizzled layout the next product reads
//     O += P . V         tcgen05.mma with V as an MN-major operand (V rows are keys, the
//                        head's dims are contiguous), O [128 x 128] float32 in tensor memory
// The running maximum is only moved (and O rescaled, through tcgen05.ld / st) when a tile
// raises it by more than 2^8; otherwise the old reference stays, which keeps P <= 256 and
// the rescale rare.  Keys and values come from the cache pages by TMA, one box of
// [16 keys x 64 dims] per page and half; a page that does not exist (a stretch before the
// window, or past the end) is fetched at an out-of-range coordinate, which TMA fills with
// zeros.  Roles: warp 0 TMA, warp 1 products and tensor-memory allocation, warps 2..5
// softmax, rescale and the final normalisation.
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
constexpr int BM = 128;            // query rows a block
constexpr int BN = 128;            // keys a tile
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr int HALF_BYTES = 128 * 64 * 2;          // a [128 x 64] bf16 swizzled half tile: 16 KB
constexpr int TILE_BYTES = 2 * HALF_BYTES;        // a [128 x 128] bf16 tile: 32 KB
constexpr float RESCALE_THRESHOLD = 8.0f;         // in log2 units

// shared memory: Q | K ring | V ring | P | barriers
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + TILE_BYTES;
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;
constexpr int SMEM_P = SMEM_V + KV_STAGES * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_P + 2 * TILE_BYTES;       // two P tiles: tile i + 1 is written while the product reads tile i
constexpr int SMEM_TOTAL = SMEM_BAR + 256 + 1024;

// tensor memory columns: S0 | S1 | O
constexpr uint32_t TM_S0 = 0, TM_S1 = 128, TM_O = 256, TM_COLS = 512;

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
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {       // 2^x, 0 for -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 32 consecutive 32-bit columns of this thread's lane into v[OFF .. OFF + 31]
template <int OFF>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[128]) {
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
};

__global__ void __launch_bounds__(THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, Args p) {
    cj::after_predecessor();
    // ---- which request and which 128-row tile of it (last tiles first) --------------------
    int tile = (int)gridDim.x - 1 - (int)blockIdx.x, req = -1, row0 = 0, rows = 0, first = 0;
    for (int r = 0; r < p.n_requests; ++r) {
        int lo = p.req_start[r], hi = p.req_start[r + 1];
        int tiles = (hi - lo + BM - 1) / BM;
        if (tile < first + tiles) {
            req = r;
            row0 = lo + (tile - first) * BM;
            rows = min(BM, hi - row0);
            break;
        }
        first += tiles;
    }
    if (req < 0) return;
    const int h = blockIdx.y, kvh = h / (p.n_heads / p.n_kv);
    const int p0 = p.req_prior[req] + (row0 - p.req_start[req]);
    const int p_last = p0 + rows - 1;
    const int key_from = (p.window > 0 && p0 + 1 > p.window) ? p0 + 1 - p.window : 0;
    const int kt_begin = key_from / BN, kt_end = p_last / BN;
    const int n_tiles = kt_end - kt_begin + 1;
    const int* tab = p.table + (size_t)req * p.table_stride;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + SMEM_BAR);
    uint64_t* q_full = bars;                      // Q tile landed
    uint64_t* k_full = bars + 1;                  // [KV_STAGES] K of a tile landed
    uint64_t* k_empty = k_full + KV_STAGES;       // [KV_STAGES] the score product has read it
    uint64_t* v_full = k_empty + KV_STAGES;       // [KV_STAGES] V of a tile landed
    uint64_t* v_empty = v_full + KV_STAGES;       // [KV_STAGES] the output product has read it
    uint64_t* s_full = v_empty + KV_STAGES;       // [2] score tile complete
    uint64_t* s_empty = s_full + 2;               // [2] softmax has read the score tile
    uint64_t* p_full = s_empty + 2;               // P written (and O rescaled): the PV product may go
    uint64_t* pv_done = p_full + 1;               // the PV product has read P and updated O
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1), mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1), mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 128); }
        mbar_init(p_full, 128);
        mbar_init(pv_done, 1);
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
            // Q: rows [row0, row0 + 128) of the [T, heads * 128] view, columns of this head; rows
            // past the step's end read as zero
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_2d(smem + SMEM_Q, &map_q, q_full, h * HD, row0);
            tma_load_2d(smem + SMEM_Q + HALF_BYTES, &map_q, q_full, h * HD + 64, row0);
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
        if (elect_one()) {
            bool ok = mbar_wait(q_full, 0, 12);
            const uint64_t dq0 = umma_desc_sw128(smem + SMEM_Q), dq1 = umma_desc_sw128(smem + SMEM_Q + HALF_BYTES);
            auto issue_qk = [&](int i) -> bool {
                const int s = i % KV_STAGES, sb = i & 1;
                if (!mbar_wait(&k_full[s], (i / KV_STAGES) & 1, 13)) return false;
                if (!mbar_wait(&s_empty[sb], ((i >> 1) & 1) ^ 1, 14)) return false;
                tcgen05_fence_after();
                const uint64_t dk0 = umma_desc_sw128(smem + SMEM_K + s * TILE_BYTES);
                const uint64_t dk1 = umma_desc_sw128(smem + SMEM_K + s * TILE_BYTES + HALF_BYTES);
                const uint32_t acc = tmem_base + (sb ? TM_S1 : TM_S0);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(acc, dq0 + 2 * k, dk0 + 2 * k, IDESC_QK, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(acc, dq1 + 2 * k, dk1 + 2 * k, IDESC_QK, 1);
                umma_commit(&k_empty[s]);        // K of this tile is free
                umma_commit(&s_full[sb]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int i = 0; i < n_tiles && ok; ++i) {
                // the next tile's scores first: they run while the softmax of tile i does
                if (i + 1 < n_tiles) { ok = issue_qk(i + 1); if (!ok) break; }
                const int s = i % KV_STAGES;
                ok = mbar_wait(&v_full[s], (i / KV_STAGES) & 1, 19) && mbar_wait(p_full, i & 1, 15);
                if (!ok) break;
                tcgen05_fence_after();
                const uint64_t dv = umma_desc_mn_sw128(smem + SMEM_V + s * TILE_BYTES);
                const uint64_t dp0 = umma_desc_sw128(smem + SMEM_P + (i & 1) * TILE_BYTES);
                const uint64_t dp1 = umma_desc_sw128(smem + SMEM_P + (i & 1) * TILE_BYTES + HALF_BYTES);
                // K of this product = keys: 16 keys = two 8-row groups = 2048 bytes a step
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + TM_O, dp0 + 2 * k, dv + (uint64_t)(k * 2048 >> 4), IDESC_PV, (i > 0 || k > 0) ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + TM_O, dp1 + 2 * k, dv + (uint64_t)((4 + k) * 2048 >> 4), IDESC_PV, 1);
                umma_commit(&v_empty[s]);        // V of this tile is free
                umma_commit(pv_done);            // P is free, O is updated
            }
        }
    } else {
        // ---- softmax: one query row per thread ---------------------------------------------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int pos = p0 + r;
        const int from = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        float m_ref = -INFINITY, l = 0.0f;
        uint8_t* prow = smem + SMEM_P + r * 128;          // this row inside each [128 x 64] half
        bool ok = true;
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int sb = i & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (i >> 1) & 1, 16));
            if (!ok) break;
            tcgen05_fence_after();
            // the whole row of scores into registers; the buffer is free for the tile after next
            uint32_t v[128];
            const uint32_t s_addr = tmem_base + (sb ? TM_S1 : TM_S0) + lane_off;
            tmem_ld32<0>(s_addr, v);
            tmem_ld32<32>(s_addr + 32, v);
            tmem_ld32<64>(s_addr + 64, v);
            tmem_ld32<96>(s_addr + 96, v);
            tmem_ld_wait();
            tcgen05_fence_before();
            mbar_arrive(&s_empty[sb]);
            // columns [lo, lo + span] of this tile are keys this row may see (span < 0: none)
            const int kbase = (kt_begin + i) * BN;
            const int lo = max(from - kbase, 0);
            const int span = min(pos - kbase, BN - 1) - lo;
            if (lo != 0 || span != BN - 1) {
#pragma unroll
                for (int c = 0; c < BN; ++c)
                    if (!((unsigned)(c - lo) <= (unsigned)span && span >= 0)) v[c] = 0xff800000u;       // -inf
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < BN; c += 4) {
                mx0 = fmaxf(mx0, __uint_as_float(v[c]));
                mx1 = fmaxf(mx1, __uint_as_float(v[c + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(v[c + 2]));
                mx3 = fmaxf(mx3, __uint_as_float(v[c + 3]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;      // scale > 0
            // the reference maximum moves only when the tile raises it by more than the threshold
            float m_new = m_ref;
            if (mx > m_ref + RESCALE_THRESHOLD || m_ref == -INFINITY) m_new = fmaxf(m_ref, mx);
            const bool rescale = m_new != m_ref && m_ref != -INFINITY;
            const float factor = rescale ? exp2f(m_ref - m_new) : 1.0f;
            const float neg_sub = m_new == -INFINITY ? 0.0f : -m_new;
            // P = exp2(S * scale - m) as bf16 into this tile's P buffer (the product that read
            // it two tiles ago finished before this tile's scores were complete)
            uint8_t* pr = prow + sb * TILE_BYTES;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 8) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    float e0 = ex2(fmaf(__uint_as_float(v[c0 + j]), p.scale_log2, neg_sub));
                    float e1 = ex2(fmaf(__uint_as_float(v[c0 + j + 1]), p.scale_log2, neg_sub));
                    sum0 += e0;
                    sum1 += e1;
                    __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
                    packed[j >> 1] = *(uint32_t*)&b;
                }
                // 8 keys = one 16-byte piece of this row's 128-byte line in half (c0 / 64)
                uint8_t* line = pr + (c0 >> 6) * HALF_BYTES;
                const int piece = (c0 & 63) >> 3;
                *(uint4*)(line + ((piece ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            l = l * factor + (sum0 + sum1);
            m_ref = m_new;
            // the product of the tile before has read its P and updated O by now, as a rule; every
            // phase of this barrier is waited for in turn, so that its parity stays unambiguous
            if (i > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (i - 1) & 1, 17));
                if (!ok) break;
            }
            // rare: bring O to the new reference
            if (__any_sync(0xffffffffu, rescale)) {
                tcgen05_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 16) {
                    uint32_t o[16];
                    tmem_ld16(tmem_base + TM_O + lane_off + c0, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
                    tmem_st16(tmem_base + TM_O + lane_off + c0, o);
                }
                tmem_st_wait();
            }
            // P is in shared memory (generic proxy): make it visible to the tensor core's reads
            fence_async_smem();
            tcgen05_fence_before();
            mbar_arrive(p_full);
        }
        // ---- the row's result: O / l ------------------------------------------------------------
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (n_tiles - 1) & 1, 18));
        if (ok) {
            tcgen05_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + r) * p.n_heads + h) * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + TM_O + lane_off + c0, v);
                tmem_ld_wait();
                if (r < rows) {
                    uint4 u0, u1;
                    __nv_bfloat162* b0 = (__nv_bfloat162*)&u0;
                    __nv_bfloat162* b1 = (__nv_bfloat162*)&u1;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        b0[j] = __floats2bfloat162_rn(__uint_as_float(v[2 * j]) * inv, __uint_as_float(v[2 * j + 1]) * inv);
                        b1[j] = __floats2bfloat162_rn(__uint_as_float(v[8 + 2 * j]) * inv, __uint_as_float(v[8 + 2 * j + 1]) * inv);
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
// req_prior [n_requests].  Head size 128 and 16-token pages only; refuses anything else.
CJ_EXPORT int cj_prefill_attention_tc(const void* q, void* out, const void* kplane, const void* vplane, int n_pages,
                                      const int* req_start, const int* req_prior, int n_requests, int total_rows,
                                      const int* table, int table_stride, int page_tokens, int n_heads, int n_kv,
                                      int hd, int window, float scale, cudaStream_t stream) {
    if (total_rows <= 0 || n_requests <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !req_start || !req_prior || !table) return CJ_ERR_ARG;
    if (hd != HD || page_tokens != 16) return CJ_ERR_SIZE;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || n_heads > 65535 || n_pages <= 0) return CJ_ERR_SIZE;
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
    Args a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, req_start, req_prior, table, n_requests, table_stride, page_tokens,
           n_heads, n_kv, window, scale * 1.4426950408889634f, (int)plane_rows};
    dim3 grid((total_rows + BM - 1) / BM + n_requests, n_heads);
    cj::launch(prefill_attention_tc_kernel, dim3(grid), dim3(THREADS), SMEM_TOTAL, stream, mq, mk, mv, a);
    return cj::launch_status();
}

CJ_EXPORT int cj_prefill_attention_tc_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_error_flag, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
