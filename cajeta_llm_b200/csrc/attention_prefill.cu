// Attention for steps that carry portions of prompts (bfloat16 path): tiles of 64 or 128 query
// rows of one request against tiles of 64 cached keys, scores and weighted values on the
// tensor cores (mma.sync m16n8k16, bf16 in, f32 out), softmax statistics in float32
// registers, keys and values fetched from cache pages through the block table with
// cp.async into swizzled shared memory, double buffered.
//
// Per row at position p: keys [from, p], from = p + 1 - w when a window is set and
// exceeded, else 0; s = (q . k) * scale; softmax with the running maximum subtracted;
// o = (sum e v) / (sum e)  (model/PagedKvCache.cajeta:374-470).  The reference's
// counterpart is its query-tiled flash prefill over the page table
// (model/AttnKernel.cajeta:2903).
//
// Rows are the step's rows: request r owns rows [req_start[r], req_start[r+1]) at
// positions req_prior[r] + i.  A block finds its (request, tile) by walking req_start.
#include "common.cuh"

using namespace cj;

namespace {


__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// element (row, col) of a [rows][HD] bf16 tile whose 16-byte chunks are XOR-swizzled by row
template <int HD>
__device__ __forceinline__ __nv_bfloat16* tile_ptr(__nv_bfloat16* base, int row, int col) {
    int chunk = (col >> 3) ^ (row & 7);
    return base + row * HD + chunk * 8 + (col & 7);
}

// HD: head size; BM: query rows a block; BN: keys a tile; MT: 16-row tiles a warp owns.  A
// warp that owns two row tiles uses every key/value fragment it reads from shared memory
// twice, which is what the legacy tensor path needs to stay ahead of shared-memory bandwidth.
template <int HD, int BM, int BN, int MT>
__global__ void __launch_bounds__(BM / (16 * MT) * 32) prefill_attention_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kplane,
    const __nv_bfloat16* __restrict__ vplane, const int* __restrict__ req_start, const int* __restrict__ req_prior,
    int n_requests, const int* __restrict__ table, int table_stride, int page_tokens, int n_heads, int n_kv, int window,
    float scale_log2) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;                 // [BM][HD]
    __nv_bfloat16* ks = qs + BM * HD;                             // [2][BN][HD]
    __nv_bfloat16* vs = ks + 2 * BN * HD;                         // [2][BN][HD]
    constexpr int CH = HD / 8;                                    // 16-byte chunks per row
    constexpr int THREADS = BM / (16 * MT) * 32;

    // ---- which request and which BM-row tile of it --------------------------------------
    // the grid walks the tiles from the last to the first: in a causal prompt the late tiles
    // have the most keys, and starting them first evens out the tail
    int tile = (int)gridDim.x - 1 - (int)blockIdx.x, req = -1, row0 = 0, rows = 0, first = 0;
    for (int r = 0; r < n_requests; ++r) {
        int lo = req_start[r], hi = req_start[r + 1];
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
    const int h = blockIdx.y, kvh = h / (n_heads / n_kv);
    const int p0 = req_prior[req] + (row0 - req_start[req]);     // position of the tile's first row
    const int p_last = p0 + rows - 1;
    const int key_from = (window > 0 && p0 + 1 > window) ? p0 + 1 - window : 0;
    const int kt_begin = key_from / BN, kt_end = p_last / BN;    // key tiles, inclusive
    const int* tab = table + (size_t)req * table_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- loads -----------------------------------------------------------------------------
    auto load_kv = [&](int kt, int buf) {
        __nv_bfloat16* kd = ks + buf * BN * HD;
        __nv_bfloat16* vd = vs + buf * BN * HD;
        for (int i = tid; i < BN * CH; i += THREADS) {
            int r = i / CH, c = i % CH;
            int key = kt * BN + r;
            bool valid = key <= p_last && key >= key_from;
            long long off = 0;
            if (valid) {
                int page = tab[key / page_tokens];
                valid = page >= 0;
                off = (((long long)(valid ? page : 0) * n_kv + kvh) * page_tokens + key % page_tokens) * HD + c * 8;
            }
            int pc = c ^ (r & 7);
            cp_async16(kd + r * HD + pc * 8, kplane + off, valid);
            cp_async16(vd + r * HD + pc * 8, vplane + off, valid);
        }
    };
    for (int i = tid; i < BM * CH; i += THREADS) {
        int r = i / CH, c = i % CH;
        bool valid = r < rows;
        const __nv_bfloat16* src = q + ((size_t)(row0 + (valid ? r : 0)) * n_heads + h) * HD + c * 8;
        cp_async16(qs + r * HD + (c ^ (r & 7)) * 8, src, valid);
    }
    load_kv(kt_begin, 0);
    cp_async_commit();

    // ---- per-warp state: MT tiles of 16 query rows; output accumulators, running max and sum ----
    const int g = lane >> 2, t4 = lane & 3;
    const int wrow = warp * 16 * MT;
    float o[MT][HD / 8][4];
    float mrun[MT][2], lrun[MT][2];                              // rows g and g + 8 of each tile
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.0f;
        mrun[mt][0] = mrun[mt][1] = -INFINITY;
        lrun[mt][0] = lrun[mt][1] = 0.0f;
    }

    for (int kt = kt_begin; kt <= kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt < kt_end) load_kv(kt + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* kb = ks + buf * BN * HD;
        const __nv_bfloat16* vb = vs + buf * BN * HD;

        // scores of MT x 16 rows x BN keys; the query fragments come from shared memory
        float s[MT][BN / 8][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            unsigned qf[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                ldmatrix_x4(qf[mt], tile_ptr<HD>(qs, wrow + mt * 16 + (lane & 15), kk * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int jp = 0; jp < BN / 16; ++jp) {
                unsigned b[4];
                int mi = lane >> 3;
                ldmatrix_x4(b, tile_ptr<HD>((__nv_bfloat16*)kb, jp * 16 + (mi >> 1) * 8 + (lane & 7), kk * 16 + (mi & 1) * 8));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16(s[mt][2 * jp], qf[mt], b[0], b[1]);
                    mma_bf16(s[mt][2 * jp + 1], qf[mt], b[2], b[3]);
                }
            }
        }
        // mask and running softmax
        const int kbase = kt * BN;
        unsigned pf[MT][BN / 16][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int pos0 = p0 + wrow + mt * 16 + g, pos1 = pos0 + 8;
            const int from0 = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
            const int from1 = (window > 0 && pos1 + 1 > window) ? pos1 + 1 - window : 0;
            float mx0 = mrun[mt][0], mx1 = mrun[mt][1];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    int key = kbase + j * 8 + 2 * t4 + e;
                    float a = (key <= pos0 && key >= from0) ? s[mt][j][e] * scale_log2 : -INFINITY;
                    float b = (key <= pos1 && key >= from1) ? s[mt][j][2 + e] * scale_log2 : -INFINITY;
                    s[mt][j][e] = a;
                    s[mt][j][2 + e] = b;
                    mx0 = fmaxf(mx0, a);
                    mx1 = fmaxf(mx1, b);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // a row that has seen no key yet (rows past the tile's end, or keys all masked so far) keeps -inf
            const float c0 = mx0 == -INFINITY ? 1.0f : exp2f(mrun[mt][0] - mx0);
            const float c1 = mx1 == -INFINITY ? 1.0f : exp2f(mrun[mt][1] - mx1);
            const float sub0 = mx0 == -INFINITY ? 0.0f : mx0, sub1 = mx1 == -INFINITY ? 0.0f : mx1;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
                float e0 = exp2f(s[mt][j][0] - sub0), e1 = exp2f(s[mt][j][1] - sub0);
                float e2 = exp2f(s[mt][j][2] - sub1), e3 = exp2f(s[mt][j][3] - sub1);
                sum0 += e0 + e1;
                sum1 += e2 + e3;
                pf[mt][j >> 1][(j & 1) * 2] = pack_bf16(e0, e1);
                pf[mt][j >> 1][(j & 1) * 2 + 1] = pack_bf16(e2, e3);
            }
            lrun[mt][0] = lrun[mt][0] * c0 + sum0;
            lrun[mt][1] = lrun[mt][1] * c1 + sum1;
            mrun[mt][0] = mx0;
            mrun[mt][1] = mx1;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[mt][i][0] *= c0; o[mt][i][1] *= c0;
                o[mt][i][2] *= c1; o[mt][i][3] *= c1;
            }
        }
        // weighted values: MT x 16 rows x HD += P[16 x BN] . V[BN x HD]
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                unsigned b[4];
                int mi = lane >> 3;
                ldmatrix_x4_trans(b, tile_ptr<HD>((__nv_bfloat16*)vb, kk * 16 + (mi & 1) * 8 + (lane & 7), dp * 16 + (mi >> 1) * 8));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16(o[mt][2 * dp], pf[mt][kk], b[0], b[1]);
                    mma_bf16(o[mt][2 * dp + 1], pf[mt][kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();                      // everyone is done with this buffer before it is refilled
    }

    // ---- finish: divide by the sum of the whole row (the quad holds the row) -------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float l0 = lrun[mt][0], l1 = lrun[mt][1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
        const int r0 = wrow + mt * 16 + g, r1 = r0 + 8;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            int col = i * 8 + 2 * t4;
            if (r0 < rows) *(unsigned*)(out + ((size_t)(row0 + r0) * n_heads + h) * HD + col) = pack_bf16(o[mt][i][0] * i0, o[mt][i][1] * i0);
            if (r1 < rows) *(unsigned*)(out + ((size_t)(row0 + r1) * n_heads + h) * HD + col) = pack_bf16(o[mt][i][2] * i1, o[mt][i][3] * i1);
        }
    }
}

}  // namespace

// q, out: [T, n_heads, hd] bf16; planes [pages, n_kv, page_tokens, hd] bf16; req_start
// [n_requests + 1], req_prior [n_requests] as the step function lays them out.  hd must be
// 64 or 128.  block_rows: 64 or 128 query rows a block, 0 = chosen from the step's shape.
CJ_EXPORT int cj_prefill_attention(const void* q, void* out, const void* kplane, const void* vplane, const int* req_start,
                                   const int* req_prior, int n_requests, int total_rows, const int* table, int table_stride,
                                   int page_tokens, int n_heads, int n_kv, int hd, int window, float scale,
                                   int block_rows, cudaStream_t stream) {
    if (total_rows <= 0 || n_requests <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !req_start || !req_prior || !table) return CJ_ERR_ARG;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0 || n_heads > 65535) return CJ_ERR_SIZE;
    if (hd != 64 && hd != 128) return CJ_ERR_SIZE;
    float scale_log2 = scale * 1.4426950408889634f;
    // long portions: 128 query rows a block, every warp two row tiles; short ones: 64 rows, one tile a warp
    const int bm = (block_rows == 128 || (block_rows == 0 && total_rows >= 128 * n_requests)) ? 128 : 64;
#define LAUNCH(HD, BM, BN, MT)                                                                                          \
    {                                                                                                                   \
        dim3 grid((total_rows + BM - 1) / BM + n_requests, n_heads);                                                    \
        size_t smem = (size_t)(BM + 4 * BN) * HD * sizeof(__nv_bfloat16);                                               \
        static bool configured = false;                                                                                 \
        if (!configured) {                                                                                              \
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<HD, BM, BN, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                        \
            configured = true;                                                                                          \
        }                                                                                                               \
        cj::launch(prefill_attention_kernel<HD, BM, BN, MT>, dim3(grid), dim3(BM / (16 * MT) * 32), smem, stream,                           \
            (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kplane, (const __nv_bfloat16*)vplane,   \
            req_start, req_prior, n_requests, table, table_stride, page_tokens, n_heads, n_kv, window, scale_log2);     \
    }
    if (hd == 128) { if (bm == 128) LAUNCH(128, 128, 32, 2) else LAUNCH(128, 64, 64, 1) }
    else { if (bm == 128) LAUNCH(64, 128, 64, 2) else LAUNCH(64, 64, 64, 1) }
#undef LAUNCH
    return launch_status();
}
