// General paged attention: one query row and head per block, keys and values read
// from cache pages through the request's block table.  It serves a portion of a prompt
// and a single decoded token alike (every row carries its own position), any head size
// up to 256, any group size, float32 or bfloat16 storage; all arithmetic is float32.
//
// For head h, kv head = h / (heads / kv_heads); keys t in [from, p] with
// from = p + 1 - w when w > 0 and p + 1 > w, else 0; s_t = (q . k_t) * scale; softmax
// with the maximum subtracted; o = (sum_t e_t v_t) / sum_t e_t
// (model/PagedKvCache.cajeta:374-470).  The keys of a row are cut into chunks of 32 that
// the block's warps take in turn, each keeping a running (max, sum, accumulator) as the
// reference's flash kernels do (model/AttnKernel.cajeta:883); the cut depends only on
// the row's own [from, p], so the result does not depend on the rest of the batch.
#include "common.cuh"

using namespace cj;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;
constexpr int DPL = MAX_HD / 32;   // output dims per lane

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kernel(
    const TQ* __restrict__ q, TO* __restrict__ out, const TC* __restrict__ kplane, const TC* __restrict__ vplane,
    const int* __restrict__ positions, const int* __restrict__ row_req, const int* __restrict__ table,
    int table_stride, int page_tokens, int n_heads, int n_kv, int hd, int window, float scale) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ float smem[];
    float* qs = smem;                       // [hd]
    float* acc_s = smem + hd;               // [WARPS][hd]
    float* m_s = acc_s + WARPS * hd;        // [WARPS]
    float* l_s = m_s + WARPS;               // [WARPS]

    int h = blockIdx.y, t = blockIdx.x;
    int kvh = h / (n_heads / n_kv);
    int p = positions[t];
    int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int* tab = table + (size_t)row_req[t] * table_stride;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const TQ* qrow = q + ((size_t)t * n_heads + h) * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f32(qrow[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;

    int n_keys = p - from + 1;
    int n_chunks = (n_keys + 31) / 32;
    for (int c = warp; c < n_chunks; c += WARPS) {
        int key = from + c * 32 + lane;
        bool valid = key <= p;
        float s = -INFINITY;
        size_t base = 0;
        if (valid) {
            int page = tab[key / page_tokens];
            base = (((size_t)page * n_kv + kvh) * page_tokens + key % page_tokens) * hd;
            const TC* kr = kplane + base;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
            s = dot * scale;
        }
        float cmax = warp_max(s);
        float m_new = fmaxf(m, cmax);
        float corr = expf(m - m_new);       // m = -inf on the first chunk: exp(-inf) = 0
        float e = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(e);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        int in_chunk = min(32, p - (from + c * 32) + 1);
        for (int j = 0; j < in_chunk; ++j) {
            float ej = __shfl_sync(0xffffffffu, e, j);
            size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
            const TC* vr = vplane + bj;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(ej, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }

    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        int d = lane + 32 * i;
        if (d < hd) acc_s[warp * hd + d] = acc[i];
    }
    __syncthreads();
    float mx = m_s[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, m_s[w]);
    float f[WARPS];
    float lsum = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - mx);
        lsum += l_s[w] * f[w];
    }
    float inv = 1.0f / lsum;
    TO* orow = out + ((size_t)t * n_heads + h) * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) o += acc_s[w * hd + d] * f[w];
        orow[d] = from_f32<TO>(o * inv);
    }
}

}  // namespace

// q, out: [T, n_heads, hd] in the activation dtype; planes: [pages, n_kv, page_tokens, hd].
CJ_EXPORT int cj_paged_attention(const void* q, void* out, int act_dtype, const void* kplane, const void* vplane,
                                 int cache_dtype, const int* positions, const int* row_req, const int* table,
                                 int table_stride, int page_tokens, int T, int n_heads, int n_kv, int hd,
                                 int window, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !row_req || !table) return CJ_ERR_ARG;
    if (hd <= 0 || hd > MAX_HD || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    if (n_heads > 65535) return CJ_ERR_SIZE;
    dim3 grid(T, n_heads);
    size_t smem = (size_t)(hd + WARPS * hd + 2 * WARPS) * sizeof(float);
#define LAUNCH(TQ, TC)                                                                                             \
    cj::launch(paged_attention_kernel<TQ, TC, TQ>, dim3(grid), dim3(WARPS * 32), smem, stream, (const TQ*)q, (TQ*)out, (const TC*)kplane, \
        (const TC*)vplane, positions, row_req, table, table_stride, page_tokens, n_heads, n_kv, hd, window, scale)
    if (act_dtype == CJ_F32 && cache_dtype == CJ_F32) LAUNCH(float, float);
    else if (act_dtype == CJ_BF16 && cache_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}
