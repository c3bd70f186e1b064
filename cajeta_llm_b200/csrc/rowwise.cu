// Row-wise kernels: embedding gather, RMSNorm, rotary encoding fused with the write
// of keys and values into cache pages, and the weighted combine of expert outputs.
// All statistics, angles and sums are float32; storage is float32 or bfloat16.
#include "common.cuh"

using namespace cj;

// ---------------------------------------------------------------------------------
// embedding: hs[t, :] = table[id_t, :] widened to float32 (the residual stream), times
// `scale` when that is not 0 (the reference's embedScale, 0 = none)
// reference: model/Embedding.cajeta:73-81, gather kernel io/QuantKernel.cajeta:40720
// ---------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                    const int* __restrict__ ids, int H, int V, float scale) {
    cj::after_predecessor();
    cj::release_successor();
    int t = blockIdx.x;
    int id = ids[t];
    bool ok = id >= 0 && id < V;   // the host checks ids; an id out of range reads nothing
    const TW* src = table + (size_t)(ok ? id : 0) * H;
    float* dst = out + (size_t)t * H;
    const float f = scale != 0.0f ? scale : 1.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? to_f32(src[i]) * f : 0.0f;
}

CJ_EXPORT int cj_embed_gather(float* out, const void* table, int table_dtype, const int* ids,
                              int T, int H, int V, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!out || !table || !ids || H <= 0 || V <= 0) return CJ_ERR_ARG;
    int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == CJ_F32)
        cj::launch(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, ids, H, V, scale);
    else if (table_dtype == CJ_BF16)
        cj::launch(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table, ids, H, V, scale);
    else
        return CJ_ERR_DTYPE;
    return launch_status();
}

// ---------------------------------------------------------------------------------
// RMSNorm: ss = sum x^2; scale = 1/sqrt(ss/dim + eps); y = x * scale * w
// reference: model/Prim.cajeta:120-151.  One block per output row; the input row may
// be picked through row_index (the rows whose logits are wanted).  Writes the result
// in the activation dtype and, when asked, a float32 copy (the router's input) or the
// same float32 value cut into three bfloat16 terms [rows, 3H] = hi | mid | lo with
// hi = bf16(y), mid = bf16(y - hi), lo = bf16(y - hi - mid): their sum is y to 2^-24, so
// a bfloat16 tensor-core product over the widened row gives float32-grade router logits.
// ---------------------------------------------------------------------------------
// The row is read once into registers (with the weight, whose load is then in flight during
// the reduction) when it fits PER elements a thread; otherwise it is read twice.
__device__ __forceinline__ void write_split(__nv_bfloat16* dst, int H, float y) {
    __nv_bfloat16 hi = __float2bfloat16_rn(y);
    float r1 = y - __bfloat162float(hi);
    __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    dst[0] = hi;
    dst[H] = mid;
    dst[2 * H] = lo;
}

template <typename TO, int PER>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ w, float eps, int H,
                               TO* __restrict__ out, float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_split,
                               const int* __restrict__ row_index, const float* __restrict__ partials, int n_partials,
                               long long partial_stride) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float partial[32];
    __shared__ float scale_s;
    int r = blockIdx.x;
    float* src = x + (size_t)(row_index ? row_index[r] : r) * H;
    float ss = 0.0f;
    float xv[PER > 0 ? PER : 1], wv[PER > 0 ? PER : 1];
    if (PER > 0) {
#pragma unroll
        for (int q = 0; q < PER; ++q) {
            int i = threadIdx.x + q * blockDim.x;
            xv[q] = i < H ? src[i] : 0.0f;
            wv[q] = i < H ? w[i] : 0.0f;
        }
        if (partials) {
            // the split sums of the product before this norm: added in split order, stored back
            for (int s = 0; s < n_partials; ++s)
#pragma unroll
                for (int q = 0; q < PER; ++q) {
                    int i = threadIdx.x + q * blockDim.x;
                    if (i < H) xv[q] += partials[s * partial_stride + (size_t)r * H + i];
                }
#pragma unroll
            for (int q = 0; q < PER; ++q) {
                int i = threadIdx.x + q * blockDim.x;
                if (i < H) src[i] = xv[q];
            }
        }
#pragma unroll
        for (int q = 0; q < PER; ++q) ss = fmaf(xv[q], xv[q], ss);
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = src[i];
            if (partials) {
                for (int s = 0; s < n_partials; ++s) v += partials[s * partial_stride + (size_t)r * H + i];
                src[i] = v;
            }
            ss = fmaf(v, v, ss);
        }
    }
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lane == 0) partial[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < nwarps ? partial[lane] : 0.0f;
        v = warp_sum(v);
        if (lane == 0) scale_s = 1.0f / sqrtf(v / (float)H + eps);
    }
    __syncthreads();
    float scale = scale_s;
    if (PER > 0) {
#pragma unroll
        for (int q = 0; q < PER; ++q) {
            int i = threadIdx.x + q * blockDim.x;
            if (i < H) {
                float y = xv[q] * scale * wv[q];
                out[(size_t)r * H + i] = from_f32<TO>(y);
                if (out_f32) out_f32[(size_t)r * H + i] = y;
                if (out_split) write_split(out_split + (size_t)r * 3 * H + i, H, y);
            }
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float y = src[i] * scale * w[i];
            out[(size_t)r * H + i] = from_f32<TO>(y);
            if (out_f32) out_f32[(size_t)r * H + i] = y;
            if (out_split) write_split(out_split + (size_t)r * 3 * H + i, H, y);
        }
    }
}

// The same norm with four elements a thread and load: the form for rows of a multiple of four
// elements (16-byte loads of the row, the weight and the partial sums; 8- or 16-byte stores).
// V = 16-byte units a thread holds in registers.
template <typename TO> __device__ __forceinline__ void store4(TO* dst, float4 y);
template <> __device__ __forceinline__ void store4<float>(float* dst, float4 y) { *(float4*)dst = y; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float4 y) {
    __nv_bfloat162 a = __floats2bfloat162_rn(y.x, y.y), b = __floats2bfloat162_rn(y.z, y.w);
    uint2 u;
    u.x = *(uint32_t*)&a;
    u.y = *(uint32_t*)&b;
    *(uint2*)dst = u;
}

__device__ __forceinline__ void write_split4(__nv_bfloat16* dst, int H, float4 y) {
    float4 hi = make_float4(__bfloat162float(__float2bfloat16_rn(y.x)), __bfloat162float(__float2bfloat16_rn(y.y)),
                            __bfloat162float(__float2bfloat16_rn(y.z)), __bfloat162float(__float2bfloat16_rn(y.w)));
    float4 r1 = make_float4(y.x - hi.x, y.y - hi.y, y.z - hi.z, y.w - hi.w);
    float4 mid = make_float4(__bfloat162float(__float2bfloat16_rn(r1.x)), __bfloat162float(__float2bfloat16_rn(r1.y)),
                             __bfloat162float(__float2bfloat16_rn(r1.z)), __bfloat162float(__float2bfloat16_rn(r1.w)));
    float4 lo = make_float4(r1.x - mid.x, r1.y - mid.y, r1.z - mid.z, r1.w - mid.w);
    store4<__nv_bfloat16>(dst, hi);             // the store's rounding leaves hi and mid as they are and rounds lo
    store4<__nv_bfloat16>(dst + H, mid);
    store4<__nv_bfloat16>(dst + 2 * H, lo);
}

template <typename TO, int V>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ w, float eps, int H,
                                   TO* __restrict__ out, float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_split,
                                   const int* __restrict__ row_index, const float* __restrict__ partials, int n_partials,
                                   long long partial_stride) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float partial[32];
    __shared__ float scale_s;
    const int r = blockIdx.x, n4 = H >> 2;
    float4* src = (float4*)(x + (size_t)(row_index ? row_index[r] : r) * H);
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 xv[V], wv[V];
#pragma unroll
    for (int q = 0; q < V; ++q) {
        int u = threadIdx.x + q * blockDim.x;
        xv[q] = u < n4 ? src[u] : zero;
        wv[q] = u < n4 ? ((const float4*)w)[u] : zero;
    }
    if (partials) {
        // the split sums of the product before this norm: added in split order, stored back
        for (int s = 0; s < n_partials; ++s)
#pragma unroll
            for (int q = 0; q < V; ++q) {
                int u = threadIdx.x + q * blockDim.x;
                if (u < n4) {
                    float4 p4 = ((const float4*)(partials + s * partial_stride + (size_t)r * H))[u];
                    xv[q].x += p4.x; xv[q].y += p4.y; xv[q].z += p4.z; xv[q].w += p4.w;
                }
            }
#pragma unroll
        for (int q = 0; q < V; ++q) {
            int u = threadIdx.x + q * blockDim.x;
            if (u < n4) src[u] = xv[q];
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int q = 0; q < V; ++q) {
        ss = fmaf(xv[q].x, xv[q].x, ss);
        ss = fmaf(xv[q].y, xv[q].y, ss);
        ss = fmaf(xv[q].z, xv[q].z, ss);
        ss = fmaf(xv[q].w, xv[q].w, ss);
    }
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lane == 0) partial[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < nwarps ? partial[lane] : 0.0f;
        v = warp_sum(v);
        if (lane == 0) scale_s = 1.0f / sqrtf(v / (float)H + eps);
    }
    __syncthreads();
    const float scale = scale_s;
#pragma unroll
    for (int q = 0; q < V; ++q) {
        int u = threadIdx.x + q * blockDim.x;
        if (u < n4) {
            float4 y = make_float4(xv[q].x * scale * wv[q].x, xv[q].y * scale * wv[q].y, xv[q].z * scale * wv[q].z,
                                   xv[q].w * scale * wv[q].w);
            store4<TO>(out + (size_t)r * H + 4 * u, y);
            if (out_f32) *(float4*)(out_f32 + (size_t)r * H + 4 * u) = y;
            if (out_split) write_split4(out_split + (size_t)r * 3 * H + 4 * u, H, y);
        }
    }
}

// The same norm by a quarter of the threads, for steps of many rows: a thread stands for the four
// threads of the kernel above whose numbers differ by 128 (their pieces, their sums, their warps'
// butterflies, then the same butterfly over the warps' sums), so a row has the same bits from either
// kernel; what changes is that a thread has four times the loads under way and an SM four times the
// rows, which is what a step of thousands of rows - wave after wave of blocks that each wait for
// one round trip to memory - is bound by.
template <typename TO, int V>
__global__ void __launch_bounds__(128) rmsnorm_vec4_kernel(float* __restrict__ x, const float* __restrict__ w, float eps, int H,
                                                           TO* __restrict__ out, float* __restrict__ out_f32,
                                                           __nv_bfloat16* __restrict__ out_split, const float* __restrict__ partials,
                                                           int n_partials, long long partial_stride) {
    cj::after_predecessor();
    cj::release_successor();
    constexpr int Q = 4, THREADS = 512;                    // the kernel above runs 512 threads when this one is chosen
    __shared__ float partial[32];
    __shared__ float scale_s;
    const int r = blockIdx.x, n4 = H >> 2;
    float4* src = (float4*)(x + (size_t)r * H);
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 xv[Q][V];
#pragma unroll
    for (int e = 0; e < Q; ++e)
#pragma unroll
        for (int q = 0; q < V; ++q) {
            int u = threadIdx.x + e * 128 + q * THREADS;
            xv[e][q] = u < n4 ? src[u] : zero;
        }
    if (partials) {
        for (int s = 0; s < n_partials; ++s)
#pragma unroll
            for (int e = 0; e < Q; ++e)
#pragma unroll
                for (int q = 0; q < V; ++q) {
                    int u = threadIdx.x + e * 128 + q * THREADS;
                    if (u < n4) {
                        float4 p4 = ((const float4*)(partials + s * partial_stride + (size_t)r * H))[u];
                        xv[e][q].x += p4.x; xv[e][q].y += p4.y; xv[e][q].z += p4.z; xv[e][q].w += p4.w;
                    }
                }
#pragma unroll
        for (int e = 0; e < Q; ++e)
#pragma unroll
            for (int q = 0; q < V; ++q) {
                int u = threadIdx.x + e * 128 + q * THREADS;
                if (u < n4) src[u] = xv[e][q];
            }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int e = 0; e < Q; ++e) {
        float ss = 0.0f;
#pragma unroll
        for (int q = 0; q < V; ++q) {
            ss = fmaf(xv[e][q].x, xv[e][q].x, ss);
            ss = fmaf(xv[e][q].y, xv[e][q].y, ss);
            ss = fmaf(xv[e][q].z, xv[e][q].z, ss);
            ss = fmaf(xv[e][q].w, xv[e][q].w, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) partial[warp + 4 * e] = ss;          // the warp of the threads this thread stands for
    }
    __syncthreads();
    if (warp == 0) {
        float v = lane < THREADS / 32 ? partial[lane] : 0.0f;
        v = warp_sum(v);
        if (lane == 0) scale_s = 1.0f / sqrtf(v / (float)H + eps);
    }
    __syncthreads();
    const float scale = scale_s;
#pragma unroll
    for (int e = 0; e < Q; ++e)
#pragma unroll
        for (int q = 0; q < V; ++q) {
            int u = threadIdx.x + e * 128 + q * THREADS;
            if (u < n4) {
                const float4 wv = ((const float4*)w)[u];
                float4 y = make_float4(xv[e][q].x * scale * wv.x, xv[e][q].y * scale * wv.y, xv[e][q].z * scale * wv.z,
                                       xv[e][q].w * scale * wv.w);
                store4<TO>(out + (size_t)r * H + 4 * u, y);
                if (out_f32) *(float4*)(out_f32 + (size_t)r * H + 4 * u) = y;
                if (out_split) write_split4(out_split + (size_t)r * 3 * H + 4 * u, H, y);
            }
        }
}

// partials (optional): [n_partials][rows][H] float32 with partial_stride elements between
// them; x[r] += sum of its partials first (the residual add of a product that was split
// along K), and x keeps the sum.  Not combined with row_index.  out_split (optional):
// bfloat16 [rows, 3H], the three-term form of the float32 result.
// rows from which on the norm runs with a quarter of the threads (measured at rows of 2,048: two norms a layer
// 27.6 -> 24.9 us at 2,048 rows, 90.6 -> 60.6 us at 8,192; a few rows are one round trip either way)
constexpr int NORM_QUARTER_MIN_ROWS = 256;

CJ_EXPORT int cj_rmsnorm(float* x, const float* w, float eps, int rows, int H, void* out, int out_dtype,
                         float* out_f32, void* out_split, const int* row_index, const float* partials, int n_partials,
                         long long partial_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!x || !w || !out || H <= 0) return CJ_ERR_ARG;
    if (partials && (row_index || n_partials < 1)) return CJ_ERR_ARG;
    // rows of a multiple of four elements, every pointer on a 16-byte boundary: four elements a load
    const bool aligned = ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out) | ((uintptr_t)out_f32) | ((uintptr_t)out_split)
                           | ((uintptr_t)partials)) & 15) == 0;
    if (H % 4 == 0 && H <= 8192 && aligned && (!partials || partial_stride % 4 == 0)) {
        const int n4 = H / 4;
        int vthreads = n4 >= 512 ? 512 : ((n4 + 31) / 32) * 32;
        int v = (n4 + vthreads - 1) / vthreads;
        if (vthreads == 512 && rows >= NORM_QUARTER_MIN_ROWS && !row_index && v <= 2) {
#define LAUNCHQ(TO, V) cj::launch(rmsnorm_vec4_kernel<TO, V>, dim3(rows), dim3(128), 0, stream, x, w, eps, H, (TO*)out, out_f32, (__nv_bfloat16*)out_split, partials, n_partials, partial_stride)
            if (out_dtype == CJ_F32) { if (v <= 1) LAUNCHQ(float, 1); else LAUNCHQ(float, 2); }
            else if (out_dtype == CJ_BF16) { if (v <= 1) LAUNCHQ(__nv_bfloat16, 1); else LAUNCHQ(__nv_bfloat16, 2); }
            else return CJ_ERR_DTYPE;
#undef LAUNCHQ
            return launch_status();
        }
#define LAUNCHV(TO, V) cj::launch(rmsnorm_vec_kernel<TO, V>, dim3(rows), dim3(vthreads), 0, stream, x, w, eps, H, (TO*)out, out_f32, (__nv_bfloat16*)out_split, row_index, partials, n_partials, partial_stride)
#define PICKV(TO)                                  \
    if (v <= 1) LAUNCHV(TO, 1);                    \
    else if (v <= 2) LAUNCHV(TO, 2);               \
    else LAUNCHV(TO, 4)
        if (out_dtype == CJ_F32) { PICKV(float); }
        else if (out_dtype == CJ_BF16) { PICKV(__nv_bfloat16); }
        else return CJ_ERR_DTYPE;
#undef PICKV
#undef LAUNCHV
        return launch_status();
    }
    int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    int per = (H + threads - 1) / threads;
#define LAUNCH(TO, PER) cj::launch(rmsnorm_kernel<TO, PER>, dim3(rows), dim3(threads), 0, stream, x, w, eps, H, (TO*)out, out_f32, (__nv_bfloat16*)out_split, row_index, partials, n_partials, partial_stride)
#define PICK(TO)                                   \
    if (per <= 4) LAUNCH(TO, 4);                   \
    else if (per <= 8) LAUNCH(TO, 8);              \
    else LAUNCH(TO, 0)
    if (out_dtype == CJ_F32) { PICK(float); }
    else if (out_dtype == CJ_BF16) { PICK(__nv_bfloat16); }
    else return CJ_ERR_DTYPE;
#undef PICK
#undef LAUNCH
    return launch_status();
}

// ---------------------------------------------------------------------------------
// Rotary encoding of q and k at each row's absolute position, fused with the write of
// the rotated k and the raw v into the cache pages of the row's request.
// Half-split pairs (d, d + rot/2): ang = float(p) * inv[d]; a' = a cos - b sin;
// b' = a sin + b cos (model/Prim.cajeta:1917-1940); dims >= rotary_dim pass through.
// reference kernels: model/AttnKernel.cajeta:128 (qkPrep), :554 (ropeAppendRows).
//
// qkv is float32 [T, ld] with q at column q_off (n_heads*hd wide), k at k_off and v at
// v_off (n_kv*hd wide each).  q_out is [T, n_heads, hd] in the activation dtype.  A
// cache plane is [pages, n_kv, page_tokens, hd]; position p of request r lies in page
// table[r * table_stride + p / page_tokens] at slot p % page_tokens.
// ---------------------------------------------------------------------------------
template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; static __device__ __forceinline__ float2 make(float a, float b) { return make_float2(a, b); } };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; static __device__ __forceinline__ __nv_bfloat162 make(float a, float b) { return __floats2bfloat162_rn(a, b); } };

// One block per row.  The row's angles are computed once (they are the same for every
// head) and kept in shared memory; then each thread takes units of two adjacent dims:
// for q and k a unit is dims (d, d+1) and their partners (d + half, d + half + 1).
template <typename TQ, typename TC>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off,
                                     TQ* __restrict__ q_out, TC* __restrict__ kplane, TC* __restrict__ vplane,
                                     const int* __restrict__ positions, const int* __restrict__ row_req,
                                     const int* __restrict__ table, int table_stride, int page_tokens,
                                     int n_heads, int n_kv, int hd, int rot, const float* __restrict__ inv_freq,
                                     int write_kv) {
    cj::release_successor();
    extern __shared__ __align__(16) float cs[];   // cos[half] then sin[half]
    const int t = blockIdx.x;
    // with few rows the units of a row are shared out over gridDim.y blocks
    const int part = blockIdx.y, parts = gridDim.y;
    // The step's positions and page tables were written before the step's first kernel, not by the
    // kernel before this one: the angles and the page's address are worked out while that kernel
    // drains.  (Read past L1: the buffers are the same from step to step.)
    const int pos = __ldcg(positions + t);
    const float* row = qkv + (size_t)t * ld;
    const int half = rot >> 1;
    for (int d = threadIdx.x; d < half; d += blockDim.x) {
        float ang = (float)pos * inv_freq[d];
        cs[d] = cosf(ang);
        cs[half + d] = sinf(ang);
    }
    size_t kv_base = 0;
    bool have_page = false;
    if (write_kv) {
        int page = __ldcg(table + (size_t)__ldcg(row_req + t) * table_stride + pos / page_tokens);
        have_page = page >= 0;                     // no page: the host never schedules this
        kv_base = ((size_t)(have_page ? page : 0) * n_kv) * page_tokens * hd + (size_t)(pos % page_tokens) * hd;
    }
    cj::after_predecessor();
    __syncthreads();
    // head sizes and rotary parts of a multiple of eight, rows on 16-byte boundaries: units of four dims
    const bool quad = (hd % 4 == 0) && (half % 4 == 0) && ((ld | q_off | k_off | v_off) % 4 == 0) &&
                      ((((uintptr_t)qkv) | ((uintptr_t)q_out) | ((uintptr_t)kplane) | ((uintptr_t)vplane)) & 15) == 0;
    if (quad) {
        const int units_per_slot = half / 4;
        const int rot_slots = n_heads + (write_kv && have_page ? n_kv : 0);
        for (int u = part * blockDim.x + threadIdx.x; u < rot_slots * units_per_slot; u += parts * blockDim.x) {
            int slot = u / units_per_slot, d = (u % units_per_slot) * 4;
            bool is_q = slot < n_heads;
            const float* src = is_q ? row + q_off + slot * hd : row + k_off + (slot - n_heads) * hd;
            float4 a = *(const float4*)(src + d), b = *(const float4*)(src + d + half);
            float4 c = *(const float4*)(cs + d), sn = *(const float4*)(cs + half + d);
            float4 lo = make_float4(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w);
            float4 hi = make_float4(a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y, a.z * sn.z + b.z * c.z, a.w * sn.w + b.w * c.w);
            if (is_q) {
                TQ* dst = q_out + ((size_t)t * n_heads + slot) * hd;
                store4<TQ>(dst + d, lo);
                store4<TQ>(dst + d + half, hi);
            } else {
                TC* dst = kplane + kv_base + (size_t)(slot - n_heads) * page_tokens * hd;
                store4<TC>(dst + d, lo);
                store4<TC>(dst + d + half, hi);
            }
        }
        const int tail = hd - rot;                 // dims past the rotary part pass through
        if (tail > 0) {
            for (int u = part * blockDim.x + threadIdx.x; u < rot_slots * (tail / 4); u += parts * blockDim.x) {
                int slot = u / (tail / 4), d = rot + (u % (tail / 4)) * 4;
                bool is_q = slot < n_heads;
                const float* src = is_q ? row + q_off + slot * hd : row + k_off + (slot - n_heads) * hd;
                float4 a = *(const float4*)(src + d);
                if (is_q) store4<TQ>(q_out + ((size_t)t * n_heads + slot) * hd + d, a);
                else store4<TC>(kplane + kv_base + (size_t)(slot - n_heads) * page_tokens * hd + d, a);
            }
        }
        if (write_kv && have_page) {
            for (int u = part * blockDim.x + threadIdx.x; u < n_kv * (hd / 4); u += parts * blockDim.x) {
                int kh = u / (hd / 4), d = (u % (hd / 4)) * 4;
                store4<TC>(vplane + kv_base + (size_t)kh * page_tokens * hd + d, *(const float4*)(row + v_off + kh * hd + d));
            }
        }
        return;
    }
    const bool even = (hd % 2 == 0) && (half % 2 == 0);
    if (even) {
        // rotated part of q and k: units of (head slot, dim pair below half)
        const int units_per_slot = half / 2;
        const int rot_slots = n_heads + (write_kv && have_page ? n_kv : 0);
        for (int u = part * blockDim.x + threadIdx.x; u < rot_slots * units_per_slot; u += parts * blockDim.x) {
            int slot = u / units_per_slot, d = (u % units_per_slot) * 2;
            bool is_q = slot < n_heads;
            const float* src = is_q ? row + q_off + slot * hd : row + k_off + (slot - n_heads) * hd;
            float2 a = *(const float2*)(src + d), b = *(const float2*)(src + d + half);
            float c0 = cs[d], c1 = cs[d + 1], s0 = cs[half + d], s1 = cs[half + d + 1];
            float lo0 = a.x * c0 - b.x * s0, lo1 = a.y * c1 - b.y * s1;
            float hi0 = a.x * s0 + b.x * c0, hi1 = a.y * s1 + b.y * c1;
            if (is_q) {
                TQ* dst = q_out + ((size_t)t * n_heads + slot) * hd;
                *(typename Pair<TQ>::type*)(dst + d) = Pair<TQ>::make(lo0, lo1);
                *(typename Pair<TQ>::type*)(dst + d + half) = Pair<TQ>::make(hi0, hi1);
            } else {
                TC* dst = kplane + kv_base + (size_t)(slot - n_heads) * page_tokens * hd;
                *(typename Pair<TC>::type*)(dst + d) = Pair<TC>::make(lo0, lo1);
                *(typename Pair<TC>::type*)(dst + d + half) = Pair<TC>::make(hi0, hi1);
            }
        }
        // dims past the rotary part of q and k pass through; v is copied whole
        const int tail = hd - rot;
        if (tail > 0) {
            for (int u = part * blockDim.x + threadIdx.x; u < rot_slots * (tail / 2); u += parts * blockDim.x) {
                int slot = u / (tail / 2), d = rot + (u % (tail / 2)) * 2;
                bool is_q = slot < n_heads;
                const float* src = is_q ? row + q_off + slot * hd : row + k_off + (slot - n_heads) * hd;
                float2 a = *(const float2*)(src + d);
                if (is_q) *(typename Pair<TQ>::type*)(q_out + ((size_t)t * n_heads + slot) * hd + d) = Pair<TQ>::make(a.x, a.y);
                else *(typename Pair<TC>::type*)(kplane + kv_base + (size_t)(slot - n_heads) * page_tokens * hd + d) = Pair<TC>::make(a.x, a.y);
            }
        }
        if (write_kv && have_page) {
            for (int u = part * blockDim.x + threadIdx.x; u < n_kv * (hd / 2); u += parts * blockDim.x) {
                int kh = u / (hd / 2), d = (u % (hd / 2)) * 2;
                float2 a = *(const float2*)(row + v_off + kh * hd + d);
                *(typename Pair<TC>::type*)(vplane + kv_base + (size_t)kh * page_tokens * hd + d) = Pair<TC>::make(a.x, a.y);
            }
        }
        return;
    }
    // general sizes: one element at a time
    const int slots = n_heads + (write_kv && have_page ? 2 * n_kv : 0);
    for (int e = part * blockDim.x + threadIdx.x; e < slots * hd; e += parts * blockDim.x) {
        int slot = e / hd, d = e % hd;
        if (slot < n_heads + n_kv) {
            bool is_q = slot < n_heads;
            const float* src = is_q ? row + q_off + slot * hd : row + k_off + (slot - n_heads) * hd;
            float v;
            if (d < rot) {
                int dd = d < half ? d : d - half;
                float a = src[dd], b = src[dd + half];
                v = d < half ? a * cs[dd] - b * cs[half + dd] : a * cs[half + dd] + b * cs[dd];
            } else {
                v = src[d];
            }
            if (is_q) q_out[((size_t)t * n_heads + slot) * hd + d] = from_f32<TQ>(v);
            else kplane[kv_base + (size_t)(slot - n_heads) * page_tokens * hd + d] = from_f32<TC>(v);
        } else {
            int kh = slot - n_heads - n_kv;
            vplane[kv_base + (size_t)kh * page_tokens * hd + d] = from_f32<TC>(row[v_off + kh * hd + d]);
        }
    }
}

CJ_EXPORT int cj_rope_kv_write(const float* qkv, int ld, int q_off, int k_off, int v_off, void* q_out, int q_dtype,
                               void* kplane, void* vplane, int cache_dtype, const int* positions,
                               const int* row_req, const int* table, int table_stride, int page_tokens, int T,
                               int n_heads, int n_kv, int hd, int rotary_dim, const float* inv_freq, int write_kv,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!qkv || !q_out || !positions || n_heads <= 0 || hd <= 0) return CJ_ERR_ARG;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return CJ_ERR_SIZE;
    if (rotary_dim > 0 && !inv_freq) return CJ_ERR_ARG;
    if (write_kv && (!kplane || !vplane || !row_req || !table || page_tokens <= 0 || n_kv <= 0)) return CJ_ERR_ARG;
    // the paired fast path reads float2: row stride and offsets must keep 8-byte alignment
    if ((ld | q_off | k_off | v_off) & 1) return CJ_ERR_ALIGN;
    int work = (n_heads + (write_kv ? 2 * n_kv : 0)) * hd / 2;
    int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
    // many rows: half the threads a row, twice the rows an SM (measured at 48 head slots of 128: 20.5 -> 19.1 us
    // at 2,048 rows, 68.8 -> 61.4 us at 8,192; 64 threads 19.7 / 64.7, 512 threads 24.6 / 84.7)
    if (T >= 256 && threads > 128) threads = 128;
    size_t smem = (size_t)rotary_dim * sizeof(float);
    int parts = T >= 128 ? 1 : (work + threads * 2 - 1) / (threads * 2);      // few rows: ~2 units a thread
    if (parts < 1) parts = 1;
    if (parts > 16) parts = 16;
    dim3 grid(T, parts);
#define LAUNCH(TQ, TC)                                                                                          \
    cj::launch(rope_kv_write_kernel<TQ, TC>, dim3(grid), dim3(threads), smem, stream, qkv, ld, q_off, k_off, v_off, (TQ*)q_out,     \
        (TC*)kplane, (TC*)vplane, positions, row_req, table, table_stride, page_tokens, n_heads, n_kv, hd,      \
        rotary_dim, inv_freq, write_kv)
    if (q_dtype == CJ_F32 && cache_dtype == CJ_F32) LAUNCH(float, float);
    else if (q_dtype == CJ_BF16 && cache_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}

// ---------------------------------------------------------------------------------
// Combine of the mixture's outputs into the residual stream, per token and in a fixed
// order: acc = sum_j w[t,j] * y[slot(t,j)] for j = 0..k-1 (selection order), then the
// shared expert: acc += gate[t] * sum_c shared[c][t] over its `chunks` partial results in
// chunk order (one chunk when it was computed whole); hs[t] += acc.  No atomics: one
// thread owns an element.
// reference: model/MoeFfn.cajeta:1849-1916 (row form), combine kernel
// io/QuantKernel.cajeta:40747; shared expert model/Prim.cajeta:1652-1664.
// ---------------------------------------------------------------------------------
// KT > 0: k is KT and the picks' loads are written out, so that a thread has all its indices
// under way at once and then all its rows (a loop over a run-time k waits for each in turn:
// ten round trips to memory instead of three).  The sums keep their order either way.
template <int VEC, int KT>
__global__ void moe_combine_kernel(float* __restrict__ hs, const float* __restrict__ y, const int* __restrict__ slot_of_pick,
                                   const float* __restrict__ w, int k, const float* __restrict__ shared, int chunks,
                                   long long chunk_stride, const float* __restrict__ shared_scale, int H) {
    cj::after_predecessor();
    cj::release_successor();
    int t = blockIdx.x;
    int i = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (i >= H) return;
    constexpr int CH = 4;                       // chunks of the shared expert whose loads are written out
    float acc[VEC], sh[VEC], res[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = sh[v] = 0.0f;
    float* dst = hs + (size_t)t * H + i;
    if (KT > 0) {
        int slot[KT > 0 ? KT : 1];
        float wj[KT > 0 ? KT : 1], row[KT > 0 ? KT : 1][VEC], part[CH][VEC];
#pragma unroll
        for (int j = 0; j < KT; ++j) {
            slot[j] = slot_of_pick[t * KT + j];
            wj[j] = w[t * KT + j];
        }
        const float g = (shared && shared_scale) ? shared_scale[t] : 1.0f;
        if (VEC == 4) *(float4*)res = *(const float4*)dst; else res[0] = dst[0];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            if (shared && c < chunks) {
                const float* src = shared + c * chunk_stride + (size_t)t * H + i;
                if (VEC == 4) *(float4*)part[c] = *(const float4*)src; else part[c][0] = src[0];
            }
        }
#pragma unroll
        for (int j = 0; j < KT; ++j) {
            const float* src = y + (size_t)slot[j] * H + i;
            if (VEC == 4) *(float4*)row[j] = *(const float4*)src; else row[j][0] = src[0];
        }
#pragma unroll
        for (int j = 0; j < KT; ++j)
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] += wj[j] * row[j][v];
        if (shared) {
#pragma unroll
            for (int c = 0; c < CH; ++c)
                if (c < chunks)
#pragma unroll
                    for (int v = 0; v < VEC; ++v) sh[v] += part[c][v];
            for (int c = CH; c < chunks; ++c) {
                const float* src = shared + c * chunk_stride + (size_t)t * H + i;
#pragma unroll
                for (int v = 0; v < VEC; ++v) sh[v] += src[v];
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] += g * sh[v];
        }
    } else {
        for (int j = 0; j < k; ++j) {
            int s = slot_of_pick[t * k + j];
            float wj = w[t * k + j];
            const float* src = y + (size_t)s * H + i;
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] += wj * src[v];
        }
        if (shared) {
            for (int c = 0; c < chunks; ++c) {
                const float* src = shared + c * chunk_stride + (size_t)t * H + i;
#pragma unroll
                for (int v = 0; v < VEC; ++v) sh[v] += src[v];
            }
            float g = shared_scale ? shared_scale[t] : 1.0f;
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] += g * sh[v];
        }
        if (VEC == 4) *(float4*)res = *(const float4*)dst; else res[0] = dst[0];
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) res[v] += acc[v];
    if (VEC == 4) *(float4*)dst = *(float4*)res; else dst[0] = res[0];
}

constexpr int COMBINE_UNROLLED_MAX_ROWS = 256;

CJ_EXPORT int cj_moe_combine(float* hs, const float* y, const int* slot_of_pick, const float* w, int k,
                             const float* shared, int chunks, long long chunk_stride, const float* shared_scale, int T,
                             int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!hs || H <= 0 || k < 0 || (k > 0 && (!y || !slot_of_pick || !w))) return CJ_ERR_ARG;
    if (shared && chunks < 1) return CJ_ERR_ARG;
    bool vec = H % 4 == 0 && chunk_stride % 4 == 0 && ((((uintptr_t)hs) | ((uintptr_t)y) | ((uintptr_t)shared)) & 15) == 0;
    int per = vec ? 4 : 1;
    int threads = H / per >= 256 ? 256 : 128;
    dim3 grid(T, (H / per + threads - 1) / threads + (H % per ? 1 : 0));
    if (grid.y > 65535) return CJ_ERR_SIZE;
#define LAUNCH(V, KT) cj::launch(moe_combine_kernel<V, KT>, dim3(grid), dim3(threads), 0, stream, hs, y, slot_of_pick, w, k, shared, chunks, chunk_stride, shared_scale, H)
    // few rows wait on latency and take the written-out form; many rows are bound by bytes, and there the
    // loop's smaller register file (more blocks an SM) measured faster
    if (vec) {
        switch (T <= COMBINE_UNROLLED_MAX_ROWS ? k : 0) {
            case 2: LAUNCH(4, 2); break;
            case 4: LAUNCH(4, 4); break;
            case 6: LAUNCH(4, 6); break;
            case 8: LAUNCH(4, 8); break;
            default: LAUNCH(4, 0);
        }
    } else {
        LAUNCH(1, 0);
    }
#undef LAUNCH
    return launch_status();
}

// ---------------------------------------------------------------------------------
// Row gather: out[s, :] = x[index[s], :] (bf16 or f32 rows).  Puts the rows of a mixture
// of experts into expert order so that each expert reads a contiguous block
// (model/MoeFfn.cajeta:2644-2777 gathers rows per expert the same way).
// ---------------------------------------------------------------------------------
// a warp a row, eight rows a block: a lane has up to eight 16-byte loads of its row in flight at once
__global__ void gather_rows16_kernel(uint4* __restrict__ out, const uint4* __restrict__ x, const int* __restrict__ index,
                                     int rows, int n16) {
    cj::after_predecessor();
    cj::release_successor();
    const int lane = threadIdx.x & 31, s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (s >= rows) return;
    const uint4* src = x + (size_t)index[s] * n16;
    uint4* dst = out + (size_t)s * n16;
    for (int i0 = lane; i0 < n16; i0 += 32 * 8) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (i0 + 32 * j < n16) v[j] = src[i0 + 32 * j];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (i0 + 32 * j < n16) dst[i0 + 32 * j] = v[j];
    }
}

template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ index, int H) {
    cj::after_predecessor();
    cj::release_successor();
    int s = blockIdx.x;
    const T* src = x + (size_t)index[s] * H;
    T* dst = out + (size_t)s * H;
    if ((H * sizeof(T)) % 16 == 0) {
        const uint4* s4 = (const uint4*)src;
        uint4* d4 = (uint4*)dst;
        int n = H * sizeof(T) / 16;
        for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    }
}

CJ_EXPORT int cj_gather_rows(void* out, const void* x, int dtype, const int* index, int rows, int H, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!out || !x || !index || H <= 0) return CJ_ERR_ARG;
    if (dtype != CJ_F32 && dtype != CJ_BF16) return CJ_ERR_DTYPE;
    const size_t row_bytes = (size_t)H * (dtype == CJ_F32 ? 4 : 2);
    if (rows >= 64 && row_bytes % 16 == 0 && ((((uintptr_t)out) | ((uintptr_t)x)) & 15) == 0) {
        cj::launch(gather_rows16_kernel, dim3((rows + 7) / 8), dim3(256), 0, stream, (uint4*)out, (const uint4*)x, index, rows,
                   (int)(row_bytes / 16));
        return launch_status();
    }
    int threads = H >= 1024 ? 256 : 128;
    if (dtype == CJ_F32) cj::launch(gather_rows_kernel<float>, dim3(rows), dim3(threads), 0, stream, (float*)out, (const float*)x, index, H);
    else if (dtype == CJ_BF16) cj::launch(gather_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, index, H);
    else return CJ_ERR_DTYPE;
    return launch_status();
}
