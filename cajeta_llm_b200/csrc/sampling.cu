// Sampling over float32 logits rows: first-occurrence argmax, and the reference's
// sampler order (gen/Sampler.cajeta:60-206): repetition penalty over emitted tokens,
// temperature, descending order, top-k cut, max-subtracted softmax over the cut, top-p
// smallest prefix with cum >= p, renormalise, one uniform draw u walked down the
// descending order.
//
// Nothing is sorted.  After e_i = exp(z_i - max z) every step is a threshold on e:
// "the k largest", "the smallest prefix of the descending order whose mass reaches P"
// and "the first element of the descending order whose cumulative mass exceeds u" are
// each the largest threshold tau for which a count or a sum over {e_i >= tau} satisfies
// a monotone condition, found bit by bit over the float's 31 magnitude bits (one pass
// over the row per bit).  Elements equal to the threshold are taken in ascending id
// order, which is this engine's deterministic tie order.
//
// One block per row.  scratch is [rows, V] float32 of global memory owned by the
// caller; on return it holds the row's e-values with every filtered token at zero
// (normalising them gives the post-filter distribution the reference's `prepare`
// exposes to tests).
#include "common.cuh"
#include "sampling_static.h"

using namespace cj;

namespace {

constexpr int ST = 1024;

struct BlockShared {
    float fsum[32];
    int isum[32];
    float fval;
    int ival;
    int ival2;
};

__device__ __forceinline__ void block_sum2(float& s, int& c, BlockShared& sh) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    s = warp_sum(s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    __syncthreads();                       // earlier readers of sh are done
    if (lane == 0) { sh.fsum[warp] = s; sh.isum[warp] = c; }
    __syncthreads();
    if (warp == 0) {
        float a = sh.fsum[lane];
        int b = sh.isum[lane];
        a = warp_sum(a);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
        if (lane == 0) { sh.fval = a; sh.ival = b; }
    }
    __syncthreads();
    s = sh.fval;
    c = sh.ival;
}

// sum and count of the elements whose bit pattern is >= tau (e >= 0, so the unsigned
// order of the bits is the order of the values)
__device__ __forceinline__ void pass_ge(const float* e, int V, unsigned tau, float& sum, int& cnt, BlockShared& sh) {
    float s = 0.0f;
    int c = 0;
    for (int i = threadIdx.x; i < V; i += ST) {
        float v = e[i];
        if (__float_as_uint(v) >= tau) { s += v; c += 1; }
    }
    block_sum2(s, c, sh);
    sum = s;
    cnt = c;
}

// exclusive scan of one int per thread over the block, in thread order
__device__ __forceinline__ int block_excl_scan(int v, BlockShared& sh) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) sh.isum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = sh.isum[lane];
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        sh.isum[lane] = winc - w;
    }
    __syncthreads();
    return sh.isum[warp] + inc - v;
}

// zero every element below tau, and every element equal to tau beyond the first `keep`
// of them in ascending id order
__device__ void cut_below(float* e, int V, unsigned tau, int keep, BlockShared& sh) {
    int chunk = (V + ST - 1) / ST;
    int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
    int ties = 0;
    for (int i = lo; i < hi; ++i) ties += __float_as_uint(e[i]) == tau ? 1 : 0;
    int rank = block_excl_scan(ties, sh);
    for (int i = lo; i < hi; ++i) {
        unsigned b = __float_as_uint(e[i]);
        if (b < tau) e[i] = 0.0f;
        else if (b == tau) {
            if (rank >= keep) e[i] = 0.0f;
            rank += 1;
        }
    }
    __syncthreads();
}

// id of the n-th (1-based) element equal to tau in ascending id order, -1 if fewer
__device__ int nth_equal(const float* e, int V, unsigned tau, int n, BlockShared& sh) {
    int chunk = (V + ST - 1) / ST;
    int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
    int ties = 0;
    for (int i = lo; i < hi; ++i) ties += __float_as_uint(e[i]) == tau ? 1 : 0;
    int rank = block_excl_scan(ties, sh);
    if (threadIdx.x == 0) sh.ival2 = -1;
    __syncthreads();
    if (rank < n && n <= rank + ties) {
        for (int i = lo; i < hi; ++i)
            if (__float_as_uint(e[i]) == tau) {
                rank += 1;
                if (rank == n) { sh.ival2 = i; break; }
            }
    }
    __syncthreads();
    return sh.ival2;
}

// largest tau in [1, 0x7f800000] for which pred(sum_ge, count_ge) holds; 0 if none
template <typename Pred>
__device__ unsigned search_threshold(const float* e, int V, Pred pred, BlockShared& sh) {
    unsigned tau = 0;
    for (int bit = 30; bit >= 0; --bit) {
        unsigned cand = tau | (1u << bit);
        if (cand > 0x7f800000u) continue;
        float s;
        int c;
        pass_ge(e, V, cand, s, c, sh);
        if (pred(s, c)) tau = cand;
    }
    return tau;
}

__device__ int block_argmax(const float* v, int V, BlockShared& sh) {
    float bv = -INFINITY;
    int bi = -1;
    for (int i = threadIdx.x; i < V; i += ST) {
        float x = v[i];
        if (bi < 0 || x > bv) { bv = x; bi = i; }      // strict '>': first occurrence
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    __syncthreads();
    if (lane == 0) { sh.fsum[warp] = bv; sh.isum[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = sh.fsum[lane];
        bi = sh.isum[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) sh.ival = bi < 0 ? 0 : bi;
    }
    __syncthreads();
    return sh.ival;
}

__global__ void __launch_bounds__(ST) argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ BlockShared sh;
    int r = blockIdx.x;
    int best = block_argmax(logits + (size_t)r * V, V, sh);
    if (threadIdx.x == 0) out[r] = best;
}

__global__ void __launch_bounds__(ST) sample_kernel(
    const float* __restrict__ logits, int V, const float* __restrict__ temperature, const int* __restrict__ top_k,
    const float* __restrict__ top_p, const float* __restrict__ repeat_penalty, const float* __restrict__ uniform,
    const int* __restrict__ history, const int* __restrict__ history_offsets, float* __restrict__ scratch,
    int* __restrict__ out) {
    __shared__ BlockShared sh;
    int r = blockIdx.x;
    const float* src = logits + (size_t)r * V;
    float* e = scratch + (size_t)r * V;

    for (int i = threadIdx.x; i < V; i += ST) e[i] = src[i];
    __syncthreads();
    float pen = repeat_penalty ? repeat_penalty[r] : 1.0f;
    if (pen != 1.0f && history && threadIdx.x == 0) {
        // one thread, in history order: a token emitted twice is penalised twice, as
        // the reference's loop does
        for (int i = history_offsets[r]; i < history_offsets[r + 1]; ++i) {
            int t = history[i];
            if (t >= 0 && t < V) {
                float lg = e[t];
                e[t] = lg > 0.0f ? lg / pen : lg * pen;
            }
        }
    }
    __syncthreads();

    float temp = temperature[r];
    int best = block_argmax(e, V, sh);
    if (temp == 0.0f) {
        for (int i = threadIdx.x; i < V; i += ST) e[i] = i == best ? 1.0f : 0.0f;
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    float mx = e[best] / temp;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += ST) e[i] = expf(e[i] / temp - mx);
    __syncthreads();

    int k = top_k ? top_k[r] : 0;
    if (k > 0 && k < V) {
        unsigned tau = search_threshold(e, V, [k](float, int c) { return c >= k; }, sh);
        float s;
        int above;
        pass_ge(e, V, tau + 1, s, above, sh);
        // tau == 0: fewer than k positive values; the zeros among the k largest carry
        // no mass, so nothing needs cutting
        if (tau > 0) cut_below(e, V, tau, k - above, sh);
    }

    float tp = top_p ? top_p[r] : 0.0f;
    if (tp > 0.0f && tp < 1.0f) {
        float total;
        int c;
        pass_ge(e, V, 1u, total, c, sh);
        float target = tp * total;
        unsigned tau = search_threshold(e, V, [target](float s, int) { return s >= target; }, sh);
        if (tau > 0) {
            float above;
            int n_above, n_ge;
            float s_ge;
            pass_ge(e, V, tau + 1, above, n_above, sh);
            pass_ge(e, V, tau, s_ge, n_ge, sh);
            float ev = __uint_as_float(tau);
            int keep = (int)ceilf((target - above) / ev);
            keep = max(1, min(keep, n_ge - n_above));
            cut_below(e, V, tau, keep, sh);
        }
    }

    float total2;
    int survivors;
    pass_ge(e, V, 1u, total2, survivors, sh);
    float target = uniform[r] * total2;
    unsigned tau = search_threshold(e, V, [target](float s, int) { return s > target; }, sh);
    int pick;
    if (tau == 0) {
        // float-sum shortfall: the last survivor of the descending order, i.e. the
        // smallest positive value and, among equals, the highest id
        unsigned small = search_threshold(e, V, [survivors](float, int c) { return c >= survivors; }, sh);
        float s;
        int n_ge, n_above;
        pass_ge(e, V, small, s, n_ge, sh);
        pass_ge(e, V, small + 1, s, n_above, sh);
        pick = nth_equal(e, V, small, n_ge - n_above, sh);
    } else {
        float above, s_ge;
        int n_above, n_ge;
        pass_ge(e, V, tau + 1, above, n_above, sh);
        pass_ge(e, V, tau, s_ge, n_ge, sh);
        float ev = __uint_as_float(tau);
        int n = (int)floorf((target - above) / ev) + 1;
        n = max(1, min(n, n_ge - n_above));
        pick = nth_equal(e, V, tau, n, sh);
    }
    if (threadIdx.x == 0) out[r] = pick < 0 ? best : pick;
}

}  // namespace

CJ_EXPORT int cj_argmax(const float* logits, int rows, int V, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!logits || !out || V <= 0) return CJ_ERR_ARG;
    argmax_kernel<<<rows, ST, 0, stream>>>(logits, V, out);
    return launch_status();
}

// Per row r: temperature[r] (0 = greedy), top_k[r] (0 = off), top_p[r] (<= 0 or >= 1 =
// off), repeat_penalty[r] (1 = off) over history[history_offsets[r] .. [r+1]), and the
// uniform draw uniform[r] in [0, 1).  top_k, top_p, repeat_penalty and history may be
// null.  scratch: [rows, V] float32.
CJ_EXPORT int cj_sample(const float* logits, int rows, int V, const float* temperature, const int* top_k,
                        const float* top_p, const float* repeat_penalty, const float* uniform, const int* history,
                        const int* history_offsets, float* scratch, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!logits || !temperature || !uniform || !scratch || !out || V <= 0) return CJ_ERR_ARG;
    if (history && !history_offsets) return CJ_ERR_ARG;
    sample_kernel<<<rows, ST, 0, stream>>>(logits, V, temperature, top_k, top_p, repeat_penalty, uniform, history,
                                           history_offsets, scratch, out);
    return launch_status();
}

// ---------------------------------------------------------------------------------
// The same sampler for callers that cannot allocate (see sampling_static.h): the scratch
// is a fixed array in the library image instead of a buffer from the caller.
//
// In host code the name of a __device__ array is only a stand-in of the host side; it is
// not an address a kernel may use.  The device address is asked for once per device, with
// that device current, and kept.
// ---------------------------------------------------------------------------------
static __device__ __align__(256) float g_sample_static_scratch[CJ_SAMPLE_STATIC_MAX_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {nullptr};
}  // namespace

CJ_EXPORT long long cj_sample_static_capacity(void) { return (long long)CJ_SAMPLE_STATIC_MAX_FLOATS; }

CJ_EXPORT int cj_sample_static(const float* logits, int rows, int V, const float* temperature, const int* top_k,
                               const float* top_p, const float* repeat_penalty, const float* uniform,
                               const int* history, const int* history_offsets, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!logits || !temperature || !uniform || !out || V <= 0) return CJ_ERR_ARG;
    if (history && !history_offsets) return CJ_ERR_ARG;
    if ((long long)rows * (long long)V > (long long)CJ_SAMPLE_STATIC_MAX_FLOATS) return CJ_SAMPLE_STATIC_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return CJ_ERR_ARG;
    if (!g_static_scratch_ptr[dev]) {
        // set-up, first call on this device: the device address of the array
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_sample_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!ptr) return CJ_ERR_ARG;
        g_static_scratch_ptr[dev] = ptr;
    }
    sample_kernel<<<rows, ST, 0, stream>>>(logits, V, temperature, top_k, top_p, repeat_penalty, uniform, history,
                                           history_offsets, g_static_scratch_ptr[dev], out);
    return launch_status();
}
