// Routing of a mixture of experts: router logits, softmax, top-k (fused, one block per
// token) and the counting sort of the picks by expert.  Everything here is float32.
#include "common.cuh"

using namespace cj;

namespace {

constexpr int ROUTER_THREADS = 256;
constexpr int MAX_EXPERTS = 1024;

// l_e = sum_j Wr[e, j] * x_j; softmax over ALL experts; top-k by repeated argmax with a
// strict '>' so that ties go to the lower index; w_k = p_sel; optional renormalisation
// with the divisor clamped at 2^-14 (model/MoeFfn.cajeta:908-988; device twin
// io/QuantKernel.cajeta:40849-40942).  Also the shared expert's gate:
// sigma(sum_j g[j] * x_j) (model/MoeFfn.cajeta:1925-1964).
__global__ void __launch_bounds__(ROUTER_THREADS) router_topk_kernel(
    const float* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ shared_gate, int H, int E,
    int k, int norm_topk, int* __restrict__ sel, float* __restrict__ w, float* __restrict__ shared_scale) {
    __shared__ float probs[MAX_EXPERTS];
    int t = blockIdx.x;
    const float* row = x + (size_t)t * H;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = ROUTER_THREADS / 32;

    for (int e = warp; e < E + (shared_gate ? 1 : 0); e += NW) {
        const float* wr = e < E ? Wr + (size_t)e * H : shared_gate;
        float dot = 0.0f;
        for (int j = lane; j < H; j += 32) dot = fmaf(wr[j], row[j], dot);
        dot = warp_sum(dot);
        if (lane == 0) {
            if (e < E) probs[e] = dot;
            else shared_scale[t] = 1.0f / (1.0f + expf(-dot));
        }
    }
    __syncthreads();
    if (warp != 0) return;

    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, probs[e]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) {
        float p = expf(probs[e] - mx);
        probs[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) probs[e] = probs[e] / sum;
    __syncwarp();

    float wsum = 0.0f;
    for (int j = 0; j < k; ++j) {
        float bp = -1.0f;
        int best = -1;
        for (int e = lane; e < E; e += 32) {
            float p = probs[e];
            if (p >= 0.0f && (best < 0 || p > bp)) { best = e; bp = p; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float op = __shfl_xor_sync(0xffffffffu, bp, o);
            int ob = __shfl_xor_sync(0xffffffffu, best, o);
            bool take = ob >= 0 && (best < 0 || op > bp || (op == bp && ob < best));
            if (take) { bp = op; best = ob; }
        }
        // every probability failed '>= 0': the logits of this row are not finite; the
        // pick falls to expert j with a NaN weight so that the fault shows in the logits
        if (best < 0) { best = j < E ? j : 0; bp = __int_as_float(0x7fc00000); }
        else if (lane == 0) probs[best] = -1.0f;
        if (lane == 0) { sel[t * k + j] = best; w[t * k + j] = bp; }
        wsum += bp;
        __syncwarp();
    }
    if (norm_topk && lane == 0) {
        if (wsum < 0.00006103515625f) wsum = 0.00006103515625f;
        for (int j = 0; j < k; ++j) w[t * k + j] = w[t * k + j] / wsum;
    }
}

// Counting sort of the picks (token t, choice j) by expert, stable.  One warp per
// expert: it counts the picks of lower experts (its first slot) and then places its own
// in pick order.  reference: model/MoeFfn.cajeta:2064-2099 (groupPicks), device
// io/QuantKernel.cajeta:41069.
__global__ void moe_group_kernel(const int* __restrict__ sel, int n, int k, int E, int* __restrict__ offsets,
                                 int* __restrict__ slot_token, int* __restrict__ slot_of_pick) {
    int e = blockIdx.x;
    int lane = threadIdx.x;
    int below = 0;
    for (int i = lane; i < n; i += 32) below += sel[i] < e ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) below += __shfl_xor_sync(0xffffffffu, below, o);
    int cursor = below;
    for (int base = 0; base < n; base += 32) {
        int i = base + lane;
        bool mine = i < n && sel[i] == e;
        unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            int pos = cursor + __popc(ballot & ((1u << lane) - 1u));
            slot_token[pos] = i / k;
            slot_of_pick[i] = pos;
        }
        cursor += __popc(ballot);
    }
    if (lane == 0) {
        offsets[e] = below;
        if (e == E - 1) offsets[E] = cursor;
    }
}

}  // namespace

CJ_EXPORT int cj_router_topk(const float* x, const float* Wr, const float* shared_gate, int T, int H, int E, int k,
                             int norm_topk, int* sel, float* w, float* shared_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!x || !Wr || !sel || !w || H <= 0) return CJ_ERR_ARG;
    if (shared_gate && !shared_scale) return CJ_ERR_ARG;
    if (E < 1 || E > MAX_EXPERTS || k < 1 || k > E) return CJ_ERR_SIZE;
    router_topk_kernel<<<T, ROUTER_THREADS, 0, stream>>>(x, Wr, shared_gate, H, E, k, norm_topk, sel, w, shared_scale);
    return launch_status();
}

// sel: [n_picks] expert of pick i = t * k + j.  Outputs: offsets [E + 1], slot_token
// [n_picks] (the token whose row feeds sorted slot s), slot_of_pick [n_picks].
CJ_EXPORT int cj_moe_group(const int* sel, int n_picks, int k, int E, int* offsets, int* slot_token,
                           int* slot_of_pick, cudaStream_t stream) {
    if (E < 1 || k < 1 || n_picks < 0) return CJ_ERR_SIZE;
    if (!sel || !offsets || !slot_token || !slot_of_pick) return CJ_ERR_ARG;
    moe_group_kernel<<<E, 32, 0, stream>>>(sel, n_picks, k, E, offsets, slot_token, slot_of_pick);
    return launch_status();
}
