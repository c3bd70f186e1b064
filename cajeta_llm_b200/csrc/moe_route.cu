// Routing of a mixture of experts: router logits, softmax and top-k, and the counting
// sort of the picks by expert.  Everything here is float32.
#include "common.cuh"

using namespace cj;

namespace {

constexpr int ROUTER_THREADS = 256;
constexpr int MAX_EXPERTS = 1024;

// Router in two launches.
//
// (1) logits: l[t, e] = sum_j Wr[e, j] * x[t, j] in float32, and in column E the shared
// expert's gate dot g . x[t].  A block stages TOKB rows of x in shared memory and each of
// its warps takes experts in turn, reading a weight row once for all TOKB rows; with few
// rows (decode) the experts are spread over several blocks instead.  A lane sums its own
// strided share of the row and the warp adds the 32 shares by butterfly, so a row's logits
// depend on nothing but the row.
// (2) select: softmax over ALL experts; top-k by repeated argmax with a strict '>' so
// that ties go to the lower index; w_k = p_sel; optional renormalisation with the divisor
// clamped at 2^-14 (model/MoeFfn.cajeta:908-988; device twin
// io/QuantKernel.cajeta:40849-40942); the gate becomes sigma(g . x)
// (model/MoeFfn.cajeta:1925-1964).
template <int TOKB>
__global__ void __launch_bounds__(ROUTER_THREADS) router_logits_kernel(
    const float* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ shared_gate, int T, int H,
    int E, int experts_per_block, float* __restrict__ logits) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ __align__(16) float xs[];         // [TOKB][H]
    const int t0 = blockIdx.x * TOKB;
    const int n_tok = min(TOKB, T - t0);
    const int n_cols = E + (shared_gate ? 1 : 0);
    const int e_begin = blockIdx.y * experts_per_block;
    const int e_end = min(n_cols, e_begin + experts_per_block);
    for (int i = threadIdx.x; i < TOKB * H; i += ROUTER_THREADS) {
        int tt = i / H;
        xs[i] = tt < n_tok ? x[(size_t)t0 * H + i] : 0.0f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = ROUTER_THREADS / 32;
    constexpr int EB = 8;                     // experts a warp keeps accumulators for at a time
    const bool vec = (H % 4) == 0;
    // a warp takes experts e_begin + warp + NW * i; EB of them at a time, so that a chunk of x
    // read from shared memory is used EB times (the loop over j is the outer one)
    for (int eb = e_begin + warp; eb < e_end; eb += NW * EB) {
        float acc[EB][TOKB];
#pragma unroll
        for (int q = 0; q < EB; ++q)
#pragma unroll
            for (int tt = 0; tt < TOKB; ++tt) acc[q][tt] = 0.0f;
        if (vec) {
            for (int j = lane * 4; j < H; j += 128) {
                float4 x4[TOKB];
#pragma unroll
                for (int tt = 0; tt < TOKB; ++tt) x4[tt] = *(const float4*)(xs + tt * H + j);
#pragma unroll
                for (int q = 0; q < EB; ++q) {
                    int e = eb + q * NW;
                    if (e < e_end) {
                        const float* wr = e < E ? Wr + (size_t)e * H : shared_gate;
                        float4 w4 = __ldg((const float4*)(wr + j));
#pragma unroll
                        for (int tt = 0; tt < TOKB; ++tt) {
                            acc[q][tt] = fmaf(w4.x, x4[tt].x, acc[q][tt]);
                            acc[q][tt] = fmaf(w4.y, x4[tt].y, acc[q][tt]);
                            acc[q][tt] = fmaf(w4.z, x4[tt].z, acc[q][tt]);
                            acc[q][tt] = fmaf(w4.w, x4[tt].w, acc[q][tt]);
                        }
                    }
                }
            }
        } else {
            for (int j = lane; j < H; j += 32) {
#pragma unroll
                for (int q = 0; q < EB; ++q) {
                    int e = eb + q * NW;
                    if (e < e_end) {
                        float wv = (e < E ? Wr + (size_t)e * H : shared_gate)[j];
#pragma unroll
                        for (int tt = 0; tt < TOKB; ++tt) acc[q][tt] = fmaf(wv, xs[tt * H + j], acc[q][tt]);
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < EB; ++q) {
            int e = eb + q * NW;
#pragma unroll
            for (int tt = 0; tt < TOKB; ++tt) {
                float v = warp_sum(acc[q][tt]);
                if (lane == 0 && e < e_end && tt < n_tok) logits[(size_t)(t0 + tt) * n_cols + e] = v;
            }
        }
    }
}

// softmax over all experts, top-k, optional renormalisation, the shared gate's sigmoid: one
// warp per row; probs is the warp's scratch of E floats in shared memory
// pin (int32 [T, k], may be null): the experts are not chosen here but given - the weights are
// still this row's own probabilities of them (how the reference replays recorded selections,
// model/MoeFfn.cajeta:626-706).  gap (float32 [T], may be null; not with pin): the row's
// routing margin (p_k - p_{k+1}) / p_k, 1 when every expert is picked - how far the row is
// from another choice (model/MoeFfn.cajeta:135-149).
__device__ __forceinline__ void select_row(const float* row, int t, int E, int k, int norm_topk, int* __restrict__ sel,
                                           float* __restrict__ w, float* __restrict__ shared_scale, float* probs, int lane,
                                           const int* __restrict__ pin, float* __restrict__ gap) {
    if (shared_scale && lane == 0) shared_scale[t] = 1.0f / (1.0f + expf(-row[E]));
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, row[e]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) {
        float p = expf(row[e] - mx);
        probs[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) probs[e] = probs[e] / sum;
    __syncwarp();

    if (pin) {
        if (lane == 0) {
            float total = 0.0f;
            for (int j = 0; j < k; ++j) {
                int e = pin[t * k + j];
                float p = (e >= 0 && e < E) ? probs[e] : __int_as_float(0x7fc00000);   // a pick outside the experts shows as NaN
                sel[t * k + j] = (e >= 0 && e < E) ? e : 0;
                w[t * k + j] = p;
                total += p;
            }
            if (norm_topk) {
                if (total < 0.00006103515625f) total = 0.00006103515625f;
                for (int j = 0; j < k; ++j) w[t * k + j] = w[t * k + j] / total;
            }
        }
        return;
    }
    float wsum = 0.0f, last = 0.0f, mine = 0.0f;
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
        // a pick's weight stays with lane j until the sum is known (picks past 31 go through memory)
        const bool held = norm_topk && j < 32;
        if (held && lane == j) mine = bp;
        if (lane == 0) {
            sel[t * k + j] = best;
            if (!held) w[t * k + j] = bp;
        }
        wsum += bp;
        last = bp;
        __syncwarp();
    }
    if (gap) {
        float next = -1.0f;                          // the largest probability left
        for (int e = lane; e < E; e += 32) next = fmaxf(next, probs[e]);
        next = warp_max(next);
        if (lane == 0) gap[t] = (k < E && last > 0.0f) ? (last - next) / last : 1.0f;
    }
    if (norm_topk) {
        if (wsum < 0.00006103515625f) wsum = 0.00006103515625f;
        if (lane < k) w[t * k + lane] = mine / wsum;
        if (lane == 0)
            for (int j = 32; j < k; ++j) w[t * k + j] = w[t * k + j] / wsum;
    }
}

// The same logits for a handful of rows (decode), and the selection, in ONE launch: a block
// is one expert and up to eight rows, one row per warp, each warp with the same
// lane-strided sum as above (so both kernels give the same bits for a row); all loads of a
// warp are independent and go out together, which matters because the weight row is cold
// (the experts' weights have flushed L2 since the last layer).  The block that finishes a
// group of rows last (a ticket in global memory, left at zero again) runs the selection for
// those rows.
constexpr int SMALL_ROWS = 8;
__global__ void __launch_bounds__(SMALL_ROWS * 32) router_small_kernel(
    const float* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ shared_gate, int T, int H,
    int E, int k, int norm_topk, float* __restrict__ logits, int* __restrict__ sel, float* __restrict__ w,
    float* __restrict__ shared_scale, int* __restrict__ tickets, const int* __restrict__ pin, float* __restrict__ gap) {
    cj::release_successor();
    __shared__ float probs[SMALL_ROWS][MAX_EXPERTS];
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_cols = E + (shared_gate ? 1 : 0);
    const int e = blockIdx.x;
    const int t = blockIdx.y * SMALL_ROWS + warp;
    const float* wr = e < E ? Wr + (size_t)e * H : shared_gate;
    const bool vec = (H % 4) == 0;
    // the weight row is written by no kernel: its loads (cold, from memory) go out before this
    // kernel waits for the one before it
    constexpr int PRE = 16;                       // float4 pieces of the row a lane holds ahead
    float4 wv[PRE];
    if (vec && t < T) {
#pragma unroll
        for (int u = 0; u < PRE; ++u) {
            int j = lane * 4 + 128 * u;
            wv[u] = j < H ? __ldg((const float4*)(wr + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    cj::after_predecessor();
    if (t < T) {
        const float* xr = x + (size_t)t * H;
        float acc = 0.0f;
        if (vec) {
            float4 xv[PRE];
#pragma unroll
            for (int u = 0; u < PRE; ++u) {
                int j = lane * 4 + 128 * u;
                xv[u] = j < H ? *(const float4*)(xr + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < PRE; ++u) {
                if (lane * 4 + 128 * u >= H) break;
                acc = fmaf(wv[u].x, xv[u].x, acc);
                acc = fmaf(wv[u].y, xv[u].y, acc);
                acc = fmaf(wv[u].z, xv[u].z, acc);
                acc = fmaf(wv[u].w, xv[u].w, acc);
            }
            // rows wider than the pieces held ahead
            for (int j = lane * 4 + 128 * PRE; j < H; j += 128) {
                float4 w4 = __ldg((const float4*)(wr + j));
                float4 x4 = *(const float4*)(xr + j);
                acc = fmaf(w4.x, x4.x, acc);
                acc = fmaf(w4.y, x4.y, acc);
                acc = fmaf(w4.z, x4.z, acc);
                acc = fmaf(w4.w, x4.w, acc);
            }
        } else {
            for (int j = lane; j < H; j += 32) acc = fmaf(wr[j], xr[j], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[(size_t)t * n_cols + e] = acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int done = atomicAdd(&tickets[blockIdx.y], 1);
        is_last = done == n_cols - 1;
        if (is_last) tickets[blockIdx.y] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (t < T) {
        select_row(logits + (size_t)t * n_cols, t, E, k, norm_topk, sel, w, shared_scale, probs[warp], lane, pin, gap);
    }
}

__global__ void __launch_bounds__(32) router_select_kernel(
    const float* __restrict__ logits, int E, int n_cols, int k, int norm_topk, int* __restrict__ sel,
    float* __restrict__ w, float* __restrict__ shared_scale, const int* __restrict__ pin, float* __restrict__ gap) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float probs[MAX_EXPERTS];
    select_row(logits + (size_t)blockIdx.x * n_cols, blockIdx.x, E, k, norm_topk, sel, w, shared_scale, probs, threadIdx.x, pin, gap);
}

// The selection from logits that a product split along K left as partial sums
// [n_partials][T][ld] (column E: the shared gate's dot): a warp adds a row's partials in
// split order and selects.  Four rows a block.
constexpr int SELECT_ROWS = 4;
__global__ void __launch_bounds__(SELECT_ROWS * 32) router_select_partials_kernel(
    const float* __restrict__ partials, int n_partials, long long partial_stride, int ld, int T, int E, int k,
    int norm_topk, int* __restrict__ sel, float* __restrict__ w, float* __restrict__ shared_scale,
    const int* __restrict__ pin, float* __restrict__ gap) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float probs[SELECT_ROWS][MAX_EXPERTS];
    __shared__ float row[SELECT_ROWS][MAX_EXPERTS + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * SELECT_ROWS + warp;
    if (t >= T) return;
    const int n_cols = E + (shared_scale ? 1 : 0);
    for (int e = lane; e < n_cols; e += 32) {
        float v = 0.0f;
        for (int s = 0; s < n_partials; ++s) v += partials[s * partial_stride + (size_t)t * ld + e];
        row[warp][e] = v;
    }
    __syncwarp();
    select_row(row[warp], t, E, k, norm_topk, sel, w, shared_scale, probs[warp], lane, pin, gap);
}

// Counting sort of the picks (token t, choice j) by expert, stable.  One block per
// expert: its warps each take a contiguous stretch of the picks, count the picks of lower
// experts (the expert's first slot) and their own, and then place their own in pick order.  reference: model/MoeFfn.cajeta:2064-2099 (groupPicks), device
// io/QuantKernel.cajeta:41069.
//
// After the E routed groups come `extra` groups that every token belongs to (the chunks
// of a shared expert run through the same grouped products): group E + c owns slots
// [n + c * T, n + (c + 1) * T) and slot n + c * T + t reads token t.
// GROUP_WARPS warps a block: 8 for the few picks of a decode step, 32 for a prompt's thousands
// (a warp walks its stretch 32 picks at a time, so the walk is as long as the stretch).
template <int GROUP_WARPS>
__global__ void __launch_bounds__(GROUP_WARPS * 32) moe_group_kernel(
    const int* __restrict__ sel, int n, int k, int E, int extra, int* __restrict__ offsets,
    int* __restrict__ slot_token, int* __restrict__ slot_of_pick) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ int lt_s[GROUP_WARPS], eq_s[GROUP_WARPS];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int T = n / k;
    if (e >= E) {
        int c = e - E;
        for (int t = threadIdx.x; t < T; t += blockDim.x) slot_token[n + c * T + t] = t;
        if (threadIdx.x == 0) {
            offsets[E + c] = n + c * T;
            if (c == extra - 1) offsets[E + extra] = n + extra * T;
        }
        return;
    }
    // each warp owns a contiguous segment of the picks (a multiple of 32 long)
    const int seg = (((n + GROUP_WARPS - 1) / GROUP_WARPS) + 31) & ~31;
    const int lo = min(n, warp * seg), hi = min(n, lo + seg);
    int lt = 0, eq = 0;
    for (int i = lo + lane; i < hi; i += 32) {
        int v = sel[i];
        lt += v < e ? 1 : 0;
        eq += v == e ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lt += __shfl_xor_sync(0xffffffffu, lt, o);
        eq += __shfl_xor_sync(0xffffffffu, eq, o);
    }
    if (lane == 0) { lt_s[warp] = lt; eq_s[warp] = eq; }
    __syncthreads();
    int below = 0, cursor = 0;
#pragma unroll
    for (int w = 0; w < GROUP_WARPS; ++w) {
        below += lt_s[w];
        if (w < warp) cursor += eq_s[w];
    }
    cursor += below;
    // placement in pick order: the segments are in order, and so is each warp's walk
    for (int base = lo; base < hi; base += 32) {
        int i = base + lane;
        bool mine = i < hi && sel[i] == e;
        unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            int pos = cursor + __popc(ballot & ((1u << lane) - 1u));
            slot_token[pos] = i / k;
            slot_of_pick[i] = pos;
        }
        cursor += __popc(ballot);
    }
    if (threadIdx.x == 0) {
        offsets[e] = below;
        if (e == E - 1 && extra == 0) {
            int total = below;
            for (int w = 0; w < GROUP_WARPS; ++w) total += eq_s[w];
            offsets[E] = total;
        }
    }
}

}  // namespace

// logits: scratch [T, E + 1] float32 (column E holds the shared gate's dot when a gate is given).
// tickets: int32 [4], zero before the first use (the kernel leaves them zero); may be null, the two-launch form is then used.
// pin: int32 [T, k] experts given instead of chosen, or null.  gap: float32 [T] routing margins out, or null.
CJ_EXPORT int cj_router_topk(const float* x, const float* Wr, const float* shared_gate, int T, int H, int E, int k,
                             int norm_topk, int* sel, float* w, float* shared_scale, float* logits, int* tickets,
                             const int* pin, float* gap, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!x || !Wr || !sel || !w || !logits || H <= 0) return CJ_ERR_ARG;
    if (shared_gate && !shared_scale) return CJ_ERR_ARG;
    if (E < 1 || E > MAX_EXPERTS || k < 1 || k > E) return CJ_ERR_SIZE;
    const int n_cols = E + (shared_gate ? 1 : 0);
    if (T <= 32 && tickets) {
        dim3 grid_small(n_cols, (T + SMALL_ROWS - 1) / SMALL_ROWS);
        cj::launch(router_small_kernel, dim3(grid_small), dim3(SMALL_ROWS * 32), 0, stream, x, Wr, shared_gate, T, H, E, k, norm_topk, logits, sel, w,
                                                                         shared_gate ? shared_scale : nullptr, tickets, pin, gap);
        return launch_status();
    }
    // rows of x staged per block: as many as fit 200 KB of shared memory, at most 8
    int tokb = 8;
    while (tokb > 1 && (size_t)tokb * H * sizeof(float) > 200 * 1024) tokb >>= 1;
    if ((size_t)tokb * H * sizeof(float) > 200 * 1024) return CJ_ERR_SIZE;
    size_t smem = (size_t)tokb * H * sizeof(float);
    int row_blocks = (T + tokb - 1) / tokb;
    // few rows: spread the experts over blocks (8 per block, one per warp)
    int per_block = row_blocks >= 128 ? n_cols : (row_blocks >= 16 ? 32 : 8);
    dim3 grid(row_blocks, (n_cols + per_block - 1) / per_block);
#define LAUNCH(TB)                                                                                                   \
    {                                                                                                                \
        static bool configured = false;                                                                              \
        if (!configured) {                                                                                           \
            cudaError_t e = cudaFuncSetAttribute(router_logits_kernel<TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e;                                                                     \
            configured = true;                                                                                       \
        }                                                                                                            \
        cj::launch(router_logits_kernel<TB>, dim3(grid), dim3(ROUTER_THREADS), smem, stream, x, Wr, shared_gate, T, H, E, per_block, logits); \
    }
    if (tokb == 8) LAUNCH(8) else if (tokb == 4) LAUNCH(4) else if (tokb == 2) LAUNCH(2) else LAUNCH(1)
#undef LAUNCH
    int st = launch_status();
    if (st) return st;
    cj::launch(router_select_kernel, dim3(T), dim3(32), 0, stream, logits, E, n_cols, k, norm_topk, sel, w, shared_gate ? shared_scale : nullptr,
               pin, gap);
    return launch_status();
}

// partials: [n_partials][T][ld] float32 logits (column E the shared gate's dot when shared_scale is given).
CJ_EXPORT int cj_router_select(const float* partials, int n_partials, long long partial_stride, int ld, int T, int E, int k,
                               int norm_topk, int* sel, float* w, float* shared_scale, const int* pin, float* gap,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!partials || !sel || !w || n_partials < 1) return CJ_ERR_ARG;
    if (E < 1 || E > MAX_EXPERTS || k < 1 || k > E || ld < E + (shared_scale ? 1 : 0)) return CJ_ERR_SIZE;
    cj::launch(router_select_partials_kernel, dim3((T + SELECT_ROWS - 1) / SELECT_ROWS), dim3(SELECT_ROWS * 32), 0, stream, 
        partials, n_partials, partial_stride, ld, T, E, k, norm_topk, sel, w, shared_scale, pin, gap);
    return launch_status();
}

// sel: [n_picks] expert of pick i = t * k + j.  Outputs: offsets [E + extra + 1], slot_token
// [n_picks + extra * T] (the token whose row feeds sorted slot s), slot_of_pick [n_picks].
CJ_EXPORT int cj_moe_group(const int* sel, int n_picks, int k, int E, int extra, int* offsets, int* slot_token,
                           int* slot_of_pick, cudaStream_t stream) {
    if (E < 1 || k < 1 || n_picks < 0 || extra < 0) return CJ_ERR_SIZE;
    if (!sel || !offsets || !slot_token || !slot_of_pick) return CJ_ERR_ARG;
    if (n_picks >= 2048)
        cj::launch(moe_group_kernel<32>, dim3(E + extra), dim3(32 * 32), 0, stream, sel, n_picks, k, E, extra, offsets, slot_token, slot_of_pick);
    else
        cj::launch(moe_group_kernel<8>, dim3(E + extra), dim3(8 * 32), 0, stream, sel, n_picks, k, E, extra, offsets, slot_token, slot_of_pick);
    return launch_status();
}
