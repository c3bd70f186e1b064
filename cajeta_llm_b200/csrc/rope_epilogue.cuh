// The q/k/v projection's epilogue that rotates and stores in one go: instead of writing the
// product's float32 sums [tokens, q | k | v] for a second kernel to read, the epilogue rotates
// q and k at each row's position, writes q in the activation dtype and puts the rotated k and
// the raw v straight into the cache pages of the row's request.
//
// For the two halves of a rotation pair (dims i and i + rot/2 of a head) to meet without a
// round trip through shared memory, the projection's weight rows (and bias) are laid out at load
// with the pairs side by side: within each q and k head the row order is 0, rot/2, 1, rot/2 + 1,
// ... (dims past the rotary part follow unchanged; v rows are not reordered).  In a product
// with the features on the accumulator's lanes the partner is then the neighbouring lane (one
// shuffle); with the tokens on the lanes it is the neighbouring column of the same thread.
//
// Formula as in the separate kernel (rowwise.cu): half-split pairs, ang = float(p) * inv[i],
// a' = a cos - b sin, b' = a sin + b cos (model/Prim.cajeta:1917-1940).  cos and sin come from
// a table [tokens, rot/2] that a small kernel fills once per step (the same for every layer);
// where each token's row of the cache starts comes from a table [tokens] filled once per step
// and cache group.
#pragma once

#include "common.cuh"

namespace cj {

struct RopeArgs {
    __nv_bfloat16* q_out;          // [tokens, q_dim]
    __nv_bfloat16* kplane;         // [pages, n_kv, page_tokens, hd]
    __nv_bfloat16* vplane;
    const float2* cos_sin;         // [tokens, rot / 2]
    const long long* kv_base;      // [tokens]: element offset of (page, kv head 0, slot, dim 0) of the token's position, or -1
    int q_dim, kv_dim, hd, rot;
    int head_stride;               // page_tokens * hd: elements between two kv heads of a page
    int write_kv;                  // 0: the product has q features only (the entry reads another entry's cache)
};

// where feature f of the stacked, pair-interleaved projection goes, for a thread that keeps it over many tokens
struct RopeFeature {
    int region;        // 0 q, 1 k, 2 v, -1 none
    int head;
    int dim;           // the dim of the head this feature is written to
    int pair;          // index into the cos / sin row, or -1: not rotated
    int high;          // 1: this feature is the pair's high half (dim = pair + rot / 2)
};

__device__ __forceinline__ RopeFeature rope_feature(const RopeArgs& r, int f, int features) {
    RopeFeature o;
    o.region = -1;
    o.head = o.dim = o.high = 0;
    o.pair = -1;
    if (f >= features) return o;
    int local = f;
    if (f < r.q_dim) o.region = 0;
    else if (f < r.q_dim + r.kv_dim) { o.region = 1; local = f - r.q_dim; }
    else { o.region = 2; local = f - r.q_dim - r.kv_dim; }
    o.head = local / r.hd;
    const int l = local - o.head * r.hd;
    if (o.region < 2 && l < r.rot) {
        o.pair = l >> 1;
        o.high = l & 1;
        o.dim = o.pair + o.high * (r.rot >> 1);
    } else {
        o.dim = l;
    }
    return o;
}

// own: this feature's sum (bias added); partner: the sum of the other half of its pair
__device__ __forceinline__ void rope_store(const RopeArgs& r, const RopeFeature& ft, int token, float own, float partner) {
    float val = own;
    if (ft.pair >= 0) {
        const float2 cs = r.cos_sin[(size_t)token * (r.rot >> 1) + ft.pair];
        val = ft.high ? fmaf(partner, cs.y, own * cs.x) : fmaf(-partner, cs.y, own * cs.x);
    }
    if (ft.region == 0) {
        r.q_out[(size_t)token * r.q_dim + ft.head * r.hd + ft.dim] = __float2bfloat16_rn(val);
    } else if (ft.region > 0) {
        const long long base = r.kv_base[token];
        if (base < 0) return;                        // no page: the host never schedules this
        __nv_bfloat16* plane = ft.region == 1 ? r.kplane : r.vplane;
        plane[base + (long long)ft.head * r.head_stride + ft.dim] = __float2bfloat16_rn(val);
    }
}

}  // namespace cj
