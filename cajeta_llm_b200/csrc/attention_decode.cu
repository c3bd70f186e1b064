// Decode attention for the bfloat16 path: few query rows, each over a long stretch of
// cached keys.  The keys of a row are cut into fixed chunks of 64 or 128 ("split-KV"); one
// block takes one (row, kv head, chunk), stages the chunk's keys and values in shared
// memory, and then four lanes share a key for the scores and each thread takes eight output
// dims of a key phase for the weighted sum of values, for every query head of the kv head's group.  A chunk leaves a partial (max, sum, unnormalised accumulator); the
// block that finishes a (row, head) last merges the partials in chunk order, so the
// result does not depend on which block arrived when, nor - the chunking being a function
// of the row's own [from, p] - on what else is in the batch.
//
// Formula as in the general kernel (model/PagedKvCache.cajeta:374-470); the split scheme
// follows the reference's flash-decode kernels and their reduce
// (model/AttnKernel.cajeta:1227-1459, :2204), which cut by a wave count instead.
#include "common.cuh"

using namespace cj;

namespace {

constexpr int THREADS = 256;     // threads per block; a block takes CHUNK (64 or 128) keys

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Two float32 multiply-adds in one instruction (sm_100 f32x2): the kernel is bound by the
// number of instructions it issues, and the dot products are half of them.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ f32x2 bf16x2_to_f32x2(uint32_t u) {       // the two bfloat16 halves widened
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(u << 16), "r"(u & 0xffff0000u));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ float2 unpack2(f32x2 v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}

// The chunk's keys and values are fetched with cp.async in one go (every load of the block
// is in flight at once) into shared memory, 16-byte pieces XOR-swizzled by row so that both
// the per-key reads of the scores and the per-column reads of the value sum are free of
// bank conflicts; all query heads of the kv head's group then work from shared memory.
template <int HD, int CHUNK>
__global__ void __launch_bounds__(THREADS) decode_attention_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kplane,
    const __nv_bfloat16* __restrict__ vplane, const int* __restrict__ positions, const int* __restrict__ row_req,
    const int* __restrict__ table, int table_stride, int page_tokens, int n_heads, int n_kv, int window, float scale,
    float* __restrict__ part_acc, float* __restrict__ part_ml, int* __restrict__ counters, int max_splits) {
    cj::after_predecessor();
    cj::release_successor();
    constexpr int VEC = 8;                        // dims one thread owns in the value sum (one 16-byte piece)
    constexpr int COLS = HD / VEC;                // pieces of a row
    constexpr int KPAR = THREADS / COLS;          // key phases working side by side in the value sum
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ks = (__nv_bfloat16*)smem_raw;             // [CHUNK][HD], pieces swizzled
    __nv_bfloat16* vs = ks + CHUNK * HD;                      // [CHUNK][HD], pieces swizzled
    __shared__ float es[CHUNK];
    __shared__ long long bases[CHUNK];
    __shared__ float red[THREADS / 32];
    __shared__ float vsum[KPAR][HD + 4];
    __shared__ float lsum[KPAR];
    __shared__ int is_last;

    const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int p = positions[t];
    const int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int n_keys = p - from + 1;
    const int n_splits = (n_keys + CHUNK - 1) / CHUNK;
    if (split >= n_splits) return;
    const int group = n_heads / n_kv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int key0 = from + split * CHUNK;
    const int count = min(CHUNK, p - key0 + 1);
    const int* tab = table + (size_t)row_req[t] * table_stride;

    // where each key of the chunk lives
    if (tid < count) {
        int key = key0 + tid;
        int page = tab[key / page_tokens];
        bases[tid] = (((long long)page * n_kv + kvh) * page_tokens + key % page_tokens) * HD;
    }
    __syncthreads();
    // all keys, then all values, on their way to shared memory: a thread fetches piece c of
    // rows r0, r0 + ROWS_STEP, ... (the swizzle of a row depends on r mod 8 only, which a step
    // of a multiple of 8 rows leaves alone, so the piece's place in the row is computed once)
    {
        constexpr int ROWS_STEP = THREADS / COLS;
        static_assert(ROWS_STEP % 8 == 0, "rows a pass apart must share their swizzle");
        const int c = tid % COLS, r0 = tid / COLS;
        const int in_row = (c ^ (r0 & 7)) * VEC;
#pragma unroll
        for (int j = 0; j < CHUNK / ROWS_STEP; ++j) {
            int r = r0 + j * ROWS_STEP;
            if (r < count) cp_async16(ks + r * HD + in_row, kplane + bases[r] + c * VEC);
        }
        cp_async_commit();
#pragma unroll
        for (int j = 0; j < CHUNK / ROWS_STEP; ++j) {
            int r = r0 + j * ROWS_STEP;
            if (r < count) cp_async16(vs + r * HD + in_row, vplane + bases[r] + c * VEC);
        }
        cp_async_commit();
    }

    // scores: four lanes share a key, each with a quarter of the head's dims (its part of q in
    // registers); lane = quarter * 8 + key, so that the eight lanes of a shared-memory
    // wavefront read eight different rows at eight different swizzled pieces
    constexpr int QD = HD / 4;                     // dims a lane owns in the score
    constexpr int KEYS_PER_PASS = THREADS / 4;     // keys the block scores side by side
    const int quarter = lane >> 3;
    for (int hg = 0; hg < group; ++hg) {
        const int h = kvh * group + hg;
        f32x2 qr[QD / 2];                            // this lane's quarter of q, in pairs of dims
        {
            const __nv_bfloat16* qp = q + ((size_t)t * n_heads + h) * HD + quarter * QD;
#pragma unroll
            for (int c = 0; c < QD / 8; ++c) {
                uint4 u = *(const uint4*)(qp + c * 8);
                qr[c * 4 + 0] = bf16x2_to_f32x2(u.x);
                qr[c * 4 + 1] = bf16x2_to_f32x2(u.y);
                qr[c * 4 + 2] = bf16x2_to_f32x2(u.z);
                qr[c * 4 + 3] = bf16x2_to_f32x2(u.w);
            }
        }
        if (hg == 0) cp_async_wait<1>();                        // this thread's key pieces have landed
        __syncthreads();                                        // everyone's; the previous head is done with es / vsum

        float sc[CHUNK / KEYS_PER_PASS];
        float m = -INFINITY;
        // a lane's keys are KEYS_PER_PASS apart (a multiple of 8): one swizzle for all of them
        const __nv_bfloat16* krow = ks + (warp * 8 + (lane & 7)) * HD;
        int in_row[QD / 8];
#pragma unroll
        for (int c = 0; c < QD / 8; ++c) in_row[c] = ((quarter * (QD / 8) + c) ^ (lane & 7)) * VEC;
#pragma unroll
        for (int pass = 0; pass < CHUNK / KEYS_PER_PASS; ++pass) {
            const int key = pass * KEYS_PER_PASS + warp * 8 + (lane & 7);
            f32x2 d0 = 0, d1 = 0;                                   // (even dims, odd dims) sums, two chains
#pragma unroll
            for (int c = 0; c < QD / 8; ++c) {
                uint4 u = *(const uint4*)(krow + pass * KEYS_PER_PASS * HD + in_row[c]);
                d0 = fma2(qr[c * 4 + 0], bf16x2_to_f32x2(u.x), d0);
                d1 = fma2(qr[c * 4 + 1], bf16x2_to_f32x2(u.y), d1);
                d0 = fma2(qr[c * 4 + 2], bf16x2_to_f32x2(u.z), d0);
                d1 = fma2(qr[c * 4 + 3], bf16x2_to_f32x2(u.w), d1);
            }
            float2 s0 = unpack2(d0), s1 = unpack2(d1);
            float dot = (s0.x + s1.x) + (s0.y + s1.y);
            dot += __shfl_xor_sync(0xffffffffu, dot, 8);
            dot += __shfl_xor_sync(0xffffffffu, dot, 16);
            sc[pass] = key < count ? dot * scale : -INFINITY;     // rows past the chunk's end hold nothing
            m = fmaxf(m, sc[pass]);
        }
        m = warp_max(m);
        if (lane == 0) red[warp] = m;
        __syncthreads();
        m = red[0];
#pragma unroll
        for (int w = 1; w < THREADS / 32; ++w) m = fmaxf(m, red[w]);
#pragma unroll
        for (int pass = 0; pass < CHUNK / KEYS_PER_PASS; ++pass) {
            const int key = pass * KEYS_PER_PASS + warp * 8 + (lane & 7);
            float e = key < count ? expf(sc[pass] - m) : 0.0f;
            if (quarter == 0) es[key] = e;
        }
        if (hg == 0) cp_async_wait<0>();                        // this thread's value pieces have landed
        __syncthreads();                                        // everyone has read red; es and values visible

        // values: thread = (8 dims, key phase); the keys of its phase in order (KPAR apart, a
        // multiple of 8: one swizzle), and with them the phase's share of the sum of e
        const int col = tid % COLS, phase = tid / COLS;
        static_assert(KPAR % 8 == 0, "keys of a phase must share their swizzle");
        const __nv_bfloat16* vcol = vs + ((col ^ (phase & 7)) * VEC);
        f32x2 acc2[VEC / 2] = {0, 0, 0, 0};
        float lpart = 0.0f;
#pragma unroll 4
        for (int j = phase; j < count; j += KPAR) {
            float ej = es[j];
            lpart += ej;
            const f32x2 e2 = pack2(ej, ej);
            uint4 u = *(const uint4*)(vcol + j * HD);
            acc2[0] = fma2(e2, bf16x2_to_f32x2(u.x), acc2[0]);
            acc2[1] = fma2(e2, bf16x2_to_f32x2(u.y), acc2[1]);
            acc2[2] = fma2(e2, bf16x2_to_f32x2(u.z), acc2[2]);
            acc2[3] = fma2(e2, bf16x2_to_f32x2(u.w), acc2[3]);
        }
#pragma unroll
        for (int d = 0; d < VEC / 2; ++d) *(float2*)&vsum[phase][VEC * col + 2 * d] = unpack2(acc2[d]);
        if (col == 0) lsum[phase] = lpart;
        __syncthreads();
        if (tid < HD / 2) {
            float2 a = make_float2(0.0f, 0.0f);
            float l = 0.0f;
#pragma unroll
            for (int ph = 0; ph < KPAR; ++ph) {
                a.x += vsum[ph][2 * tid];
                a.y += vsum[ph][2 * tid + 1];
                l += lsum[ph];
            }
            if (n_splits == 1) {
                float inv = 1.0f / l;
                *(__nv_bfloat162*)(out + ((size_t)t * n_heads + h) * HD + 2 * tid) = __floats2bfloat162_rn(a.x * inv, a.y * inv);
            } else {
                size_t slot = ((size_t)t * n_heads + h) * max_splits + split;
                *(float2*)(part_acc + slot * HD + 2 * tid) = a;
                if (tid == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
            }
        }
    }
    if (n_splits == 1) return;

    // the last chunk of this (row, kv head) to finish merges all chunks, in chunk order.  The
    // barrier orders the block's partial stores before thread 0, whose fence (cumulative)
    // orders them before its ticket.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        int done = atomicAdd(&counters[t * n_kv + kvh], 1);
        is_last = done == n_splits - 1;
        if (is_last) {
            counters[t * n_kv + kvh] = 0;                       // ready for the next launch
            __threadfence();                                    // the other chunks' partials, published before their tickets
        }
    }
    __syncthreads();
    if (!is_last) return;
    for (int hg = 0; hg < group; ++hg) {
        const int h = kvh * group + hg;
        size_t slot0 = ((size_t)t * n_heads + h) * max_splits;
        float M = -INFINITY;
        for (int sidx = 0; sidx < n_splits; ++sidx) M = fmaxf(M, part_ml[(slot0 + sidx) * 2]);
        float L = 0.0f;
        for (int sidx = 0; sidx < n_splits; ++sidx) L += part_ml[(slot0 + sidx) * 2 + 1] * expf(part_ml[(slot0 + sidx) * 2] - M);
        if (tid < HD / 2) {
            float2 a = make_float2(0.0f, 0.0f);
            for (int sidx = 0; sidx < n_splits; ++sidx) {
                float f = expf(part_ml[(slot0 + sidx) * 2] - M);
                float2 v = *(const float2*)(part_acc + (slot0 + sidx) * HD + 2 * tid);
                a.x = fmaf(v.x, f, a.x);
                a.y = fmaf(v.y, f, a.y);
            }
            float inv = 1.0f / L;
            *(__nv_bfloat162*)(out + ((size_t)t * n_heads + h) * HD + 2 * tid) = __floats2bfloat162_rn(a.x * inv, a.y * inv);
        }
    }
}


// ---------------------------------------------------------------------------------------------
// The same chunk on the tensor cores (mma.sync m16n8k16, bf16 in, f32 out): a chunk's scores
// and weighted values are 256 tensor instructions and a few dozen fragment loads instead of
// thousands of multiply-adds, and ALL query heads of a kv head's group (up to 8 at a time) share
// them - the product's 16 rows are those heads (the rest fed zeros), its columns the chunk's 128
// keys.  Warp w takes keys [32 w, 32 w + 32) for both products; the warps exchange row maxima
// through shared memory and add their partial outputs there in warp order.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
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
// the same product with rows 8..15 of A zero: c0, c1 are rows 0..7; rows 8..15 land in d0, d1
__device__ __forceinline__ void mma_bf16_top(float& c0, float& c1, float& d0, float& d1, unsigned a0, unsigned a2, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c0), "+f"(c1), "+f"(d0), "+f"(d1)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}
// element (row, col) of a [rows][HD] bf16 tile whose 16-byte pieces are XOR-swizzled by row
template <int HD>
__device__ __forceinline__ const __nv_bfloat16* tile_at(const __nv_bfloat16* base, int row, int col) {
    return base + row * HD + (((col >> 3) ^ (row & 7)) << 3) + (col & 7);
}

constexpr int TC_CHUNK = 128;
constexpr int TC_HEADS = 8;          // query heads of a kv head a block takes at a time

// One tile of shared memory holds the chunk's keys and then its values: the keys are fetched and
// scored, the values fetched over them while the exponentials run.  A chunk is a chain of round
// trips (position -> page table -> keys -> values -> partial result) whose length the bytes hardly
// change; what an SM streams is the chunks it has side by side times their bytes over that
// length.  With keys and values in tiles of their own (64 KB) and 256 threads, three blocks fit
// an SM and the kernel streamed 3.9-4.0 TB/s; with one tile (32 KB) and 128 threads - four warps
// of 32 keys - five do, for a chain one round trip longer: 5.4 TB/s at 32 rows x 4,096 keys (a
// step 9 % shorter), batch 64 x 576 keys 3.6 % shorter, batch 1 0.6 % longer.  Six blocks an SM
// (80 registers, a few spilled) measured 1-2 % slower than five.
constexpr int TC_THREADS = 128;
constexpr int TC_WARPS = TC_THREADS / 32;
constexpr int TC_BLOCKS = 5;         // blocks an SM

template <int HD>
__global__ void __launch_bounds__(TC_THREADS, TC_BLOCKS) decode_attention_tc_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kplane,
    const __nv_bfloat16* __restrict__ vplane, const int* __restrict__ positions, const int* __restrict__ row_req,
    const int* __restrict__ table, int table_stride, int page_tokens, int n_heads, int n_kv, int head_batches,
    int window, float scale, float* __restrict__ part_acc, float* __restrict__ part_ml, int* __restrict__ counters,
    int max_splits, int merge_later) {
    cj::release_successor();
    constexpr int COLS = HD / 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* kv = (__nv_bfloat16*)smem_raw;             // [128][HD] swizzled: the keys, then the values, then the warps' partial outputs
    __nv_bfloat16* qs = kv + TC_CHUNK * HD;                   // [8][HD] swizzled: the group's heads, zero rows below them
    __shared__ int bases[TC_CHUNK];                           // the key's row in the plane (pages x kv heads x page tokens)
    __shared__ float smax[TC_WARPS][TC_HEADS];
    __shared__ float ssum[TC_WARPS][TC_HEADS];
    __shared__ int is_last;

    const int t = blockIdx.x, split = blockIdx.z;
    const int kvh = blockIdx.y / head_batches, hb = blockIdx.y % head_batches;
    const int group = n_heads / n_kv;
    const int h0 = kvh * group + hb * TC_HEADS;
    const int n_h = min(TC_HEADS, group - hb * TC_HEADS);
    const int p = __ldcg(positions + t);
    const int req = __ldcg(row_req + t);
    const int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int n_keys = p - from + 1;
    const int n_splits = (n_keys + TC_CHUNK - 1) / TC_CHUNK;
    if (split >= n_splits) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int key0 = from + split * TC_CHUNK;
    const int count = min(TC_CHUNK, p - key0 + 1);
    const int* tab = table + (size_t)req * table_stride;
    {
        int b = 0;
        if (tid < count) {
            int key = key0 + tid;
            int page = __ldcg(tab + key / page_tokens);
            b = (page * n_kv + kvh) * page_tokens + key % page_tokens;
        }
        bases[tid] = b;
    }
    // only the row's own position was written by the kernel before this one; it lies in the row's last chunk
    const bool older_keys_only = split < n_splits - 1;
    if (!older_keys_only) cj::after_predecessor();
    __syncthreads();
    constexpr int ROWS_STEP = TC_THREADS / COLS;
    const int c = tid % COLS, r0 = tid / COLS;
#pragma unroll
    for (int j = 0; j < TC_CHUNK / ROWS_STEP; ++j) {
        const int r = r0 + j * ROWS_STEP;
        cp_async16_zfill(kv + r * HD + ((c ^ (r & 7)) * 8), kplane + (size_t)bases[r] * HD + c * 8, r < count);
    }
    cp_async_commit();
    if (older_keys_only) cj::after_predecessor();
    static_assert(ROWS_STEP >= TC_HEADS, "one pass of the block's threads covers the query tile");
    if (r0 < TC_HEADS) {
        // the queries (the kernel before wrote them): q rows, zero below the heads taken
        uint4 qv = make_uint4(0u, 0u, 0u, 0u);
        if (r0 < n_h) qv = __ldcg((const uint4*)(q + ((size_t)t * n_heads + h0 + r0) * HD + c * 8));
        *(uint4*)(qs + r0 * HD + ((c ^ (r0 & 7)) * 8)) = qv;
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- scores of this warp's 32 keys (two blocks of 16) ---------------------------------------------
    // The product has 16 rows and the block at most 8 heads: rows 8..15 of both products are fed
    // zeros and their sums land in two registers that nothing reads.
    const int g = lane >> 2, t4 = lane & 3, mi = lane >> 3;
    float idle0 = 0.0f, idle1 = 0.0f;
    float s[2][2][2];
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int j = 0; j < 2; ++j) s[kb][j][0] = s[kb][j][1] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        unsigned qf[2];
        ldmatrix_x2(qf, tile_at<HD>(qs, lane & 7, kk * 16 + ((lane >> 3) & 1) * 8));
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            unsigned b[4];
            ldmatrix_x4(b, tile_at<HD>(kv, warp * 32 + kb * 16 + (mi >> 1) * 8 + (lane & 7), kk * 16 + (mi & 1) * 8));
            mma_bf16_top(s[kb][0][0], s[kb][0][1], idle0, idle1, qf[0], qf[1], b[0], b[1]);
            mma_bf16_top(s[kb][1][0], s[kb][1][1], idle0, idle1, qf[0], qf[1], b[2], b[3]);
        }
    }
    // s[kb][j][e]: row g, key warp * 32 + kb * 16 + j * 8 + 2 t4 + e
    float mx0 = -INFINITY;
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool in = warp * 32 + kb * 16 + j * 8 + 2 * t4 + e < count;
                s[kb][j][e] = in ? s[kb][j][e] * scale : -INFINITY;
                mx0 = fmaxf(mx0, s[kb][j][e]);
            }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    if (t4 == 0) smax[warp][g] = mx0;
    __syncthreads();                                            // every warp is done with the keys
    // the values over the keys; their fetch runs during the exponentials.  Rows past the chunk's end
    // are filled with zeros (a stale value row times a zero weight could still be NaN)
#pragma unroll
    for (int j = 0; j < TC_CHUNK / ROWS_STEP; ++j) {
        const int r = r0 + j * ROWS_STEP;
        cp_async16_zfill(kv + r * HD + ((c ^ (r & 7)) * 8), vplane + (size_t)bases[r] * HD + c * 8, r < count);
    }
    cp_async_commit();
    float m0 = smax[0][g];
#pragma unroll
    for (int w = 1; w < TC_WARPS; ++w) m0 = fmaxf(m0, smax[w][g]);
    // the chunk has at least one key, so the maximum is finite
    unsigned pf[2][2];
    float sum0 = 0.0f;
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
        float e00 = expf(s[kb][0][0] - m0), e01 = expf(s[kb][0][1] - m0);
        float e10 = expf(s[kb][1][0] - m0), e11 = expf(s[kb][1][1] - m0);
        sum0 += (e00 + e01) + (e10 + e11);
        pf[kb][0] = pack_bf16(e00, e01);
        pf[kb][1] = pack_bf16(e10, e11);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    if (t4 == 0) ssum[warp][g] = sum0;
    cp_async_wait<0>();
    __syncthreads();                                            // everyone's value pieces have landed

    // ---- this warp's keys' share of the weighted values -----------------------------------------------
    float o[HD / 8][2];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = 0.0f;
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            unsigned b[4];
            ldmatrix_x4_trans(b, tile_at<HD>(kv, warp * 32 + kb * 16 + (mi & 1) * 8 + (lane & 7), dp * 16 + (mi >> 1) * 8));
            mma_bf16_top(o[2 * dp][0], o[2 * dp][1], idle0, idle1, pf[kb][0], pf[kb][1], b[0], b[1]);
            mma_bf16_top(o[2 * dp + 1][0], o[2 * dp + 1][1], idle0, idle1, pf[kb][0], pf[kb][1], b[2], b[3]);
        }
    __syncthreads();                                            // every warp is done with the values: the tile is free
    float* osum = (float*)kv;                                   // [warp][row][HD] float32
    if (g < n_h) {
#pragma unroll
        for (int i = 0; i < HD / 8; ++i)
            *(float2*)(osum + ((size_t)warp * TC_HEADS + g) * HD + i * 8 + 2 * t4) = make_float2(o[i][0], o[i][1]);
    }
    __syncthreads();
    // ---- the chunk's result per head: warps added in order ---------------------------------------------
    for (int i = tid; i < n_h * (HD / 2); i += TC_THREADS) {
        const int row = i / (HD / 2), d2 = i % (HD / 2);
        float2 a = make_float2(0.0f, 0.0f);
        float l = 0.0f;
#pragma unroll
        for (int w = 0; w < TC_WARPS; ++w) {
            float2 v = *(const float2*)(osum + ((size_t)w * TC_HEADS + row) * HD + 2 * d2);
            a.x += v.x;
            a.y += v.y;
            l += ssum[w][row];
        }
        const int h = h0 + row;
        if (n_splits == 1) {
            float inv = 1.0f / l;
            *(__nv_bfloat162*)(out + ((size_t)t * n_heads + h) * HD + 2 * d2) = __floats2bfloat162_rn(a.x * inv, a.y * inv);
        } else {
            size_t slot = ((size_t)t * n_heads + h) * max_splits + split;
            *(float2*)(part_acc + slot * HD + 2 * d2) = a;
            if (d2 == 0) {
                float m = smax[0][row];
#pragma unroll
                for (int w = 1; w < TC_WARPS; ++w) m = fmaxf(m, smax[w][row]);
                part_ml[slot * 2] = m;
                part_ml[slot * 2 + 1] = l;
            }
        }
    }
    if (n_splits == 1 || merge_later) return;

    // the last chunk of this (row, kv head, head batch) to finish merges all chunks, in chunk order
    __syncthreads();
    int* counter = counters + ((size_t)t * n_kv + kvh) * head_batches + hb;
    if (tid == 0) {
        __threadfence();
        int done = atomicAdd(counter, 1);
        is_last = done == n_splits - 1;
        if (is_last) {
            *counter = 0;
            __threadfence();
        }
    }
    __syncthreads();
    if (!is_last) return;
    for (int i = tid; i < n_h * (HD / 2); i += TC_THREADS) {
        const int row = i / (HD / 2), d2 = i % (HD / 2);
        const int h = h0 + row;
        size_t slot0 = ((size_t)t * n_heads + h) * max_splits;
        float M = -INFINITY;
        for (int sidx = 0; sidx < n_splits; ++sidx) M = fmaxf(M, part_ml[(slot0 + sidx) * 2]);
        float L = 0.0f;
        float2 a = make_float2(0.0f, 0.0f);
        for (int sidx = 0; sidx < n_splits; ++sidx) {
            float f = expf(part_ml[(slot0 + sidx) * 2] - M);
            L += part_ml[(slot0 + sidx) * 2 + 1] * f;
            float2 v = *(const float2*)(part_acc + (slot0 + sidx) * HD + 2 * d2);
            a.x = fmaf(v.x, f, a.x);
            a.y = fmaf(v.y, f, a.y);
        }
        float inv = 1.0f / L;
        *(__nv_bfloat162*)(out + ((size_t)t * n_heads + h) * HD + 2 * d2) = __floats2bfloat162_rn(a.x * inv, a.y * inv);
    }
}

// The merge of the chunks of every (row, head) as a kernel of its own, for steps whose attention
// kernel left it out: a warp a (row, head), the chunks added in chunk order with the same
// arithmetic as the in-kernel merge, so both ways give the same bits.
template <int HD>
__global__ void __launch_bounds__(128) decode_merge_kernel(
    __nv_bfloat16* __restrict__ out, const float* __restrict__ part_acc, const float* __restrict__ part_ml,
    const int* __restrict__ positions, int T, int n_heads, int window, int max_splits) {
    cj::release_successor();
    const int lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const bool in_range = idx < (long long)T * n_heads;
    int n_splits = 1;
    if (in_range) {
        const int p = __ldcg(positions + (int)(idx / n_heads));     // the step's metadata: settled before the step's first kernel
        const int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
        n_splits = (p - from + TC_CHUNK) / TC_CHUNK;
    }
    // Every warp waits, also one with nothing to merge: a grid none of whose blocks waited could
    // complete while the attention kernel still runs, and the kernel after this one - which
    // waits for this grid only - would then read `out` too early.
    cj::after_predecessor();
    if (n_splits == 1) return;                                  // out of range, or that row's only chunk wrote the result itself
    const size_t slot0 = (size_t)idx * max_splits;
    float M = -INFINITY;
    for (int sidx = 0; sidx < n_splits; ++sidx) M = fmaxf(M, part_ml[(slot0 + sidx) * 2]);
    for (int d2 = lane; d2 < HD / 2; d2 += 32) {
        float L = 0.0f;
        float2 a = make_float2(0.0f, 0.0f);
        for (int sidx = 0; sidx < n_splits; ++sidx) {
            float f = expf(part_ml[(slot0 + sidx) * 2] - M);
            L += part_ml[(slot0 + sidx) * 2 + 1] * f;
            float2 v = *(const float2*)(part_acc + (slot0 + sidx) * HD + 2 * d2);
            a.x = fmaf(v.x, f, a.x);
            a.y = fmaf(v.y, f, a.y);
        }
        float inv = 1.0f / L;
        *(__nv_bfloat162*)(out + (size_t)idx * HD + 2 * d2) = __floats2bfloat162_rn(a.x * inv, a.y * inv);
    }
}

}  // namespace

// q, out: [T, n_heads, hd] bf16; planes [pages, n_kv, page_tokens, hd] bf16.  max_context
// bounds position + 1 over the rows.  chunk: keys a block takes, 64 or 128.  part_acc: scratch float32 [T, n_heads, max_splits, hd],
// part_ml: [T, n_heads, max_splits, 2], counters: int32 [T * n_kv], zero before the first use
// (the kernel leaves them zero).  hd must be 64 or 128.
CJ_EXPORT int cj_decode_attention(const void* q, void* out, const void* kplane, const void* vplane, const int* positions,
                                  const int* row_req, const int* table, int table_stride, int page_tokens, int T,
                                  int n_heads, int n_kv, int hd, int window, float scale, int max_context,
                                  float* part_acc, float* part_ml, int* counters, int max_splits, int chunk,
                                  cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !row_req || !table || !part_acc || !part_ml || !counters) return CJ_ERR_ARG;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    if (hd != 64 && hd != 128) return CJ_ERR_SIZE;
    if (chunk != 64 && chunk != 128) return CJ_ERR_SIZE;
    int span = window > 0 ? min(window, max_context) : max_context;
    int splits = (span + chunk - 1) / chunk;
    if (splits < 1) splits = 1;
    if (splits > max_splits || splits > 65535 || n_kv > 65535) return CJ_ERR_SIZE;
    dim3 grid(T, n_kv, splits);
#define LAUNCH(HD, CH)                                                                                                 \
    {                                                                                                                  \
        constexpr int smem = 2 * CH * HD * (int)sizeof(__nv_bfloat16);                                                 \
        static bool configured = false;                                                                                \
        if (!configured) {                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<HD, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e != cudaSuccess) return (int)e;                                                                       \
            configured = true;                                                                                         \
        }                                                                                                              \
        cj::launch(decode_attention_kernel<HD, CH>, dim3(grid), dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, \
            (const __nv_bfloat16*)kplane, (const __nv_bfloat16*)vplane, positions, row_req, table, table_stride,       \
            page_tokens, n_heads, n_kv, window, scale, part_acc, part_ml, counters, max_splits);                       \
    }
    if (hd == 128 && chunk == 128) LAUNCH(128, 128)
    else if (hd == 128) LAUNCH(128, 64)
    else if (chunk == 128) LAUNCH(64, 128)
    else LAUNCH(64, 64)
#undef LAUNCH
    return launch_status();
}

// The same on the tensor cores (chunks of 128 keys; up to 8 query heads of a kv head a block).
// counters: int32 [T * n_heads] here (one per row, kv head and batch of 8 heads).
CJ_EXPORT int cj_decode_attention_tc(const void* q, void* out, const void* kplane, const void* vplane, const int* positions,
                                     const int* row_req, const int* table, int table_stride, int page_tokens, int T,
                                     int n_heads, int n_kv, int hd, int window, float scale, int max_context,
                                     float* part_acc, float* part_ml, int* counters, int max_splits, int merge_later,
                                     cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !row_req || !table || !part_acc || !part_ml || !counters) return CJ_ERR_ARG;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    if (hd != 64 && hd != 128) return CJ_ERR_SIZE;
    int span = window > 0 ? min(window, max_context) : max_context;
    int splits = (span + TC_CHUNK - 1) / TC_CHUNK;
    if (splits < 1) splits = 1;
    const int group = n_heads / n_kv;
    const int head_batches = (group + TC_HEADS - 1) / TC_HEADS;
    if (splits > max_splits || splits > 65535 || (long long)n_kv * head_batches > 65535) return CJ_ERR_SIZE;
    dim3 grid(T, n_kv * head_batches, splits);
#define LAUNCH(HD)                                                                                                     \
    {                                                                                                                  \
        constexpr int smem = (TC_CHUNK + TC_HEADS) * HD * (int)sizeof(__nv_bfloat16);                                  \
        static_assert(TC_WARPS * TC_HEADS * HD * 4 <= TC_CHUNK * HD * 2, "the warps' partial outputs must fit the tile"); \
        static bool configured = false;                                                                                \
        if (!configured) {                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(decode_attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e != cudaSuccess) return (int)e;                                                                       \
            configured = true;                                                                                         \
        }                                                                                                              \
        cj::launch(decode_attention_tc_kernel<HD>, dim3(grid), dim3(TC_THREADS), smem, stream, (const __nv_bfloat16*)q, \
            (__nv_bfloat16*)out, (const __nv_bfloat16*)kplane, (const __nv_bfloat16*)vplane, positions, row_req, table, \
            table_stride, page_tokens, n_heads, n_kv, head_batches, window, scale, part_acc, part_ml, counters,        \
            max_splits, merge_later && splits > 1 ? 1 : 0);                                                            \
        if (merge_later && splits > 1)                                                                                 \
            cj::launch(decode_merge_kernel<HD>, dim3((unsigned)(((long long)T * n_heads + 3) / 4)), dim3(128), 0, stream, \
                (__nv_bfloat16*)out, (const float*)part_acc, (const float*)part_ml, positions, T, n_heads, window, max_splits); \
    }
    if (hd == 128) LAUNCH(128) else LAUNCH(64)
#undef LAUNCH
    return launch_status();
}
