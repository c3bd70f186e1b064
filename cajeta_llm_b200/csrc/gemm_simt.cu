// Matrix products on the float32 FMA pipe:  C[M,N] (+)= A[M,K] . W[N,K]^T (+ bias).
//
// This is the true 32-bit path of every projection (no reduced-precision matrix mode)
// and the general fallback of the bfloat16 path for sizes the tensor-core kernels
// refuse.  Every output element is one sequential chain of fused multiply-adds over
// k = 0..K-1, so a row's result does not depend on which other rows share the launch.
//
// Variants, all one kernel template:
//   * plain / accumulate into C (the residual add of an output projection);
//   * SwiGLU: two weight matrices, C = silu(A.Wg^T) * (A.Wu^T)
//     (model/Prim.cajeta:1822-1847);
//   * grouped: rows of A are "sorted slots" of a mixture of experts; group g owns slots
//     [offsets[g], offsets[g+1]) and its own weight slab W + g * w_group_stride;
//     a_row_index maps a slot to its row of A (the token), as the reference's grouped
//     forward gathers rows per expert (model/MoeFfn.cajeta:2644-2777).
#include "common.cuh"

using namespace cj;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

struct GemmArgs {
    const void* A; long long lda;
    const void* W; const void* W2; long long ldw;
    const float* bias;
    void* C; long long ldc;
    int M, N, K;
    int accumulate;
    const int* group_offsets;     // [num_groups + 1] or null
    const int* a_row_index;       // [M] or null
    long long w_group_stride;
    int num_groups;
};

template <typename TA, typename TW, typename TC, bool SWIGLU>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs p) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float W2s[SWIGLU ? BK : 1][BN + 4];

    // which rows: a plain launch tiles M directly; a grouped launch walks the groups to
    // find the (group, tile) this block owns and leaves when there is none
    int row_begin, row_end;
    const TW* W = (const TW*)p.W;
    const TW* W2 = (const TW*)p.W2;
    if (p.group_offsets) {
        int tile = blockIdx.y, g = 0, first = 0;
        bool found = false;
        for (; g < p.num_groups; ++g) {
            int lo = p.group_offsets[g], hi = p.group_offsets[g + 1];
            int tiles = (hi - lo + BM - 1) / BM;
            if (tile < first + tiles) {
                row_begin = lo + (tile - first) * BM;
                row_end = min(hi, row_begin + BM);
                found = true;
                break;
            }
            first += tiles;
        }
        if (!found) return;
        W += (size_t)g * p.w_group_stride;
        if (SWIGLU) W2 += (size_t)g * p.w_group_stride;
    } else {
        row_begin = blockIdx.y * BM;
        row_end = min(p.M, row_begin + BM);
    }
    int col_begin = blockIdx.x * BN;

    const TA* A = (const TA*)p.A;
    int tid = threadIdx.x;
    int tx = tid % (BN / TN), ty = tid / (BN / TN);

    float acc[TM][TN];
    float acc2[SWIGLU ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.0f;
            if (SWIGLU) acc2[i][j] = 0.0f;
        }

    // each thread loads 4 elements of the A tile and 4 of each W tile per k-step
    int ld_row = tid / 4;            // 0..63
    int ld_k = (tid % 4) * 4;        // 0,4,8,12
    int a_row = row_begin + ld_row;
    long long a_src = -1;
    if (a_row < row_end) a_src = p.a_row_index ? (long long)p.a_row_index[a_row] : (long long)a_row;
    int w_row = col_begin + ld_row;

    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int k = k0 + ld_k + i;
            float av = 0.0f, wv = 0.0f, w2v = 0.0f;
            if (k < p.K) {
                if (a_src >= 0) av = to_f32(A[a_src * p.lda + k]);
                if (w_row < p.N) {
                    wv = to_f32(W[(size_t)w_row * p.ldw + k]);
                    if (SWIGLU) w2v = to_f32(W2[(size_t)w_row * p.ldw + k]);
                }
            }
            As[ld_k + i][ld_row] = av;
            Ws[ld_k + i][ld_row] = wv;
            if (SWIGLU) W2s[ld_k + i][ld_row] = w2v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN], b2[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                b[j] = Ws[kk][tx * TN + j];
                if (SWIGLU) b2[j] = W2s[kk][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (SWIGLU) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }

    TC* C = (TC*)p.C;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int r = row_begin + ty * TM + i;
        if (r >= row_end) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int c = col_begin + tx * TN + j;
            if (c >= p.N) continue;
            float v = acc[i][j];
            if (SWIGLU) v = silu(v) * acc2[i][j];
            if (p.bias) v += p.bias[c];
            size_t o = (size_t)r * p.ldc + c;
            if (p.accumulate) v += to_f32(C[o]);
            C[o] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(const GemmArgs& p, bool swiglu, cudaStream_t stream) {
    int row_tiles = p.group_offsets ? (p.M + BM - 1) / BM + p.num_groups : (p.M + BM - 1) / BM;
    dim3 grid((p.N + BN - 1) / BN, row_tiles);
    if (grid.y > 65535) return CJ_ERR_SIZE;
    if (swiglu) cj::launch(gemm_simt_kernel<TA, TW, TC, true>, dim3(grid), dim3(256), 0, stream, p);
    else cj::launch(gemm_simt_kernel<TA, TW, TC, false>, dim3(grid), dim3(256), 0, stream, p);
    return launch_status();
}

}  // namespace

// a_dtype / w_dtype / c_dtype: CJ_F32 or CJ_BF16.  Instantiated: (f32,f32,f32),
// (bf16,bf16,f32), (bf16,bf16,bf16).  w2 non-null selects the SwiGLU form.
CJ_EXPORT int cj_gemm_simt(const void* A, long long lda, int a_dtype, const void* W, const void* W2, long long ldw,
                           int w_dtype, const float* bias, void* C, long long ldc, int c_dtype, int M, int N, int K,
                           int accumulate, const int* group_offsets, int num_groups, long long w_group_stride,
                           const int* a_row_index, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!A || !W || !C || K <= 0) return CJ_ERR_ARG;
    if (group_offsets && num_groups <= 0) return CJ_ERR_ARG;
    GemmArgs p{A, lda, W, W2, ldw, bias, C, ldc, M, N, K, accumulate, group_offsets, a_row_index, w_group_stride, num_groups};
    bool sw = W2 != nullptr;
    if (a_dtype == CJ_F32 && w_dtype == CJ_F32 && c_dtype == CJ_F32) return launch<float, float, float>(p, sw, stream);
    if (a_dtype == CJ_BF16 && w_dtype == CJ_BF16 && c_dtype == CJ_F32) return launch<__nv_bfloat16, __nv_bfloat16, float>(p, sw, stream);
    if (a_dtype == CJ_BF16 && w_dtype == CJ_BF16 && c_dtype == CJ_BF16) return launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(p, sw, stream);
    return CJ_ERR_DTYPE;
}
