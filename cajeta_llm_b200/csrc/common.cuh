// Shared helpers of the hand-written sm_100a kernels.
//
// Every exported function has C linkage, takes raw device pointers plus a stream,
// launches asynchronously and returns 0 or a negative "refused" code / positive
// cudaError_t.  Storage types are passed as small integer codes so that one entry
// point serves the 32-bit path and the bfloat16 path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CJ_F32 0
#define CJ_BF16 1

// refusal codes (negative so they never collide with cudaError_t)
#define CJ_ERR_DTYPE (-2)     // dtype combination not instantiated
#define CJ_ERR_SIZE (-3)      // a size this kernel does not take
#define CJ_ERR_ALIGN (-4)     // pointer or stride alignment this kernel needs
#define CJ_ERR_ARG (-5)       // null pointer or negative count

#define CJ_EXPORT extern "C" __attribute__((visibility("default")))

namespace cj {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x / (1 + exp(-x)), the reference's SiLU (model/Prim.cajeta:1822-1847)
__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace cj
