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
#include <stdlib.h>

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

// Launches overlap their neighbours in the stream (programmatic dependent launch): a kernel
// may be set up on the SMs while the one before it is still draining.  Every kernel of this
// library therefore begins with after_predecessor(), which returns once all earlier work in
// the stream is complete and visible - before it nothing that another kernel writes may be
// read and nothing it reads may be written - and release_successor(), which lets the next
// kernel's blocks be scheduled as SM resources free up (they wait at their own
// after_predecessor()).  In a kernel launched the ordinary way both are no-ops.
__device__ __forceinline__ void after_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void release_successor() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// CAJETA_B200_SERIAL_LAUNCH=1 turns the overlap off (every kernel then starts after the one before has ended)
inline bool overlap_launches() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("CAJETA_B200_SERIAL_LAUNCH");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v != 0;
}

template <typename... P, typename... A>
inline void launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<A&&>(args)...);      // an error is left for launch_status()
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace cj
