// Sampling without any allocation: declaration of cj_sample_static.
//
// This entry point has no counterpart in the reference (its sampler is host code with
// two arrays sized at construction, gen/Sampler.cajeta:24-38); it exists for callers of
// this library that must not, or cannot, allocate device memory at the moment they
// sample:
//   * a C or C++ host that links the kernel library by its exported symbols and brings no
//     allocator of its own (no PyTorch caching allocator behind it);
//   * a serving process that has handed all free device memory to its cache pool at
//     start-up, so that a later cudaMalloc would fail;
//   * a latency-critical loop in which cudaMalloc / cudaFree are unwelcome because they
//     synchronise the whole device.
// The regular entry point, cj_sample, takes the scratch buffer ([rows, V] float32) from
// the caller.  cj_sample_static runs the same kernel with the scratch in a fixed array that
// is part of the library image: CJ_SAMPLE_STATIC_MAX_FLOATS floats (4 MiB), which every
// GPU that loads the library holds until the process exits.
//
// Rules of use
//   * rows * V must not exceed CJ_SAMPLE_STATIC_MAX_FLOATS; a larger request is refused with
//     CJ_SAMPLE_STATIC_TOO_LARGE and nothing is launched.  cj_sample_static_capacity() returns
//     the limit.
//   * The first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
//     on a device before you begin any stream capture on it.  Later calls only launch.
//   * All calls on a device share the one array.  It keeps what the last call left in it;
//     nothing in it has to start at zero, because the kernel writes every element of a row
//     before it reads it.  Two calls whose kernels overlap on the GPU (different streams
//     without an ordering between them) race on the array: order them.
//   * Two host threads that make the first call on a device at the same moment both look the
//     address up and both store the same value: harmless, so the look-up takes no lock.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine.
//
// Arguments and result are those of cj_sample without `scratch`: per row r, temperature[r]
// (0 = greedy), top_k[r] (0 = off), top_p[r] (<= 0 or >= 1 = off), repeat_penalty[r]
// (1 = off) over history[history_offsets[r] .. history_offsets[r + 1]), and the uniform
// draw uniform[r] in [0, 1); top_k, top_p, repeat_penalty and history may be null.  All
// pointers are device pointers.  Returns 0, a negative refusal code, or a cudaError_t.
#pragma once

#include <cuda_runtime.h>

#define CJ_SAMPLE_STATIC_MAX_FLOATS (1 << 20)
#define CJ_SAMPLE_STATIC_TOO_LARGE (-6)     // its own code: -3 is the kernels' general "a size this kernel does not take"

#ifdef __cplusplus
extern "C" {
#endif

int cj_sample_static(const float* logits, int rows, int V, const float* temperature, const int* top_k,
                     const float* top_p, const float* repeat_penalty, const float* uniform, const int* history,
                     const int* history_offsets, int* out, cudaStream_t stream);

long long cj_sample_static_capacity(void);

#ifdef __cplusplus
}
#endif
