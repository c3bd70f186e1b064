// Random weights drawn on the device, element by element from a counter: the value of element
// i of a tensor depends on (key, i) only - not on the launch shape, not on the device - and is
// made of integer arithmetic plus ONE float32 multiply, so that the same few lines in numpy
// (weights/random_fill.py) give the same bits on the host.  A model folder written on the CPU
// and a model drawn in place on the GPU from the same seed therefore hold the same tensors.
//
// The draw: two rounds of the splitmix64 finaliser over key + i * golden give 128 bits, read
// as eight 16-bit integers u_0..u_7; n = 2 * sum(u) - 8 * 65535 is a symmetric integer whose
// distribution (Irwin-Hall of eight) is bell-shaped with tails bounded at +-4.9 standard
// deviations; the value is float32(n) * scale with scale = std / (2 * sqrt(8 * (65536^2 - 1) / 12)).
// (The reference has random weights only as test fixtures, selftest/ToyModel.cajeta:116-120.)
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

__device__ __forceinline__ int sum16(unsigned long long h) {
    return (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) + (int)(h >> 48);
}

template <typename T>
__global__ void __launch_bounds__(256) random_fill_kernel(T* __restrict__ out, long long n, unsigned long long key, float scale) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long h1 = mix64(key + (unsigned long long)i * 0x9E3779B97F4A7C15ull);
        const unsigned long long h2 = mix64(h1 + 0x9E3779B97F4A7C15ull);
        const int centred = 2 * (sum16(h1) + sum16(h2)) - 8 * 65535;
        out[i] = cj::from_f32<T>(__fmul_rn((float)centred, scale));
    }
}

}  // namespace

// out[i] = float32(n(key, i)) * scale for i in [0, count), stored as float32 or bfloat16 (rounded
// to nearest even).
CJ_EXPORT int cj_random_fill(void* out, int dtype, long long count, unsigned long long key, float scale, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (!out) return CJ_ERR_ARG;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == CJ_F32) random_fill_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)out, count, key, scale);
    else if (dtype == CJ_BF16) random_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16*)out, count, key, scale);
    else return CJ_ERR_DTYPE;
    return cj::launch_status();
}
