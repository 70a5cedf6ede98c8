// Random weights that every implementation can reproduce bit for bit: a counter-based fill.
//
// Element i of the tensor whose stream starts at `base` (a 64-bit number the host derives from the seed and the
// tensor's name) is
//
//     h0 = mix64(base + (2i) * G),  h1 = mix64(base + (2i + 1) * G),       G = 0x9E3779B97F4A7C15
//     c  = (sum of the eight 16-bit fields of h0 and h1) - 4 * 65535        an integer, |c| <= 262140
//     value = float(c) * scale                                              one rounding
//
// mix64 is the finalizer of splitmix64.  The sum of eight uniform 16-bit integers is close to normal
// (Irwin-Hall), c converts to float exactly, and the one multiplication rounds the same way on every IEEE
// machine, so host code, this kernel and a test's own restatement agree in every bit; the value is then rounded
// to the storage type (to nearest even).  The reference has no random weights at all: it only reads files
// (models/llama/common/src/storage.rs:29-88).
#include "common.cuh"

__host__ __device__ __forceinline__ unsigned long long tb_mix64(unsigned long long z) {
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

__device__ __forceinline__ float counter_normal(unsigned long long base, unsigned long long i, float scale) {
    const unsigned long long G = 0x9E3779B97F4A7C15ull;
    const unsigned long long h0 = tb_mix64(base + (2 * i) * G), h1 = tb_mix64(base + (2 * i + 1) * G);
    int sum = 0;
#pragma unroll
    for (int f = 0; f < 4; ++f) sum += (int)((h0 >> (16 * f)) & 0xFFFF) + (int)((h1 >> (16 * f)) & 0xFFFF);
    return __fmul_rn((float)(sum - 4 * 65535), scale);
}

// Each thread fills eight consecutive elements (one 16-byte store of bfloat16, two of float).
template <typename T>
__global__ void __launch_bounds__(256) random_fill_kernel(T* out, long long n, unsigned long long base, long long first,
                                                          float scale) {
    const long long at = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (at >= n) return;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = counter_normal(base, (unsigned long long)(first + at + j), scale);
    if (at + 8 <= n && ((uintptr_t)(out + at) & 15) == 0) {
        store8(out + at, v);
    } else {
        for (int j = 0; j < 8 && at + j < n; ++j) stf(out + at + j, v[j]);
    }
}

template <typename T>
static int random_fill(void* out, long long n, unsigned long long base, long long first, float scale, cudaStream_t s) {
    if (n < 0 || first < 0) return TB_ERR_ARG;
    if (n == 0) return 0;
    const long long threads = (n + 7) / 8, blocks = (threads + 255) / 256;
    if (blocks > 0x7fffffffll) return TB_ERR_UNSUPPORTED;
    random_fill_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((T*)out, n, base, first, scale);
    return tb_last_error();
}

extern "C" {
// out[j] = value(first + j) for j in [0, n): a slab of a tensor can be filled by itself.
int tb_random_fill_bf16(void* out, long long n, unsigned long long base, long long first, float scale, cudaStream_t s) {
    return random_fill<__nv_bfloat16>(out, n, base, first, scale, s);
}
int tb_random_fill_f32(void* out, long long n, unsigned long long base, long long first, float scale, cudaStream_t s) {
    return random_fill<float>(out, n, base, first, scale, s);
}
}
