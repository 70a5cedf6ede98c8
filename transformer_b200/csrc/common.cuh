// Shared device helpers for the sm_100a kernels of transformer_b200.
//
// Conventions used by every kernel file:
//  * activations and matrices are `T` = float (the true 32-bit path) or __nv_bfloat16 (serving);
//    all arithmetic happens in float, one rounding to T at the store;
//  * the residual stream, router logits, softmax statistics, norm statistics and logits are float;
//  * every launcher is `extern "C"`, takes raw device pointers, sizes and a cudaStream_t, checks
//    its sizes, and returns 0 or a cudaError_t / negative argument error; it never allocates.
#pragma once
#include <mutex>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TB_PAGE 64  // tokens in one cache page

// argument errors returned by launchers (cudaError_t values are positive)
#define TB_ERR_ARG (-1)
#define TB_ERR_UNSUPPORTED (-2)

template <typename T> struct Elem;
template <> struct Elem<float> {
    __device__ __forceinline__ static float load(const float* p) { return *p; }
    __device__ __forceinline__ static void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    __device__ __forceinline__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ __forceinline__ static void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float ldf(const T* p) { return Elem<T>::load(p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { Elem<T>::store(p, v); }

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

// Sum over a block of up to 1024 threads; `red` holds at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// One 16-byte load as floats: 8 bfloat16 or 4 float values.
template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
        unpack(*reinterpret_cast<const uint4*>(p), f);
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float (&f)[8]) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    }
};
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void load(const float* p, float (&f)[4]) {
        unpack(*reinterpret_cast<const uint4*>(p), f);
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
};

// Eight consecutive values as floats (and back): two 16-byte accesses for float, one for bfloat16.
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) { Vec16<__nv_bfloat16>::load(p, f); }
__device__ __forceinline__ void store8(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(f[0], f[1]); v.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[2], f[3]); v.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[4], f[5]); v.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[6], f[7]); v.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(p) = v;
}

// ---- launches with programmatic dependent launch ------------------------------------------------
// Every kernel of this package begins with pdl_sync(): it lets the next kernel in the stream start
// launching (its blocks become resident and wait), then waits until the previous kernel has finished
// and its writes are visible.  Nothing is read or written before that wait, so the overlap never
// changes a result; what it removes is the launch gap between the many small kernels of a decode step.
__device__ __forceinline__ void pdl_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Every kernel states how much of the SM's unified L1/shared memory it wants as shared memory: what the
// blocks that fit by threads and registers need together, and no more.  Without the statement the split
// that a kernel with a large ring asked for stays in force, and the kernels after it run with a sliver
// of L1 (measured: a decode step of small kernels lost a third of its speed behind one 200 KB kernel).
// Looked up per kernel, set again only when a launch needs more than any before it.
// A CUDA call of a launcher's set-up that failed (an attribute query, an attribute that was refused) is kept here
// until the launcher returns: tb_last_error() hands it out before anything else, so it reaches the caller as the
// launcher's result instead of vanishing.  One word per host thread, shared by all files of the library.
inline int& tb_pending_error() {
    static thread_local int code = 0;
    return code;
}
static inline void tb_note_error(cudaError_t e) {
    if (e != cudaSuccess) {
        cudaGetLastError();   // the runtime's own copy would otherwise be blamed on a later, innocent call
        if (!tb_pending_error()) tb_pending_error() = (int)e;
    }
}

static inline void tb_state_carveout(const void* kernel, unsigned threads, size_t dyn_smem) {
    struct Seen { const void* kernel; size_t need; };
    static Seen seen[128];
    static int n_seen = 0;
    static std::mutex lock;
    std::lock_guard<std::mutex> hold(lock);
    int at = -1;
    for (int i = 0; i < n_seen; ++i)
        if (seen[i].kernel == kernel) { at = i; break; }
    if (at >= 0 && dyn_smem <= seen[at].need) return;
    if (at < 0) {
        if (n_seen == 128) return;
        at = n_seen++;
        seen[at].kernel = kernel;
    }
    seen[at].need = dyn_smem;
    cudaFuncAttributes fa;
    {
        const cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
        if (e != cudaSuccess) {
            seen[at].need = 0;    // not stated: the next launch tries again
            tb_note_error(e);
            return;
        }
    }
    const unsigned warps = (threads + 31) / 32;
    const unsigned regs_per_warp = ((unsigned)fa.numRegs * 32 + 255) / 256 * 256;
    unsigned blocks = 2048 / (warps * 32);
    if (regs_per_warp) blocks = blocks < 65536 / (regs_per_warp * warps) ? blocks : 65536 / (regs_per_warp * warps);
    if (blocks > 32) blocks = 32;
    if (blocks < 1) blocks = 1;
    const size_t per_block = fa.sharedSizeBytes + dyn_smem + 1024, sm_total = 228 * 1024;
    size_t want = blocks * per_block;
    if (want > sm_total) want = sm_total / per_block ? sm_total / per_block * per_block : per_block;
    int pct = (int)((want * 100 + sm_total - 1) / sm_total);
    pct = pct < 12 ? 12 : pct > 100 ? 100 : pct;
    tb_note_error(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, pct));
}

template <typename... KArgs, typename... Args>
static inline void tb_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    tb_state_carveout((const void*)kernel, block.x * block.y * block.z, smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface through cudaGetLastError
}
#define TB_LAUNCH(kernel, grid, block, smem, stream, ...) \
    tb_launch_pdl(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__)

static inline int tb_last_error() {
    const int launch = (int)cudaGetLastError(), pending = tb_pending_error();
    tb_pending_error() = 0;
    return pending ? pending : launch;
}
