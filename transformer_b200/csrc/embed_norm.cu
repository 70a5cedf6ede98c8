// Embedding gather and the fused residual-add + RMSNorm.
//
// The residual stream is float on both paths, so the residual sum is a 32-bit sum.
#include "common.cuh"
#include "router_pick.cuh"

// x[i, :] = table[tokens[i], :]   (models/llama/cuda/src/infer.rs:98-104 copies row by row)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ x, int d) {
    pdl_sync();
    const int i = blockIdx.x;
    const T* src = table + (size_t)tokens[i] * d;
    float* dst = x + (size_t)i * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = ldf(src + c);
}

// Row r = rows ? rows[i] : i.
//   v = x[r] + delta(r)                                    float sum
//   if (!rows && there is a delta) x[r] = v                the stream is updated in place
//   y[i] = v / sqrt(mean(v^2) + eps) * w                   statistics in float, one rounding to T
// delta(r) is delta[r] (a part's output), or, when wy is given, the weighted sum of rows of wy:
//   sum_j topk_w[r, j] * wy[pair_row[r * k + j]]           j ascending, in float
// which is the combine of the experts' outputs (compute.rs:329-330) fused into the norm that follows.
// (call sites of rms_norm: models/llama/common/src/compute.rs:207,275,362; the residual sum is the
//  beta = 1 of the output products, :270,:330.)
// Bytes that the kernel AFTER this one reads first and that are weights (a router's matrix: 128 KB that one block
// per token would otherwise wait for from HBM): the last block asks for them to be brought into L2, before it
// waits for the kernel before it.  Weights do not change, so asking early is always safe.
__device__ __forceinline__ void warm_l2(const void* warm, int warm_bytes) {
    if (warm && blockIdx.x == gridDim.x - 1)
        for (int off = threadIdx.x * 128; off < warm_bytes; off += blockDim.x * 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char*>(warm) + off));
}

template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                   const T* __restrict__ wy, const int* __restrict__ pair_row,
                                   const float* __restrict__ topk_w, int k,
                                   const int* __restrict__ rows, const float* __restrict__ w,
                                   float eps, T* __restrict__ y, int d, const void* warm, int warm_bytes) {
    warm_l2(warm, warm_bytes);
    pdl_sync();
    __shared__ float red[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* xr = x + (size_t)r * d;
    const T* dr = delta ? delta + (size_t)r * d : nullptr;
    const bool has_delta = dr != nullptr || wy != nullptr;
    const bool write_back = (rows == nullptr) && has_delta;
    auto delta_at = [&](int c) -> float {
        if (dr) return ldf(dr + c);
        float acc = 0.f;
        for (int j = 0; j < k; ++j)
            acc += topk_w[(size_t)r * k + j] * ldf(wy + (size_t)pair_row[(size_t)r * k + j] * d + c);
        return acc;
    };
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = xr[c];
        if (has_delta) v += delta_at(c);
        if (write_back) xr[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    T* yr = y + (size_t)i * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = xr[c];
        if (has_delta && !write_back) v += delta_at(c);
        stf(yr + c, v * rs * w[c]);
    }
}

// The same, eight values at a time with 16-byte accesses, the row kept in registers between the two
// passes.  For widths that are a multiple of 8 and at most threads * 8 * NORM_CHUNKS.
#define NORM_CHUNKS 4
// Two forms: for a few rows (decoding) 512 threads per row and the weights read before the dependency wait; for
// many rows (prompts) 256 lean threads, four blocks to an SM, since there the kernel is bound by memory traffic
// and the registers of the early read would halve what is resident.
// What a feed-forward may ask the norm before it to do in the same kernel (TAIL): the router of the row it has
// just normalized, i.e. the row's k experts and their weights, by the rules of router_kernel.  The row goes to
// shared memory as it goes to y (rounded to T), one warp per expert takes its dot product with the router's
// matrix (whose first part it has read before the dependency wait), one warp picks.  A router kernel of its
// own would first wait for this kernel to end and then read the row back.
template <typename T> struct RouterTail {
    const T* w;        // [E, d], or null: none
    int E, k;
    int* idx;          // [rows, k]
    float* wts;        // [rows, k]
};

template <typename T, int NORM_THREADS, bool EARLY, bool TAIL>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ wy,
                       const int* __restrict__ pair_row, const float* __restrict__ topk_w, int k,
                       const int* __restrict__ rows, const float* __restrict__ w, float eps, T* __restrict__ y,
                       int d, const void* warm, int warm_bytes, const RouterTail<T> tail) {
    constexpr int EPL = Vec16<T>::N, UN = 8;
    extern __shared__ __align__(16) unsigned char tail_smem[];      // TAIL: the row as T [d], then logits [E]
    uint4 first[TAIL ? UN : 1];
    if (TAIL) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (warp < tail.E) {
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int c = (lane + u * 32) * EPL;
                first[u] = make_uint4(0u, 0u, 0u, 0u);
                if (c < d) first[u] = *reinterpret_cast<const uint4*>(tail.w + (size_t)warp * d + c);
            }
        }
    }
    warm_l2(warm, warm_bytes);
    // this kernel's own weights do not depend on the kernel before it either: they are in registers by the time
    // the wait is over (they are read once per layer and have left L2 since the last step)
    float ww[EARLY ? NORM_CHUNKS : 1][8];
    if (EARLY) {
#pragma unroll
        for (int j = 0; j < NORM_CHUNKS; ++j) {
            const int c = (threadIdx.x + j * NORM_THREADS) * 8;
            if (c < d) load8(w + c, ww[j]);
        }
    }
    pdl_sync();
    __shared__ float red[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* xr = x + (size_t)r * d;
    const T* dr = delta ? delta + (size_t)r * d : nullptr;
    const bool has_delta = dr != nullptr || wy != nullptr;
    const bool write_back = (rows == nullptr) && has_delta;
    float v[NORM_CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_CHUNKS; ++j) {
        const int c = (threadIdx.x + j * NORM_THREADS) * 8;
        if (c < d) {
            load8(xr + c, v[j]);
            if (dr) {
                float t[8];
                load8(dr + c, t);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j][e] += t[e];
            } else if (wy) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int q = 0; q < k; ++q) {
                    float t[8];
                    load8(wy + (size_t)pair_row[(size_t)r * k + q] * d + c, t);
                    const float wq = topk_w[(size_t)r * k + q];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] += wq * t[e];
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j][e] += acc[e];
            }
            if (write_back) store8(xr + c, v[j]);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[j][e] * v[j][e];
        }
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    T* yr = y + (size_t)i * d;
#pragma unroll
    for (int j = 0; j < NORM_CHUNKS; ++j) {
        const int c = (threadIdx.x + j * NORM_THREADS) * 8;
        if (c < d) {
            float o[8];
            if (!EARLY) load8(w + c, ww[0]);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = v[j][e] * rs * ww[EARLY ? j : 0][e];
            store8(yr + c, o);
            if (TAIL) store8(reinterpret_cast<T*>(tail_smem) + c, o);
        }
    }
    if (!TAIL) return;
    __syncthreads();
    const T* ys = reinterpret_cast<const T*>(tail_smem);
    float* lg = reinterpret_cast<float*>(tail_smem + (size_t)d * sizeof(T));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = warp; e < tail.E; e += NORM_THREADS / 32) {
        const T* we = tail.w + (size_t)e * d;
        float acc = 0.f;
        for (int c0 = lane * EPL; c0 < d; c0 += 32 * EPL * UN) {
            uint4 xv[UN], wv[UN];
            const bool have = e == warp && c0 == lane * EPL;     // the batch read before the wait
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int c = c0 + u * 32 * EPL;
                xv[u] = wv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (c < d) {
                    xv[u] = *reinterpret_cast<const uint4*>(ys + c);
                    wv[u] = have ? first[u] : *reinterpret_cast<const uint4*>(we + c);
                }
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                float xf[EPL], wf[EPL];
                Vec16<T>::unpack(xv[u], xf);
                Vec16<T>::unpack(wv[u], wf);
#pragma unroll
                for (int q = 0; q < EPL; ++q) acc += xf[q] * wf[q];
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) lg[e] = acc;
    }
    __syncthreads();
    if (warp == 0) router_pick(lg, tail.idx + (size_t)i * tail.k, tail.wts + (size_t)i * tail.k, tail.E, tail.k, lane);
}

template <typename T>
__global__ void embed_vec_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ x,
                                 int d) {
    pdl_sync();
    const int i = blockIdx.x;
    const T* src = table + (size_t)tokens[i] * d;
    float* dst = x + (size_t)i * d;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
        float f[8];
        load8(src + c, f);
        store8(dst + c, f);
    }
}

template <typename T>
static int embed_launch(const int* tokens, const void* table, float* x, int nt, int d, cudaStream_t s) {
    if (nt < 0 || d <= 0) return TB_ERR_ARG;
    if (nt == 0) return 0;
    if (d % 8 == 0)
        TB_LAUNCH((embed_vec_kernel<T>), nt, 128, 0, s, tokens, (const T*)table, x, d);
    else
        TB_LAUNCH((embed_kernel<T>), nt, 256, 0, s, tokens, (const T*)table, x, d);
    return tb_last_error();
}
template <typename T>
static int add_rmsnorm_launch(float* x, const void* delta, const void* wy, const int* pair_row,
                              const float* topk_w, int k, const int* rows, const float* w, float eps,
                              void* y, int n_out, int d, const void* warm, int warm_bytes, cudaStream_t s,
                              RouterTail<T> tail = RouterTail<T>{nullptr, 0, 0, nullptr, nullptr}) {
    if (n_out < 0 || d <= 0) return TB_ERR_ARG;
    if (wy && (delta || !pair_row || !topk_w || k <= 0)) return TB_ERR_ARG;
    if (tail.w && (tail.E <= 0 || tail.k <= 0 || tail.k > tail.E || !tail.idx || !tail.wts)) return TB_ERR_ARG;
    if (n_out == 0) return 0;
    if (tail.w) {
        // the form that also routes: a few rows, a width of 16-byte pieces, the row and the logits in 40 KB
        const size_t smem = (size_t)d * sizeof(T) + (size_t)tail.E * sizeof(float);
        if (d % 8 || d > 512 * 8 * NORM_CHUNKS || n_out > 256 || smem > 40 * 1024 ||
            (reinterpret_cast<uintptr_t>(tail.w) & 15))
            return TB_ERR_UNSUPPORTED;           // the caller runs the router by itself
        TB_LAUNCH((add_rmsnorm_vec_kernel<T, 512, true, true>), n_out, 512, smem, s, x, (const T*)delta, (const T*)wy,
                  pair_row, topk_w, k, rows, w, eps, (T*)y, d, nullptr, 0, tail);
        return tb_last_error();
    }
    if (d % 8 == 0 && n_out <= 256 && d <= 512 * 8 * NORM_CHUNKS) {
        TB_LAUNCH((add_rmsnorm_vec_kernel<T, 512, true, false>), n_out, 512, 0, s, x, (const T*)delta, (const T*)wy,
                  pair_row, topk_w, k, rows, w, eps, (T*)y, d, warm, warm_bytes, tail);
        return tb_last_error();
    }
    if (d % 8 == 0 && d <= 256 * 8 * NORM_CHUNKS) {
        TB_LAUNCH((add_rmsnorm_vec_kernel<T, 256, false, false>), n_out, 256, 0, s, x, (const T*)delta, (const T*)wy,
                  pair_row, topk_w, k, rows, w, eps, (T*)y, d, warm, warm_bytes, tail);
        return tb_last_error();
    }
    int threads = d >= 2048 ? 512 : 256;
    TB_LAUNCH((add_rmsnorm_kernel<T>), n_out, threads, 0, s, x, (const T*)delta, (const T*)wy, pair_row, topk_w, k, rows, w, eps,
                                                   (T*)y, d, warm, warm_bytes);
    return tb_last_error();
}

extern "C" {
int tb_embed_f32(const int* tokens, const void* table, float* x, int nt, int d, cudaStream_t s) {
    return embed_launch<float>(tokens, table, x, nt, d, s);
}
int tb_embed_bf16(const int* tokens, const void* table, float* x, int nt, int d, cudaStream_t s) {
    return embed_launch<__nv_bfloat16>(tokens, table, x, nt, d, s);
}
// warm / warm_bytes: weights that the next kernel reads first, to be asked into L2 meanwhile (or null / 0).
int tb_add_rmsnorm_f32(float* x, const void* delta, const void* wy, const int* pair_row, const float* topk_w, int k,
                       const int* rows, const float* w, float eps, void* y, int n_out, int d, const void* warm,
                       int warm_bytes, cudaStream_t s) {
    return add_rmsnorm_launch<float>(x, delta, wy, pair_row, topk_w, k, rows, w, eps, y, n_out, d, warm, warm_bytes, s);
}
int tb_add_rmsnorm_bf16(float* x, const void* delta, const void* wy, const int* pair_row, const float* topk_w, int k,
                        const int* rows, const float* w, float eps, void* y, int n_out, int d, const void* warm,
                        int warm_bytes, cudaStream_t s) {
    return add_rmsnorm_launch<__nv_bfloat16>(x, delta, wy, pair_row, topk_w, k, rows, w, eps, y, n_out, d, warm,
                                             warm_bytes, s);
}
// The same, and the router of the rows just normalized in the same kernel (router_w [E, d]; each row's route_k
// experts and weights into route_idx / route_w [n_out, route_k]).  TB_ERR_UNSUPPORTED for what it does not take
// (many rows, widths that are no multiple of 8 or do not fit shared memory): nothing has been done then.
int tb_add_rmsnorm_router_f32(float* x, const void* delta, const void* wy, const int* pair_row, const float* topk_w,
                              int k, const int* rows, const float* w, float eps, void* y, const void* router_w,
                              int* route_idx, float* route_w, int n_out, int d, int E, int route_k, cudaStream_t s) {
    if (!router_w) return TB_ERR_ARG;
    return add_rmsnorm_launch<float>(x, delta, wy, pair_row, topk_w, k, rows, w, eps, y, n_out, d, nullptr, 0, s,
                                     RouterTail<float>{(const float*)router_w, E, route_k, route_idx, route_w});
}
int tb_add_rmsnorm_router_bf16(float* x, const void* delta, const void* wy, const int* pair_row, const float* topk_w,
                               int k, const int* rows, const float* w, float eps, void* y, const void* router_w,
                               int* route_idx, float* route_w, int n_out, int d, int E, int route_k, cudaStream_t s) {
    if (!router_w) return TB_ERR_ARG;
    return add_rmsnorm_launch<__nv_bfloat16>(
        x, delta, wy, pair_row, topk_w, k, rows, w, eps, y, n_out, d, nullptr, 0, s,
        RouterTail<__nv_bfloat16>{(const __nv_bfloat16*)router_w, E, route_k, route_idx, route_w});
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_embed_f32)
TB_TAPE_REGISTER(tb_embed_bf16)
TB_TAPE_REGISTER(tb_add_rmsnorm_f32)
TB_TAPE_REGISTER(tb_add_rmsnorm_bf16)
TB_TAPE_REGISTER(tb_add_rmsnorm_router_f32)
TB_TAPE_REGISTER(tb_add_rmsnorm_router_bf16)
