// Mixture-of-experts routing on the device: router logits + top-k + weights, the token -> expert
// dispatch lists, and the weighted combine.
//
// The reference copies the router logits to the host in every layer, sorts them there and then
// loops over tokens and experts (models/llama/common/src/compute.rs:294-333,375-394).  Here nothing
// leaves the device: a step has no synchronisation point.
#include "common.cuh"
#include "router_pick.cuh"

#define ROUTER_WARPS 16
#define ROUTER_MAX_E 1024

// One block per token, one warp per expert (warps loop when there are more experts than warps).
//   logits[e] = x1 . Wr[e]                       float accumulation, kept in float
//   keep the k largest, ties to the lower expert (the reference sorts descending, compute.rs:381)
//   w_j = exp(v_j - v_0) / sum_kept exp(v_i - v_0)    softmax over the kept logits (compute.rs:383-392)
// topk_idx / topk_w are in descending-logit order.
__device__ void dispatch_lists(const int* topk_idx, int* __restrict__ group_offsets, int* __restrict__ sorted_token,
                               int* __restrict__ pair_row, int M, int k, int E, int* count, int* cursor);

// With `lists` set, the block that finishes last (counted in lists.done, which it leaves at zero again) also
// builds the dispatch lists from every token's choice: one kernel less between the router and the experts.
struct DispatchLists {
    int* group_offsets;
    int* sorted_token;
    int* pair_row;
    unsigned* done;
};

template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_kernel(const T* __restrict__ x1, const T* __restrict__ wr, int* __restrict__ topk_idx,
              float* __restrict__ topk_w, float* __restrict__ logits_out, int nt, int d, int E, int k,
              const DispatchLists lists) {
    constexpr int EPL = Vec16<T>::N;
    constexpr int UN = 8;
    extern __shared__ float lg[];   // [E]
    __shared__ int count[ROUTER_MAX_E + 1];
    __shared__ int cursor[ROUTER_MAX_E];
    __shared__ bool last_block;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const T* xr = x1 + (size_t)t * d;
    const bool vec = (d % EPL) == 0;
    // The router's weights do not depend on the kernel before this one: the first batch of this warp's first
    // expert is in registers by the time the wait for the activations is over.
    uint4 first[UN];
    if (vec && warp < E) {
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int c = (lane + u * 32) * EPL;
            first[u] = make_uint4(0u, 0u, 0u, 0u);
            if (c < d) first[u] = *reinterpret_cast<const uint4*>(wr + (size_t)warp * d + c);
        }
    }
    pdl_sync();
    for (int e = warp; e < E; e += nwarps) {
        const T* w = wr + (size_t)e * d;
        float acc = 0.f;
        if (vec) {
            // eight 16-byte loads of each operand are asked for before any is used: the dot product of one
            // row is short, so what it costs is memory latency, paid once per batch instead of once per load
            for (int c0 = lane * EPL; c0 < d; c0 += 32 * EPL * UN) {
                uint4 xv[UN], wv[UN];
                const bool have = e == warp && c0 == lane * EPL;     // the batch read before the wait
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    const int c = c0 + u * 32 * EPL;
                    xv[u] = wv[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (c < d) {
                        xv[u] = *reinterpret_cast<const uint4*>(xr + c);
                        wv[u] = have ? first[u] : *reinterpret_cast<const uint4*>(w + c);
                    }
                }
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    float xf[EPL], wf[EPL];
                    Vec16<T>::unpack(xv[u], xf);
                    Vec16<T>::unpack(wv[u], wf);
#pragma unroll
                    for (int i = 0; i < EPL; ++i) acc += xf[i] * wf[i];
                }
            }
        } else {
            for (int c = lane; c < d; c += 32) acc += ldf(xr + c) * ldf(w + c);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            lg[e] = acc;
            if (logits_out) logits_out[(size_t)t * E + e] = acc;
        }
    }
    __syncthreads();
    if (warp != 0 && !lists.done) return;
    if (warp == 0) router_pick(lg, topk_idx + (size_t)t * k, topk_w + (size_t)t * k, E, k, lane);
    if (!lists.done) return;
    __threadfence();          // this token's choice is visible before the count says so
    __syncthreads();
    if (threadIdx.x == 0) {
        last_block = atomicAdd(lists.done, 1u) == gridDim.x - 1;
        if (last_block) *lists.done = 0;
    }
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    dispatch_lists(topk_idx, lists.group_offsets, lists.sorted_token, lists.pair_row, nt * k, k, E, count, cursor);
}

// Many tokens, bfloat16: the logits of 16 tokens x up to 64 experts are tiles of mma.sync.m16n8k16, accumulated in
// float.  A block's eight warps split the width; every lane reads 16 bytes (8 values) of its token's row and of its
// expert's row per 32 columns and feeds them to two k-steps: which of the 16 k-slots of an instruction a value sits
// in does not matter as long as the token's and the expert's value of one column sit in the same slot.  The
// activations are read once (the per-token kernel above reads the router's matrix once per token).  The warps' sums
// meet in shared memory, are added in a fixed order, and the same router_pick finishes each token, a warp per token.
#define RR_ROWS 16

template <int NT, int RR_WARPS>   // tiles of 8 experts; warps that split the width
__global__ void __launch_bounds__(RR_WARPS * 32)
router_rows_kernel(const __nv_bfloat16* __restrict__ x1, const __nv_bfloat16* __restrict__ wr,
                   int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ logits_out, int nt, int d,
                   int E, int k, const DispatchLists lists) {
    constexpr int EP = 8 * NT;
    constexpr int U = NT <= 2 ? 4 : NT == 4 ? 2 : 1;     // chunks of 32 columns in flight per warp
    __shared__ float part[RR_WARPS][RR_ROWS][EP + 1];
    __shared__ int count[ROUTER_MAX_E + 1];
    __shared__ int cursor[ROUTER_MAX_E];
    __shared__ bool last_block;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int row0 = blockIdx.x * RR_ROWS;
    const int chunks = d / 32;
    const bool lo = row0 + g < nt, hi = row0 + g + 8 < nt;
    const __nv_bfloat16* xa = x1 + (size_t)(row0 + g) * d + t4 * 8;
    const __nv_bfloat16* xb = xa + (size_t)8 * d;
    const __nv_bfloat16* wb = wr + (size_t)g * d + t4 * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    // the router's rows of this warp's first chunks do not depend on the kernel before: read before the wait
    uint4 wv[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = warp + u * RR_WARPS;
#pragma unroll
        for (int j = 0; j < NT; ++j)
            wv[u][j] = (c < chunks && 8 * j + g < E) ? *reinterpret_cast<const uint4*>(wb + (size_t)8 * j * d + c * 32) : zero;
    }
    pdl_sync();
    for (int c0 = warp; c0 < chunks; c0 += RR_WARPS * U) {
        uint4 av[U], bv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + u * RR_WARPS;
            av[u] = (lo && c < chunks) ? *reinterpret_cast<const uint4*>(xa + c * 32) : zero;
            bv[u] = (hi && c < chunks) ? *reinterpret_cast<const uint4*>(xb + c * 32) : zero;
            if (c0 != warp) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
                    wv[u][j] = (c < chunks && 8 * j + g < E)
                                   ? *reinterpret_cast<const uint4*>(wb + (size_t)8 * j * d + c * 32) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                asm volatile(
                    "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                    : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                    : "r"(av[u].x), "r"(bv[u].x), "r"(av[u].y), "r"(bv[u].y), "r"(wv[u][j].x), "r"(wv[u][j].y));
                asm volatile(
                    "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                    : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                    : "r"(av[u].z), "r"(bv[u].z), "r"(av[u].w), "r"(bv[u].w), "r"(wv[u][j].z), "r"(wv[u][j].w));
            }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        part[warp][g][8 * j + 2 * t4] = acc[j][0];
        part[warp][g][8 * j + 2 * t4 + 1] = acc[j][1];
        part[warp][g + 8][8 * j + 2 * t4] = acc[j][2];
        part[warp][g + 8][8 * j + 2 * t4 + 1] = acc[j][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < RR_ROWS * EP; i += RR_WARPS * 32) {
        const int r = i / EP, e = i - r * EP;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < RR_WARPS; ++w) v += part[w][r][e];
        part[0][r][e] = v;
        if (logits_out && row0 + r < nt && e < E) logits_out[(size_t)(row0 + r) * E + e] = v;
    }
    __syncthreads();
    if (k <= ROUTER_PICK_SERIAL_K && E * k <= 256) {
        const int t = row0 + (int)threadIdx.x;
        if (threadIdx.x < RR_ROWS && t < nt)
            router_pick_serial(&part[0][threadIdx.x][0], topk_idx + (size_t)t * k, topk_w + (size_t)t * k, E, k);
    } else {
        for (int r = warp; r < RR_ROWS; r += RR_WARPS) {
            const int t = row0 + r;
            if (t < nt) router_pick(&part[0][r][0], topk_idx + (size_t)t * k, topk_w + (size_t)t * k, E, k, lane);
        }
    }
    if (!lists.done) return;
    __threadfence();          // these tokens' choices are visible before the count says so
    __syncthreads();
    if (threadIdx.x == 0) {
        last_block = atomicAdd(lists.done, 1u) == gridDim.x - 1;
        if (last_block) *lists.done = 0;
    }
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    dispatch_lists(topk_idx, lists.group_offsets, lists.sorted_token, lists.pair_row, nt * k, k, E, count, cursor);
}

// One block builds the dispatch lists for M = nt * k (token, choice) pairs:
//   group_offsets[e] .. group_offsets[e+1]   rows of expert e in the sorted order
//   sorted_token[r]                          token whose activation row r reads
//   pair_row[t * k + j]                      row r that holds the pair's result
// The order of the rows inside one expert is not fixed; no result depends on it (every row of a
// product is computed alone, and the combine reads rows through pair_row in the order of j).
__device__ void dispatch_lists(const int* topk_idx, int* __restrict__ group_offsets, int* __restrict__ sorted_token,
                               int* __restrict__ pair_row, int M, int k, int E, int* count, int* cursor) {
    // One block, two passes over the pairs, and what they cost is the latency of reading each pair's expert: the
    // reads of eight rounds are asked for together, before any of them is used (a prompt of 2,048 tokens is eight
    // rounds of a 1,024-thread block: 9 -> 5 us for this kernel, which nothing runs beside).
    constexpr int U = 8;
    for (int e = threadIdx.x; e <= E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p0 = threadIdx.x; p0 < M; p0 += U * blockDim.x) {
        int ex[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = p0 + u * blockDim.x;
            ex[u] = p < M ? __ldcg(topk_idx + p) : -1;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (ex[u] >= 0) atomicAdd(&count[ex[u]], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = count[e];
            cursor[e] = run;
            group_offsets[e] = run;
            run += c;
        }
        group_offsets[E] = run;
    }
    __syncthreads();
    for (int p0 = threadIdx.x; p0 < M; p0 += U * blockDim.x) {
        int ex[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = p0 + u * blockDim.x;
            ex[u] = p < M ? __ldcg(topk_idx + p) : -1;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = p0 + u * blockDim.x;
            if (ex[u] >= 0) {
                const int r = atomicAdd(&cursor[ex[u]], 1);
                sorted_token[r] = p / k;
                pair_row[p] = r;
            }
        }
    }
}

__global__ void __launch_bounds__(1024)
moe_dispatch_kernel(const int* __restrict__ topk_idx, int* __restrict__ group_offsets,
                    int* __restrict__ sorted_token, int* __restrict__ pair_row, int M, int k, int E) {
    pdl_sync();
    __shared__ int count[ROUTER_MAX_E + 1];
    __shared__ int cursor[ROUTER_MAX_E];
    dispatch_lists(topk_idx, group_offsets, sorted_token, pair_row, M, k, E, count, cursor);
}

// delta[t, :] = sum_j w[t, j] * y[pair_row[t, j], :]   in float, j ascending = descending logit,
// the order in which the reference accumulates the experts (compute.rs:319-330); one rounding.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ pair_row,
                                   const float* __restrict__ topk_w, T* __restrict__ delta, int d, int k) {
    pdl_sync();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < k; ++j)
            acc += topk_w[(size_t)t * k + j] * ldf(y + (size_t)pair_row[(size_t)t * k + j] * d + c);
        stf(delta + (size_t)t * d + c, acc);
    }
}

template <typename T>
static int router_launch(const void* x1, const void* wr, int* topk_idx, float* topk_w, float* logits_out, int nt,
                         int d, int E, int k, const DispatchLists& lists, cudaStream_t s) {
    if (nt < 0 || d <= 0 || E <= 0 || k <= 0 || k > E) return TB_ERR_ARG;
    if (E > ROUTER_MAX_E) return TB_ERR_UNSUPPORTED;
    if (nt == 0) return 0;
    int warps = E < ROUTER_WARPS ? E : ROUTER_WARPS;
    if (nt >= 1024 && warps > 4) warps = 4;   // many tokens: fewer, longer-lived warps per token
    TB_LAUNCH((router_kernel<T>), nt, warps * 32, (size_t)E * sizeof(float), s, 
        (const T*)x1, (const T*)wr, topk_idx, topk_w, logits_out, nt, d, E, k, lists);
    return tb_last_error();
}
template <typename T>
static int combine_launch(const void* y, const int* pair_row, const float* topk_w, void* delta, int nt, int d,
                          int k, cudaStream_t s) {
    if (nt < 0 || d <= 0 || k <= 0) return TB_ERR_ARG;
    if (nt == 0) return 0;
    TB_LAUNCH((moe_combine_kernel<T>), nt, 256, 0, s, (const T*)y, pair_row, topk_w, (T*)delta, d, k);
    return tb_last_error();
}

extern "C" {
// With `done` (one zeroed word that the kernel leaves zeroed) the dispatch lists of tb_moe_dispatch are built
// by the same kernel; the three list pointers are then required.
int tb_router_f32(const void* x1, const void* wr, int* topk_idx, float* topk_w, float* logits_out, int* group_offsets,
                  int* sorted_token, int* pair_row, unsigned* done, int nt, int d, int E, int k, cudaStream_t s) {
    if (done && !(group_offsets && sorted_token && pair_row)) return TB_ERR_ARG;
    return router_launch<float>(x1, wr, topk_idx, topk_w, logits_out, nt, d, E, k,
                                DispatchLists{group_offsets, sorted_token, pair_row, done}, s);
}
int tb_router_bf16(const void* x1, const void* wr, int* topk_idx, float* topk_w, float* logits_out, int* group_offsets,
                   int* sorted_token, int* pair_row, unsigned* done, int nt, int d, int E, int k, cudaStream_t s) {
    if (done && !(group_offsets && sorted_token && pair_row)) return TB_ERR_ARG;
    return router_launch<__nv_bfloat16>(x1, wr, topk_idx, topk_w, logits_out, nt, d, E, k,
                                        DispatchLists{group_offsets, sorted_token, pair_row, done}, s);
}
// Router for many tokens (bfloat16, up to 64 experts, a width that is a multiple of 32); `done` as in tb_router_*.
int tb_router_rows_bf16(const void* x1, const void* wr, int* topk_idx, float* topk_w, float* logits_out,
                        int* group_offsets, int* sorted_token, int* pair_row, unsigned* done, int nt, int d, int E,
                        int k, cudaStream_t s) {
    if (nt < 0 || d <= 0 || E <= 0 || k <= 0 || k > E) return TB_ERR_ARG;
    if (done && !(group_offsets && sorted_token && pair_row)) return TB_ERR_ARG;
    if (E > 64 || d % 32 || (((uintptr_t)x1 | (uintptr_t)wr) & 15)) return TB_ERR_UNSUPPORTED;
    if (nt == 0) return 0;
    const DispatchLists lists{group_offsets, sorted_token, pair_row, done};
    const int grid = (nt + RR_ROWS - 1) / RR_ROWS;
    const __nv_bfloat16* x = (const __nv_bfloat16*)x1;
    const __nv_bfloat16* w = (const __nv_bfloat16*)wr;
    if (E <= 8) TB_LAUNCH((router_rows_kernel<1, 16>), grid, 512, 0, s, x, w, topk_idx, topk_w, logits_out, nt, d, E, k, lists);
    else if (E <= 16) TB_LAUNCH((router_rows_kernel<2, 16>), grid, 512, 0, s, x, w, topk_idx, topk_w, logits_out, nt, d, E, k, lists);
    else if (E <= 32) TB_LAUNCH((router_rows_kernel<4, 16>), grid, 512, 0, s, x, w, topk_idx, topk_w, logits_out, nt, d, E, k, lists);
    else TB_LAUNCH((router_rows_kernel<8, 8>), grid, 256, 0, s, x, w, topk_idx, topk_w, logits_out, nt, d, E, k, lists);
    return tb_last_error();
}
int tb_moe_dispatch(const int* topk_idx, int* group_offsets, int* sorted_token, int* pair_row, int M, int k, int E,
                    cudaStream_t s) {
    if (M < 0 || k <= 0 || E <= 0) return TB_ERR_ARG;
    if (E > ROUTER_MAX_E) return TB_ERR_UNSUPPORTED;
    TB_LAUNCH((moe_dispatch_kernel), 1, 1024, 0, s, topk_idx, group_offsets, sorted_token, pair_row, M, k, E);
    return tb_last_error();
}
int tb_moe_combine_f32(const void* y, const int* pair_row, const float* topk_w, void* delta, int nt, int d, int k,
                       cudaStream_t s) {
    return combine_launch<float>(y, pair_row, topk_w, delta, nt, d, k, s);
}
int tb_moe_combine_bf16(const void* y, const int* pair_row, const float* topk_w, void* delta, int nt, int d, int k,
                        cudaStream_t s) {
    return combine_launch<__nv_bfloat16>(y, pair_row, topk_w, delta, nt, d, k, s);
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_router_f32)
TB_TAPE_REGISTER(tb_router_bf16)
TB_TAPE_REGISTER(tb_router_rows_bf16)
TB_TAPE_REGISTER(tb_moe_dispatch)
TB_TAPE_REGISTER(tb_moe_combine_f32)
TB_TAPE_REGISTER(tb_moe_combine_bf16)
