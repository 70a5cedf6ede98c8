// The router's choice, shared by the kernels that end in it (moe.cu, and the norm that also routes, embed_norm.cu):
//   keep the k largest logits, ties to the lower expert (the reference sorts descending, compute.rs:381)
//   w_j = exp(v_j - v_0) / sum_kept exp(v_i - v_0)    softmax over the kept logits (compute.rs:383-392)
#pragma once
#include "common.cuh"

// The k largest of lg[0..E) and their softmax weights, by one warp; lg is consumed.  Up to 32 choices stay in
// registers (choice j in lane j) and leave in one store each; more go through memory.
__device__ __forceinline__ void router_pick(float* lg, int* __restrict__ idx_out, float* __restrict__ w_out, int E, int k,
                                            int lane) {
    float v0 = 0.f, sum = 0.f, my_p = 0.f;
    int my_i = 0;
    const bool in_regs = k <= 32;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = lg[e];
            if (v > best) {   // strictly greater: the lower index stays on ties (e ascends)
                best = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (bi >= E) bi = 0;   // only when every remaining logit is -inf or NaN
        if (j == 0) v0 = best;
        const float p = expf(best - v0);
        sum += p;
        if (in_regs) {
            if (lane == j) {
                my_p = p;
                my_i = bi;
            }
        } else if (lane == 0) {
            idx_out[j] = bi;
            w_out[j] = p;
        }
        if (lane == 0) lg[bi] = __int_as_float(0x7fc00000);   // NaN compares false with everything: taken
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    if (in_regs) {
        if (lane < k) {
            idx_out[lane] = my_i;
            w_out[lane] = my_p * inv;
        }
    } else {
        for (int j = lane; j < k; j += 32) w_out[j] *= inv;
    }
}

// The same choice by ONE thread, for a few experts and choices (E * k steps): where many tokens' logits lie in shared
// memory at once, a thread per token costs far fewer instructions than a warp per token.
#define ROUTER_PICK_SERIAL_K 8
__device__ __forceinline__ void router_pick_serial(float* lg, int* __restrict__ idx_out, float* __restrict__ w_out, int E,
                                                   int k) {
    float p[ROUTER_PICK_SERIAL_K];
    float v0 = 0.f, sum = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTER_PICK_SERIAL_K; ++j) {
        if (j >= k) break;
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = 0; e < E; ++e) {
            const float v = lg[e];
            if (v > best) {   // strictly greater: the lower index stays on ties (e ascends)
                best = v;
                bi = e;
            }
        }
        if (bi >= E) bi = 0;
        if (j == 0) v0 = best;
        p[j] = expf(best - v0);
        sum += p[j];
        idx_out[j] = bi;
        lg[bi] = __int_as_float(0x7fc00000);
    }
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < ROUTER_PICK_SERIAL_K; ++j)
        if (j < k) w_out[j] = p[j] * inv;
}
