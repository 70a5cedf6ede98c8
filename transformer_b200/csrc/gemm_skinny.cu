// Skinny (few-token) matrix products for decoding, bfloat16 on the tensor cores:
//     Y[m, :] = X[row(m), :] . W[g(m)]^T        with a handful of rows m per weight matrix.
//
// A decode step multiplies a few activation rows with every weight it uses, so the step is bound
// by reading the weights once from HBM.  The weight matrix is therefore the streamed operand:
// it is the A operand (16 output columns x 16 k) of mma.sync.m16n8k16, loaded straight from
// global memory with 16-byte loads, and the tokens are the n = 8 side.  Accumulation is float.
//
//  * grouped: W holds G matrices; rows of the problem are sorted by group (the experts of
//    models/llama/common/src/compute.rs:319-330: every DISTINCT expert is read once per layer, not
//    once per (token, expert) pair as in the reference's loop); G = 1 without offsets is dense.
//  * x_rows gathers activation rows (token -> expert dispatch).
//  * row_group: the rows are NOT sorted; row m belongs to group row_group[m] (a (token, choice) pair and the
//    expert it chose).  Every block picks its group's rows out of that list by itself, which takes one load
//    and a ballot, so a decode step needs no dispatch lists at all between the router and the experts.
//  * DUAL: W[g] is [2N, K]; gate = X.W[g][n], up = X.W[g][N + n]; stores silu(gate) * up
//    (swiglu, compute.rs:324-326).
//  * output bfloat16 or float (logits, router).
//
// A block covers 16 * WN output columns of one group.  WK warps split K (warp w takes the 32-wide
// k-steps w, w + WK, ...: neighbouring warps read neighbouring 64-byte pieces of a weight row) and
// add their partial sums through shared memory; long rows use 8 x 1 warps, short ones (an expert's
// down projection) 2 x 1.  Rows are taken 8 * NT at a time.  What bounds the kernel is the number of
// bytes in flight, so every thread issues UNR k-steps of loads before it multiplies any of them.
// (Measured and dropped: staging the weights through shared memory with cp.async, persistent or
// not; cp.async.bulk.prefetch.L2 of the block's weight rows; a tcgen05 variant with the weights as
// the M = 128 side behind a 12-stage TMA ring.  All were correct and all were slower than this.)
//
// The 8 values a thread loads per row with one 16-byte load are consecutive in k; the mma's
// k-slots are fed in that order for both operands (a dot product does not care about the order of
// its terms as long as both sides agree), so no shuffle or shared-memory transpose is needed.
//
// Sizes: K a multiple of 8 (16-byte loads), any N, any number of rows; others are refused.
#include "common.cuh"

#define SK_WARPS 8
#define SK_COLS 16

struct SkinnyArgs {
    const __nv_bfloat16* X;
    const int* x_rows;
    const __nv_bfloat16* W;
    void* Y;
    const int* group_offsets;
    long long w_group_stride;
    int ldx, ldw, ldy;
    int M, N, K, G;
    const int* row_group;   // [M] group of every row, rows in any order (instead of group_offsets and x_rows), or null
    int x_div;              // with row_group: row m reads X[m / x_div] and writes Y[m]
    int w_constant;         // W is a weight: nothing the kernel before this one may have written
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Weights are read once: no L1 allocation, and each L2 miss brings 256 bytes from HBM (its neighbours
// are wanted a moment later by the next warps).
__device__ __forceinline__ uint4 ld16w(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// The same stream of W when W is itself a result of the step (the router product with the roles swapped reads the
// normalized activations as W): the read-only path promises that nothing writes the data during the kernel's
// lifetime, which does not hold while the kernel before this one may still be draining, so the plain path is taken.
__device__ __forceinline__ uint4 ld16s(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p) {
    return *reinterpret_cast<const uint4*>(p);
}

// WK warps split K, WN warps take 16 columns each: a block covers 16 * WN columns.
// UNR k-steps are loaded before any of them is multiplied, so that every thread keeps several
// 16-byte loads in flight (the step is bound by memory latency x bytes in flight otherwise).
template <int NT, bool DUAL, typename TY, int WK, int WN, int UNR>
__global__ void __launch_bounds__(WK * WN * 32) gemm_skinny_kernel(const SkinnyArgs a) {
    constexpr int ROWS = 8 * NT;
    constexpr int NMAT = DUAL ? 2 : 1;
    __shared__ float red[WN][WK][NMAT][ROWS][SK_COLS + 1];

    __shared__ int list[SK_WARPS * 32];     // with row_group: the rows of this block's group
    __shared__ unsigned list_mask[WK * WN];

    const int g_idx = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wk = warp % WK, wn = warp / WK;
    const int n0 = (blockIdx.x * WN + wn) * SK_COLS;
    const int g = lane >> 2, t = lane & 3;

    const __nv_bfloat16* Wg = a.W + (size_t)g_idx * a.w_group_stride;
    // weight rows of this thread: columns n0 + g and n0 + g + 8 (clamped; never stored when out of range)
    const int c0 = min(n0 + g, a.N - 1), c1 = min(n0 + g + 8, a.N - 1);
    const __nv_bfloat16* w0 = Wg + (size_t)c0 * a.ldw + t * 8;
    const __nv_bfloat16* w1 = Wg + (size_t)c1 * a.ldw + t * 8;
    const __nv_bfloat16* u0 = DUAL ? Wg + (size_t)(a.N + c0) * a.ldw + t * 8 : nullptr;
    const __nv_bfloat16* u1 = DUAL ? Wg + (size_t)(a.N + c1) * a.ldw + t * 8 : nullptr;
    const int k_steps = (a.K + 31) / 32;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    // Which weights this block reads does not depend on the kernel before it, so the first batch of them is in
    // flight before the wait for the activations is over.  With groups (experts) the block cannot know yet whether
    // its group has rows at all: it reads ahead only when most groups do (twice as many rows as groups), so that
    // what is read for nothing stays a few percent.
    const bool early = a.w_constant && ((!a.group_offsets && !a.row_group) || a.M >= 2 * a.G);
    uint4 wa[UNR], wb[UNR], ua[DUAL ? UNR : 1], ub[DUAL ? UNR : 1];
    if (early) {
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int k = (wk + u * WK) * 32;
            const bool live = k + t * 8 < a.K;
            wa[u] = live ? ld16w(w0 + k) : zero4;
            wb[u] = live ? ld16w(w1 + k) : zero4;
            if (DUAL) {
                ua[u] = live ? ld16w(u0 + k) : zero4;
                ub[u] = live ? ld16w(u1 + k) : zero4;
            }
        }
    }
    pdl_sync();
    int row_lo = 0, row_hi = a.M;
    const bool listed = a.row_group != nullptr;
    if (listed) {
        // a thread looks at one row per round of the block's threads (M <= SK_WARPS * 32, the size of the list);
        // rows keep their order inside the group
        int total = 0;
        for (int base = 0; base < a.M; base += WK * WN * 32) {
            const int m = base + threadIdx.x;
            const bool mine = m < a.M && a.row_group[m] == g_idx;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (lane == 0) list_mask[warp] = mask;
            __syncthreads();
            int before = 0, round = 0;
            for (int w = 0; w < WK * WN; ++w) {
                const int c = __popc(list_mask[w]);
                if (w < warp) before += c;
                round += c;
            }
            if (mine) list[total + before + __popc(mask & ((1u << lane) - 1u))] = m;
            total += round;
            __syncthreads();
        }
        row_hi = total;
    } else if (a.group_offsets) {
        row_lo = a.group_offsets[g_idx];
        row_hi = a.group_offsets[g_idx + 1];
    }
    if (row_lo >= row_hi) return;
    for (int chunk = row_lo; chunk < row_hi; chunk += ROWS) {
        const int rows = min(ROWS, row_hi - chunk);
        const int nta = (rows + 7) >> 3;
        // activation rows of this thread: token g of every n-tile
        const __nv_bfloat16* xp[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = chunk + nt * 8 + g;
            xp[nt] = nullptr;
            if (m < row_hi)
                xp[nt] = a.X + (size_t)(listed ? list[m] / a.x_div : a.x_rows ? a.x_rows[m] : m) * a.ldx + t * 8;
        }
        float acc[NMAT][NT][4];
#pragma unroll
        for (int i = 0; i < NMAT; ++i)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][nt][j] = 0.f;

        for (int s0 = wk; s0 < k_steps; s0 += WK * UNR) {
            uint4 xv[UNR][NT];
            const bool have = early && s0 == wk && chunk == row_lo;     // the batch read before the wait
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int k = (s0 + u * WK) * 32;
                const bool live = k + t * 8 < a.K;      // also false past the last step
                if (!have) {
                    if (a.w_constant) {
                        wa[u] = live ? ld16w(w0 + k) : zero4;
                        wb[u] = live ? ld16w(w1 + k) : zero4;
                        if (DUAL) {
                            ua[u] = live ? ld16w(u0 + k) : zero4;
                            ub[u] = live ? ld16w(u1 + k) : zero4;
                        }
                    } else {
                        wa[u] = live ? ld16s(w0 + k) : zero4;
                        wb[u] = live ? ld16s(w1 + k) : zero4;
                        if (DUAL) {
                            ua[u] = live ? ld16s(u0 + k) : zero4;
                            ub[u] = live ? ld16s(u1 + k) : zero4;
                        }
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) xv[u][nt] = (live && nt < nta && xp[nt]) ? ld16(xp[nt] + k) : zero4;
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if (nt < nta) {
                        const uint4 x = xv[u][nt];
                        mma_bf16_16816(acc[0][nt], wa[u].x, wb[u].x, wa[u].y, wb[u].y, x.x, x.y);
                        mma_bf16_16816(acc[0][nt], wa[u].z, wb[u].z, wa[u].w, wb[u].w, x.z, x.w);
                        if (DUAL) {
                            mma_bf16_16816(acc[1][nt], ua[u].x, ub[u].x, ua[u].y, ub[u].y, x.x, x.y);
                            mma_bf16_16816(acc[1][nt], ua[u].z, ub[u].z, ua[u].w, ub[u].w, x.z, x.w);
                        }
                    }
                }
            }
        }
        // partial sums of this warp: d0 (col g, token 2t), d1 (col g, token 2t+1), d2/d3 the same for col g+8
        __syncthreads();   // the previous chunk's reduction has been read
#pragma unroll
        for (int i = 0; i < NMAT; ++i)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                red[wn][wk][i][nt * 8 + 2 * t][g] = acc[i][nt][0];
                red[wn][wk][i][nt * 8 + 2 * t + 1][g] = acc[i][nt][1];
                red[wn][wk][i][nt * 8 + 2 * t][g + 8] = acc[i][nt][2];
                red[wn][wk][i][nt * 8 + 2 * t + 1][g + 8] = acc[i][nt][3];
            }
        __syncthreads();
        const int nb0 = blockIdx.x * WN * SK_COLS;
        for (int idx = threadIdx.x; idx < rows * SK_COLS * WN; idx += blockDim.x) {
            const int r = idx / (SK_COLS * WN), cc = idx - r * (SK_COLS * WN);
            const int w_n = cc / SK_COLS, c = cc - w_n * SK_COLS;
            if (nb0 + cc >= a.N) continue;
            float v = 0.f, v2 = 0.f;
#pragma unroll
            for (int w = 0; w < WK; ++w) {
                v += red[w_n][w][0][r][c];
                if (DUAL) v2 += red[w_n][w][NMAT - 1][r][c];
            }
            if (DUAL) v = v / (1.0f + expf(-v)) * v2;
            stf(static_cast<TY*>(a.Y) + (size_t)(listed ? list[chunk + r] : chunk + r) * a.ldy + nb0 + cc, v);
        }
    }
}

template <int NT, bool DUAL, typename TY>
static int skinny_launch_shape(const SkinnyArgs& a, cudaStream_t s) {
    // long rows: all 8 warps of a block share 16 columns and split K;
    // short rows (an expert's down projection): 2 warps on K
    if (a.K >= 2048) {
        constexpr int WK = 8, WN = 1, UNR = NT >= 4 ? 2 : 4;
        dim3 grid((a.N + SK_COLS * WN - 1) / (SK_COLS * WN), a.G);
        // up to 8 rows and one matrix per group: registers allow twice as many loads in flight per thread
        // (measured in the decode step: -1.5 us per layer on the q-k-v product; for the gate/up pair 4 is best)
        if constexpr (NT == 1 && !DUAL)
            TB_LAUNCH((gemm_skinny_kernel<NT, DUAL, TY, WK, WN, 8>), grid, WK * WN * 32, 0, s, a);
        else
            TB_LAUNCH((gemm_skinny_kernel<NT, DUAL, TY, WK, WN, UNR>), grid, WK * WN * 32, 0, s, a);
    } else {
        // 16 columns per block, as for long rows: few sequences touch few experts, and the smaller the pieces
        // of their weights, the more evenly they fall on the SMs (with 4 x 16 columns per block the whole decode
        // step at batch 8 took 2.4 % longer; 4 or 1 warps on K, or 8 loads ahead, are slower too).  Tried on the
        // gate/up pair as well (8 gate and 8 up rows per tile, half the bytes per block): no gain.
        constexpr int WK = 2, WN = 1, UNR = NT >= 4 ? 2 : 4;
        dim3 grid((a.N + SK_COLS * WN - 1) / (SK_COLS * WN), a.G);
        TB_LAUNCH((gemm_skinny_kernel<NT, DUAL, TY, WK, WN, UNR>), grid, WK * WN * 32, 0, s, a);
    }
    return tb_last_error();
}

template <int NT>
static int skinny_launch_nt(const SkinnyArgs& a, int out_kind, cudaStream_t s) {
    if (out_kind == 0) return skinny_launch_shape<NT, false, __nv_bfloat16>(a, s);
    if (out_kind == 1) return skinny_launch_shape<NT, false, float>(a, s);
    if (out_kind == 2) return skinny_launch_shape<NT, true, __nv_bfloat16>(a, s);
    return TB_ERR_ARG;
}

extern "C" {
// out_kind: 0 = bfloat16 out, 1 = float out, 2 = swiglu pair (bfloat16 out).  M is the number of rows
// over all groups; max_group_rows bounds the rows of any ONE group (for experts: the number of tokens,
// since a token picks an expert at most once) and only chooses how many rows a pass takes at once.
// w_constant: W holds weights, which no kernel writes, so a block may read its first weights before it waits for
// the kernel before it; 0 when W is itself a result (the router of prompts passes the activations as W).
int tb_gemm_skinny_bf16(const void* X, const int* x_rows, const void* W, void* Y, const int* group_offsets,
                        long long w_group_stride, int ldx, int ldw, int ldy, int M, int N, int K, int G, int out_kind,
                        int max_group_rows, const int* row_group, int x_div, int w_constant, cudaStream_t s) {
    if (M < 0 || N <= 0 || K <= 0 || G <= 0) return TB_ERR_ARG;
    if (row_group && (group_offsets || x_rows || x_div < 1)) return TB_ERR_ARG;
    if (row_group && M > SK_WARPS * 32) return TB_ERR_UNSUPPORTED;
    if (K % 8 || ldx % 8 || ldw % 8 || (w_group_stride % 8)) return TB_ERR_UNSUPPORTED;
    if (((uintptr_t)X | (uintptr_t)W) & 15) return TB_ERR_UNSUPPORTED;
    if (M == 0) return 0;
    SkinnyArgs a{(const __nv_bfloat16*)X, x_rows, (const __nv_bfloat16*)W, Y, group_offsets, w_group_stride,
                 ldx, ldw, ldy, M, N, K, G, row_group, x_div, w_constant};
    int rows = (max_group_rows > 0 && max_group_rows < M) ? max_group_rows : M;
    if (G > 1) {
        // A pass takes 8, 16 or 32 rows of a group and a thread's registers are sized by the pass (with 16 rows the
        // gate/up kernel fits one block on an SM instead of two).  So the pass is sized by what most groups hold,
        // one and a half times the mean, not by the largest group there could be: a group with more rows takes
        // another pass over its weights, which come from L2 that time.  (Decode steps of 12 to 32 sequences: 4..10 %.)
        const long long usual = (3ll * M / G + 1) / 2;
        if (usual < rows) rows = usual < 1 ? 1 : (int)usual;
    }
    if (rows <= 8) return skinny_launch_nt<1>(a, out_kind, s);
    if (rows <= 16) return skinny_launch_nt<2>(a, out_kind, s);
    return skinny_launch_nt<4>(a, out_kind, s);
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_gemm_skinny_bf16)
