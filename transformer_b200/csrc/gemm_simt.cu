// Grouped matrix product on the CUDA cores, float accumulation:  C[m, :] = A[row(m), :] . B[g(m)]^T
//
// This is the matrix product of the true 32-bit path (plain FFMA, no reduced-precision matrix
// mode) and the fallback of the bfloat16 path for shapes the tensor-core kernels refuse.
//
//  * B holds G matrices [N, K] row-major (weights as stored: y = x W^T,
//    models/llama/common/src/lib.rs:168-180); rows of the problem are sorted by group and
//    group_offsets[g] .. group_offsets[g+1] are the rows of group g (the experts of
//    models/llama/common/src/compute.rs:319-330, all tokens of one expert in one product instead of
//    a product per token).  G = 1 with no offsets is the plain product.
//  * a_rows, when given, gathers: row m reads A[a_rows[m]].
//  * DUAL: B[g] is [2N, K]; the block computes gate = A.B[g][n] and up = A.B[g][N + n] together and
//    stores silu(gate) * up  (swiglu, compute.rs:324-326), in float, rounded once.
//  Any M, N, K >= 1; edges are predicated.
#include "common.cuh"

struct GemmArgs {
    const void* A;
    const int* a_rows;
    const void* B;
    void* C;
    const int* group_offsets;
    long long b_group_stride;   // elements between B[g] and B[g+1]
    int lda, ldb, ldc;
    int M, N, K, G;
};

#define GB_N 64
#define GB_K 16

template <typename T, typename TC, int BM, bool DUAL>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const GemmArgs a) {
    pdl_sync();
    constexpr int TM = BM / 16;
    __shared__ float As[GB_K][BM + 1];
    __shared__ float Bs[GB_K][GB_N + 1];
    __shared__ float B2s[DUAL ? GB_K : 1][GB_N + 1];

    // which group and rows does this block own?
    int g = 0, row0 = 0, row_end = a.M;
    if (a.group_offsets) {
        int tile = blockIdx.x, cum = 0;
        bool found = false;
        for (g = 0; g < a.G; ++g) {
            const int lo = a.group_offsets[g], hi = a.group_offsets[g + 1];
            const int tiles = (hi - lo + BM - 1) / BM;
            if (tile < cum + tiles) {
                row0 = lo + (tile - cum) * BM;
                row_end = hi;
                found = true;
                break;
            }
            cum += tiles;
        }
        if (!found) return;
    } else {
        row0 = blockIdx.x * BM;
        if (row0 >= a.M) return;
    }
    const int n0 = blockIdx.y * GB_N;
    const T* A = static_cast<const T*>(a.A);
    const T* B = static_cast<const T*>(a.B) + (size_t)g * a.b_group_stride;

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;   // tx: columns (4 each), ty: rows (TM each)
    float acc[TM][4], acc2[DUAL ? TM : 1][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int i = 0; i < (DUAL ? TM : 1); ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = 0.f;

    // loader roles: B tile 64 x 16 -> 4 elements a thread; A tile BM x 16 -> BM*16/256 a thread
    const int lb_r = tid >> 2, lb_k = (tid & 3) * 4;
    constexpr int A_PER = BM * GB_K / 256;   // 4 (BM 64) or 1 (BM 16)
    const int la_r = (tid * A_PER) / GB_K, la_k = (tid * A_PER) % GB_K;
    const int a_row = row0 + la_r;
    const T* a_ptr = nullptr;
    if (a_row < row_end) a_ptr = A + (size_t)(a.a_rows ? a.a_rows[a_row] : a_row) * a.lda;
    const int b_row = n0 + lb_r;
    const T* b_ptr = b_row < a.N ? B + (size_t)b_row * a.ldb : nullptr;
    const T* b2_ptr = (DUAL && b_row < a.N) ? B + (size_t)(a.N + b_row) * a.ldb : nullptr;

    for (int k0 = 0; k0 < a.K; k0 += GB_K) {
#pragma unroll
        for (int i = 0; i < A_PER; ++i) {
            const int k = k0 + la_k + i;
            As[la_k + i][la_r] = (a_ptr && k < a.K) ? ldf(a_ptr + k) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lb_k + i;
            Bs[lb_k + i][lb_r] = (b_ptr && k < a.K) ? ldf(b_ptr + k) : 0.f;
            if (DUAL) B2s[lb_k + i][lb_r] = (b2_ptr && k < a.K) ? ldf(b2_ptr + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GB_K; ++k) {
            float av[TM], bv[4], b2v[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j] = Bs[k][tx * 4 + j];
                if (DUAL) b2v[j] = B2s[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] += av[i] * bv[j];
                    if (DUAL) acc2[i][j] += av[i] * b2v[j];
                }
        }
        __syncthreads();
    }

    TC* C = static_cast<TC*>(a.C);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = row0 + ty * TM + i;
        if (m >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (DUAL) {
                const float gate = v;
                v = gate / (1.0f + expf(-gate)) * acc2[i][j];
            }
            stf(C + (size_t)m * a.ldc + n, v);
        }
    }
}

template <typename T, typename TC, bool DUAL>
static int gemm_simt_launch(const GemmArgs& a, cudaStream_t s) {
    if (a.M < 0 || a.N <= 0 || a.K <= 0 || a.G <= 0) return TB_ERR_ARG;
    if (a.M == 0) return 0;
    const bool small = a.M <= 16 * a.G;
    const int bm = small ? 16 : 64;
    // every group may end in a partly filled tile
    const int tiles = a.group_offsets ? (a.M + bm - 1) / bm + a.G : (a.M + bm - 1) / bm;
    dim3 grid(tiles, (a.N + GB_N - 1) / GB_N);
    if (small)
        TB_LAUNCH((gemm_simt_kernel<T, TC, 16, DUAL>), grid, 256, 0, s, a);
    else
        TB_LAUNCH((gemm_simt_kernel<T, TC, 64, DUAL>), grid, 256, 0, s, a);
    return tb_last_error();
}

extern "C" {
// out_kind: 0 = C has the type of A and B, 1 = C is float, 2 = swiglu pair (C has the type of A)
#define TB_GEMM(NAME, T)                                                                                        \
    int NAME(const void* A, const int* a_rows, const void* B, void* C, const int* group_offsets,               \
             long long b_group_stride, int lda, int ldb, int ldc, int M, int N, int K, int G, int out_kind,    \
             cudaStream_t s) {                                                                                  \
        GemmArgs a{A, a_rows, B, C, group_offsets, b_group_stride, lda, ldb, ldc, M, N, K, G};                  \
        if (out_kind == 0) return gemm_simt_launch<T, T, false>(a, s);                                          \
        if (out_kind == 1) return gemm_simt_launch<T, float, false>(a, s);                                      \
        if (out_kind == 2) return gemm_simt_launch<T, T, true>(a, s);                                           \
        return TB_ERR_ARG;                                                                                      \
    }
TB_GEMM(tb_gemm_simt_f32, float)
TB_GEMM(tb_gemm_simt_bf16, __nv_bfloat16)
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_gemm_simt_f32)
TB_TAPE_REGISTER(tb_gemm_simt_bf16)
