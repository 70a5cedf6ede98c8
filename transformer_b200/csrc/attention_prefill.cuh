// Causal attention for prompts over the paged cache, bfloat16, on the tensor cores.
//
// Same mathematics as the general kernel (attention_kernels.cuh): score = q.k / sqrt(dh) over the
// positions <= the token's own (models/llama/common/src/compute.rs:243-264), softmax statistics and
// the output accumulator in float, no score matrix in memory (the reference sizes a workspace for
// the whole [nh, seq, att_len] matrix, compute.rs:172).
//
// A block = one tile of up to 64 query tokens of ONE sequence x one query head; its 4 warps own 16
// query rows each.  It walks the sequence's pages (64 keys each): K and V of a page are copied to
// shared memory with cp.async (K double buffered, V fetched behind the score product; XOR swizzle), S = Q K^T and O += P V run
// as mma.sync.m16n8k16 with ldmatrix-fed fragments, and the softmax is the online form kept in
// registers.  The step's own keys are already in the cache.
// Head sizes that are a multiple of 16 up to 256 (a row of shared memory is padded to a multiple of 64 values so
// that the XOR swizzle stays inside it); others are answered with TB_ERR_UNSUPPORTED and the caller takes the
// general kernel.  The instantiations are spread over two source files so that they compile side by side.
#pragma once
#include "common.cuh"

#define AP_BM 64
#define AP_BN 64
#define AP_THREADS 128

struct PrefillArgs {
    const __nv_bfloat16* q;    // [nt, q_stride]
    __nv_bfloat16* out;        // [nt, nh * dh]
    const __nv_bfloat16* kc;   // [pages, nkvh, TB_PAGE, dh]
    const __nv_bfloat16* vc;
    const int* tile_seq;
    const int* tile_t0;
    const int* tile_nq;
    const int* tok_pos;
    const int* page_table;
    int tiles, max_pages, q_stride, nh, nkvh;
    float scale_log2e;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// values of a row of shared memory: dh rounded up to a multiple of 64 (8 chunks of 16 bytes)
__host__ __device__ constexpr int ap_row(int dh) { return (dh + 63) / 64 * 64; }
// blocks that the registers of a block of this head size leave room for on an SM (the output accumulator is dh/2
// floats per thread)
__host__ __device__ constexpr int ap_blocks(int dh) { return dh <= 128 ? 3 : dh <= 192 ? 2 : 1; }

template <int DH>
__global__ void __launch_bounds__(AP_THREADS, ap_blocks(DH)) attention_prefill_kernel(const PrefillArgs a) {
    pdl_sync();
    constexpr int CH = DH / 8;                 // 16-byte chunks in a row
    constexpr int RS = ap_row(DH);             // values from one row of shared memory to the next
    constexpr int TILE = AP_BN * RS;           // elements of one K or V tile
    extern __shared__ __align__(128) __nv_bfloat16 sm[];
    __nv_bfloat16* sq = sm;                    // [64][RS]
    __nv_bfloat16* sk = sq + AP_BM * RS;       // [2][64][RS]  K of tile j and of tile j + 1
    __nv_bfloat16* sv = sk + 2 * TILE;         // [64][RS]     V of tile j only: three blocks fit on an SM (dh <= 128)
    // element offset of (row, 16-byte chunk) under the XOR swizzle
    auto swz = [](int row, int chunk) { return row * RS + ((chunk ^ (row & 7)) << 3); };

    const int tile = a.tiles - 1 - (int)blockIdx.x;     // the last tiles of a sequence see the most keys: start them first
    const int h = blockIdx.y;
    const int g = h / (a.nh / a.nkvh);
    const int b = a.tile_seq[tile], t0 = a.tile_t0[tile], nq = a.tile_nq[tile];
    const int pos_first = a.tok_pos[t0];
    const int pos_last = pos_first + nq - 1;
    const int n_tiles = pos_last / AP_BN + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tid4 = lane & 3;
    const int* pt = a.page_table + (size_t)b * a.max_pages;

    auto load_tile = [&](const __nv_bfloat16* cache, int j, __nv_bfloat16* dst_tile) {
        const __nv_bfloat16* src = cache + ((size_t)pt[j] * a.nkvh + g) * TB_PAGE * DH;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(dst_tile);
        for (int idx = threadIdx.x; idx < AP_BN * CH; idx += AP_THREADS) {
            const int row = idx / CH, c = idx - row * CH;
            cp_async16(dst + swz(row, c) * 2, src + row * DH + c * 8);
        }
    };

    // Q tile (rows past nq are zero), then the first K/V tile
    for (int idx = threadIdx.x; idx < AP_BM * CH; idx += AP_THREADS) {
        const int row = idx / CH, c = idx - row * CH;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < nq) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + row) * a.q_stride + (size_t)h * DH + c * 8);
        *reinterpret_cast<uint4*>(sq + swz(row, c)) = v;
    }
    load_tile(a.kc, 0, sk);
    cp_async_commit();

    float o[DH / 8][4];
#pragma unroll
    for (int i = 0; i < DH / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_a = warp * 16 + gid, row_b = row_a + 8;          // this thread's two query rows in the tile
    const int pos_a = pos_first + row_a, pos_b = pos_first + row_b;
    const uint32_t sq_addr = (uint32_t)__cvta_generic_to_shared(sq);

    for (int j = 0; j < n_tiles; ++j) {
        const int buf = j & 1;
        cp_async_wait<0>();
        __syncthreads();                       // K of tile j has landed; everyone is done with tile j - 1 (its V too)
        load_tile(a.vc, j, sv);                // V of tile j flies while S = Q K^T is computed
        cp_async_commit();
        if (j + 1 < n_tiles) load_tile(a.kc, j + 1, sk + (buf ^ 1) * TILE);
        cp_async_commit();
        const uint32_t sk_addr = (uint32_t)__cvta_generic_to_shared(sk + buf * TILE);
        const uint32_t sv_addr = (uint32_t)__cvta_generic_to_shared(sv);

        // ---- S = Q K^T : 16 rows x 64 keys per warp ----
        float s[AP_BN / 8][4];
#pragma unroll
        for (int i = 0; i < AP_BN / 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DH / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunk = ks * 2 + (lane >> 4);
                ldsm_x4(sq_addr + swz(row, chunk) * 2, a0, a1, a2, a3);
            }
#pragma unroll
            for (int nb = 0; nb < AP_BN / 8; nb += 2) {
                uint32_t b0, b1, b2, b3;
                const int key = nb * 8 + (lane & 7) + (lane >> 4) * 8;
                const int chunk = ks * 2 + ((lane >> 3) & 1);
                ldsm_x4(sk_addr + swz(key, chunk) * 2, b0, b1, b2, b3);
                mma16816(s[nb], a0, a1, a2, a3, b0, b1);
                mma16816(s[nb + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- scale, mask, online softmax ----
        const int key0 = j * AP_BN;
        const bool edge = key0 + AP_BN - 1 > pos_first;       // some key of the tile may be invisible to some row
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nb = 0; nb < AP_BN / 8; ++nb) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v = s[nb][c] * a.scale_log2e;
                if (edge) {
                    const int key = key0 + nb * 8 + tid4 * 2 + (c & 1);
                    if (key > ((c & 2) ? pos_b : pos_a)) v = -INFINITY;
                }
                s[nb][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        float corr[2], mref[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mref[r] = (mx[r] == -INFINITY) ? 0.f : mx[r];      // a row with no visible key yet
            corr[r] = exp2f(m_run[r] - mref[r]);
            m_run[r] = mx[r];
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        uint32_t p[AP_BN / 8][2];
#pragma unroll
        for (int nb = 0; nb < AP_BN / 8; ++nb) {
            const float p0 = exp2f(s[nb][0] - mref[0]), p1 = exp2f(s[nb][1] - mref[0]);
            const float p2 = exp2f(s[nb][2] - mref[1]), p3 = exp2f(s[nb][3] - mref[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            p[nb][0] = pack_bf16(p0, p1);
            p[nb][1] = pack_bf16(p2, p3);
        }
        // ---- O += P V ----
        cp_async_wait<1>();                    // all but the newest group (K of tile j + 1): V of tile j is here
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < AP_BN / 16; ++kk) {
            const uint32_t a0 = p[2 * kk][0], a1 = p[2 * kk][1], a2 = p[2 * kk + 1][0], a3 = p[2 * kk + 1][1];
#pragma unroll
            for (int db = 0; db < DH / 8; db += 2) {
                uint32_t b0, b1, b2, b3;
                const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunk = db + (lane >> 4);
                ldsm_x4_t(sv_addr + swz(key, chunk) * 2, b0, b1, b2, b3);
                mma16816(o[db], a0, a1, a2, a3, b0, b1);
                mma16816(o[db + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    }
    cp_async_wait<0>();

    // ---- normalise and store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv_a = 1.0f / l_run[0], inv_b = 1.0f / l_run[1];
    if (row_a < nq) {
        __nv_bfloat16* dst = a.out + ((size_t)(t0 + row_a) * a.nh + h) * DH + tid4 * 2;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
    }
    if (row_b < nq) {
        __nv_bfloat16* dst = a.out + ((size_t)(t0 + row_b) * a.nh + h) * DH + tid4 * 2;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

template <int DH>
static int prefill_launch(const PrefillArgs& a, cudaStream_t s) {
    const size_t smem = (size_t)(AP_BM + 3 * AP_BN) * ap_row(DH) * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.tiles, a.nh);
    TB_LAUNCH((attention_prefill_kernel<DH>), grid, AP_THREADS, smem, s, a);
    return tb_last_error();
}

// head sizes above 128 (attention_prefill_large.cu)
int prefill_launch_large(const PrefillArgs& a, int dh, cudaStream_t s);
