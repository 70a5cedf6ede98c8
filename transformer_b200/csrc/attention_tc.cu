// Causal attention for prompts over the paged cache on the 5th-generation tensor cores (tcgen05),
// bfloat16 in, float accumulation in tensor memory.
//
// Same mathematics as the other attention kernels (score = q.k / sqrt(dh) over positions <= the
// token's own, models/llama/common/src/compute.rs:243-264; softmax statistics and the output
// accumulator in float).  A block = 128 query tokens of ONE sequence x one query head; it walks the
// sequence's pages (64 keys each):
//
//   warp 0   TMA: the Q tile once, then K and V of each page into a two-stage ring (the cache of a
//            layer is one 2-D tensor [pages * nkvh * 64, dh], so a page of a head is a box of rows)
//   warp 1   one thread issues  S = Q K^T  (128 x 64, accumulator S in TMEM) and  O += P V
//            (128 x dh, accumulator O in TMEM; P from TMEM, V is the MN-major B operand, straight as cached)
//   warps 2-5  128 threads = the 128 query rows: read their row of S from TMEM, mask, running
//            maximum and sum, P = exp2(s - m) rounded to bfloat16 and written back into tensor memory
//            where the row of S was (tcgen05.st): the second product takes its A operand from there
//            (tcgen05.mma with A in tensor memory), so P never passes through shared memory; and at
//            the end O / l to memory.
//
// The running maximum is only raised when it grows by more than 8 (in the exponent's log2 units):
// then the row of O in TMEM is rescaled; otherwise P is simply computed against the older maximum
// (it stays below 2^8, exact enough in bfloat16 and float), so the costly read-modify-write of O is
// rare.  Every wait on an mbarrier is bounded (see gemm_tc.cu); a wait that runs out sets the error
// word that tb_gemm_tc_status() reports.
//
// Head sizes 64 and 128.
#include <cuda.h>

#include "tc_common.cuh"

#define AT_BM 128
#define AT_BN 64
#define AT_STAGES 2
#define AT_THREADS 192

struct AtArgs {
    __nv_bfloat16* out;       // [nt, nh * dh]
    const int* tile_seq;
    const int* tile_t0;
    const int* tile_nq;
    const int* tok_pos;
    const int* page_table;
    int* error;
    int tiles, max_pages, nh, nkvh;
    float scale_log2e;
    unsigned v_lbo, v_sbo;    // descriptor strides of the MN-major V operand, in bytes
};

// Shared-memory descriptor with explicit strides (K-major operands use umma_desc of tc_common.cuh).
__device__ __forceinline__ uint64_t umma_desc_strides(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// 32 columns of this thread's lane without waiting for them (tcgen05.wait::ld comes before their first use)
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Two floats in one 64-bit register, for the packed arithmetic of sm_100 (fma.rn.f32x2, add.rn.f32x2).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 consecutive 32-bit columns of this thread's lane, as they are (packed bfloat16 pairs)
__device__ __forceinline__ void tmem_st32_words(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

template <int DH>
__global__ void __launch_bounds__(AT_THREADS) attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                 const __grid_constant__ CUtensorMap map_k,
                                                                 const __grid_constant__ CUtensorMap map_v,
                                                                 const AtArgs a) {
    pdl_sync();
    constexpr int KB = DH / 64;                          // 64-wide column boxes of a row of dh values
    constexpr uint32_t Q_BYTES = AT_BM * DH * 2, KV_BYTES = AT_BN * DH * 2;
    constexpr uint32_t STAGE_BYTES = 2 * KV_BYTES;
    constexpr uint32_t TMEM_COLS = 256;                  // S twice (2 x 64 columns) and O (dh columns)
    // All shared memory is dynamic and the kernel has no static shared memory, so the tiles start at the
    // base of the block's window (1024-byte aligned, as the 128-byte swizzle needs); two blocks then fit
    // on an SM.  The barriers and the TMEM slot follow the tiles.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    const uint32_t sq = smem_base, skv = sq + Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + Q_BYTES + AT_STAGES * STAGE_BYTES);   // 4 * stages + 7
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 4 * AT_STAGES + 7);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (smem_base & 1023u) {                              // never expected; refuse rather than compute garbage
        if (threadIdx.x == 0) atomicCAS(a.error, 0, 19);
        return;
    }

    // blocks start in the order of blockIdx.x fastest: all heads of the last tile (the one that sees the most
    // keys) first, then all heads of the tile before it, ... : the longest jobs first over the whole grid
    const int tile = a.tiles - 1 - (int)blockIdx.y;
    const int h = blockIdx.x, g = h / (a.nh / a.nkvh);
    const int b = a.tile_seq[tile], t0 = a.tile_t0[tile], nq = a.tile_nq[tile];
    const int pos_first = a.tok_pos[t0], pos_last = pos_first + nq - 1;
    const int n_tiles = pos_last / AT_BN + 1;
    const int* pt = a.page_table + (size_t)b * a.max_pages;

    const uint32_t bar0 = smem_u32(bars);
    // K and V have barriers of their own: a K slot is free as soon as the scores that read it are done,
    // a whole iteration before the V slot, so the next K is already on its way while P V still runs
    auto k_full = [&](int s) { return bar0 + 8u * s; };
    auto k_empty = [&](int s) { return bar0 + 8u * (AT_STAGES + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (2 * AT_STAGES + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (3 * AT_STAGES + s); };
    const uint32_t q_full = bar0 + 8u * (4 * AT_STAGES), o_done = q_full + 16;
    auto s_full = [&](int i) { return q_full + 24 + 8u * i; };      // one per S buffer
    // ... and one per S buffer for "P is in it": a softmax warp may be a tile ahead of the others (nothing holds it
    // back but the scores), and its arrival for the next tile must not count towards this one
    auto p_ready = [&](int i) { return i == 0 ? q_full + 8 : q_full + 40; };
    if (threadIdx.x == 0) {
        for (int s = 0; s < AT_STAGES; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        mbar_init(q_full, 1);
        mbar_init(s_full(0), 1);
        mbar_init(s_full(1), 1);
        mbar_init(p_ready(0), 4);    // one arrival per softmax warp
        mbar_init(p_ready(1), 4);
        mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + 2 * AT_BN;     // S of tile j at tmem_s + (j & 1) * 64

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) tma_load_2d(sq + kb * (AT_BM * 128), &map_q, q_full, h * DH + kb * 64, t0);
            bool ok = true;
            int issued = 0;
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % AT_STAGES;
                const int row = (pt[j] * a.nkvh + g) * TB_PAGE;
                const uint32_t sk = skv + s * STAGE_BYTES, sv = sk + KV_BYTES;
                if (j >= AT_STAGES) ok = mbar_wait(k_empty(s), ((j / AT_STAGES) - 1) & 1, a.error, 11);
                if (!ok) break;
                mbar_expect_tx(k_full(s), KV_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) tma_load_2d(sk + kb * (AT_BN * 128), &map_k, k_full(s), kb * 64, row);
                if (j >= AT_STAGES) ok = mbar_wait(v_empty(s), ((j / AT_STAGES) - 1) & 1, a.error, 11);
                if (!ok) break;
                mbar_expect_tx(v_full(s), KV_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) tma_load_2d(sv + kb * (AT_BN * 128), &map_v, v_full(s), kb * 64, row);
                issued = j + 1;
            }
            if (*(volatile int*)a.error != 0) {
                mbar_wait(q_full, 0, a.error, 14);
                for (int j = max(0, issued - AT_STAGES); j < issued; ++j) {
                    mbar_wait(k_full(j % AT_STAGES), (j / AT_STAGES) & 1, a.error, 14);
                    mbar_wait(v_full(j % AT_STAGES), (j / AT_STAGES) & 1, a.error, 14);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(AT_BM, AT_BN);                       // both operands K-major
            const uint32_t idesc_o = umma_idesc(AT_BM, DH) | (1u << 16);             // B (= V) is MN-major
            // S = Q K^T of tile j into S buffer j & 1: K = dh in steps of 16; step k lives in column box k / 4,
            // 32 bytes * (k % 4) along the row
            auto issue_s = [&](int j) {
                const uint32_t sk = skv + (j % AT_STAGES) * STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const uint64_t dq = umma_desc(sq + (k / 4) * (AT_BM * 128)) + 2 * (k % 4);
                    const uint64_t dk = umma_desc(sk + (k / 4) * (AT_BN * 128)) + 2 * (k % 4);
                    umma_bf16(tmem_s + (j & 1) * AT_BN, dq, dk, idesc_s, k != 0);
                }
                umma_commit(s_full(j & 1));
                umma_commit(k_empty(j % AT_STAGES));          // K of tile j is free once these scores are done
            };
            bool ok = mbar_wait(q_full, 0, a.error, 12);
            if (ok) ok = mbar_wait(k_full(0), 0, a.error, 12);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % AT_STAGES;
                // the scores of the NEXT tile are computed while the softmax warps work on this one
                if (j + 1 < n_tiles) {
                    ok = mbar_wait(k_full((j + 1) % AT_STAGES), ((j + 1) / AT_STAGES) & 1, a.error, 12);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(j + 1);
                }
                ok = mbar_wait(p_ready(j & 1), (j >> 1) & 1, a.error, 13);   // P is in tensor memory, where S of tile j was
                if (ok) ok = mbar_wait(v_full(s), (j / AT_STAGES) & 1, a.error, 12);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sv = skv + s * STAGE_BYTES + KV_BYTES;
                // O += P V: K = 64 keys in steps of 16 (16 keys = two 8-row groups = 2048 bytes along V's rows;
                // 32 bytes along P's rows); N = dh spans KB column boxes of V
#pragma unroll
                for (int k = 0; k < AT_BN / 16; ++k) {
                    // P of tile j lies where S of tile j lay: 16 keys = 8 columns of packed pairs per step
                    const uint64_t dv = umma_desc_strides(sv + k * 2048, a.v_lbo, a.v_sbo);
                    umma_bf16_ts(tmem_o, tmem_s + (j & 1) * AT_BN + 8 * k, dv, idesc_o, (j | k) != 0);
                }
                umma_commit(v_empty(s));
                umma_commit(o_done);
            }
        }
    } else {
        // ---------------- softmax / correction / epilogue: thread = query row ----------------
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int pos_r = pos_first + row;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        float m_used = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = mbar_wait(s_full(j & 1), (j >> 1) & 1, a.error, 15);
            tc_fence_after();
            if (!ok) break;
            float s[AT_BN];
            {
                uint32_t lo[32], hi[32];                 // both halves asked for, one wait
                tmem_ld32_nowait(tmem_s + (j & 1) * AT_BN + lane_sel, lo);
                tmem_ld32_nowait(tmem_s + (j & 1) * AT_BN + lane_sel + 32, hi);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    s[i] = __uint_as_float(lo[i]);
                    s[32 + i] = __uint_as_float(hi[i]);
                }
            }
            // The softmax warps are bound by instruction issue and by the exponential unit, so the row is
            // handled with as few instructions as will do: the maximum on the raw scores (the scale is
            // positive), the mask only on tiles that reach past the row's own position, and
            // p = 2^(s * scale - m) as one fused multiply-add and one ex2.approx each.
            const int key0 = j * AT_BN;
            if (key0 + AT_BN - 1 > pos_first) {             // uniform over the block: a tile on or past the diagonal
#pragma unroll
                for (int i = 0; i < AT_BN; ++i)
                    if (key0 + i > pos_r) s[i] = -INFINITY;
            }
            // two chains of three-input maxima: 32 instructions for the 64 scores
            float mx = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < AT_BN; i += 4) {
                asm("max.f32 %0, %0, %1, %2;" : "+f"(mx) : "f"(s[i]), "f"(s[i + 1]));
                asm("max.f32 %0, %0, %1, %2;" : "+f"(mx1) : "f"(s[i + 2]), "f"(s[i + 3]));
            }
            mx = fmaxf(mx, mx1) * a.scale_log2e;
            // raise the maximum only when it has grown by more than 8; then O must be rescaled
            const bool raise = mx > m_used + 8.0f;          // also true for the first visible keys (m_used = -inf)
            const float m_new = raise ? mx : m_used;
            const float rescale = (raise && m_used != -INFINITY) ? exp2f(m_used - m_new) : 1.0f;
            m_used = m_new;
            const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
            // computed BEFORE waiting for the previous tile's P V: the exponentials overlap that product,
            // only the stores below come after it
            uint32_t pk[AT_BN / 2];
            // two scores at a time through the packed forms of multiply-add and add (half the instructions)
            const uint64_t sc2 = pack_f32x2(a.scale_log2e, a.scale_log2e), nm2 = pack_f32x2(neg_m, neg_m);
            uint64_t psum_a = 0ull, psum_b = 0ull;              // two pairs of +0.0f
#pragma unroll
            for (int i = 0; i < AT_BN; i += 4) {
                uint64_t t0, t1;
                asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(t0) : "l"(pack_f32x2(s[i], s[i + 1])), "l"(sc2), "l"(nm2));
                asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(t1) : "l"(pack_f32x2(s[i + 2], s[i + 3])), "l"(sc2), "l"(nm2));
                float e0, e1, e2, e3, p0, p1, p2, p3;
                unpack_f32x2(t0, e0, e1);
                unpack_f32x2(t1, e2, e3);
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(e0));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(e1));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p2) : "f"(e2));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p3) : "f"(e3));
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(psum_a) : "l"(pack_f32x2(p0, p1)));
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(psum_b) : "l"(pack_f32x2(p2, p3)));
                __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
                pk[i / 2] = *reinterpret_cast<uint32_t*>(&h0);
                pk[i / 2 + 1] = *reinterpret_cast<uint32_t*>(&h1);
            }
            float ps0, ps1, ps2, ps3;
            unpack_f32x2(psum_a, ps0, ps1);
            unpack_f32x2(psum_b, ps2, ps3);
            l_run = l_run * rescale + ((ps0 + ps1) + (ps2 + ps3));
            // O may only be touched once the previous tile's P V is done (P itself goes where this tile's S was,
            // which nothing reads any more: no wait for that)
            const bool touch_o = __any_sync(0xffffffffu, rescale != 1.0f) && j > 0;
            if (touch_o) {
                ok = mbar_wait(o_done, (j - 1) & 1, a.error, 16);
                tc_fence_after();
                if (!ok) break;
#pragma unroll
                for (int c0 = 0; c0 < DH; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_sel + c0, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= rescale;
                    tmem_st32(tmem_o + lane_sel + c0, o);
                }
            }
            // P as the A operand of the second product, in tensor memory: this row's 64 values as 32 packed pairs
            // over the first 32 columns of the S buffer they came from
            tmem_st32_words(tmem_s + (j & 1) * AT_BN + lane_sel, pk);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_ready(j & 1)) : "memory");
            // Keep in step with the products' completions, one phase at a time (a wait on a phase's parity cannot
            // tell "two behind" from "done").  Here it costs nothing: P has been handed over, and the product
            // waited for was issued a whole tile ago.
            if (j > 0 && !touch_o) {
                ok = mbar_wait(o_done, (j - 1) & 1, a.error, 16);
                tc_fence_after();
            }
        }
        if (ok) {
            ok = mbar_wait(o_done, (n_tiles - 1) & 1, a.error, 17);
            tc_fence_after();
        }
        if (ok) {
            const float inv = 1.0f / l_run;
            __nv_bfloat16* dst = a.out + ((size_t)(t0 + row) * a.nh + h) * DH;
#pragma unroll
            for (int c0 = 0; c0 < DH; c0 += 32) {
                float o[32];
                tmem_ld32(tmem_o + lane_sel + c0, o);       // warp-collective: rows past nq take part, store nothing
                if (row < nq) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float f8[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) f8[e] = o[i + e] * inv;
                        store8(dst + c0 + i, f8);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_slot, TMEM_COLS);
}

template <int DH>
static int attention_tc_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AtArgs& a,
                               cudaStream_t s) {
    const size_t smem = (size_t)AT_BM * DH * 2 + (size_t)AT_STAGES * 2 * AT_BN * DH * 2 + 160;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.nh, a.tiles);
    TB_LAUNCH((attention_tc_kernel<DH>), grid, AT_THREADS, smem, s, mq, mk, mv, a);
    return tb_last_error();
}

extern "C" {
// Query tiles hold up to this many tokens of one sequence.
int tb_attention_tc_tile_tokens() { return AT_BM; }

// q: [nt, q_stride] (first q head of each token), out: [nt, nh * dh], kc / vc: one layer's cache
// [cache_pages, nkvh, 64, dh].
int tb_attention_tc_bf16(const void* q, void* out, const void* kc, const void* vc, const int* tile_seq,
                         const int* tile_t0, const int* tile_nq, const int* tok_pos, const int* page_table, int tiles,
                         int nt, int max_pages, int q_stride, int nh, int nkvh, int dh, int cache_pages, float scale,
                         cudaStream_t s) {
    if (nh <= 0 || nkvh <= 0 || nh % nkvh || tiles < 0 || nt < 0 || cache_pages <= 0) return TB_ERR_ARG;
    if (dh != 64 && dh != 128) return TB_ERR_UNSUPPORTED;
    if (q_stride % 8 || (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kc | (uintptr_t)vc) & 15)) return TB_ERR_UNSUPPORTED;
    if (tiles == 0) return 0;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, nt, nh * dh, q_stride, AT_BM);
    if (rc) return rc;
    const long long rows = (long long)cache_pages * nkvh * TB_PAGE;
    rc = make_map(&mk, kc, rows, dh, dh, AT_BN);
    if (rc) return rc;
    rc = make_map(&mv, vc, rows, dh, dh, AT_BN);
    if (rc) return rc;
    int* err_ptr = tc_error_ptr();
    if (!err_ptr) return tb_last_error();
    AtArgs a{(__nv_bfloat16*)out, tile_seq, tile_t0, tile_nq, tok_pos, page_table, err_ptr, tiles, max_pages, nh, nkvh,
             scale * 1.4426950408889634f, (unsigned)(AT_BN * 128), 1024u};
    return dh == 64 ? attention_tc_launch<64>(mq, mk, mv, a, s) : attention_tc_launch<128>(mq, mk, mv, a, s);
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_attention_tc_bf16)
