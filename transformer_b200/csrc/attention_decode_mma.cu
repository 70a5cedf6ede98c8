// Attention for decoding, bfloat16, head sizes 64, 128, 192 and 256: the cache pages come by TMA, the products run on the
// tensor cores.
//
// Same mathematics and the same cut of the work as attention_decode.cu (a block = one query token x one key/value
// head x one slice of the keys; partial results and a merge when the keys are sliced).  Two things differ.
//
// How K and V reach the block: one elected thread of a fifth warp asks the TMA unit for whole pages (64 keys x dh of
// one head are a box of rows of the layer's cache seen as a 2-D tensor) into a ring of stages, so that well over a
// hundred kilobytes are in flight per SM whatever the register budget of the arithmetic warps, which only read
// shared memory.  A decode step is bound by reading the cache once; bytes in flight are what buys bandwidth.  The
// pages arrive as tiles with the 128-byte swizzle, so that ldmatrix reads them without bank conflicts.
//
// Who multiplies: with multiply-adds on the CUDA cores every query head of a group pays for each key again, and
// from four query heads per key/value head on the arithmetic, not the read of the cache, sets the time (measured:
// 3.0 TB/s at 4 heads per group, 2.0 at 6, against 5.9 with one).  Here up to 16 query heads of the group are the M
// dimension of mma.sync.m16n8k16, and a page costs the same instructions whether 1 or 16 heads look at it:
//
//   S[16 heads, 16 keys] = Q[16 heads, dh] . K[16 keys, dh]^T      (A = Q in registers for the whole kernel,
//                                                                   B = K from shared memory by ldmatrix)
//   online softmax per head row in 32-bit (a row lives in the four lanes of a quad)
//   O[16 heads, dh]     += P[16 heads, 16 keys] . V[16 keys, dh]   (A = P: the accumulators of S, rounded to
//                                                                   bfloat16, are already laid out as an A operand;
//                                                                   B = V by ldmatrix.trans)
//
// The fused form (FUSE) also does what the rotary kernel does for a decode step, so that a layer has one launch
// less: the queries are rotated as they are loaded into registers; the new token's key (rotated) and value are taken
// from the q-k-v product's result, laid over the row of the last page in shared memory that TMA brought in its old
// state, and written to the cache by the block of the group's first 16 heads.
//
// Each of the four arithmetic warps takes 16 of a page's 64 keys and keeps a running (max, sum, O) of its own; they
// are merged once at the end, in the ring's memory.  With the keys in slices, the block that finishes a (token, head
// group)'s last slice merges the slices (a counter per group), so no kernel of its own is needed for that.
#include "attention_kernels.cuh"
#include "tc_common.cuh"

#define DM_WARPS 4
#define DM_THREADS ((DM_WARPS + 1) * 32)
#define DM_MAX_STAGES 8
#define DM_HEADS 16                    // query heads of one key/value head per block

struct DecodeMmaArgs {
    const __nv_bfloat16* q;   // [nt, q_stride]
    __nv_bfloat16* out;       // [nt, nh * dh]
    const int* tok_seq;
    const int* tok_pos;
    const int* page_table;
    float* partial;           // [nt, nh, splits, dh + 2] when splits > 1
    unsigned* done;           // [nt, gridDim.y] zeroed counters of finished slices (left zeroed), or null
    int* error;
    int max_pages, q_stride, nh, nkvh, splits, stages;
    float scale_log2e;
    // fused rotary encoding and cache write (FUSE): angle tables [positions, dh / 2]; pairing (i, i + dh/2) or
    // (2i, 2i + 1); patch: the new token's key and value come from the row of q (behind the query heads) and go to
    // kc_out / vc_out; without patch they are in the cache already (a layer that reads another layer's cache)
    const float* cos_t;
    const float* sin_t;
    __nv_bfloat16* kc_out;
    __nv_bfloat16* vc_out;
    int half_pairing, patch;
};

__device__ __forceinline__ float2 dm_unpack(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}
// (x0, x1) turned by the angle whose cosine and sine are c and s
__device__ __forceinline__ void dm_turn(float x0, float x1, float c, float s, float& y0, float& y1) {
    y0 = x0 * c - x1 * s;
    y1 = x0 * s + x1 * c;
}

__device__ __forceinline__ void dm_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dm_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// Byte offset of the 16-byte chunk `chunk` (8 channels) of row `row` in a page that TMA wrote as boxes of 64
// channels x 64 rows with the 128-byte swizzle.
__device__ __forceinline__ uint32_t dm_at(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (TB_PAGE * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int DH, bool FUSE>
__global__ void __launch_bounds__(DM_THREADS)
attention_decode_mma_kernel(const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv,
                            const DecodeMmaArgs a) {
    // The next kernel may start launching at once.  This one waits for the kernel before it (which wrote the
    // step's queries and the newest key and value) as late as it can: page numbers, positions and every cache
    // page but the sequence's last two were written long before the step began, so the ring is filled meanwhile.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int KS = DH / 16;                         // k-steps of Q.K^T
    constexpr int DT = DH / 8;                          // 8-channel tiles of O
    constexpr uint32_t PAGE_BYTES = TB_PAGE * DH * 2, STAGE_BYTES = 2 * PAGE_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_dm[];
    const uint32_t smem_base = (smem_u32(smem_dm) + 1023u) & ~1023u;
    uint8_t* smem_al = smem_dm + (smem_base - smem_u32(smem_dm));
    const int S = a.stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + (size_t)S * STAGE_BYTES);   // full[S], empty[S]
    float* sm_m = reinterpret_cast<float*>(bars + 2 * DM_MAX_STAGES);                   // [DM_WARPS][DM_HEADS]
    float* sm_l = sm_m + DM_WARPS * DM_HEADS;
    float* sm_o = reinterpret_cast<float*>(smem_al);   // [DM_WARPS][DM_HEADS][DH], over the ring once it is drained

    const int t = blockIdx.x;
    const int group = a.nh / a.nkvh;
    const int chunks = (group + DM_HEADS - 1) / DM_HEADS;
    const int g = blockIdx.y / chunks;
    const int h0 = g * group + (blockIdx.y % chunks) * DM_HEADS;
    const int nheads = min(DM_HEADS, g * group + group - h0);
    const int split = blockIdx.z;
    const int b = a.tok_seq[t], pos = a.tok_pos[t];
    const int n_pages = pos / TB_PAGE + 1;
    const int slices = decode_slices(n_pages, a.splits);
    if (split >= slices) return;
    const int per = (n_pages + slices - 1) / slices;
    const int p_lo = split * per, p_hi = min(n_pages, p_lo + per);
    const int np = max(0, p_hi - p_lo);
    const int* pt = a.page_table + (size_t)b * a.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (DM_MAX_STAGES + s); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), DM_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int r0 = lane >> 2, c2 = (lane & 3) * 2;      // this thread's rows r0 and r0 + 8, columns c2 and c2 + 1
    float o[DT][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    bool ok = true;
    if (warp == DM_WARPS) {
        // ---------------- producer: the whole warp reads page numbers, lane 0 asks for the tiles ----------------
        bool waited = false;
        int issued = 0, mine = 0;
        for (int i = 0; i < np && ok; ++i) {
            if ((i & 31) == 0) mine = (i + lane < np) ? pt[p_lo + i + lane] : 0;
            const int page = __shfl_sync(0xffffffffu, mine, i & 31);
            const int s = i % S;
            if (lane == 0) {
                if (i >= S) ok = mbar_wait(empty_bar(s), ((i / S) - 1) & 1, a.error, 25);
                if (ok) {
                    // The sequence's last two pages hold what this step and the 64 or more steps before it
                    // wrote: they are asked for after the wait.  Older pages were written so many launches ago
                    // that their writers cannot still be running (a chain of dependent launches is no deeper than
                    // the grids the device holds at once), and are fetched before it.
                    if (!waited && p_lo + i >= n_pages - 2) {
                        asm volatile("griddepcontrol.wait;" ::: "memory");
                        waited = true;
                    }
                    const int row = (page * a.nkvh + g) * TB_PAGE;       // of the layer's cache as [rows, DH]
                    const uint32_t sk = smem_base + s * STAGE_BYTES, sv = sk + PAGE_BYTES;
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
                    for (int kb = 0; kb < DH / 64; ++kb) {
                        tma_load_2d(sk + kb * (TB_PAGE * 128), &mk, full_bar(s), kb * 64, row);
                        tma_load_2d(sv + kb * (TB_PAGE * 128), &mv, full_bar(s), kb * 64, row);
                    }
                    issued = i + 1;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        if (lane == 0 && *(volatile int*)a.error != 0)
            for (int i = max(0, issued - S); i < issued; ++i) mbar_wait(full_bar(i % S), (i / S) & 1, a.error, 27);
    } else {
        // ---------------- arithmetic warps: keys 16 warp .. 16 warp + 15 of every page ----------------
        uint32_t qa[KS][4];
#pragma unroll
        for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
        // Fused: the angles of this token's position were there before the step began; they are read before the
        // wait, the q-k-v row's new key and value (by the warp that owns their row of the last page) right after it.
        float ang[FUSE ? KS * 4 : 1];                     // this thread's cosines and sines for the queries
        constexpr int NPL = (DH / 2 + 31) / 32;           // pairs of the new key per lane: lane, lane + 32, ...
        float pc[NPL], ps[NPL];                           // their cosines and sines
        const bool patcher = FUSE && a.patch && p_hi == n_pages && np > 0 && warp == (pos % TB_PAGE) / 16;
        if (FUSE) {
            const float* cs = a.cos_t + (size_t)pos * (DH / 2);
            const float* sn = a.sin_t + (size_t)pos * (DH / 2);
            if (a.half_pairing) {
#pragma unroll
                for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = 16 * ks + c2 + 8 * hh;
                        const float2 c = *reinterpret_cast<const float2*>(cs + i);
                        const float2 sv2 = *reinterpret_cast<const float2*>(sn + i);
                        float* dst = ang + (ks * 2 + hh) * 4;
                        dst[0] = c.x, dst[1] = c.y, dst[2] = sv2.x, dst[3] = sv2.y;
                    }
            } else {
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = 8 * ks + (c2 >> 1) + 4 * hh;
                        ang[(ks * 2 + hh) * 2] = cs[i];
                        ang[(ks * 2 + hh) * 2 + 1] = sn[i];
                    }
            }
            if (patcher) {
#pragma unroll
                for (int u = 0; u < NPL; ++u)
                    if (lane + 32 * u < DH / 2) {
                        pc[u] = cs[lane + 32 * u];
                        ps[u] = sn[lane + 32 * u];
                    }
            }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");     // the queries come from the kernel before
        float kx0[NPL], kx1[NPL];
        uint4 vnew = make_uint4(0u, 0u, 0u, 0u);
        if (patcher) {
            const __nv_bfloat16* kn = a.q + (size_t)t * a.q_stride + (size_t)(a.nh + g) * DH;
#pragma unroll
            for (int u = 0; u < NPL; ++u) {
                const int p = lane + 32 * u;
                if (p < DH / 2) {
                    kx0[u] = __bfloat162float(kn[a.half_pairing ? p : 2 * p]);
                    kx1[u] = __bfloat162float(kn[a.half_pairing ? p + DH / 2 : 2 * p + 1]);
                }
            }
            if (lane < DH / 8) vnew = *reinterpret_cast<const uint4*>(kn + (size_t)a.nkvh * DH + lane * 8);
        }
        const __nv_bfloat16* qg = a.q + (size_t)t * a.q_stride + (size_t)h0 * DH + c2;
        const bool lo = r0 < nheads, hi = r0 + 8 < nheads;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const __nv_bfloat16* q0 = qg + (size_t)r0 * DH + ks * 16;
            const __nv_bfloat16* q1 = q0 + 8 * DH;
            qa[ks][0] = lo ? *reinterpret_cast<const uint32_t*>(q0) : 0u;
            qa[ks][1] = hi ? *reinterpret_cast<const uint32_t*>(q1) : 0u;
            qa[ks][2] = lo ? *reinterpret_cast<const uint32_t*>(q0 + 8) : 0u;
            qa[ks][3] = hi ? *reinterpret_cast<const uint32_t*>(q1 + 8) : 0u;
        }
        if (FUSE) {
            if (a.half_pairing) {
                // dims d and d + DH/2 make a pair: the same register slot, KS/2 k-steps apart
#pragma unroll
                for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float* an = ang + (ks * 2 + hh) * 4;
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            const float2 xl = dm_unpack(qa[ks][2 * hh + rr]), xh = dm_unpack(qa[ks + KS / 2][2 * hh + rr]);
                            float l0, l1, h0f, h1f;
                            dm_turn(xl.x, xh.x, an[0], an[2], l0, h0f);
                            dm_turn(xl.y, xh.y, an[1], an[3], l1, h1f);
                            qa[ks][2 * hh + rr] = dm_pack(l0, l1);
                            qa[ks + KS / 2][2 * hh + rr] = dm_pack(h0f, h1f);
                        }
                    }
            } else {
                // dims 2i and 2i + 1 make a pair: the two halves of one register
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float c = ang[(ks * 2 + hh) * 2], sv1 = ang[(ks * 2 + hh) * 2 + 1];
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            const float2 x = dm_unpack(qa[ks][2 * hh + rr]);
                            float y0, y1;
                            dm_turn(x.x, x.y, c, sv1, y0, y1);
                            qa[ks][2 * hh + rr] = dm_pack(y0, y1);
                        }
                    }
            }
        }
        const int mi = lane >> 3, lr = lane & 7;
        const int krow = 16 * warp + (mi >> 1) * 8 + lr, kch = mi & 1;     // K: matrices (keys lo/hi) x (channels lo/hi)
        const int vrow = 16 * warp + (mi & 1) * 8 + lr, vch = mi >> 1;     // V: matrices (channels lo/hi) x (keys lo/hi)
        for (int i = 0; i < np && ok; ++i) {
            const int s = i % S;
            ok = mbar_wait(full_bar(s), (i / S) & 1, a.error, 26);
            if (!ok) break;
            const uint32_t sk = smem_base + s * STAGE_BYTES, sv = sk + PAGE_BYTES;
            if (patcher && i == np - 1) {
                // The newest key and value: into this page's row in shared memory (only this warp reads that row),
                // and into the cache by the block of the group's first heads.
                const int row = pos % TB_PAGE, half = DH / 2;
                uint8_t* pk = smem_al + (size_t)s * STAGE_BYTES;
                uint8_t* pv = pk + PAGE_BYTES;
                const bool writer = blockIdx.y % chunks == 0;
                const size_t at = (((size_t)pt[n_pages - 1] * a.nkvh + g) * TB_PAGE + row) * DH;
#pragma unroll
                for (int u = 0; u < NPL; ++u) {
                    const int p = lane + 32 * u;
                    if (p < half) {
                        const int d0 = a.half_pairing ? p : 2 * p, d1 = a.half_pairing ? p + half : 2 * p + 1;
                        float y0, y1;
                        dm_turn(kx0[u], kx1[u], pc[u], ps[u], y0, y1);
                        const __nv_bfloat16 b0 = __float2bfloat16_rn(y0), b1 = __float2bfloat16_rn(y1);
                        *reinterpret_cast<__nv_bfloat16*>(pk + dm_at(row, d0 >> 3) + (d0 & 7) * 2) = b0;
                        *reinterpret_cast<__nv_bfloat16*>(pk + dm_at(row, d1 >> 3) + (d1 & 7) * 2) = b1;
                        if (writer) {
                            a.kc_out[at + d0] = b0;
                            a.kc_out[at + d1] = b1;
                        }
                    }
                }
                if (lane < DH / 8) {                       // the value: 16 bytes per lane
                    *reinterpret_cast<uint4*>(pv + dm_at(row, lane)) = vnew;
                    if (writer) *reinterpret_cast<uint4*>(a.vc_out + at + lane * 8) = vnew;
                }
                __syncwarp();
            }
            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b0, b1, b2, b3;
                dm_ldsm_x4(sk + dm_at(krow, 2 * ks + kch), b0, b1, b2, b3);
                dm_mma(sc[0], qa[ks], b0, b1);
                dm_mma(sc[1], qa[ks], b2, b3);
            }
            const int key0 = (p_lo + i) * TB_PAGE + 16 * warp + c2;
            const bool edge = (p_lo + i) * TB_PAGE + TB_PAGE - 1 > pos;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = sc[j][e] * a.scale_log2e;
                    sc[j][e] = (edge && key0 + 8 * j + (e & 1) > pos) ? -INFINITY : v;
                }
            uint32_t pa[4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {          // row r0 (accumulator elements 0, 1) and row r0 + 8 (2, 3)
                float mx = fmaxf(fmaxf(sc[0][2 * r], sc[0][2 * r + 1]), fmaxf(sc[1][2 * r], sc[1][2 * r + 1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m[r], mx);
                const float mref = (m_new == -INFINITY) ? 0.f : m_new;
                const float corr = exp2f(m[r] - mref);
                const float p00 = exp2f(sc[0][2 * r] - mref), p01 = exp2f(sc[0][2 * r + 1] - mref);
                const float p10 = exp2f(sc[1][2 * r] - mref), p11 = exp2f(sc[1][2 * r + 1] - mref);
                l[r] = l[r] * corr + (p00 + p01 + p10 + p11);
                m[r] = m_new;
#pragma unroll
                for (int d = 0; d < DT; ++d) {
                    o[d][2 * r] *= corr;
                    o[d][2 * r + 1] *= corr;
                }
                pa[r] = dm_pack(p00, p01);          // keys 0..7 of this warp's 16
                pa[2 + r] = dm_pack(p10, p11);      // keys 8..15
            }
#pragma unroll
            for (int dp = 0; dp < DT / 2; ++dp) {
                uint32_t b0, b1, b2, b3;
                dm_ldsm_x4_t(sv + dm_at(vrow, 2 * dp + vch), b0, b1, b2, b3);
                dm_mma(o[2 * dp], pa, b0, b1);
                dm_mma(o[2 * dp + 1], pa, b2, b3);
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(s)) : "memory");
        }
    }
    // Every warp has read its last page: the ring becomes the place where the warps' results meet.
    __syncthreads();
    if (warp < DM_WARPS && ok) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int hc = r0 + 8 * r;
            float lt = l[r];
            lt += __shfl_xor_sync(0xffffffffu, lt, 1);
            lt += __shfl_xor_sync(0xffffffffu, lt, 2);
            if (hc < nheads) {
                float* dst = sm_o + ((size_t)warp * DM_HEADS + hc) * DH + c2;
#pragma unroll
                for (int d = 0; d < DT; ++d)
                    *reinterpret_cast<float2*>(dst + 8 * d) = make_float2(o[d][2 * r], o[d][2 * r + 1]);
                if ((lane & 3) == 0) {
                    sm_m[warp * DM_HEADS + hc] = m[r];
                    sm_l[warp * DM_HEADS + hc] = lt;
                }
            }
        }
    }
    __syncthreads();
    if (warp < DM_WARPS) {
        const float ln2 = 0.6931471805599453f;
        for (int idx = threadIdx.x; idx < nheads * DH; idx += DM_WARPS * 32) {
            const int hc = idx / DH, c = idx - hc * DH;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < DM_WARPS; ++j) mx = fmaxf(mx, sm_m[j * DM_HEADS + hc]);
            float den = 0.f, acc = 0.f;
            if (mx != -INFINITY) {
#pragma unroll
                for (int j = 0; j < DM_WARPS; ++j) {
                    const float mj = sm_m[j * DM_HEADS + hc];
                    if (mj == -INFINITY) continue;
                    const float w = exp2f(mj - mx);
                    den += sm_l[j * DM_HEADS + hc] * w;
                    acc += sm_o[((size_t)j * DM_HEADS + hc) * DH + c] * w;
                }
            }
            const int h = h0 + hc;
            if (a.splits == 1) {
                a.out[((size_t)t * a.nh + h) * DH + c] = __float2bfloat16_rn(acc / den);
            } else {
                float* dst = a.partial + (((size_t)t * a.nh + h) * a.splits + split) * (DH + 2);
                dst[c] = acc;
                if (c == 0) {
                    dst[DH] = mx == -INFINITY ? -INFINITY : mx * ln2;   // natural-log units, as the merge kernel expects
                    dst[DH + 1] = den;
                }
            }
        }
    }
    if (a.splits == 1 || !a.done) return;
    // The block that finishes a (token, head group)'s last slice merges the slices: no kernel of its own for it.
    __shared__ bool last_slice;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* count = a.done + (size_t)t * gridDim.y + blockIdx.y;
        last_slice = atomicAdd(count, 1u) == (unsigned)slices - 1;
        if (last_slice) *count = 0;
    }
    __syncthreads();
    if (!last_slice) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < nheads * DH; idx += DM_THREADS) {
        const int hc = idx / DH, c = idx - hc * DH, h = h0 + hc;
        const float* p = a.partial + ((size_t)t * a.nh + h) * a.splits * (DH + 2);
        float mx = -INFINITY;
        for (int s = 0; s < slices; ++s) mx = fmaxf(mx, __ldcg(p + s * (DH + 2) + DH));
        float den = 0.f, acc = 0.f;
        for (int s = 0; s < slices; ++s) {
            const float ms = __ldcg(p + s * (DH + 2) + DH);
            if (ms == -INFINITY) continue;
            const float w = expf(ms - mx);
            den += __ldcg(p + s * (DH + 2) + DH + 1) * w;
            acc += __ldcg(p + s * (DH + 2) + c) * w;
        }
        a.out[((size_t)t * a.nh + h) * DH + c] = __float2bfloat16_rn(acc / den);
    }
}

template <int DH, bool FUSE>
static int decode_mma_launch(const CUtensorMap& mk, const CUtensorMap& mv, DecodeMmaArgs a, int nt, cudaStream_t s) {
    const size_t stage = (size_t)2 * TB_PAGE * DH * 2;
    const size_t tail = 2 * DM_MAX_STAGES * 8 + (size_t)2 * DM_WARPS * DM_HEADS * sizeof(float);
    // about half of an SM's shared memory per block: two blocks per SM keep their rings in flight together; heads
    // above 128 leave room for one block only (registers), which then takes most of the shared memory
    int stages = (int)(((DH <= 128 ? 110 : 200) * 1024 - 1024 - tail) / stage);
    if (stages > DM_MAX_STAGES) stages = DM_MAX_STAGES;
    if (stages < 2) stages = 2;
    a.stages = stages;
    // the warps' results (DM_WARPS x DM_HEADS x DH floats) meet in the ring: one stage's worth
    static_assert((size_t)DM_WARPS * DM_HEADS * DH * sizeof(float) <= (size_t)2 * 2 * TB_PAGE * DH * 2, "ring too small");
    const size_t smem = stage * stages + tail + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<DH, FUSE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = a.nh / a.nkvh;
    dim3 grid(nt, a.nkvh * ((group + DM_HEADS - 1) / DM_HEADS), a.splits);
    TB_LAUNCH((attention_decode_mma_kernel<DH, FUSE>), grid, DM_THREADS, smem, s, mk, mv, a);
    return tb_last_error();
}

static int decode_mma(const void* q, void* out, void* kc, void* vc, const int* tok_seq, const int* tok_pos,
                      const int* page_table, float* partial, unsigned* done, const float* cos_t, const float* sin_t,
                      int nt, int max_pages, int q_stride, int nh, int nkvh, int dh, int splits, int cache_pages,
                      int half_pairing, int patch, bool fuse, float scale, cudaStream_t s) {
    if (nh <= 0 || nkvh <= 0 || nh % nkvh || splits < 1 || cache_pages <= 0) return TB_ERR_ARG;
    if (splits > 1 && !partial) return TB_ERR_ARG;
    if (fuse && !(cos_t && sin_t)) return TB_ERR_ARG;
    if (dh != 64 && dh != 128 && dh != 192 && dh != 256) return TB_ERR_UNSUPPORTED;
    if (q_stride % 8 || (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc) & 15)) return TB_ERR_UNSUPPORTED;
    if (fuse && (((uintptr_t)cos_t | (uintptr_t)sin_t) & 7)) return TB_ERR_UNSUPPORTED;
    if (nt <= 0) return nt == 0 ? 0 : TB_ERR_ARG;
    CUtensorMap mk, mv;
    const long long rows = (long long)cache_pages * nkvh * TB_PAGE;
    if (rows > 0x7fffffffLL) return TB_ERR_UNSUPPORTED;
    int rc = make_map(&mk, kc, rows, dh, dh, TB_PAGE);
    if (rc) return rc;
    rc = make_map(&mv, vc, rows, dh, dh, TB_PAGE);
    if (rc) return rc;
    int* err = tc_error_ptr();
    if (!err) return tb_last_error();
    DecodeMmaArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, tok_seq, tok_pos, page_table, partial, done, err,
                    max_pages, q_stride, nh, nkvh, splits, 0, scale * 1.4426950408889634f,
                    cos_t, sin_t, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, half_pairing, patch};
    switch (dh + (fuse ? 1 : 0)) {
        case 64: rc = decode_mma_launch<64, false>(mk, mv, a, nt, s); break;
        case 65: rc = decode_mma_launch<64, true>(mk, mv, a, nt, s); break;
        case 128: rc = decode_mma_launch<128, false>(mk, mv, a, nt, s); break;
        case 129: rc = decode_mma_launch<128, true>(mk, mv, a, nt, s); break;
        case 192: rc = decode_mma_launch<192, false>(mk, mv, a, nt, s); break;
        case 193: rc = decode_mma_launch<192, true>(mk, mv, a, nt, s); break;
        case 256: rc = decode_mma_launch<256, false>(mk, mv, a, nt, s); break;
        default: rc = decode_mma_launch<256, true>(mk, mv, a, nt, s); break;
    }
    if (rc) return rc;
    if (splits > 1 && !done) {
        dim3 grid(nt, nh);
        TB_LAUNCH((attention_merge_kernel<__nv_bfloat16>), grid, dh < 128 ? 64 : 128, 0, s, partial,
                  (__nv_bfloat16*)out, nh, dh, splits, tok_pos);
        rc = tb_last_error();
    }
    return rc;
}

extern "C" {
// q: [nt, q_stride] (first q head of each token, already rotated), out: [nt, nh * dh], kc / vc: one layer's cache
// [cache_pages, nkvh, 64, dh] with the new token's key and value in it; done: [nt * nkvh * ceil(group / 16)] zeroed
// counters, or null (then a merge kernel runs).
int tb_attention_decode_mma_bf16(const void* q, void* out, const void* kc, const void* vc, const int* tok_seq,
                                 const int* tok_pos, const int* page_table, float* partial, unsigned* done, int nt,
                                 int max_pages, int q_stride, int nh, int nkvh, int dh, int splits, int cache_pages,
                                 float scale, cudaStream_t s) {
    return decode_mma(q, out, const_cast<void*>(kc), const_cast<void*>(vc), tok_seq, tok_pos, page_table, partial, done,
                      nullptr, nullptr, nt, max_pages, q_stride, nh, nkvh, dh, splits, cache_pages, 0, 0, false, scale, s);
}
// The same with the rotary encoding and the cache write of a decode step inside: qkv is the q-k-v product's result
// [nt, q_stride] (heads ordered q, k, v; nothing rotated yet; left as it is), cos_t / sin_t the angle tables
// [positions, dh / 2].  write_kv = 1: the new token's key (rotated) and value go into kc / vc; 0: they are there
// already (a layer that reads another layer's cache) and only the queries are rotated.
int tb_attention_decode_rope_bf16(const void* qkv, void* out, void* kc, void* vc, const int* tok_seq, const int* tok_pos,
                                  const int* page_table, float* partial, unsigned* done, const float* cos_t,
                                  const float* sin_t, int nt, int max_pages, int q_stride, int nh, int nkvh, int dh,
                                  int splits, int cache_pages, int half_pairing, int write_kv, float scale,
                                  cudaStream_t s) {
    if (q_stride < (nh + 2 * nkvh) * dh) return TB_ERR_ARG;
    return decode_mma(qkv, out, kc, vc, tok_seq, tok_pos, page_table, partial, done, cos_t, sin_t, nt, max_pages,
                      q_stride, nh, nkvh, dh, splits, cache_pages, half_pairing, write_kv ? 1 : 0, true, scale, s);
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_attention_decode_mma_bf16)
TB_TAPE_REGISTER(tb_attention_decode_rope_bf16)
