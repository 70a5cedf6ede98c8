// Attention for decoding, bfloat16, with the cache pages fetched by TMA.
//
// Same mathematics and the same work split as attention_decode.cu (a block = one query token x one
// key/value head x up to GC of its query heads x one slice of the keys; a sub-warp of dh/8 lanes per
// key, an online softmax per sub-warp, one merge at the end; partial results + attention_merge_kernel
// when the keys are sliced).  What differs is how K and V reach the block: one elected thread asks
// the TMA unit for whole pages (64 keys x dh of one head are a box of rows of the layer's cache seen as
// a 2-D tensor) into a ring of DT_STAGES stages, so that well over a hundred kilobytes are in flight
// per SM whatever the register budget of the arithmetic warps, which only read shared memory.
// A decode step is bound by reading the cache once; bytes in flight are what buys bandwidth.
//
// Head sizes 64 and 128 (the box is 64 columns wide); others use attention_decode.cu.
#include "attention_kernels.cuh"
#include "tc_common.cuh"

#define DT_WARPS 4                     // arithmetic warps; one more warp feeds the ring
#define DT_THREADS ((DT_WARPS + 1) * 32)
#define DT_MAX_STAGES 8

struct DecodeTmaArgs {
    const __nv_bfloat16* q;   // [nt, q_stride]
    const __nv_bfloat16* kc;  // [pages, nkvh, TB_PAGE, dh]
    const __nv_bfloat16* vc;
    __nv_bfloat16* out;       // [nt, nh * dh]
    const int* tok_seq;
    const int* tok_pos;
    const int* page_table;
    float* partial;           // [nt, nh, splits, dh + 2] when splits > 1
    unsigned* done;           // [nt, gridDim.y] zeroed counters of finished slices (left zeroed), or null
    int* error;
    int max_pages, q_stride, nh, nkvh, splits, stages;
    float scale_log2e;
};

template <int DH, int GC>
__global__ void __launch_bounds__(DT_THREADS) attention_decode_tma_kernel(const DecodeTmaArgs a) {
    // The next kernel may start launching at once.  This one waits for the kernel before it (which wrote the
    // step's queries and the newest key and value) as late as it can: page numbers, positions and every cache
    // page but the sequence's last were written before the step began, so the ring is filled meanwhile.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int TPK = DH / 8;                         // lanes per key (8 or 16)
    constexpr int NSW = DT_WARPS * 32 / TPK;            // sub-warps among the arithmetic warps
    constexpr int KPS = TB_PAGE / NSW;                  // keys of a page per sub-warp (4 or 8)
    constexpr int KU = 4;                               // of which this many are in registers at a time
    constexpr uint32_t PAGE_BYTES = TB_PAGE * DH * 2, STAGE_BYTES = 2 * PAGE_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_dt[];
    const uint32_t smem_base = (smem_u32(smem_dt) + 1023u) & ~1023u;
    uint8_t* smem_al = smem_dt + (smem_base - smem_u32(smem_dt));
    const int S = a.stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + (size_t)S * STAGE_BYTES);   // full[S], empty[S]
    float* sm_o = reinterpret_cast<float*>(bars + 2 * DT_MAX_STAGES);                   // [NSW][GC][DH]
    float* sm_m = sm_o + NSW * GC * DH;                                                 // [NSW][GC]
    float* sm_l = sm_m + NSW * GC;

    const int t = blockIdx.x;
    const int group = a.nh / a.nkvh;
    const int chunks = (group + GC - 1) / GC;
    const int g = blockIdx.y / chunks;
    const int h0 = g * group + (blockIdx.y % chunks) * GC;
    const int nheads = min(GC, g * group + group - h0);
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
    auto empty_bar = [&](int s) { return bar0 + 8u * (DT_MAX_STAGES + s); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), DT_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == DT_WARPS) {
        // ---------------- producer: the whole warp reads page numbers, lane 0 asks for the copies ----------------
        bool ok = true, waited = false;
        int issued = 0, mine = 0;
        for (int i = 0; i < np && ok; ++i) {
            if ((i & 31) == 0) mine = (i + lane < np) ? pt[p_lo + i + lane] : 0;
            const int page = __shfl_sync(0xffffffffu, mine, i & 31);
            const int s = i % S;
            if (lane == 0) {
                if (i >= S) ok = mbar_wait(empty_bar(s), ((i / S) - 1) & 1, a.error, 21);
                if (ok) {
                    if (!waited && p_lo + i == n_pages - 1) {   // the page the kernel before this one wrote to
                        asm volatile("griddepcontrol.wait;" ::: "memory");
                        waited = true;
                    }
                    // one head's keys of a page are TB_PAGE * DH contiguous elements of the cache
                    const size_t at = ((size_t)page * a.nkvh + g) * (TB_PAGE * DH);
                    const uint32_t sk = smem_base + s * STAGE_BYTES, sv = sk + PAGE_BYTES;
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
                    bulk_load(sk, a.kc + at, PAGE_BYTES, full_bar(s));
                    bulk_load(sv, a.vc + at, PAGE_BYTES, full_bar(s));
                    issued = i + 1;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        if (lane == 0 && *(volatile int*)a.error != 0)
            for (int i = max(0, issued - S); i < issued; ++i) mbar_wait(full_bar(i % S), (i / S) & 1, a.error, 24);
    } else {
        // ---------------- arithmetic warps ----------------
        const int tid = threadIdx.x;                 // 0 .. 127
        const int sw = tid / TPK, li = tid % TPK;    // sub-warp, lane in it: channels li * 8 .. + 8
        float q[GC][8], o[GC][8], m[GC], l[GC];
        asm volatile("griddepcontrol.wait;" ::: "memory");     // the queries come from the kernel before
        const __nv_bfloat16* qg = a.q + (size_t)t * a.q_stride + (size_t)h0 * DH + li * 8;
#pragma unroll
        for (int hc = 0; hc < GC; ++hc) {
            m[hc] = -INFINITY;
            l[hc] = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) o[hc][e] = q[hc][e] = 0.f;
            if (hc < nheads) {
                load8(qg + (size_t)hc * DH, q[hc]);
#pragma unroll
                for (int e = 0; e < 8; ++e) q[hc][e] *= a.scale_log2e;
            }
        }
        bool ok = true;
        for (int i = 0; i < np && ok; ++i) {
            const int s = i % S;
            ok = mbar_wait(full_bar(s), (i / S) & 1, a.error, 22);
            if (!ok) break;
            const uint8_t* sk = smem_al + (size_t)s * STAGE_BYTES + li * 16;
            const uint8_t* sv = sk + PAGE_BYTES;
            const int key0 = (p_lo + i) * TB_PAGE;
            // this sub-warp's keys of the page: r = sw, sw + NSW, ..., four at a time; a quarter-warp reads
            // 128 contiguous bytes, so the plain row-major page has no bank conflicts
#pragma unroll
            for (int u0 = 0; u0 < KPS; u0 += KU) {
                float kf[KU][8], vf[KU][8];
                bool live[KU];
#pragma unroll
                for (int u = 0; u < KU; ++u) {
                    const int r = sw + (u0 + u) * NSW;
                    const int off = r * (DH * 2);
                    live[u] = key0 + r <= pos;
                    Vec16<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(sk + off), kf[u]);
                    Vec16<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(sv + off), vf[u]);
                }
                if (u0 + KU >= KPS) {
                    // the whole page is in registers: hand the stage back before the arithmetic
                    __syncwarp();
                    if (lane == 0)
                        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(s)) : "memory");
                }
#pragma unroll
                for (int hc = 0; hc < GC; ++hc) {
                    if (hc >= nheads) continue;
                    float sc[KU];
#pragma unroll
                    for (int u = 0; u < KU; ++u) {
                        float d = 0.f;
#pragma unroll
                        for (int e = 0; e < 8; ++e) d += q[hc][e] * kf[u][e];
#pragma unroll
                        for (int w = TPK >> 1; w > 0; w >>= 1) d += __shfl_xor_sync(0xffffffffu, d, w);
                        sc[u] = live[u] ? d : -INFINITY;
                    }
                    float m_new = m[hc];
#pragma unroll
                    for (int u = 0; u < KU; ++u) m_new = fmaxf(m_new, sc[u]);
                    const float mref = (m_new == -INFINITY) ? 0.f : m_new;
                    const float corr = exp2f(m[hc] - mref);
                    float psum = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[hc][e] *= corr;
#pragma unroll
                    for (int u = 0; u < KU; ++u) {
                        const float p = exp2f(sc[u] - mref);
                        psum += p;
#pragma unroll
                        for (int e = 0; e < 8; ++e) o[hc][e] += p * vf[u][e];
                    }
                    l[hc] = l[hc] * corr + psum;
                    m[hc] = m_new;
                }
            }
        }
        // every sub-warp's running state to shared memory
#pragma unroll
        for (int hc = 0; hc < GC; ++hc) {
            if (hc >= nheads) continue;
#pragma unroll
            for (int e = 0; e < 8; ++e) sm_o[(sw * GC + hc) * DH + li * 8 + e] = o[hc][e];
            if (li == 0) {
                sm_m[sw * GC + hc] = m[hc];
                sm_l[sw * GC + hc] = l[hc];
            }
        }
    }
    __syncthreads();
    if (warp < DT_WARPS) {
        const float ln2 = 0.6931471805599453f;
        for (int idx = threadIdx.x; idx < nheads * DH; idx += DT_WARPS * 32) {
            const int hc = idx / DH, c = idx - hc * DH;
            float mx = -INFINITY;
            for (int j = 0; j < NSW; ++j) mx = fmaxf(mx, sm_m[j * GC + hc]);
            float den = 0.f, acc = 0.f;
            if (mx != -INFINITY) {
                for (int j = 0; j < NSW; ++j) {
                    const float mj = sm_m[j * GC + hc];
                    if (mj == -INFINITY) continue;
                    const float w = exp2f(mj - mx);
                    den += sm_l[j * GC + hc] * w;
                    acc += sm_o[(j * GC + hc) * DH + c] * w;
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
    for (int idx = threadIdx.x; idx < nheads * DH; idx += DT_THREADS) {
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

template <int DH, int GC>
static int decode_tma_launch(DecodeTmaArgs a, int nt, cudaStream_t s) {
    constexpr int NSW = DT_WARPS * 32 / (DH / 8);
    const size_t stage = (size_t)2 * TB_PAGE * DH * 2;
    const size_t tail = 2 * DT_MAX_STAGES * 8 + (size_t)(NSW * GC * DH + 2 * NSW * GC) * sizeof(float);
    // about half of an SM's shared memory per block: two blocks per SM keep their rings in flight together
    int stages = (int)((110 * 1024 - 1024 - tail) / stage);
    if (stages > DT_MAX_STAGES) stages = DT_MAX_STAGES;
    if (stages < 2) stages = 2;
    a.stages = stages;
    const size_t smem = stage * stages + tail + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<DH, GC>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = a.nh / a.nkvh;
    dim3 grid(nt, a.nkvh * ((group + GC - 1) / GC), a.splits);
    TB_LAUNCH((attention_decode_tma_kernel<DH, GC>), grid, DT_THREADS, smem, s, a);
    return tb_last_error();
}

extern "C" int tb_attention_decode_tma_bf16(const void* q, void* out, const void* kc, const void* vc, const int* tok_seq,
                                            const int* tok_pos, const int* page_table, float* partial,
                                            unsigned* done, int nt, int max_pages, int q_stride, int nh, int nkvh, int dh, int splits,
                                            float scale, cudaStream_t s) {
    if (nh <= 0 || nkvh <= 0 || nh % nkvh || splits < 1) return TB_ERR_ARG;
    if (splits > 1 && !partial) return TB_ERR_ARG;
    if (dh != 64 && dh != 128) return TB_ERR_UNSUPPORTED;
    if (q_stride % 8 || (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc) & 15)) return TB_ERR_UNSUPPORTED;
    if (nt <= 0) return nt == 0 ? 0 : TB_ERR_ARG;
    int rc = 0;
    int* err = tc_error_ptr();
    if (!err) return tb_last_error();
    DecodeTmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, tok_seq, tok_pos, page_table, partial, done, err,
                    max_pages, q_stride, nh, nkvh, splits, 0, scale * 1.4426950408889634f};
    const int group = nh / nkvh;
    const int gc = group == 1 ? 1 : group == 2 ? 2 : 4;
    if (dh == 64)
        rc = gc == 1 ? decode_tma_launch<64, 1>(a, nt, s)
                     : gc == 2 ? decode_tma_launch<64, 2>(a, nt, s) : decode_tma_launch<64, 4>(a, nt, s);
    else
        rc = gc == 1 ? decode_tma_launch<128, 1>(a, nt, s)
                     : gc == 2 ? decode_tma_launch<128, 2>(a, nt, s) : decode_tma_launch<128, 4>(a, nt, s);
    if (rc) return rc;
    if (splits > 1 && !done) {
        dim3 grid(nt, nh);
        TB_LAUNCH((attention_merge_kernel<__nv_bfloat16>), grid, dh < 128 ? 64 : 128, 0, s, partial,
                  (__nv_bfloat16*)out, nh, dh, splits, tok_pos);
        rc = tb_last_error();
    }
    return rc;
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_attention_decode_tma_bf16)
