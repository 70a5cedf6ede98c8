// Attention for decoding: one query token per block against its sequence's cache, at the speed
// the cache can be read.
//
// Same mathematics as the general kernel (attention_kernels.cuh): score = q.k / sqrt(dh) over the
// positions <= the token's own, softmax and P.V in float, query head h reads key/value head
// h / (nh / nkvh).  What differs is the work split, made for one query row per head:
//
//   * a block = (token, key/value head, up to GC of its query heads, one slice of the keys);
//   * a key row is read by a "sub-warp" of dh / EPL lanes, each lane one 16-byte load (EPL = 8
//     bfloat16 or 4 float values); the 128 threads of a block form 128 / (dh / EPL) sub-warps that
//     take consecutive keys, so a block streams whole 64-token pages with full-width loads;
//   * every sub-warp runs its own online softmax (running max, sum, output slice) over its keys,
//     four keys at a time, the next four already in flight; the sub-warps are merged once at the end through shared memory;
//   * with several key slices the block writes (unnormalised output, max, sum) per slice in the
//     layout of the general kernel and attention_merge_kernel combines them.
//
// Head sizes whose sub-warp is a power of two lanes (bfloat16: 16, 32, 64, 128, 256; float: 16,
// 32, 64, 128) are taken; the launcher answers TB_ERR_UNSUPPORTED for others and the caller uses
// the general kernel.
#include "attention_kernels.cuh"

#define AD_THREADS 128
#define AD_UNROLL 4

struct DecodeArgs {
    const void* q;          // [nt, q_stride]
    void* out;              // [nt, nh * dh]
    const void* kc;         // [pages, nkvh, TB_PAGE, dh]
    const void* vc;
    const int* tok_seq;     // [nt] row of page_table
    const int* tok_pos;     // [nt]
    const int* page_table;  // [B, max_pages]
    float* partial;         // [nt, nh, splits, dh + 2] when splits > 1
    int max_pages, q_stride, nh, nkvh, dh, splits;
    float scale_log2e;      // log2(e) / sqrt(dh)
};

template <typename T, int GC>
__global__ void __launch_bounds__(AD_THREADS) attention_decode_kernel(const DecodeArgs a) {
    pdl_sync();
    constexpr int EPL = Vec16<T>::N;
    extern __shared__ __align__(16) float sm[];
    const int dh = a.dh;
    const int tpk = dh / EPL;                  // lanes per key (power of two, <= 32)
    const int nsw = AD_THREADS / tpk;          // sub-warps in the block
    const int sw = threadIdx.x / tpk;          // my sub-warp
    const int li = threadIdx.x % tpk;          // my lane in it: channels li * EPL .. + EPL
    float* sm_o = sm;                          // [nsw][GC][dh]
    float* sm_m = sm_o + (size_t)nsw * GC * dh;   // [nsw][GC]
    float* sm_l = sm_m + nsw * GC;             // [nsw][GC]

    const int t = blockIdx.x;
    const int group = a.nh / a.nkvh;
    const int chunks = (group + GC - 1) / GC;
    const int g = blockIdx.y / chunks;
    const int h0 = g * group + (blockIdx.y % chunks) * GC;
    const int nheads = min(GC, g * group + group - h0);
    const int split = blockIdx.z;
    const int b = a.tok_seq[t], pos = a.tok_pos[t];
    const int n_keys = pos + 1;
    const int n_pages = pos / TB_PAGE + 1, slices = decode_slices(n_pages, a.splits);
    if (split >= slices) return;
    const int per = (n_pages + slices - 1) / slices * TB_PAGE;
    const int k_lo = split * per, k_hi = min(n_keys, k_lo + per);

    const T* qg = static_cast<const T*>(a.q) + (size_t)t * a.q_stride + (size_t)h0 * dh + li * EPL;
    float q[GC][EPL], o[GC][EPL], m[GC], l[GC];
#pragma unroll
    for (int hc = 0; hc < GC; ++hc) {
        m[hc] = -INFINITY;
        l[hc] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            o[hc][e] = 0.f;
            q[hc][e] = 0.f;
        }
        if (hc < nheads) {
            Vec16<T>::load(qg + (size_t)hc * dh, q[hc]);
#pragma unroll
            for (int e = 0; e < EPL; ++e) q[hc][e] *= a.scale_log2e;
        }
    }
    const T* kc = static_cast<const T*>(a.kc);
    const T* vc = static_cast<const T*>(a.vc);
    // the pages of this block's key slice, once, into shared memory
    int* sm_pages = reinterpret_cast<int*>(sm_l + nsw * GC);
    {
        const int* pt = a.page_table + (size_t)b * a.max_pages;
        const int p_lo = k_lo / TB_PAGE, p_hi = (k_hi + TB_PAGE - 1) / TB_PAGE;
        for (int i = p_lo + threadIdx.x; i < p_hi; i += blockDim.x) sm_pages[i - p_lo] = pt[i];
    }
    __syncthreads();
    const int page0 = k_lo / TB_PAGE;
    const size_t lane_off = (size_t)li * EPL;

    // raw 16-byte loads for the AD_UNROLL keys of one round; keys past the slice load nothing
    auto fetch = [&](int base, uint4 (&kr)[AD_UNROLL], uint4 (&vr)[AD_UNROLL]) {
#pragma unroll
        for (int u = 0; u < AD_UNROLL; ++u) {
            const int key = base + sw + u * nsw;
            kr[u] = make_uint4(0u, 0u, 0u, 0u);
            vr[u] = make_uint4(0u, 0u, 0u, 0u);
            if (key < k_hi) {
                const int page = sm_pages[key / TB_PAGE - page0];
                const size_t off = (((size_t)page * a.nkvh + g) * TB_PAGE + (key % TB_PAGE)) * dh + lane_off;
                kr[u] = *reinterpret_cast<const uint4*>(kc + off);
                vr[u] = *reinterpret_cast<const uint4*>(vc + off);
            }
        }
    };

    uint4 kr[AD_UNROLL], vr[AD_UNROLL];
    fetch(k_lo, kr, vr);
    // the trip count is the same for every lane of a warp (the shuffles below need all of them)
    for (int base = k_lo; base < k_hi; base += nsw * AD_UNROLL) {
        float kf[AD_UNROLL][EPL], vf[AD_UNROLL][EPL];
        bool live[AD_UNROLL];
#pragma unroll
        for (int u = 0; u < AD_UNROLL; ++u) {
            live[u] = base + sw + u * nsw < k_hi;
            Vec16<T>::unpack(kr[u], kf[u]);
            Vec16<T>::unpack(vr[u], vf[u]);
        }
        fetch(base + nsw * AD_UNROLL, kr, vr);     // the next round's loads fly while this one is computed
#pragma unroll
        for (int hc = 0; hc < GC; ++hc) {
            if (hc >= nheads) continue;
            float s[AD_UNROLL];
#pragma unroll
            for (int u = 0; u < AD_UNROLL; ++u) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) d += q[hc][e] * kf[u][e];
                for (int w = tpk >> 1; w > 0; w >>= 1) d += __shfl_xor_sync(0xffffffffu, d, w);
                s[u] = live[u] ? d : -INFINITY;
            }
            float m_new = m[hc];
#pragma unroll
            for (int u = 0; u < AD_UNROLL; ++u) m_new = fmaxf(m_new, s[u]);
            const float mref = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = exp2f(m[hc] - mref);
            float psum = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[hc][e] *= corr;
#pragma unroll
            for (int u = 0; u < AD_UNROLL; ++u) {
                const float p = exp2f(s[u] - mref);
                psum += p;
#pragma unroll
                for (int e = 0; e < EPL; ++e) o[hc][e] += p * vf[u][e];
            }
            l[hc] = l[hc] * corr + psum;
            m[hc] = m_new;
        }
    }

    // merge the sub-warps
#pragma unroll
    for (int hc = 0; hc < GC; ++hc) {
        if (hc >= nheads) continue;
#pragma unroll
        for (int e = 0; e < EPL; ++e) sm_o[((size_t)sw * GC + hc) * dh + li * EPL + e] = o[hc][e];
        if (li == 0) {
            sm_m[sw * GC + hc] = m[hc];
            sm_l[sw * GC + hc] = l[hc];
        }
    }
    __syncthreads();
    const float ln2 = 0.6931471805599453f;
    for (int idx = threadIdx.x; idx < nheads * dh; idx += blockDim.x) {
        const int hc = idx / dh, c = idx - hc * dh;
        float mx = -INFINITY;
        for (int j = 0; j < nsw; ++j) mx = fmaxf(mx, sm_m[j * GC + hc]);
        float den = 0.f, acc = 0.f;
        if (mx != -INFINITY) {
            for (int j = 0; j < nsw; ++j) {
                const float mj = sm_m[j * GC + hc];
                if (mj == -INFINITY) continue;
                const float w = exp2f(mj - mx);
                den += sm_l[j * GC + hc] * w;
                acc += sm_o[((size_t)j * GC + hc) * dh + c] * w;
            }
        }
        const int h = h0 + hc;
        if (a.splits == 1) {
            stf(static_cast<T*>(a.out) + ((size_t)t * a.nh + h) * dh + c, acc / den);
        } else {
            float* dst = a.partial + (((size_t)t * a.nh + h) * a.splits + split) * (dh + 2);
            dst[c] = acc;
            if (c == 0) {
                dst[dh] = mx == -INFINITY ? -INFINITY : mx * ln2;   // natural-log units, as the merge kernel expects
                dst[dh + 1] = den;
            }
        }
    }
}

template <typename T, int GC>
static int decode_launch_gc(const DecodeArgs& a, int nt, cudaStream_t s) {
    constexpr int EPL = Vec16<T>::N;
    const int tpk = a.dh / EPL, nsw = AD_THREADS / tpk;
    const size_t smem = ((size_t)nsw * GC * a.dh + 2 * (size_t)nsw * GC) * sizeof(float) + (size_t)a.max_pages * sizeof(int);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<T, GC>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int group = a.nh / a.nkvh;
    dim3 grid(nt, a.nkvh * ((group + GC - 1) / GC), a.splits);
    TB_LAUNCH((attention_decode_kernel<T, GC>), grid, AD_THREADS, smem, s, a);
    return tb_last_error();
}

template <typename T>
static int decode_launch(const DecodeArgs& a, int nt, cudaStream_t s) {
    constexpr int EPL = Vec16<T>::N;
    if (a.nh <= 0 || a.nkvh <= 0 || a.nh % a.nkvh || a.splits < 1) return TB_ERR_ARG;
    if (a.splits > 1 && !a.partial) return TB_ERR_ARG;
    if (a.dh <= 0 || a.dh % EPL) return TB_ERR_UNSUPPORTED;
    const int tpk = a.dh / EPL;
    if (tpk > 32 || (tpk & (tpk - 1))) return TB_ERR_UNSUPPORTED;
    if (a.q_stride % EPL) return TB_ERR_UNSUPPORTED;
    if (nt <= 0) return nt == 0 ? 0 : TB_ERR_ARG;
    const int group = a.nh / a.nkvh;
    int rc;
    if (group == 1)
        rc = decode_launch_gc<T, 1>(a, nt, s);
    else if (group == 2)
        rc = decode_launch_gc<T, 2>(a, nt, s);
    else
        rc = decode_launch_gc<T, 4>(a, nt, s);
    if (rc) return rc;
    if (a.splits > 1) {
        dim3 grid(nt, a.nh);
        TB_LAUNCH((attention_merge_kernel<T>), grid, a.dh < 128 ? 64 : 128, 0, s, a.partial, (T*)a.out, a.nh, a.dh, a.splits,
                  a.tok_pos);
        rc = tb_last_error();
    }
    return rc;
}

extern "C" {
#define TB_ATT_DECODE(NAME, T)                                                                                     \
    int NAME(const void* q, void* out, const void* kc, const void* vc, const int* tok_seq, const int* tok_pos,    \
             const int* page_table, float* partial, int nt, int max_pages, int q_stride, int nh, int nkvh, int dh, \
             int splits, float scale, cudaStream_t s) {                                                            \
        DecodeArgs a{q, out, kc, vc, tok_seq, tok_pos, page_table, partial, max_pages, q_stride, nh, nkvh, dh,     \
                     splits, scale * 1.4426950408889634f};                                                         \
        return decode_launch<T>(a, nt, s);                                                                          \
    }
TB_ATT_DECODE(tb_attention_decode_f32, float)
TB_ATT_DECODE(tb_attention_decode_bf16, __nv_bfloat16)
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_attention_decode_f32)
TB_TAPE_REGISTER(tb_attention_decode_bf16)
