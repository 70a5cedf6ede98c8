// Causal attention over the paged cache: the general kernel.
//
// It serves prompts (many query tokens per sequence), decoding (one) and anything between, in
// float or bfloat16 storage, for every head size that is a multiple of 16 up to 256 and any number
// of heads and groups.  All arithmetic is float: scores, running maximum, sum and the output
// accumulator (flash form, no score matrix in memory).  The keys and values of the step's own
// tokens are already in the cache when it runs (rope_cache.cu wrote them).
//
//   score(q at position p, key at position j) = q.k / sqrt(dh),   visible iff j <= p
//   query head h reads key/value head h / (nh / nkvh)
// (models/llama/common/src/compute.rs:243-264; scale and mask are inside the reference's external
//  attention operator.)
//
// Work split: one block = one tile of query tokens of ONE sequence x one key/value head x up to 16
// of its query heads x one slice of the key range.  The block's rows (token, head) share every key
// tile in shared memory.  A warp owns rows warp, warp+4, ...; inside a warp the 32 lanes are 32
// keys for the scores and 32 output channels for P.V.
// With more than one key slice each block writes (max, sum, unnormalised output) and
// attention_merge_kernel combines them.
#pragma once
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_ROWS 16               // rows (token, head) per block
#define ATT_QPW (ATT_ROWS / ATT_WARPS)
#define ATT_KEYS 32               // keys per tile (divides TB_PAGE)

struct AttnArgs {
    const void* q;          // [nt, q_stride] first q head of each token
    void* out;              // [nt, nh * dh]
    const void* kc;         // [pages, nkvh, TB_PAGE, dh]
    const void* vc;
    const int* tile_seq;    // [tiles] sequence (row of page_table) of the tile
    const int* tile_t0;     // [tiles] first token (index in the step) of the tile
    const int* tile_nq;     // [tiles] tokens in the tile
    const int* tok_pos;     // [nt]
    const int* page_table;  // [B, max_pages]
    float* partial;         // [nt, nh, splits, dh + 2] when splits > 1
    int max_pages, q_stride, nh, nkvh, dh, hc /*heads per block*/, splits;
    float scale;
};

template <typename T, int DPL>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_kernel(const AttnArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dh = a.dh;
    const int kstride = dh + (sizeof(T) == 4 ? 1 : 2);   // odd word stride: lanes hit distinct banks
    float* qs = reinterpret_cast<float*>(smem_raw);                 // [ATT_ROWS][dh]
    T* ks = reinterpret_cast<T*>(qs + ATT_ROWS * dh);               // [ATT_KEYS][kstride]
    T* vs = ks + ATT_KEYS * kstride;                                // [ATT_KEYS][dh]

    const int tile = blockIdx.x;
    const int group = a.nh / a.nkvh;
    const int chunks = (group + a.hc - 1) / a.hc;
    const int g = blockIdx.y / chunks;                 // key/value head
    const int h0 = g * group + (blockIdx.y % chunks) * a.hc;   // first query head of the block
    const int nheads = min(a.hc, g * group + group - h0);
    const int split = blockIdx.z;
    const int b = a.tile_seq[tile], t0 = a.tile_t0[tile], nq = a.tile_nq[tile];
    const int rows = nq * nheads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* qg = static_cast<const T*>(a.q);

    // queries of the block, as float
    for (int idx = threadIdx.x; idx < rows * dh; idx += blockDim.x) {
        const int r = idx / dh, c = idx - r * dh;
        const int tq = r / nheads, hh = r - tq * nheads;
        qs[r * dh + c] = ldf(qg + (size_t)(t0 + tq) * a.q_stride + (size_t)(h0 + hh) * dh + c);
    }
    const int pos_first = a.tok_pos[t0];
    const int pos_last = pos_first + nq - 1;
    const int n_kt = pos_last / ATT_KEYS + 1;
    const int per = (n_kt + a.splits - 1) / a.splits;
    const int kt_lo = split * per, kt_hi = min(n_kt, kt_lo + per);

    float m[ATT_QPW], l[ATT_QPW], o[ATT_QPW][DPL];
#pragma unroll
    for (int i = 0; i < ATT_QPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) o[i][c] = 0.f;
    }
    const T* kc = static_cast<const T*>(a.kc);
    const T* vc = static_cast<const T*>(a.vc);

    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int key0 = kt * ATT_KEYS;
        const int page = a.page_table[(size_t)b * a.max_pages + key0 / TB_PAGE];
        const size_t base = (((size_t)page * a.nkvh + g) * TB_PAGE + (key0 % TB_PAGE)) * dh;
        __syncthreads();   // the previous tile is consumed (and qs is written, first time round)
        for (int idx = threadIdx.x; idx < ATT_KEYS * dh; idx += blockDim.x) {
            const int j = idx / dh, c = idx - j * dh;
            const bool live = key0 + j <= pos_last;
            ks[j * kstride + c] = live ? kc[base + idx] : T(0.f);
            vs[idx] = live ? vc[base + idx] : T(0.f);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < ATT_QPW; ++i) {
            const int r = warp + i * ATT_WARPS;
            if (r >= rows) continue;                       // uniform in the warp
            const int pos_r = pos_first + r / nheads;
            const float* qr = qs + r * dh;
            const T* kr = ks + lane * kstride;
            float s = 0.f;
            for (int c = 0; c < dh; ++c) s += qr[c] * ldf(kr + c);
            s = (key0 + lane <= pos_r) ? s * a.scale : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            if (m_new == -INFINITY) continue;              // no visible key yet for this row
            const float p = expf(s - m_new);               // exp(-inf) = 0 for masked keys
            const float corr = expf(m[i] - m_new);
            l[i] = l[i] * corr + warp_sum(p);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) o[i][c] *= corr;
            for (int j = 0; j < ATT_KEYS; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int c = 0; c < DPL; ++c) {
                    const int ch = lane + 32 * c;
                    if (ch < dh) o[i][c] += pj * ldf(vs + j * dh + ch);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < ATT_QPW; ++i) {
        const int r = warp + i * ATT_WARPS;
        if (r >= rows) continue;
        const int tq = r / nheads, hh = r - tq * nheads;
        const int t = t0 + tq, h = h0 + hh;
        if (a.splits == 1) {
            T* dst = static_cast<T*>(a.out) + (size_t)t * a.nh * dh + (size_t)h * dh;
            const float inv = 1.0f / l[i];
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int ch = lane + 32 * c;
                if (ch < dh) stf(dst + ch, o[i][c] * inv);
            }
        } else {
            float* dst = a.partial + (((size_t)t * a.nh + h) * a.splits + split) * (dh + 2);
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int ch = lane + 32 * c;
                if (ch < dh) dst[ch] = o[i][c];
            }
            if (lane == 0) {
                dst[dh] = m[i];
                dst[dh + 1] = l[i];
            }
        }
    }
}

// Slices into which a decode kernel cuts a sequence of n_pages pages: at most `splits` (the depth of its grid,
// a function of the batch's shape alone so that a captured graph can keep it) and none shorter than two pages.
// The kernels and the merge agree through this one function; blocks of slices beyond it write nothing.
__host__ __device__ inline int decode_slices(int n_pages, int splits) {
    const int s = n_pages / 2;
    return s < 1 ? 1 : s > splits ? splits : s;
}

// out[t, h, :] = sum_s o_s exp(m_s - m) / sum_s l_s exp(m_s - m),  m = max_s m_s.
// tok_pos (decoding) limits the sum to the slices that the token's sequence was cut into.
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, int nh, int dh,
                                       int splits, const int* __restrict__ tok_pos) {
    pdl_sync();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* p = partial + ((size_t)t * nh + h) * splits * (dh + 2);
    if (tok_pos) splits = decode_slices(tok_pos[t] / TB_PAGE + 1, splits);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, p[s * (dh + 2) + dh]);
    float den = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = p[s * (dh + 2) + dh];
        if (ms != -INFINITY) den += p[s * (dh + 2) + dh + 1] * expf(ms - m);
    }
    for (int c = threadIdx.x; c < dh; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = p[s * (dh + 2) + dh];
            if (ms != -INFINITY) acc += p[s * (dh + 2) + c] * expf(ms - m);
        }
        stf(out + ((size_t)t * nh + h) * dh + c, acc / den);
    }
}

static size_t attention_smem(int dh, size_t elem) {
    const int kstride = dh + (elem == 4 ? 1 : 2);
    return (size_t)ATT_ROWS * dh * 4 + (size_t)ATT_KEYS * kstride * elem + (size_t)ATT_KEYS * dh * elem;
}

template <typename T, int DPL>
static int attention_launch_dpl(const AttnArgs& a, int tiles, cudaStream_t s) {
    const size_t smem = attention_smem(a.dh, sizeof(T));
    static size_t configured = 0;   // per instantiation
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_kernel<T, DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int group = a.nh / a.nkvh;
    const int chunks = (group + a.hc - 1) / a.hc;
    dim3 grid(tiles, a.nkvh * chunks, a.splits);
    TB_LAUNCH((attention_kernel<T, DPL>), grid, ATT_WARPS * 32, smem, s, a);
    return tb_last_error();
}

template <typename T>
static int attention_launch(AttnArgs a, int tiles, int nt, cudaStream_t s) {
    if (a.nh <= 0 || a.nkvh <= 0 || a.nh % a.nkvh) return TB_ERR_ARG;
    if (a.dh <= 0 || a.dh % 16 || a.dh > 256) return TB_ERR_UNSUPPORTED;
    if (a.splits < 1 || (a.splits > 1 && !a.partial)) return TB_ERR_ARG;
    if (tiles <= 0 || nt <= 0) return tiles == 0 || nt == 0 ? 0 : TB_ERR_ARG;
    const int group = a.nh / a.nkvh;
    a.hc = group < ATT_ROWS ? group : ATT_ROWS;
    int rc;
    switch ((a.dh + 31) / 32) {
        case 1: rc = attention_launch_dpl<T, 1>(a, tiles, s); break;
        case 2: rc = attention_launch_dpl<T, 2>(a, tiles, s); break;
        case 3: rc = attention_launch_dpl<T, 3>(a, tiles, s); break;
        case 4: rc = attention_launch_dpl<T, 4>(a, tiles, s); break;
        case 5: rc = attention_launch_dpl<T, 5>(a, tiles, s); break;
        case 6: rc = attention_launch_dpl<T, 6>(a, tiles, s); break;
        case 7: rc = attention_launch_dpl<T, 7>(a, tiles, s); break;
        default: rc = attention_launch_dpl<T, 8>(a, tiles, s); break;
    }
    if (rc) return rc;
    if (a.splits > 1) {
        dim3 grid(nt, a.nh);
        TB_LAUNCH((attention_merge_kernel<T>), grid, a.dh < 128 ? 64 : 128, 0, s, a.partial, (T*)a.out, a.nh, a.dh, a.splits,
                  (const int*)nullptr);
        rc = tb_last_error();
    }
    return rc;
}

