// Rotary position encoding of q and k, fused with the write of k and v into the paged cache.
//
// qkv is [nt, (nh + 2 nkvh) dh] with the heads ordered q, k, v
// (models/llama/common/src/compute.rs:225-227).  q is rotated in place; k is rotated and stored,
// v is copied, into the page that holds the token's position
// (the reference stores k, v at pos..pos+seq of the request's cache, compute.rs:244-263).
// Angles come from a float table [positions, dh/2] built on the host in double precision:
// angle(p, i) = p * theta^(-2i/dh).
//
// Cache of one layer: K and V each [pages, nkvh, TB_PAGE, dh].
#include "common.cuh"

#define ROPE_HEADS 4   // heads per block when there are few tokens; 32 (a full block of 16-byte items) for prompts

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                  int max_pages, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, T* __restrict__ kc, T* __restrict__ vc,
                                  int nh, int nkvh, int dh, int half_pairing, int hpb) {
    pdl_sync();
    // grid: (token, chunk of hpb heads out of q heads, k heads, v heads in that order)
    const int t = blockIdx.x;
    const int head_lo = blockIdx.y * hpb;
    const int head_hi = min(head_lo + hpb, nh + 2 * nkvh);
    const int pos = tok_pos[t];
    const int half = dh >> 1;
    T* row = qkv + (size_t)t * (nh + 2 * nkvh) * dh;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    size_t cache_row = 0;
    if (kc) {
        const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
        cache_row = ((size_t)page * nkvh * TB_PAGE + (pos % TB_PAGE)) * dh;  // + g * TB_PAGE * dh
    }
    const int rot_hi = min(head_hi, nh + nkvh);
    for (int idx = threadIdx.x; idx < (rot_hi - head_lo) * half; idx += blockDim.x) {
        const int head = head_lo + idx / half, i = idx % half;
        const int i0 = half_pairing ? i : 2 * i;
        const int i1 = half_pairing ? i + half : 2 * i + 1;
        T* h = row + (size_t)head * dh;
        const float x0 = ldf(h + i0), x1 = ldf(h + i1);
        const float c = cs[i], s = sn[i];
        const float y0 = x0 * c - x1 * s;
        const float y1 = x0 * s + x1 * c;
        if (head < nh) {
            stf(h + i0, y0);
            stf(h + i1, y1);
        } else if (kc) {
            T* dst = kc + cache_row + (size_t)(head - nh) * TB_PAGE * dh;
            stf(dst + i0, y0);
            stf(dst + i1, y1);
        }
    }
    if (vc && head_hi > nh + nkvh) {
        const int v_lo = max(head_lo, nh + nkvh);
        for (int idx = threadIdx.x; idx < (head_hi - v_lo) * dh; idx += blockDim.x) {
            const int head = v_lo + idx / dh, c = idx % dh;
            vc[cache_row + (size_t)(head - nh - nkvh) * TB_PAGE * dh + c] = row[(size_t)head * dh + c];
        }
    }
}

// The same with 8 values per thread and 16-byte accesses (head sizes that are a multiple of 16).  EARLY (a few
// tokens: decoding) reads the angles before the dependency wait; with many tokens the kernel is bound by memory
// traffic and does better with the registers that would cost.
template <typename T, bool EARLY>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, const int* __restrict__ tok_seq,
                                      const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                      int max_pages, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, T* __restrict__ kc, T* __restrict__ vc,
                                      int nh, int nkvh, int dh, int half_pairing, int hpb) {
    // Positions and the angle table were there before the step began: the angles of this thread's first item are
    // read before the wait for the kernel that wrote q, k and v (the table is touched once per layer and has
    // left L2 since the last step).
    const int t = blockIdx.x;
    const int head_lo = blockIdx.y * hpb;
    const int head_hi = min(head_lo + hpb, nh + 2 * nkvh);
    const int pos = tok_pos[t];
    const int half = dh >> 1;
    T* row = qkv + (size_t)t * (nh + 2 * nkvh) * dh;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    float c0[8], s0[8];
    if (EARLY) {
        const int u = threadIdx.x % (dh / 16);
        load8(cs + u * 8, c0);
        load8(sn + u * 8, s0);
    }
    size_t cache_row = 0;
    if (kc) {
        const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
        cache_row = ((size_t)page * nkvh * TB_PAGE + (pos % TB_PAGE)) * dh;
    }
    pdl_sync();
    const int rot_hi = min(head_hi, nh + nkvh);
    const int units = dh / 16;                 // work items per head: 16 values = 8 pairs each
    for (int idx = threadIdx.x; idx < (rot_hi - head_lo) * units; idx += blockDim.x) {
        const int head = head_lo + idx / units, u = idx % units;
        T* h = row + (size_t)head * dh;
        T* dst = head < nh ? h : (kc ? kc + cache_row + (size_t)(head - nh) * TB_PAGE * dh : nullptr);
        float a[8], b[8], c[8], s[8], ya[8], yb[8];
        if (EARLY && idx == (int)threadIdx.x) {   // the item whose angles are in registers already
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                c[e] = c0[e];
                s[e] = s0[e];
            }
        } else {
            load8(cs + u * 8, c);              // pairs 8u .. 8u+7
            load8(sn + u * 8, s);
        }
        if (half_pairing) {                    // pair i = (x[i], x[i + half])
            load8(h + u * 8, a);
            load8(h + half + u * 8, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ya[e] = a[e] * c[e] - b[e] * s[e];
                yb[e] = a[e] * s[e] + b[e] * c[e];
            }
            if (dst) {
                store8(dst + u * 8, ya);
                store8(dst + half + u * 8, yb);
            }
        } else {                               // pair i = (x[2i], x[2i+1]): 16 consecutive values
            load8(h + u * 16, a);
            load8(h + u * 16 + 8, b);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                ya[2 * e] = a[2 * e] * c[e] - a[2 * e + 1] * s[e];
                ya[2 * e + 1] = a[2 * e] * s[e] + a[2 * e + 1] * c[e];
                yb[2 * e] = b[2 * e] * c[4 + e] - b[2 * e + 1] * s[4 + e];
                yb[2 * e + 1] = b[2 * e] * s[4 + e] + b[2 * e + 1] * c[4 + e];
            }
            if (dst) {
                store8(dst + u * 16, ya);
                store8(dst + u * 16 + 8, yb);
            }
        }
    }
    if (vc && head_hi > nh + nkvh) {
        const int v_lo = max(head_lo, nh + nkvh);
        const int per = dh / 8;
        for (int idx = threadIdx.x; idx < (head_hi - v_lo) * per; idx += blockDim.x) {
            const int head = v_lo + idx / per, c8 = (idx % per) * 8;
            float f[8];
            load8(row + (size_t)head * dh + c8, f);
            store8(vc + cache_row + (size_t)(head - nh - nkvh) * TB_PAGE * dh + c8, f);
        }
    }
}

template <typename T>
static int rope_cache_launch(void* qkv, const int* tok_seq, const int* tok_pos, const int* page_table,
                             int max_pages, const float* cos_t, const float* sin_t, void* kc, void* vc,
                             int nt, int nh, int nkvh, int dh, int half_pairing, cudaStream_t s) {
    if (nt < 0 || nh <= 0 || nkvh <= 0 || dh <= 0 || (dh & 1)) return TB_ERR_ARG;
    if ((kc == nullptr) != (vc == nullptr)) return TB_ERR_ARG;
    if (nt == 0) return 0;
    // few tokens (decoding): many small blocks, so that every SM has some; prompts: blocks of 256 full threads
    const int hpb = nt >= 256 ? 8 * ROPE_HEADS : ROPE_HEADS;
    dim3 grid(nt, (nh + 2 * nkvh + hpb - 1) / hpb);
    if (dh % 16 == 0 && (((uintptr_t)qkv | (uintptr_t)kc | (uintptr_t)vc) & 15) == 0) {
        int threads = (hpb * (dh / 16) + 31) / 32 * 32;
        threads = threads < 64 ? 64 : threads > 256 ? 256 : threads;
        if (nt < 256)
            TB_LAUNCH((rope_cache_vec_kernel<T, true>), grid, threads, 0, s, (T*)qkv, tok_seq, tok_pos, page_table,
                      max_pages, cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dh, half_pairing, hpb);
        else
            TB_LAUNCH((rope_cache_vec_kernel<T, false>), grid, threads, 0, s, (T*)qkv, tok_seq, tok_pos, page_table,
                      max_pages, cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dh, half_pairing, hpb);
        return tb_last_error();
    }
    TB_LAUNCH((rope_cache_kernel<T>), grid, nt >= 256 ? 256 : 128, 0, s, (T*)qkv, tok_seq, tok_pos, page_table, max_pages,
              cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dh, half_pairing, hpb);
    return tb_last_error();
}

extern "C" {
int tb_rope_cache_f32(void* qkv, const int* tok_seq, const int* tok_pos, const int* page_table, int max_pages,
                      const float* cos_t, const float* sin_t, void* kc, void* vc, int nt, int nh, int nkvh,
                      int dh, int half_pairing, cudaStream_t s) {
    return rope_cache_launch<float>(qkv, tok_seq, tok_pos, page_table, max_pages, cos_t, sin_t, kc, vc, nt, nh,
                                    nkvh, dh, half_pairing, s);
}
int tb_rope_cache_bf16(void* qkv, const int* tok_seq, const int* tok_pos, const int* page_table, int max_pages,
                       const float* cos_t, const float* sin_t, void* kc, void* vc, int nt, int nh, int nkvh,
                       int dh, int half_pairing, cudaStream_t s) {
    return rope_cache_launch<__nv_bfloat16>(qkv, tok_seq, tok_pos, page_table, max_pages, cos_t, sin_t, kc, vc,
                                            nt, nh, nkvh, dh, half_pairing, s);
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_rope_cache_f32)
TB_TAPE_REGISTER(tb_rope_cache_bf16)
