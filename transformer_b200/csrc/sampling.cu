// Sampling from one row of float logits per block: argmax, or temperature / top-k / top-p and an
// inverse-CDF draw with a uniform number the caller supplies.
//
// The reference hands one logits row, SampleArgs{temperature, top_p, top_k} and one uniform
// number to an external operator and gets back {index, value}
// (tensor/src/operators/random_sample.rs:64-75; temperature 0 is the default and means argmax,
// test-utils/src/lib.rs:78-80).  The rules chosen here, in this order:
//   1. temperature == 0 or top_k == 1: the largest logit, the lowest id among equals;
//   2. z = logit / temperature;
//   3. keep the top_k largest z (0 = all); equals at the edge: lower ids first;
//   4. p = softmax over the kept;
//   5. keep the shortest prefix, in descending p (equals: lower ids first), whose mass >= top_p;
//   6. draw in ASCENDING id order: the first kept id whose running mass exceeds u * (kept mass).
// Selection of the edges is exact (a radix select over the order-preserving bit pattern of z),
// so no sort and no scratch memory is needed; every pass reads the row again (it sits in L2).
#include "common.cuh"

#define SAMP_THREADS 1024

__device__ __forceinline__ unsigned order_key(float z) {   // larger float <=> larger unsigned
    unsigned b = __float_as_uint(z);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Cut {        // the set {key > key_cut} plus {key == key_cut and id <= id_cut}
    unsigned key;
    int id;
};
__device__ __forceinline__ bool in_cut(const Cut& c, unsigned key, int id) {
    return key > c.key || (key == c.key && id <= c.id);
}

// Find the cut that keeps, in descending key order inside `outer`, the shortest prefix whose
// count reaches need_count (by_mass = false) or whose mass reaches need_mass (by_mass = true).
// mass(i) = exp(z_i - zmax).  Shared arrays: hist_c[256], hist_m[256], misc.
__device__ Cut select_cut(const float* __restrict__ row, int V, float inv_t, float zmax, const Cut outer,
                          bool by_mass, int need_count, float need_mass, int* hist_c, float* hist_m,
                          int* sh_i, float* sh_f) {
    unsigned prefix = 0, mask = 0;
    int count_gt = 0;       // kept so far (strictly above the current prefix range)
    float mass_gt = 0.f;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            hist_c[i] = 0;
            hist_m[i] = 0.f;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float z = row[i] * inv_t;
            const unsigned key = order_key(z);
            if ((key & mask) == prefix && in_cut(outer, key, i)) {
                const int bin = (key >> shift) & 255;
                atomicAdd(&hist_c[bin], 1);
                if (by_mass) atomicAdd(&hist_m[bin], expf(z - zmax));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int bin = 255;
            for (; bin > 0; --bin) {
                if (hist_c[bin] == 0) continue;
                const bool reached = by_mass ? (mass_gt + hist_m[bin] >= need_mass)
                                             : (count_gt + hist_c[bin] >= need_count);
                if (reached) break;
                count_gt += hist_c[bin];
                mass_gt += hist_m[bin];
            }
            sh_i[0] = bin;
            sh_i[1] = count_gt;
            sh_f[0] = mass_gt;
        }
        __syncthreads();
        prefix |= (unsigned)sh_i[0] << shift;
        mask |= 255u << shift;
        count_gt = sh_i[1];
        mass_gt = sh_f[0];
        __syncthreads();
    }
    // `prefix` is now the key at the edge.  How many of its equals (lowest ids first) are kept?
    // Count them, then find the id of the last one kept by bisection over the id range.
    int n_eq = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const unsigned key = order_key(row[i] * inv_t);
        if (key == prefix && in_cut(outer, key, i)) ++n_eq;
    }
    {
        __syncthreads();
        if (threadIdx.x == 0) sh_i[2] = 0;
        __syncthreads();
        if (n_eq) atomicAdd(&sh_i[2], n_eq);
        __syncthreads();
        n_eq = sh_i[2];
    }
    int keep_eq;
    if (by_mass) {
        unsigned b = prefix;   // invert order_key to get z at the edge
        b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
        const float pe = expf(__uint_as_float(b) - zmax);
        const float lack = need_mass - mass_gt;
        keep_eq = pe > 0.f ? (int)ceilf(lack / pe) : n_eq;
    } else {
        keep_eq = need_count - count_gt;
    }
    keep_eq = max(1, min(keep_eq, n_eq));
    Cut c{prefix, V - 1};
    if (keep_eq < n_eq) {
        int lo = 0, hi = V - 1;   // smallest id such that #equals with id <= it == keep_eq
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            __syncthreads();
            if (threadIdx.x == 0) sh_i[2] = 0;
            __syncthreads();
            int n = 0;
            for (int i = threadIdx.x; i <= mid; i += blockDim.x) {
                const unsigned key = order_key(row[i] * inv_t);
                if (key == prefix && in_cut(outer, key, i)) ++n;
            }
            if (n) atomicAdd(&sh_i[2], n);
            __syncthreads();
            if (sh_i[2] >= keep_eq) hi = mid; else lo = mid + 1;
        }
        c.id = lo;
    }
    if (outer.key == prefix) c.id = min(c.id, outer.id);
    return c;
}

// logits [rows, V] float (row stride ld); u [rows] uniform numbers in [0, 1);
// out_idx [rows], out_val [rows] (the chosen token's logit).
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ u, int V, float temperature,
              int top_k, float top_p, int* __restrict__ out_idx, float* __restrict__ out_val) {
    pdl_sync();
    __shared__ float red_f[SAMP_THREADS];
    __shared__ int red_i[SAMP_THREADS];
    __shared__ int hist_c[256];
    __shared__ float hist_m[256];
    __shared__ int sh_i[4];
    __shared__ float sh_f[4];
    const float* row = logits + (size_t)blockIdx.x * ld;
    const int tid = threadIdx.x;

    // argmax with the lowest id among equals
    float best = -INFINITY;
    int bi = 0x7fffffff;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // four 16-byte loads in flight per thread: the row is read once and what it costs is latency
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = V >> 2;
        for (int i0 = tid; i0 < n4; i0 += 4 * blockDim.x) {
            float4 q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * blockDim.x;
                q[j] = i < n4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {       // ascending ids within the thread: strictly greater keeps the lowest
                const int i = (i0 + j * blockDim.x) << 2;
                if (q[j].x > best) { best = q[j].x; bi = i; }
                if (q[j].y > best) { best = q[j].y; bi = i + 1; }
                if (q[j].z > best) { best = q[j].z; bi = i + 2; }
                if (q[j].w > best) { best = q[j].w; bi = i + 3; }
            }
        }
        done = n4 << 2;
    }
    for (int i = done + tid; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
        }
    }
    red_f[tid] = best;
    red_i[tid] = bi;
    __syncthreads();
    for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
        if (tid < o) {
            const float ov = red_f[tid + o];
            const int oi = red_i[tid + o];
            if (ov > red_f[tid] || (ov == red_f[tid] && oi < red_i[tid])) {
                red_f[tid] = ov;
                red_i[tid] = oi;
            }
        }
        __syncthreads();
    }
    const float vmax = red_f[0];
    const int imax = red_i[0] < V ? red_i[0] : 0;
    __syncthreads();
    if (temperature == 0.f || top_k == 1) {
        if (tid == 0) {
            out_idx[blockIdx.x] = imax;
            out_val[blockIdx.x] = vmax;
        }
        return;
    }
    const float inv_t = 1.0f / temperature;
    const float zmax = vmax * inv_t;
    Cut cut{0u, V - 1};   // everything
    if (top_k > 0 && top_k < V)
        cut = select_cut(row, V, inv_t, zmax, cut, false, top_k, 0.f, hist_c, hist_m, sh_i, sh_f);
    if (top_p < 1.0f) {
        float mass = 0.f;
        for (int i = tid; i < V; i += blockDim.x) {
            const float z = row[i] * inv_t;
            if (in_cut(cut, order_key(z), i)) mass += expf(z - zmax);
        }
        mass = block_sum(mass, red_f);
        __syncthreads();
        cut = select_cut(row, V, inv_t, zmax, cut, true, 0, top_p * mass, hist_c, hist_m, sh_i, sh_f);
    }
    // inverse CDF in ascending id: each thread owns one contiguous segment of ids
    const int seg = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min(V, tid * seg), hi = min(V, lo + seg);
    float mine = 0.f;
    int last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const float z = row[i] * inv_t;
        if (in_cut(cut, order_key(z), i)) {
            mine += expf(z - zmax);
            last_kept = i;
        }
    }
    __syncthreads();
    red_f[tid] = mine;
    red_i[tid] = last_kept;
    __syncthreads();
    if (tid == 0) {   // sequential scan over 1024 partial sums: fixed order, cheap
        float total = 0.f;
        for (int t = 0; t < (int)blockDim.x; ++t) total += red_f[t];
        const float target = u[blockIdx.x] * total;
        float run = 0.f;
        int owner = -1, fallback = -1;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (red_i[t] >= 0) fallback = t;
            if (owner < 0 && red_i[t] >= 0 && run + red_f[t] > target) {
                owner = t;
                sh_f[1] = run;
            }
            if (owner < 0) run += red_f[t];
        }
        if (owner < 0) {   // rounding left the target at or above the total: the last kept id
            owner = fallback;
            sh_f[1] = INFINITY;
        }
        sh_i[3] = owner;
        sh_f[2] = target;
    }
    __syncthreads();
    if (tid == sh_i[3]) {
        float run = sh_f[1];
        const float target = sh_f[2];
        int pick = last_kept;
        if (run != INFINITY) {
            for (int i = lo; i < hi; ++i) {
                const float z = row[i] * inv_t;
                if (in_cut(cut, order_key(z), i)) {
                    run += expf(z - zmax);
                    if (run > target) {
                        pick = i;
                        break;
                    }
                }
            }
        }
        out_idx[blockIdx.x] = pick;
        out_val[blockIdx.x] = row[pick];
    }
}

extern "C" int tb_sample(const float* logits, long long ld, const float* u, int rows, int V, float temperature,
                         int top_k, float top_p, int* out_idx, float* out_val, cudaStream_t s) {
    if (rows < 0 || V <= 0 || ld < V) return TB_ERR_ARG;
    if (!(temperature >= 0.f) || !(top_p > 0.f && top_p <= 1.f) || top_k < 0) return TB_ERR_ARG;
    if (rows == 0) return 0;
    TB_LAUNCH((sample_kernel), rows, SAMP_THREADS, 0, s, logits, ld, u, V, temperature, top_k, top_p, out_idx, out_val);
    return tb_last_error();
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_sample)
