// tb_attention_split_static: split-key attention whose scratch memory lives in the library.
// See no_alloc.h for who this is for and the rules of use.  No counterpart in the reference.
#include <mutex>

#include "attention_kernels.cuh"
#include "no_alloc.h"

// The scratch itself.  In host code this name is only a handle for the runtime's symbol calls, not
// a device address: a kernel must be given the address that cudaGetSymbolAddress returns.
static __device__ __align__(256) float tb_static_scratch[TB_STATIC_SCRATCH_BYTES / sizeof(float)];

#define TB_MAX_DEVICES 64
static float* g_scratch_addr[TB_MAX_DEVICES];   // device address of the array on each device
static std::mutex g_scratch_lock;

// Once per device, with that device current: ask the runtime where the array lives there.
static int scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= TB_MAX_DEVICES) return TB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> hold(g_scratch_lock);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, tb_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_addr[dev];
    return 0;
}

extern "C" int tb_attention_split_static(const void* q, void* out, const void* kc, const void* vc,
                                         const int* tile_seq, const int* tile_t0, const int* tile_nq,
                                         const int* tok_pos, const int* page_table, int tiles, int nt, int max_pages,
                                         int q_stride, int nh, int nkvh, int dh, int splits, float scale, int is_bf16,
                                         cudaStream_t stream) {
    if (nt < 0 || nh <= 0 || dh <= 0 || splits < 1) return TB_ERR_ARG;
    float* scratch = nullptr;
    if (splits > 1) {
        const unsigned long long need = (unsigned long long)nt * nh * splits * (dh + 2) * sizeof(float);
        if (need > TB_STATIC_SCRATCH_BYTES) return TB_ERR_TOO_LARGE;
        const int rc = scratch_address(&scratch);
        if (rc) return rc;
    }
    AttnArgs a{q, out, kc, vc, tile_seq, tile_t0, tile_nq, tok_pos, page_table, scratch,
               max_pages, q_stride, nh, nkvh, dh, 0, splits, scale};
    return is_bf16 ? attention_launch<__nv_bfloat16>(a, tiles, nt, stream) : attention_launch<float>(a, tiles, nt, stream);
}
