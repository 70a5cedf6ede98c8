// Entry points of the general attention kernel (see attention_kernels.cuh).
#include "attention_kernels.cuh"

extern "C" {
// Tokens of one sequence that one block takes: the host cuts each sequence's new tokens into
// tiles of this many.
int tb_attention_tile_tokens(int nh, int nkvh) {
    const int group = nh / nkvh;
    const int hc = group < ATT_ROWS ? group : ATT_ROWS;
    return ATT_ROWS / hc;
}
#define TB_ATTENTION(NAME, T)                                                                                       \
    int NAME(const void* q, void* out, const void* kc, const void* vc, const int* tile_seq, const int* tile_t0,    \
             const int* tile_nq, const int* tok_pos, const int* page_table, float* partial, int tiles, int nt,     \
             int max_pages, int q_stride, int nh, int nkvh, int dh, int splits, float scale, cudaStream_t s) {     \
        AttnArgs a{q, out, kc, vc, tile_seq, tile_t0, tile_nq, tok_pos, page_table, partial,                       \
                   max_pages, q_stride, nh, nkvh, dh, 0, splits, scale};                                           \
        return attention_launch<T>(a, tiles, nt, s);                                                                \
    }
TB_ATTENTION(tb_attention_f32, float)
TB_ATTENTION(tb_attention_bf16, __nv_bfloat16)
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_attention_f32)
TB_TAPE_REGISTER(tb_attention_bf16)
