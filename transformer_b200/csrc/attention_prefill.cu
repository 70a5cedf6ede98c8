// The prompt attention on mma.sync (attention_prefill.cuh): head sizes up to 128 and the entry point.
#include "attention_prefill.cuh"

extern "C" {
// Query tiles hold up to this many tokens of one sequence.
int tb_attention_prefill_tile_tokens() { return AP_BM; }

int tb_attention_prefill_bf16(const void* q, void* out, const void* kc, const void* vc, const int* tile_seq,
                              const int* tile_t0, const int* tile_nq, const int* tok_pos, const int* page_table,
                              int tiles, int max_pages, int q_stride, int nh, int nkvh, int dh, float scale,
                              cudaStream_t s) {
    if (nh <= 0 || nkvh <= 0 || nh % nkvh || tiles < 0) return TB_ERR_ARG;
    if (dh <= 0 || dh % 16 || dh > 256) return TB_ERR_UNSUPPORTED;
    if (q_stride % 8 || (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kc | (uintptr_t)vc) & 15)) return TB_ERR_UNSUPPORTED;
    if (tiles == 0) return 0;
    PrefillArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                  tile_seq, tile_t0, tile_nq, tok_pos, page_table, tiles, max_pages, q_stride, nh, nkvh,
                  scale * 1.4426950408889634f};
    switch (dh) {
        case 16: return prefill_launch<16>(a, s);
        case 32: return prefill_launch<32>(a, s);
        case 48: return prefill_launch<48>(a, s);
        case 64: return prefill_launch<64>(a, s);
        case 80: return prefill_launch<80>(a, s);
        case 96: return prefill_launch<96>(a, s);
        case 112: return prefill_launch<112>(a, s);
        case 128: return prefill_launch<128>(a, s);
        default: return prefill_launch_large(a, dh, s);
    }
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_attention_prefill_bf16)
