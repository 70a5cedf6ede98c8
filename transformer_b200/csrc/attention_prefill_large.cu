// The prompt attention on mma.sync (attention_prefill.cuh): head sizes 144 to 256.
#include "attention_prefill.cuh"

int prefill_launch_large(const PrefillArgs& a, int dh, cudaStream_t s) {
    switch (dh) {
        case 144: return prefill_launch<144>(a, s);
        case 160: return prefill_launch<160>(a, s);
        case 176: return prefill_launch<176>(a, s);
        case 192: return prefill_launch<192>(a, s);
        case 208: return prefill_launch<208>(a, s);
        case 224: return prefill_launch<224>(a, s);
        case 240: return prefill_launch<240>(a, s);
        case 256: return prefill_launch<256>(a, s);
        default: return TB_ERR_UNSUPPORTED;
    }
}
