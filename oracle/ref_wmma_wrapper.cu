// C-ABI wrapper around the REFERENCE's own fused kernel, compiled from the reference checkout
// where it lies (the header is included by path at build time; nothing of it is copied here).
// TEST INFRASTRUCTURE: the built library lands in oracle/_ref/ and is only used by tests and the
// benchmark's context line as a second comparator next to the CPU oracle.
//
// Exposes launch_attention_kernel<head_dim, chunk_size> (include/fused_attn.cuh:860-894) for the
// twelve instances the reference binding dispatches (src/fused_attn_extention.cu:72-111).
#include <cstdint>
#include "fused_attn.cuh"

#define REF_CASE(H, C)                                                                          \
    if (head_dim == H && chunk_size == C) {                                                     \
        launch_attention_kernel<H, C>(B, L, F, (const half_t*)q, (const half_t*)k,              \
                                      (const half_t*)v, (const half_t*)mask, (half_t*)y, true); \
        return 0;                                                                               \
    }

extern "C" int ref_wmma_attention_forward(const void* q, const void* k, const void* v, const void* mask,
                                          void* y, uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim,
                                          uint32_t chunk_size) {
    if (L % chunk_size != 0 || F % head_dim != 0) return -1;  // src/fused_attn_extention.cu:63-64
    REF_CASE(16, 16) REF_CASE(16, 32)
    REF_CASE(32, 16) REF_CASE(32, 32) REF_CASE(32, 64)
    REF_CASE(64, 16) REF_CASE(64, 32) REF_CASE(64, 64) REF_CASE(64, 128)
    REF_CASE(128, 32) REF_CASE(128, 64) REF_CASE(128, 128)
    return -2;
}
