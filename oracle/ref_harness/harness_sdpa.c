/* Exports the CPU reference functions that the reference's own test carries as file-local
 * statics (tests/test_sdpa_varlen.c:122-371,599-677) so that the oracle can be pinned against
 * them. The test file is included from the reference tree where it lies; nothing is copied.
 * Test infrastructure only. */
#define main gdref_sdpa_unused_main
#include GDREF_TEST_SDPA
#undef main

int gdref_allowed(int i, int j, int causal, int window, int prefix_len) { return allowed(i, j, causal, window, prefix_len); }
void gdref_fill_tokens(uint16_t *x, uint32_t count, float base) { fill_tokens(x, count, base); }
void gdref_varlen_fwd(const uint16_t *q, const uint16_t *k, const uint16_t *v, const int32_t *cu, uint32_t B, uint32_t Hq,
                      uint32_t Hkv, uint32_t Dh, float scale, int causal, int window, int prefix_len, float *out)
{
    ref_varlen_fwd(q, k, v, cu, B, Hq, Hkv, Dh, scale, causal, window, prefix_len, out);
}
void gdref_varlen_bwd(const uint16_t *go, const uint16_t *q, const uint16_t *k, const uint16_t *v, const int32_t *cu,
                      uint32_t B, uint32_t Hq, uint32_t Hkv, uint32_t Dh, float scale, int causal, int window,
                      int prefix_len, float *dq, float *dk, float *dv)
{
    ref_varlen_bwd(go, q, k, v, cu, B, Hq, Hkv, Dh, scale, causal, window, prefix_len, dq, dk, dv);
}
void gdref_decode(const uint16_t *q, const uint16_t *k, const uint16_t *v, int cache_pos, uint32_t B, uint32_t Tq,
                  uint32_t Tmax, uint32_t Hq, uint32_t Hkv, uint32_t Dh, float scale, int window, int prefix_len, float *out)
{
    ref_decode(q, k, v, cache_pos, B, Tq, Tmax, Hq, Hkv, Dh, scale, window, prefix_len, out);
}
uint16_t gdref_f32_to_f16_bits(float v) { return f32_to_f16_bits(v); }
float gdref_f16_bits_to_f32(uint16_t b) { return f16_bits_to_f32(b); }
