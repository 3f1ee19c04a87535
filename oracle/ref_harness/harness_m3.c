/* Exports the CPU references of tests/test_minimax_m3_sparse_attention.c: ref_topk (:145-213), ref_sparse_fwd_gqa
 * (:423-483) and ref_sparse_bwd_gqa (:485-600). Test infrastructure only. */
#define main gdref_m3_unused_main
#include GDREF_TEST_M3
#undef main

/* topk <= 4 (capacity of the test's reference). out: I32 [H, N, topk]. */
void gdref_m3_topk(const uint16_t *q, const uint16_t *k, const int32_t *cu, uint32_t B, uint32_t H, uint32_t Dh, uint32_t block_size,
                   uint32_t topk, uint32_t init_blocks, uint32_t local_blocks, int32_t *out)
{
    ref_topk(q, k, cu, B, H, Dh, block_size, topk, init_blocks, local_blocks, out);
}

void gdref_m3_fwd(const uint16_t *q, const uint16_t *k, const uint16_t *v, const int32_t *cu, const int32_t *topk, uint32_t B, uint32_t Hq,
                  uint32_t Hkv, uint32_t Dh, uint32_t block_size, uint32_t topk_count, float scale, float *out)
{
    ref_sparse_fwd_gqa(q, k, v, cu, topk, B, Hq, Hkv, Dh, block_size, topk_count, scale, out);
}

void gdref_m3_bwd(const uint16_t *go, const uint16_t *q, const uint16_t *k, const uint16_t *v, const int32_t *cu, const int32_t *topk,
                  uint32_t B, uint32_t Hq, uint32_t Hkv, uint32_t Dh, uint32_t block_size, uint32_t topk_count, float scale, float *dq,
                  float *dk, float *dv)
{
    ref_sparse_bwd_gqa(go, q, k, v, cu, topk, B, Hq, Hkv, Dh, block_size, topk_count, scale, dq, dk, dv);
}
