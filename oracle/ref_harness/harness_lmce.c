/* Exports the soft-capped LM cross-entropy oracle of tests/test_lm_cross_entropy.c:141-296
 * (fixed case: 6 rows, dim 8, vocab 32). Test infrastructure only. */
#define main gdref_lmce_unused_main
#include GDREF_TEST_LMCE
#undef main

void gdref_lmce_dims(int *rows, int *dim, int *vocab) { *rows = SOFT_ROWS; *dim = SOFT_DIM; *vocab = SOFT_VOCAB; }
void gdref_lmce_fill(uint16_t *hidden, uint16_t *weight, uint16_t *bias)
{
    fill_hidden(hidden, SOFT_HCOUNT);
    fill_weight(weight, SOFT_WCOUNT);
    fill_bias(bias, SOFT_VOCAB);
}
void gdref_lmce_oracle(const uint16_t *hidden, const uint16_t *weight, const uint16_t *bias, const int32_t *targets,
                       float cap, float *loss, uint16_t *dh, uint16_t *dw, uint16_t *db)
{
    compute_softcapped_oracle(hidden, weight, bias, targets, cap, loss, dh, dw, db);
}
