/* Exports rope_ref of tests/test_rope.c:67-103. Test infrastructure only. */
#define main gdref_rope_unused_main
#include GDREF_TEST_ROPE
#undef main

void gdref_rope(const float *x, const int32_t *pos, float *out, const int64_t *shape, uint32_t rank, float theta,
                int32_t n_dims, int interleaved, float sin_sign)
{
    rope_ref(x, pos, out, shape, rank, theta, n_dims, interleaved, sin_sign);
}
