/* Exports rms_reference of tests/test_rms_norm.c:56-105. Test infrastructure only. */
#define main gdref_rms_unused_main
#include GDREF_TEST_RMS
#undef main

void gdref_rms(const float *x, const float *weight, const float *grad_out, uint32_t rows, uint32_t cols, float eps,
               float *out, float *dx, float *dw)
{
    rms_reference(x, weight, grad_out, rows, cols, eps, out, dx, dw);
}
