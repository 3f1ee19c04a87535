#include "common.cuh"
gd_status gdb_gemm_tcgen05(gd_backend *, int, int, uint32_t, const void *, size_t, const void *, size_t, void *, size_t, const void *, uint32_t, uint32_t, uint32_t) { return GD_ERR_UNSUPPORTED; }
void gdb_tmap_cache_destroy(gd_backend *) {}
