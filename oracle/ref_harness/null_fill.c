/* The reference's null backend (src/backends/null/) does not define six entries that its host
 * code calls (rope, rope_backward, swiglu_forward/backward, swiglu_split_forward/backward), so a
 * shared library of host + null backend has unresolved symbols. These fillers answer
 * GD_ERR_UNSUPPORTED like every other null entry. Test infrastructure only. */
#include <core/backend.h>

#define TV const gd_backend_tensor_view *
gd_status gd_backend_rope(gd_backend *b, TV x, TV p, TV o, const gd_backend_rope_args *a) { (void)b; (void)x; (void)p; (void)o; (void)a; return GD_ERR_UNSUPPORTED; }
gd_status gd_backend_rope_backward(gd_backend *b, TV g, TV p, TV d, const gd_backend_rope_args *a) { (void)b; (void)g; (void)p; (void)d; (void)a; return GD_ERR_UNSUPPORTED; }
gd_status gd_backend_swiglu_forward(gd_backend *b, TV x1, TV x2, TV o) { (void)b; (void)x1; (void)x2; (void)o; return GD_ERR_UNSUPPORTED; }
gd_status gd_backend_swiglu_backward(gd_backend *b, TV x1, TV x2, TV g, TV d1, TV d2) { (void)b; (void)x1; (void)x2; (void)g; (void)d1; (void)d2; return GD_ERR_UNSUPPORTED; }
gd_status gd_backend_swiglu_split_forward(gd_backend *b, TV x, TV o) { (void)b; (void)x; (void)o; return GD_ERR_UNSUPPORTED; }
gd_status gd_backend_swiglu_split_backward(gd_backend *b, TV x, TV g, TV d) { (void)b; (void)x; (void)g; (void)d; return GD_ERR_UNSUPPORTED; }
