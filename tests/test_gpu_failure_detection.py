"""GPU: a device-side give-up reaches the host as GD_ERR_INTERNAL at flush, names its code, is cleared, and leaves the
backend usable. The failure is made without a fault: a code stored in the backend's error word in stream order, and a
one-warp kernel whose bounded wait on a barrier nobody arrives at runs out (a few thousand polls) and returns."""
import numpy as np
import pytest

from gpu_util import F16, abi, dev, host, pkg

pytestmark = pytest.mark.gpu


def still_usable(ctx):
    ctx.begin_step()
    x = np.arange(64, dtype=np.float32).reshape(8, 8)
    t = dev(ctx, x, F16)
    out = ctx.scratch_empty(F16, (8, 8))
    ctx.check(ctx.lib.gd_backend_scale(ctx.backend, out.buffer, out.offset, t.buffer, t.offset, 64, F16, 2.0), "scale")
    got = host(out)
    ctx.end_step()
    return np.array_equal(got, 2 * x)


@pytest.mark.parametrize("how", ["injected", "bounded_wait"])
def test_device_give_up_surfaces_at_flush_once_and_the_backend_stays_usable(how):
    with pkg.runtime.Context(params_bytes=16 << 20, state_bytes=16 << 20, scratch_bytes=64 << 20) as ctx:
        lib, be = ctx.lib, ctx.backend
        assert lib.gd_backend_flush(be) == abi.GD_OK
        if how == "injected":
            assert lib.gdb200_inject_device_error(be, 777) == abi.GD_OK
            code = 777
        else:
            assert lib.gdb200_selftest_bounded_wait(be, 4096) == abi.GD_OK
            code = 399
        assert lib.gd_backend_flush(be) == abi.GD_ERR_INTERNAL
        assert f"code {code}".encode() in lib.gdb200_last_error(be)
        assert lib.gd_backend_flush(be) == abi.GD_OK          # reported once, then cleared
        assert still_usable(ctx)
        assert lib.gdb200_inject_device_error(be, 0) == abi.GD_ERR_INVALID_ARGUMENT
        assert lib.gdb200_selftest_bounded_wait(be, 0) == abi.GD_ERR_INVALID_ARGUMENT
