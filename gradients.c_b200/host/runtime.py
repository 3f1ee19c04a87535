"""Host runtime above the backend ABI: context, arenas, tensors, step scopes and the tape.

This mirrors the part of the reference's core that the gpt_lm path exercises
(src/core/memory.c: params / state arenas, per-step scratch and data slots, one fence per
step, :1350-1474; src/core/tensor.c descriptors; src/autograd/autograd.c:128,943-1135 tape
and gradient slots) with the same names and call order, so that the op capsules in ops.py
read like the reference's core_*.c files. It holds no numerics: every byte of tensor data is
produced by a gd_backend_* call.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Sequence

import numpy as np

from . import abi
from .abi import BackendError, DTYPE_SIZE, F16, BF16, F32, I32, U8

ALIGN = 256

NP_DTYPES = {F16: np.float16, F32: np.float32, I32: np.int32, U8: np.uint8, BF16: np.uint16, abi.U16: np.uint16}


def bf16_bits_from_f32(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def f32_from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


class Arena:
    """One backend buffer with bump allocation (reference gd_arena, src/core/memory.c:214-258)."""

    def __init__(self, ctx: "Context", name: str, nbytes: int):
        self.ctx, self.name, self.capacity = ctx, name, int(nbytes)
        out = C.c_void_p()
        st = ctx.lib.gd_backend_buffer_create(ctx.backend, self.capacity, C.byref(out))
        if st != abi.GD_OK:
            raise BackendError(st, f"buffer_create({name}, {nbytes})", ctx.last_error())
        self.buffer = out
        self.top = 0
        self.high_water = 0

    def alloc(self, nbytes: int, align: int = ALIGN) -> int:
        off = (self.top + align - 1) & ~(align - 1)
        if off + nbytes > self.capacity:
            raise MemoryError(f"arena {self.name}: need {off + nbytes} bytes, capacity {self.capacity}")
        self.top = off + int(nbytes)
        self.high_water = max(self.high_water, self.top)
        return off

    def reset(self) -> None:
        self.top = 0

    def destroy(self) -> None:
        if self.buffer:
            self.ctx.lib.gd_backend_buffer_destroy(self.buffer)
            self.buffer = None


class Tensor:
    """Descriptor of contiguous tensor bytes inside an arena (reference gd_tensor)."""

    __slots__ = ("ctx", "arena", "offset", "dtype", "shape", "requires_grad", "grad", "is_leaf", "name", "_tv")

    def __init__(self, ctx: "Context", arena: Arena, offset: int, dtype: int, shape: Sequence[int], name: str = ""):
        self.ctx, self.arena, self.offset, self.dtype = ctx, arena, int(offset), dtype
        self.shape = tuple(int(s) for s in shape)
        self.requires_grad = False
        self.grad: Optional[Tensor] = None
        self.is_leaf = False
        self.name = name
        self._tv = None

    @property
    def count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return self.count * DTYPE_SIZE[self.dtype]

    @property
    def buffer(self):
        return self.arena.buffer

    def tv(self) -> abi.TensorView:
        """gd_backend_tensor_view of the whole tensor (cached; descriptors are immutable)."""
        if self._tv is None:
            v = abi.TensorView()
            v.buffer, v.offset, v.count, v.dtype, v.rank = self.arena.buffer, self.offset, self.count, self.dtype, len(self.shape)
            stride = 1
            for d in range(len(self.shape) - 1, -1, -1):
                v.shape[d] = self.shape[d]
                v.strides[d] = stride
                stride *= self.shape[d]
            self._tv = v
        return self._tv

    def mv(self, rows: int, cols: int, row_offset: int = 0, row_bytes: Optional[int] = None) -> abi.MatrixView:
        es = DTYPE_SIZE[self.dtype]
        rb = cols * es if row_bytes is None else row_bytes
        v = abi.MatrixView()
        v.buffer, v.offset, v.rows, v.cols, v.row_bytes, v.dtype = self.arena.buffer, self.offset + row_offset * rb, rows, cols, rb, self.dtype
        return v

    def vv(self, start: int = 0, length: Optional[int] = None) -> abi.VectorView:
        v = abi.VectorView()
        v.buffer, v.offset = self.arena.buffer, self.offset + start * DTYPE_SIZE[self.dtype]
        v.length, v.dtype = (self.count - start) if length is None else length, self.dtype
        return v

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        t = Tensor(self.ctx, self.arena, self.offset, self.dtype, shape, self.name)
        assert t.count == self.count
        return t

    def rows(self, start: int, n: int) -> "Tensor":
        """View of n leading-dimension rows starting at `start`."""
        inner = self.count // self.shape[0]
        return Tensor(self.ctx, self.arena, self.offset + start * inner * DTYPE_SIZE[self.dtype], self.dtype,
                      (n,) + self.shape[1:], self.name)

    # ---- transfers (gd_tensor_write / gd_tensor_read: flush + synchronous copy) ----
    def write(self, host: np.ndarray) -> None:
        if self.dtype == BF16 and host.dtype != np.uint16:
            host = bf16_bits_from_f32(host)
        a = np.ascontiguousarray(host, dtype=NP_DTYPES[self.dtype])
        assert a.size == self.count, (a.shape, self.shape)
        self.ctx.check(self.ctx.lib.gd_backend_upload(self.ctx.backend, self.buffer, self.offset,
                                                      a.ctypes.data_as(C.c_void_p), a.nbytes), "upload")

    def write_async(self, pinned: np.ndarray) -> None:
        """Stream-ordered upload from page-locked memory (Context.pinned_copy); not waited for. `pinned` must
        keep its contents until a fence recorded after this call has completed."""
        assert pinned.dtype == NP_DTYPES[self.dtype] and pinned.size == self.count and pinned.flags.c_contiguous
        self.ctx.check(self.ctx.lib.gdb200_upload_async(self.ctx.backend, self.buffer, self.offset,
                                                        pinned.ctypes.data_as(C.c_void_p), pinned.nbytes), "upload_async")

    def read_async(self, pinned_out: np.ndarray) -> None:
        """Stream-ordered download into page-locked memory; valid once a later fence has completed."""
        assert pinned_out.dtype == NP_DTYPES[self.dtype] and pinned_out.size == self.count and pinned_out.flags.c_contiguous
        self.ctx.check(self.ctx.lib.gdb200_download_async(self.ctx.backend, self.buffer, self.offset,
                                                          pinned_out.ctypes.data_as(C.c_void_p), pinned_out.nbytes), "download_async")

    def read(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=NP_DTYPES[self.dtype])
        self.ctx.check(self.ctx.lib.gd_backend_download(self.ctx.backend, self.buffer, self.offset,
                                                        out.ctypes.data_as(C.c_void_p), out.nbytes), "download")
        return out

    def read_f32(self) -> np.ndarray:
        a = self.read()
        return f32_from_bf16_bits(a) if self.dtype == BF16 else a.astype(np.float32)


class Context:
    """gd_context: one backend, params/state arenas, one scratch slot and one data slot.

    The reference keeps `scratch_slots` ring buffers and waits on the slot's fence before
    reuse (memory.c:701); with one slot that is a wait for the previous step's fence at
    begin_step, which is what this class does by default (`run_ahead` 0). With `run_ahead` = n the
    host may enqueue up to n steps beyond the one the device is executing: begin_step then waits
    only for the fence of step k - n. The device arenas need no ring for that, because every
    kernel and every stream-ordered copy of step k + 1 is queued behind step k on the one in-order
    stream; only host memory handed to write_async / read_async must be rotated by the caller.
    """

    def __init__(self, params_bytes: int = 256 << 20, state_bytes: int = 512 << 20,
                 scratch_bytes: int = 6 << 30, data_bytes: int = 64 << 20):
        self.lib = abi.load_library()
        be = C.c_void_p()
        st = self.lib.gd_backend_create_default(C.byref(be))
        if st != abi.GD_OK:
            raise BackendError(st, "gd_backend_create_default", "no sm_100a CUDA device or library mismatch")
        self.backend = be
        self.params = Arena(self, "params", params_bytes)
        self.state = Arena(self, "state", state_bytes)
        self.scratch = Arena(self, "scratch", scratch_bytes)
        self.data = Arena(self, "data", data_bytes)
        self.tape: list[Callable[[], None]] = []
        self.grad_enabled = True
        self._fences: list[abi.Fence] = []
        self.run_ahead = 0
        self.in_step = False
        self.grad_ready_hook: Optional[Callable[[Tensor], None]] = None

    # ---- plumbing ----
    def last_error(self) -> str:
        s = self.lib.gdb200_last_error(self.backend) if getattr(self, "backend", None) else b""
        return (s or b"").decode()

    def check(self, status: int, what: str) -> None:
        if status != abi.GD_OK:
            raise BackendError(status, what, self.last_error())

    def destroy(self) -> None:
        if getattr(self, "backend", None):
            self.flush()
            for f in self._fences:
                self.lib.gd_backend_fence_destroy(C.byref(f))
            self._fences = []
            for a in (self.params, self.state, self.scratch, self.data):
                a.destroy()
            self.lib.gd_backend_destroy(self.backend)
            self.backend = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()

    def flush(self) -> None:
        self.check(self.lib.gd_backend_flush(self.backend), "flush")

    def launch_count(self) -> int:
        return int(self.lib.gdb200_launch_count(self.backend))

    def pinned_copy(self, a: np.ndarray) -> np.ndarray:
        """Copy of `a` in page-locked host memory (kept alive by the context)."""
        a = np.ascontiguousarray(a)
        ptr = self.lib.gdb200_pinned_alloc(max(a.nbytes, 1))
        if not ptr:
            raise MemoryError("pinned host allocation failed")
        self._pinned = getattr(self, "_pinned", [])
        self._pinned.append(ptr)
        buf = (C.c_byte * a.nbytes).from_address(ptr)
        out = np.frombuffer(buf, dtype=a.dtype).reshape(a.shape)
        out[...] = a
        return out

    # ---- step scope (reference gd_begin_step / gd_end_step) ----
    def begin_step(self) -> None:
        assert not self.in_step
        self.wait_steps(self.run_ahead)
        self.scratch.reset()
        self.data.reset()
        self.tape.clear()
        self.check(self.lib.gd_backend_scope_begin(self.backend), "scope_begin")
        self.in_step = True

    def end_step(self) -> None:
        assert self.in_step
        f = abi.Fence()
        self.check(self.lib.gd_backend_record_fence(self.backend, C.byref(f)), "record_fence")
        self._fences.append(f)
        self.tape.clear()
        self.in_step = False

    def wait_steps(self, keep: int = 0) -> None:
        """Waits until at most `keep` recorded steps are still in flight (oldest first)."""
        while len(self._fences) > keep:
            f = self._fences.pop(0)
            st = self.lib.gd_backend_fence_wait(C.byref(f))
            self.lib.gd_backend_fence_destroy(C.byref(f))
            self.check(st, "fence_wait")

    # ---- tensors ----
    def empty(self, arena: Arena, dtype: int, shape: Sequence[int], name: str = "") -> Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        off = arena.alloc(max(n, 1) * DTYPE_SIZE[dtype])
        return Tensor(self, arena, off, dtype, shape, name)

    def scratch_empty(self, dtype: int, shape: Sequence[int], name: str = "") -> Tensor:
        return self.empty(self.scratch, dtype, shape, name)

    def fill(self, t: Tensor, pattern: int) -> None:
        self.check(self.lib.gd_backend_fill(self.backend, t.buffer, t.offset, t.count, DTYPE_SIZE[t.dtype], pattern), "fill")

    def zeros(self, arena: Arena, dtype: int, shape: Sequence[int], name: str = "") -> Tensor:
        t = self.empty(arena, dtype, shape, name)
        self.fill(t, 0)
        return t

    def from_numpy(self, arena: Arena, dtype: int, host: np.ndarray, name: str = "") -> Tensor:
        t = self.empty(arena, dtype, host.shape, name)
        t.write(host)
        return t

    # ---- tape (reference gd_autograd_record + reverse walk) ----
    def record(self, backward: Callable[[], None]) -> None:
        if self.grad_enabled:
            self.tape.append(backward)

    def accumulate_grad(self, t: Tensor, g: Tensor) -> None:
        """First contribution is adopted, later ones are added with gd_backend_accumulate
        (16-bit storage rounds after every add), as src/autograd/autograd.c:517-685 does."""
        if not t.requires_grad:
            return
        if t.grad is None:
            t.grad = g
        else:
            assert t.grad.count == g.count and t.grad.dtype == g.dtype
            self.check(self.lib.gd_backend_accumulate(self.backend, t.grad.buffer, t.grad.offset, g.buffer, g.offset,
                                                      g.count, g.dtype), "accumulate")

    def run_backward(self) -> None:
        for fn in reversed(self.tape):
            fn()
        self.tape.clear()
