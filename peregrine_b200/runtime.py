"""GPU context and buffers: the B200 counterpart of the reference's `metal` seam.

Mirrors `peregrine::metal::{init_gpu, with_gpu, GpuContext, GpuBuffer}`
(src/metal/context.rs:45, 188-204, 2472-2510): one context per thread, work enqueued on a
stream without synchronisation, explicit `sync()` / `read()` by the caller.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Callable, Optional, TypeVar

import numpy as np

from . import _lib

T = TypeVar("T")


def _ptr(a) -> C.c_void_p:
    """Host pointer of a numpy array, or the integer/None passed through as a device pointer."""
    if a is None:
        return C.c_void_p(0)
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    if isinstance(a, GpuBuffer):
        return C.c_void_p(a.ptr)
    if hasattr(a, "data_ptr"):  # torch tensor on the device
        return C.c_void_p(a.data_ptr())
    return C.c_void_p(int(a))


class GpuBuffer:
    """A typed device allocation (reference: `GpuBuffer<T>`); `read()` blocks and copies back."""

    def __init__(self, ctx: "GpuContext", count: int, dtype):
        self.ctx = ctx
        self.dtype = np.dtype(dtype)
        self.count = int(count)
        out = C.c_void_p()
        _lib.check(ctx.lib.pg_mem_alloc(ctx.handle, self.nbytes, C.byref(out)))
        self.ptr = out.value or 0

    @property
    def nbytes(self) -> int:
        return self.count * self.dtype.itemsize

    def write(self, host: np.ndarray) -> None:
        host = np.ascontiguousarray(host, self.dtype)
        assert host.size == self.count
        _lib.check(self.ctx.lib.pg_mem_upload(self.ctx.handle, self.ptr, _ptr(host), self.nbytes))
        # the source array may be a temporary: make the copy complete before it can be freed
        self.ctx.sync()

    def read(self) -> np.ndarray:
        out = np.empty(self.count, self.dtype)
        _lib.check(self.ctx.lib.pg_mem_download(self.ctx.handle, _ptr(out), self.ptr, self.nbytes))
        return out

    def free(self) -> None:
        if self.ptr:
            _lib.check(self.ctx.lib.pg_mem_free(self.ctx.handle, self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GpuContext:
    """One CUDA device + stream.  `stream` may be a raw cudaStream_t (int) to share, e.g.
    `torch.cuda.current_stream().cuda_stream`."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self.lib = _lib.load()
        h = C.c_void_p()
        _lib.check(self.lib.pg_ctx_create(int(device), C.c_void_p(stream or 0), C.byref(h)))
        self.handle = h
        self.device = int(device)

    # GpuContext::alloc / upload / sync
    def alloc(self, count: int, dtype=np.float32) -> GpuBuffer:
        return GpuBuffer(self, count, dtype)

    def upload(self, host: np.ndarray) -> GpuBuffer:
        host = np.ascontiguousarray(host)
        buf = GpuBuffer(self, host.size, host.dtype)
        buf.write(host)
        return buf

    def sync(self) -> None:
        _lib.check(self.lib.pg_ctx_sync(self.handle))

    @property
    def stream(self) -> int:
        return self.lib.pg_ctx_stream(self.handle) or 0

    def device_status(self) -> int:
        v = C.c_int32(0)
        _lib.check(self.lib.pg_ctx_device_status(self.handle, C.byref(v)))
        return v.value

    # batched submission (CUDA graph): `with gpu.record() as g: ...` then `g.launch()`
    def record(self) -> "Graph":
        return Graph(self)

    def close(self) -> None:
        if self.handle:
            self.lib.pg_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Graph:
    """Records the calls made on a context inside the `with` block and replays them with one
    submission (`launch`).  Run the calls once before recording so that scratch memory is sized."""

    def __init__(self, ctx: GpuContext):
        self.ctx = ctx
        self.handle = None
        self.kernels = 0

    def __enter__(self):
        self._n0 = self.ctx.lib.pg_launch_count()
        _lib.check(self.ctx.lib.pg_graph_begin(self.ctx.handle))
        return self

    def __exit__(self, exc_type, exc, tb):
        h = C.c_void_p()
        rc = self.ctx.lib.pg_graph_end(self.ctx.handle, C.byref(h))
        if exc_type is None:
            _lib.check(rc)
            self.handle = h
            self.kernels = int(self.ctx.lib.pg_launch_count() - self._n0)
        return False

    def launch(self) -> None:
        _lib.check(self.ctx.lib.pg_graph_launch(self.ctx.handle, self.handle))

    def free(self) -> None:
        if self.handle is not None and self.ctx.handle:
            self.ctx.lib.pg_graph_free(self.ctx.handle, self.handle)
        self.handle = None


_tls = threading.local()


def init_gpu(device: int = 0, stream: Optional[int] = None) -> GpuContext:
    """`metal::init_gpu()`: creates this thread's context (idempotent).  Raises if no B200 is usable."""
    ctx = getattr(_tls, "ctx", None)
    if ctx is None or ctx.handle is None:
        ctx = GpuContext(device, stream)
        _tls.ctx = ctx
    return ctx


def with_gpu(f: Callable[[GpuContext], T]) -> Optional[T]:
    """`metal::with_gpu`: runs `f` with the thread's context, or returns None if there is none."""
    ctx = getattr(_tls, "ctx", None)
    if ctx is None or ctx.handle is None:
        return None
    return f(ctx)


def current_gpu() -> GpuContext:
    """The thread's context, created on device 0 on first use.  There is no CPU path behind this."""
    return init_gpu()
