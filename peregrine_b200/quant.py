"""Host-side mirror of `peregrine::quant` (src/quant.rs) on top of the C ABI.

Same names, argument order and error behaviour as the reference:

    quantize_weights(data, rows, cols) -> QuantizedTensor          src/quant.rs:27-75
    quantize_activations(data, rows, cols) -> (i8, scales)         src/quant.rs:79-112
    dequantize(qt) -> f32                                          src/quant.rs:115-123
    matmul_quantized(a, m, k, w) -> f32 [m*n]                      src/quant.rs:129-169
    QuantizedTensor.to_gpu / from_gpu                              src/quant.rs:172-191
    matmul_quantized_gpu(gpu, a, m, k, w) -> GpuBuffer (no sync)   src/quant.rs:195-218

Where the reference `assert!`s, these raise `InvalidArgument` (an AssertionError).
Every function runs on the GPU; none has a CPU implementation.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np

from . import _lib
from .runtime import GpuBuffer, GpuContext, _ptr, current_gpu


def _f32(a, n: int, what: str) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32).reshape(-1)
    if a.size != n:
        raise _lib.InvalidArgument(_lib.PG_ERR_INVALID, f"{what}: data.len() = {a.size}, expected {n}")
    return a


class QuantizedTensor:
    """`peregrine::quant::QuantizedTensor` (src/quant.rs:12-23): host arrays plus the optional
    device copy that `to_gpu` creates (the reference's `gpu_data_i8` / `gpu_scales`)."""

    def __init__(self, data_i8: np.ndarray, data_i8_t: np.ndarray, scales: np.ndarray, rows: int, cols: int):
        self.data_i8 = data_i8
        self.data_i8_t = data_i8_t
        self.scales = scales
        self.rows = int(rows)
        self.cols = int(cols)
        self._gpu: Optional[C.c_void_p] = None
        self._gpu_ctx: Optional[GpuContext] = None
        self.col_range: Tuple[int, int] = (0, self.cols)

    @property
    def on_gpu(self) -> bool:
        return self._gpu is not None

    def to_gpu(self, gpu: GpuContext, col_begin: int = 0, col_end: Optional[int] = None) -> None:
        """Uploads once (idempotent, like src/quant.rs:174-181).  A column range keeps only that
        shard of the output columns on this GPU."""
        if self._gpu is not None:
            return
        col_end = self.cols if col_end is None else col_end
        h = C.c_void_p()
        _lib.check(gpu.lib.pg_qtensor_upload(gpu.handle, _ptr(self.data_i8), _ptr(self.data_i8_t), _ptr(self.scales),
                                             self.rows, self.cols, col_begin, col_end, C.byref(h)))
        self._gpu, self._gpu_ctx, self.col_range = h, gpu, (col_begin, col_end)

    def from_gpu(self, gpu: GpuContext) -> None:
        """Reads the device copy back into the host arrays (src/quant.rs:183-190)."""
        if self._gpu is None:
            return
        b, e = self.col_range
        n = e - b
        qt = np.empty((n, self.rows), np.int8)
        s = np.empty(n, np.float32)
        q = np.empty((self.rows, n), np.int8) if self.data_i8 is not None else None
        _lib.check(gpu.lib.pg_qtensor_download(gpu.handle, self._gpu, _ptr(q), _ptr(qt), _ptr(s)))
        self.data_i8_t[b:e] = qt
        self.scales[b:e] = s
        if q is not None:
            self.data_i8[:, b:e] = q

    def free_gpu(self) -> None:
        if self._gpu is not None and self._gpu_ctx is not None and self._gpu_ctx.handle:
            self._gpu_ctx.lib.pg_qtensor_free(self._gpu_ctx.handle, self._gpu)
        self._gpu = None

    def __del__(self):
        try:
            self.free_gpu()
        except Exception:
            pass


def quantize_weights(data, rows: int, cols: int, gpu: Optional[GpuContext] = None) -> QuantizedTensor:
    gpu = gpu or current_gpu()
    data = _f32(data, rows * cols, "quantize_weights")
    q = np.empty((rows, cols), np.int8)
    qt = np.empty((cols, rows), np.int8)
    s = np.empty(cols, np.float32)
    _lib.check(gpu.lib.pg_quantize_weights_host(gpu.handle, _ptr(data), rows, cols, _ptr(q), _ptr(qt), _ptr(s)))
    return QuantizedTensor(q, qt, s, rows, cols)


def quantize_activations(data, rows: int, cols: int, gpu: Optional[GpuContext] = None):
    gpu = gpu or current_gpu()
    data = _f32(data, rows * cols, "quantize_activations")
    q = np.empty((rows, cols), np.int8)
    s = np.empty(rows, np.float32)
    _lib.check(gpu.lib.pg_quantize_activations_host(gpu.handle, _ptr(data), rows, cols, _ptr(q), _ptr(s)))
    return q, s


def dequantize(qt: QuantizedTensor, gpu: Optional[GpuContext] = None) -> np.ndarray:
    gpu = gpu or current_gpu()
    d_q = gpu.upload(qt.data_i8)
    d_s = gpu.upload(qt.scales)
    d_o = gpu.alloc(qt.rows * qt.cols, np.float32)
    _lib.check(gpu.lib.pg_dequantize(gpu.handle, d_q.ptr, d_s.ptr, qt.rows, qt.cols, d_o.ptr))
    return d_o.read().reshape(qt.rows, qt.cols)


def matmul_quantized(a_data, m: int, k: int, w: QuantizedTensor, gpu: Optional[GpuContext] = None) -> np.ndarray:
    """Host slices in, host result out; the weights are uploaded on first use and stay resident."""
    gpu = gpu or current_gpu()
    if w.rows != k:
        raise _lib.InvalidArgument(_lib.PG_ERR_INVALID, f"matmul_quantized: w.rows ({w.rows}) != k ({k})")
    a = _f32(a_data, m * k, "matmul_quantized")
    w.to_gpu(gpu)
    n = w.col_range[1] - w.col_range[0]
    y = np.empty((m, n), np.float32)
    _lib.check(gpu.lib.pg_matmul_quantized_host(gpu.handle, _ptr(a), m, k, w._gpu, _ptr(y)))
    return y


def matmul_quantized_gpu(gpu: GpuContext, a_data, m: int, k: int, w: QuantizedTensor, dequant: bool = False,
                         sequential: bool = False) -> GpuBuffer:
    """Uploads A, enqueues the product and returns the device buffer WITHOUT synchronising;
    the weights must already be on the GPU ("weights not on GPU" otherwise, src/quant.rs:208).

    By default the product is the CPU path's W8A8 (quantised activations, integer sums), which is what the parity
    target of this library is.  dequant=True gives what the reference's own GPU kernels compute behind this function
    (src/metal/shaders.rs:2329-2465): f32 activations times weights dequantised on the fly ("W8A32");
    sequential=True takes the one-thread-per-output form of it, which adds in the order of the reference's loops."""
    if w.rows != k:
        raise _lib.InvalidArgument(_lib.PG_ERR_INVALID, f"matmul_quantized_gpu: w.rows ({w.rows}) != k ({k})")
    a = _f32(a_data, m * k, "matmul_quantized_gpu")
    if w._gpu is None:
        raise _lib.InvalidArgument(_lib.PG_ERR_INVALID, "weights not on GPU")
    a_buf = gpu.upload(a)
    n = w.col_range[1] - w.col_range[0]
    out = gpu.alloc(m * n, np.float32)
    if dequant:
        _lib.check(gpu.lib.pg_matmul_dequant_w8a32(gpu.handle, a_buf.ptr, m, k, w._gpu, out.ptr, 1 if sequential else 0))
    else:
        _lib.check(gpu.lib.pg_matmul_quantized(gpu.handle, a_buf.ptr, m, k, w._gpu, out.ptr))
    out._keepalive = a_buf  # A must outlive the enqueued kernels
    return out


def matmul_quantized_parts(gpu: GpuContext, a_data, m: int, k: int, w: QuantizedTensor, algo: int = _lib.ALGO_AUTO):
    """The same product with every intermediate returned: (y, acc_i32, a_i8, a_scales).
    For parity tests: the reference keeps these as locals (src/quant.rs:140-165)."""
    a = _f32(a_data, m * k, "matmul_quantized")
    w.to_gpu(gpu)
    n = w.col_range[1] - w.col_range[0]
    d_a = gpu.upload(a) if a.size else gpu.alloc(1, np.float32)
    d_y = gpu.alloc(max(m * n, 1), np.float32)
    d_acc = gpu.alloc(max(m * n, 1), np.int32)
    d_q = gpu.alloc(max(m * k, 1) + 16, np.int8)
    d_s = gpu.alloc(max(m, 1), np.float32)
    _lib.check(gpu.lib.pg_matmul_quantized_ex(gpu.handle, d_a.ptr, m, k, w._gpu, d_y.ptr, d_acc.ptr, d_q.ptr, d_s.ptr, algo))
    y = d_y.read()[: m * n].reshape(m, n)
    acc = d_acc.read()[: m * n].reshape(m, n)
    q = d_q.read()[: m * k].reshape(m, k)
    s = d_s.read()[:m]
    return y, acc, q, s
