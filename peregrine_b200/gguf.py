"""Host-side mirror of the block codecs of `peregrine::gguf` (src/gguf.rs) on top of the C ABI.

    dequant_q8_0 / dequant_q4_0 / dequant_q4_1(data, num_elements) -> f32   src/gguf.rs:286-351
    f16_to_f32(bits) -> f32                                                 src/gguf.rs:354-382
    load_tensor_q8_as_quantized(data, rows, cols) -> QuantizedTensor        src/gguf.rs:386-401

and the operation the Llama linears perform on such a tensor (dequantise, transpose, f32
matmul: src/gguf.rs:485-517, src/models/llama/model.rs:243-257, src/tensor.rs:1342-1354) as one
device-resident object, `GgufWeight`, whose `matmul` never materialises the f32 weight.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib
from .quant import QuantizedTensor
from .runtime import GpuContext, _ptr, current_gpu

BLOCK_BYTES = {_lib.GGUF_Q8_0: 34, _lib.GGUF_Q4_0: 18, _lib.GGUF_Q4_1: 20}
TYPE_BY_NAME = {"q8_0": _lib.GGUF_Q8_0, "q4_0": _lib.GGUF_Q4_0, "q4_1": _lib.GGUF_Q4_1}


def _dequant(kind: int, data, num_elements: int, gpu: Optional[GpuContext]) -> np.ndarray:
    gpu = gpu or current_gpu()
    data = np.ascontiguousarray(data, np.uint8).reshape(-1)
    out = np.empty(max(num_elements, 0), np.float32)
    _lib.check(gpu.lib.pg_dequant_blocks_host(gpu.handle, kind, _ptr(data), data.size, num_elements, _ptr(out)))
    return out


def dequant_q8_0(data, num_elements: int, gpu: Optional[GpuContext] = None) -> np.ndarray:
    return _dequant(_lib.GGUF_Q8_0, data, num_elements, gpu)


def dequant_q4_0(data, num_elements: int, gpu: Optional[GpuContext] = None) -> np.ndarray:
    return _dequant(_lib.GGUF_Q4_0, data, num_elements, gpu)


def dequant_q4_1(data, num_elements: int, gpu: Optional[GpuContext] = None) -> np.ndarray:
    return _dequant(_lib.GGUF_Q4_1, data, num_elements, gpu)


def f16_to_f32(bits, gpu: Optional[GpuContext] = None):
    """Scalar or array of f16 bit patterns -> f32 (bit-exact, NaN payloads included)."""
    gpu = gpu or current_gpu()
    arr = np.ascontiguousarray(np.atleast_1d(bits), np.uint16)
    d_in = gpu.upload(arr)
    d_out = gpu.alloc(arr.size, np.float32)
    _lib.check(gpu.lib.pg_f16_to_f32(gpu.handle, d_in.ptr, arr.size, d_out.ptr))
    out = d_out.read()
    return out[0] if np.isscalar(bits) else out


def load_tensor_q8_as_quantized(data, rows: int, cols: int, gpu: Optional[GpuContext] = None) -> QuantizedTensor:
    """Q8_0 blocks of a [rows, cols] tensor -> dequantise -> per-column requantise, on the device.
    The result is already resident (`on_gpu`), with host copies filled in."""
    gpu = gpu or current_gpu()
    data = np.ascontiguousarray(data, np.uint8).reshape(-1)
    h = C.c_void_p()
    _lib.check(gpu.lib.pg_qtensor_from_q8_0(gpu.handle, _ptr(data), data.size, rows, cols, C.byref(h)))
    qt = QuantizedTensor(np.empty((rows, cols), np.int8), np.empty((cols, rows), np.int8), np.empty(cols, np.float32), rows, cols)
    qt._gpu, qt._gpu_ctx = h, gpu
    qt.from_gpu(gpu)
    return qt


class GgufWeight:
    """A GGUF block-quantised weight [N=out, K=in] resident on the GPU.

    `rows` selects the shard of output rows this GPU keeps.  `matmul(x, m)` returns
    y[m, N] = x[m, K] . dequant(W)^T in f32."""

    def __init__(self, kind, raw, n: int, k: int, gpu: Optional[GpuContext] = None, rows: Optional[tuple] = None):
        self.gpu = gpu or current_gpu()
        self.kind = TYPE_BY_NAME[kind] if isinstance(kind, str) else int(kind)
        raw = np.ascontiguousarray(raw, np.uint8).reshape(-1)
        b, e = rows if rows is not None else (0, n)
        h = C.c_void_p()
        _lib.check(self.gpu.lib.pg_gguf_upload(self.gpu.handle, self.kind, _ptr(raw), raw.size, n, k, b, e, C.byref(h)))
        self.handle = h
        self.n = e - b
        self.k = k
        self.raw_bytes = self.n * (k // 32) * BLOCK_BYTES[self.kind]

    def matmul(self, x, m: int) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        if x.size != m * self.k:
            raise _lib.InvalidArgument(_lib.PG_ERR_INVALID, f"matmul: x holds {x.size} values, expected {m * self.k}")
        y = np.empty((m, self.n), np.float32)
        _lib.check(self.gpu.lib.pg_matmul_gguf_host(self.gpu.handle, _ptr(x), m, self.handle, _ptr(y)))
        return y

    def matmul_device(self, d_x, m: int, d_y) -> None:
        """Device pointers (ints, GpuBuffers or torch tensors); enqueued, not synchronised."""
        _lib.check(self.gpu.lib.pg_matmul_gguf(self.gpu.handle, _ptr(d_x), m, self.handle, _ptr(d_y)))

    def free(self) -> None:
        if self.handle is not None and self.gpu.handle:
            self.gpu.lib.pg_gguf_free(self.gpu.handle, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
