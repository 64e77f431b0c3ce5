"""The quantised serial formats: host-side mirror of `write_quantized_tensor` / `read_quantized_tensor`
(src/serial.rs:124-222) and of `write_huffman_tensor` / `read_huffman_tensor` (src/serial.rs:315-443).

    [name_len: u32][name: utf-8][dtype = 1: u8][ndim = 2: u32][rows: u32][cols: u32]
    [data_i8: rows * cols bytes, row-major][scales: cols x f32]                      (all little-endian)

Writing is byte bookkeeping.  Reading hands the int8 matrix to the GPU, where the GEMM layout
`data_i8_t` [cols, rows] is rebuilt (the reference transposes on the host, src/serial.rs:203-208): the
tensor comes back resident, with its host arrays filled in.

A Huffman record keeps the int8 matrix as bitstreams:

    [name_len: u32][name][dtype = 3: u8][ndim = 2: u32][rows: u32][cols: u32][code book: 256 bit lengths]
    [num_streams: u32][symbols per stream: u32 each][bytes per stream: u32 each][bitstreams][scales: cols x f32]

and is read back as a `HuffmanTensor`, whose `to_gpu` sends the compressed bytes to the device and decodes there.

Where the reference returns `io::Error` (short reads, invalid UTF-8) this raises `ValueError`; where
it asserts (`expected dtype=1`, `quantized tensors must be 2D`) this raises `SerialPanic`.
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import BinaryIO, Optional, Tuple

import numpy as np

from . import _lib
from .quant import QuantizedTensor
from .runtime import GpuContext, _ptr, current_gpu


class SerialPanic(RuntimeError):
    """A condition on which the reference panics (`assert_eq!`)."""


def write_quantized_tensor(file: BinaryIO, name: str, qt: QuantizedTensor) -> None:
    """src/serial.rs:124-157"""
    name_bytes = name.encode("utf-8")
    data = np.ascontiguousarray(qt.data_i8, np.int8).reshape(-1)
    scales = np.ascontiguousarray(qt.scales, np.float32).reshape(-1)
    if data.size != qt.rows * qt.cols or scales.size != qt.cols:
        raise ValueError("write_quantized_tensor: array sizes do not match rows x cols")
    file.write(struct.pack("<I", len(name_bytes)))
    file.write(name_bytes)
    file.write(b"\x01")                                   # dtype tag: 1 = i8 quantised
    file.write(struct.pack("<III", 2, qt.rows, qt.cols))
    file.write(data.tobytes())
    file.write(scales.astype("<f4", copy=False).tobytes())


def _read_exact(file: BinaryIO, n: int) -> bytes:
    b = file.read(n)
    if len(b) != n:
        raise ValueError("failed to fill whole buffer")   # what io::Read::read_exact reports
    return b


def read_quantized_tensor(file: BinaryIO, gpu: Optional[GpuContext] = None) -> Tuple[str, QuantizedTensor]:
    """src/serial.rs:159-222.  The returned tensor is already on the GPU (`on_gpu`)."""
    (name_len,) = struct.unpack("<I", _read_exact(file, 4))
    try:
        name = _read_exact(file, name_len).decode("utf-8")
    except UnicodeDecodeError as e:
        raise ValueError(f"invalid utf-8 sequence: {e}") from e
    dtype = _read_exact(file, 1)[0]
    if dtype != 1:
        raise SerialPanic("expected dtype=1 (i8) for quantized tensor")
    (ndim,) = struct.unpack("<I", _read_exact(file, 4))
    if ndim != 2:
        raise SerialPanic("quantized tensors must be 2D")
    rows, cols = struct.unpack("<II", _read_exact(file, 8))
    data_i8 = np.frombuffer(_read_exact(file, rows * cols), np.int8).reshape(rows, cols).copy()
    scales = np.frombuffer(_read_exact(file, cols * 4), "<f4").astype(np.float32)
    gpu = gpu or current_gpu()
    h = C.c_void_p()
    _lib.check(gpu.lib.pg_qtensor_from_i8(gpu.handle, _ptr(data_i8), _ptr(scales), rows, cols, C.byref(h)))
    qt = QuantizedTensor(data_i8, np.empty((cols, rows), np.int8), scales, rows, cols)
    qt._gpu, qt._gpu_ctx = h, gpu
    if rows * cols:
        # the pre-transposed layout, built on the device, read back so that the host fields are whole
        keep_q, keep_s = qt.data_i8.copy(), qt.scales.copy()
        qt.from_gpu(gpu)
        assert np.array_equal(qt.data_i8, keep_q) and np.array_equal(qt.scales.view(np.uint32), keep_s.view(np.uint32))
    return name, qt


def write_huffman_tensor(file: BinaryIO, name: str, ht) -> None:
    """src/serial.rs:320-365"""
    name_bytes = name.encode("utf-8")
    scales = np.ascontiguousarray(ht.scales, np.float32).reshape(-1)
    if len(ht.streams) != ht.num_streams or len(ht.stream_lengths) != ht.num_streams:
        raise ValueError("write_huffman_tensor: one stream and one length per stream")
    file.write(struct.pack("<I", len(name_bytes)))
    file.write(name_bytes)
    file.write(b"\x03")                                   # dtype tag: 3 = Huffman coded
    file.write(struct.pack("<III", 2, ht.rows, ht.cols))
    file.write(ht.table.to_bytes())
    file.write(struct.pack("<I", ht.num_streams))
    file.write(struct.pack(f"<{ht.num_streams}I", *ht.stream_lengths))
    file.write(struct.pack(f"<{ht.num_streams}I", *[len(s) for s in ht.streams]))
    for s in ht.streams:
        file.write(bytes(s))
    file.write(scales.astype("<f4", copy=False).tobytes())


def read_huffman_tensor(file: BinaryIO):
    """src/serial.rs:367-443 -> (name, HuffmanTensor)."""
    from .huffman import HuffmanTable, HuffmanTensor

    (name_len,) = struct.unpack("<I", _read_exact(file, 4))
    try:
        name = _read_exact(file, name_len).decode("utf-8")
    except UnicodeDecodeError as e:
        raise ValueError(f"invalid utf-8 sequence: {e}") from e
    dtype = _read_exact(file, 1)[0]
    if dtype != 3:
        raise SerialPanic("expected dtype=3 (Huffman) for huffman tensor")
    (ndim,) = struct.unpack("<I", _read_exact(file, 4))
    if ndim != 2:
        raise SerialPanic("huffman tensors must be 2D")
    rows, cols = struct.unpack("<II", _read_exact(file, 8))
    table = HuffmanTable.from_bytes(_read_exact(file, 256))
    (num_streams,) = struct.unpack("<I", _read_exact(file, 4))
    lengths = list(struct.unpack(f"<{num_streams}I", _read_exact(file, 4 * num_streams)))
    sizes = struct.unpack(f"<{num_streams}I", _read_exact(file, 4 * num_streams))
    streams = [_read_exact(file, n) for n in sizes]
    scales = np.frombuffer(_read_exact(file, cols * 4), "<f4").astype(np.float32)
    return name, HuffmanTensor(table, streams, lengths, scales, rows, cols, num_streams)

