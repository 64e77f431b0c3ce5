"""The quantised serial formats: host-side mirror of `write_quantized_tensor` / `read_quantized_tensor`
(src/serial.rs:124-222), of `write_huffman_tensor` / `read_huffman_tensor` (src/serial.rs:315-443), of
`save_model` / `load_model` (src/serial.rs:10-86) and of the two converters the reference ships as scripts
(scripts/convert_weights_int8.py, scripts/convert_huffman.py).

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
import os
import struct
from typing import BinaryIO, List, Optional, Sequence, Tuple

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


def _read_name(file: BinaryIO) -> str:
    (name_len,) = struct.unpack("<I", _read_exact(file, 4))
    try:
        return _read_exact(file, name_len).decode("utf-8")
    except UnicodeDecodeError as e:
        raise ValueError(f"invalid utf-8 sequence: {e}") from e


def _read_i8_body(file: BinaryIO, gpu: Optional[GpuContext]) -> QuantizedTensor:
    """What follows the dtype byte of an i8 record (src/serial.rs:188-222)."""
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
    return qt


def read_quantized_tensor(file: BinaryIO, gpu: Optional[GpuContext] = None) -> Tuple[str, QuantizedTensor]:
    """src/serial.rs:159-222.  The returned tensor is already on the GPU (`on_gpu`)."""
    name = _read_name(file)
    dtype = _read_exact(file, 1)[0]
    if dtype != 1:
        raise SerialPanic("expected dtype=1 (i8) for quantized tensor")
    return name, _read_i8_body(file, gpu)


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


def _read_huffman_body(file: BinaryIO):
    """What follows the dtype byte of a Huffman record (src/serial.rs:385-443)."""
    from .huffman import HuffmanTable, HuffmanTensor

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
    return HuffmanTensor(table, streams, lengths, scales, rows, cols, num_streams)


def read_huffman_tensor(file: BinaryIO):
    """src/serial.rs:367-443 -> (name, HuffmanTensor)."""
    name = _read_name(file)
    dtype = _read_exact(file, 1)[0]
    if dtype != 3:
        raise SerialPanic("expected dtype=3 (Huffman) for huffman tensor")
    return name, _read_huffman_body(file)


# ---- whole model files ---------------------------------------------------------------------------------------------
def load_model(path: str) -> List[Tuple[str, List[int], np.ndarray]]:
    """serial::load_model (src/serial.rs:44-86): [num_tensors: u32] then [name][ndim: u32][shape: u32 each][f32 data] per
    tensor -> (name, shape, flat f32 data) triples."""
    out = []
    with open(path, "rb") as f:
        (count,) = struct.unpack("<I", _read_exact(f, 4))
        for _ in range(count):
            name = _read_name(f)
            (ndim,) = struct.unpack("<I", _read_exact(f, 4))
            shape = list(struct.unpack(f"<{ndim}I", _read_exact(f, 4 * ndim)))
            n = int(np.prod(shape, dtype=np.int64)) if shape else 1
            out.append((name, shape, np.frombuffer(_read_exact(f, 4 * n), "<f4").astype(np.float32)))
    return out


def save_model(params: Sequence[Tuple[str, Sequence[int], np.ndarray]], path: str) -> None:
    """serial::save_model (src/serial.rs:10-41) for (name, shape, data) triples."""
    with open(path, "wb") as f:
        f.write(struct.pack("<I", len(params)))
        for name, shape, data in params:
            nb = name.encode("utf-8")
            f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", len(shape)) + struct.pack(f"<{len(shape)}I", *shape))
            f.write(np.ascontiguousarray(data, np.float32).astype("<f4", copy=False).tobytes())


def load_typed_model(path: str, gpu: Optional[GpuContext] = None) -> List[Tuple[str, object]]:
    """A file of typed records, as scripts/convert_weights_int8.py:44-81 and scripts/convert_huffman.py:266-300 write them:
    [num_tensors: u32] then per tensor [name][dtype: u8] and
        dtype 0   [ndim][shape][f32 data]         -> (shape, flat f32 array)
        dtype 1   an i8 record                    -> QuantizedTensor, resident on the GPU
        dtype 3   a Huffman record                -> HuffmanTensor (`to_gpu` decodes it on the device)
    The 2:4 sparse records (dtype 2, src/serial.rs:226-313) are not read."""
    out: List[Tuple[str, object]] = []
    with open(path, "rb") as f:
        (count,) = struct.unpack("<I", _read_exact(f, 4))
        for _ in range(count):
            name = _read_name(f)
            dtype = _read_exact(f, 1)[0]
            if dtype == 0:
                (ndim,) = struct.unpack("<I", _read_exact(f, 4))
                shape = list(struct.unpack(f"<{ndim}I", _read_exact(f, 4 * ndim)))
                n = int(np.prod(shape, dtype=np.int64)) if shape else 1
                out.append((name, (shape, np.frombuffer(_read_exact(f, 4 * n), "<f4").astype(np.float32))))
            elif dtype == 1:
                out.append((name, _read_i8_body(f, gpu)))
            elif dtype == 3:
                out.append((name, _read_huffman_body(f)))
            else:
                raise SerialPanic(f"unsupported dtype {dtype} for tensor '{name}'")
    return out


def convert_weights_int8(input_path: str, output_path: str, gpu: Optional[GpuContext] = None) -> None:
    """scripts/convert_weights_int8.py: an f32 model file -> a typed file in which every 2-D tensor whose name contains
    ".weight" is an i8 record and everything else an f32 record.  The quantiser is `quantize_weights` on the GPU
    (src/quant.rs:27-75: half away from zero; the script's numpy rounding is half to even, so a value that lies
    exactly on a tie differs by one step, and nothing else does)."""
    from .quant import quantize_weights

    tensors = load_model(input_path)
    with open(output_path, "wb") as f:
        f.write(struct.pack("<I", len(tensors)))
        for name, shape, data in tensors:
            if len(shape) == 2 and ".weight" in name:
                write_quantized_tensor(f, name, quantize_weights(data, shape[0], shape[1], gpu))
            else:
                nb = name.encode("utf-8")
                f.write(struct.pack("<I", len(nb)) + nb + b"\x00" + struct.pack("<I", len(shape)) + struct.pack(f"<{len(shape)}I", *shape))
                f.write(data.astype("<f4", copy=False).tobytes())


def _walk(path: str, typed: bool) -> bool:
    """True when the file's records, read as typed (a dtype byte after every name) or as plain f32 records, follow one
    another consistently and end exactly at the end of the file.  Only headers are read."""
    size = os.path.getsize(path)
    try:
        with open(path, "rb") as f:
            (count,) = struct.unpack("<I", _read_exact(f, 4))
            for _ in range(count):
                (name_len,) = struct.unpack("<I", _read_exact(f, 4))
                if name_len > size:
                    return False
                _read_exact(f, name_len).decode("utf-8")
                dtype = _read_exact(f, 1)[0] if typed else 0
                (ndim,) = struct.unpack("<I", _read_exact(f, 4))
                if ndim > 8:
                    return False
                shape = struct.unpack(f"<{ndim}I", _read_exact(f, 4 * ndim))
                n = int(np.prod(shape, dtype=np.int64)) if shape else 1
                if dtype == 0:
                    skip = 4 * n
                elif dtype == 1 and ndim == 2:
                    skip = n + 4 * shape[1]
                elif dtype == 3 and ndim == 2:
                    f.seek(256, 1)
                    (streams,) = struct.unpack("<I", _read_exact(f, 4))
                    if streams > size:
                        return False
                    f.seek(4 * streams, 1)
                    skip = sum(struct.unpack(f"<{streams}I", _read_exact(f, 4 * streams))) + 4 * shape[1]
                else:
                    return False
                if f.tell() + skip > size:
                    return False
                f.seek(skip, 1)
            return f.tell() == size
    except (ValueError, struct.error, UnicodeDecodeError):
        return False


def file_kind(path: str) -> str:
    """"typed" (records with a dtype byte, scripts/convert_weights_int8.py) or "plain" (serial::save_model).  The two
    layouts differ by one byte per record, so the whole chain of record headers is followed under each reading and must
    end at the end of the file; the reference's script looks at one byte of each record instead and takes the rank of a
    plain tensor for a dtype.  A file that fits neither reading, or both, is refused."""
    typed, plain = _walk(path, True), _walk(path, False)
    if typed == plain:
        with open(path, "rb") as f:
            empty = os.path.getsize(path) == 4 and f.read(4) == b"\0\0\0\0"
        if empty:
            return "plain"
        raise SerialPanic(f"{path}: " + ("reads both as a typed and as a plain model file" if typed else "neither a typed nor a plain model file"))
    return "typed" if typed else "plain"


def convert_huffman(input_path: str, output_path: str, num_streams: int = 4, limit_lengths: bool = False,
                    gpu: Optional[GpuContext] = None) -> None:
    """scripts/convert_huffman.py: a typed file (or a plain f32 model file) -> a file of Huffman records for its 2-D
    tensors; f32 tensors are quantised first, tensors of other ranks are left out, as the script leaves them out.
    The code is built by HuffmanTable.from_frequencies (the tie rules of src/huffman.rs, not those of the script's
    heap): both are optimal prefix codes, the bytes may differ, the decoded tensors do not."""
    from .huffman import HuffmanTensor
    from .quant import quantize_weights

    kind = file_kind(input_path)
    records: List[Tuple[str, QuantizedTensor]] = []
    if kind == "typed":
        for name, item in load_typed_model(input_path, gpu):
            if isinstance(item, QuantizedTensor):
                records.append((name, item))
            elif isinstance(item, tuple):
                shape, data = item
                if len(shape) == 2:               # an f32 record of a typed file: quantised like a plain file's tensor
                    records.append((name, quantize_weights(data, shape[0], shape[1], gpu)))
            else:
                raise ValueError(f"Unsupported dtype for conversion: tensor '{name}'")
    else:
        for name, shape, data in load_model(input_path):
            if len(shape) == 2:
                records.append((name, quantize_weights(data, shape[0], shape[1], gpu)))
    with open(output_path, "wb") as f:
        f.write(struct.pack("<I", len(records)))
        for name, qt in records:
            write_huffman_tensor(f, name, HuffmanTensor.from_quantized(qt, num_streams, limit_lengths))
