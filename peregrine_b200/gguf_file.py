"""The GGUF container: host-side mirror of `GgufFile` (src/gguf.rs:140-283, 403-567).

    GgufFile.load(path) / GgufFile.parse(bytes)        src/gguf.rs:405-482
    .metadata, .tensors[name] -> GgufTensor            src/gguf.rs:142-177
    .load_tensor_f32(name)                             src/gguf.rs:485-517
    .load_tensor_q8(name)                              src/gguf.rs:519-537
    .get_metadata / get_u32 / get_f32 / tensor_shape / tensor_names   src/gguf.rs:539-566

Parsing is byte bookkeeping and stays on the host; everything that touches tensor DATA goes to the
GPU through the library: block dequantisation (`pg_dequant_blocks_host`), f16 widening
(`pg_f16_to_f32`), the Q8_0 -> per-column int8 requantisation (`pg_qtensor_from_q8_0`).  On top of
the reference's API, `load_tensor_blocks` keeps a Q4_0 / Q8_0 / Q4_1 matrix in block form on the GPU
(`GgufWeight`), which is what a Llama linear then multiplies by, never materialising the f32 weight.

Where the reference returns `io::Error` this raises `ValueError` with the same message; where it
panics (`unknown GGUF metadata value type`, `unsupported GGML type`, `tensor ... not found`) this
raises `GgufPanic`.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from . import _lib
from .gguf import GgufWeight, _dequant, f16_to_f32, load_tensor_q8_as_quantized
from .quant import QuantizedTensor
from .runtime import GpuContext

GGUF_MAGIC = 0x46554747  # "GGUF" read as a little-endian u32 (src/gguf.rs:10)

# GgmlType (src/gguf.rs:13-56): value -> (name, elements per block, bytes per block)
GGML_TYPES = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 8: ("Q8_0", 32, 34)}
_BLOCK_KIND = {2: _lib.GGUF_Q4_0, 3: _lib.GGUF_Q4_1, 8: _lib.GGUF_Q8_0}


class GgufPanic(RuntimeError):
    """A condition on which the reference panics."""


@dataclass
class GgufTensor:
    """src/gguf.rs:142-161.  `shape` is in file order (innermost dimension first)."""
    name: str
    dtype: int
    shape: List[int]
    data_offset: int

    def num_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def data_size(self) -> int:
        _, bs, bb = GGML_TYPES[self.dtype]
        n = self.num_elements()
        if n % bs != 0:
            raise GgufPanic(f"tensor elements {n} not divisible by block size {bs}")
        return (n // bs) * bb


class _Reader:
    """Little-endian cursor over the file bytes (src/gguf.rs:180-283).  Reads past the end raise GgufPanic
    (the reference's slice indexing panics)."""

    def __init__(self, data: bytes):
        self.data, self.pos = data, 0

    def _take(self, fmt: str, size: int):
        if self.pos + size > len(self.data):
            raise GgufPanic(f"GGUF header truncated at byte {self.pos}")
        (v,) = struct.unpack_from(fmt, self.data, self.pos)
        self.pos += size
        return v

    def u8(self): return self._take("<B", 1)
    def i8(self): return self._take("<b", 1)
    def u16(self): return self._take("<H", 2)
    def i16(self): return self._take("<h", 2)
    def u32(self): return self._take("<I", 4)
    def i32(self): return self._take("<i", 4)
    def u64(self): return self._take("<Q", 8)
    def i64(self): return self._take("<q", 8)
    def f32(self): return np.frombuffer(struct.pack("<I", self.u32()), np.float32)[0]   # bit pattern kept
    def f64(self): return self._take("<d", 8)
    def boolean(self): return self.u8() != 0

    def string(self) -> str:
        n = self.u64()
        if self.pos + n > len(self.data):
            raise GgufPanic(f"GGUF string of {n} bytes runs past the end of the file")
        try:
            s = self.data[self.pos:self.pos + n].decode("utf-8")
        except UnicodeDecodeError as e:
            raise GgufPanic("invalid UTF-8 in GGUF string") from e
        self.pos += n
        return s

    def value(self, vtype: int):
        simple = {0: self.u8, 1: self.i8, 2: self.u16, 3: self.i16, 4: self.u32, 5: self.i32, 6: self.f32, 7: self.boolean,
                  8: self.string, 10: self.u64, 11: self.i64, 12: self.f64}
        if vtype in simple:
            return simple[vtype]()
        if vtype == 9:
            arr_type, arr_len = self.u32(), self.u64()
            return [self.value(arr_type) for _ in range(arr_len)]
        raise GgufPanic(f"unknown GGUF metadata value type: {vtype}")


def _as_u32(v) -> Optional[int]:
    """MetadataValue::as_u32 (src/gguf.rs:78-86): the integer types the reference accepts, truncated to 32 bits."""
    if isinstance(v, bool) or not isinstance(v, (int, np.integer)):
        return None
    return int(v) & 0xFFFFFFFF


class GgufFile:
    def __init__(self, metadata: Dict[str, object], tensors: Dict[str, GgufTensor], data: bytes, data_start: int,
                 gpu: Optional[GpuContext] = None):
        self.metadata, self.tensors, self._data, self.data_start, self.gpu = metadata, tensors, data, data_start, gpu

    # ---- parsing (src/gguf.rs:405-482) -------------------------------------------------------
    @classmethod
    def load(cls, path: str, gpu: Optional[GpuContext] = None) -> "GgufFile":
        with open(path, "rb") as f:
            return cls.parse(f.read(), gpu)

    @classmethod
    def parse(cls, data: bytes, gpu: Optional[GpuContext] = None) -> "GgufFile":
        data = bytes(data)
        r = _Reader(data)
        magic = r.u32()
        if magic != GGUF_MAGIC:
            raise ValueError(f"invalid GGUF magic: 0x{magic:08X}, expected 0x{GGUF_MAGIC:08X}")
        version = r.u32()
        if version < 2 or version > 3:
            raise ValueError(f"unsupported GGUF version: {version}")
        n_tensors, n_kv = r.u64(), r.u64()
        metadata: Dict[str, object] = {}
        # value types are kept beside the values: as_u32 / as_f32 depend on them (an integer is not a float)
        kinds: Dict[str, int] = {}
        for _ in range(n_kv):
            key = r.string()
            vtype = r.u32()
            metadata[key] = r.value(vtype)
            kinds[key] = vtype
        tensors: Dict[str, GgufTensor] = {}
        for _ in range(n_tensors):
            name = r.string()
            n_dims = r.u32()
            shape = [r.u64() for _ in range(n_dims)]
            dtype_raw = r.u32()
            if dtype_raw not in GGML_TYPES:
                raise GgufPanic(f"unsupported GGML type {dtype_raw} for tensor '{name}'")
            tensors[name] = GgufTensor(name, dtype_raw, shape, r.u64())
        # data starts at the next alignment boundary after the header (general.alignment, default 32)
        alignment = None
        if "general.alignment" in metadata and kinds["general.alignment"] in (4, 5, 10, 11):
            alignment = _as_u32(metadata["general.alignment"])
        if alignment is None:
            alignment = 32
        if alignment == 0:
            raise GgufPanic("attempt to divide by zero")   # what the reference's arithmetic does with alignment 0
        data_start = (r.pos + alignment - 1) // alignment * alignment
        out = cls(metadata, tensors, data, data_start, gpu)
        out._kinds = kinds
        return out

    # ---- metadata (src/gguf.rs:539-552) ------------------------------------------------------
    def get_metadata(self, key: str):
        return self.metadata.get(key)

    def get_u32(self, key: str) -> Optional[int]:
        if key not in self.metadata or self._kinds[key] not in (4, 5, 10, 11):
            return None
        return _as_u32(self.metadata[key])

    def get_f32(self, key: str) -> Optional[np.float32]:
        if key not in self.metadata or self._kinds[key] not in (6, 12):
            return None
        return np.float32(self.metadata[key])

    def tensor_shape(self, name: str) -> List[int]:
        """Shape in the reference's convention: the file's order reversed (src/gguf.rs:554-561)."""
        if name not in self.tensors:
            raise GgufPanic(f"tensor '{name}' not found")
        return list(reversed(self.tensors[name].shape))

    def tensor_names(self) -> List[str]:
        return list(self.tensors.keys())

    # ---- tensor data -------------------------------------------------------------------------
    def _raw(self, name: str):
        if name not in self.tensors:
            raise GgufPanic(f"tensor '{name}' not found in GGUF file")
        info = self.tensors[name]
        off, size = self.data_start + info.data_offset, info.data_size()
        if off + size > len(self._data):
            raise GgufPanic(f"tensor '{name}' runs past the end of the file")
        return info, np.frombuffer(self._data, np.uint8, size, off)

    def load_tensor_f32(self, name: str, gpu: Optional[GpuContext] = None) -> np.ndarray:
        """The tensor as flat f32 (src/gguf.rs:485-517); quantised and f16 data are widened on the GPU."""
        info, raw = self._raw(name)
        n = info.num_elements()
        if info.dtype == 0:
            return raw.view(np.float32).copy()
        gpu = gpu or self.gpu
        if info.dtype == 1:
            return f16_to_f32(raw.view(np.uint16), gpu) if n else np.empty(0, np.float32)
        return _dequant(_BLOCK_KIND[info.dtype], raw, n, gpu)

    @staticmethod
    def _rows_cols(info: GgufTensor):
        # GGUF shapes are [cols, rows] (src/gguf.rs:529-534)
        if len(info.shape) == 1:
            return 1, info.shape[0]
        if len(info.shape) == 2:
            return info.shape[1], info.shape[0]
        raise GgufPanic(f"expected 1D or 2D tensor for q8 load, got {info.shape}")

    def load_tensor_q8(self, name: str, gpu: Optional[GpuContext] = None) -> QuantizedTensor:
        """src/gguf.rs:519-537: the bytes are read as Q8_0 blocks of a [rows, cols] tensor, dequantised and
        requantised per column (the tensor's stored orientation, no transposition)."""
        info, raw = self._raw(name)
        rows, cols = self._rows_cols(info)
        return load_tensor_q8_as_quantized(raw, rows, cols, gpu or self.gpu)

    def load_tensor_blocks(self, name: str, gpu: Optional[GpuContext] = None, rows: Optional[tuple] = None) -> GgufWeight:
        """A 2-D Q4_0 / Q4_1 / Q8_0 tensor [out, in] kept in block form on the GPU: `matmul(x, m)` gives
        x . dequant(W)^T, what load_tensor_f32 + load_transposed_weight + Tensor::matmul compute
        (src/models/llama/model.rs:243-257).  `rows` keeps only a range of output rows (a column shard of the linear)."""
        info, raw = self._raw(name)
        if info.dtype not in _BLOCK_KIND:
            raise GgufPanic(f"tensor '{name}' is {GGML_TYPES[info.dtype][0]}, not a block-quantised type")
        n, k = self._rows_cols(info)
        return GgufWeight(_BLOCK_KIND[info.dtype], raw, n, k, gpu or self.gpu, rows)
