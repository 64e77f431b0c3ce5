"""Huffman-coded int8 weights: host-side mirror of `HuffmanTable`, `HuffmanTensor` and `matmul_huffman`
(src/huffman.rs:19-476, 726-737).

    HuffmanTable.from_frequencies / from_bytes / to_bytes / encode / decode / to_gpu_lut
    HuffmanTensor.from_quantized / decode_to_quantized / to_gpu / compressed_size / uncompressed_size / compression_ratio
    matmul_huffman(a, m, k, ht)

Building the code (256 symbols) and writing the bitstreams is offline conversion work and stays on the
host.  Everything on the loading side runs on the GPU: `decode`, `decode_to_quantized` and `to_gpu` send the
COMPRESSED bytes to the device, where every stream is decoded by thousands of threads and the GEMM
layout is built; the reference decodes on the host and uploads the decoded bytes
(src/huffman.rs:430-437).  `HuffmanKVCache` (src/huffman.rs:484-724) is not part of this package.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from .quant import QuantizedTensor, matmul_quantized
from .runtime import GpuContext, _ptr, current_gpu

NUM_SYMBOLS = 256     # src/huffman.rs:10
MAX_LUT_BITS = 12     # src/huffman.rs:13


def _canonical_codes(bit_lengths: np.ndarray) -> np.ndarray:
    """src/huffman.rs:155-190: codes in order of (length, symbol)."""
    codes = np.zeros(NUM_SYMBOLS, np.uint32)
    longest = int(bit_lengths.max())
    if longest == 0:
        return codes
    per_len = np.bincount(bit_lengths, minlength=longest + 1).astype(np.uint64)
    per_len[0] = 0
    first = [0] * (longest + 1)
    code = 0
    for bits in range(1, longest + 1):
        code = ((code + int(per_len[bits - 1])) << 1) & 0xFFFFFFFF
        first[bits] = code
    for s in range(NUM_SYMBOLS):
        bl = int(bit_lengths[s])
        if bl:
            codes[s] = first[bl] & 0xFFFFFFFF
            first[bl] += 1
    return codes


def _fit_lengths(lengths: np.ndarray, freqs: List[int]) -> np.ndarray:
    """Lengths of at most 12 bits whose Kraft sum exceeds 1 -> lengths of a prefix code (not in the reference)."""
    full = 1 << MAX_LUT_BITS
    lens = [int(v) for v in lengths]
    used = sum(full >> l for l in lens if l)
    if used <= full:
        return lengths
    rare_first = sorted((i for i in range(NUM_SYMBOLS) if lens[i]), key=lambda i: (freqs[i], i))
    while used > full:
        # the rarest symbol among the longest codes that can still grow
        grow = max((i for i in rare_first if lens[i] < MAX_LUT_BITS), key=lambda i: (lens[i], -freqs[i], -i))
        used -= full >> (lens[grow] + 1)
        lens[grow] += 1
    for i in reversed(rare_first):                      # most frequent first: take back the slack
        while lens[i] > 1 and used + (full >> lens[i]) <= full:
            used += full >> lens[i]
            lens[i] -= 1
    return np.array(lens, np.uint8)


class HuffmanTable:
    """A canonical code over the 256 int8 values; index = value + 128 (src/huffman.rs:19-30)."""

    def __init__(self, bit_lengths: np.ndarray):
        self.bit_lengths = np.ascontiguousarray(bit_lengths, np.uint8).reshape(NUM_SYMBOLS).copy()
        self.codes = _canonical_codes(self.bit_lengths)
        # the reference builds its decode table with the code (build_decode_lut, src/huffman.rs:193-213) and panics
        # there when the lengths over-subscribe the 12-bit table; so does this
        self.decode_lut = self.to_gpu_lut()

    # ---- construction ---------------------------------------------------------------------------
    @classmethod
    def from_frequencies(cls, freqs: Sequence[int], limit_lengths: bool = False) -> "HuffmanTable":
        """src/huffman.rs:35-152.  The tree is built with two queues over the symbols in (frequency, symbol)
        order; a leaf wins a tie against an inner node; depths beyond 12 are cut to 12 afterwards, as the
        reference does it.  A histogram whose tree is deeper than 12 therefore ends in `HuffmanPanic`, as it
        ends in a panic there (the cut lengths no longer fit the 4096-entry table): int8 weights of a few
        million values with a Gaussian tail are such a histogram.

        `limit_lengths=True` is an addition to the reference's interface: the cut lengths are repaired into a
        complete code of at most 12 bits (rare symbols give up a bit until the lengths fit, then frequent ones
        take back what is left).  The code book it writes is an ordinary one: the reference's `from_bytes`
        and `decode` read it."""
        f = [int(v) for v in np.asarray(freqs).reshape(NUM_SYMBOLS)]
        active = [i for i in range(NUM_SYMBOLS) if f[i] > 0]
        lengths = np.zeros(NUM_SYMBOLS, np.uint8)
        if len(active) == 1:
            lengths[active[0]] = 1
        elif len(active) > 1:
            n = len(active)
            leaves = sorted(range(n), key=lambda i: f[active[i]])          # stable, like sort_by_key
            leaf_q = [(f[active[i]], i) for i in leaves]
            inner_q: List[tuple] = []
            lh = ih = 0
            parent = [0] * (2 * n - 1)
            for node in range(n, 2 * n - 1):
                pair = []
                for _ in range(2):
                    if lh < len(leaf_q) and (ih >= len(inner_q) or leaf_q[lh][0] <= inner_q[ih][0]):
                        pair.append(leaf_q[lh])
                        lh += 1
                    else:
                        pair.append(inner_q[ih])
                        ih += 1
                parent[pair[0][1]] = parent[pair[1][1]] = node
                inner_q.append((pair[0][0] + pair[1][0], node))
            depth = [0] * (2 * n - 1)
            for i in range(2 * n - 3, -1, -1):
                depth[i] = (depth[parent[i]] + 1) & 0xFF                    # the reference counts in u8
            for i in range(n):
                lengths[active[i]] = min(depth[i], MAX_LUT_BITS)
            if limit_lengths:
                lengths = _fit_lengths(lengths, f)
        return cls(lengths)

    @classmethod
    def from_bytes(cls, data: bytes) -> "HuffmanTable":
        """src/huffman.rs:292-307"""
        if len(data) < NUM_SYMBOLS:
            raise HuffmanPanic("codebook too short")
        return cls(np.frombuffer(bytes(data[:NUM_SYMBOLS]), np.uint8))

    def to_bytes(self) -> bytes:
        """src/huffman.rs:287-289: the 256 bit lengths."""
        return self.bit_lengths.tobytes()

    def to_gpu_lut(self) -> np.ndarray:
        """The 4096-entry decode table as the reference packs it for a GPU (src/huffman.rs:193-213, 726-737):
        (bit_length << 8) | (value + 128); (length 0, value 0) where no code starts with the 12 bits."""
        lut = np.full(1 << MAX_LUT_BITS, 128, np.uint32)
        for s in range(NUM_SYMBOLS):
            bl = int(self.bit_lengths[s])
            if bl == 0 or bl > MAX_LUT_BITS:
                continue
            shift = MAX_LUT_BITS - bl
            base = int(self.codes[s]) << shift
            if base + (1 << shift) > lut.size:
                raise HuffmanPanic("index out of bounds: the bit lengths do not describe a code of at most 12 bits")
            lut[base:base + (1 << shift)] = (bl << 8) | s
        return lut

    # ---- coding ---------------------------------------------------------------------------------
    def encode(self, data) -> bytes:
        """src/huffman.rs:216-251: code words MSB first, the last byte padded with zeros."""
        d = np.ascontiguousarray(data, np.int8).reshape(-1)
        if d.size == 0:
            return b""
        out = []
        carry = np.zeros(0, np.uint8)           # bits that did not fill a byte yet
        step = 1 << 22
        for i in range(0, d.size, step):
            idx = d[i:i + step].astype(np.int16) + 128
            lens = self.bit_lengths[idx].astype(np.int64)
            codes = self.codes[idx]
            ends = np.cumsum(lens)
            bits = np.zeros(int(ends[-1]) + carry.size, np.uint8)
            bits[:carry.size] = carry
            first = ends - lens + carry.size
            for b in range(int(lens.max()) if lens.size else 0):
                sel = lens > b
                bits[first[sel] + b] = (codes[sel] >> (lens[sel] - 1 - b).astype(np.uint32)) & 1
            whole = bits.size // 8 * 8
            out.append(np.packbits(bits[:whole]).tobytes())
            carry = bits[whole:].copy()
        if carry.size:
            out.append(np.packbits(carry).tobytes())     # packbits pads the last byte with zeros
        return b"".join(out)

    def decode(self, bitstream, num_symbols: int, gpu: Optional[GpuContext] = None) -> np.ndarray:
        """src/huffman.rs:254-284, on the GPU."""
        return _decode_streams(self, [bitstream], [num_symbols], gpu)


class HuffmanPanic(RuntimeError):
    """A condition on which the reference panics."""


def _stream_tables(streams, stream_lengths):
    blobs = [np.frombuffer(bytes(s), np.uint8) if not isinstance(s, np.ndarray) else np.ascontiguousarray(s, np.uint8).reshape(-1)
             for s in streams]
    sizes = np.array([b.size for b in blobs], np.uint64)
    lens = np.array([int(n) for n in stream_lengths], np.uint64)
    if len(blobs) != len(lens):
        raise ValueError("one length per stream")
    packed = np.concatenate(blobs) if blobs and int(sizes.sum()) else np.zeros(1, np.uint8)
    return np.ascontiguousarray(packed), sizes, lens


def _decode_streams(table: HuffmanTable, streams, stream_lengths, gpu: Optional[GpuContext]) -> np.ndarray:
    gpu = gpu or current_gpu()
    packed, sizes, lens = _stream_tables(streams, stream_lengths)
    out = np.empty(int(lens.sum()), np.int8)
    if out.size:
        _lib.check(gpu.lib.pg_huffman_decode_host(gpu.handle, _ptr(table.bit_lengths), len(lens), _ptr(lens), _ptr(sizes),
                                                  _ptr(packed), _ptr(out)))
    return out


class HuffmanTensor:
    """src/huffman.rs:311-325: per-column scales plus the int8 matrix as `num_streams` Huffman bitstreams."""

    def __init__(self, table: HuffmanTable, streams: List[bytes], stream_lengths: List[int], scales: np.ndarray, rows: int, cols: int,
                 num_streams: int):
        self.table, self.streams, self.stream_lengths = table, streams, [int(n) for n in stream_lengths]
        self.scales = np.ascontiguousarray(scales, np.float32).reshape(-1)
        self.rows, self.cols, self.num_streams = int(rows), int(cols), int(num_streams)

    @classmethod
    def from_quantized(cls, qt: QuantizedTensor, num_streams: int, limit_lengths: bool = False) -> "HuffmanTensor":
        """src/huffman.rs:332-371: one code from the histogram of the whole matrix; the row-major bytes cut into
        `num_streams` equal chunks (the last ones may be short or empty), each coded on its own.
        `limit_lengths`: see HuffmanTable.from_frequencies."""
        num_streams = max(int(num_streams), 1)
        data = np.ascontiguousarray(qt.data_i8, np.int8).reshape(-1)
        total = data.size
        freqs = np.bincount(data.astype(np.int16) + 128, minlength=NUM_SYMBOLS)
        table = HuffmanTable.from_frequencies(freqs, limit_lengths)
        chunk = (total + num_streams - 1) // num_streams
        streams, lengths = [], []
        for s in range(num_streams):
            lo = s * chunk
            part = data[lo:min(lo + chunk, total)] if lo < total else data[:0]
            streams.append(table.encode(part))
            lengths.append(part.size)
        return cls(table, streams, lengths, qt.scales.copy(), qt.rows, qt.cols, num_streams)

    def to_gpu(self, gpu: Optional[GpuContext] = None) -> QuantizedTensor:
        """src/huffman.rs:430-437, with the decode on the device: the resident tensor `pg_matmul_quantized` multiplies
        by.  Its host arrays are left empty (`from_gpu` fills them)."""
        gpu = gpu or current_gpu()
        if sum(self.stream_lengths) != self.rows * self.cols:
            raise HuffmanPanic(f"assertion failed: the streams hold {sum(self.stream_lengths)} symbols, {self.rows * self.cols} expected")
        # the streams back to back, as a file holds them; kept for the next call while the streams stay the same objects
        key = (tuple(id(x) for x in self.streams), tuple(self.stream_lengths))
        if getattr(self, "_packed_key", None) != key:
            self._packed, self._packed_key = _stream_tables(self.streams, self.stream_lengths), key
        packed, sizes, lens = self._packed
        h = C.c_void_p()
        _lib.check(gpu.lib.pg_qtensor_from_huffman(gpu.handle, _ptr(self.table.bit_lengths), len(lens), _ptr(lens), _ptr(sizes),
                                                   _ptr(packed), _ptr(self.scales), self.rows, self.cols, C.byref(h)))
        qt = QuantizedTensor(np.empty((self.rows, self.cols), np.int8), np.empty((self.cols, self.rows), np.int8), self.scales.copy(),
                             self.rows, self.cols)
        qt._gpu, qt._gpu_ctx = h, gpu
        return qt

    def decode_to_quantized(self, gpu: Optional[GpuContext] = None) -> QuantizedTensor:
        """src/huffman.rs:374-404: the tensor with all its host fields, and resident on the GPU that decoded it."""
        qt = self.to_gpu(gpu)
        if self.rows * self.cols:
            qt.from_gpu(qt._gpu_ctx)
        return qt

    def compressed_size(self) -> int:
        """src/huffman.rs:407-412: bitstreams + code book + scales, in bytes."""
        return sum(len(s) for s in self.streams) + NUM_SYMBOLS + self.cols * 4

    def uncompressed_size(self) -> int:
        return self.rows * self.cols + self.cols * 4

    def compression_ratio(self) -> np.float32:
        return np.float32(self.uncompressed_size()) / np.float32(self.compressed_size())


def matmul_huffman(a_data, m: int, k: int, ht: HuffmanTensor, gpu: Optional[GpuContext] = None) -> np.ndarray:
    """src/huffman.rs:465-476: decode, then `matmul_quantized`."""
    if ht.rows != k:
        raise HuffmanPanic(f"assertion `left == right` failed: ht.rows = {ht.rows}, k = {k}")
    qt = ht.to_gpu(gpu)
    try:
        return matmul_quantized(a_data, m, k, qt, gpu)
    finally:
        qt.free_gpu()
