"""numpy front end of the CPU oracle (oracle/peregrine_oracle.c, oracle/gguf_encode.c, oracle/huffman_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports it.

Function names and argument order follow the reference's Rust API
(src/quant.rs, src/gguf.rs) so that tests read like the reference's own.
`Oracle(mt=False)` is the reference-equivalent single-thread build,
`Oracle(mt=True)` the OpenMP build (identical results, all host cores).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
_sz = C.c_size_t


def build(force: bool = False) -> None:
    """Compile both oracle libraries with oracle/Makefile (gcc only)."""
    libs = [os.path.join(_BUILD, n) for n in ("libpgoracle.so", "libpgoracle_mt.so")]
    srcs = [os.path.join(_HERE, n) for n in ("peregrine_oracle.c", "gguf_encode.c", "huffman_oracle.c", "Makefile")]
    stale = force or any(
        not os.path.exists(l) or os.path.getmtime(l) < max(os.path.getmtime(s) for s in srcs) for l in libs
    )
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)


@dataclass
class QuantizedTensor:
    """Mirror of `peregrine::quant::QuantizedTensor` (src/quant.rs:12-23)."""

    data_i8: np.ndarray    # [rows, cols] = [K, N]
    data_i8_t: np.ndarray  # [cols, rows] = [N, K]
    scales: np.ndarray     # [cols]
    rows: int
    cols: int


class Oracle:
    def __init__(self, mt: bool = False):
        build()
        path = os.path.join(_BUILD, "libpgoracle_mt.so" if mt else "libpgoracle.so")
        self.lib = lib = C.CDLL(path)
        self.mt = mt
        lib.pgo_num_threads.restype = C.c_int
        lib.pgo_f16_to_f32.restype = C.c_float
        lib.pgo_f16_to_f32.argtypes = [C.c_uint16]
        lib.pgo_f16_to_f32_bits.argtypes = [np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS"), _sz,
                                            np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")]
        lib.pgo_f32_to_f16.restype = C.c_uint16
        lib.pgo_f32_to_f16.argtypes = [C.c_float]
        lib.pgo_quantize_weights.argtypes = [_f32p, _sz, _sz, _i8p, _i8p, _f32p]
        lib.pgo_quantize_activations.argtypes = [_f32p, _sz, _sz, _i8p, _f32p]
        lib.pgo_dequantize.argtypes = [_i8p, _f32p, _sz, _sz, _f32p]
        lib.pgo_gemm_i8.argtypes = [_i8p, _f32p, _i8p, _f32p, _sz, _sz, _sz, _f32p, _i32p]
        lib.pgo_gemm_i8_sampled.argtypes = [_i8p, _i8p, _sz, _sz, _i64p, _sz, _i32p]
        lib.pgo_matmul_quantized.argtypes = [_f32p, _sz, _sz, _i8p, _f32p, _sz, _f32p, _i32p, _i8p, _f32p]
        for name in ("pgo_dequant_q8_0", "pgo_dequant_q4_0", "pgo_dequant_q4_1"):
            f = getattr(lib, name)
            f.restype = C.c_int
            f.argtypes = [_u8p, _sz, _sz, _f32p]
        lib.pgo_matmul_f32.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _f32p]
        lib.pgo_matmul_f32_wt.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _f32p]
        lib.pgo_matmul_f64acc_wt.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _f64p]
        lib.pgo_matmul_dequant_w8a32.argtypes = [_f32p, _i8p, _f32p, _sz, _sz, _sz, _f32p]
        _u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
        _u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
        lib.pgo_huffman_from_frequencies.argtypes = [_u64p, _u8p, _u32p]
        lib.pgo_huffman_canonical_codes.argtypes = [_u8p, _u32p]
        lib.pgo_huffman_build_lut.argtypes = [_u8p, _u32p, _u32p]
        lib.pgo_huffman_encode.argtypes = [_u8p, _u32p, _i8p, _sz, _u8p]
        lib.pgo_huffman_encode.restype = _sz
        lib.pgo_huffman_decode.argtypes = [_u32p, _u8p, _sz, _sz, _i8p]
        for name in ("pgo_encode_q8_0", "pgo_encode_q4_0", "pgo_encode_q4_1"):
            getattr(lib, name).argtypes = [_f32p, _sz, _u8p]

    @property
    def threads(self) -> int:
        return int(self.lib.pgo_num_threads())

    # ---- src/quant.rs -------------------------------------------------
    def quantize_weights(self, data: np.ndarray, rows: int, cols: int) -> QuantizedTensor:
        data = np.ascontiguousarray(data, np.float32).reshape(-1)
        assert data.size == rows * cols
        q = np.empty((rows, cols), np.int8)
        qt = np.empty((cols, rows), np.int8)
        s = np.empty(cols, np.float32)
        self.lib.pgo_quantize_weights(data, rows, cols, q, qt, s)
        return QuantizedTensor(q, qt, s, rows, cols)

    def quantize_activations(self, data: np.ndarray, rows: int, cols: int):
        data = np.ascontiguousarray(data, np.float32).reshape(-1)
        assert data.size == rows * cols
        q = np.empty((rows, cols), np.int8)
        s = np.empty(rows, np.float32)
        self.lib.pgo_quantize_activations(data, rows, cols, q, s)
        return q, s

    def dequantize(self, qt: QuantizedTensor) -> np.ndarray:
        out = np.empty((qt.rows, qt.cols), np.float32)
        self.lib.pgo_dequantize(qt.data_i8, qt.scales, qt.rows, qt.cols, out)
        return out

    def matmul_quantized(self, a: np.ndarray, m: int, k: int, w: QuantizedTensor, return_parts: bool = False):
        assert w.rows == k
        a = np.ascontiguousarray(a, np.float32).reshape(-1)
        assert a.size == m * k
        n = w.cols
        out = np.empty((m, n), np.float32)
        acc = np.empty((m, n), np.int32)
        a_i8 = np.empty((m, k), np.int8)
        a_s = np.empty(m, np.float32)
        self.lib.pgo_matmul_quantized(a, m, k, w.data_i8_t, w.scales, n, out, acc, a_i8, a_s)
        if return_parts:
            return out, acc, a_i8, a_s
        return out

    def gemm_i8(self, a_i8, a_scales, b_t, w_scales, m, n, k):
        out = np.empty((m, n), np.float32)
        acc = np.empty((m, n), np.int32)
        self.lib.pgo_gemm_i8(np.ascontiguousarray(a_i8), np.ascontiguousarray(a_scales, np.float32),
                             np.ascontiguousarray(b_t), np.ascontiguousarray(w_scales, np.float32),
                             m, n, k, out, acc)
        return out, acc

    def gemm_i8_sampled(self, a_i8, b_t, n, k, idx):
        idx = np.ascontiguousarray(idx, np.int64)
        acc = np.empty(idx.size, np.int32)
        self.lib.pgo_gemm_i8_sampled(np.ascontiguousarray(a_i8), np.ascontiguousarray(b_t), n, k, idx, idx.size, acc)
        return acc

    def matmul_dequant_w8a32(self, a, m, k, w: QuantizedTensor):
        out = np.empty((m, w.cols), np.float32)
        self.lib.pgo_matmul_dequant_w8a32(np.ascontiguousarray(a, np.float32).reshape(-1), w.data_i8, w.scales,
                                          m, w.cols, k, out)
        return out

    # ---- src/gguf.rs --------------------------------------------------
    def f16_to_f32(self, bits: int) -> np.float32:
        return np.float32(self.lib.pgo_f16_to_f32(bits))

    def f16_to_f32_bits(self, bits: np.ndarray) -> np.ndarray:
        """f32 bit patterns (uint32) of an array of f16 bit patterns."""
        bits = np.ascontiguousarray(bits, np.uint16)
        out = np.empty(bits.size, np.uint32)
        self.lib.pgo_f16_to_f32_bits(bits, bits.size, out)
        return out

    def f32_to_f16(self, v: float) -> int:
        return int(self.lib.pgo_f32_to_f16(float(v)))

    def _dequant(self, fn, data, num_elements):
        data = np.ascontiguousarray(data, np.uint8).reshape(-1)
        out = np.empty(num_elements, np.float32)
        if fn(data, data.size, num_elements, out) != 0:
            raise AssertionError("block count / length check failed (reference asserts here)")
        return out

    def dequant_q8_0(self, data, num_elements):
        return self._dequant(self.lib.pgo_dequant_q8_0, data, num_elements)

    def dequant_q4_0(self, data, num_elements):
        return self._dequant(self.lib.pgo_dequant_q4_0, data, num_elements)

    def dequant_q4_1(self, data, num_elements):
        return self._dequant(self.lib.pgo_dequant_q4_1, data, num_elements)

    def dequant(self, kind: str, data, num_elements):
        return {"q8_0": self.dequant_q8_0, "q4_0": self.dequant_q4_0, "q4_1": self.dequant_q4_1}[kind](data, num_elements)

    # ---- src/tensor.rs:1342-1354 and the Llama linear on a GGUF weight ----
    def matmul_f32(self, a, b, m, k, n):
        out = np.empty((m, n), np.float32)
        self.lib.pgo_matmul_f32(np.ascontiguousarray(a, np.float32).reshape(-1),
                                np.ascontiguousarray(b, np.float32).reshape(-1), m, k, n, out)
        return out

    def gguf_matmul(self, x, m, k, raw, kind: str, n):
        """y[m,n] = sum_p x[m,p] * dequant(W)[n,p], f32, ascending p."""
        wd = self.dequant(kind, raw, n * k)
        out = np.empty((m, n), np.float32)
        self.lib.pgo_matmul_f32_wt(np.ascontiguousarray(x, np.float32).reshape(-1), wd, m, k, n, out)
        return out

    def gguf_matmul_f64(self, x, m, k, raw, kind: str, n):
        wd = self.dequant(kind, raw, n * k)
        out = np.empty((m, n), np.float64)
        self.lib.pgo_matmul_f64acc_wt(np.ascontiguousarray(x, np.float32).reshape(-1), wd, m, k, n, out)
        return out

    # ---- generators (no reference counterpart) ------------------------
    def encode(self, kind: str, w: np.ndarray) -> np.ndarray:
        w = np.ascontiguousarray(w, np.float32).reshape(-1)
        assert w.size % 32 == 0
        bs = {"q8_0": 34, "q4_0": 18, "q4_1": 20}[kind]
        out = np.empty(w.size // 32 * bs, np.uint8)
        getattr(self.lib, "pgo_encode_" + kind)(w, w.size, out)
        return out

    # ---- Huffman-coded int8 weights (src/huffman.rs) ------------------------------------------
    def huffman_from_frequencies(self, freqs):
        """HuffmanTable::from_frequencies -> (bit_lengths[256] u8, codes[256] u32)."""
        f = np.ascontiguousarray(freqs, np.uint64)
        assert f.size == 256
        bl, codes = np.zeros(256, np.uint8), np.zeros(256, np.uint32)
        self.lib.pgo_huffman_from_frequencies(f, bl, codes)
        return bl, codes

    def huffman_canonical_codes(self, bit_lengths):
        bl = np.ascontiguousarray(bit_lengths, np.uint8)
        codes = np.zeros(256, np.uint32)
        self.lib.pgo_huffman_canonical_codes(bl, codes)
        return codes

    def huffman_lut(self, bit_lengths, codes):
        """The 4096-entry decode table in the packing of to_gpu_lut: (bit_length << 8) | (symbol + 128)."""
        lut = np.zeros(4096, np.uint32)
        self.lib.pgo_huffman_build_lut(np.ascontiguousarray(bit_lengths, np.uint8), np.ascontiguousarray(codes, np.uint32), lut)
        return lut

    def huffman_encode(self, bit_lengths, codes, data):
        d = np.ascontiguousarray(data, np.int8).reshape(-1)
        bl = np.ascontiguousarray(bit_lengths, np.uint8)
        out = np.zeros(int(bl[(d.astype(np.int16) + 128)].astype(np.int64).sum() + 7) // 8 + 1, np.uint8)
        n = self.lib.pgo_huffman_encode(bl, np.ascontiguousarray(codes, np.uint32), d, d.size, out)
        return out[:n].copy()

    def huffman_decode(self, lut, bitstream, num_symbols):
        bs = np.ascontiguousarray(bitstream, np.uint8).reshape(-1)
        out = np.zeros(num_symbols, np.int8)
        self.lib.pgo_huffman_decode(np.ascontiguousarray(lut, np.uint32), bs if bs.size else np.zeros(1, np.uint8), bs.size, num_symbols, out)
        return out

