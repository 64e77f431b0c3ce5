"""Huffman-coded int8 weights on the host: the C oracle (oracle/huffman_oracle.c) against the reference's own tests
(src/huffman.rs:740-847, tests/huffman_parity.rs), and the package's table builder and encoder against the oracle."""
import io
import struct

import numpy as np
import pytest

from _inputs import lcg, rng
from peregrine_b200.huffman import HuffmanPanic, HuffmanTable, HuffmanTensor
from peregrine_b200.quant import QuantizedTensor
from peregrine_b200.serial import SerialPanic, read_huffman_tensor, write_huffman_tensor


def random_i8(n, seed):
    """The biased LCG bytes of src/huffman.rs:743-754 (i32 remainder and i8 division truncate toward zero)."""
    out = np.empty(n, np.int8)
    state = seed
    for i in range(n):
        state = (state * 1103515245 + 12345) & 0xFFFFFFFF
        raw = (state >> 16) % 256 - 128
        out[i] = raw if (state >> 8) % 4 == 0 else int(raw / 4)
    return out


def histogram(d):
    return np.bincount(np.asarray(d, np.int8).astype(np.int16) + 128, minlength=256).astype(np.uint64)


def oracle_roundtrip(oracle, data):
    bl, codes = oracle.huffman_from_frequencies(histogram(data))
    enc = oracle.huffman_encode(bl, codes, data)
    return bl, codes, enc, oracle.huffman_decode(oracle.huffman_lut(bl, codes), enc, len(data))


# ---- the reference's own tests, run on the oracle ------------------------------------------------
def test_encode_decode_roundtrip(oracle):
    data = random_i8(1024, 42)
    _, _, _, dec = oracle_roundtrip(oracle, data)
    assert np.array_equal(dec, data)


def test_empty_input(oracle):
    bl, codes = oracle.huffman_from_frequencies(np.zeros(256, np.uint64))
    assert not bl.any() and not codes.any()
    assert oracle.huffman_encode(bl, codes, np.zeros(0, np.int8)).size == 0
    assert oracle.huffman_decode(oracle.huffman_lut(bl, codes), np.zeros(0, np.uint8), 0).size == 0


def test_all_same_symbol(oracle):
    data = np.full(512, 42, np.int8)
    bl, _, enc, dec = oracle_roundtrip(oracle, data)
    assert np.array_equal(dec, data)
    assert bl[42 + 128] == 1 and enc.size == 64          # the reference asserts <= 65 bytes


def test_table_correctness(oracle):
    f = np.zeros(256, np.uint64)
    f[128], f[129] = 100, 50
    bl, codes = oracle.huffman_from_frequencies(f)
    assert 0 < bl[128] <= bl[129] and bl[129] > 0
    assert (bl[128], bl[129], codes[128], codes[129]) == (1, 1, 0, 1)


def test_known_code(oracle):
    """Frequencies 1,1,2,4 -> depths 3,3,2,1; canonical codes by (length, symbol)."""
    f = np.zeros(256, np.uint64)
    f[10], f[20], f[30], f[40] = 1, 1, 2, 4
    bl, codes = oracle.huffman_from_frequencies(f)
    assert [int(bl[i]) for i in (10, 20, 30, 40)] == [3, 3, 2, 1]
    assert [int(codes[i]) for i in (10, 20, 30, 40)] == [0b110, 0b111, 0b10, 0b0]
    enc = oracle.huffman_encode(bl, codes, np.array([40 - 128, 30 - 128, 10 - 128, 20 - 128], np.int8))
    assert enc.tobytes() == bytes([0b01011011, 0b10000000])   # 0 | 10 | 110 | 111, then padding


# ---- the package's host side against the oracle --------------------------------------------------
def histograms():
    g = rng(7)
    yield histogram(random_i8(4096, 1))
    yield histogram((g.standard_normal(20000) * 12).clip(-127, 127).astype(np.int8))
    yield histogram(g.integers(-128, 128, 50000).astype(np.int8))               # flat: every code 8 bits
    f = np.zeros(256, np.uint64)
    f[:40] = [2 ** i for i in range(40)]                                        # a chain deeper than 12: lengths are cut
    yield f
    f = np.zeros(256, np.uint64)
    f[200] = 9
    yield f
    yield np.zeros(256, np.uint64)
    f = g.integers(0, 5, 256).astype(np.uint64)                                 # many ties
    yield f
    yield np.full(256, 1, np.uint64)


def kraft(bl):
    return sum(2.0 ** -int(b) for b in bl if b)


def test_table_builder_matches_oracle(oracle):
    for f in histograms():
        bl, codes = oracle.huffman_from_frequencies(f)
        if kraft(bl) > 1.0:          # depths cut to 12 over-subscribe the reference's table: a panic there, and here
            with pytest.raises(HuffmanPanic, match="index out of bounds"):
                HuffmanTable.from_frequencies(f)
            continue
        t = HuffmanTable.from_frequencies(f)
        assert np.array_equal(t.bit_lengths, bl)
        assert np.array_equal(t.codes, codes)
        assert np.array_equal(HuffmanTable.from_bytes(t.to_bytes()).codes, codes)
        assert np.array_equal(t.to_gpu_lut(), oracle.huffman_lut(bl, codes))


def test_limited_lengths_make_a_code_the_reference_reads(oracle):
    """limit_lengths=True (not in the reference): a complete prefix code of at most 12 bits, written as an ordinary
    code book, that the oracle's from_bytes path (canonical_codes + build_decode_lut + decode) round-trips."""
    g = rng(21)
    cases = [np.array([2 ** i for i in range(40)] + [0] * 216, np.uint64),
             histogram((g.standard_normal(3_000_000) * 11).clip(-127, 127).astype(np.int8)),
             histogram(random_i8(4096, 1))]
    for f in cases:
        t = HuffmanTable.from_frequencies(f, limit_lengths=True)
        active = f > 0
        assert np.all(t.bit_lengths[active] >= 1) and np.all(t.bit_lengths[~active] == 0) and int(t.bit_lengths.max()) <= 12
        assert kraft(t.bit_lengths) == 1.0
        codes = oracle.huffman_canonical_codes(t.bit_lengths)
        assert np.array_equal(codes, t.codes)
        data = np.repeat(np.arange(-128, 128)[active], 3).astype(np.int8)
        g.shuffle(data)
        enc = np.frombuffer(t.encode(data), np.uint8)
        assert np.array_equal(oracle.huffman_decode(oracle.huffman_lut(t.bit_lengths, codes), enc, data.size), data)
    # where the reference's own lengths fit, nothing changes
    f = histogram(random_i8(4096, 1))
    assert np.array_equal(HuffmanTable.from_frequencies(f, True).bit_lengths, HuffmanTable.from_frequencies(f).bit_lengths)


def test_encoder_matches_oracle(oracle):
    g = rng(11)
    for n in (1, 7, 8, 1000, 70001):
        data = (g.standard_normal(n) * 9).clip(-127, 127).astype(np.int8)
        t = HuffmanTable.from_frequencies(histogram(data), limit_lengths=True)
        assert t.encode(data) == oracle.huffman_encode(t.bit_lengths, t.codes, data).tobytes()
    assert HuffmanTable.from_frequencies(np.zeros(256, np.uint64)).encode(np.zeros(0, np.int8)) == b""


def _weights(oracle, rows, cols, seed):
    o = oracle.quantize_weights(lcg(rows * cols, seed), rows, cols)
    return QuantizedTensor(o.data_i8, o.data_i8_t, o.scales, rows, cols)


def test_huffman_tensor_streams(oracle):
    """from_quantized (src/huffman.rs:332-371): equal chunks of the row-major bytes, empty streams past the end."""
    qt = _weights(oracle, 5, 3, 3)                      # 15 bytes in 4 streams: 4 + 4 + 4 + 3
    ht = HuffmanTensor.from_quantized(qt, 4)
    assert ht.stream_lengths == [4, 4, 4, 3] and ht.num_streams == 4
    flat = qt.data_i8.reshape(-1)
    lut = oracle.huffman_lut(ht.table.bit_lengths, ht.table.codes)
    got = np.concatenate([oracle.huffman_decode(lut, np.frombuffer(s, np.uint8), n) for s, n in zip(ht.streams, ht.stream_lengths)])
    assert np.array_equal(got, flat)
    ht = HuffmanTensor.from_quantized(_weights(oracle, 1, 2, 4), 4)          # 2 bytes in 4 streams: 1 + 1 + 0 + 0
    assert ht.stream_lengths == [1, 1, 0, 0] and ht.streams[2] == b"" and ht.streams[3] == b""
    assert HuffmanTensor.from_quantized(qt, 0).num_streams == 1


def test_huffman_tensor_compression(oracle):
    """src/huffman.rs:831-847"""
    rows = cols = 256
    data = np.array([((i * 7 + 3) % 200) / 200.0 - 0.5 for i in range(rows * cols)], np.float32)
    o = oracle.quantize_weights(data, rows, cols)
    ht = HuffmanTensor.from_quantized(QuantizedTensor(o.data_i8, o.data_i8_t, o.scales, rows, cols), 4)
    assert ht.uncompressed_size() == rows * cols + cols * 4
    assert ht.compressed_size() == sum(len(x) for x in ht.streams) + 256 + cols * 4
    assert ht.compression_ratio() > 1.0


def test_serial_record_layout_and_roundtrip(oracle):
    """tests/huffman_parity.rs:104-134 without the decode (that part needs the GPU)."""
    qt = _weights(oracle, 32, 64, 77)
    ht = HuffmanTensor.from_quantized(qt, 4)
    buf = io.BytesIO()
    write_huffman_tensor(buf, "test.huffman", ht)
    raw = buf.getvalue()
    head = struct.pack("<I", 12) + b"test.huffman" + b"\x03" + struct.pack("<III", 2, 32, 64) + ht.table.to_bytes() + struct.pack("<I", 4)
    assert raw.startswith(head)
    assert raw[len(head):len(head) + 32] == struct.pack("<4I", *ht.stream_lengths) + struct.pack("<4I", *[len(s) for s in ht.streams])
    assert raw.endswith(qt.scales.tobytes()) and len(raw) == len(head) + 32 + sum(len(s) for s in ht.streams) + 64 * 4
    name, ht2 = read_huffman_tensor(io.BytesIO(raw))
    assert name == "test.huffman" and (ht2.rows, ht2.cols, ht2.num_streams) == (32, 64, 4)
    assert np.array_equal(ht2.scales.view(np.uint32), ht.scales.view(np.uint32))
    assert ht2.stream_lengths == ht.stream_lengths and ht2.streams == ht.streams
    assert np.array_equal(ht2.table.codes, ht.table.codes)
    with pytest.raises(SerialPanic, match="expected dtype=3"):
        read_huffman_tensor(io.BytesIO(raw[:16] + b"\x01" + raw[17:]))
    with pytest.raises(ValueError, match="failed to fill whole buffer"):
        read_huffman_tensor(io.BytesIO(raw[:-1]))
