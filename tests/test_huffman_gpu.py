"""Huffman-coded int8 weights through the GPU decoder: the reference's tests (src/huffman.rs:755-829,
tests/huffman_parity.rs:23-43, 104-134) and the decoder against the C oracle, bit for bit, on codes and stream
layouts that exercise every path of the parallel decode."""
import io

import numpy as np
import pytest

from _inputs import bits_equal, lcg, rng
from test_huffman_cpu import histogram, random_i8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def oracle_decode(oracle, table, stream, n):
    return oracle.huffman_decode(oracle.huffman_lut(table.bit_lengths, table.codes), np.frombuffer(bytes(stream), np.uint8), n)


# ---- the reference's own tests --------------------------------------------------------------------
def test_encode_decode_roundtrip(pg, gpu):
    data = random_i8(1024, 42)
    t = pg.huffman.HuffmanTable.from_frequencies(histogram(data))
    assert np.array_equal(t.decode(t.encode(data), data.size, gpu), data)


def test_empty_input(pg, gpu):
    t = pg.huffman.HuffmanTable.from_frequencies(np.zeros(256, np.uint64))
    assert t.decode(t.encode(np.zeros(0, np.int8)), 0, gpu).size == 0


def test_all_same_symbol(pg, gpu):
    data = np.full(512, 42, np.int8)
    t = pg.huffman.HuffmanTable.from_frequencies(histogram(data))
    enc = t.encode(data)
    assert len(enc) <= 65 and np.array_equal(t.decode(enc, data.size, gpu), data)


def test_huffman_tensor_roundtrip(pg, gpu):
    rows, cols = 64, 32
    data = np.array([((i * 7 + 3) % 200) / 200.0 - 0.5 for i in range(rows * cols)], np.float32)
    qt = pg.quant.quantize_weights(data, rows, cols, gpu)
    qt2 = pg.huffman.HuffmanTensor.from_quantized(qt, 4).decode_to_quantized(gpu)
    assert np.array_equal(qt2.data_i8, qt.data_i8) and bits_equal(qt2.scales, qt.scales)
    assert np.array_equal(qt2.data_i8_t, qt.data_i8_t) and (qt2.rows, qt2.cols) == (rows, cols)


@pytest.mark.parametrize("m,k,n", [(8, 32, 16), (1, 64, 1), (32, 128, 64), (16, 256, 32)])
def test_huffman_vs_quantized_matmul_parity(pg, gpu, oracle, m, k, n):
    """tests/huffman_parity.rs:23-43; here the two products are equal bit for bit, and equal to the oracle's."""
    a, w = lcg(m * k, 42), lcg(k * n, 123)
    qt = pg.quant.quantize_weights(w, k, n, gpu)
    ht = pg.huffman.HuffmanTensor.from_quantized(qt, 4)
    quant = pg.quant.matmul_quantized(a, m, k, qt, gpu)
    huff = pg.huffman.matmul_huffman(a, m, k, ht, gpu)
    assert bits_equal(quant, huff)
    assert bits_equal(huff, oracle.matmul_quantized(a, m, k, oracle.quantize_weights(w, k, n)))


def test_huffman_serialization_roundtrip(pg, gpu):
    """tests/huffman_parity.rs:104-134"""
    rows, cols = 32, 64
    qt = pg.quant.quantize_weights(lcg(rows * cols, 77), rows, cols, gpu)
    ht = pg.huffman.HuffmanTensor.from_quantized(qt, 4)
    buf = io.BytesIO()
    pg.serial.write_huffman_tensor(buf, "test.huffman", ht)
    buf.seek(0)
    name, ht2 = pg.serial.read_huffman_tensor(buf)
    assert name == "test.huffman" and (ht2.rows, ht2.cols, ht2.num_streams) == (rows, cols, 4)
    assert bits_equal(ht2.scales, ht.scales) and ht2.stream_lengths == ht.stream_lengths
    assert np.array_equal(ht.decode_to_quantized(gpu).data_i8, ht2.decode_to_quantized(gpu).data_i8)
    assert np.array_equal(ht2.decode_to_quantized(gpu).data_i8, qt.data_i8)


# ---- the parallel decoder against the oracle ---------------------------------------------------------
def _sources():
    g = rng(5)
    yield "gaussian", lambda n: (g.standard_normal(n) * 10).clip(-127, 127).astype(np.int8)
    yield "narrow", lambda n: (g.standard_normal(n) * 1.2).clip(-127, 127).astype(np.int8)      # code words of 1-2 bits dominate
    yield "flat", lambda n: g.integers(-128, 128, n).astype(np.int8)                            # every code word 8 bits
    yield "two", lambda n: g.integers(0, 2, n).astype(np.int8)                                  # 1-bit code words: 2048 symbols per subsequence
    yield "skewed", lambda n: np.where(g.random(n) < 0.97, 0, g.integers(-128, 128, n)).astype(np.int8)   # 12-bit code words


@pytest.mark.parametrize("n", [1, 5, 255, 256, 257, 4096, 300_001, 5_000_000])
def test_decode_matches_oracle(pg, gpu, oracle, n):
    """One stream; the sizes straddle one subsequence (256 bytes), one block (128 subsequences) and many blocks."""
    for name, make in _sources():
        data = make(n)
        t = pg.huffman.HuffmanTable.from_frequencies(histogram(data), limit_lengths=True)   # a few million Gaussian values: deeper than 12
        enc = t.encode(data)
        got = t.decode(enc, n, gpu)
        assert np.array_equal(got, oracle_decode(oracle, t, enc, n)), name
        assert np.array_equal(got, data), name


@pytest.mark.parametrize("rows,cols,streams", [(64, 48, 1), (64, 48, 4), (333, 77, 7), (1000, 1024, 4), (1000, 1024, 1000), (3, 5, 64),
                                               (2048, 4096, 4)])
def test_tensor_decode_matches_oracle(pg, gpu, oracle, rows, cols, streams):
    """Streams of ragged sizes at odd byte offsets, empty streams, more streams than blocks."""
    g = rng(rows + cols + streams)
    q = (g.standard_normal((rows, cols)) * 14).clip(-127, 127).astype(np.int8)
    s = (g.random(cols, dtype=np.float32) + np.float32(0.01)).astype(np.float32)
    qt = pg.quant.QuantizedTensor(q, np.ascontiguousarray(q.T), s, rows, cols)
    ht = pg.huffman.HuffmanTensor.from_quantized(qt, streams, limit_lengths=True)
    want = np.concatenate([oracle_decode(oracle, ht.table, st, n) for st, n in zip(ht.streams, ht.stream_lengths)])
    assert np.array_equal(want, q.reshape(-1))
    back = ht.decode_to_quantized(gpu)
    assert np.array_equal(back.data_i8, q) and np.array_equal(back.data_i8_t, q.T) and bits_equal(back.scales, s)


def test_codes_the_reference_decodes_oddly(pg, gpu, oracle):
    """What a damaged or hand-made code book does in the reference's sequential loop, bit for bit: a window no code
    starts with yields value 0 and leaves the cursor where it is; a stream that ends early is read on as zeros."""
    HuffmanTable = pg.huffman.HuffmanTable
    lengths = np.zeros(256, np.uint8)
    lengths[128 + 5], lengths[128 + 9] = 1, 3                         # codes 0 and 100: windows 101, 11x start no code
    t = HuffmanTable(lengths)
    g = rng(3)
    for n, nbytes in ((40, 8), (5000, 700), (100_000, 9000)):
        stream = g.integers(0, 256, nbytes).astype(np.uint8).tobytes()
        assert np.array_equal(t.decode(stream, n, gpu), oracle_decode(oracle, t, stream, n))
    data = (g.standard_normal(20_000) * 6).clip(-127, 127).astype(np.int8)
    t = HuffmanTable.from_frequencies(histogram(data), limit_lengths=True)
    enc = t.encode(data)
    short = enc[:len(enc) // 2]
    assert np.array_equal(t.decode(short, data.size, gpu), oracle_decode(oracle, t, short, data.size))
    assert np.array_equal(t.decode(b"", 100, gpu), oracle_decode(oracle, t, b"", 100))
    # more bytes than the symbols need: the rest is ignored
    long = enc + bytes(g.integers(0, 256, 999).astype(np.uint8))
    assert np.array_equal(t.decode(long, data.size, gpu), data)


def test_deep_tree_panics_like_the_reference(pg):
    """A histogram whose Huffman tree is deeper than 12: the reference cuts the depths and then indexes past its
    4096-entry table (src/huffman.rs:135-141, 193-213)."""
    f = np.zeros(256, np.uint64)
    f[:40] = [2 ** i for i in range(40)]
    with pytest.raises(pg.huffman.HuffmanPanic, match="index out of bounds"):
        pg.huffman.HuffmanTable.from_frequencies(f)


def test_symbol_count_is_checked(pg, gpu):
    q = np.zeros((4, 4), np.int8)
    ht = pg.huffman.HuffmanTensor.from_quantized(pg.quant.QuantizedTensor(q, q.T.copy(), np.ones(4, np.float32), 4, 4), 2)
    ht.stream_lengths[1] -= 1
    with pytest.raises(pg.huffman.HuffmanPanic, match="symbols"):
        ht.to_gpu(gpu)
    from peregrine_b200 import _lib
    import ctypes as C
    lens, sizes = np.array([8, 7], np.uint64), np.array([len(s) for s in ht.streams], np.uint64)
    packed = np.frombuffer(b"".join(ht.streams), np.uint8)
    h = C.c_void_p()
    rc = gpu.lib.pg_qtensor_from_huffman(gpu.handle, ht.table.bit_lengths.ctypes.data, 2, lens.ctypes.data, sizes.ctypes.data,
                                         packed.ctypes.data, ht.scales.ctypes.data, 4, 4, C.byref(h))
    assert rc == _lib.PG_ERR_INVALID and not h.value


def test_random_tensors_and_damaged_streams(pg, gpu, oracle):
    """80 seeded random tensors (five symbol distributions, 1 to 300 streams): the decode gives the source back, and a
    damaged, shortened copy of the first stream decodes to what the oracle's sequential loop makes of it."""
    g = rng(77)
    for _ in range(80):
        rows, cols = int(g.choice([1, 3, 16, 100, 333, 1024])), int(g.choice([1, 5, 32, 77, 256, 1000]))
        kind = int(g.integers(0, 5))
        if kind == 0:
            q = (g.standard_normal((rows, cols)) * g.choice([0.5, 3, 12, 40])).clip(-127, 127).astype(np.int8)
        elif kind == 1:
            q = g.integers(-128, 128, (rows, cols)).astype(np.int8)
        elif kind == 2:
            q = g.integers(0, int(g.choice([1, 2, 3, 5, 17])), (rows, cols)).astype(np.int8)
        elif kind == 3:
            q = np.where(g.random((rows, cols)) < 0.95, 7, g.integers(-128, 128, (rows, cols))).astype(np.int8)
        else:
            q = (g.geometric(0.3, (rows, cols)) % 120).astype(np.int8)
        qt = pg.quant.QuantizedTensor(q, np.ascontiguousarray(q.T), g.random(cols, dtype=np.float32), rows, cols)
        ht = pg.huffman.HuffmanTensor.from_quantized(qt, int(g.choice([1, 2, 4, 7, 64, 300])), limit_lengths=True)
        back = ht.decode_to_quantized(gpu)
        assert np.array_equal(back.data_i8, q) and np.array_equal(back.data_i8_t, q.T), (rows, cols, kind)
        back.free_gpu()
        if len(ht.streams[0]) > 4:
            bad = bytearray(ht.streams[0])
            for _ in range(3):
                bad[int(g.integers(0, len(bad)))] ^= int(g.integers(1, 256))
            bad = bytes(bad[:max(1, len(bad) - int(g.integers(0, 3)))])
            n0 = ht.stream_lengths[0]
            assert np.array_equal(ht.table.decode(bad, n0, gpu), oracle_decode(oracle, ht.table, bad, n0)), (rows, cols, kind)
