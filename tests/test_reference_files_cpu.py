"""Model files written by the reference's own converters (scripts/convert_weights_int8.py, scripts/convert_huffman.py;
fixtures made by tests/golden/make_reference_files.py): the oracle's weight quantiser and its Huffman code, table,
encoder and decoder are held to those bytes, and the package's host-side readers parse them."""
import os
import struct

import numpy as np

from _inputs import bits_equal
from peregrine_b200.huffman import HuffmanTable, HuffmanTensor
from peregrine_b200.serial import load_model, load_typed_model, save_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
F32, INT8, HUFF = (os.path.join(GOLDEN, n) for n in ("reference_model_f32.bin", "reference_model_int8.bin", "reference_model_huffman.bin"))


def parse_int8_file(path):
    """A reader of the typed file that touches no GPU: {name: (shape, f32 data)} or {name: (rows, cols, i8, scales)}."""
    out, raw, pos = {}, open(path, "rb").read(), 4
    (count,) = struct.unpack_from("<I", raw, 0)
    for _ in range(count):
        (n,) = struct.unpack_from("<I", raw, pos)
        name = raw[pos + 4:pos + 4 + n].decode()
        pos += 4 + n
        dtype = raw[pos]
        (ndim,) = struct.unpack_from("<I", raw, pos + 1)
        shape = struct.unpack_from(f"<{ndim}I", raw, pos + 5)
        pos += 5 + 4 * ndim
        size = int(np.prod(shape))
        if dtype == 0:
            out[name] = (list(shape), np.frombuffer(raw, "<f4", size, pos).copy())
            pos += 4 * size
        else:
            assert dtype == 1 and ndim == 2
            q = np.frombuffer(raw, np.int8, size, pos).reshape(shape).copy()
            s = np.frombuffer(raw, "<f4", shape[1], pos + size).copy()
            out[name] = (shape[0], shape[1], q, s)
            pos += size + 4 * shape[1]
    assert pos == len(raw)
    return out


def test_f32_model_file_round_trip(tmp_path):
    model = load_model(F32)
    assert [(n, s) for n, s, _ in model] == [("layers.0.attn.weight", [24, 16]), ("layers.0.attn.bias", [16]), ("layers.0.mlp.weight", [16, 40]),
                                              ("norm.scale", [16]), ("head.weight", [40, 33])]
    save_model(model, str(tmp_path / "again.bin"))
    assert open(tmp_path / "again.bin", "rb").read() == open(F32, "rb").read()


def test_oracle_quantiser_matches_the_reference_converter(oracle):
    """quantize_weights (src/quant.rs:27-75) against scripts/convert_weights_int8.py:58-70 on the same tensors."""
    ref = parse_int8_file(INT8)
    seen = 0
    for name, shape, data in load_model(F32):
        if len(shape) == 2:
            rows, cols, q, s = ref[name]
            o = oracle.quantize_weights(data, rows, cols)
            assert np.array_equal(o.data_i8.reshape(rows, cols), q) and bits_equal(o.scales, s), name
            assert np.array_equal(o.data_i8_t.reshape(cols, rows), q.T), name
            seen += 1
        else:
            assert ref[name][0] == shape and bits_equal(ref[name][1], data)
    assert seen == 3


def test_oracle_huffman_matches_the_reference_converter(oracle):
    """The streams scripts/convert_huffman.py:161-237 wrote: the oracle's canonical codes, table and decoder read them
    back to the int8 tensors, and its encoder (and the package's) writes the same bytes from the same code book."""
    ref = parse_int8_file(INT8)
    records = load_typed_model(HUFF)            # Huffman records only: parsed on the host
    assert [n for n, _ in records] == ["layers.0.attn.weight", "layers.0.mlp.weight", "head.weight"]
    for name, ht in records:
        assert isinstance(ht, HuffmanTensor) and ht.num_streams == 4
        rows, cols, q, s = ref[name]
        assert (ht.rows, ht.cols) == (rows, cols) and bits_equal(ht.scales, s)
        flat = q.reshape(-1)
        chunk = (flat.size + 3) // 4
        assert ht.stream_lengths == [max(0, min(chunk, flat.size - i * chunk)) for i in range(4)]
        codes = oracle.huffman_canonical_codes(ht.table.bit_lengths)
        assert np.array_equal(codes, ht.table.codes)
        lut = oracle.huffman_lut(ht.table.bit_lengths, codes)
        at = 0
        for stream, n in zip(ht.streams, ht.stream_lengths):
            part = flat[at:at + n]
            assert np.array_equal(oracle.huffman_decode(lut, np.frombuffer(stream, np.uint8), n), part), name
            assert oracle.huffman_encode(ht.table.bit_lengths, codes, part).tobytes() == stream, name
            assert HuffmanTable.from_bytes(ht.table.to_bytes()).encode(part) == stream, name
            at += n
        assert at == flat.size
