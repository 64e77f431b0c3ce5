"""The quantised serial format through the GPU: the reference's round-trip test (tests/quant_parity.rs:148-173), the
device-built transposed layout, and a product from a tensor that was read back."""
import io

import numpy as np
import pytest

from _inputs import bits_equal, linear_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def test_reference_roundtrip(pg, gpu):
    """tests/quant_parity.rs:148-173"""
    rows, cols = 16, 32
    data = np.array([((i * 11 + 3) % 100) / 50.0 - 1.0 for i in range(rows * cols)], np.float32)
    qt = pg.quant.quantize_weights(data, rows, cols, gpu)
    buf = io.BytesIO()
    pg.serial.write_quantized_tensor(buf, "test.weight", qt)
    buf.seek(0)
    name, qt2 = pg.serial.read_quantized_tensor(buf, gpu)
    assert name == "test.weight" and qt2.rows == rows and qt2.cols == cols
    assert np.array_equal(qt2.data_i8.reshape(-1), qt.data_i8.reshape(-1)) and bits_equal(qt2.scales, qt.scales)
    assert np.array_equal(qt2.data_i8_t.reshape(cols, rows), qt.data_i8.reshape(rows, cols).T)


@pytest.mark.parametrize("m,k,n", [(4, 256, 40), (16, 1000, 333), (3, 64, 1), (70, 130, 65)])
def test_product_from_a_tensor_read_back(pg, gpu, oracle_mt, m, k, n):
    """Several tensors in one stream; the transposed layout is rebuilt on the device (tile edges in both directions) and
    the product from it equals the oracle's on the original tensor, bit for bit."""
    x, w = linear_inputs(m, k, n, 40 + m + n)
    ref = oracle_mt.quantize_weights(w, k, n)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    buf = io.BytesIO()
    pg.serial.write_quantized_tensor(buf, "first", qt)
    pg.serial.write_quantized_tensor(buf, "second.bias", qt)
    buf.seek(0)
    name1, a = pg.serial.read_quantized_tensor(buf, gpu)
    name2, b = pg.serial.read_quantized_tensor(buf, gpu)
    assert (name1, name2) == ("first", "second.bias") and a.on_gpu and b.on_gpu
    assert np.array_equal(a.data_i8_t.reshape(n, k), ref.data_i8_t.reshape(n, k))
    out_o = oracle_mt.matmul_quantized(x, m, k, ref)
    assert bits_equal(pg.quant.matmul_quantized(x, m, k, b, gpu), out_o)
    a.free_gpu()
    b.free_gpu()


def test_convert_huffman_from_a_mixed_typed_file(pg, gpu, oracle_mt, tmp_path):
    """A typed file as scripts/convert_weights_int8.py writes it, with an f32 scalar first, an f32 matrix (a 2-D tensor
    whose name has no ".weight": the int8 converter leaves it f32), an i8 record and an f32 vector: the Huffman file must
    hold the i8 tensor as it is and the f32 matrix quantised per column, and leave the scalar and the vector out."""
    import struct

    g = np.random.Generator(np.random.PCG64(77))
    k, n = 48, 40
    w_i8 = (g.standard_normal((k, n)) * 0.05).astype(np.float32)
    w_f32 = (g.standard_normal((24, 16)) * 0.05).astype(np.float32)
    ref_i8 = oracle_mt.quantize_weights(w_i8, k, n)
    ref_f32 = oracle_mt.quantize_weights(w_f32, 24, 16)

    def f32_record(name, shape, data):
        nb = name.encode()
        return (struct.pack("<I", len(nb)) + nb + b"\x00" + struct.pack("<I", len(shape)) + struct.pack(f"<{len(shape)}I", *shape) +
                np.asarray(data, "<f4").tobytes())

    src = tmp_path / "mixed.bin"
    with open(src, "wb") as f:
        f.write(struct.pack("<I", 4))
        f.write(f32_record("step", [], [3.0]))
        f.write(f32_record("proj.kernel", [24, 16], w_f32))
        pg.serial.write_quantized_tensor(f, "blk.weight", pg.quant.QuantizedTensor(ref_i8.data_i8, ref_i8.data_i8_t, ref_i8.scales, k, n))
        f.write(f32_record("blk.bias", [n], np.zeros(n)))
    assert pg.serial.file_kind(str(src)) == "typed"
    out = tmp_path / "mixed_huff.bin"
    pg.serial.convert_huffman(str(src), str(out), 3, limit_lengths=True, gpu=gpu)
    got = pg.serial.load_typed_model(str(out), gpu)
    assert [name for name, _ in got] == ["proj.kernel", "blk.weight"]
    for (name, ht), ref in zip(got, (ref_f32, ref_i8)):
        qt = ht.decode_to_quantized(gpu)
        assert np.array_equal(np.asarray(qt.data_i8).reshape(-1), ref.data_i8.reshape(-1)), name
        assert bits_equal(qt.scales, ref.scales), name
