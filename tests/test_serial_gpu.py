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
