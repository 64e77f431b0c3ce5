"""The reference's GPU form of the quantised linear (quant::matmul_quantized_gpu -> matmul_dequant_i8 /
matmul_dequant_simd_i8, src/quant.rs:195-218, src/metal/shaders.rs:2329-2465): f32 activations times int8 weights
dequantised on the fly, on the CUDA kernels of csrc/pg_w8a32.cu, against the CPU restatement of that arithmetic."""
import numpy as np
import pytest

from _inputs import bits_equal, linear_inputs, normal, rng

pytestmark = pytest.mark.gpu


def _closed_form(m, k, n, mod):
    i = np.arange(m * k, dtype=np.int64)
    a = (((i * 7 + 3) % mod).astype(np.float32) / np.float32(mod) - np.float32(0.5)).astype(np.float32)
    j = np.arange(k * n, dtype=np.int64)
    w = (((j * 13 + 7) % mod).astype(np.float32) / np.float32(mod) - np.float32(0.5)).astype(np.float32)
    return a, w


def _run(pg, gpu, x, m, k, qt, sequential):
    qt.to_gpu(gpu)
    buf = pg.quant.matmul_quantized_gpu(gpu, x, m, k, qt, dequant=True, sequential=sequential)
    gpu.sync()                                   # the caller syncs (tests/quant_parity.rs:102-107)
    return buf.read().reshape(m, qt.cols)


def test_reference_metal_parity_test(gpu, oracle):
    """tests/quant_parity.rs:79-146: M 32, K 128, N 64, closed-form inputs; GPU W8A32 against the f32 product,
    rtol < 0.10 or diff < 0.02 -- on both forms of the CUDA kernel."""
    import peregrine_b200 as pg

    m, k, n = 32, 128, 64
    a, w = _closed_form(m, k, n, 200)
    expected = oracle.matmul_f32(a, w, m, k, n)
    ref = oracle.quantize_weights(w, k, n)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    for sequential in (True, False):
        got = _run(pg, gpu, a, m, k, qt, sequential)
        diff = np.abs(got - expected)
        rtol = diff / np.maximum(np.abs(expected), 1e-6)
        assert np.all((rtol < 0.10) | (diff < 0.02))
    qt.free_gpu()


@pytest.mark.parametrize("m,k,n", [(1, 4096, 1024), (8, 4096, 515), (16, 1024, 300), (3, 48, 7), (5, 100, 33), (33, 272, 19), (2, 16, 1)])
def test_w8a32_against_the_restatement(gpu, oracle_mt, m, k, n):
    """Sequential form: the same additions in the same order, bit for bit.  Streaming form: 1e-5 of max|C|, and no
    further from an f64 sum than the sequential f32 loop is."""
    import peregrine_b200 as pg

    x, w = linear_inputs(m, k, n, 900 + m + n, outliers=(k >= 1024))
    ref = oracle_mt.quantize_weights(w, k, n)
    want = oracle_mt.matmul_dequant_w8a32(x, m, k, ref)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    assert bits_equal(_run(pg, gpu, x, m, k, qt, True), want)
    got = _run(pg, gpu, x, m, k, qt, False)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-5 * scale
    exact = x.astype(np.float64) @ (ref.data_i8.astype(np.float32) * ref.scales[None, :]).astype(np.float64)
    assert np.abs(got - exact).max() <= max(1e-6 * scale, 2 * np.abs(want - exact).max())
    qt.free_gpu()


def test_w8a32_errors_and_empty(gpu, oracle):
    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    w = normal(rng(3), (64, 8), 0.02)
    qt = pg.quant.quantize_weights(w, 64, 8, gpu)
    with pytest.raises(AssertionError, match="weights not on GPU"):          # expect("weights not on GPU"), src/quant.rs:208-209
        pg.quant.matmul_quantized_gpu(gpu, np.zeros(128, np.float32), 2, 64, qt, dequant=True)
    qt.to_gpu(gpu)
    with pytest.raises(AssertionError):                                       # w.rows != k
        pg.quant.matmul_quantized_gpu(gpu, np.zeros(64, np.float32), 2, 32, qt, dequant=True)
    assert gpu.lib.pg_matmul_dequant_w8a32(gpu.handle, None, 0, 64, qt._gpu, None, 0) == 0     # no rows: nothing to do
    qt.free_gpu()
