"""The CUDA path against the committed golden fixtures alone (no oracle in the loop): bit-exact for the int8 path and the
block decoders, 1e-5 of max|y| for the GGUF product."""
import os

import numpy as np
import pytest

from _inputs import bits_equal, lcg, linear_inputs, normal, rng

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = np.load(os.path.join(HERE, "golden", "peregrine_quant_path.npz"))
# the case lists of tests/golden/make_golden.py, repeated here so that this file does not import the oracle
W8A8_CASES = [(1, 64, 8, 3), (8, 32, 16, 4), (16, 256, 40, 5), (5, 1040, 33, 6), (64, 192, 24, 7), (130, 144, 72, 8)]
LCG_CASES = [(8, 32, 16), (1, 64, 1), (32, 128, 64), (16, 256, 32)]
GGUF_CASES = [("q8_0", 24, 256, 3, 9), ("q4_0", 24, 256, 3, 10), ("q4_1", 16, 128, 2, 11), ("q4_0", 40, 512, 9, 12)]


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def test_w8a8_path_matches_golden(pg, gpu):
    for m, k, n, seed in W8A8_CASES:
        x, w = linear_inputs(m, k, n, seed, outliers=True)
        tag = f"w8a8_{m}_{k}_{n}"
        qt = pg.quant.quantize_weights(w, k, n, gpu)
        assert np.array_equal(qt.data_i8_t.reshape(n, k), GOLD[tag + "_wq_t"].reshape(n, k)) and bits_equal(qt.scales, GOLD[tag + "_ws"])
        for algo in (0, 1, 2, 3, 4):                              # automatic, checker, both streaming kernels, tcgen05
            if algo == 4 and not (m <= 16 and k % 64 == 0):
                continue
            if algo == 2 and not (m <= 64 and k % 16 == 0):
                continue
            y, acc, q, s = pg.quant.matmul_quantized_parts(gpu, x, m, k, qt, algo)
            assert np.array_equal(q.reshape(m, k), GOLD[tag + "_aq"].reshape(m, k)) and bits_equal(s, GOLD[tag + "_as"]), (tag, algo)
            assert np.array_equal(acc.reshape(m, n), GOLD[tag + "_acc"].reshape(m, n)), (tag, algo)
            assert bits_equal(y.reshape(m, n), GOLD[tag + "_y"].reshape(m, n)), (tag, algo)
        qt.free_gpu()
    for m, k, n in LCG_CASES:
        a, w = lcg(m * k, 42), lcg(k * n, 123)
        tag = f"lcg_{m}_{k}_{n}"
        qt = pg.quant.quantize_weights(w, k, n, gpu)
        y, acc, _, _ = pg.quant.matmul_quantized_parts(gpu, a, m, k, qt)
        assert bits_equal(qt.scales, GOLD[tag + "_ws"]) and np.array_equal(acc.reshape(-1), GOLD[tag + "_acc"].reshape(-1))
        assert bits_equal(y.reshape(-1), GOLD[tag + "_y"].reshape(-1))
    assert gpu.device_status() == 0


def test_gguf_path_matches_golden(pg, gpu):
    for kind, n, k, m, seed in GGUF_CASES:
        g = rng(seed)
        normal(g, (n, k), 0.02)                                   # the weights: only their encoding (in the fixture) is needed
        x = normal(g, (m, k))
        tag = f"gguf_{kind}_{n}_{k}_{m}"
        raw = GOLD[tag + "_raw"]
        deq = getattr(pg.gguf, "dequant_" + kind)(raw, n * k, gpu)
        assert bits_equal(deq, GOLD[tag + "_deq"]), tag
        y = pg.gguf.GgufWeight(kind, raw, n, k, gpu).matmul(x, m)
        ref = GOLD[tag + "_y"].reshape(m, n)
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max(), tag
    got = pg.gguf.f16_to_f32(GOLD["f16_bits"], gpu)
    ref = GOLD["f16_as_f32_bits"].view(np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan) and bits_equal(got[~nan], ref[~nan])
