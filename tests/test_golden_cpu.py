"""The committed golden fixtures against the CPU oracle: both oracle builds must reproduce them bit for bit
(tests/golden/make_golden.py wrote them from the one-thread build)."""
import os

import numpy as np
import pytest

from _inputs import bits_equal, lcg, linear_inputs, normal, rng
from golden.make_golden import GGUF_CASES, LCG_CASES, W8A8_CASES

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "peregrine_quant_path.npz"))


@pytest.mark.parametrize("which", ["oracle", "oracle_mt"])
def test_oracle_reproduces_golden(which, request):
    orc = request.getfixturevalue(which)
    for m, k, n, seed in W8A8_CASES:
        x, w = linear_inputs(m, k, n, seed, outliers=True)
        qt = orc.quantize_weights(w, k, n)
        y, acc, q, s = orc.matmul_quantized(x, m, k, qt, return_parts=True)
        tag = f"w8a8_{m}_{k}_{n}"
        assert np.array_equal(qt.data_i8_t, GOLD[tag + "_wq_t"]) and bits_equal(qt.scales, GOLD[tag + "_ws"])
        assert np.array_equal(q, GOLD[tag + "_aq"]) and bits_equal(s, GOLD[tag + "_as"])
        assert np.array_equal(acc, GOLD[tag + "_acc"]) and bits_equal(y, GOLD[tag + "_y"])
    for m, k, n in LCG_CASES:
        a, w = lcg(m * k, 42), lcg(k * n, 123)
        qt = orc.quantize_weights(w, k, n)
        y, acc, _, _ = orc.matmul_quantized(a, m, k, qt, return_parts=True)
        tag = f"lcg_{m}_{k}_{n}"
        assert np.array_equal(acc, GOLD[tag + "_acc"]) and bits_equal(y, GOLD[tag + "_y"]) and bits_equal(qt.scales, GOLD[tag + "_ws"])
    for kind, n, k, m, seed in GGUF_CASES:
        g = rng(seed)
        w = normal(g, (n, k), 0.02)
        x = normal(g, (m, k))
        tag = f"gguf_{kind}_{n}_{k}_{m}"
        raw = orc.encode(kind, w)
        assert np.array_equal(raw, GOLD[tag + "_raw"])
        assert bits_equal(getattr(orc, "dequant_" + kind)(raw, n * k), GOLD[tag + "_deq"])
        assert bits_equal(orc.gguf_matmul(x, m, k, raw, kind, n), GOLD[tag + "_y"])
    assert np.array_equal(orc.f16_to_f32_bits(GOLD["f16_bits"]), GOLD["f16_as_f32_bits"])
