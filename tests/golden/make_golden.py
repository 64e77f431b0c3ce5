"""Writes the golden fixtures of this folder from the CPU oracle (the one-thread, reference-equivalent build).

    python tests/golden/make_golden.py

Inputs are regenerated from their seeds by the tests, so the files hold OUTPUTS only: what the reference's scalar code
produces for them (the oracle restates that code and is pinned against the reference's own known-answer tests).
The fixtures let the GPU tests compare with fixed bytes even where the oracle cannot be built, and catch an oracle
whose results drift with compiler or flags."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from _inputs import lcg, linear_inputs, normal, rng  # noqa: E402
from oracle.pgoracle import Oracle  # noqa: E402

W8A8_CASES = [(1, 64, 8, 3), (8, 32, 16, 4), (16, 256, 40, 5), (5, 1040, 33, 6), (64, 192, 24, 7), (130, 144, 72, 8)]   # m, k, n, seed
LCG_CASES = [(8, 32, 16), (1, 64, 1), (32, 128, 64), (16, 256, 32)]                                                       # tests/huffman_parity.rs:23-41
GGUF_CASES = [("q8_0", 24, 256, 3, 9), ("q4_0", 24, 256, 3, 10), ("q4_1", 16, 128, 2, 11), ("q4_0", 40, 512, 9, 12)]      # kind, n, k, m, seed


def main() -> None:
    orc = Oracle(mt=False)
    out = {}
    for m, k, n, seed in W8A8_CASES:
        x, w = linear_inputs(m, k, n, seed, outliers=True)
        qt = orc.quantize_weights(w, k, n)
        y, acc, q, s = orc.matmul_quantized(x, m, k, qt, return_parts=True)
        tag = f"w8a8_{m}_{k}_{n}"
        out[tag + "_wq_t"], out[tag + "_ws"], out[tag + "_aq"], out[tag + "_as"] = qt.data_i8_t, qt.scales, q, s
        out[tag + "_acc"], out[tag + "_y"] = acc, y
    for m, k, n in LCG_CASES:
        a, w = lcg(m * k, 42), lcg(k * n, 123)
        qt = orc.quantize_weights(w, k, n)
        y, acc, q, s = orc.matmul_quantized(a, m, k, qt, return_parts=True)
        tag = f"lcg_{m}_{k}_{n}"
        out[tag + "_acc"], out[tag + "_y"], out[tag + "_ws"] = acc, y, qt.scales
    for kind, n, k, m, seed in GGUF_CASES:
        g = rng(seed)
        w = normal(g, (n, k), 0.02)
        x = normal(g, (m, k))
        raw = orc.encode(kind, w)
        tag = f"gguf_{kind}_{n}_{k}_{m}"
        out[tag + "_raw"] = raw
        out[tag + "_deq"] = getattr(orc, "dequant_" + kind)(raw, n * k)
        out[tag + "_y"] = orc.gguf_matmul(x, m, k, raw, kind, n)
    halves = np.concatenate([np.arange(0, 65536, 37, dtype=np.uint16), np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00, 0x7C01, 0x7E00, 0xFFFF], np.uint16)])
    out["f16_bits"], out["f16_as_f32_bits"] = halves, orc.f16_to_f32_bits(halves)
    np.savez_compressed(os.path.join(HERE, "peregrine_quant_path.npz"), **out)
    print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "peregrine_quant_path.npz")), "bytes")


if __name__ == "__main__":
    main()
