"""Tensor data of a GGUF file through the GPU (src/gguf.rs:485-537), against the CPU oracle."""
import numpy as np
import pytest

import _gguf_writer as W
from _inputs import bits_equal, normal, rng

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def _file(pg, gpu, oracle_mt):
    g = rng(11)
    n, k = 96, 256
    w = normal(g, (n, k), 0.02)
    raws = {kind: oracle_mt.encode(kind, w) for kind in ("q8_0", "q4_0", "q4_1")}
    f16 = g.integers(0, 65536, 300, dtype=np.uint16)           # every kind of half: NaN, inf, denormal included
    f32 = normal(g, (7, 9))
    tensors = [("w.q8", [k, n], 8, raws["q8_0"]), ("w.q4", [k, n], 2, raws["q4_0"]), ("w.q41", [k, n], 3, raws["q4_1"]),
               ("h", [300], 1, f16.tobytes()), ("f", [9, 7], 0, f32.tobytes()), ("v.q8", [64], 8, oracle_mt.encode("q8_0", w[0, :64]))]
    data = W.build([("llama.block_count", W.U32, 2), ("llama.rope.freq_base", W.F32, 500000.0)], tensors, alignment=64)
    return pg.GgufFile.parse(data, gpu), w, raws, f16, f32, n, k


def test_load_tensor_f32_every_type(pg, gpu, oracle_mt):
    f, w, raws, f16, f32, n, k = _file(pg, gpu, oracle_mt)
    assert f.get_u32("llama.block_count") == 2 and f.get_f32("llama.rope.freq_base") == np.float32(500000.0)
    for name, kind in (("w.q8", "q8_0"), ("w.q4", "q4_0"), ("w.q41", "q4_1")):
        ref = getattr(oracle_mt, "dequant_" + kind)(raws[kind], n * k)
        assert bits_equal(f.load_tensor_f32(name), ref), name
        assert f.tensor_shape(name) == [n, k]
    got, ref = f.load_tensor_f32("h"), oracle_mt.f16_to_f32_bits(f16).view(np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan) and bits_equal(got[~nan], ref[~nan])
    assert np.array_equal(f.load_tensor_f32("f"), f32.reshape(-1))


def test_load_tensor_q8_and_blocks(pg, gpu, oracle_mt):
    f, w, raws, _, _, n, k = _file(pg, gpu, oracle_mt)
    # load_tensor_q8: Q8_0 bytes -> dequantise -> per-column requantise in the stored [rows = out, cols = in] orientation
    qt = f.load_tensor_q8("w.q8")
    ref = oracle_mt.quantize_weights(oracle_mt.dequant_q8_0(raws["q8_0"], n * k), n, k)
    assert (qt.rows, qt.cols) == (n, k)
    assert np.array_equal(qt.data_i8.reshape(-1), ref.data_i8.reshape(-1)) and np.array_equal(qt.data_i8_t.reshape(-1), ref.data_i8_t.reshape(-1))
    assert bits_equal(qt.scales, ref.scales)
    v = f.load_tensor_q8("v.q8")                                 # 1-D tensor: one row
    assert (v.rows, v.cols) == (1, 64)
    # the block form kept on the GPU multiplies like dequantise + transpose + f32 matmul
    x = normal(rng(12), (3, k))
    for name, kind in (("w.q8", "q8_0"), ("w.q4", "q4_0"), ("w.q41", "q4_1")):
        y = f.load_tensor_blocks(name).matmul(x, 3)
        ref = oracle_mt.gguf_matmul(x, 3, k, raws[kind], kind, n)
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max(), name
    part = f.load_tensor_blocks("w.q4", rows=(32, 64)).matmul(x, 3)
    assert bits_equal(part, f.load_tensor_blocks("w.q4").matmul(x, 3)[:, 32:64])
    with pytest.raises(pg.gguf_file.GgufPanic, match="not a block-quantised type"):
        f.load_tensor_blocks("f")
