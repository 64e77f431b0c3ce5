"""Parity of the CUDA GGUF block decoders and the dequantising product with the CPU oracle,
through the C ABI.

Decoders: bit for bit (one rounded multiply per element; Q4_1 a rounded multiply then a rounded
add).  Product: f32 accumulation order differs from the reference's sequential loop, so the bar is
the path's stated tolerance, max|y - ref| <= 1e-5 * max|ref|, and an f64-accumulated product is
used as arbiter: the CUDA result must be at least as close to it as the tolerance allows."""
import numpy as np
import pytest

from _inputs import bits_equal, normal, rng

pytestmark = pytest.mark.gpu
KINDS = ["q8_0", "q4_0", "q4_1"]
BS = {"q8_0": 34, "q4_0": 18, "q4_1": 20}
REL_TOL = 1e-5  # relative to max|ref|, as the path's contract states


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def _dq(pg, kind):
    return getattr(pg.gguf, "dequant_" + kind)


# ---- the reference's single-block known answers (src/gguf.rs:588-631, tests/gguf_parity.rs:7-76)
def test_reference_kats(pg, gpu):
    b = np.zeros(34, np.uint8); b[1] = 0x3C; b[2:] = np.arange(32)
    assert np.all(np.abs(pg.gguf.dequant_q8_0(b, 32, gpu) - np.arange(32)) < 1e-3)
    b = np.zeros(34, np.uint8); b[1] = 0x38; b[2:] = np.arange(1, 33)
    assert np.all(np.abs(pg.gguf.dequant_q8_0(b, 32, gpu) - (np.arange(32) + 1.0) * 0.5) < 0.01)
    b = np.zeros(18, np.uint8); b[1] = 0x3C; b[2] = 0x98
    r = pg.gguf.dequant_q4_0(b, 32, gpu)
    assert abs(r[0]) < 1e-3 and abs(r[1] - 1.0) < 1e-3          # pins the nibble order
    b = np.zeros(18, np.uint8); b[1] = 0x40; b[2:] = 0x88
    assert np.all(np.abs(pg.gguf.dequant_q4_0(b, 32, gpu)) < 0.01)
    b = np.zeros(20, np.uint8); b[1] = 0x3C; b[4] = 0x53
    r = pg.gguf.dequant_q4_1(b, 32, gpu)
    assert abs(r[0] - 3.0) < 1e-3 and abs(r[1] - 5.0) < 1e-3
    b = np.zeros(20, np.uint8); b[1] = 0x3C; b[3] = 0x49
    assert np.all(np.abs(pg.gguf.dequant_q4_1(b, 32, gpu) - 10.0) < 0.1)
    for bits, want in ((0x0000, 0.0), (0x3C00, 1.0), (0xBC00, -1.0), (0x3800, 0.5), (0x8000, -0.0)):   # src/gguf.rs:574-585
        got = pg.gguf.f16_to_f32(np.uint16(bits), gpu)
        assert got == np.float32(want) and np.signbit(got) == np.signbit(np.float32(want))


def test_f16_to_f32_all_patterns(pg, gpu, oracle):
    bits = np.arange(65536, dtype=np.uint16)
    got = pg.gguf.f16_to_f32(bits, gpu).view(np.uint32)
    assert np.array_equal(got, oracle.f16_to_f32_bits(bits))


@pytest.mark.parametrize("kind", KINDS)
def test_dequant_bit_exact_random_bytes(pg, gpu, oracle, kind):
    """Arbitrary bytes: every scale pattern (subnormal, inf, NaN) and every quant value."""
    g = rng(40)
    nb = 4096 + 3
    raw = g.integers(0, 256, nb * BS[kind], dtype=np.uint8)
    got = _dq(pg, kind)(raw, nb * 32, gpu)
    want = oracle.dequant(kind, raw, nb * 32)
    # a NaN scale gives NaN on both sides; which NaN payload an arithmetic op returns is a property
    # of the processor, not of the algorithm, so NaNs are compared by position only
    nan = np.isnan(want)
    assert nan.any() and np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])


@pytest.mark.parametrize("kind", KINDS)
def test_dequant_encoded_weights(pg, gpu, oracle_mt, kind):
    w = normal(rng(41), (512, 4096), 0.02)
    raw = oracle_mt.encode(kind, w)
    got = _dq(pg, kind)(raw, w.size, gpu)
    assert bits_equal(got, oracle_mt.dequant(kind, raw, w.size))


@pytest.mark.parametrize("kind", KINDS)
def test_dequant_asserts_and_empty(pg, gpu, kind):
    with pytest.raises(AssertionError):       # assert!(num_elements % 32 == 0)
        _dq(pg, kind)(np.zeros(BS[kind], np.uint8), 31, gpu)
    with pytest.raises(AssertionError):       # assert!(data.len() >= num_blocks * block_size)
        _dq(pg, kind)(np.zeros(BS[kind], np.uint8), 64, gpu)
    assert _dq(pg, kind)(np.zeros(0, np.uint8), 0, gpu).size == 0
    # a longer buffer than needed is accepted, like the reference's `>=`
    assert _dq(pg, kind)(np.zeros(BS[kind] * 3, np.uint8), 32, gpu).size == 32


def _check_matmul(pg, gpu, orc, kind, n, k, m, seed):
    g = rng(seed)
    w = normal(g, (n, k), 0.02)
    x = normal(g, (m, k))
    raw = orc.encode(kind, w)
    ref = orc.gguf_matmul(x, m, k, raw, kind, n)
    gw = pg.gguf.GgufWeight(kind, raw, n, k, gpu)
    y = gw.matmul(x, m)
    scale = np.abs(ref).max()
    err = np.abs(y - ref).max() / scale
    assert err <= REL_TOL, f"{kind} M={m}: max|d|/max|ref| = {err:.3e}"
    exact = orc.gguf_matmul_f64(x, m, k, raw, kind, n)
    err_gpu = np.abs(y - exact).max() / scale
    err_ref = np.abs(ref - exact).max() / scale
    assert err_gpu <= max(REL_TOL, 2 * err_ref)
    # per element, relative to the element itself (floored at a thousandth of the output's rms so that exact zeros do
    # not divide): elements that nearly cancel exceed 1e-5 for ANY f32 summation order, the reference's own loop included,
    # so where that happens the f64-accumulated product arbitrates: the GPU result must be no further from it than the
    # reference's loop is (root mean square over those elements)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    den = np.maximum(np.abs(ref), 1e-3 * rms)
    per_elem = np.abs(y - ref) / den
    over = per_elem > REL_TOL
    if over.any():
        rms_gpu = np.sqrt(np.mean((y[over] - exact[over]) ** 2))
        rms_ref = np.sqrt(np.mean((ref[over] - exact[over]) ** 2))
        assert rms_gpu <= rms_ref + 1e-7 * scale, (f"{kind} M={m}: {int(over.sum())} elements beyond 1e-5 of themselves "
                                                     f"(max {per_elem.max():.2e}); GPU rms distance to the f64 product {rms_gpu:.3e} "
                                                     f"against the reference loop's {rms_ref:.3e}")
    gw.free()
    return err, err_gpu, err_ref, float(per_elem.max()), float(over.mean())


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("m,n,k", [(1, 64, 32), (1, 37, 96), (3, 130, 1024), (8, 257, 4096), (5, 1000, 160), (16, 48, 2048),
                                   # the streaming kernel's row groups: two rows, eight + one, eight + two, seven; K beyond one chunk of planes
                                   (2, 300, 512), (9, 100, 1024), (10, 2400, 768), (7, 33, 2048), (2, 64, 16640), (1, 50, 16640), (4, 40, 8448)])
def test_matmul_gguf_small(pg, gpu, oracle_mt, kind, m, n, k):
    _check_matmul(pg, gpu, oracle_mt, kind, n, k, m, 3000 + m + n)


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m", [1, 8])
def test_matmul_gguf_config(pg, gpu, oracle_mt, kind, m):
    """N=14336, K=4096 (the FFN up-projection shape), seed 3000."""
    _check_matmul(pg, gpu, oracle_mt, kind, 14336, 4096, m, 3000)


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
def test_matmul_gguf_cuda_core_path(pg, gpu, oracle_mt, kind):
    """The CUDA-core kernel (used for Q4_1 and for K not a multiple of 128) on shapes the tensor-core
    kernel would otherwise take."""
    gpu.lib.pg_tune_gguf_simple(1)
    try:
        _check_matmul(pg, gpu, oracle_mt, kind, 200, 1024, 5, 3100)
    finally:
        gpu.lib.pg_tune_gguf_simple(0)


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
@pytest.mark.parametrize("m,n,k", [(1, 33, 256), (9, 40, 768), (17, 100, 4096 + 256), (2, 4096, 14336)])
def test_matmul_gguf_tensor_core_path_edges(pg, gpu, oracle_mt, kind, m, n, k):
    """More than eight activation rows (two passes), K longer than one 4096-element chunk
    (accumulating launches), ragged N, outlier activations."""
    g = rng(3200 + m + n)
    w = normal(g, (n, k), 0.02)
    x = normal(g, (m, k))
    x[:, g.choice(k, size=max(1, k // 100), replace=False)] *= np.float32(20.0)
    raw = oracle_mt.encode(kind, w)
    ref = oracle_mt.gguf_matmul(x, m, k, raw, kind, n)
    y = pg.gguf.GgufWeight(kind, raw, n, k, gpu).matmul(x, m)
    assert np.abs(y - ref).max() <= REL_TOL * np.abs(ref).max()


def test_matmul_gguf_row_shard_and_errors(pg, gpu, oracle_mt):
    g = rng(7)
    n, k, m = 96, 256, 4
    w = normal(g, (n, k), 0.02)
    x = normal(g, (m, k))
    raw = oracle_mt.encode("q4_0", w)
    full = pg.gguf.GgufWeight("q4_0", raw, n, k, gpu).matmul(x, m)
    for b, e in ((0, 48), (48, 96), (10, 11)):
        part = pg.gguf.GgufWeight("q4_0", raw, n, k, gpu, rows=(b, e)).matmul(x, m)
        assert bits_equal(part, full[:, b:e])
    with pytest.raises(AssertionError):
        pg.gguf.GgufWeight("q4_0", raw, n, 250, gpu)          # k % 32 != 0
    with pytest.raises(AssertionError):
        pg.gguf.GgufWeight("q4_0", raw[:-1], n, k, gpu)       # short buffer
    with pytest.raises(AssertionError):
        pg.gguf.GgufWeight("q4_0", raw, n, k, gpu).matmul(x[:, :-1], m)


def test_load_tensor_q8_as_quantized(pg, gpu, oracle_mt):
    """src/gguf.rs:386-401: Q8_0 [rows, cols] -> dequantise -> quantize_weights(rows, cols)."""
    rows, cols = 96, 128
    w = normal(rng(12), (rows, cols), 0.02)
    raw = oracle_mt.encode("q8_0", w)
    qt = pg.gguf.load_tensor_q8_as_quantized(raw, rows, cols, gpu)
    ref = oracle_mt.quantize_weights(oracle_mt.dequant_q8_0(raw, rows * cols), rows, cols)
    assert bits_equal(qt.scales, ref.scales) and np.array_equal(qt.data_i8, ref.data_i8) and np.array_equal(qt.data_i8_t, ref.data_i8_t)
    with pytest.raises(AssertionError):       # assert!(cols % 32 == 0)
        pg.gguf.load_tensor_q8_as_quantized(raw, rows, 100, gpu)


def test_matmul_f32_checker_is_bit_exact(pg, gpu, oracle):
    """The naive f32 product (src/tensor.rs:1342-1354) keeps the reference's summation order."""
    import ctypes as C
    from peregrine_b200 import _lib

    g = rng(3)
    m, k, n = 7, 300, 41
    a, b = normal(g, (m, k)), normal(g, (k, n), 0.02)
    d_a, d_b, d_o = gpu.upload(a.reshape(-1)), gpu.upload(b.reshape(-1)), gpu.alloc(m * n, np.float32)
    _lib.check(gpu.lib.pg_matmul_f32(gpu.handle, d_a.ptr, d_b.ptr, m, k, n, d_o.ptr))
    assert bits_equal(d_o.read().reshape(m, n), oracle.matmul_f32(a, b, m, k, n))
