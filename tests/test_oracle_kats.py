"""Pins the CPU oracle against every known-answer test the reference holds for
the quantized path.  Inputs and tolerances are the reference tests' own
(cited per test); the assertions that go beyond them (bit-level checks) are
marked as such."""
import numpy as np
import pytest


# ---- src/gguf.rs:574-585 (test_f16_to_f32): exact equality -------------------
@pytest.mark.parametrize("bits,expected", [(0x0000, 0.0), (0x3C00, 1.0), (0xBC00, -1.0), (0x3800, 0.5), (0x8000, -0.0)])
def test_f16_to_f32_kats(oracle, bits, expected):
    got = oracle.f16_to_f32(bits)
    assert got == np.float32(expected)
    assert np.signbit(got) == np.signbit(np.float32(expected))


def test_f16_to_f32_all_bit_patterns_match_ieee(oracle):
    """Beyond the reference: all 65536 halves against numpy's IEEE conversion, bit for bit."""
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32).view(np.uint32)
    got = oracle.f16_to_f32_bits(bits)
    nan = np.isnan(bits.view(np.float16))
    assert np.array_equal(got[~nan], want[~nan])
    # NaN: the reference shifts the payload up by 13 and keeps it (gguf.rs:376-378)
    exp_nan = ((bits[nan].astype(np.uint32) >> 15) << 31) | (0xFF << 23) | ((bits[nan].astype(np.uint32) & 0x3FF) << 13)
    assert np.array_equal(got[nan], exp_nan)


# ---- src/gguf.rs:588-601 (test_dequant_q8_0_simple) --------------------------
def test_dequant_q8_0_simple(oracle):
    block = np.zeros(34, np.uint8)
    block[0], block[1] = 0x00, 0x3C
    block[2:] = np.arange(32, dtype=np.uint8)
    r = oracle.dequant_q8_0(block, 32)
    assert r.shape == (32,)
    assert np.all(np.abs(r - np.arange(32, dtype=np.float32)) < 1e-3)


# ---- tests/gguf_parity.rs:7-28 (test_dequant_q8_0_roundtrip) -----------------
def test_dequant_q8_0_roundtrip(oracle):
    block = np.zeros(34, np.uint8)
    block[0], block[1] = 0x00, 0x38  # f16 0.5
    block[2:] = np.arange(1, 33, dtype=np.uint8)
    r = oracle.dequant_q8_0(block, 32)
    assert np.all(np.abs(r - (np.arange(32) + 1.0) * 0.5) < 0.01)


def test_dequant_q8_0_negative_bytes(oracle):
    """Beyond the reference: bytes >= 0x80 are read as negative i8 (gguf.rs:297)."""
    block = np.zeros(34, np.uint8)
    block[0], block[1] = 0x00, 0x3C
    block[2:] = np.arange(224, 256, dtype=np.uint8)
    r = oracle.dequant_q8_0(block, 32)
    assert np.array_equal(r, np.arange(-32, 0, dtype=np.float32))


# ---- src/gguf.rs:604-615 (test_dequant_q4_0_simple): pins the nibble order ---
def test_dequant_q4_0_simple(oracle):
    block = np.zeros(18, np.uint8)
    block[0], block[1] = 0x00, 0x3C
    block[2] = 0x98
    r = oracle.dequant_q4_0(block, 32)
    assert r.shape == (32,)
    assert abs(r[0] - 0.0) < 1e-3
    assert abs(r[1] - 1.0) < 1e-3
    # bytes 1..15 are zero: both nibbles 0 -> -8 * 1.0
    assert np.array_equal(r[2:], np.full(30, -8.0, np.float32))


# ---- tests/gguf_parity.rs:31-50 (test_dequant_q4_0_symmetry) -----------------
def test_dequant_q4_0_symmetry(oracle):
    block = np.zeros(18, np.uint8)
    block[0], block[1] = 0x00, 0x40  # f16 2.0
    block[2:] = 0x88
    r = oracle.dequant_q4_0(block, 32)
    assert np.all(np.abs(r) < 0.01)


# ---- src/gguf.rs:618-631 (test_dequant_q4_1_simple) --------------------------
def test_dequant_q4_1_simple(oracle):
    block = np.zeros(20, np.uint8)
    block[0], block[1] = 0x00, 0x3C
    block[4] = 0x53
    r = oracle.dequant_q4_1(block, 32)
    assert abs(r[0] - 3.0) < 1e-3
    assert abs(r[1] - 5.0) < 1e-3


# ---- tests/gguf_parity.rs:53-76 (test_dequant_q4_1_with_min) -----------------
def test_dequant_q4_1_with_min(oracle):
    block = np.zeros(20, np.uint8)
    block[0], block[1] = 0x00, 0x3C
    block[2], block[3] = 0x00, 0x49  # f16 10.0
    r = oracle.dequant_q4_1(block, 32)
    assert np.all(np.abs(r - 10.0) < 0.1)


@pytest.mark.parametrize("kind", ["q8_0", "q4_0", "q4_1"])
def test_dequant_asserts_like_reference(oracle, kind):
    """gguf.rs:287-290 / 308-311 / 332-335: num_elements % 32 and the length check."""
    bs = {"q8_0": 34, "q4_0": 18, "q4_1": 20}[kind]
    with pytest.raises(AssertionError):
        oracle.dequant(kind, np.zeros(bs, np.uint8), 31)
    with pytest.raises(AssertionError):
        oracle.dequant(kind, np.zeros(bs, np.uint8), 64)
    assert oracle.dequant(kind, np.zeros(0, np.uint8), 0).size == 0


# ---- src/quant.rs:225-249 (test_quantize_dequantize_roundtrip) ---------------
def test_quantize_dequantize_roundtrip(oracle):
    rows, cols = 32, 64
    data = ((np.arange(rows * cols, dtype=np.float32)) - np.float32(rows * cols // 2)) * np.float32(0.01)
    qt = oracle.quantize_weights(data, rows, cols)
    rec = oracle.dequantize(qt)
    d = data.reshape(rows, cols)
    amax = np.abs(d).max(axis=0)
    scale = np.where(amax == 0, np.float32(1), amax / np.float32(127))
    assert np.array_equal(qt.scales, scale.astype(np.float32))
    assert np.all(np.abs(d - rec) <= scale[None, :] + 1e-6)
    assert np.array_equal(qt.data_i8_t, qt.data_i8.T)


# ---- tests/quant_parity.rs:6-32 ---------------------------------------------
def test_quantize_dequantize_roundtrip_max_error(oracle):
    rows, cols = 64, 128
    i = np.arange(rows * cols, dtype=np.int64)
    data = (((i * 17 + 5) % 400).astype(np.float32) / np.float32(100.0) - np.float32(2.0)).astype(np.float32)
    qt = oracle.quantize_weights(data, rows, cols)
    rec = oracle.dequantize(qt)
    d = data.reshape(rows, cols)
    amax = np.abs(d).max(axis=0)
    scale = np.where(amax == 0, np.float32(1), amax / np.float32(127))
    assert np.all(np.abs(d - rec) <= scale[None, :] + 1e-7)


def _closed_form(m, k, n, mod):
    i = np.arange(m * k, dtype=np.int64)
    a = (((i * 7 + 3) % mod).astype(np.float32) / np.float32(mod) - np.float32(0.5)).astype(np.float32)
    j = np.arange(k * n, dtype=np.int64)
    w = (((j * 13 + 7) % mod).astype(np.float32) / np.float32(mod) - np.float32(0.5)).astype(np.float32)
    return a, w


# ---- src/quant.rs:252-291 (test_matmul_quantized_vs_f32) ---------------------
def test_matmul_quantized_vs_f32(oracle):
    m, k, n = 16, 64, 32
    a, w = _closed_form(m, k, n, 100)
    expected = oracle.matmul_f32(a, w, m, k, n)
    qt = oracle.quantize_weights(w, k, n)
    result = oracle.matmul_quantized(a, m, k, qt)
    diff = np.abs(result - expected)
    rtol = diff / np.maximum(np.abs(expected), 1e-6)
    assert np.all((rtol < 0.05) | (diff < 0.01))


# ---- tests/quant_parity.rs:35-77 (test_i8_matmul_vs_f32_matmul) --------------
def test_i8_matmul_vs_f32_matmul(oracle):
    m, k, n = 32, 128, 64
    a, w = _closed_form(m, k, n, 200)
    expected = oracle.matmul_f32(a, w, m, k, n)
    qt = oracle.quantize_weights(w, k, n)
    result = oracle.matmul_quantized(a, m, k, qt)
    diff = np.abs(result - expected)
    rtol = diff / np.maximum(np.abs(expected), 1e-6)
    assert np.all((rtol < 0.15) | (diff < 0.05))


# ---- tests/quant_parity.rs:79-146: the Metal W8A32 arithmetic vs f32 ---------
def test_w8a32_vs_f32(oracle):
    m, k, n = 32, 128, 64
    a, w = _closed_form(m, k, n, 200)
    expected = oracle.matmul_f32(a, w, m, k, n)
    qt = oracle.quantize_weights(w, k, n)
    got = oracle.matmul_dequant_w8a32(a, m, k, qt)
    diff = np.abs(got - expected)
    rtol = diff / np.maximum(np.abs(expected), 1e-6)
    assert np.all((rtol < 0.10) | (diff < 0.02))


# ---- tests/huffman_parity.rs:9-41: the LCG inputs and shapes -----------------
def _lcg(n, seed):
    out = np.empty(n, np.float32)
    state = seed
    for i in range(n):
        state = (state * 1103515245 + 12345) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(state) / np.float32(0xFFFFFFFF)) * np.float32(2.0) - np.float32(1.0)
    return out


@pytest.mark.parametrize("m,k,n", [(8, 32, 16), (1, 64, 1), (32, 128, 64), (16, 256, 32)])
def test_matmul_quantized_lcg_shapes(oracle, oracle_mt, m, k, n):
    """The reference checks Huffman-decoded weights against matmul_quantized on these
    inputs; here they check that the two oracle builds agree bit for bit and that the
    i32 sums equal an int64 numpy product."""
    a, w = _lcg(m * k, 42), _lcg(k * n, 123)
    qt = oracle.quantize_weights(w, k, n)
    out, acc, a_i8, a_s = oracle.matmul_quantized(a, m, k, qt, return_parts=True)
    qt2 = oracle_mt.quantize_weights(w, k, n)
    out2, acc2, a_i82, a_s2 = oracle_mt.matmul_quantized(a, m, k, qt2, return_parts=True)
    assert np.array_equal(qt.data_i8, qt2.data_i8) and np.array_equal(qt.scales.view(np.uint32), qt2.scales.view(np.uint32))
    assert np.array_equal(a_i8, a_i82) and np.array_equal(acc, acc2)
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))
    want = a_i8.astype(np.int64) @ qt.data_i8.astype(np.int64)
    assert np.array_equal(acc.astype(np.int64), want)
    ep = (acc.astype(np.float32) * a_s[:, None]) * qt.scales[None, :]
    assert np.array_equal(out.view(np.uint32), ep.astype(np.float32).view(np.uint32))


# ---- semantics the reference source fixes but no reference test exercises ----
def test_activation_rounding_is_half_away_and_reciprocal(oracle):
    """quant.rs:101-106: scale = amax/127, inv = 1/scale, q = round(x*inv) half away from zero."""
    x = np.array([[127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5]], np.float32)
    q, s = oracle.quantize_activations(x, 1, 8)
    assert s[0] == np.float32(1.0)
    assert q.tolist() == [[127, 1, -1, 2, -2, 3, -3, 127]]


def test_activation_special_values(oracle):
    nan, inf = np.float32(np.nan), np.float32(np.inf)
    # all-zero row: scale 1.0 (quant.rs:102)
    q, s = oracle.quantize_activations(np.zeros((1, 8), np.float32), 1, 8)
    assert s[0] == 1.0 and not q.any()
    # NaN is ignored by the absmax fold and quantises to 0 (f32::max, `as i8`)
    x = np.array([[nan, 2.0, -4.0, 1.0]], np.float32)
    q, s = oracle.quantize_activations(x, 1, 4)
    assert s[0] == np.float32(4.0) / np.float32(127.0)
    assert q.tolist() == [[0, 64, -127, 32]]
    # +-inf: scale inf, inv 0, inf*0 = NaN -> 0, finite*0 -> 0
    x = np.array([[inf, 2.0, -inf, -1.0]], np.float32)
    q, s = oracle.quantize_activations(x, 1, 4)
    assert np.isinf(s[0]) and q.tolist() == [[0, 0, 0, 0]]
    # absmax so small that amax/127 underflows to 0: inv = inf, nonzero -> +-127, zero -> NaN -> 0
    tiny = np.float32(1e-45)
    x = np.array([[tiny, -tiny, 0.0, tiny]], np.float32)
    q, s = oracle.quantize_activations(x, 1, 4)
    assert s[0] == 0.0 and q.tolist() == [[127, -127, 0, 127]]


def test_weight_quant_divides_and_ignores_nan(oracle):
    """quant.rs:34-36 (strict '>' so NaN never wins), :51 (true division)."""
    w = np.array([[np.nan, 3.0], [2.0, -1.0], [-1.0, 0.4]], np.float32)
    qt = oracle.quantize_weights(w, 3, 2)
    assert qt.scales[0] == np.float32(2.0) / np.float32(127.0)
    assert qt.data_i8[:, 0].tolist() == [0, 127, -64]  # 63.5 rounds away from zero
    assert qt.data_i8[:, 1].tolist() == [127, -42, 17]
    assert qt.cols == 2 and qt.rows == 3


def test_encoder_output_is_what_the_decoder_reads(oracle):
    """Generator contract: the reference decoder layout reads the encoded bytes back
    to within half a quantisation step, and f32->f16 matches numpy's."""
    rng = np.random.Generator(np.random.PCG64(7))
    w = (rng.standard_normal(32 * 64) * 0.02).astype(np.float32)
    for kind, steps in (("q8_0", 127), ("q4_0", 7), ("q4_1", 15)):
        raw = oracle.encode(kind, w)
        back = oracle.dequant(kind, raw, w.size)
        blk = w.reshape(-1, 32)
        span = np.abs(blk).max(axis=1) if kind != "q4_1" else (blk.max(axis=1) - blk.min(axis=1))
        tol = span / steps * (1.01 if kind != "q4_0" else 1.01)
        err = np.abs(back.reshape(-1, 32) - blk).max(axis=1)
        assert np.all(err <= tol + 1e-7), kind
    vals = np.concatenate([rng.standard_normal(2000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 2000),
                           np.array([0, -0.0, 65504, 65519.99, 65520, 1e10, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5], np.float32)])
    vals = vals.astype(np.float32)
    got = np.array([oracle.f32_to_f16(v) for v in vals], np.uint16)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
