"""Parity of the CUDA int8 path with the CPU oracle, through the C ABI (ctypes).

Bars: quantised i8 activations/weights, f32 scales and i32 accumulators are compared
bit for bit; the f32 output of the W8A8 product is also compared bit for bit (the epilogue is two
rounded multiplies in a fixed order), which is stricter than the 1e-5 relative the path requires.
The reference's own tolerance tests (src/quant.rs:225-291, tests/quant_parity.rs:6-77) are
re-run against the CUDA path with their inputs and tolerances."""
import numpy as np
import pytest

from _inputs import bits_equal, linear_inputs, normal, rng

pytestmark = pytest.mark.gpu

ALGOS = {"naive": 1, "stream": 2, "tcgen05": 3, "wstream": 4}


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


# ------------------------------------------------------------ activations ----
@pytest.mark.parametrize("m,k,seed,outliers", [
    (32, 4096, 0, False),      # single-linear config
    (1, 4096, 1000, True), (4, 4096, 1001, True), (16, 4096, 1002, True),
    (16, 14336, 1008, True),   # widest decode row
    (512, 4096, 2000, False),
    (3, 20000, 5, False),      # longer than the register-resident part of a row
    (7, 1027, 6, False), (5, 1, 7, False), (2, 3, 8, False), (1, 18, 9, False),  # unaligned: scalar kernel
])
def test_quantize_activations_bit_exact(pg, gpu, oracle_mt, m, k, seed, outliers):
    x, _ = linear_inputs(m, k, 1, seed, outliers)
    q, s = pg.quant.quantize_activations(x, m, k, gpu)
    qo, so = oracle_mt.quantize_activations(x, m, k)
    assert bits_equal(s, so)
    assert np.array_equal(q, qo)


def test_quantize_activations_special_rows(pg, gpu, oracle):
    k = 256
    g = rng(11)
    x = normal(g, (10, k))
    x[0] = 0.0                                   # all-zero row: scale 1.0
    x[1, 5] = np.nan                             # NaN ignored by absmax, quantises to 0
    x[2, 7] = np.inf                             # scale inf, everything -> 0
    x[3, 9] = -np.inf
    x[4] = np.float32(1e-45) * np.sign(x[4])     # amax/127 underflows to 0: inv = inf
    x[5] = x[5] * np.float32(1e-38)              # subnormal scale
    x[6, :] = np.nan                             # all NaN: amax 0 -> scale 1, q = 0
    x[7] = x[7] * np.float32(1e30)               # large finite
    x[8, :4] = [3.4e38, -3.4e38, 1.0, 0.0]
    x[9, 0] = -0.0
    q, s = pg.quant.quantize_activations(x, 10, k, gpu)
    qo, so = oracle.quantize_activations(x, 10, k)
    assert bits_equal(s, so)
    assert np.array_equal(q, qo)
    assert s[0] == 1.0 and not q[0].any() and not q[2].any() and not q[6].any()


def test_quantize_activations_ties_round_half_away(pg, gpu, oracle):
    """absmax 127 makes scale = inv = 1, so x.5 inputs are exact ties: the scalar reference rounds
    them away from zero (src/quant.rs:106)."""
    k = 512
    x = np.zeros((2, k), np.float32)
    x[0, 0] = 127.0
    x[0, 1:255] = np.arange(-127, 127, dtype=np.float32) + 0.5
    x[1, 0] = -127.0
    x[1, 1:255] = -(np.arange(-127, 127, dtype=np.float32) + 0.5)
    q, s = pg.quant.quantize_activations(x, 2, k, gpu)
    qo, so = oracle.quantize_activations(x, 2, k)
    assert s[0] == 1.0 and np.array_equal(q, qo) and bits_equal(s, so)
    assert q[0, 1 + 127] == 1 and q[0, 1 + 126] == -1  # 0.5 -> 1, -0.5 -> -1


def test_quantize_activations_empty(pg, gpu):
    q, s = pg.quant.quantize_activations(np.zeros(0, np.float32), 0, 64, gpu)
    assert q.shape == (0, 64) and s.shape == (0,)
    q, s = pg.quant.quantize_activations(np.zeros(0, np.float32), 3, 0, gpu)
    assert q.shape == (3, 0) and np.array_equal(s, np.ones(3, np.float32))
    with pytest.raises(AssertionError):  # the reference's assert_eq!(data.len(), rows * cols)
        pg.quant.quantize_activations(np.zeros(5, np.float32), 2, 3, gpu)


# ---------------------------------------------------------------- weights ----
@pytest.mark.parametrize("k,n,seed", [(4096, 4096, 0), (4096, 1024, 1), (33, 65, 2), (1, 7, 3), (129, 31, 4), (64, 1, 5)])
def test_quantize_weights_bit_exact(pg, gpu, oracle_mt, k, n, seed):
    w = normal(rng(seed), (k, n), 0.02)
    qt = pg.quant.quantize_weights(w, k, n, gpu)
    ref = oracle_mt.quantize_weights(w, k, n)
    assert bits_equal(qt.scales, ref.scales)
    assert np.array_equal(qt.data_i8, ref.data_i8)
    assert np.array_equal(qt.data_i8_t, ref.data_i8_t)
    assert (qt.rows, qt.cols) == (k, n)


def test_quantize_weights_special_columns(pg, gpu, oracle):
    g = rng(21)
    w = normal(g, (40, 12), 0.02)
    w[:, 0] = 0.0              # zero column: scale 1
    w[3, 1] = np.nan           # NaN never wins the absmax, quantises to 0
    w[5, 2] = np.inf           # scale inf: inf/inf = NaN -> 0, finite/inf -> 0
    w[:, 3] = np.float32(1e-44)
    w[:, 4] *= np.float32(1e-38)
    w[:, 5] = np.nan
    w[0, 6], w[1, 6] = 127.0, 63.5   # tie after a true division
    qt = pg.quant.quantize_weights(w, 40, 12, gpu)
    ref = oracle.quantize_weights(w, 40, 12)
    assert bits_equal(qt.scales, ref.scales)
    assert np.array_equal(qt.data_i8, ref.data_i8) and np.array_equal(qt.data_i8_t, ref.data_i8_t)


def test_dequantize_bit_exact(pg, gpu, oracle):
    w = normal(rng(31), (96, 50), 0.02)
    qt = pg.quant.quantize_weights(w, 96, 50, gpu)
    ref = oracle.quantize_weights(w, 96, 50)
    assert bits_equal(pg.quant.dequantize(qt, gpu), oracle.dequantize(ref))


# ----- the reference's own tests, against the CUDA path (same inputs and tolerances) -----
def test_reference_roundtrip_tests(pg, gpu):
    for rows, cols, gen, eps in (
        (32, 64, lambda i: (i.astype(np.float32) - np.float32(32 * 64 // 2)) * np.float32(0.01), 1e-6),   # src/quant.rs:225-249
        (64, 128, lambda i: ((i * 17 + 5) % 400).astype(np.float32) / np.float32(100.0) - np.float32(2.0), 1e-7),  # tests/quant_parity.rs:6-32
    ):
        data = gen(np.arange(rows * cols, dtype=np.int64)).astype(np.float32)
        qt = pg.quant.quantize_weights(data, rows, cols, gpu)
        rec = pg.quant.dequantize(qt, gpu)
        d = data.reshape(rows, cols)
        amax = np.abs(d).max(axis=0)
        scale = np.where(amax == 0, np.float32(1), amax / np.float32(127))
        assert np.all(np.abs(d - rec) <= scale[None, :] + eps)


@pytest.mark.parametrize("m,k,n,mod,rt,at", [(16, 64, 32, 100, 0.05, 0.01), (32, 128, 64, 200, 0.15, 0.05)])
def test_reference_i8_vs_f32_matmul(pg, gpu, oracle, m, k, n, mod, rt, at):
    """src/quant.rs:252-291 and tests/quant_parity.rs:35-77."""
    a = (((np.arange(m * k, dtype=np.int64) * 7 + 3) % mod).astype(np.float32) / np.float32(mod) - np.float32(0.5)).astype(np.float32)
    w = (((np.arange(k * n, dtype=np.int64) * 13 + 7) % mod).astype(np.float32) / np.float32(mod) - np.float32(0.5)).astype(np.float32)
    expected = oracle.matmul_f32(a, w, m, k, n)
    qt = pg.quant.quantize_weights(w, k, n, gpu)
    result = pg.quant.matmul_quantized(a, m, k, qt, gpu)
    diff = np.abs(result - expected)
    rtol = diff / np.maximum(np.abs(expected), 1e-6)
    assert np.all((rtol < rt) | (diff < at))
    # and bit-exact against the oracle's W8A8 result
    assert bits_equal(result, oracle.matmul_quantized(a, m, k, oracle.quantize_weights(w, k, n)))


def _lcg(n, seed):
    out = np.empty(n, np.float32)
    state = seed
    for i in range(n):
        state = (state * 1103515245 + 12345) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(state) / np.float32(0xFFFFFFFF)) * np.float32(2.0) - np.float32(1.0)
    return out


@pytest.mark.parametrize("m,k,n", [(8, 32, 16), (1, 64, 1), (32, 128, 64), (16, 256, 32)])
def test_reference_lcg_shapes(pg, gpu, oracle, m, k, n):
    """Inputs and shapes of tests/huffman_parity.rs:23-41."""
    a, w = _lcg(m * k, 42), _lcg(k * n, 123)
    ref = oracle.quantize_weights(w, k, n)
    out_o, acc_o, q_o, s_o = oracle.matmul_quantized(a, m, k, ref, return_parts=True)
    qt = pg.quant.quantize_weights(w, k, n, gpu)
    y, acc, q, s = pg.quant.matmul_quantized_parts(gpu, a, m, k, qt)
    assert np.array_equal(q, q_o) and bits_equal(s, s_o) and np.array_equal(acc, acc_o) and bits_equal(y, out_o)


# ------------------------------------------------ the product, every kernel ----
def _check_product(pg, gpu, orc, x, w, m, k, n, algos):
    ref = orc.quantize_weights(w, k, n)
    out_o, acc_o, q_o, s_o = orc.matmul_quantized(x, m, k, ref, return_parts=True)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    qt.to_gpu(gpu)
    for name in algos:
        y, acc, q, s = pg.quant.matmul_quantized_parts(gpu, x, m, k, qt, ALGOS[name])
        assert np.array_equal(q, q_o) and bits_equal(s, s_o), name
        assert np.array_equal(acc, acc_o), f"{name}: i32 accumulators differ"
        assert bits_equal(y, out_o), f"{name}: f32 outputs differ"
    y = pg.quant.matmul_quantized(x, m, k, qt, gpu)      # host API, automatic kernel choice
    assert bits_equal(y, out_o)
    qt.free_gpu()


def test_single_linear_config(pg, gpu, oracle_mt):
    """M=32, K=4096, N=4096, seed 0."""
    x, w = linear_inputs(32, 4096, 4096, 0)
    _check_product(pg, gpu, oracle_mt, x, w, 32, 4096, 4096, ["naive", "stream", "tcgen05"])


@pytest.mark.parametrize("idx,m,k,n", [(i, m, k, n) for i, (m, (k, n)) in enumerate(
    [(m, kn) for kn in [(4096, 4096), (4096, 14336), (14336, 4096)] for m in (1, 4, 16)])])
def test_decode_gemv_sweep(pg, gpu, oracle_mt, idx, m, k, n):
    """Llama-3-8B projection shapes, activations with 1 % outlier channels (x20)."""
    x, w = linear_inputs(m, k, n, 1000 + idx, outliers=True)
    _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["wstream", "stream", "tcgen05"])


@pytest.mark.parametrize("m,k,n", [
    (1, 64, 1), (2, 128, 9), (8, 192, 8), (9, 64, 17), (16, 576, 24), (16, 4096 + 64, 100), (5, 1088, 1000), (12, 2048, 130),
    (3, 8192, 40), (8, 8192 + 128, 33), (16, 4160, 3000), (8, 14336, 100), (2, 65536 - 64, 20), (7, 512, 2369 * 16 + 3),
])
def test_warp_stream_kernel_ragged_shapes(pg, gpu, oracle_mt, m, k, n):
    """Edges of the persistent decode kernel: N not a multiple of the 8-column tile, K not a multiple of the 512-byte
    ring segment, K beyond one shared-memory range of activations (forced split), more tiles than warps."""
    x, w = linear_inputs(m, k, n, 177 + m + n)
    _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["naive", "wstream"])
    assert gpu.device_status() == 0


@pytest.mark.parametrize("cs", [2, 4])
@pytest.mark.parametrize("kw", [0, 1, 4, 16])
def test_warp_stream_k_split_over_a_cluster(pg, gpu, oracle_mt, kw, cs):
    """K split over the 2 or 4 CTAs of a cluster (each holds its part of the activations; the other CTAs add their sums
    into the first one's shared memory once per round of tiles): forced on small shapes, several rounds included, and
    taken by itself when the rows of K do not fit beside the ring in one CTA."""
    gpu.lib.pg_tune_wstream_kw(kw)
    gpu.lib.pg_tune_wstream_cluster(cs)
    try:
        for m, k, n in ((1, 4096, 520), (16, 4096, 8), (7, 4032, 33), (16, 4096, 3000), (9, 4096, 2369 * 16 + 5)):
            x, w = linear_inputs(m, k, n, 850 + kw + m)
            _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["wstream", "wstream"])
        gpu.lib.pg_tune_wstream_cluster(0)
        gpu.lib.pg_tune_wstream_kw(0)
        if cs == 2 and kw == 0:
            for m, k, n in ((16, 14336, 264), (8, 14336, 100), (12, 8192 + 512, 100), (16, 16384 - 64, 40)):
                x, w = linear_inputs(m, k, n, 870 + kw + m)
                _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["naive", "wstream"])
        assert gpu.device_status() == 0
    finally:
        gpu.lib.pg_tune_wstream_kw(0)
        gpu.lib.pg_tune_wstream_cluster(0)


@pytest.mark.parametrize("kw", [1, 2, 4, 8, 16])
def test_warp_stream_every_k_split(pg, gpu, oracle_mt, kw):
    """1..16 warps share a tile, each with its own part of K (uneven last parts included); run twice back to back."""
    gpu.lib.pg_tune_wstream_kw(kw)
    try:
        for m, k, n in ((1, 4096, 520), (16, 4096, 72), (7, 1984, 33), (16, 2048, 3000), (4, 14336, 264), (8, 14336, 40)):
            x, w = linear_inputs(m, k, n, 800 + kw + m)
            _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["wstream", "wstream"])
        assert gpu.device_status() == 0
    finally:
        gpu.lib.pg_tune_wstream_kw(0)


@pytest.mark.parametrize("m,k,n", [
    (1, 16, 1), (2, 32, 9), (8, 48, 8), (9, 64, 17), (16, 80, 24), (17, 128, 40), (33, 144, 7), (64, 4096 + 16, 100),
    (5, 1040, 1000), (12, 2048, 130),
])
def test_stream_kernel_ragged_shapes(pg, gpu, oracle_mt, m, k, n):
    x, w = linear_inputs(m, k, n, 77 + m + n)
    _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["naive", "stream"])


@pytest.mark.parametrize("m,k,n", [
    (1, 16, 1), (128, 128, 256), (127, 112, 255), (129, 144, 257), (200, 1040, 300), (300, 4096, 520), (65, 272, 64),
    (256, 2048, 1000),
])
def test_tcgen05_kernel_ragged_shapes(pg, gpu, oracle_mt, m, k, n):
    """Tile edges in M, N and K (K not a multiple of the 128-byte stage, N not of the tile)."""
    x, w = linear_inputs(m, k, n, 99 + m + n)
    _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["naive", "tcgen05"])


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_tcgen05_every_tile_width(pg, gpu, oracle_mt, bn):
    x, w = linear_inputs(384, 1024, 1280, 500 + bn)
    gpu.lib.pg_tune_tcgen05_bn(bn)
    try:
        _check_product(pg, gpu, oracle_mt, x, w, 384, 1024, 1280, ["tcgen05"])
    finally:
        gpu.lib.pg_tune_tcgen05_bn(0)


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
@pytest.mark.parametrize("m", [1, 17, 32, 33, 64, 65, 128])
def test_tcgen05_small_row_counts(pg, gpu, oracle_mt, m, bn):
    """One row of tiles: the A tile is copied with 32, 64 or 128 rows (the MMA reads 128 either way; what lies behind the
    copied rows must not reach the output), every tile width, ragged K and N, and K shorter than the ring."""
    gpu.lib.pg_tune_tcgen05_bn(bn)
    try:
        for k, n in ((1040, 520), (144, 257), (4096, 96)):
            x, w = linear_inputs(m, k, n, 900 + m + bn + n)
            _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["tcgen05"])
    finally:
        gpu.lib.pg_tune_tcgen05_bn(0)


@pytest.mark.parametrize("m,k,n", [(17, 4096, 14336), (48, 4096, 6144), (64, 14336, 4096), (100, 4096, 4096), (24, 1040, 12000)])
def test_mid_batch_dispatch(pg, gpu, oracle_mt, m, k, n):
    """17 <= M <= 128 with the automatic kernel choice (tcgen05 with the modelled tile width, or the FIFO kernel)."""
    x, w = linear_inputs(m, k, n, 40 + m)
    _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["naive"])


@pytest.mark.parametrize("split", [0, 2, 4, 8])
@pytest.mark.parametrize("m,k,n,bn", [(17, 14336, 4096, 0), (64, 4096, 4096, 0), (128, 4096, 520, 64), (33, 1040, 1000, 32), (100, 2048, 14336, 256),
                                      (20, 384, 96, 0)])
def test_tcgen05_k_split_over_ctas(pg, gpu, oracle_mt, m, k, n, bn, split):
    """One row of tiles with K divided over CTAs: the parts add their s32 sums into the zeroed workspace, the last part
    in applies the scales.  Every number of parts (0 = the library's own choice), ragged N and K, more parts than k-blocks
    (384 bytes of K are three k-blocks), twice in a row and once more from a recorded graph: the workspace must be back
    at zero after every call."""
    x, w = linear_inputs(m, k, n, 4000 + m + n)
    gpu.lib.pg_tune_tcgen05_split(split)
    gpu.lib.pg_tune_tcgen05_bn(bn)
    try:
        _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["tcgen05", "tcgen05"])
        ref = oracle_mt.quantize_weights(w, k, n)
        out_o = oracle_mt.matmul_quantized(x, m, k, ref)
        qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
        qt.to_gpu(gpu)
        d_x = gpu.upload(x.reshape(-1))
        d_y = gpu.alloc(m * n, np.float32)
        call = lambda: pg._lib.check(gpu.lib.pg_matmul_quantized_ex(gpu.handle, d_x.ptr, m, k, qt._gpu, d_y.ptr, None, None, None, pg._lib.ALGO_TCGEN05))
        call()
        with gpu.record() as graph:
            call()
            call()
        for _ in range(3):
            graph.launch()
        gpu.sync()
        assert bits_equal(d_y.read().reshape(m, n), out_o)
        graph.free()
        qt.free_gpu()
        assert gpu.device_status() == 0
    finally:
        gpu.lib.pg_tune_tcgen05_split(0)
        gpu.lib.pg_tune_tcgen05_bn(0)


@pytest.mark.parametrize("m,k,n", [(256, 128, 256), (512, 1024, 768), (300, 1040, 520), (1000, 4096, 1000), (129, 144, 257)])
def test_tcgen05_cta_pairs(pg, gpu, oracle_mt, m, k, n):
    """cta_group::2: two CTAs share one 256 x 256 tile; full and ragged tiles in M, N and K."""
    x, w = linear_inputs(m, k, n, 900 + m + n)
    gpu.lib.pg_tune_tcgen05_pair(2)
    try:
        _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["tcgen05"])
        assert gpu.device_status() == 0
    finally:
        gpu.lib.pg_tune_tcgen05_pair(0)


@pytest.mark.parametrize("ng", [1, 2, 4])
def test_stream_every_column_group(pg, gpu, oracle_mt, ng):
    gpu.lib.pg_tune_stream_ng(ng)
    try:
        for m in (3, 16):
            x, w = linear_inputs(m, 1024, 333, 600 + ng + m)
            _check_product(pg, gpu, oracle_mt, x, w, m, 1024, 333, ["stream"])
    finally:
        gpu.lib.pg_tune_stream_ng(0)


@pytest.mark.parametrize("split", [1, 2, 4])
@pytest.mark.parametrize("depth", [4, 8])
def test_stream_cluster_split_and_fifo_depth(pg, gpu, oracle_mt, split, depth):
    """K split over a thread-block cluster (partial sums through distributed shared memory) and
    both FIFO depths, on shapes whose K does not divide evenly."""
    gpu.lib.pg_tune_stream_split(split)
    gpu.lib.pg_tune_stream_depth(depth)
    try:
        for m, k, n in ((1, 4096, 520), (16, 14336, 72), (7, 1040, 33), (33, 2064, 40), (64, 192, 9)):
            x, w = linear_inputs(m, k, n, 700 + split + depth + m)
            _check_product(pg, gpu, oracle_mt, x, w, m, k, n, ["stream"])
    finally:
        gpu.lib.pg_tune_stream_split(0)
        gpu.lib.pg_tune_stream_depth(0)


def test_unaligned_k_uses_the_checker_kernel(pg, gpu, oracle):
    """K not a multiple of 16: neither fast kernel takes it; the result is still exact."""
    for m, k, n in ((3, 17, 5), (20, 1001, 33), (70, 250, 19)):
        x, w = linear_inputs(m, k, n, 42 + k)
        ref = oracle.quantize_weights(w, k, n)
        out_o = oracle.matmul_quantized(x, m, k, ref)
        qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
        assert bits_equal(pg.quant.matmul_quantized(x, m, k, qt, gpu), out_o)


@pytest.mark.parametrize("idx,n", [(0, 4096), (1, 14336)])
def test_prefill_m512(pg, gpu, oracle_mt, idx, n):
    """Prefill configs M=512, K=4096, N in {4096, 14336}: full i32 and f32 comparison with the CPU oracle."""
    x, w = linear_inputs(512, 4096, n, 2000 + idx)
    _check_product(pg, gpu, oracle_mt, x, w, 512, 4096, n, ["tcgen05"])


@pytest.mark.parametrize("idx,m,n", [(2, 2048, 4096), (3, 2048, 14336), (4, 8192, 4096), (5, 8192, 14336)])
def test_prefill_large_vs_checker_and_sampled_oracle(pg, gpu, oracle_mt, idx, m, n):
    """Too large to sweep on the CPU: the tcgen05 result is compared over the whole output with the
    independent one-thread-per-output kernel, and on 200k random outputs with the CPU oracle."""
    import ctypes as C

    k = 4096
    g = rng(2000 + idx)
    x = normal(g, (m, k))
    # weights: quantise on the GPU (bit-exact with the oracle, checked above) to keep the test short
    w = normal(g, (k, n), 0.02)
    qt = pg.quant.quantize_weights(w, k, n, gpu)
    qt.to_gpu(gpu)
    lib = gpu.lib
    d_x = gpu.upload(x.reshape(-1))
    d_q = gpu.alloc(m * k + 16, np.int8)
    d_s = gpu.alloc(m, np.float32)
    d_y1, d_y2 = gpu.alloc(m * n, np.float32), gpu.alloc(m * n, np.float32)
    d_a1, d_a2 = gpu.alloc(m * n, np.int32), gpu.alloc(m * n, np.int32)
    from peregrine_b200 import _lib

    _lib.check(lib.pg_matmul_quantized_ex(gpu.handle, d_x.ptr, m, k, qt._gpu, d_y1.ptr, d_a1.ptr, d_q.ptr, d_s.ptr, 3))
    _lib.check(lib.pg_gemm_i8(gpu.handle, d_q.ptr, d_s.ptr, m, k, qt._gpu, d_y2.ptr, d_a2.ptr, 1))
    gpu.sync()
    assert gpu.device_status() == 0
    a1, a2 = d_a1.read(), d_a2.read()
    assert np.array_equal(a1, a2)
    y1 = d_y1.read()
    assert bits_equal(y1, d_y2.read())
    q = d_q.read()[: m * k].reshape(m, k)
    qo, so = oracle_mt.quantize_activations(x, m, k)
    assert np.array_equal(q, qo) and bits_equal(d_s.read(), so)
    idx_s = rng(9).integers(0, m * n, 200_000)
    acc_s = oracle_mt.gemm_i8_sampled(qo, qt.data_i8_t, n, k, idx_s)
    assert np.array_equal(a1[idx_s], acc_s)
    ep = (acc_s.astype(np.float32) * so[idx_s // n]) * qt.scales[idx_s % n]
    assert bits_equal(y1[idx_s], ep.astype(np.float32))
    # linearity in the integer domain: A and -A give negated sums
    for b in (d_x, d_q, d_s, d_y1, d_y2, d_a1, d_a2):
        b.free()
    qt.free_gpu()


def test_shape_errors_match_reference_asserts(pg, gpu):
    w = normal(rng(1), (64, 8), 0.02)
    qt = pg.quant.quantize_weights(w, 64, 8, gpu)
    with pytest.raises(AssertionError):   # assert_eq!(w.rows, k)
        pg.quant.matmul_quantized(np.zeros(2 * 32, np.float32), 2, 32, qt, gpu)
    with pytest.raises(AssertionError):   # assert_eq!(a_data.len(), m * k)
        pg.quant.matmul_quantized(np.zeros(10, np.float32), 2, 64, qt, gpu)
    with pytest.raises(AssertionError):   # expect("weights not on GPU")
        pg.quant.matmul_quantized_gpu(gpu, np.zeros(128, np.float32), 2, 64, pg.quant.quantize_weights(w, 64, 8, gpu))
    assert pg.quant.matmul_quantized(np.zeros(0, np.float32), 0, 64, qt, gpu).shape == (0, 8)


def test_matmul_quantized_gpu_is_async_and_resident(pg, gpu, oracle):
    """to_gpu is idempotent, the result buffer is returned unsynchronised and read() blocks
    (tests/quant_parity.rs:98-107)."""
    x, w = linear_inputs(4, 256, 48, 5)
    ref = oracle.quantize_weights(w, 256, 48)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, 256, 48)
    qt.to_gpu(gpu)
    h = qt._gpu
    qt.to_gpu(gpu)
    assert qt._gpu is h
    buf = pg.quant.matmul_quantized_gpu(gpu, x, 4, 256, qt)
    gpu.sync()
    assert bits_equal(buf.read().reshape(4, 48), oracle.matmul_quantized(x, 4, 256, ref))
    qt.data_i8_t[:] = 0
    qt.scales[:] = 0
    qt.from_gpu(gpu)
    assert np.array_equal(qt.data_i8_t, ref.data_i8_t) and bits_equal(qt.scales, ref.scales)


def test_column_shard_equals_slice_of_full_result(pg, gpu, oracle):
    """A GPU holding columns [b,e) produces exactly y[:, b:e] of the unsharded product."""
    x, w = linear_inputs(16, 512, 96, 8)
    ref = oracle.quantize_weights(w, 512, 96)
    full = oracle.matmul_quantized(x, 16, 512, ref)
    for b, e in ((0, 48), (48, 96), (24, 25), (96, 96)):
        qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, 512, 96)
        qt.to_gpu(gpu, b, e)
        assert bits_equal(pg.quant.matmul_quantized(x, 16, 512, qt, gpu), full[:, b:e])


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (1, 1024, 320), (4, 4096, 512), (16, 4096, 4096), (16, 14336, 64), (3, 1000, 40)])
def test_page_locked_host_buffers_give_the_same_bits(pg, gpu, oracle_mt, m, k, n):
    """pg_matmul_quantized_host lets kernels address page-locked host buffers themselves where that is faster (the
    quantiser reads x, a copy kernel pushes y) and uses the copy engines otherwise: pageable, page-locked, misaligned
    page-locked buffers and every path forced on or off all give the oracle's bits."""
    import torch

    from peregrine_b200 import _lib

    x, w = linear_inputs(m, k, n, 700 + m + n)
    ref = oracle_mt.quantize_weights(w, k, n)
    want = oracle_mt.matmul_quantized(x, m, k, ref)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    qt.to_gpu(gpu)
    lib = gpu.lib
    x_pin = torch.from_numpy(x.reshape(-1)).pin_memory()
    x_off = torch.empty(m * k + 1).pin_memory()          # a view that starts 4 bytes into a page-locked block
    x_off[1:].copy_(torch.from_numpy(x.reshape(-1)))
    y_pin = torch.empty(m * n + 1).pin_memory()
    try:
        for x_bytes, y_bytes, push in ((-1, -1, -1), (0, 0, 0), (1 << 24, 1 << 24, 0), (0, 0, 1 << 24), (1 << 24, 1024, 1 << 24)):
            lib.pg_tune_host_direct(x_bytes, y_bytes)
            lib.pg_tune_host_push(push)
            for xp, yp in ((x_pin.data_ptr(), y_pin.data_ptr()), (x_off.data_ptr() + 4, y_pin.data_ptr() + 4),
                           (x.ctypes.data, y_pin.data_ptr())):
                y_pin.fill_(float("nan"))
                _lib.check(lib.pg_matmul_quantized_host(gpu.handle, xp, m, k, qt._gpu, yp))
                off = 1 if yp != y_pin.data_ptr() else 0
                assert bits_equal(y_pin.numpy()[off:off + m * n].reshape(m, n), want), (x_bytes, y_bytes)
        # new contents in the same page-locked buffer are what the next call computes with: -x gives exactly -y
        lib.pg_tune_host_direct(-1, -1)
        lib.pg_tune_host_push(-1)
        for sign in (-1.0, 1.0, -1.0):
            x_pin.copy_(torch.from_numpy(x.reshape(-1)) * sign)
            _lib.check(lib.pg_matmul_quantized_host(gpu.handle, x_pin.data_ptr(), m, k, qt._gpu, y_pin.data_ptr()))
            assert np.array_equal(y_pin.numpy()[:m * n].reshape(m, n), want * np.float32(sign))
    finally:
        lib.pg_tune_host_direct(-1, -1)
        lib.pg_tune_host_push(-1)
        qt.free_gpu()


def test_repeated_host_calls_replayed_from_a_graph(pg, gpu, oracle_mt):
    """A blocking host call that comes back with the same page-locked buffers, shape and weights is recorded the second
    time and replayed afterwards: every call must still compute with what the buffers hold at that moment, count its
    kernels, survive other calls in between, and stop using a recording when its weights are freed (a new tensor may
    get the same address)."""
    import torch

    from peregrine_b200 import _lib

    lib = gpu.lib
    g = rng(31)
    shapes = [(1, 4096, 512), (16, 1024, 320), (4, 14336, 64)]
    refs, qts, xs, ys = [], [], [], []
    for m, k, n in shapes:
        x, w = linear_inputs(m, k, n, 800 + n)
        ref = oracle_mt.quantize_weights(w, k, n)
        qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
        qt.to_gpu(gpu)
        refs.append(ref)
        qts.append(qt)
        xs.append(torch.empty(m * k).pin_memory())
        ys.append(torch.empty(m * n).pin_memory())
    try:
        for on in (1, 0, 1):
            lib.pg_tune_host_graph(on)
            for rnd in range(5):
                for i, (m, k, n) in enumerate(shapes):
                    x = g.standard_normal((m, k), dtype=np.float32)
                    xs[i].copy_(torch.from_numpy(x.reshape(-1)))
                    ys[i].fill_(float("nan"))
                    before = lib.pg_launch_count()
                    _lib.check(lib.pg_matmul_quantized_host(gpu.handle, xs[i].data_ptr(), m, k, qts[i]._gpu, ys[i].data_ptr()))
                    assert lib.pg_launch_count() - before == 3, "quantiser, product, copy kernel"
                    want = oracle_mt.matmul_quantized(x, m, k, refs[i])
                    assert bits_equal(ys[i].numpy().reshape(m, n), want), (on, rnd, i)
        # the weights of shape 0 go away; new weights of the same size (possibly at the same addresses) with other values
        m, k, n = shapes[0]
        qts[0].free_gpu()
        x, w = linear_inputs(m, k, n, 999)
        refs[0] = oracle_mt.quantize_weights(w, k, n)
        qts[0] = pg.quant.QuantizedTensor(refs[0].data_i8, refs[0].data_i8_t, refs[0].scales, k, n)
        qts[0].to_gpu(gpu)
        for rnd in range(3):
            x = g.standard_normal((m, k), dtype=np.float32)
            xs[0].copy_(torch.from_numpy(x.reshape(-1)))
            _lib.check(lib.pg_matmul_quantized_host(gpu.handle, xs[0].data_ptr(), m, k, qts[0]._gpu, ys[0].data_ptr()))
            assert bits_equal(ys[0].numpy().reshape(m, n), oracle_mt.matmul_quantized(x, m, k, refs[0])), rnd
        assert gpu.device_status() == 0
    finally:
        lib.pg_tune_host_graph(1)
        for qt in qts:
            qt.free_gpu()


def test_random_shapes_every_kernel_agrees(pg, gpu):
    """150 seeded random (M, K, N) around every switch point of the automatic kernel choice: the chosen kernel, the
    one-thread-per-output checker and the blocking host call give the same accumulators and the same f32 bits."""
    import ctypes as C

    from peregrine_b200 import _lib

    lib = gpu.lib
    g = rng(2024)
    ms = [1, 2, 3, 4, 7, 8, 15, 16, 17, 24, 31, 32, 33, 48, 63, 64, 65, 100, 127, 128, 129, 200, 300]
    ks = [16, 32, 48, 64, 128, 144, 256, 512, 992, 1040, 2048, 4096, 4112]
    ns = [1, 7, 8, 16, 31, 40, 64, 96, 127, 128, 257, 520, 1000, 2048, 4100, 6144]
    for _ in range(150):
        m, k, n = int(g.choice(ms)), int(g.choice(ks)), int(g.choice(ns))
        wt = g.integers(-127, 128, (n, k), dtype=np.int8)
        ws = (g.random(n, dtype=np.float32) * np.float32(1e-2) + np.float32(1e-4)).astype(np.float32)
        x = normal(g, (m, k))
        d_w = gpu.alloc(n * k + 1024, np.int8)
        _lib.check(lib.pg_mem_upload(gpu.handle, d_w.ptr, wt.ctypes.data, n * k))
        gpu.sync()
        d_ws, d_x = gpu.upload(ws), gpu.upload(x.reshape(-1))
        h = C.c_void_p()
        _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, d_w.ptr, d_ws.ptr, k, n, C.byref(h)))
        d_q, d_s = gpu.alloc(m * k + 16, np.int8), gpu.alloc(m, np.float32)
        _lib.check(lib.pg_quantize_activations(gpu.handle, d_x.ptr, m, k, d_q.ptr, d_s.ptr))
        outs = []
        for algo in (_lib.ALGO_NAIVE, _lib.ALGO_AUTO):
            d_y, d_a = gpu.alloc(m * n, np.float32), gpu.alloc(m * n, np.int32)
            _lib.check(lib.pg_gemm_i8(gpu.handle, d_q.ptr, d_s.ptr, m, k, h, d_y.ptr, d_a.ptr, algo))
            gpu.sync()
            outs.append((d_y.read(), d_a.read()))
        y_host = np.empty((m, n), np.float32)
        _lib.check(lib.pg_matmul_quantized_host(gpu.handle, x.ctypes.data, m, k, h, y_host.ctypes.data))
        assert np.array_equal(outs[0][1], outs[1][1]), (m, k, n)
        assert bits_equal(outs[0][0], outs[1][0]) and bits_equal(y_host.reshape(-1), outs[0][0]), (m, k, n)
        assert gpu.device_status() == 0
        lib.pg_qtensor_free(gpu.handle, h)
