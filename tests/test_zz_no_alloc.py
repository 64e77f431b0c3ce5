"""pg_matmul_quantized_static: the W8A8 product for callers that may not allocate device memory
(hosts with a memory budget fixed before inference starts, loops in which cudaMalloc is forbidden).

Its intermediates live in an array built into the library instead of growable context scratch, so
its output must equal pg_matmul_quantized's bit for bit.  Two calls in a row with different shapes
check that nothing depends on what the previous call left in the shared array.  The file is named
so that pytest collects it last."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bits_equal(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_static_scratch_product_matches_allocating_product(gpu):
    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    lib = gpu.lib
    assert lib.pg_static_scratch_bytes() >= 256 * 1024
    g = np.random.Generator(np.random.PCG64(99))
    # first call: decode shape; second call: smaller M and K, so stale bytes of the first call stay in the array
    for m, k, n in ((16, 4096, 1536), (5, 1040, 333)):
        x = g.standard_normal((m, k), dtype=np.float32)
        w = (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        qt = pg.quant.quantize_weights(w, k, n, gpu)
        qt.to_gpu(gpu)
        d_x = gpu.upload(x.reshape(-1))
        d_ref, d_out = gpu.alloc(m * n, np.float32), gpu.alloc(m * n, np.float32)
        _lib.check(lib.pg_matmul_quantized(gpu.handle, d_x.ptr, m, k, qt._gpu, d_ref.ptr))
        _lib.check(lib.pg_matmul_quantized_static(gpu.handle, d_x.ptr, m, k, qt._gpu, d_out.ptr))
        ref, out = d_ref.read(), d_out.read()
        assert _bits_equal(out, ref), f"M={m} K={k} N={n}"
        qt.free_gpu()


def test_static_scratch_rejects_shapes_beyond_its_size(gpu):
    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    lib = gpu.lib
    k, n, m = 4096, 64, 65          # 65 * 4096 > 262144
    g = np.random.Generator(np.random.PCG64(5))
    w = (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    qt = pg.quant.quantize_weights(w, k, n, gpu)
    qt.to_gpu(gpu)
    d_x = gpu.alloc(m * k, np.float32)
    d_y = gpu.alloc(m * n, np.float32)
    rc = lib.pg_matmul_quantized_static(gpu.handle, d_x.ptr, m, k, qt._gpu, d_y.ptr)
    assert rc == _lib.PG_ERR_UNSUPPORTED
    assert b"exceeds the built-in scratch" in lib.pg_last_error()
    qt.free_gpu()
