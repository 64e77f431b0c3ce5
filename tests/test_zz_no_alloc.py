"""pg_matmul_quantized_static: the W8A8 product for callers that may not allocate device memory
(hosts with a memory budget fixed before inference starts, loops in which cudaMalloc is forbidden).

Its intermediates live in an array built into the library instead of growable context scratch, so
its output must equal pg_matmul_quantized's bit for bit.  Two calls in a row with different shapes
check that nothing depends on what the previous call left in the shared array; a context that has
served nothing but this entry point must own no scratch memory, and the device's free memory must not
move across the calls.  The file is named so that pytest collects it last."""
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


def test_static_scratch_product_allocates_nothing(gpu):
    """The property the entry point exists for.  The shapes include the two corners of its limit (M*K = 262144 with
    M = 64, and M = 256) and one of every kernel family the product can choose (decode, streaming, tcgen05)."""
    import torch

    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    lib = gpu.lib
    shapes = ((64, 4096, 256), (256, 1024, 512), (1, 4096, 4096), (16, 4096, 1024), (24, 1024, 640), (3, 80, 17))
    g = np.random.Generator(np.random.PCG64(7))
    cases = []
    for m, k, n in shapes:
        x = g.standard_normal((m, k), dtype=np.float32)
        w = (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        qt = pg.quant.quantize_weights(w, k, n, gpu)
        qt.to_gpu(gpu)
        d_x = gpu.upload(x.reshape(-1))
        d_ref, d_out = gpu.alloc(m * n, np.float32), gpu.alloc(m * n, np.float32)
        # the allocating entry on the shared context: the reference result, and every kernel is loaded before the count starts
        _lib.check(lib.pg_matmul_quantized(gpu.handle, d_x.ptr, m, k, qt._gpu, d_ref.ptr))
        cases.append((m, k, n, qt, d_x, d_ref, d_out))
    gpu.sync()
    fresh = pg.GpuContext(0)                     # has served nothing yet
    assert lib.pg_ctx_scratch_bytes(fresh.handle) == 0
    m, k, n, qt, d_x, d_ref, d_out = cases[0]
    _lib.check(lib.pg_matmul_quantized_static(fresh.handle, d_x.ptr, m, k, qt._gpu, d_out.ptr))   # the documented set-up call
    fresh.sync()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for rep in range(2):
        for m, k, n, qt, d_x, d_ref, d_out in cases:
            _lib.check(lib.pg_matmul_quantized_static(fresh.handle, d_x.ptr, m, k, qt._gpu, d_out.ptr))
            fresh.sync()
            assert _bits_equal(d_out.read(), d_ref.read()), f"M={m} K={k} N={n}"
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes across the calls"
    assert lib.pg_ctx_scratch_bytes(fresh.handle) == 0, "the context allocated scratch memory"
    assert fresh.device_status() == 0
    fresh.close()
    for c in cases:
        c[3].free_gpu()


def test_static_scratch_rejects_shapes_beyond_its_size(gpu):
    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    lib = gpu.lib
    g = np.random.Generator(np.random.PCG64(5))
    for m, k, n in ((65, 4096, 64), (257, 64, 64)):          # M*K one row past 262144; M past 256
        w = (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        qt = pg.quant.quantize_weights(w, k, n, gpu)
        qt.to_gpu(gpu)
        d_x = gpu.alloc(m * k, np.float32)
        d_y = gpu.alloc(m * n, np.float32)
        rc = lib.pg_matmul_quantized_static(gpu.handle, d_x.ptr, m, k, qt._gpu, d_y.ptr)
        assert rc == _lib.PG_ERR_UNSUPPORTED
        assert b"exceeds the built-in scratch" in lib.pg_last_error()
        qt.free_gpu()
