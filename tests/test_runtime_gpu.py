"""Run-time behaviour of the context that is not arithmetic: bounded waits that run out, recorded graphs that outlive
a growth of the scratch memory, the wait limit as a context setting.  No test here faults, traps or hangs the GPU: the
one failure that is provoked is a flag that nobody raises, and the kernel that waits for it gives up after two
milliseconds and returns."""
import ctypes as C
import time

import numpy as np
import pytest

from _inputs import bits_equal, linear_inputs, rng

pytestmark = pytest.mark.gpu


def _product_is_exact(pg, gpu, oracle, seed):
    m, k, n = 7, 512, 200
    x, w = linear_inputs(m, k, n, seed)
    ref = oracle.quantize_weights(w, k, n)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    y = pg.quant.matmul_quantized(x, m, k, qt, gpu)
    qt.free_gpu()
    return bits_equal(y, oracle.matmul_quantized(x, m, k, ref))


def test_a_wait_that_runs_out_returns_and_leaves_the_context_usable(gpu, oracle):
    import peregrine_b200 as pg
    from peregrine_b200 import _lib
    from peregrine_b200.sharded import Exchange

    lib = gpu.lib
    _lib.check(lib.pg_ctx_set_wait_limit_ns(gpu.handle, 2_000_000))       # 2 ms
    try:
        # (1) the wait kernel: an exchange on which nothing was ever stored
        ex = Exchange(gpu, 0, 1, 4096)
        ex.connect()
        t0 = time.perf_counter()
        ex.wait()
        gpu.sync()
        assert time.perf_counter() - t0 < 0.5, "the wait did not end at its limit"
        assert gpu.device_status() == _lib.PG_ERR_DEVICE_TIMEOUT
        assert gpu.device_status() == 0                                    # reading clears it
        ex.destroy()
        # (2) a consumer with the wait inside it: two ranks in this process, only rank 0 delivers its half
        m, n = 4, 256
        exs = [Exchange(gpu, r, 2, m * n * 4) for r in range(2)]
        Exchange.connect_local(exs)
        half = gpu.upload(np.arange(m * n // 2, dtype=np.float32))
        exs[0].store_cells(half, m, n // 2, n, 0)
        d_q, d_s = gpu.alloc(m * n + 64, np.int8), gpu.alloc(m, np.float32)
        _lib.check(lib.pg_quantize_activations_exchange(gpu.handle, exs[0].handle, m, n, d_q.ptr, d_s.ptr))
        gpu.sync()
        assert gpu.device_status() == _lib.PG_ERR_DEVICE_TIMEOUT          # rank 1's flag never came
        # rank 1 delivers: the same consumer now passes without a word
        other = gpu.upload(np.arange(m * n // 2, dtype=np.float32) + 1000)
        exs[1].store_cells(other, m, n // 2, n, n // 2)
        _lib.check(lib.pg_quantize_activations_exchange(gpu.handle, exs[0].handle, m, n, d_q.ptr, d_s.ptr))
        exs[0].gather(m, n)
        gpu.sync()
        assert gpu.device_status() == 0
        full = exs[0].read(m * n).reshape(m, n)
        want = np.concatenate([np.arange(m * n // 2, dtype=np.float32).reshape(m, n // 2),
                               (np.arange(m * n // 2, dtype=np.float32) + 1000).reshape(m, n // 2)], axis=1)
        assert np.array_equal(full, want)
        qo, so = oracle.quantize_activations(want, m, n)
        assert np.array_equal(d_q.read()[: m * n].reshape(m, n), qo) and np.array_equal(d_s.read(), so)
        for e in exs:
            e.destroy()
    finally:
        _lib.check(lib.pg_ctx_set_wait_limit_ns(gpu.handle, 1_000_000_000))
    # the context went through two timeouts: its next product is still bit-exact
    assert _product_is_exact(pg, gpu, oracle, 5)
    assert lib.pg_ctx_set_wait_limit_ns(gpu.handle, 10) == _lib.PG_ERR_INVALID


def test_recorded_graph_survives_growth_of_the_scratch_memory(oracle):
    """A graph keeps the scratch address it was recorded with; a later, larger call makes the scratch grow.  The old
    block must stay alive for the graph: launching it again gives the recorded product, not a write into freed memory."""
    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    gpu = pg.GpuContext(0)                                                 # a context of its own: its scratch starts empty
    lib = gpu.lib
    m, k, n = 8, 1024, 384
    x, w = linear_inputs(m, k, n, 41)
    ref = oracle.quantize_weights(w, k, n)
    qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
    qt.to_gpu(gpu)
    want = oracle.matmul_quantized(x, m, k, ref)
    d_x, d_y = gpu.upload(x.reshape(-1)), gpu.alloc(m * n, np.float32)
    _lib.check(lib.pg_matmul_quantized(gpu.handle, d_x.ptr, m, k, qt._gpu, d_y.ptr))     # sizes the scratch
    gpu.sync()
    small = lib.pg_ctx_scratch_bytes(gpu.handle)
    with gpu.record() as graph:
        _lib.check(lib.pg_matmul_quantized(gpu.handle, d_x.ptr, m, k, qt._gpu, d_y.ptr))
    # a much larger call: the scratch has to grow while the graph is alive
    m2 = 700
    x2 = rng(42).standard_normal((m2, k), dtype=np.float32)
    d_x2, d_y2 = gpu.upload(x2.reshape(-1)), gpu.alloc(m2 * n, np.float32)
    _lib.check(lib.pg_matmul_quantized(gpu.handle, d_x2.ptr, m2, k, qt._gpu, d_y2.ptr))
    gpu.sync()
    assert lib.pg_ctx_scratch_bytes(gpu.handle) > small
    assert bits_equal(d_y2.read().reshape(m2, n), oracle.matmul_quantized(x2, m2, k, ref))
    # poison what a freed-and-reused block would look like, then replay the old graph twice
    filler = [gpu.alloc(small // 4 + 64, np.float32) for _ in range(4)]
    for it in range(2):
        _lib.check(lib.pg_mem_upload(gpu.handle, d_y.ptr, np.zeros(m * n, np.float32).ctypes.data_as(C.c_void_p), m * n * 4))
        gpu.sync()
        graph.launch()
        gpu.sync()
        assert bits_equal(d_y.read().reshape(m, n), want), f"replay {it}"
    assert gpu.device_status() == 0
    graph.free()
    del filler
    qt.free_gpu()
    gpu.close()


def test_several_exchanges_gathered_by_one_launch(gpu, oracle):
    """pg_exchange_gather_many over three exchanges of different shapes (two ranks in this process): one launch writes all
    three gathered matrices, twice in a row with new data (the second round must not be served the first round's cells),
    into the exchanges' own buffers and into caller buffers; wrong arguments are refused."""
    from peregrine_b200 import _lib
    from peregrine_b200.sharded import Exchange

    g = np.random.Generator(np.random.PCG64(9))
    shapes = [(1, 4096), (4, 520), (16, 64)]
    ranks = [[Exchange(gpu, r, 2, m * n * 4) for (m, n) in shapes] for r in range(2)]
    for i in range(len(shapes)):
        Exchange.connect_local([ranks[0][i], ranks[1][i]])
    outs = [gpu.alloc(m * n, np.float32) for (m, n) in shapes]
    for rnd in range(2):
        want = []
        for i, (m, n) in enumerate(shapes):
            full = g.standard_normal((m, n), dtype=np.float32)
            want.append(full)
            cut = (n // 2) & ~3
            for r, (c0, c1) in enumerate(((0, cut), (cut, n))):
                part = gpu.upload(np.ascontiguousarray(full[:, c0:c1]).reshape(-1))
                ranks[r][i].store_cells(part, m, c1 - c0, n, c0)
        for r in range(2):
            Exchange.gather_many(ranks[r], [m for m, _ in shapes], [n for _, n in shapes], outs if (r == 0 and rnd == 1) else None)
        gpu.sync()
        assert gpu.device_status() == 0
        for i, (m, n) in enumerate(shapes):
            for r in range(2):
                if r == 0 and rnd == 1:
                    got = outs[i].read().reshape(m, n)
                else:
                    got = ranks[r][i].read(m * n).reshape(m, n)
                assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32)), (rnd, i, r)
    # a matrix whose size is not a multiple of four, and more exchanges than one launch takes
    odd = [Exchange(gpu, r, 2, 3 * 5 * 4) for r in range(2)]
    Exchange.connect_local(odd)
    with pytest.raises(_lib.InvalidArgument, match="multiple of four"):
        Exchange.gather_many([odd[0]], [3], [5])
    with pytest.raises(_lib.InvalidArgument, match="between 0 and 16"):
        Exchange.gather_many([odd[0]] * 17, [1] * 17, [4] * 17)
    for e in odd + ranks[0] + ranks[1]:
        e.destroy()


def test_sharded_product_from_f32_activations(gpu, oracle):
    """pg_matmul_quantized_exchange over two ranks in this process: f32 activations in, gathered product out, bit for bit
    the oracle's matmul_quantized (one to sixteen rows, K split over a cluster of CTAs, a zero row, an infinite activation)."""
    import peregrine_b200 as pg
    from peregrine_b200 import _lib
    from peregrine_b200.sharded import Exchange

    lib = gpu.lib
    if True:
        for m, k, n in ((1, 4096, 256), (2, 1024, 96), (3, 14336, 128), (4, 4096, 520), (4, 65536 - 64, 64), (1, 64, 8), (5, 4096, 128), (16, 2048, 64)):
            x, w = linear_inputs(m, k, n, 60 + m + n)
            if m == 3:
                x[1] = 0.0                                   # a zero row: scale 1
                x[2, 7] = np.float32(np.inf)
            ref = oracle.quantize_weights(w, k, n)
            want = oracle.matmul_quantized(x, m, k, ref)
            exs = [Exchange(gpu, r, 2, m * n * 4) for r in range(2)]
            Exchange.connect_local(exs)
            cut = (n // 2) & ~7
            d_x = gpu.upload(x.reshape(-1))
            shards = []
            for r, (c0, c1) in enumerate(((0, cut), (cut, n))):
                sh = pg.quant.QuantizedTensor(None, np.ascontiguousarray(ref.data_i8_t[c0:c1]), np.ascontiguousarray(ref.scales[c0:c1]), k, c1 - c0)
                sh.to_gpu(gpu)
                shards.append(sh)
                tmp = gpu.alloc(m * (c1 - c0), np.float32)
                _lib.check(lib.pg_matmul_quantized_exchange(gpu.handle, d_x.ptr, m, k, sh._gpu, exs[r].handle, n, c0, tmp.ptr))
            for r in range(2):
                exs[r].gather(m, n)
            gpu.sync()
            assert gpu.device_status() == 0
            for r in range(2):
                got = exs[r].read(m * n).reshape(m, n)
                # (a row with an infinite activation is NaN throughout: which NaN a multiplication returns is the processor's choice)
                nan = np.isnan(want)
                assert np.array_equal(np.isnan(got), nan) and np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32)), (m, k, n, r)
            for sh in shards:
                sh.free_gpu()
            for e in exs:
                e.destroy()
