"""Host-side logic of the column-sharded linear, on CPU: world_size-2 `gloo` ranks, with the CPU
oracle standing in for the per-rank compute (the CUDA path itself is covered by the GPU tests,
including `test_column_shard_equals_slice_of_full_result`).  What is checked here: the shard plans
partition the columns, keep heads / gate-up pairs on one rank, and the all-gather reassembles a
matrix that is bit-identical to the unsharded product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from peregrine_b200 import sharded


def test_shard_bounds_and_plans():
    assert sharded.shard_bounds(10, 3) == [(0, 4), (4, 7), (7, 10)]
    assert sharded.shard_bounds(4096, 8)[-1] == (3584, 4096)
    assert sharded.shard_bounds(0, 2) == [(0, 0), (0, 0)]
    # Llama-3-8B: 32 query heads, 8 KV heads, head_dim 128 -> 6144 fused columns
    for world in (1, 2, 4, 8):
        plan = sharded.llama_qkv_columns(32, 8, 128, world)
        allc = np.sort(np.concatenate(plan))
        assert np.array_equal(allc, np.arange(6144))
        for r, cols in enumerate(plan):
            assert len(cols) == 6144 // world
            q = cols[cols < 4096] // 128
            k = (cols[(cols >= 4096) & (cols < 5120)] - 4096) // 128
            v = (cols[cols >= 5120] - 5120) // 128
            assert np.array_equal(np.unique(k), np.unique(v))            # K and V of the same heads
            assert np.array_equal(np.unique(q // 4), np.unique(k))       # query heads with their KV head
        gu = sharded.llama_gate_up_columns(14336, world)
        assert np.array_equal(np.sort(np.concatenate(gu)), np.arange(28672))
        for cols in gu:
            half = len(cols) // 2
            assert np.array_equal(cols[:half] + 14336, cols[half:])     # gate and up of the same channels
    with pytest.raises(ValueError):
        sharded.llama_qkv_columns(32, 8, 128, 3)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.pgoracle import Oracle

        orc = Oracle(mt=False)
        g = np.random.Generator(np.random.PCG64(11))
        m, k = 5, 96
        hq, hkv, hd = 8, 4, 16
        n = (hq + 2 * hkv) * hd
        x = g.standard_normal((m, k), dtype=np.float32)
        w = (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        qt = orc.quantize_weights(w, k, n)
        full = orc.matmul_quantized(x, m, k, qt)
        compute = lambda xx, mm, kk, shard: orc.matmul_quantized(xx, mm, kk, shard)
        # contiguous shards (uneven: 15 columns over 2 ranks exercises the padding)
        for cols_n in (n, 15):
            sub = sharded.take_columns(qt, np.arange(cols_n))
            lin = sharded.ColumnShardedLinear(sub, rank, world, compute=compute)
            y = lin.forward(x, m)
            assert y.shape == (m, cols_n)
            assert np.array_equal(y.view(np.uint32), full[:, :cols_n].view(np.uint32))
        # head-aware plan for the fused QKV weight
        plan = sharded.llama_qkv_columns(hq, hkv, hd, world)
        lin = sharded.ColumnShardedLinear(qt, rank, world, columns=plan, compute=compute)
        assert lin.shard.cols == n // world and lin.local(x, m).shape == (m, n // world)
        y = lin.forward(x, m)
        assert np.array_equal(y.view(np.uint32), full.view(np.uint32))
        # a plan that is not a partition is rejected
        try:
            sharded.ColumnShardedLinear(qt, rank, world, columns=[np.arange(n), np.arange(n)], compute=compute)
            raise AssertionError("overlapping plan accepted")
        except ValueError:
            pass
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_allgather_is_bit_identical(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
