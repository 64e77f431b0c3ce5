"""Column-sharded W8A8 linear on two GPUs: one process per GPU, NCCL all-gather of the output
slices, result bit-identical to the single-device oracle product.  Needs >= 2 GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import peregrine_b200 as pg
        from oracle.pgoracle import Oracle
        from peregrine_b200 import sharded

        gpu = pg.GpuContext(rank)
        orc = Oracle(mt=True)
        g = np.random.Generator(np.random.PCG64(21))
        m, k = 16, 4096
        hq, hkv, hd = 32, 8, 128
        n = (hq + 2 * hkv) * hd
        x = g.standard_normal((m, k), dtype=np.float32)
        w = (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        ref = orc.quantize_weights(w, k, n)
        full = orc.matmul_quantized(x, m, k, ref)
        qt = pg.quant.QuantizedTensor(ref.data_i8, ref.data_i8_t, ref.scales, k, n)
        for plan in (None, sharded.llama_qkv_columns(hq, hkv, hd, world)):
            lin = sharded.ColumnShardedLinear(qt, rank, world, columns=plan, gpu=gpu)
            y = lin.forward(x, m)
            assert np.array_equal(y.view(np.uint32), full.view(np.uint32))
        # the same product with the peer-store all-gather: slices computed on the device, stored into every
        # rank's result buffer over NVLink, two exchanges in a row on the same object pair
        from peregrine_b200 import _lib

        b, e = sharded.shard_bounds(n, world)[rank]
        shard = pg.quant.QuantizedTensor(None, np.ascontiguousarray(ref.data_i8_t[b:e]), np.ascontiguousarray(ref.scales[b:e]), k, e - b)
        shard.to_gpu(gpu)
        exs = [sharded.PeerExchange(gpu, rank, world, m, n) for _ in range(2)]
        d_x = gpu.upload(x.reshape(-1))
        d_slice = gpu.alloc(m * (e - b), np.float32)
        for it in range(4):
            ex = exs[it & 1]
            _lib.check(gpu.lib.pg_matmul_quantized(gpu.handle, d_x.ptr, m, k, shard._gpu, d_slice.ptr))
            ex.allgather(d_slice, m, e - b, b)
            y = ex.read(m)
            assert gpu.device_status() == 0
            assert np.array_equal(y.view(np.uint32), full.view(np.uint32)), f"exchange {it}"
        dist.barrier()
        for ex in exs:
            ex.destroy()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_column_sharded_linear(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
