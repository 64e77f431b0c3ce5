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
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_column_sharded_linear(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
