"""Column-sharded W8A8 linear and column-sharded Llama decode step on two GPUs: one process per GPU, output slices
gathered by NCCL, by the separate peer-store kernels and by the products' own epilogues; every gathered result
bit-identical to the single-device oracle product / the single-GPU step.  Needs >= 2 GPUs (the same step with all
ranks played on one GPU is in test_llama_gpu.py)."""
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
        d_slice = gpu.alloc(m * (e - b), np.float32)
        d_q = gpu.alloc(m * max(k, n) + 64, np.int8)
        d_s = gpu.alloc(m, np.float32)
        for it in range(6):
            # new activations every time: a slice read stale (or a flag believed too early) would show
            xi = g.standard_normal((m, k), dtype=np.float32)
            want = orc.matmul_quantized(xi, m, k, ref)
            d_x = gpu.upload(xi.reshape(-1))
            ex = exs[it & 1]
            if it < 3:
                # separate kernels: product, copy into every rank, wait
                _lib.check(gpu.lib.pg_matmul_quantized(gpu.handle, d_x.ptr, m, k, shard._gpu, d_slice.ptr))
                ex.allgather(d_slice, m, e - b, b)
            else:
                # the product's own epilogue stores flagged cells into every rank
                if it == 4:
                    # f32 activations in: quantiser and product with the exchange in one call
                    _lib.check(gpu.lib.pg_matmul_quantized_exchange(gpu.handle, d_x.ptr, m, k, shard._gpu, ex.handle, n, b, d_slice.ptr))
                else:
                    _lib.check(gpu.lib.pg_quantize_activations(gpu.handle, d_x.ptr, m, k, d_q.ptr, d_s.ptr))
                    _lib.check(gpu.lib.pg_gemm_i8_exchange(gpu.handle, d_q.ptr, d_s.ptr, m, k, shard._gpu, ex.handle, n, b, None))
                # consumers with the wait inside: quantise the gathered rows; write them out as plain floats
                _lib.check(gpu.lib.pg_quantize_activations_exchange(gpu.handle, ex.handle, m, n, d_q.ptr, d_s.ptr))
                if it == 5:
                    sharded.Exchange.gather_many([ex], [m], [n])      # the batched form of the same consumer
                else:
                    ex.gather(m, n)
            y = ex.read(m)
            assert gpu.device_status() == 0
            assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), f"exchange {it}"
            if it >= 3:
                qo, so = orc.quantize_activations(want, m, n)
                assert np.array_equal(d_q.read()[: m * n].reshape(m, n), qo) and np.array_equal(d_s.read(), so)
            dist.barrier()          # the next round reuses the buffer the other rank may still be reading
        _sharded_llama(rank, world, gpu)
        dist.barrier()
        for ex in exs:
            ex.destroy()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def _sharded_llama(rank, world, gpu):
    """Three decode steps (one eager, two replayed from the recorded graph) of a small Llama, heads / channels / columns
    split over the ranks, against the same step on this GPU alone: bit-identical logits, tokens and caches."""
    import torch.distributed as dist

    from peregrine_b200.llama import LlamaConfig, LlamaInt8Decoder

    cfg = LlamaConfig(layers=2, hidden=1024, n_q_heads=16, n_kv_heads=4, head_dim=128, ffn=2048, vocab=4096, batch=16, capacity=300)
    g = np.random.Generator(np.random.PCG64(31))
    nrm = lambda shape, s: (g.standard_normal(shape, dtype=np.float32) * np.float32(s)).astype(np.float32)
    W = {"embedding": nrm((cfg.vocab, cfg.hidden), 0.5), "final_norm": (1 + nrm((cfg.hidden,), 0.1)).astype(np.float32),
         "lm_head": nrm((cfg.hidden, cfg.vocab), 0.02)}
    for i in range(cfg.layers):
        W[f"l{i}.attn_norm"] = (1 + nrm((cfg.hidden,), 0.1)).astype(np.float32)
        W[f"l{i}.ffn_norm"] = (1 + nrm((cfg.hidden,), 0.1)).astype(np.float32)
        W[f"l{i}.qkv"] = nrm((cfg.hidden, cfg.qkv_dim), 0.05)
        W[f"l{i}.o"] = nrm((cfg.n_q_heads * cfg.head_dim, cfg.hidden), 0.05)
        W[f"l{i}.gate_up"] = nrm((cfg.hidden, 2 * cfg.ffn), 0.05)
        W[f"l{i}.down"] = nrm((cfg.ffn, cfg.hidden), 0.05)
    start = 200
    K = [nrm((cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim), 1.0) for _ in range(cfg.layers)]
    V = [nrm((cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim), 1.0) for _ in range(cfg.layers)]
    tokens = g.integers(0, cfg.vocab, cfg.batch).astype(np.int32)

    def prime(m):
        for i in range(cfg.layers):
            m.load_cache(i, K[i], V[i])
        m.set_position(start)
        m.set_tokens(tokens)
        torch.cuda.synchronize()
        m.embed()
        gpu.sync()

    one = LlamaInt8Decoder(cfg, gpu, W, device_index=rank)
    prime(one)
    ref = []
    for _ in range(3):
        one.enqueue_step()
        gpu.sync()
        ref.append((one.logits.cpu().numpy().copy(), one.tokens.cpu().numpy().copy()))
    ref_k = one.kcache.cpu().numpy().copy()
    one.free()
    model = LlamaInt8Decoder(cfg, gpu, W, device_index=rank, rank=rank, world=world, attn_splits="match")
    prime(model)
    lo_, hi_ = rank * model.v_l, (rank + 1) * model.v_l
    graph = None
    for step in range(3):
        if step == 0:
            model.enqueue_step()
        else:
            if graph is None:
                graph = model.record()
            graph.launch()
        gpu.sync()
        assert gpu.device_status() == 0
        logits, toks = ref[step]
        assert np.array_equal(model.logits.cpu().numpy().view(np.uint32), logits[:, lo_:hi_].view(np.uint32)), f"step {step}"
        assert np.array_equal(model.tokens.cpu().numpy(), toks)
        dist.barrier()
    klo, khi = rank * model.hkv_l, (rank + 1) * model.hkv_l
    assert np.array_equal(model.kcache.cpu().numpy(), ref_k[:, :, klo:khi])
    graph.free()
    model.free()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_column_sharded_linear(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
