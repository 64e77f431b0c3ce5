"""Runs one case of one kernel a few times, for profiling under `ncu` or quick timing.

    python profile_case.py --op w8a8 --algo stream --m 16 --k 4096 --n 32768 --reps 3
    python profile_case.py --op w8a8 --algo tcgen05 --m 2048 --k 4096 --n 4096
    python profile_case.py --op gguf --kind q4_0 --m 1 --k 4096 --n 32768
    python profile_case.py --op quant --m 8192 --k 4096
    python profile_case.py --op llama --layers 2 --m 16 --context 2048 --reps 2
    python profile_case.py --op huffman --k 4096 --n 14336 --streams 4 --reps 3
    python profile_case.py --op host --reps 1500

Inputs are seeded random values generated on the host; weights for `w8a8` are random int8 (no
quantisation pass), so start-up stays short.  Prints the mean time per call in microseconds
(host clock around a synchronised loop, adequate for kernels of tens of microseconds and up).
"""
from __future__ import annotations

import argparse
import ctypes as C
import time

import numpy as np

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from peregrine_b200 import _lib  # noqa: E402
from peregrine_b200.gguf import BLOCK_BYTES, TYPE_BY_NAME, GgufWeight  # noqa: E402
from peregrine_b200.runtime import GpuContext  # noqa: E402

ALGOS = {"auto": _lib.ALGO_AUTO, "naive": _lib.ALGO_NAIVE, "stream": _lib.ALGO_STREAM, "tcgen05": _lib.ALGO_TCGEN05, "wstream": _lib.ALGO_WSTREAM}


def llama_case(a) -> None:
    """Eager decode steps (one launch per kernel, batch = --m) of a Llama-3-8B-shaped stack cut to --layers layers."""
    import torch

    from peregrine_b200.llama import LlamaConfig, LlamaInt8Decoder

    dev = torch.device("cuda", 0)
    cfg = LlamaConfig(layers=a.layers, batch=a.m, capacity=a.context + 64)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)

    class Lazy(dict):
        """weights drawn on the device when asked for; the embedding (replicated on every rank) once"""

        emb = None

        def __getitem__(self, key):
            if key == "embedding":
                if Lazy.emb is None:
                    Lazy.emb = torch.randn(cfg.vocab, cfg.hidden, generator=gen, device=dev) * 0.02
                return Lazy.emb
            if key.endswith("norm"):
                return torch.ones(cfg.hidden, device=dev)
            shape = {"lm_head": (cfg.hidden, cfg.vocab), "qkv": (cfg.hidden, cfg.qkv_dim), "o": (cfg.hidden, cfg.hidden),
                     "gate_up": (cfg.hidden, 2 * cfg.ffn), "down": (cfg.ffn, cfg.hidden)}[key.split(".")[-1]]
            return torch.randn(*shape, generator=gen, device=dev) * 0.02

        def columns(self, key, cols):
            rows = {"lm_head": cfg.hidden, "qkv": cfg.hidden, "o": cfg.n_q_heads * cfg.head_dim, "gate_up": cfg.hidden,
                    "down": cfg.ffn}[key.split(".")[-1]]
            return torch.randn(rows, len(cols), generator=gen, device=dev) * 0.02

    gpu = GpuContext(0)
    if a.world > 1 and a.solo:
        # rank 0 of a.world alone: its kernels at the sharded shapes, recorded into one graph, nothing exchanged
        gpu.lib.pg_tune_exchange_solo(1)
        model = LlamaInt8Decoder(cfg, gpu, Lazy(), rank=0, world=a.world, connect=False)
        for e in model.ex.values():
            _lib.check(gpu.lib.pg_exchange_connect_local(gpu.handle, e.handle, None))   # solo: no peers to name
        ranks = [model]
        model.kcache[:, :, :, :a.context].normal_(generator=gen)
        model.vcache[:, :, :, :a.context].normal_(generator=gen)
        model.set_position(a.context)
        model.set_tokens(np.arange(cfg.batch) * 977 % cfg.vocab)
        model.embed()
        graph = model.record()
        for _ in range(5):
            graph.launch()
        gpu.sync()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        model.set_position(a.context)
        torch.cuda.synchronize()
        stream = torch.cuda.ExternalStream(gpu.stream)
        ev0.record(stream)
        for _ in range(a.reps):
            graph.launch()
        ev1.record(stream)
        gpu.sync()
        us = ev0.elapsed_time(ev1) / a.reps * 1e3
        print(f"op=llama layers={cfg.layers} batch={cfg.batch} context={a.context} rank 0 of {a.world} alone (no exchange): "
              f"{us:.1f} us/step from a graph of {graph.kernels} kernels")
        gpu.device_status()
        gpu.lib.pg_tune_exchange_solo(0)
        return
    if a.world > 1:
        # every rank of a column-sharded step played on this one GPU, advanced in turn launch by launch (a launch that
        # waits for the other ranks' cells is then always enqueued behind the launches that store them): the launch list
        # of such a run shows what each rank's kernels cost at the sharded shapes, without the other GPUs
        lazy = Lazy()
        ranks = [LlamaInt8Decoder(cfg, gpu, lazy, rank=r, world=a.world, connect=False) for r in range(a.world)]
        LlamaInt8Decoder.connect_local(ranks)
        for m in ranks:
            m.kcache[:, :, :, :a.context].normal_(generator=gen)
            m.vcache[:, :, :, :a.context].normal_(generator=gen)
            m.set_position(a.context)
            m.set_tokens(np.arange(cfg.batch) * 977 % cfg.vocab)
            m.embed()

        def step():
            for _ in zip(*[m.step_ops() for m in ranks]):
                pass

        model = ranks[0]
    else:
        model = LlamaInt8Decoder(cfg, gpu, Lazy())
        ranks = [model]
        model.kcache[:, :, :, :a.context].normal_(generator=gen)
        model.vcache[:, :, :, :a.context].normal_(generator=gen)
        model.set_position(a.context)
        model.set_tokens(np.arange(cfg.batch) * 977 % cfg.vocab)
        model.embed()
        step = model.enqueue_step
    step()
    gpu.sync()
    t0 = time.perf_counter()
    for _ in range(a.reps):
        step()
    gpu.sync()
    us = (time.perf_counter() - t0) / a.reps * 1e6
    status = gpu.device_status()
    print(f"op=llama layers={cfg.layers} batch={cfg.batch} context={a.context} ranks on this GPU={a.world}: {us:.1f} us/step eager, "
          f"device_status={status}")
    for m in ranks:
        m.free()
    if status != 0:
        raise SystemExit(1)


def huffman_case(a) -> None:
    """Loads a Huffman-coded [k, n] int8 weight (N(0, 0.02) quantised per column, --sparsity of it zeroed first) with
    pg_qtensor_from_huffman, beside the plain upload of the decoded bytes (pg_qtensor_from_i8).  Host clock around
    the whole call: upload from pageable memory, decode, transposition."""
    from peregrine_b200 import quant
    from peregrine_b200.huffman import HuffmanTensor, _stream_tables
    from peregrine_b200.runtime import _ptr

    gpu = GpuContext(0)
    g = np.random.Generator(np.random.PCG64(1))
    w = g.standard_normal((a.k, a.n), dtype=np.float32) * np.float32(0.02)
    if a.sparsity > 0:
        w[g.random((a.k, a.n)) < a.sparsity] = 0
    qt = quant.quantize_weights(w, a.k, a.n, gpu)
    ht = HuffmanTensor.from_quantized(qt, a.streams, limit_lengths=True)
    packed, sizes, lens = _stream_tables(ht.streams, ht.stream_lengths)

    def timed(fn):
        best = 1e9
        for _ in range(a.reps + 1):
            h = C.c_void_p()
            t0 = time.perf_counter()
            _lib.check(fn(h))
            best = min(best, time.perf_counter() - t0)
            last = h
            if _ < a.reps:
                gpu.lib.pg_qtensor_free(gpu.handle, h)
        return best * 1e3, last

    ms_h, h = timed(lambda h: gpu.lib.pg_qtensor_from_huffman(gpu.handle, _ptr(ht.table.bit_lengths), len(lens), _ptr(lens), _ptr(sizes),
                                                              _ptr(packed), _ptr(ht.scales), a.k, a.n, C.byref(h)))
    back_t, back_s = np.empty((a.n, a.k), np.int8), np.empty(a.n, np.float32)
    _lib.check(gpu.lib.pg_qtensor_download(gpu.handle, h, None, _ptr(back_t), _ptr(back_s)))
    same = np.array_equal(back_t, qt.data_i8_t)
    gpu.lib.pg_qtensor_free(gpu.handle, h)
    ms_p, h = timed(lambda h: gpu.lib.pg_qtensor_from_i8(gpu.handle, _ptr(qt.data_i8), _ptr(qt.scales), a.k, a.n, C.byref(h)))
    gpu.lib.pg_qtensor_free(gpu.handle, h)
    print(f"op=huffman k={a.k} n={a.n} streams={a.streams} sparsity={a.sparsity}: {packed.size} compressed bytes for {a.k * a.n} "
          f"(ratio {ht.compression_ratio():.3f}), from_huffman {ms_h:.2f} ms, from_i8 {ms_p:.2f} ms, identical={same}")


def host_case(a) -> None:
    """pg_matmul_quantized_host (host x in, host y out, blocking) over the nine decode cases of the benchmark, with
    page-locked buffers and each way of moving x and y: copy engines only, x read by the quantiser, y pushed by a copy
    kernel (launch by launch, and replayed from the recorded graph of a repeated call), y written by the product itself.  Microseconds per call, host clock."""
    import torch

    gpu = GpuContext(0)
    lib = gpu.lib
    g = np.random.Generator(np.random.PCG64(1))
    modes = [("copies", (0, 0, 0)), ("x direct", (1 << 20, 0, 0)), ("x direct + y pushed", (-1, -1, -1)),
             ("x direct + y pushed, replayed from a graph (default)", (-1, -1, -1)),
             ("x direct + y written by the product", (1 << 20, 1 << 20, 0))]
    total = {name: 0.0 for name, _ in modes}
    for k, n in ((4096, 4096), (4096, 14336), (14336, 4096)):
        wt = g.integers(-127, 128, n * k, dtype=np.int8)
        d_w = gpu.alloc(n * k + 1024, np.int8)
        _lib.check(lib.pg_mem_upload(gpu.handle, d_w.ptr, wt.ctypes.data, n * k))
        gpu.sync()
        d_ws = gpu.upload(np.full(n, 1e-3, np.float32))
        h = C.c_void_p()
        _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, d_w.ptr, d_ws.ptr, k, n, C.byref(h)))
        for m in (1, 4, 16):
            x = torch.randn(m, k).pin_memory()
            y = torch.empty(m, n).pin_memory()
            line = []
            for name, (bx, by, bp) in modes:
                lib.pg_tune_host_direct(bx, by)
                lib.pg_tune_host_push(bp)
                lib.pg_tune_host_graph(1 if "replayed" in name else 0)
                for _ in range(300):
                    lib.pg_matmul_quantized_host(gpu.handle, x.data_ptr(), m, k, h, y.data_ptr())
                t0 = time.perf_counter()
                for _ in range(a.reps):
                    _lib.check(lib.pg_matmul_quantized_host(gpu.handle, x.data_ptr(), m, k, h, y.data_ptr()))
                us = (time.perf_counter() - t0) / a.reps * 1e6
                total[name] += us
                line.append(f"{name} {us:.1f}")
            print(f"op=host m={m} k={k} n={n}: " + " | ".join(line), flush=True)
        lib.pg_qtensor_free(gpu.handle, h)
    lib.pg_tune_host_direct(-1, -1)
    lib.pg_tune_host_push(-1)
    lib.pg_tune_host_graph(1)
    print("sum over the nine cases, us: " + " | ".join(f"{k} {v:.1f}" for k, v in total.items()))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["w8a8", "gguf", "quant", "llama", "huffman", "host"], default="w8a8")
    ap.add_argument("--streams", type=int, default=4, help="huffman: bitstreams per tensor")
    ap.add_argument("--sparsity", type=float, default=0.0, help="huffman: share of the weights set to zero before quantisation")
    ap.add_argument("--algo", choices=list(ALGOS), default="auto")
    ap.add_argument("--kind", choices=list(TYPE_BY_NAME), default="q4_0")
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--copies", type=int, default=1, help="rotate over this many copies of the weights")
    ap.add_argument("--ng", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--pair", type=int, default=0, help="tcgen05: 0 heuristic, 1 one CTA per tile, 2 CTA pairs")
    ap.add_argument("--layers", type=int, default=2, help="llama: decoder layers (Llama-3-8B shapes otherwise)")
    ap.add_argument("--context", type=int, default=2048, help="llama: KV positions already filled")
    ap.add_argument("--solo", action="store_true", help="llama with --world: rank 0 alone, nothing exchanged (timing diagnostic)")
    ap.add_argument("--world", type=int, default=1, help="llama: ranks of a column-sharded step, all played on this one GPU")
    a = ap.parse_args()
    if a.op == "llama":
        return llama_case(a)
    if a.op == "huffman":
        return huffman_case(a)
    if a.op == "host":
        return host_case(a)

    gpu = GpuContext(0)
    lib = gpu.lib
    lib.pg_tune_stream_ng(a.ng)
    lib.pg_tune_tcgen05_bn(a.bn)
    lib.pg_tune_tcgen05_pair(a.pair)
    g = np.random.Generator(np.random.PCG64(1))
    m, k, n = a.m, a.k, a.n
    x = g.standard_normal((m, k), dtype=np.float32)
    d_x = gpu.upload(x.reshape(-1))

    if a.op == "quant":
        d_q, d_s = gpu.alloc(m * k + 16, np.int8), gpu.alloc(m, np.float32)
        call = lambda i: _lib.check(lib.pg_quantize_activations(gpu.handle, d_x.ptr, m, k, d_q.ptr, d_s.ptr))
        nbytes = 5 * m * k + 4 * m
    elif a.op == "gguf":
        bs = BLOCK_BYTES[TYPE_BY_NAME[a.kind]]
        raw = g.integers(0, 256, n * (k // 32) * bs, dtype=np.uint8)
        blocks = raw.reshape(-1, bs)
        blocks[:, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)   # a sane f16 scale
        if a.kind == "q4_1":
            blocks[:, 2:4] = np.frombuffer(np.float16(-0.08).tobytes(), np.uint8)
        ws = [GgufWeight(a.kind, raw, n, k, gpu) for _ in range(a.copies)]
        d_y = gpu.alloc(m * n, np.float32)
        call = lambda i: ws[i % a.copies].matmul_device(d_x.ptr, m, d_y.ptr)
        nbytes = n * (k // 32) * bs + 4 * m * k + 4 * m * n
    else:
        hs, keep = [], []
        for _ in range(a.copies):
            wt = g.integers(-127, 128, n * k, dtype=np.int8)
            d_w = gpu.alloc(n * k + 1024, np.int8)
            _lib.check(lib.pg_mem_upload(gpu.handle, d_w.ptr, wt.ctypes.data, n * k))
            gpu.sync()
            d_ws = gpu.upload(np.full(n, 1e-3, np.float32))
            h = C.c_void_p()
            _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, d_w.ptr, d_ws.ptr, k, n, C.byref(h)))
            hs.append(h)
            keep += [d_w, d_ws]
        d_q, d_s, d_y = gpu.alloc(m * k + 16, np.int8), gpu.alloc(m, np.float32), gpu.alloc(m * n, np.float32)
        _lib.check(lib.pg_quantize_activations(gpu.handle, d_x.ptr, m, k, d_q.ptr, d_s.ptr))
        call = lambda i: _lib.check(lib.pg_gemm_i8(gpu.handle, d_q.ptr, d_s.ptr, m, k, hs[i % a.copies], d_y.ptr, None, ALGOS[a.algo]))
        nbytes = m * k + 4 * m + k * n + 4 * n + 4 * m * n

    call(0)
    gpu.sync()
    t0 = time.perf_counter()
    for i in range(a.reps):
        call(i + 1)
    gpu.sync()
    us = (time.perf_counter() - t0) / a.reps * 1e6
    status = gpu.device_status()
    ops = 2.0 * m * n * k
    print(f"op={a.op} algo={a.algo} m={m} k={k} n={n}: {us:.1f} us/call, {nbytes / us / 1e3:.1f} GB/s algorithmic, "
          f"{ops / us / 1e6:.1f} TOPS, device_status={status}")
    if status != 0:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
