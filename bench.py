#!/usr/bin/env python
"""Benchmark of the W8A8 decode path (quant::matmul_quantized at M <= 16) on B200.

Workload: the decode GEMV sweep -- M in {1,4,16} x (K,N) in {(4096,4096),(4096,14336),(14336,4096)}
(Llama-3-8B projection shapes), activations ~N(0,1) with 1 % of channels scaled x20, weights
~N(0,0.02) quantised per column to i8.  One "step" is one pass over the nine cases:
per case, per-row activation quantisation followed by the int8 product and the scale epilogue.

Metric: achieved HBM bandwidth in GB/s = algorithmic bytes of the sweep / time, with
  bytes(M,K,N) = 4*M*K (x f32) + K*N (weights i8) + 4*N (scales) + 4*M*N (y f32).

    python bench.py --gpus N --steps K --warmup W            this library
    python bench.py --impl reference ...                     the reference's CPU algorithm (C port)

With N > 1 (one process per GPU, torchrun) the weights are sharded by output column over the ranks: one
sweep, every rank quantises the (replicated) activations and computes its columns, and the products' own
epilogues store the slices into every rank's result buffer over NVLink (`--collective nccl`: eager NCCL
all-gathers instead); `scaling: strong`, `value` is the sweep's bytes over the slowest rank's time.  The
same line carries the column-sharded Llama-3-8B-shape decode stack (`also.llama8b_int8_decode`).
`--parallel replicas` runs the other layout, labelled as what it is: a full copy of the weights and an
own sweep per GPU, no collective (`scaling: weak`).

Cache discipline: every case of a step reads its own copy of the weights (three copies per shape,
402 MB in total), so a weight matrix is re-read only after ~400 MB of other traffic (L2 is 126 MB).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]
MS = [1, 4, 16]
# order of a step: all shapes at M=1, then M=4, then M=16; case index = position in BASELINE's sweep
CASES = [(mi, si) for mi in range(3) for si in range(3)]
L2_BYTES = 126 * 1024 * 1024


def bytes_w8a8(m, k, n):
    return 4 * m * k + k * n + 4 * n + 4 * m * n


def bytes_gemv_kernel(m, k, n):
    """The product kernel alone: quantised activations in (i8 + scales) instead of f32."""
    return m * k + 4 * m + k * n + 4 * n + 4 * m * n


def sweep_bytes():
    return sum(bytes_w8a8(MS[mi], *SHAPES[si]) for mi, si in CASES)


def make_inputs(case_idx, m, k):
    g = np.random.Generator(np.random.PCG64(1000 + case_idx))
    x = g.standard_normal((m, k), dtype=np.float32)
    ch = g.choice(k, size=int(np.ceil(0.01 * k)), replace=False)
    x[:, ch] *= np.float32(20.0)
    return x


RESULT_OUT = sys.stdout
WORKLOAD = {"workload": "decode_gemv_sweep M{1,4,16} x (K,N){(4096,4096),(4096,14336),(14336,4096)}", "cases": 9}


def make_weight(shape_idx, k, n):
    g = np.random.Generator(np.random.PCG64(7000 + shape_idx))
    return (g.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)


# --------------------------------------------------------------------- clocks ----
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        self.t_mark = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def mark(self):
        self.t_mark = time.time()

    def stop(self, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "nvidia-smi unavailable"}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for t, r in self.rows if self.t_mark is not None and self.t_mark <= t <= t_end + 0.06]
        window = "timed region"
        if not inside:
            inside = [r for _, r in self.rows[-4:]]
            window = "timed region shorter than the sampling period: last samples under load (warm-up + timed)"
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            p = [c.strip() for c in r.split(",")]
            if len(p) < 8:
                continue
            try:
                sm.append(float(p[0]))
                smax.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(names, p[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


# ------------------------------------------------------------ reference (CPU) ----
def run_reference(args):
    """The reference's algorithm for this path (scalar branch of src/quant.rs, C port) on the host
    cores.  The reference itself runs this path on one thread; here every output element is an
    independent OpenMP task, so all cores are used and the result is unchanged."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if "LOCAL_RANK" in os.environ and os.environ.get("OMP_NUM_THREADS") == "1":
        # torch.distributed.run gives every rank one OpenMP thread unless told otherwise; the other ranks of this arm do no
        # work, so rank 0 takes the host's cores (the setting is read when the OpenMP library loads, below)
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    from oracle.pgoracle import Oracle

    orc = Oracle(mt=True)
    qts = []
    for si, (k, n) in enumerate(SHAPES):
        qts.append(orc.quantize_weights(make_weight(si, k, n), k, n))
    xs = [make_inputs(ci, MS[mi], SHAPES[si][0]) for ci, (mi, si) in enumerate(CASES)]

    from oracle.pgoracle import QuantizedTensor

    def make_step(frac):
        part = []
        for qt in qts:
            nf = max(1, int(qt.cols * frac))
            part.append(QuantizedTensor(qt.data_i8, np.ascontiguousarray(qt.data_i8_t[:nf]), np.ascontiguousarray(qt.scales[:nf]), qt.rows, nf))

        def step():
            for ci, (mi, si) in enumerate(CASES):
                orc.matmul_quantized(xs[ci], MS[mi], SHAPES[si][0], part[si])

        return step, sum(bytes_w8a8(MS[mi], SHAPES[si][0], part[si].cols) for mi, si in CASES)

    # A step is one pass over the sweep; when K passes would not finish in about 90 s, each step
    # covers the same leading fraction of every case's output columns (columns are independent).
    step, nbytes = make_step(1.0)
    t0 = time.perf_counter()
    step()
    t_full = time.perf_counter() - t0
    frac = 1.0
    budget = 90.0 / max(args.steps + args.warmup, 1)
    if t_full > budget:
        frac = max(budget / t_full, 1.0 / 64)
        step, nbytes = make_step(frac)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = nbytes * args.steps / dt / 1e9
    sample = (f"{args.steps} passes of the nine-case sweep" if frac == 1.0 else
              f"{args.steps} passes over the first {frac:.4f} of each case's output columns (full pass takes {t_full * 1e3:.0f} ms)")
    line = {
        "impl": "reference", "metric": "w8a8_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        # the host's throughput does not depend on how many sweeps it is given: the label follows the GPU arm's layout
        "scaling": "weak" if (args.gpus > 1 and args.parallel == "replicas") else "strong", "vs_baseline": None, "dtype": "i8",
        "data": "synthetic",
        "config": dict(WORKLOAD),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": orc.threads, "kind": "port",
                         "sample": sample + "; OpenMP over independent outputs (the reference itself runs this path on one thread)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=RESULT_OUT, flush=True)


# -------------------------------------------------------------------- our arm ----
def run_ours(args):
    import torch
    import torch.distributed as dist

    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.Stream(device=dev)
    gpu = pg.GpuContext(local, stream.cuda_stream)
    lib = gpu.lib
    if world > 1:
        # a flag that another rank raises arrives within microseconds; a rank that waits a tenth of a second for one has lost
        # its peer, and the run should end with the status word set rather than wait a second per kernel
        _lib.check(lib.pg_ctx_set_wait_limit_ns(gpu.handle, 100_000_000))
    warmup = max(args.warmup, 3)
    # N > 1: "shard" splits every weight matrix by output column over the ranks and all-gathers the slices (strong
    # scaling of one sweep); "replicas" gives every rank the whole matrices and its own copy of the sweep, with no
    # data-path collective (weak scaling: what a server does with independent batches when the model fits one GPU)
    replicas = world > 1 and args.parallel == "replicas"
    sw, srank = (1, 0) if replicas else (world, rank)

    # ---- weights: quantise on the GPU, keep this rank's column shard, three copies per shape ----
    COPIES = 3
    pool = []      # pool[si][c] = (pg_qtensor handle, torch tensors kept alive)
    shard = []
    for si, (k, n) in enumerate(SHAPES):
        w = make_weight(si, k, n)
        qt = pg.quant.quantize_weights(w, k, n, gpu)
        b, e = (n * srank) // sw, (n * (srank + 1)) // sw
        shard.append((b, e))
        t_w = torch.from_numpy(np.ascontiguousarray(qt.data_i8_t[b:e])).to(dev)
        t_s = torch.from_numpy(np.ascontiguousarray(qt.scales[b:e])).to(dev)
        copies = []
        for c in range(COPIES):
            # 1 KiB of slack after the weights keeps tiled loads of the last rows inside the allocation
            buf = torch.empty(t_w.numel() + 1024, dtype=torch.int8, device=dev)
            buf[: t_w.numel()].copy_(t_w.view(-1))
            sc = t_s.clone()
            h = _lib.C.c_void_p()
            _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, buf.data_ptr(), sc.data_ptr(), k, e - b, _lib.C.byref(h)))
            copies.append((h, buf, sc))
        pool.append(copies)
        del w, qt
    torch.cuda.synchronize()

    xs_host = [torch.from_numpy(make_inputs(ci, MS[mi], SHAPES[si][0])).pin_memory() for ci, (mi, si) in enumerate(CASES)]
    xs = [x.to(dev) for x in xs_host]
    ys = [torch.empty(MS[mi], shard[si][1] - shard[si][0], dtype=torch.float32, device=dev) for mi, si in CASES]
    ys_full = [torch.empty(sw, MS[mi], shard[si][1] - shard[si][0], dtype=torch.float32, device=dev) if sw > 1 else None
               for mi, si in CASES]
    ys_host = [torch.empty(MS[mi], SHAPES[si][1], dtype=torch.float32).pin_memory() for mi, si in CASES]
    even = all(SHAPES[si][1] % sw == 0 for si in range(3))
    if sw > 1 and not even:
        raise SystemExit("column shards must be equal for the all-gather")

    from peregrine_b200.sharded import PeerExchange

    peer = sw > 1 and args.collective == "peer"
    exs = [PeerExchange(gpu, rank, world, MS[mi], SHAPES[si][1]) for mi, si in CASES] if peer else None
    qs = [torch.empty(MS[mi] * SHAPES[si][0] + 64, dtype=torch.int8, device=dev) for mi, si in CASES] if peer else None
    qss = [torch.empty(MS[mi], dtype=torch.float32, device=dev) for mi, si in CASES] if peer else None

    def enqueue_products():
        for ci, (mi, si) in enumerate(CASES):
            k, n = SHAPES[si]
            h = pool[si][mi][0]
            if peer:
                # the product's own epilogue stores this rank's columns into every rank's [M, N] buffer over NVLink and
                # publishes the exchange: no all-gather launch
                _lib.check(lib.pg_matmul_quantized_exchange(gpu.handle, xs[ci].data_ptr(), MS[mi], k, h, exs[ci].handle, n, shard[si][0],
                                                            ys[ci].data_ptr()))
            else:
                _lib.check(lib.pg_matmul_quantized(gpu.handle, xs[ci].data_ptr(), MS[mi], k, h, ys[ci].data_ptr()))
        if peer:
            # the nine products of the sweep are independent, so the consumers (bounded waits for the other ranks' cells,
            # results written out as plain [M, N] matrices) come after the last product: the step ends when every rank
            # holds all nine full results
            # -- collected by ONE launch
            PeerExchange.gather_many(exs, [MS[mi] for mi, si in CASES], [SHAPES[si][1] for mi, si in CASES])

    def step_eager():
        if peer:
            return enqueue_products()
        for ci, (mi, si) in enumerate(CASES):
            k, _ = SHAPES[si]
            h = pool[si][mi][0]
            _lib.check(lib.pg_matmul_quantized(gpu.handle, xs[ci].data_ptr(), MS[mi], k, h, ys[ci].data_ptr()))
            if sw > 1:
                dist.all_gather_into_tensor(ys_full[ci], ys[ci])

    n0 = lib.pg_launch_count()
    with torch.cuda.stream(stream):
        step_eager()
    stream.synchronize()
    launches_per_step = int(lib.pg_launch_count() - n0)
    st = gpu.device_status()
    if st != 0:
        raise SystemExit(f"rank {rank}: device status {st} after the first step (a bounded wait ran out): not measuring")

    # One submission per step at N = 1 (the library's own graph recorder).  With NCCL in the step the
    # launches stay eager: replaying a captured step that contained the all-gathers did not complete
    # on this pool, so that form is not used.
    graph = None
    if sw == 1 or peer:
        if world > 1:
            dist.barrier()
        with gpu.record() as graph:
            enqueue_products()

    def step():
        if graph is not None:
            graph.launch()
        else:
            step_eager()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: exactly K steps, device time, max over ranks ----
    sampler = ClockSampler(local) if rank == 0 else None
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.mark()
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        barrier()
    t_end = time.time()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_end) if sampler else None
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total_bytes = sweep_bytes() * (world if replicas else 1)   # every replica runs the whole sweep
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9
    assert gpu.device_status() == 0

    # ---- end to end: host buffers in, host result out, every step ----
    e2e_steps = min(args.steps, 2000)
    h2d = sum(4 * MS[mi] * SHAPES[si][0] for mi, si in CASES)
    d2h = sum(4 * MS[mi] * SHAPES[si][1] for mi, si in CASES)

    def e2e_step():
        for ci, (mi, si) in enumerate(CASES):
            k, n = SHAPES[si]
            h = pool[si][mi][0]
            if sw == 1:
                # the C-ABI call with the exact shape of quant::matmul_quantized: copies x up, runs, copies y back, blocks
                _lib.check(lib.pg_matmul_quantized_host(gpu.handle, xs_host[ci].data_ptr(), MS[mi], k, h, ys_host[ci].data_ptr()))
            else:
                xs[ci].copy_(xs_host[ci], non_blocking=True)
                _lib.check(lib.pg_matmul_quantized(gpu.handle, xs[ci].data_ptr(), MS[mi], k, h, ys[ci].data_ptr()))
                if peer:
                    _lib.check(lib.pg_quantize_activations(gpu.handle, xs[ci].data_ptr(), MS[mi], k, qs[ci].data_ptr(), qss[ci].data_ptr()))
                    _lib.check(lib.pg_gemm_i8_exchange(gpu.handle, qs[ci].data_ptr(), qss[ci].data_ptr(), MS[mi], k, h, exs[ci].handle, n,
                                                       shard[si][0], ys[ci].data_ptr()))
                    exs[ci].gather(MS[mi], n)
                    _lib.check(lib.pg_mem_download(gpu.handle, ys_host[ci].data_ptr(), exs[ci].result_ptr, MS[mi] * n * 4))
                else:
                    dist.all_gather_into_tensor(ys_full[ci], ys[ci])
                    ys_host[ci].view(MS[mi], sw, -1).copy_(ys_full[ci].permute(1, 0, 2), non_blocking=True)
                    stream.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = total_bytes * e2e_steps / e2e_s / 1e9

    line = None
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"

        # ---- roofline of the dominant kernel (the int8 product): kernel-only replay of the nine launches
        d_q, d_s = [], []
        with torch.cuda.stream(stream):
            for ci, (mi, si) in enumerate(CASES):
                k = SHAPES[si][0]
                q = torch.empty(MS[mi] * k + 16, dtype=torch.int8, device=dev)
                s = torch.empty(MS[mi], dtype=torch.float32, device=dev)
                _lib.check(lib.pg_quantize_activations(gpu.handle, xs[ci].data_ptr(), MS[mi], k, q.data_ptr(), s.data_ptr()))
                d_q.append(q)
                d_s.append(s)

            def products_only():
                for ci, (mi, si) in enumerate(CASES):
                    k = SHAPES[si][0]
                    _lib.check(lib.pg_gemm_i8(gpu.handle, d_q[ci].data_ptr(), d_s[ci].data_ptr(), MS[mi], k, pool[si][mi][0],
                                              ys[ci].data_ptr(), None, _lib.ALGO_AUTO))

            products_only()
            with gpu.record() as g2:
                products_only()
            for _ in range(5):
                g2.launch()
            reps = max(20, min(args.steps, 2000))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g2.launch()
            e1.record(stream)
            stream.synchronize()
        k_ms = e0.elapsed_time(e1) / reps
        kern_bytes = sum(bytes_gemv_kernel(MS[mi], SHAPES[si][0], shard[si][1] - shard[si][0]) for mi, si in CASES)
        achieved = kern_bytes / (k_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "gemv_wstream_kernel", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                    "frac": achieved / hbm_peak,
                    # DRAM bytes (read + write) of this kernel under ncu: 139.3 MB for 136.5 MB algorithmic at K 4096,
                    # N 32768, M 16 (1.02 x), and 58.9 MB for 59.8 MB at K 4096, N 14336, M 16, a case of this sweep
                    # (0.99 x: part of y is still in L2 when the kernel ends).  The larger ratio, scaled by the bytes an
                    # average launch of the sweep moves (traffic grows in proportion to K * N)
                    "traffic": 1.02 * kern_bytes / 9,
                    "traffic_source": "ncu captures of gemv_wstream_kernel (profiles/), ratio to algorithmic bytes 0.99-1.02, scaled",
                    "peak_source": peak_src,
                    "bytes_per_launch_avg": kern_bytes / 9, "us_per_launch_avg": k_ms * 1e3 / 9,
                    "how": f"{reps} replays of a graph holding only the nine product launches, CUDA events on the launch stream"}

        # ---- CPU baseline: the oracle's single-thread port (what the reference runs), bounded sample
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            from oracle.pgoracle import Oracle

            orc = Oracle(mt=False)
            qts = [orc.quantize_weights(make_weight(si, k, n), k, n) for si, (k, n) in enumerate(SHAPES)]
            xn = [x.numpy() for x in xs_host]
            passes = 0
            t0 = time.perf_counter()
            while passes < 2 or (time.perf_counter() - t0 < 10.0 and passes < 8):
                for ci, (mi, si) in enumerate(CASES):
                    orc.matmul_quantized(xn[ci], MS[mi], SHAPES[si][0], qts[si])
                passes += 1
            dt = time.perf_counter() - t0
            cpu = {"value": total_bytes * passes / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                   "sample": f"{passes} full passes of the nine-case sweep, single thread (the reference's quant path is single-threaded)",
                   "ms_per_step": dt / passes * 1e3, "host_cpus": os.cpu_count()}

        line = {
            "metric": "w8a8_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak" if replicas else "strong",
            "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "config": dict(WORKLOAD),
            "config_detail": {
                "parallelism": (f"{world} replicas, one sweep each, no collective" if replicas else
                                f"column-sharded x{world}" + ((", slices stored into every rank by the product's epilogue over NVLink as flagged cells; the nine gathered results collected by one launch at the end of the step (bounded waits)"
                                                               if peer else ", NCCL all-gather of output slices") if world > 1 else "")),
                "l2": "inputs larger than L2: each case reads its own copy of the weights (3 copies per shape, 402 MB per step)",
                "submission": "one CUDA graph per step" if graph is not None else "eager launches + NCCL",
                "collective": ("peer-store (fused)" if peer else "nccl") if sw > 1 else None,
                "bytes_per_step": total_bytes},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_s / e2e_steps * 1e3,
                    "api": "pg_matmul_quantized_host (pinned host x in, host y out, blocking)" if sw == 1 else
                           "pinned H2D + pg_matmul_quantized + all-gather + D2H of the full result"},
            "gpu_launches": launches_per_step * args.steps,
            "kernels_per_step": launches_per_step,
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        if world == 1 and not args.no_extra:
            line["also"] = extra_measurements(gpu, torch, stream, dev, hbm_peak, peaks)
    # The Llama-3-8B-shape decode stack: on one GPU; column-sharded over the ranks (one model, one batch of 16 sequences);
    # or (replicas) one full model and one batch per GPU
    if not args.no_llama:
        peak_l = 6532.9
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak_l = float(json.load(f).get("hbm_gbs", peak_l))
        except (OSError, ValueError):
            pass
        if world > 1 and not replicas:
            ll = llama_decode_measurement(gpu, torch, stream, dev, peak_l, rank=rank, world=world)
            t = torch.tensor([ll["ms_per_step"], ll["e2e_ms_per_step"]], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ll["ms_per_step"], ll["e2e_ms_per_step"] = float(t[0].item()), float(t[1].item())
            ll["tok_s"] = ll["batch"] * 1e3 / ll["ms_per_step"]
            ll["e2e_tok_s"] = ll["batch"] * 1e3 / ll["e2e_ms_per_step"]
            # bytes of one step over all ranks (every rank reads its shard of the weights and of the KV cache)
            ll["bytes_per_step"] *= world
            ll["hbm_gbs"] = ll["bytes_per_step"] / (ll["ms_per_step"] * 1e-3) / 1e9
            ll["frac_of_measured_hbm"] = ll["hbm_gbs"] / (world * peak_l)
            ll["parallelism"] = (f"column-sharded x{world}: heads / gate-up channels / O, down and vocabulary columns per rank, four exchanges per "
                                 "layer stored by the producing kernels, awaited by the consuming ones")
        else:
            ll = llama_decode_measurement(gpu, torch, stream, dev, peak_l)
        if world > 1 and replicas:
            # whole-job tokens per second: all replicas' tokens over the slowest replica's time
            t = torch.tensor([ll["ms_per_step"]], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ll["ms_per_step"] = float(t.item())
            ll["tok_s"] = world * ll["batch"] * 1e3 / ll["ms_per_step"]
            ll["replicas"] = world
            ll["hbm_gbs"] = world * ll["bytes_per_step"] / (ll["ms_per_step"] * 1e-3) / 1e9
            ll["frac_of_measured_hbm"] = ll["hbm_gbs"] / (world * peak_l)
            t = torch.tensor([ll["e2e_tok_s"]], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            ll["e2e_tok_s"] = float(t.item())
        if rank == 0:
            line.setdefault("also", {})["llama8b_int8_decode"] = ll
    if world > 1:
        dist.barrier()
        if exs:
            for ex in exs:
                ex.destroy()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), file=RESULT_OUT, flush=True)


def extra_measurements(gpu, torch, stream, dev, hbm_peak, peaks):
    """Secondary figures of the same path: prefill GEMM TOPS, GGUF dequant-product GB/s, Huffman-coded weight load."""
    import peregrine_b200 as pg
    from peregrine_b200 import _lib

    lib = gpu.lib
    out = {}
    g = np.random.Generator(np.random.PCG64(2002))
    bf16 = float(peaks.get("bf16_tflops", 1590.0))
    with torch.cuda.stream(stream):
        # the single linear of the first benchmark config: M 32, K = N = 4096, seed 0, quantiser + product; eight copies of the
        # weights (134 MB) walked in one graph so that no copy is found in L2
        m, k, n = 32, 4096, 4096
        g0 = np.random.Generator(np.random.PCG64(0))
        x = torch.from_numpy(g0.standard_normal((m, k), dtype=np.float32)).to(dev)
        w0 = (g0.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        qt0 = pg.quant.quantize_weights(w0, k, n, gpu)
        t_w = torch.from_numpy(qt0.data_i8_t).to(dev)
        t_s = torch.from_numpy(qt0.scales).to(dev)
        copies = []
        for _ in range(8):
            buf = torch.empty(t_w.numel() + 1024, dtype=torch.int8, device=dev)
            buf[: t_w.numel()].copy_(t_w.view(-1))
            h = _lib.C.c_void_p()
            _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, buf.data_ptr(), t_s.data_ptr(), k, n, _lib.C.byref(h)))
            copies.append((h, buf))
        y = torch.empty(m, n, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        for h, _ in copies:
            _lib.check(lib.pg_matmul_quantized(gpu.handle, x.data_ptr(), m, k, h, y.data_ptr()))
        with gpu.record() as gg:
            for h, _ in copies:
                _lib.check(lib.pg_matmul_quantized(gpu.handle, x.data_ptr(), m, k, h, y.data_ptr()))
        gg.launch()
        reps = 50
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            gg.launch()
        e1.record(stream)
        stream.synchronize()
        gg.free()
        us = e0.elapsed_time(e1) / (reps * len(copies)) * 1e3
        gbs = bytes_w8a8(m, k, n) / (us * 1e-6) / 1e9
        out["w8a8_linear_M32_K4096_N4096_seed0"] = {"us": us, "gbs": gbs, "frac_of_measured_hbm": gbs / hbm_peak,
                                                    "tops": 2.0 * m * n * k / (us * 1e-6) / 1e12}
        for h, _ in copies:
            lib.pg_qtensor_free(gpu.handle, h)
        del copies, x, y, t_w
        # the six prefill shapes, with the kernel the library chooses by itself
        for (m, k, n) in ((512, 4096, 4096), (512, 4096, 14336), (2048, 4096, 4096), (2048, 4096, 14336), (8192, 4096, 4096),
                          (8192, 4096, 14336)):
            x = torch.from_numpy(g.standard_normal((m, k), dtype=np.float32)).to(dev)
            wq = torch.randint(-127, 128, (n * k + 1024,), dtype=torch.int8, device=dev)
            sc = torch.rand(n, dtype=torch.float32, device=dev) * 1e-3
            h = _lib.C.c_void_p()
            _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, wq.data_ptr(), sc.data_ptr(), k, n, _lib.C.byref(h)))
            y = torch.empty(m, n, dtype=torch.float32, device=dev)
            q = torch.empty(m * k + 16, dtype=torch.int8, device=dev)
            s = torch.empty(m, dtype=torch.float32, device=dev)
            _lib.check(lib.pg_quantize_activations(gpu.handle, x.data_ptr(), m, k, q.data_ptr(), s.data_ptr()))
            for _ in range(3):
                _lib.check(lib.pg_gemm_i8(gpu.handle, q.data_ptr(), s.data_ptr(), m, k, h, y.data_ptr(), None, _lib.ALGO_AUTO))
            reps = 20
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                _lib.check(lib.pg_gemm_i8(gpu.handle, q.data_ptr(), s.data_ptr(), m, k, h, y.data_ptr(), None, _lib.ALGO_AUTO))
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) / reps * 1e3
            tops = 2.0 * m * n * k / (us * 1e-6) / 1e12
            out[f"w8a8_gemm_M{m}_K{k}_N{n}"] = {"us": us, "tops": tops, "frac_of_2x_measured_bf16": tops / (2 * bf16),
                                                  "frac_of_4500_nominal": tops / 4500.0}
            lib.pg_qtensor_free(gpu.handle, h)
            del x, wq, y, q
    # per-shape table of the decode and mid-batch products (quantiser + product, the library's own kernel choice): every
    # shape with enough copies of its weights (>= 134 MB) walked in one graph, so that no copy is found in L2
    table = {}
    with torch.cuda.stream(stream):
        for (k, n) in SHAPES:
            ncopies = max(3, -(-134_000_000 // (k * n)))
            sc = torch.rand(n, dtype=torch.float32, device=dev) * 1e-3
            copies = []
            for _ in range(ncopies):
                wq = torch.randint(-127, 128, (n * k + 1024,), dtype=torch.int8, device=dev)
                h = _lib.C.c_void_p()
                _lib.check(lib.pg_qtensor_wrap(gpu.handle, None, wq.data_ptr(), sc.data_ptr(), k, n, _lib.C.byref(h)))
                copies.append((h, wq))
            for m in (1, 4, 16, 17, 64, 128):
                x = torch.from_numpy(g.standard_normal((m, k), dtype=np.float32)).to(dev)
                y = torch.empty(m, n, dtype=torch.float32, device=dev)
                for h, _ in copies:
                    _lib.check(lib.pg_matmul_quantized(gpu.handle, x.data_ptr(), m, k, h, y.data_ptr()))
                with gpu.record() as gg:
                    for h, _ in copies:
                        _lib.check(lib.pg_matmul_quantized(gpu.handle, x.data_ptr(), m, k, h, y.data_ptr()))
                gg.launch()
                reps = 30
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    gg.launch()
                e1.record(stream)
                stream.synchronize()
                gg.free()
                us = e0.elapsed_time(e1) / (reps * ncopies) * 1e3
                gbs = bytes_w8a8(m, k, n) / (us * 1e-6) / 1e9
                table[f"M{m}_K{k}_N{n}"] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / hbm_peak, 3)}
                del x, y
            for h, _ in copies:
                lib.pg_qtensor_free(gpu.handle, h)
            del copies
    out["w8a8_quantise_and_product_per_shape"] = table
    n, k = 14336, 4096
    for kind, bs in (("q4_0", 18), ("q8_0", 34)):
        # random quants under one sane f16 scale per block: the product's speed does not depend on the values
        blocks = g.integers(0, 256, (n * (k // 32), bs), dtype=np.uint8)
        blocks[:, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)
        raw = blocks.reshape(-1)
        copies = [pg.gguf.GgufWeight(kind, raw, n, k, gpu) for _ in range(6 if kind == "q4_0" else 3)]
        for m in (1, 8):
            with torch.cuda.stream(stream):
                x = torch.from_numpy(g.standard_normal((m, k), dtype=np.float32)).to(dev)
                y = torch.empty(m, n, dtype=torch.float32, device=dev)
                for c in copies:
                    c.matmul_device(x, m, y)
                with gpu.record() as gg:
                    for c in copies:
                        c.matmul_device(x, m, y)
                gg.launch()
                reps = 20
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    gg.launch()
                e1.record(stream)
                stream.synchronize()
                gg.free()
            us = e0.elapsed_time(e1) / (reps * len(copies)) * 1e3
            nbytes = n * (k // 32) * bs + 4 * m * k + 4 * m * n
            gbs = nbytes / (us * 1e-6) / 1e9
            out[f"gguf_{kind}_M{m}"] = {"us": us, "gbs": gbs, "frac_of_measured_hbm": gbs / hbm_peak}
        for c in copies:
            c.free()
    out["huffman_load"] = huffman_load_measurement(gpu, g)
    return out


def huffman_load_measurement(gpu, g, rows=4096, cols=4096, sparsity=0.5, reps=5):
    """A Huffman-coded [rows, cols] int8 weight (N(0, 0.02), half of it zeroed, quantised per column) loaded with
    pg_qtensor_from_huffman (compressed bytes up, parallel decode and transposition on the device) beside the plain load
    of the decoded bytes (pg_qtensor_from_i8).  Host clock around the blocking calls, pinned host memory, best of `reps`."""
    import torch

    import peregrine_b200 as pg
    from peregrine_b200 import _lib
    from peregrine_b200.huffman import HuffmanTensor, _stream_tables
    from peregrine_b200.runtime import _ptr

    C = _lib.C
    w = g.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
    w[g.random((rows, cols)) < sparsity] = 0
    qt = pg.quant.quantize_weights(w, rows, cols, gpu)
    ht = HuffmanTensor.from_quantized(qt, 4, limit_lengths=True)
    packed, sizes, lens = _stream_tables(ht.streams, ht.stream_lengths)
    pinned_bits = torch.from_numpy(packed).pin_memory()
    pinned_q = torch.from_numpy(np.ascontiguousarray(qt.data_i8)).pin_memory()

    def best(fn):
        t_best, keep = 1e9, None
        for i in range(reps + 1):
            h = C.c_void_p()
            t0 = time.perf_counter()
            _lib.check(fn(h))
            dt = time.perf_counter() - t0
            if i:
                t_best = min(t_best, dt)
            if keep is not None:
                gpu.lib.pg_qtensor_free(gpu.handle, keep)
            keep = h
        return t_best * 1e3, keep

    ms_h, h = best(lambda h: gpu.lib.pg_qtensor_from_huffman(gpu.handle, _ptr(ht.table.bit_lengths), len(lens), _ptr(lens), _ptr(sizes),
                                                             pinned_bits.data_ptr(), _ptr(ht.scales), rows, cols, C.byref(h)))
    back = np.empty((cols, rows), np.int8)
    _lib.check(gpu.lib.pg_qtensor_download(gpu.handle, h, None, _ptr(back), None))
    identical = bool(np.array_equal(back, qt.data_i8_t))
    gpu.lib.pg_qtensor_free(gpu.handle, h)
    ms_p, h = best(lambda h: gpu.lib.pg_qtensor_from_i8(gpu.handle, pinned_q.data_ptr(), _ptr(qt.scales), rows, cols, C.byref(h)))
    gpu.lib.pg_qtensor_free(gpu.handle, h)
    return {"tensor": f"{rows}x{cols} int8, {int(sparsity * 100)}% zeros, 4 streams", "compressed_bytes": int(packed.size),
            "ratio": float(ht.compression_ratio()), "from_huffman_ms": ms_h, "from_i8_ms": ms_p, "sweeps": int(gpu.lib.pg_huffman_last_sweeps()),
            "decoded_gb_s": rows * cols / (ms_h * 1e-3) / 1e9, "identical_to_source": identical, "host_memory": "pinned"}


def llama_decode_measurement(gpu, torch, stream, dev, hbm_peak, steps=128, warmup=8, layers=32, rank=0, world=1):
    """Llama-3-8B-shape int8 decode stack: 32 layers, hidden 4096, GQA 32/8 heads of 128, SwiGLU 14336,
    vocab 128256, all linears ~N(0,0.02) quantised per column, batch 16, KV cache pre-filled with N(0,1)
    to context 2048, greedy decode of `steps` tokens from one recorded graph."""
    from peregrine_b200.llama import LlamaConfig, LlamaInt8Decoder

    cfg = LlamaConfig(layers=layers, capacity=2048 + 128)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4000)

    class Lazy(dict):
        """weights are drawn on the device when the model asks for them, so only one f32 matrix lives at a time"""

        def __getitem__(self, k):
            if k == "embedding":
                return torch.randn(cfg.vocab, cfg.hidden, generator=gen, device=dev) * 0.02
            if k.endswith("norm"):
                return torch.ones(cfg.hidden, device=dev)            # nn.rs:569: RMSNorm weights start at 1
            shape = {"lm_head": (cfg.hidden, cfg.vocab), "qkv": (cfg.hidden, cfg.qkv_dim), "o": (cfg.hidden, cfg.hidden),
                     "gate_up": (cfg.hidden, 2 * cfg.ffn), "down": (cfg.ffn, cfg.hidden)}[k.split(".")[-1]]
            return torch.randn(*shape, generator=gen, device=dev) * 0.02

        def columns(self, name, cols):
            """only this rank's columns of a linear are ever drawn (values differ from the single-GPU run's; timing does not care)"""
            rows = {"lm_head": cfg.hidden, "qkv": cfg.hidden, "o": cfg.n_q_heads * cfg.head_dim, "gate_up": cfg.hidden, "down": cfg.ffn}[name.split(".")[-1]]
            return torch.randn(rows, len(cols), generator=gen, device=dev) * 0.02

    with torch.cuda.stream(stream):
        model = LlamaInt8Decoder(cfg, gpu, Lazy(), device_index=dev.index, rank=rank, world=world)
        ctx0 = 2048
        for i in range(cfg.layers):
            model.kcache[i, :, :, :ctx0].normal_(generator=gen)
            model.vcache[i, :, :, :ctx0].normal_(generator=gen)
        model.set_position(ctx0)
        model.set_tokens(np.random.Generator(np.random.PCG64(4000)).integers(0, cfg.vocab, cfg.batch).astype(np.int32))
        torch.cuda.synchronize()
        model.embed()
        graph = model.record()
        for _ in range(warmup):
            graph.launch()
        stream.synchronize()
        st = gpu.device_status()
        if st != 0:
            raise SystemExit(f"rank {rank}: device status {st} in the warm-up steps of the decode stack (a bounded wait ran out): not measuring")
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        model.set_position(ctx0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.launch()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1)
        assert gpu.device_status() == 0
        # end to end: tokens leave and enter through host memory every step
        host_tok = torch.zeros(cfg.batch, dtype=torch.int32).pin_memory()
        model.set_position(ctx0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            graph.launch()
            host_tok.copy_(model.tokens, non_blocking=True)
            stream.synchronize()
        e2e_s = time.perf_counter() - t0
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
    mean_len = ctx0 + (steps + 1) / 2.0
    bytes_per_step = model.weight_bytes() + model.kv_bytes(int(mean_len))
    out = {"tok_s": cfg.batch * steps / (ms * 1e-3), "ms_per_step": ms / steps, "steps": steps, "batch": cfg.batch, "context": ctx0,
           "layers": cfg.layers, "kernels_per_step": graph.kernels,
           "bytes_per_step": bytes_per_step, "weight_bytes": model.weight_bytes(), "kv_bytes_mean": model.kv_bytes(int(mean_len)),
           "hbm_gbs": bytes_per_step / (ms / steps * 1e-3) / 1e9, "frac_of_measured_hbm": bytes_per_step / (ms / steps * 1e-3) / 1e9 / hbm_peak,
           "e2e_tok_s": cfg.batch * steps / e2e_s, "e2e_ms_per_step": e2e_s / steps * 1e3,
           "attention_slices": int(model.splits)}
    graph.free()
    model.free()
    del model
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extra", action="store_true", help="(default at N=1; kept for old command lines)")
    ap.add_argument("--no-extra", action="store_true", help="skip the prefill GEMM, GGUF product and Huffman load figures")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-llama", action="store_true", help="skip the Llama-8B-shape decode stack measurement (N = 1 only)")
    ap.add_argument("--parallel", default="shard", choices=["shard", "replicas"],
                    help="N > 1: weights sharded by output column over the GPUs, output slices gathered (strong scaling of one sweep and "
                         "of the Llama decode stack; default), or one full replica of the weights and one sweep per GPU with no collective "
                         "(weak scaling)")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1, sharded: slices stored into every rank by the products' own epilogues, recorded in the step graph "
                         "(default), or eager NCCL all-gathers")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: libraries that print there (NCCL's version banner) are sent to
    # stderr by pointing file descriptor 1 at it; the line itself goes to a duplicate of the original stdout
    global RESULT_OUT
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
