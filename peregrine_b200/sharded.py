"""Column-sharded quantised linears over the GPUs of one node (one process per GPU).

Each rank keeps the rows [n0, n1) of `data_i8_t [N,K]` (= output columns n0..n1) and the matching
scales, quantises the replicated activations itself and computes Y[:, n0:n1].  Integer accumulation
is exact and the epilogue is per column, so the all-gathered matrix is bit-identical to the
single-GPU product.  The one exchange is an all-gather of output slices over NCCL (gloo in the CPU
tests), whose API precedent in the reference is `Communicator::allgather`
(src/comm/communicator.rs:162-191: concatenation of equal chunks in rank order).

For the Llama layer the reference's fused layouts `[Q | K | V]` (src/models/llama/attention.rs:51-71)
and `[gate | up]` (src/models/llama/decoder.rs:49-67) must not be cut contiguously: `llama_qkv_columns`
and `llama_gate_up_columns` give each rank whole heads (query heads with the KV head they attend to)
and matching gate/up column ranges, so attention and SiLU(g)*u stay local to a rank.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np


def shard_bounds(n: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous, as-equal-as-possible column ranges; the first n % world ranks get one more."""
    if world < 1 or n < 0:
        raise ValueError("shard_bounds: need world >= 1 and n >= 0")
    base, extra = divmod(n, world)
    out, b = [], 0
    for r in range(world):
        e = b + base + (1 if r < extra else 0)
        out.append((b, e))
        b = e
    return out


def llama_qkv_columns(n_q_heads: int, n_kv_heads: int, head_dim: int, world: int) -> List[np.ndarray]:
    """Columns of the fused `[Q | K | V]` weight that rank r owns: its query heads, then the KV
    heads those query heads use (GQA groups stay together), in Q, K, V order."""
    if n_kv_heads % world or n_q_heads % n_kv_heads:
        raise ValueError("llama_qkv_columns: world must divide the KV heads, KV heads must divide the query heads")
    per_kv = n_q_heads // n_kv_heads
    kv_per_rank = n_kv_heads // world
    q_off, k_off, v_off = 0, n_q_heads * head_dim, (n_q_heads + n_kv_heads) * head_dim
    out = []
    for r in range(world):
        kv = range(r * kv_per_rank, (r + 1) * kv_per_rank)
        qh = [h for g in kv for h in range(g * per_kv, (g + 1) * per_kv)]
        cols = [q_off + h * head_dim + i for h in qh for i in range(head_dim)]
        cols += [k_off + g * head_dim + i for g in kv for i in range(head_dim)]
        cols += [v_off + g * head_dim + i for g in kv for i in range(head_dim)]
        out.append(np.asarray(cols, np.int64))
    return out


def llama_gate_up_columns(ffn: int, world: int) -> List[np.ndarray]:
    """Columns of the fused `[gate | up]` weight for rank r: the same range of both halves."""
    out = []
    for b, e in shard_bounds(ffn, world):
        out.append(np.concatenate([np.arange(b, e, dtype=np.int64), np.arange(ffn + b, ffn + e, dtype=np.int64)]))
    return out


def take_columns(qt, cols: Sequence[int]):
    """A QuantizedTensor-like holding only `cols` (in that order) of `qt` (host arrays)."""
    cols = np.asarray(cols, np.int64)
    data_i8 = None if qt.data_i8 is None else np.ascontiguousarray(qt.data_i8[:, cols])
    return type(qt)(data_i8, np.ascontiguousarray(qt.data_i8_t[cols]), np.ascontiguousarray(qt.scales[cols]), qt.rows, len(cols))


def unshard_columns(parts: Sequence[np.ndarray], columns: Sequence[np.ndarray], n: int) -> np.ndarray:
    """Inverse of a column plan: parts[r] is [M, len(columns[r])]; returns [M, n]."""
    m = parts[0].shape[0]
    y = np.empty((m, n), parts[0].dtype)
    for p, c in zip(parts, columns):
        y[:, c] = p
    return y


class ColumnShardedLinear:
    """y = matmul_quantized(x, W) with W's output columns split over the ranks of `group`.

    `columns` is this rank's column index array (default: the contiguous shard).  `compute(x, m,
    k, shard)` produces the local slice; by default it is the CUDA path (`quant.matmul_quantized`
    on this rank's GPU).  The CPU tests pass the oracle here to exercise the plan and the gather."""

    def __init__(self, qt, rank: int, world: int, columns: Optional[Sequence[np.ndarray]] = None, gpu=None,
                 compute: Optional[Callable] = None, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.n, self.k = qt.cols, qt.rows
        if columns is None:
            columns = [np.arange(b, e, dtype=np.int64) for b, e in shard_bounds(self.n, world)]
        if len(columns) != world:
            raise ValueError("ColumnShardedLinear: one column set per rank is required")
        seen = np.sort(np.concatenate([np.asarray(c) for c in columns]))
        if seen.size != self.n or not np.array_equal(seen, np.arange(self.n)):
            raise ValueError("ColumnShardedLinear: the column sets must partition 0..N-1")
        self.columns = [np.asarray(c, np.int64) for c in columns]
        self.width = max(len(c) for c in self.columns)     # slices are padded to this for the gather
        self.shard = take_columns(qt, self.columns[rank])
        self.gpu = gpu
        if compute is None:
            from . import quant

            def compute(x, m, k, shard, _gpu=gpu):
                return quant.matmul_quantized(x, m, k, shard, _gpu)

        self.compute = compute

    def local(self, x, m: int) -> np.ndarray:
        return np.asarray(self.compute(x, m, self.k, self.shard), np.float32).reshape(m, len(self.columns[self.rank]))

    def forward(self, x, m: int) -> np.ndarray:
        """All ranks call this with the same x; every rank returns the full [m, N] result."""
        import torch
        import torch.distributed as dist

        mine = self.local(x, m)
        if self.world == 1:
            return unshard_columns([mine], self.columns, self.n)
        pad = np.zeros((m, self.width), np.float32)
        pad[:, : mine.shape[1]] = mine
        send = torch.from_numpy(pad)
        device = None
        if dist.get_backend(self.group) == "nccl":
            device = torch.device("cuda", torch.cuda.current_device())
            send = send.to(device)
        recv = torch.empty((self.world * m, self.width), dtype=torch.float32, device=send.device)
        dist.all_gather_into_tensor(recv, send, group=self.group)   # rank-major concatenation
        full = recv.cpu().numpy().reshape(self.world, m, self.width)
        parts = [full[r][:, : len(self.columns[r])] for r in range(self.world)]
        return unshard_columns(parts, self.columns, self.n)


class Exchange:
    """One rank's end of an all-gather by direct stores into the other GPUs' result buffers (`pg_exchange_*`): a
    buffer of `y_bytes` that every rank writes its part of, plus the flags that say whose part has arrived.  No
    library collective runs in a step, so a whole sharded step can be recorded into one CUDA graph.  The 64-byte
    handles are swapped once through `torch.distributed` (any backend); ranks that live in one process use
    `connect_local`."""

    def __init__(self, gpu, rank: int, world: int, y_bytes: int):
        import ctypes as C

        from . import _lib

        self.gpu, self.rank, self.world, self.y_bytes = gpu, rank, world, int(y_bytes)
        self._ipc = (C.c_ubyte * 64)()
        h = C.c_void_p()
        _lib.check(gpu.lib.pg_exchange_create(gpu.handle, rank, world, self.y_bytes, self._ipc, C.byref(h)))
        self.handle = h
        self.result_ptr = gpu.lib.pg_exchange_result(h)

    def connect(self, group=None) -> None:
        import ctypes as C

        import torch
        import torch.distributed as dist

        from . import _lib

        if self.world > 1:
            mine = torch.tensor(list(bytes(self._ipc)), dtype=torch.uint8)
            dev = torch.device("cuda", self.gpu.device) if dist.get_backend(group) == "nccl" else torch.device("cpu")
            allh = torch.empty(self.world * 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(allh, mine.to(dev), group=group)
            blob = bytes(allh.cpu().numpy().tobytes())
        else:
            blob = bytes(self._ipc)
        buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        _lib.check(self.gpu.lib.pg_exchange_connect(self.gpu.handle, self.handle, buf))
        if self.world > 1:
            dist.barrier(group=group)   # nobody stores into a peer before that peer exists

    @staticmethod
    def connect_local(ranks: Sequence["Exchange"]) -> None:
        """All ranks of the exchange live in this process: no IPC, the peers' buffers are plain device pointers."""
        import ctypes as C

        from . import _lib

        arr = (C.c_void_p * len(ranks))(*[e.handle for e in ranks])
        for e in ranks:
            _lib.check(e.gpu.lib.pg_exchange_connect_local(e.gpu.handle, e.handle, arr))

    def store(self, d_slice, m: int, n_local: int, n_total: int, col0: int) -> None:
        """Hand this rank's [m, n_local] slice to every rank (columns col0.. of their [m, n_total]); do not wait."""
        from . import _lib
        from .runtime import _ptr

        _lib.check(self.gpu.lib.pg_exchange_store(self.gpu.handle, self.handle, _ptr(d_slice), m, n_local, n_total, col0))

    def store_cells(self, d_slice, m: int, n_local: int, n_total: int, col0: int) -> None:
        """The same hand-over in the flagged-cell form (what `pg_gemm_i8_exchange` does from inside the product);
        consume with `gather` or one of the `pg_*_exchange` entry points."""
        from . import _lib
        from .runtime import _ptr

        _lib.check(self.gpu.lib.pg_exchange_store_cells(self.gpu.handle, self.handle, _ptr(d_slice), m, n_local, n_total, col0))

    def gather(self, rows: int, cols: int, d_out=None) -> None:
        """Bounded wait for every rank's cells of the exchange this rank produced last; the plain [rows, cols] matrix goes
        to `d_out` (default: the exchange's own result buffer, `result_ptr`)."""
        from . import _lib
        from .runtime import _ptr

        _lib.check(self.gpu.lib.pg_exchange_gather(self.gpu.handle, self.handle, rows, cols, _ptr(d_out)))

    @staticmethod
    def gather_many(exchanges: Sequence["Exchange"], rows: Sequence[int], cols: Sequence[int], d_outs=None) -> None:
        """`gather` for up to 16 exchanges in one launch: results of independent products that nothing consumes one by one."""
        import ctypes as C

        from . import _lib
        from .runtime import _ptr

        n = len(exchanges)
        gpu = exchanges[0].gpu
        exs = (C.c_void_p * n)(*[e.handle for e in exchanges])
        r = (C.c_int64 * n)(*rows)
        c = (C.c_int64 * n)(*cols)
        outs = None
        if d_outs is not None:
            outs = (C.c_void_p * n)(*[_ptr(o) for o in d_outs])
        _lib.check(gpu.lib.pg_exchange_gather_many(gpu.handle, exs, r, c, outs, n))

    def wait(self) -> None:
        """Bounded wait for every rank's slice of the oldest store not yet waited for."""
        from . import _lib

        _lib.check(self.gpu.lib.pg_exchange_wait(self.gpu.handle, self.handle))

    def read(self, count: int, dtype=np.float32) -> np.ndarray:
        from . import _lib
        from .runtime import _ptr

        out = np.empty(count, dtype)
        _lib.check(self.gpu.lib.pg_mem_download(self.gpu.handle, _ptr(out), self.result_ptr, out.nbytes))
        return out

    def destroy(self) -> None:
        if self.handle is not None and self.gpu.handle:
            self.gpu.lib.pg_exchange_destroy(self.gpu.handle, self.handle)
        self.handle = None


class PeerExchange(Exchange):
    """An `Exchange` sized for one [m_max, n_total] f32 result, connected on construction."""

    def __init__(self, gpu, rank: int, world: int, m_max: int, n_total: int, group=None):
        super().__init__(gpu, rank, world, m_max * n_total * 4)
        self.n_total = n_total
        self.connect(group)

    def allgather(self, d_slice, m: int, n_local: int, col0: int) -> None:
        """Enqueue on the context's stream; afterwards `result_ptr` holds the full [m, n_total] matrix."""
        from . import _lib
        from .runtime import _ptr

        _lib.check(self.gpu.lib.pg_exchange_allgather(self.gpu.handle, self.handle, _ptr(d_slice), m, n_local, self.n_total, col0))

    def store(self, d_slice, m: int, n_local: int, col0: int) -> None:   # noqa: D401 (the fixed-width form)
        Exchange.store(self, d_slice, m, n_local, self.n_total, col0)

    def read(self, m: int) -> np.ndarray:
        return Exchange.read(self, m * self.n_total).reshape(m, self.n_total)
