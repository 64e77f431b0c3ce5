"""Llama decode step on the int8 path: the wiring the reference left open.

The reference's `Llama` (src/models/llama/model.rs:100-237) dequantises every weight to f32 and
calls `Tensor::matmul`; its int8 hooks exist but are unwired (`GgufFile::load_tensor_q8`,
`Tensor::matmul_quantized`, peregrine-py/src/py_inference.rs:183).  This module holds the five
linears of every layer as device-resident `QuantizedTensor`s -- fused `[Q | K | V]`
(src/models/llama/attention.rs:51-71), O, fused `[gate | up]` (src/models/llama/decoder.rs:49-67), down,
and the output head -- and runs one decode step for a batch of independent sequences:

    x -> [RMSNorm+quantise] -> QKV -> [RoPE, KV append, GQA attention + quantise] -> O
      -> [residual+RMSNorm+quantise] -> gate|up -> [SwiGLU+quantise] -> down -> (residual into the next norm)
    final: [residual+RMSNorm+quantise] -> lm_head -> [argmax, position += 1] -> [embedding] -> x

Bracketed stages are the f32 glue kernels of csrc/pg_llama.cu; the products are `pg_gemm_i8`.
torch is used only to hold device memory.  A step can be recorded once into a graph and replayed:
the position lives in device memory.

Column-sharded form (`world` > 1, one process per GPU): every linear keeps only this rank's output
columns -- whole KV heads with the query heads that attend to them, the same channel range of gate
and up, contiguous ranges of O, down and the vocabulary -- so attention, the KV cache and SiLU(g)*u
stay local to a rank, and four exchanges per layer gather what the next linear needs as whole rows
(attention rows, O, SwiGLU rows, down).  Each exchange is stored into every rank's buffer by the
kernel that produces the slice and awaited by the kernel that consumes the rows (`pg_*_exchange`):

    x -> [RMSNorm+quantise] -> QKV_r -> [attention on rank r's heads] => rows -> [quantise] -> O_r => delta
      -> [residual+RMSNorm+quantise] -> gate|up_r -> [SwiGLU_r] => rows -> [quantise] -> down_r => delta
    final: [residual+RMSNorm+quantise] -> lm_head_r -> [local argmax] => 8 bytes -> [pick, position += 1, embedding]

(`=>` is a store into all ranks over NVLink.)  The integer sums and per-column epilogues make every
linear's gathered output bit-identical to the unsharded product of the same rows.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence

import numpy as np

from . import _lib, sharded


@dataclass
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_base: float = 500000.0    # src/models/llama/model.rs:36
    eps: float = 1e-5              # src/models/llama/model.rs:37
    batch: int = 16
    capacity: int = 2176           # KV positions per sequence

    @property
    def qkv_dim(self) -> int:
        return (self.n_q_heads + 2 * self.n_kv_heads) * self.head_dim


def rope_tables(head_dim: int, max_pos: int, base: float):
    """cos/sin tables as RoPE::new builds them (src/nn.rs:1258-1283), f32: [max_pos, head_dim/2]."""
    half = head_dim // 2
    i = np.arange(half, dtype=np.float32)
    inv = np.power(np.float32(base), np.float32(2.0) * i / np.float32(head_dim)).astype(np.float32)
    theta = (np.arange(max_pos, dtype=np.float32)[:, None] / inv[None, :]).astype(np.float32)
    return np.cos(theta).astype(np.float32), np.sin(theta).astype(np.float32)


class LlamaInt8Decoder:
    """weights: name -> f32 array ([in, out] for linears), numpy or torch (any device):
    `embedding` [V, hidden], `final_norm` [hidden], `lm_head` [hidden, V], and per layer i
    `l{i}.attn_norm`, `l{i}.qkv` [hidden, qkv_dim], `l{i}.o` [hidden, hidden], `l{i}.ffn_norm`,
    `l{i}.gate_up` [hidden, 2*ffn], `l{i}.down` [ffn, hidden].  If `weights` has a method
    `columns(name, cols)` it is asked for just this rank's columns of a linear (so that a sharded
    rank never holds a whole matrix); otherwise the whole matrix is taken and sliced.

    rank / world: this process's place among the ranks that share the model by output column; the
    exchanges are connected over `group` (torch.distributed, any backend) or, for ranks that live in
    one process, with `connect_local`.  attn_splits: "match" cuts the context into as many slices per
    (sequence, KV head) as the single-GPU step does, which makes the whole step bit-identical to it;
    "auto" lets each rank cut for its own number of heads (faster, f32 sums in another order)."""

    def __init__(self, cfg: LlamaConfig, gpu, weights, device_index: int = 0, rank: int = 0, world: int = 1, group=None,
                 attn_splits: str = "auto", connect: bool = True):
        import torch

        self.torch = torch
        self.cfg, self.gpu, self.lib = cfg, gpu, gpu.lib
        self.dev = torch.device("cuda", device_index)
        self.rank, self.world, self.group = rank, world, group
        c = cfg
        B = c.batch
        f32, i8, i32 = torch.float32, torch.int8, torch.int32
        dev = self.dev
        if world > 1:
            if c.n_kv_heads % world or c.hidden % world or c.ffn % (4 * world) or c.vocab % world:
                raise ValueError("sharded Llama: world must divide the KV heads, hidden, vocab and ffn / 4")
            if (c.n_q_heads // c.n_kv_heads) not in (4, 8):
                raise ValueError("sharded Llama: the fused attention kernel needs 4 or 8 query heads per KV head")
        self.hq_l, self.hkv_l = c.n_q_heads // world, c.n_kv_heads // world
        self.f_l, self.h_l, self.v_l = c.ffn // world, c.hidden // world, c.vocab // world
        self.qkv_l = (self.hq_l + 2 * self.hkv_l) * c.head_dim
        plans = {
            "qkv": sharded.llama_qkv_columns(c.n_q_heads, c.n_kv_heads, c.head_dim, world)[rank],
            "gate_up": sharded.llama_gate_up_columns(c.ffn, world)[rank],
            "o": np.arange(*sharded.shard_bounds(c.hidden, world)[rank], dtype=np.int64),
            "down": np.arange(*sharded.shard_bounds(c.hidden, world)[rank], dtype=np.int64),
            "lm_head": np.arange(*sharded.shard_bounds(c.vocab, world)[rank], dtype=np.int64),
        }
        self.plans = plans

        def dev_f32(a):
            t = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a, np.float32))
            return t.to(dev, torch.float32).contiguous()

        def qtensor(name, rows, cols_total):
            cols = plans[name.split(".")[-1]]
            if world == 1:
                t = dev_f32(weights[name])
                assert tuple(t.shape) == (rows, cols_total), (name, tuple(t.shape), rows, cols_total)
            elif hasattr(weights, "columns"):
                t = dev_f32(weights.columns(name, cols))
            else:
                t = dev_f32(weights[name])
                assert tuple(t.shape) == (rows, cols_total), (name, tuple(t.shape), rows, cols_total)
                t = t[:, torch.from_numpy(cols).to(dev)].contiguous()
            assert tuple(t.shape) == (rows, len(cols)), (name, tuple(t.shape))
            h = C.c_void_p()
            # per-column scales: quantising this rank's columns alone gives the same bytes as slicing the quantised whole
            _lib.check(self.lib.pg_qtensor_from_f32(gpu.handle, t.data_ptr(), rows, len(cols), 0, C.byref(h)))
            gpu.sync()
            return h

        self.embedding = dev_f32(weights["embedding"])
        self.final_norm = dev_f32(weights["final_norm"])
        self.lm_head = qtensor("lm_head", c.hidden, c.vocab)
        self.layers = []
        for i in range(c.layers):
            self.layers.append({
                "attn_norm": dev_f32(weights[f"l{i}.attn_norm"]),
                "qkv": qtensor(f"l{i}.qkv", c.hidden, c.qkv_dim),
                "o": qtensor(f"l{i}.o", c.n_q_heads * c.head_dim, c.hidden),
                "ffn_norm": dev_f32(weights[f"l{i}.ffn_norm"]),
                "gate_up": qtensor(f"l{i}.gate_up", c.hidden, 2 * c.ffn),
                "down": qtensor(f"l{i}.down", c.ffn, c.hidden),
            })
        cos, sin = rope_tables(c.head_dim, c.capacity, c.rope_base)
        self.cos, self.sin = dev_f32(cos), dev_f32(sin)
        # KV caches [layers][B, Hkv on this rank, cap, hd]
        self.kcache = torch.zeros(c.layers, B, self.hkv_l, c.capacity, c.head_dim, dtype=f32, device=dev)
        self.vcache = torch.zeros_like(self.kcache)
        self.pos = torch.zeros(1, dtype=i32, device=dev)
        self.tokens = torch.zeros(B, dtype=i32, device=dev)
        # activations
        wide = max(c.hidden, c.ffn, c.n_q_heads * c.head_dim)
        self.x = torch.zeros(B, c.hidden, dtype=f32, device=dev)
        self.q8 = torch.zeros(B * wide + 64, dtype=i8, device=dev)
        self.q8s = torch.zeros(B, dtype=f32, device=dev)
        self.qkv = torch.zeros(B, self.qkv_l, dtype=f32, device=dev)
        self.q_rot = torch.zeros(B, self.hq_l, c.head_dim, dtype=f32, device=dev)
        self.gate_up = torch.zeros(B, 2 * self.f_l, dtype=f32, device=dev)
        self.logits = torch.zeros(B, self.v_l, dtype=f32, device=dev)     # this rank's vocabulary columns
        if world == 1:
            self.o = torch.zeros(B, c.hidden, dtype=f32, device=dev)
            self.down = torch.zeros(B, c.hidden, dtype=f32, device=dev)
        # context slices per (sequence, KV head)
        S_own = self.lib.pg_gqa_decode_splits(gpu.handle, B, self.hq_l, self.hkv_l, c.capacity)
        S_one = self.lib.pg_gqa_decode_splits(gpu.handle, B, c.n_q_heads, c.n_kv_heads, c.capacity)
        if attn_splits not in ("auto", "match"):
            raise ValueError("attn_splits: 'auto' or 'match'")
        self.splits = S_one if (attn_splits == "match" or world == 1) else S_own
        self.work = torch.zeros(B * self.hq_l * max(self.splits, S_own) * 130, dtype=f32, device=dev)
        self.graph = None
        # RoPE and the KV append run inside the attention kernel when it has the streaming form (4 or 8 query heads per KV head)
        self.fuse_rope = (c.n_q_heads // c.n_kv_heads) in (4, 8)
        # exchanges of the sharded step, one set for all layers (four other exchanges lie between two uses of one)
        self.ex: Dict[str, sharded.Exchange] = {}
        if world > 1:
            sizes = {"attn": B * c.n_q_heads * c.head_dim * 4, "o": B * c.hidden * 4, "act": B * c.ffn * 4, "down": B * c.hidden * 4,
                     "arg": B * world * 8}
            for name, nbytes in sizes.items():
                self.ex[name] = sharded.Exchange(gpu, rank, world, nbytes)
            if connect:
                for e in self.ex.values():
                    e.connect(group)
        torch.cuda.synchronize()   # torch filled the buffers on its own stream; the kernels use the context's

    @staticmethod
    def connect_local(decoders: Sequence["LlamaInt8Decoder"]) -> None:
        """Ranks that live in one process (built with connect=False): wire their exchanges to each other."""
        for name in decoders[0].ex:
            sharded.Exchange.connect_local([d.ex[name] for d in decoders])

    # ---- state --------------------------------------------------------------------------------
    def set_position(self, pos: int) -> None:
        self.pos.fill_(int(pos))

    def set_tokens(self, tokens) -> None:
        t = self.torch.as_tensor(np.asarray(tokens, np.int32)).to(self.dev)
        self.tokens.copy_(t)
        self.torch.cuda.synchronize()

    def embed(self) -> None:
        c = self.cfg
        _lib.check(self.lib.pg_embedding(self.gpu.handle, self.embedding.data_ptr(), self.tokens.data_ptr(), c.batch, c.hidden, self.x.data_ptr()))

    def load_cache(self, layer: int, k, v) -> None:
        """k, v: [B, Hkv (all heads), cap, hd] host or device arrays; this rank keeps its KV heads."""
        t = self.torch
        lo, hi = self.rank * self.hkv_l, (self.rank + 1) * self.hkv_l
        for dst, src in ((self.kcache, k), (self.vcache, v)):
            s = src if isinstance(src, t.Tensor) else t.from_numpy(np.ascontiguousarray(src))
            dst[layer].copy_(s[:, lo:hi].to(self.dev))

    # ---- one decode step: x (already embedded) -> logits -> next tokens -> next x ----------------
    def step_ops(self) -> Iterator[str]:
        """Enqueues the step launch by launch, yielding a label after each one (tests stop at the labels to read
        intermediate buffers; ranks that share one process and one GPU are advanced in turn, launch by launch, so that
        every wait finds its flags already raised)."""
        c, lib, h = self.cfg, self.lib, self.gpu.handle
        B, hd = c.batch, c.head_dim
        P = lambda t: t.data_ptr()
        ck = _lib.check
        sh = self.world > 1
        ex = {k: v.handle for k, v in self.ex.items()}
        attn_dim = c.n_q_heads * hd
        delta = None
        for i, L in enumerate(self.layers):
            if sh and i > 0:
                ck(lib.pg_add_rmsnorm_quantize_exchange(h, P(self.x), ex["down"], P(L["attn_norm"]), B, c.hidden, c.eps, P(self.q8), P(self.q8s), None))
            else:
                ck(lib.pg_add_rmsnorm_quantize(h, P(self.x), P(delta) if delta is not None else None, P(L["attn_norm"]), B, c.hidden,
                                               c.eps, P(self.q8), P(self.q8s), None))
            yield f"l{i}.qkv.in"
            ck(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, L["qkv"], P(self.qkv), None, _lib.ALGO_AUTO))
            yield f"l{i}.qkv.out"
            if sh:
                ck(lib.pg_gqa_attention_decode_fused_exchange(h, P(self.qkv), P(self.pos), P(self.cos), P(self.sin), P(self.kcache[i]),
                                                              P(self.vcache[i]), B, self.hq_l, self.hkv_l, hd, c.capacity, P(self.work),
                                                              self.splits, ex["attn"], attn_dim, self.rank * self.hq_l * hd))
                yield f"l{i}.attn"
                ck(lib.pg_quantize_activations_exchange(h, ex["attn"], B, attn_dim, P(self.q8), P(self.q8s)))
            elif self.fuse_rope:
                ck(lib.pg_gqa_attention_decode_fused(h, P(self.qkv), P(self.pos), P(self.cos), P(self.sin), P(self.kcache[i]),
                                                     P(self.vcache[i]), B, c.n_q_heads, c.n_kv_heads, hd, c.capacity,
                                                     P(self.work), None, P(self.q8), P(self.q8s)))
            else:
                ck(lib.pg_rope_kv_append(h, P(self.qkv), P(self.pos), P(self.cos), P(self.sin), B, c.n_q_heads, c.n_kv_heads,
                                         hd, c.capacity, P(self.q_rot), P(self.kcache[i]), P(self.vcache[i])))
                ck(lib.pg_gqa_attention_decode(h, P(self.q_rot), P(self.kcache[i]), P(self.vcache[i]), P(self.pos), B, c.n_q_heads,
                                               c.n_kv_heads, hd, c.capacity, P(self.work), None, P(self.q8), P(self.q8s)))
            yield f"l{i}.o.in"
            if sh:
                ck(lib.pg_gemm_i8_exchange(h, P(self.q8), P(self.q8s), B, attn_dim, L["o"], ex["o"], c.hidden, self.rank * self.h_l, P(self.gate_up)))
                yield f"l{i}.o.out"
                ck(lib.pg_add_rmsnorm_quantize_exchange(h, P(self.x), ex["o"], P(L["ffn_norm"]), B, c.hidden, c.eps, P(self.q8), P(self.q8s), None))
            else:
                ck(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, attn_dim, L["o"], P(self.o), None, _lib.ALGO_AUTO))
                yield f"l{i}.o.out"
                ck(lib.pg_add_rmsnorm_quantize(h, P(self.x), P(self.o), P(L["ffn_norm"]), B, c.hidden, c.eps, P(self.q8), P(self.q8s), None))
            yield f"l{i}.gate_up.in"
            ck(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, L["gate_up"], P(self.gate_up), None, _lib.ALGO_AUTO))
            yield f"l{i}.gate_up.out"
            if sh:
                ck(lib.pg_swiglu_exchange(h, P(self.gate_up), B, self.f_l, ex["act"], c.ffn, self.rank * self.f_l))
                yield f"l{i}.act"
                ck(lib.pg_quantize_activations_exchange(h, ex["act"], B, c.ffn, P(self.q8), P(self.q8s)))
            else:
                ck(lib.pg_swiglu_quantize(h, P(self.gate_up), B, c.ffn, P(self.q8), P(self.q8s), None))
            yield f"l{i}.down.in"
            if sh:
                # the slice buffer of shapes the fused epilogue does not take: the gate|up output is free by now
                ck(lib.pg_gemm_i8_exchange(h, P(self.q8), P(self.q8s), B, c.ffn, L["down"], ex["down"], c.hidden, self.rank * self.h_l, P(self.gate_up)))
            else:
                ck(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.ffn, L["down"], P(self.down), None, _lib.ALGO_AUTO))
                delta = self.down
            yield f"l{i}.down.out"
        if sh and self.layers:
            ck(lib.pg_add_rmsnorm_quantize_exchange(h, P(self.x), ex["down"], P(self.final_norm), B, c.hidden, c.eps, P(self.q8), P(self.q8s), None))
        else:
            ck(lib.pg_add_rmsnorm_quantize(h, P(self.x), P(delta) if delta is not None else None, P(self.final_norm), B, c.hidden, c.eps,
                                           P(self.q8), P(self.q8s), None))
        yield "lm_head.in"
        ck(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, self.lm_head, P(self.logits), None, _lib.ALGO_AUTO))
        yield "lm_head.out"
        if sh:
            ck(lib.pg_argmax_exchange(h, P(self.logits), B, self.v_l, self.rank * self.v_l, ex["arg"]))
            yield "argmax"
            ck(lib.pg_pick_embed(h, ex["arg"], B, P(self.tokens), P(self.pos), c.capacity, P(self.embedding), c.hidden, P(self.x)))
        else:
            ck(lib.pg_argmax_advance(h, P(self.logits), B, c.vocab, P(self.tokens), P(self.pos), c.capacity))
            yield "argmax"
            self.embed()
        yield "embed"

    def enqueue_step(self) -> None:
        for _ in self.step_ops():
            pass

    def record(self):
        """Runs one step eagerly (sizes scratch), restores the position, records the step.  Sharded: every rank calls
        this at the same point; the eager step is itself a complete exchange round, so the ranks stay in step."""
        pos0 = int(self.pos.item())
        tok0 = self.tokens.clone()
        x0 = self.x.clone()
        self.enqueue_step()
        self.gpu.sync()
        self.pos.fill_(pos0)
        self.tokens.copy_(tok0)
        self.x.copy_(x0)
        self.torch.cuda.synchronize()
        if self.world > 1 and self.group is not False:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.barrier(group=self.group)   # nobody replays into a rank that is still restoring its state
        with self.gpu.record() as g:
            self.enqueue_step()
        self.graph = g
        return g

    def gather_logits(self) -> np.ndarray:
        """This rank's [B, V / world] logits (world == 1: all of them), on the host."""
        return self.logits.cpu().numpy()

    def weight_bytes(self) -> int:
        """int8 weight bytes one step reads on THIS rank."""
        c = self.cfg
        per_layer = c.hidden * self.qkv_l + c.n_q_heads * c.head_dim * self.h_l + c.hidden * 2 * self.f_l + c.ffn * self.h_l
        return c.layers * per_layer + c.hidden * self.v_l

    def kv_bytes(self, length: int) -> int:
        c = self.cfg
        return c.layers * c.batch * self.hkv_l * length * c.head_dim * 4 * 2

    def free(self) -> None:
        for L in self.layers:
            for k in ("qkv", "o", "gate_up", "down"):
                self.lib.pg_qtensor_free(self.gpu.handle, L[k])
        if self.layers or self.lm_head is not None:
            self.lib.pg_qtensor_free(self.gpu.handle, self.lm_head)
            self.lm_head = None
        self.layers = []
        for e in self.ex.values():
            e.destroy()
        self.ex = {}
