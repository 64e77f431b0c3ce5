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
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np

from . import _lib


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
    `l{i}.gate_up` [hidden, 2*ffn], `l{i}.down` [ffn, hidden]."""

    def __init__(self, cfg: LlamaConfig, gpu, weights: Dict[str, object], device_index: int = 0):
        import torch

        self.torch = torch
        self.cfg, self.gpu, self.lib = cfg, gpu, gpu.lib
        self.dev = torch.device("cuda", device_index)
        self._keep = []
        c = cfg
        B = c.batch
        f32, i8, i32 = torch.float32, torch.int8, torch.int32
        dev = self.dev

        def dev_f32(a):
            t = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a, np.float32))
            return t.to(dev, torch.float32).contiguous()

        def qtensor(a, rows, cols):
            t = dev_f32(a)
            assert tuple(t.shape) == (rows, cols), (tuple(t.shape), rows, cols)
            h = C.c_void_p()
            _lib.check(self.lib.pg_qtensor_from_f32(gpu.handle, t.data_ptr(), rows, cols, 0, C.byref(h)))
            gpu.sync()
            return h

        self.embedding = dev_f32(weights["embedding"])
        self.final_norm = dev_f32(weights["final_norm"])
        self.lm_head = qtensor(weights["lm_head"], c.hidden, c.vocab)
        self.layers = []
        for i in range(c.layers):
            self.layers.append({
                "attn_norm": dev_f32(weights[f"l{i}.attn_norm"]),
                "qkv": qtensor(weights[f"l{i}.qkv"], c.hidden, c.qkv_dim),
                "o": qtensor(weights[f"l{i}.o"], c.hidden, c.hidden),
                "ffn_norm": dev_f32(weights[f"l{i}.ffn_norm"]),
                "gate_up": qtensor(weights[f"l{i}.gate_up"], c.hidden, 2 * c.ffn),
                "down": qtensor(weights[f"l{i}.down"], c.ffn, c.hidden),
            })
        cos, sin = rope_tables(c.head_dim, c.capacity, c.rope_base)
        self.cos, self.sin = dev_f32(cos), dev_f32(sin)
        # KV caches [layers][B, Hkv, cap, hd]
        self.kcache = torch.zeros(c.layers, B, c.n_kv_heads, c.capacity, c.head_dim, dtype=f32, device=dev)
        self.vcache = torch.zeros_like(self.kcache)
        self.pos = torch.zeros(1, dtype=i32, device=dev)
        self.tokens = torch.zeros(B, dtype=i32, device=dev)
        # activations
        wide = max(c.hidden, c.ffn)
        self.x = torch.zeros(B, c.hidden, dtype=f32, device=dev)
        self.q8 = torch.zeros(B * wide + 64, dtype=i8, device=dev)
        self.q8s = torch.zeros(B, dtype=f32, device=dev)
        self.qkv = torch.zeros(B, c.qkv_dim, dtype=f32, device=dev)
        self.q_rot = torch.zeros(B, c.n_q_heads, c.head_dim, dtype=f32, device=dev)
        self.attn = torch.zeros(B, c.hidden, dtype=f32, device=dev)
        self.o = torch.zeros(B, c.hidden, dtype=f32, device=dev)
        self.gate_up = torch.zeros(B, 2 * c.ffn, dtype=f32, device=dev)
        self.down = torch.zeros(B, c.hidden, dtype=f32, device=dev)
        self.logits = torch.zeros(B, c.vocab, dtype=f32, device=dev)
        S = self.lib.pg_gqa_decode_splits(gpu.handle, B, c.n_q_heads, c.n_kv_heads, c.capacity)
        self.work = torch.zeros(B * c.n_q_heads * S * 130, dtype=f32, device=dev)
        self.graph = None
        # RoPE and the KV append run inside the attention kernel when it has the streaming form (4 or 8 query heads per KV head)
        self.fuse_rope = (c.n_q_heads // c.n_kv_heads) in (4, 8)
        torch.cuda.synchronize()   # torch filled the buffers on its own stream; the kernels use the context's

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

    # ---- one decode step: x (already embedded) -> logits -> next tokens -> next x ----------------
    def enqueue_step(self) -> None:
        c, lib, h = self.cfg, self.lib, self.gpu.handle
        B = c.batch
        P = lambda t: t.data_ptr()
        delta = None
        for i, L in enumerate(self.layers):
            _lib.check(lib.pg_add_rmsnorm_quantize(h, P(self.x), P(delta) if delta is not None else None, P(L["attn_norm"]), B, c.hidden,
                                                   c.eps, P(self.q8), P(self.q8s), None))
            _lib.check(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, L["qkv"], P(self.qkv), None, _lib.ALGO_AUTO))
            if self.fuse_rope:
                _lib.check(lib.pg_gqa_attention_decode_fused(h, P(self.qkv), P(self.pos), P(self.cos), P(self.sin), P(self.kcache[i]),
                                                             P(self.vcache[i]), B, c.n_q_heads, c.n_kv_heads, c.head_dim, c.capacity,
                                                             P(self.work), None, P(self.q8), P(self.q8s)))
            else:
                _lib.check(lib.pg_rope_kv_append(h, P(self.qkv), P(self.pos), P(self.cos), P(self.sin), B, c.n_q_heads, c.n_kv_heads,
                                                 c.head_dim, c.capacity, P(self.q_rot), P(self.kcache[i]), P(self.vcache[i])))
                _lib.check(lib.pg_gqa_attention_decode(h, P(self.q_rot), P(self.kcache[i]), P(self.vcache[i]), P(self.pos), B, c.n_q_heads,
                                                       c.n_kv_heads, c.head_dim, c.capacity, P(self.work), None, P(self.q8), P(self.q8s)))
            _lib.check(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, L["o"], P(self.o), None, _lib.ALGO_AUTO))
            _lib.check(lib.pg_add_rmsnorm_quantize(h, P(self.x), P(self.o), P(L["ffn_norm"]), B, c.hidden, c.eps, P(self.q8), P(self.q8s), None))
            _lib.check(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, L["gate_up"], P(self.gate_up), None, _lib.ALGO_AUTO))
            _lib.check(lib.pg_swiglu_quantize(h, P(self.gate_up), B, c.ffn, P(self.q8), P(self.q8s), None))
            _lib.check(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.ffn, L["down"], P(self.down), None, _lib.ALGO_AUTO))
            delta = self.down
        _lib.check(lib.pg_add_rmsnorm_quantize(h, P(self.x), P(delta) if delta is not None else None, P(self.final_norm), B, c.hidden, c.eps,
                                               P(self.q8), P(self.q8s), None))
        _lib.check(lib.pg_gemm_i8(h, P(self.q8), P(self.q8s), B, c.hidden, self.lm_head, P(self.logits), None, _lib.ALGO_AUTO))
        _lib.check(lib.pg_argmax_advance(h, P(self.logits), B, c.vocab, P(self.tokens), P(self.pos)))
        self.embed()

    def record(self):
        """Runs one step eagerly (sizes scratch), restores the position, records the step."""
        pos0 = int(self.pos.item())
        tok0 = self.tokens.clone()
        x0 = self.x.clone()
        self.enqueue_step()
        self.gpu.sync()
        self.pos.fill_(pos0)
        self.tokens.copy_(tok0)
        self.x.copy_(x0)
        self.torch.cuda.synchronize()
        with self.gpu.record() as g:
            self.enqueue_step()
        self.graph = g
        return g

    def weight_bytes(self) -> int:
        c = self.cfg
        per_layer = c.hidden * c.qkv_dim + c.hidden * c.hidden + c.hidden * 2 * c.ffn + c.ffn * c.hidden
        return c.layers * per_layer + c.hidden * c.vocab

    def kv_bytes(self, length: int) -> int:
        c = self.cfg
        return c.layers * c.batch * c.n_kv_heads * length * c.head_dim * 4 * 2

    def free(self) -> None:
        for L in self.layers:
            for k in ("qkv", "o", "gate_up", "down"):
                self.lib.pg_qtensor_free(self.gpu.handle, L[k])
        self.lib.pg_qtensor_free(self.gpu.handle, self.lm_head)
        self.layers = []
