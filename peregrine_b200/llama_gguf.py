"""`Llama::from_gguf` on the int8 path: a GGUF model file -> `LlamaInt8Decoder`.

Mirrors the loader of the reference (src/models/llama/model.rs:28-62, 100-213, 243-257), with the one
step the reference left open: its `Llama` keeps every linear as an f32 tensor, and its int8 hook
`GgufFile::load_tensor_q8` (src/gguf.rs:519-537) quantises a tensor in its STORED `[out, in]`
orientation, i.e. per input channel, which `matmul_quantized` (scales per output column of an
`[in, out]` matrix, src/quant.rs:129-169) cannot use.  Here the order is the one the f32 loader
has: `load_tensor_f32` -> `[out, in]` -> transpose to `[in, out]` (`load_transposed_weight`) -> column
concatenation `[Q | K | V]` and `[gate | up]` (`fuse_qkv`, src/models/llama/attention.rs:51-71;
`fuse_gate_up`, src/models/llama/decoder.rs:49-67) -> `quantize_weights` per output column, on the GPU.

Tensor names and metadata keys are the reference's (llama.cpp's): `token_embd.weight`,
`output.weight` (absent: tied to the embedding), `output_norm.weight`, `blk.{i}.attn_norm.weight`,
`blk.{i}.ffn_norm.weight`, `blk.{i}.attn_{q,k,v,output}.weight`, `blk.{i}.ffn_{gate,up,down}.weight`.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from .gguf_file import GgufFile, GgufPanic
from .llama import LlamaConfig, LlamaInt8Decoder


def config_from_gguf(gguf: GgufFile, batch: int = 1, capacity: Optional[int] = None) -> LlamaConfig:
    """LlamaConfig::from_gguf (src/models/llama/model.rs:28-62): same keys, same defaults, same panics."""

    def need(key: str) -> int:
        v = gguf.get_u32(key)
        if v is None:
            raise GgufPanic(f"missing {key}")          # .expect("missing ...")
        return int(v)

    hidden = need("llama.embedding_length")
    layers = need("llama.block_count")
    n_q = need("llama.attention.head_count")
    n_kv = gguf.get_u32("llama.attention.head_count_kv")
    n_kv = n_q if n_kv is None else int(n_kv)
    ffn = need("llama.feed_forward_length")
    rope_base = gguf.get_f32("llama.rope.freq_base")
    eps = gguf.get_f32("llama.attention.layer_norm_rms_epsilon")
    max_seq = gguf.get_u32("llama.context_length")
    tokens = gguf.get_metadata("tokenizer.ggml.tokens")
    vocab = len(tokens) if isinstance(tokens, (list, tuple)) else 128256
    return LlamaConfig(layers=layers, hidden=hidden, n_q_heads=n_q, n_kv_heads=n_kv, head_dim=hidden // n_q, ffn=ffn, vocab=vocab,
                       rope_base=float(500000.0 if rope_base is None else rope_base), eps=float(1e-5 if eps is None else eps),
                       batch=batch, capacity=int(capacity if capacity is not None else (8192 if max_seq is None else max_seq)))


def load_transposed_weight(gguf: GgufFile, name: str, gpu=None) -> np.ndarray:
    """src/models/llama/model.rs:243-257: the tensor as f32 `[out, in]` (reversed file shape), returned as `[in, out]`."""
    shape = gguf.tensor_shape(name)
    if len(shape) != 2:
        raise GgufPanic(f"expected 2D weight for {name}")
    rows, cols = shape
    data = gguf.load_tensor_f32(name, gpu).reshape(rows, cols)
    return np.ascontiguousarray(data.T)


def fuse_qkv(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """src/models/llama/attention.rs:51-71: `[model_dim, q_dim + 2 kv_dim]`, columns Q then K then V."""
    return np.ascontiguousarray(np.concatenate([q, k, v], axis=1), np.float32)


def fuse_gate_up(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """src/models/llama/decoder.rs:49-67: `[model_dim, 2 ffn_dim]`, columns gate then up."""
    return np.ascontiguousarray(np.concatenate([gate, up], axis=1), np.float32)


def weights_from_gguf(gguf: GgufFile, cfg: LlamaConfig, gpu=None) -> Dict[str, np.ndarray]:
    """Every tensor `Llama::from_gguf` reads (src/models/llama/model.rs:110-205), as the f32 arrays
    `LlamaInt8Decoder` takes: linears `[in, out]`, Q|K|V and gate|up fused."""
    W: Dict[str, np.ndarray] = {}
    emb_shape = gguf.tensor_shape("token_embd.weight")                       # [vocab, dim]
    emb = gguf.load_tensor_f32("token_embd.weight", gpu).reshape(emb_shape)
    if emb.shape != (cfg.vocab, cfg.hidden):
        # the reference takes the vocabulary size from the tokenizer list and would index out of range here
        raise GgufPanic(f"token_embd.weight is {list(emb.shape)}, the metadata says [{cfg.vocab}, {cfg.hidden}]")
    W["embedding"] = emb
    if "output.weight" in gguf.tensors:
        W["lm_head"] = load_transposed_weight(gguf, "output.weight", gpu)    # [vocab, dim] -> [dim, vocab]
    else:
        W["lm_head"] = np.ascontiguousarray(emb.T)                           # tied weights (model.rs:139-151)
    W["final_norm"] = gguf.load_tensor_f32("output_norm.weight", gpu)
    for i in range(cfg.layers):
        p = f"blk.{i}."
        W[f"l{i}.attn_norm"] = gguf.load_tensor_f32(p + "attn_norm.weight", gpu)
        W[f"l{i}.ffn_norm"] = gguf.load_tensor_f32(p + "ffn_norm.weight", gpu)
        W[f"l{i}.qkv"] = fuse_qkv(load_transposed_weight(gguf, p + "attn_q.weight", gpu), load_transposed_weight(gguf, p + "attn_k.weight", gpu),
                                  load_transposed_weight(gguf, p + "attn_v.weight", gpu))
        W[f"l{i}.o"] = load_transposed_weight(gguf, p + "attn_output.weight", gpu)
        W[f"l{i}.gate_up"] = fuse_gate_up(load_transposed_weight(gguf, p + "ffn_gate.weight", gpu),
                                          load_transposed_weight(gguf, p + "ffn_up.weight", gpu))
        W[f"l{i}.down"] = load_transposed_weight(gguf, p + "ffn_down.weight", gpu)
    c = cfg
    expect = {"qkv": (c.hidden, c.qkv_dim), "o": (c.n_q_heads * c.head_dim, c.hidden), "gate_up": (c.hidden, 2 * c.ffn), "down": (c.ffn, c.hidden)}
    for i in range(cfg.layers):
        for k, shp in expect.items():
            if W[f"l{i}.{k}"].shape != shp:
                raise GgufPanic(f"blk.{i}: fused {k} weight is {list(W[f'l{i}.{k}'].shape)}, the metadata says {list(shp)}")
    if W["lm_head"].shape != (c.hidden, c.vocab):
        raise GgufPanic(f"output weight is {list(W['lm_head'].shape)}, the metadata says [{c.hidden}, {c.vocab}]")
    return W


def from_gguf(source, gpu, batch: int = 1, capacity: Optional[int] = None, device_index: int = 0, rank: int = 0, world: int = 1,
              group=None, attn_splits: str = "auto"):
    """`Llama::from_gguf(path)` (src/models/llama/model.rs:100-213) for the int8 decode step.  `source`: a path, the
    file's bytes, or a parsed `GgufFile`.  Returns `(decoder, gguf)` like the reference returns `(model, gguf)`."""
    if isinstance(source, GgufFile):
        gguf = source
    elif isinstance(source, (bytes, bytearray, memoryview)):
        gguf = GgufFile.parse(bytes(source), gpu)
    else:
        gguf = GgufFile.load(source, gpu)
    cfg = config_from_gguf(gguf, batch, capacity)
    W = weights_from_gguf(gguf, cfg, gpu)
    return LlamaInt8Decoder(cfg, gpu, W, device_index=device_index, rank=rank, world=world, group=group, attn_splits=attn_splits), gguf
