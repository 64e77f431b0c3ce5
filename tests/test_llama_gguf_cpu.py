"""Llama::from_gguf on the host side (no GPU: every tensor of the test file is F32): metadata keys and defaults of
LlamaConfig::from_gguf (src/models/llama/model.rs:28-62), tensor names, the [out, in] -> [in, out] transposition
(model.rs:243-257) and the fused column orders [Q | K | V] (attention.rs:51-71) and [gate | up] (decoder.rs:49-67)."""
import numpy as np
import pytest

import _gguf_writer as gw
from _llama_gguf import make_model, reference_weights
from peregrine_b200 import llama_gguf
from peregrine_b200.gguf_file import GgufFile, GgufPanic


def test_config_and_weights_from_an_f32_file():
    g = np.random.Generator(np.random.PCG64(8))
    blob, stored = make_model(g, layers=2, hidden=256, n_q=4, n_kv=2, ffn=384, vocab=320)
    gguf = GgufFile.parse(blob)
    cfg = llama_gguf.config_from_gguf(gguf, batch=3)
    assert (cfg.layers, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab) == (2, 256, 4, 2, 64, 384, 320)
    assert cfg.rope_base == 10000.0 and abs(cfg.eps - 1e-6) < 1e-12 and cfg.capacity == 96 and cfg.batch == 3
    W = llama_gguf.weights_from_gguf(gguf, cfg)
    ref = reference_weights(stored, 2)
    assert sorted(W) == sorted(ref)
    for k in ref:
        assert W[k].shape == ref[k].shape and np.array_equal(W[k], ref[k]), k
    # the fused orders, spelled out: x @ qkv gives [q heads | k heads | v heads]; gate before up
    q, k_, v = stored["blk.1.attn_q.weight"], stored["blk.1.attn_k.weight"], stored["blk.1.attn_v.weight"]
    assert np.array_equal(W["l1.qkv"][:, :256], q.T) and np.array_equal(W["l1.qkv"][:, 256:384], k_.T) and np.array_equal(W["l1.qkv"][:, 384:], v.T)
    assert np.array_equal(W["l1.gate_up"][:, :384], stored["blk.1.ffn_gate.weight"].T)
    assert np.array_equal(W["l1.gate_up"][:, 384:], stored["blk.1.ffn_up.weight"].T)
    assert W["l0.o"].shape == (256, 256) and W["l0.down"].shape == (384, 256) and W["lm_head"].shape == (256, 320)


def test_tied_output_weights_and_defaults():
    g = np.random.Generator(np.random.PCG64(9))
    blob, stored = make_model(g, layers=1, hidden=128, n_q=2, n_kv=2, ffn=128, vocab=64, tied=True)
    gguf = GgufFile.parse(blob)
    cfg = llama_gguf.config_from_gguf(gguf)
    W = llama_gguf.weights_from_gguf(gguf, cfg)
    assert np.array_equal(W["lm_head"], stored["token_embd.weight"].T)          # model.rs:139-151
    # defaults (model.rs:35-38): no kv head count -> the query head count; rope base 500000; eps 1e-5; context 8192;
    # vocabulary 128256 when the tokenizer list is missing
    kvs = [("llama.embedding_length", gw.U32, 128), ("llama.block_count", gw.U32, 1), ("llama.attention.head_count", gw.U32, 2),
           ("llama.feed_forward_length", gw.U32, 128)]
    bare = GgufFile.parse(gw.build(kvs, []))
    c = llama_gguf.config_from_gguf(bare)
    assert (c.n_kv_heads, c.rope_base, c.capacity, c.vocab) == (2, 500000.0, 8192, 128256) and abs(c.eps - 1e-5) < 1e-12
    with pytest.raises(GgufPanic, match="missing llama.block_count"):
        llama_gguf.config_from_gguf(GgufFile.parse(gw.build(kvs[:1], [])))
    with pytest.raises(GgufPanic, match="not found"):
        llama_gguf.weights_from_gguf(bare, c)
