"""Llama::from_gguf -> int8 decode step on the GPU: a small model stored as Q8_0 / Q4_0 / F16 / F32 tensors is loaded
through the library's loader (block decoders on the GPU, transposition, Q|K|V and gate|up fusion, per-column quantiser on
the GPU) and one decode step is checked stage by stage against the oracle built from the same stored tensors."""
import numpy as np
import pytest

from _inputs import normal, rng
from _llama_gguf import make_model, reference_weights
from test_llama_gpu import check_stages, run_step_with_taps

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["q8_0", "q4_0", "f16"])
def test_from_gguf_decode_step(gpu, oracle_mt, kind):
    import torch
    from oracle import llama_oracle as lo
    from peregrine_b200 import llama_gguf
    from peregrine_b200.llama import rope_tables

    g = rng(50)
    ggml = {"q8_0": 8, "q4_0": 2, "f16": 1}[kind]

    def encode(name, a):
        if name == "token_embd.weight" and kind != "f16":
            return None                                        # embedding stays F32 in the block-quantised files
        if kind == "f16":
            h = a.astype(np.float16)
            return 1, h.tobytes(), h.astype(np.float32)
        raw = oracle_mt.encode(kind, a)
        return ggml, raw, oracle_mt.dequant(kind, raw, a.size).reshape(a.shape)

    blob, stored = make_model(g, layers=2, hidden=512, n_q=4, n_kv=1, ffn=768, vocab=512, encode=encode)
    model, gguf = llama_gguf.from_gguf(blob, gpu, batch=3, capacity=64)
    cfg = model.cfg
    assert (cfg.layers, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab) == (2, 512, 4, 1, 128, 768, 512)
    assert cfg.rope_base == 10000.0 and cfg.capacity == 64
    W = reference_weights(stored, cfg.layers)
    Q = {k: oracle_mt.quantize_weights(v, v.shape[0], v.shape[1]) for k, v in W.items() if v.ndim == 2 and k != "embedding"}
    # the loader's quantised linears are the oracle's, bit for bit (fused column order included)
    from peregrine_b200 import _lib

    for name, h in (("l0.qkv", model.layers[0]["qkv"]), ("l1.gate_up", model.layers[1]["gate_up"]), ("lm_head", model.lm_head)):
        n, k = Q[name].cols, Q[name].rows
        wt, ws = np.empty((n, k), np.int8), np.empty(n, np.float32)
        _lib.check(gpu.lib.pg_qtensor_download(gpu.handle, h, None, wt.ctypes.data, ws.ctypes.data))
        assert np.array_equal(wt, Q[name].data_i8_t) and np.array_equal(ws.view(np.uint32), Q[name].scales.view(np.uint32)), name
    assert np.array_equal(model.embedding.cpu().numpy(), W["embedding"])
    start = 9
    K = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    V = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    for i in range(cfg.layers):
        model.load_cache(i, K[i], V[i])
    cos, sin = rope_tables(cfg.head_dim, cfg.capacity, cfg.rope_base)
    tokens = g.integers(0, cfg.vocab, cfg.batch).astype(np.int32)
    model.set_position(start)
    model.set_tokens(tokens)
    torch.cuda.synchronize()
    model.embed()
    gpu.sync()
    taps = run_step_with_taps(model, gpu)
    assert gpu.device_status() == 0
    stats, logits = check_stages(oracle_mt, cfg, W, Q, taps, W["embedding"][tokens], K, V, start, cos, sin, f"from_gguf {kind}")
    assert np.array_equal(logits, model.logits.cpu().numpy())
    ref = lo.decode_step(oracle_mt, cfg, W, Q, W["embedding"][tokens], [k.copy() for k in K], [v.copy() for v in V], start, cos, sin)
    # K, V above were advanced by check_stages with the GPU's rows; the free-running oracle overwrites the same position
    assert np.abs(logits - ref).max() <= 2e-2 * np.abs(ref).max()
    model.free()
