"""A small Llama model written as a GGUF file in memory (tests/_gguf_writer.py), with the tensor names, shapes
([out, in] linears, file shape = reversed) and metadata keys the reference's loader reads
(src/models/llama/model.rs:28-62, 110-205)."""
import numpy as np

import _gguf_writer as gw


def make_model(g, layers=2, hidden=256, n_q=2, n_kv=2, ffn=384, vocab=320, encode=None, tied=False, sigma=0.05):
    """Returns (file bytes, f32 tensors by GGUF name as the file stores them, i.e. [out, in] for linears).
    encode(name, f32 [rows, cols]) -> (ggml_type, raw bytes, f32 array the decoder will give back) or None for F32."""
    hd = hidden // n_q
    nrm = lambda shape, s: (g.standard_normal(shape, dtype=np.float32) * np.float32(s)).astype(np.float32)
    T = {"token_embd.weight": nrm((vocab, hidden), 0.5), "output_norm.weight": (1 + nrm((hidden,), 0.1)).astype(np.float32)}
    if not tied:
        T["output.weight"] = nrm((vocab, hidden), 0.02)
    for i in range(layers):
        p = f"blk.{i}."
        T[p + "attn_norm.weight"] = (1 + nrm((hidden,), 0.1)).astype(np.float32)
        T[p + "ffn_norm.weight"] = (1 + nrm((hidden,), 0.1)).astype(np.float32)
        T[p + "attn_q.weight"] = nrm((n_q * hd, hidden), sigma)
        T[p + "attn_k.weight"] = nrm((n_kv * hd, hidden), sigma)
        T[p + "attn_v.weight"] = nrm((n_kv * hd, hidden), sigma)
        T[p + "attn_output.weight"] = nrm((hidden, n_q * hd), sigma)
        T[p + "ffn_gate.weight"] = nrm((ffn, hidden), sigma)
        T[p + "ffn_up.weight"] = nrm((ffn, hidden), sigma)
        T[p + "ffn_down.weight"] = nrm((hidden, ffn), sigma)
    kvs = [("general.architecture", gw.STR, "llama"), ("llama.embedding_length", gw.U32, hidden), ("llama.block_count", gw.U32, layers),
           ("llama.attention.head_count", gw.U32, n_q), ("llama.attention.head_count_kv", gw.U32, n_kv),
           ("llama.feed_forward_length", gw.U32, ffn), ("llama.rope.freq_base", gw.F32, 10000.0),
           ("llama.attention.layer_norm_rms_epsilon", gw.F32, 1e-6), ("llama.context_length", gw.U32, 96),
           ("tokenizer.ggml.tokens", gw.ARR, (gw.STR, [f"t{i}" for i in range(vocab)]))]
    tensors, stored = [], {}
    for name, a in T.items():
        file_shape = list(reversed(a.shape))
        enc = encode(name, a) if (encode and a.ndim == 2) else None
        if enc is None:
            tensors.append((name, file_shape, 0, a.tobytes()))
            stored[name] = a
        else:
            ggml_type, raw, back = enc
            tensors.append((name, file_shape, ggml_type, bytes(raw)))
            stored[name] = back
    return gw.build(kvs, tensors), stored


def reference_weights(stored, layers, tied=False):
    """What Llama::from_gguf builds from the stored tensors: transposed linears, fused Q|K|V and gate|up
    (src/models/llama/model.rs:243-257, attention.rs:51-71, decoder.rs:49-67), keyed like LlamaInt8Decoder's weights."""
    from oracle import llama_oracle as lo

    W = {"embedding": stored["token_embd.weight"], "final_norm": stored["output_norm.weight"],
         "lm_head": lo.load_transposed_weight(stored["token_embd.weight" if tied else "output.weight"])}
    for i in range(layers):
        p = f"blk.{i}."
        W[f"l{i}.attn_norm"] = stored[p + "attn_norm.weight"]
        W[f"l{i}.ffn_norm"] = stored[p + "ffn_norm.weight"]
        W[f"l{i}.qkv"] = lo.fuse_qkv(*(lo.load_transposed_weight(stored[p + f"attn_{x}.weight"]) for x in "qkv"))
        W[f"l{i}.o"] = lo.load_transposed_weight(stored[p + "attn_output.weight"])
        W[f"l{i}.gate_up"] = lo.fuse_gate_up(lo.load_transposed_weight(stored[p + "ffn_gate.weight"]), lo.load_transposed_weight(stored[p + "ffn_up.weight"]))
        W[f"l{i}.down"] = lo.load_transposed_weight(stored[p + "ffn_down.weight"])
    return W
