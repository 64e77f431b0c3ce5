"""The Llama decode glue (csrc/pg_llama.cu) and the int8 decode step built from it
(peregrine_b200/llama.py), against a numpy restatement of the reference's host code
(src/nn.rs RMSNorm / RoPE, src/attention.rs gqa_attention_cpu, src/models/llama/{attention,decoder,model}.rs)
with the CPU oracle's matmul_quantized for the linears.

Bars: RoPE, KV append, embedding, argmax: bit-exact.  RMSNorm, SwiGLU, attention: f32 sums in another
order, 1e-5 of the row maximum.  Whole step (teacher-forced tokens): logits within 5e-3 of max|logit| --
a quantised activation can land on the other side of a rounding tie when its f32 input differs in the
last bit, which moves a logit by about one quantisation step of one activation."""
import ctypes as C

import numpy as np
import pytest

from _inputs import normal, rng

pytestmark = pytest.mark.gpu


def _t(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rmsnorm_ref(x, w, eps):
    ss = (x.astype(np.float32) ** 2).sum(axis=1, dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(ss * np.float32(1.0 / x.shape[1]) + np.float32(eps), dtype=np.float32)
    return (x * inv[:, None] * w[None, :]).astype(np.float32)


def rope_ref(v, cos, sin):
    half = v.shape[-1] // 2
    x0, x1 = v[..., :half], v[..., half:]
    return np.concatenate([x0 * cos - x1 * sin, x0 * sin + x1 * cos], axis=-1).astype(np.float32)


def attention_ref(q, K, V, length, group):
    """q [B,Hq,hd]; K,V [B,Hkv,cap,hd]; softmax(q.k / sqrt(hd)) V over positions < length."""
    B, Hq, hd = q.shape
    out = np.zeros((B, Hq * hd), np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(hd)))
    for b in range(B):
        for h in range(Hq):
            k = K[b, h // group, :length]
            s = (k @ q[b, h]).astype(np.float32) * scale
            p = np.exp(s - s.max(), dtype=np.float32)
            p = p / p.sum(dtype=np.float32)
            out[b, h * hd:(h + 1) * hd] = (p[:, None] * V[b, h // group, :length]).sum(axis=0, dtype=np.float32)
    return out


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def test_add_rmsnorm_quantize(pg, gpu, oracle):
    import torch
    from peregrine_b200 import _lib

    g = rng(1)
    for rows, dim, with_delta in ((16, 4096, True), (3, 256, False), (5, 14336, True)):
        x = normal(g, (rows, dim))
        d = normal(g, (rows, dim), 0.5)
        w = (1.0 + normal(g, (dim,), 0.1)).astype(np.float32)
        tx, td, tw = _t(x), _t(d), _t(w)
        q = torch.zeros(rows * dim, dtype=torch.int8, device="cuda")
        s = torch.zeros(rows, device="cuda")
        n = torch.zeros(rows, dim, device="cuda")
        torch.cuda.synchronize()
        _lib.check(gpu.lib.pg_add_rmsnorm_quantize(gpu.handle, tx.data_ptr(), td.data_ptr() if with_delta else None, tw.data_ptr(), rows, dim,
                                                   1e-5, q.data_ptr(), s.data_ptr(), n.data_ptr()))
        gpu.sync()
        xs = (x + d).astype(np.float32) if with_delta else x
        assert np.array_equal(tx.cpu().numpy(), xs)                     # residual stream updated exactly
        ref = rmsnorm_ref(xs, w, 1e-5)
        got = n.cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
        # the quantiser applied to the kernel's own normalised rows is the oracle's, bit for bit
        qo, so = oracle.quantize_activations(got, rows, dim)
        assert np.array_equal(q.cpu().numpy().reshape(rows, dim), qo) and np.array_equal(s.cpu().numpy(), so)


def test_swiglu_quantize(pg, gpu, oracle):
    import torch
    from peregrine_b200 import _lib

    g = rng(2)
    for rows, F in ((16, 14336), (2, 64)):
        gu = normal(g, (rows, 2 * F), 2.0)
        tgu = _t(gu)
        q = torch.zeros(rows * F, dtype=torch.int8, device="cuda")
        s = torch.zeros(rows, device="cuda")
        a = torch.zeros(rows, F, device="cuda")
        torch.cuda.synchronize()
        _lib.check(gpu.lib.pg_swiglu_quantize(gpu.handle, tgu.data_ptr(), rows, F, q.data_ptr(), s.data_ptr(), a.data_ptr()))
        gpu.sync()
        gate, up = gu[:, :F], gu[:, F:]
        ref = (gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)) * up).astype(np.float32)
        got = a.cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
        qo, so = oracle.quantize_activations(got, rows, F)
        assert np.array_equal(q.cpu().numpy().reshape(rows, F), qo) and np.array_equal(s.cpu().numpy(), so)


def test_rope_append_attention_embedding_argmax(pg, gpu, oracle):
    import torch
    from peregrine_b200 import _lib
    from peregrine_b200.llama import rope_tables

    g = rng(3)
    lib = gpu.lib
    hd = 128
    # 4 and 8 query heads per KV head take the streaming kernel, 1 and 2 the chunked one; first position, ragged slices,
    # more (sequence, head, slice) units than the GPU has warps
    for B, Hq, Hkv, cap, pos in ((3, 8, 2, 300, 7), (3, 8, 2, 1100, 1099), (3, 8, 2, 2200, 2047), (2, 16, 2, 700, 0), (2, 16, 2, 700, 650),
                                 (1, 4, 2, 600, 333), (2, 2, 2, 300, 299), (40, 32, 8, 200, 130), (16, 32, 8, 2176, 2048),
                                 # capacities whose slices are not multiples of four positions (chunked kernel: 513 per slice)
                                 (2, 2, 1, 4100, 0), (2, 2, 2, 4100, 901), (3, 2, 1, 2178, 2158), (1, 8, 8, 66, 10), (5, 8, 1, 301, 86)):
        cos, sin = rope_tables(hd, cap, 500000.0)
        qkv = normal(g, (B, (Hq + 2 * Hkv) * hd))
        K = normal(g, (B, Hkv, cap, hd))
        V = normal(g, (B, Hkv, cap, hd))
        tq, tK, tV, tc, ts = _t(qkv), _t(K), _t(V), _t(cos), _t(sin)
        tpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        qrot = torch.zeros(B, Hq, hd, device="cuda")
        S = lib.pg_gqa_decode_splits(gpu.handle, B, Hq, Hkv, cap)
        work = torch.zeros(B * Hq * S * 130, device="cuda")
        out = torch.zeros(B, Hq * hd, device="cuda")
        torch.cuda.synchronize()
        _lib.check(lib.pg_rope_kv_append(gpu.handle, tq.data_ptr(), tpos.data_ptr(), tc.data_ptr(), ts.data_ptr(), B, Hq, Hkv, hd, cap,
                                         qrot.data_ptr(), tK.data_ptr(), tV.data_ptr()))
        o8 = torch.zeros(B, Hq * hd, dtype=torch.int8, device="cuda")
        o8s = torch.zeros(B, device="cuda")
        _lib.check(lib.pg_gqa_attention_decode(gpu.handle, qrot.data_ptr(), tK.data_ptr(), tV.data_ptr(), tpos.data_ptr(), B, Hq, Hkv, hd, cap,
                                               work.data_ptr(), out.data_ptr(), o8.data_ptr(), o8s.data_ptr()))
        gpu.sync()
        heads = qkv.reshape(B, Hq + 2 * Hkv, hd)
        q_ref = rope_ref(heads[:, :Hq], cos[pos], sin[pos])
        k_ref = rope_ref(heads[:, Hq:Hq + Hkv], cos[pos], sin[pos])
        assert np.array_equal(qrot.cpu().numpy(), q_ref)                       # RoPE: same table, same two products -> bit-exact
        K2, V2 = K.copy(), V.copy()
        K2[:, :, pos], V2[:, :, pos] = k_ref, heads[:, Hq + Hkv:]
        assert np.array_equal(tK.cpu().numpy(), K2) and np.array_equal(tV.cpu().numpy(), V2)
        ref = attention_ref(q_ref, K2, V2, pos + 1, Hq // Hkv)
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
        # the fused quantiser: bit-exact with the oracle's quantiser applied to the f32 rows the kernel produced
        qo, so = oracle.quantize_activations(out.cpu().numpy(), B, Hq * hd)
        assert np.array_equal(o8.cpu().numpy(), qo) and np.array_equal(o8s.cpu().numpy(), so)
        if Hq // Hkv in (4, 8):
            # RoPE + append inside the attention kernel: the same cache bits, the same output to the last few ulps
            fK, fV = _t(K), _t(V)
            fout = torch.zeros(B, Hq * hd, device="cuda")
            torch.cuda.synchronize()
            _lib.check(lib.pg_gqa_attention_decode_fused(gpu.handle, tq.data_ptr(), tpos.data_ptr(), tc.data_ptr(), ts.data_ptr(), fK.data_ptr(),
                                                         fV.data_ptr(), B, Hq, Hkv, hd, cap, work.data_ptr(), fout.data_ptr(), None, None))
            gpu.sync()
            assert np.array_equal(fK.cpu().numpy(), K2) and np.array_equal(fV.cpu().numpy(), V2)
            assert np.abs(fout.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
            assert gpu.device_status() == 0
    # embedding and argmax (first maximum; the position is advanced once)
    table = normal(g, (50, 64))
    tok = np.array([3, 49, 0], np.int32)
    o = torch.zeros(3, 64, device="cuda")
    tt, ttok = _t(table), _t(tok)
    torch.cuda.synchronize()
    _lib.check(lib.pg_embedding(gpu.handle, tt.data_ptr(), ttok.data_ptr(), 3, 64, o.data_ptr()))
    logits = normal(g, (3, 5000))
    logits[0, 77] = logits[0, 4000] = 9.0
    logits[1, :] = -1.0
    tl = _t(logits)
    picks = torch.zeros(3, dtype=torch.int32, device="cuda")
    p = torch.tensor([5], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.pg_argmax_advance(gpu.handle, tl.data_ptr(), 3, 5000, picks.data_ptr(), p.data_ptr()))
    gpu.sync()
    assert np.array_equal(o.cpu().numpy(), table[tok])
    assert picks.cpu().numpy().tolist() == [77, 0, int(np.argmax(logits[2]))] and int(p.item()) == 6
    # a vocabulary wide enough for the row to be spread over a cluster: ties across segment borders, maximum in the last segment
    big = normal(g, (5, 128256))
    big[0, 100] = big[0, 128255] = 11.0
    big[1, 128255] = 12.0
    big[2, 16031] = big[2, 16032] = 13.0
    big[3, :] = 0.5
    tb = _t(big)
    picks = torch.zeros(5, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.pg_argmax_advance(gpu.handle, tb.data_ptr(), 5, 128256, picks.data_ptr(), p.data_ptr()))
    gpu.sync()
    assert picks.cpu().numpy().tolist() == [100, 128255, 16031, 0, int(np.argmax(big[4]))] and int(p.item()) == 7


def _ref_step(orc, cfg, W, Q, x, K, V, pos, cos, sin):
    """One decode step in numpy; returns logits and the updated residual stream is discarded."""
    B, H, Hq, Hkv, hd = cfg.batch, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    delta = None
    for i in range(cfg.layers):
        if delta is not None:
            x = (x + delta).astype(np.float32)
        n = rmsnorm_ref(x, W[f"l{i}.attn_norm"], cfg.eps)
        qkv = orc.matmul_quantized(n, B, H, Q[f"l{i}.qkv"]).reshape(B, Hq + 2 * Hkv, hd)
        q = rope_ref(qkv[:, :Hq], cos[pos], sin[pos])
        K[i][:, :, pos] = rope_ref(qkv[:, Hq:Hq + Hkv], cos[pos], sin[pos])
        V[i][:, :, pos] = qkv[:, Hq + Hkv:]
        a = attention_ref(q, K[i], V[i], pos + 1, Hq // Hkv)
        o = orc.matmul_quantized(a, B, H, Q[f"l{i}.o"])
        x = (x + o).astype(np.float32)
        n = rmsnorm_ref(x, W[f"l{i}.ffn_norm"], cfg.eps)
        gu = orc.matmul_quantized(n, B, H, Q[f"l{i}.gate_up"])
        gate, up = gu[:, :cfg.ffn], gu[:, cfg.ffn:]
        act = (gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)) * up).astype(np.float32)
        delta = orc.matmul_quantized(act, B, cfg.ffn, Q[f"l{i}.down"])
    x = (x + delta).astype(np.float32)
    n = rmsnorm_ref(x, W["final_norm"], cfg.eps)
    return orc.matmul_quantized(n, B, H, Q["lm_head"])


@pytest.mark.parametrize("heads,kv_heads,ffn,vocab,batch,capacity", [
    (4, 2, 512, 1000, 3, 40),       # two query heads per KV head: RoPE and attention as separate kernels
    (8, 2, 1024, 2000, 2, 70),      # four: RoPE and the cache append inside the attention kernel
    (8, 1, 768, 520, 17, 33),       # eight, and more than 16 sequences: the products leave the decode kernel
    (2, 2, 640, 300, 1, 37),        # one, a single sequence
])
def test_decode_steps_teacher_forced(pg, gpu, oracle_mt, heads, kv_heads, ffn, vocab, batch, capacity):
    import torch
    from peregrine_b200.llama import LlamaConfig, LlamaInt8Decoder, rope_tables

    cfg = LlamaConfig(layers=2, hidden=heads * 128, n_q_heads=heads, n_kv_heads=kv_heads, head_dim=128, ffn=ffn, vocab=vocab, batch=batch,
                      capacity=capacity)        # o_proj input = heads * head_dim = hidden, as in Llama
    g = rng(4 + heads + batch)
    W = {"embedding": normal(g, (cfg.vocab, cfg.hidden), 0.5), "final_norm": (1 + normal(g, (cfg.hidden,), 0.1)).astype(np.float32),
         "lm_head": normal(g, (cfg.hidden, cfg.vocab), 0.02)}
    for i in range(cfg.layers):
        W[f"l{i}.attn_norm"] = (1 + normal(g, (cfg.hidden,), 0.1)).astype(np.float32)
        W[f"l{i}.ffn_norm"] = (1 + normal(g, (cfg.hidden,), 0.1)).astype(np.float32)
        W[f"l{i}.qkv"] = normal(g, (cfg.hidden, cfg.qkv_dim), 0.05)
        W[f"l{i}.o"] = normal(g, (cfg.hidden, cfg.hidden), 0.05)
        W[f"l{i}.gate_up"] = normal(g, (cfg.hidden, 2 * cfg.ffn), 0.05)
        W[f"l{i}.down"] = normal(g, (cfg.ffn, cfg.hidden), 0.05)
    Q = {k: oracle_mt.quantize_weights(v, v.shape[0], v.shape[1]) for k, v in W.items() if v.ndim == 2 and k != "embedding"}
    model = LlamaInt8Decoder(cfg, gpu, W)
    # a short synthetic history in the cache
    start = 5
    K = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    V = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    for i in range(cfg.layers):
        model.kcache[i].copy_(_t(K[i]))
        model.vcache[i].copy_(_t(V[i]))
    cos, sin = rope_tables(cfg.head_dim, cfg.capacity, cfg.rope_base)
    tokens = g.integers(0, cfg.vocab, cfg.batch).astype(np.int32)
    tokens[0] = cfg.vocab - 1
    model.set_position(start)
    model.set_tokens(tokens)
    torch.cuda.synchronize()
    model.embed()
    graph = model.record()
    for step in range(3):
        x = W["embedding"][tokens]
        ref_logits = _ref_step(oracle_mt, cfg, W, Q, x, K, V, start + step, cos, sin)
        graph.launch()
        gpu.sync()
        assert gpu.device_status() == 0
        got = model.logits.cpu().numpy()
        # f32 sums in another order can move an activation across a rounding boundary of one of the eleven quantisers on
        # the way: that sequence's logits then differ by a quantisation step's worth (seen: 6e-3 of max|logit|), all
        # others agree to f32 accuracy.  Every sequence within 2e-2, and all but a few within 5e-3.
        scale = np.abs(ref_logits).max()
        tol = 2e-2 * scale
        rows_err = np.abs(got - ref_logits).max(axis=1)
        assert rows_err.max() <= tol, f"step {step}: per-sequence max error {np.array2string(rows_err, precision=2)} > {tol}"
        assert int((rows_err > 5e-3 * scale).sum()) <= max(1, cfg.batch // 8), f"step {step}: {np.array2string(rows_err, precision=2)}"
        assert int(model.pos.item()) == start + step + 1
        picked = model.tokens.cpu().numpy()
        srt = np.sort(ref_logits, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 2 * tol
        assert np.array_equal(picked[clear], np.argmax(ref_logits, axis=1)[clear])
        # teacher forcing: continue from the oracle's greedy choice on both sides
        tokens = np.argmax(ref_logits, axis=1).astype(np.int32)
        model.set_tokens(tokens)
        model.embed()
        gpu.sync()
        # the caches must agree too (same rounding path for k, v up to the f32 tolerance of their inputs)
        assert np.abs(model.kcache[0][:, :, start + step].cpu().numpy() - K[0][:, :, start + step]).max() <= 1e-2
    model.free()
