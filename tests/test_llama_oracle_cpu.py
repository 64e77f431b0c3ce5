"""Pins oracle/llama_oracle.py (the CPU restatement of the reference's Llama glue that the GPU tests
check against) to the reference's own tests for those functions: same closed-form inputs, same
expected values, same tolerances.  Each test names the reference test it re-runs."""
import numpy as np
import pytest

from oracle import llama_oracle as lo

F = np.float32


def naive_attention(q, k, v, seq_q, seq_kv, head_dim, scale, causal, offset):
    """The single-head check the reference's tests carry themselves (tests/attention.rs:5-56)."""
    q = np.asarray(q, F).reshape(seq_q, head_dim)
    k = np.asarray(k, F).reshape(seq_kv, head_dim)
    v = np.asarray(v, F).reshape(seq_kv, head_dim)
    out = np.zeros((seq_q, head_dim), F)
    for qt in range(seq_q):
        scores = np.zeros(seq_kv, F)
        for kt in range(seq_kv):
            if causal and kt > offset + qt:
                scores[kt] = -np.inf
            else:
                dot = F(0.0)
                for d in range(head_dim):
                    dot = F(dot + F(q[qt, d] * k[kt, d]))
                scores[kt] = F(dot * F(scale))
        max_s = scores.max()
        scores = np.exp(scores - max_s, dtype=F)
        exp_sum = F(0.0)
        for s in scores:
            exp_sum = F(exp_sum + s)
        if exp_sum > 0:
            scores = (scores / exp_sum).astype(F)
        for kt in range(seq_kv):
            if scores[kt] > 0:
                out[qt] = (out[qt] + scores[kt] * v[kt]).astype(F)
    return out


def _seq(n, step, fn):
    return fn(np.arange(n, dtype=F) * F(step)).astype(F)


def _run_grouped(num_q_heads, num_kv_heads, head_dim, seq_q, seq_kv):
    # inputs of tests/attention.rs:66-81, 137-152, 216-231: sin(0.1 i), cos(0.2 i), sin(0.15 i)
    q = _seq(num_q_heads * seq_q * head_dim, 0.1, np.sin)
    k = _seq(num_kv_heads * seq_kv * head_dim, 0.2, np.cos)
    v = _seq(num_kv_heads * seq_kv * head_dim, 0.15, np.sin)
    cache = lo.StandardKVCache(num_kv_heads, head_dim)
    cache.append(k, v, seq_kv)
    scale = F(1.0) / np.sqrt(F(head_dim))
    out = lo.gqa_attention_cpu(q, cache, cache, num_q_heads, num_kv_heads, seq_q, head_dim, scale, None)
    group = num_q_heads // num_kv_heads
    for qh in range(num_q_heads):
        kvh = qh // group
        q_head = q.reshape(num_q_heads, seq_q, head_dim)[qh]
        expected = naive_attention(q_head, cache.k[kvh, :seq_kv], cache.v[kvh, :seq_kv], seq_q, seq_kv, head_dim, scale, False, 0)
        got = out[:, qh * head_dim:(qh + 1) * head_dim]
        assert np.abs(got - expected).max() < 1e-5, f"head {qh}"


def test_gqa_matches_naive_mha():
    """tests/attention.rs:58-127: 2 heads of 8, 3 queries, 5 cached positions, no grouping."""
    _run_grouped(2, 2, 8, 3, 5)


def test_gqa_with_grouping():
    """tests/attention.rs:129-200: 4 query heads on 2 KV heads."""
    _run_grouped(4, 2, 4, 2, 3)


def test_mqa_fallback():
    """tests/attention.rs:202-266: 4 query heads on one KV head."""
    _run_grouped(4, 1, 4, 2, 3)


@pytest.mark.parametrize("seq_q,seq_kv,offset", [(3, 3, 0), (1, 6, 5)])
def test_causal_mask(seq_q, seq_kv, offset):
    """tests/attention.rs:268-311 (offset 0) and :313-354 (one query after a prompt of five)."""
    head_dim = 4
    q = _seq(seq_q * head_dim, 0.1, np.sin)
    k = _seq(seq_kv * head_dim, 0.2, np.cos)
    v = _seq(seq_kv * head_dim, 0.15, np.sin)
    cache = lo.StandardKVCache(1, head_dim)
    cache.append(k, v, seq_kv)
    scale = F(1.0) / np.sqrt(F(head_dim))
    out = lo.gqa_attention_cpu(q, cache, cache, 1, 1, seq_q, head_dim, scale, ("causal", offset))
    expected = naive_attention(q, k, v, seq_q, seq_kv, head_dim, scale, True, offset)
    assert np.abs(out - expected).max() < 1e-5


def test_kv_cache_growth_keeps_rows():
    """StandardKVCache::ensure_capacity (src/attention.rs:31-62): rows survive the re-layout to a larger capacity."""
    g = np.random.Generator(np.random.PCG64(3))
    cache = lo.StandardKVCache(2, 4)
    rows_k, rows_v = [], []
    for n in (3, 20, 1, 40):
        k, v = g.standard_normal((2, n, 4)).astype(F), g.standard_normal((2, n, 4)).astype(F)
        cache.append(k, v, n)
        rows_k.append(k)
        rows_v.append(v)
    assert cache.len == 64 and cache.capacity >= 64
    assert np.array_equal(cache.k[:, :64], np.concatenate(rows_k, axis=1))
    assert np.array_equal(cache.v[:, :64], np.concatenate(rows_v, axis=1))
    cache.rollback_to(10)
    assert cache.len == 10
    with pytest.raises(AssertionError):
        cache.rollback_to(11)


def test_rmsnorm_forward():
    """src/nn.rs:4036-4057: [1, 2, 3, 4], eps 1e-5, unit weights."""
    out = lo.rmsnorm_rows(np.array([[1, 2, 3, 4]], F), np.ones(4, F), 1e-5)
    rms = np.sqrt(F(7.5) + F(1e-5))
    for fn in (lo.rmsnorm_rows, lo.rmsnorm):
        out = fn(np.array([[1, 2, 3, 4]], F), np.ones(4, F), 1e-5)
        assert np.abs(out[0] - np.arange(1, 5, dtype=F) / rms).max() < 1e-4


def test_rmsnorm_batch():
    """src/nn.rs:4060-4076: rows [3, 4] and [1, 0]."""
    for fn in (lo.rmsnorm_rows, lo.rmsnorm):
        out = fn(np.array([[3, 4], [1, 0]], F), np.ones(2, F), 1e-5)
        rms0, rms1 = np.sqrt(F(12.5)), np.sqrt(F(0.5))
        assert abs(out[0, 0] - 3 / rms0) < 1e-4 and abs(out[0, 1] - 4 / rms0) < 1e-4
        assert abs(out[1, 0] - 1 / rms1) < 1e-4 and abs(out[1, 1]) < 1e-4


def test_rope():
    """src/nn.rs:4167-4177: position 0 leaves the input unchanged; plus the rotation itself at a later position."""
    cos, sin = lo.rope_tables(4, 128, 10000.0)
    x = np.array([[1, 0, 1, 0], [0, 1, 0, 1]], F)
    out = np.stack([lo.rope_apply(x[t], cos[t], sin[t]) for t in range(2)])
    assert abs(out[0, 0] - 1.0) < 1e-5 and abs(out[0, 1]) < 1e-5
    # row 1 at position 1: pairs (x[i], x[half + i]) rotated by theta_i = 1 / 10000^(2i/4)
    th = np.array([1.0, 1.0 / 100.0])
    exp = np.array([0 * np.cos(th[0]) - 0 * np.sin(th[0]), 1 * np.cos(th[1]) - 1 * np.sin(th[1]),
                    0 * np.sin(th[0]) + 0 * np.cos(th[0]), 1 * np.sin(th[1]) + 1 * np.cos(th[1])])
    assert np.abs(out[1] - exp).max() < 1e-6


def test_greedy_and_embedding():
    """examples/llama/main.rs:15-26 (first maximum, NaN never wins) and src/nn.rs:217-227."""
    assert lo.greedy_decode(np.array([1, 5, 5, 2], F)) == 1
    assert lo.greedy_decode(np.array([np.nan, np.nan], F)) == 0
    assert lo.greedy_decode(np.array([np.nan, -3, np.nan], F)) == 1
    t = np.arange(12, dtype=F).reshape(4, 3)
    assert np.array_equal(lo.embedding(t, [3, 0]), t[[3, 0]])


def test_weight_layout():
    """load_transposed_weight (model.rs:243-257), fuse_qkv (attention.rs:51-71), fuse_gate_up (decoder.rs:49-67)."""
    g = np.random.Generator(np.random.PCG64(5))
    wq, wk, wv = (g.standard_normal(s).astype(F) for s in ((8, 6), (4, 6), (4, 6)))      # GGUF [out, in]
    q, k, v = (lo.load_transposed_weight(w) for w in (wq, wk, wv))
    assert q.shape == (6, 8) and q[2, 5] == wq[5, 2]
    fused = lo.fuse_qkv(q, k, v)
    assert fused.shape == (6, 16)
    assert np.array_equal(fused[:, :8], q) and np.array_equal(fused[:, 8:12], k) and np.array_equal(fused[:, 12:], v)
    gu = lo.fuse_gate_up(q, q * 2)
    assert np.array_equal(gu[:, :8], q) and np.array_equal(gu[:, 8:], q * 2)


def test_vectorised_forms_match_the_loops():
    """attention_decode / rmsnorm (numpy reductions) against the statement-by-statement forms."""
    g = np.random.Generator(np.random.PCG64(11))
    B, Hq, Hkv, hd, length, cap = 2, 4, 2, 16, 37, 40
    q = g.standard_normal((B, Hq, hd)).astype(F)
    K = g.standard_normal((B, Hkv, cap, hd)).astype(F)
    V = g.standard_normal((B, Hkv, cap, hd)).astype(F)
    fast = lo.attention_decode(q, K, V, length, Hq // Hkv)
    for b in range(B):
        cache = lo.StandardKVCache(Hkv, hd)
        cache.append(K[b, :, :length], V[b, :, :length], length)
        slow = lo.gqa_attention_cpu(q[b], cache, cache, Hq, Hkv, 1, hd, F(1.0) / np.sqrt(F(hd)), ("causal", length - 1))
        assert np.abs(fast[b] - slow[0]).max() <= 2e-6 * np.abs(slow).max()
    x = g.standard_normal((3, 200)).astype(F)
    w = (1 + 0.1 * g.standard_normal(200)).astype(F)
    a, b_ = lo.rmsnorm(x, w, 1e-5), lo.rmsnorm_rows(x, w, 1e-5)
    assert np.abs(a - b_).max() <= 1e-6 * np.abs(b_).max()
    gate, up = g.standard_normal((2, 50)).astype(F), g.standard_normal((2, 50)).astype(F)
    ref = np.array([[F(F(gg / F(F(1.0) + np.exp(F(-gg), dtype=F))) * uu) for gg, uu in zip(gr, ur)] for gr, ur in zip(gate, up)], F)
    assert np.abs(lo.silu_mul(gate, up) - ref).max() <= 1e-7
