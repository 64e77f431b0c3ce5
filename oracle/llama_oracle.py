"""CPU restatement of the f32 glue of the reference's Llama step (TEST INFRASTRUCTURE: only tests/,
__graft_entry__.smoke() and bench.py's CPU legs may import this; the product never does).

What is restated, in numpy, each function citing the reference code it follows (paths inside
etam103/peregrine):

    StandardKVCache.append         src/attention.rs:65-83      [heads, capacity, head_dim] rows
    gqa_attention_cpu              src/attention.rs:141-265    the scalar (non-aarch64) branch, masks None / Causal
    rmsnorm                        src/nn.rs:577-652           the scalar branch of the inference path
    rope_tables / rope_apply_one   src/nn.rs:1258-1338
    silu_mul                       src/models/llama/decoder.rs:143-150 (non-macOS loop)
    greedy_decode                  examples/llama/main.rs:15-26 (first maximum wins)
    embedding                      src/nn.rs:217-227
    fuse_qkv / fuse_gate_up        src/models/llama/attention.rs:51-71, decoder.rs:49-67
    load_transposed_weight         src/models/llama/model.rs:243-257
    decode_step                    src/models/llama/{attention.rs:73-195, decoder.rs:69-155, model.rs:223-237}
                                   with every `Tensor::matmul` replaced by quant::matmul_quantized (the wiring the
                                   reference left open), the linears taken from the C oracle.

The loop forms (`gqa_attention_cpu`, `rmsnorm_rows`) follow the reference statement by statement and are
what the reference's own tests are re-run on (tests/test_llama_oracle_cpu.py: tests/attention.rs:58-354,
src/nn.rs:4036-4072, 4167-4177).  The vectorised forms (`attention_decode`, `rmsnorm`) compute the same
quantities with numpy reductions (sums in another order) and are held to the loop forms in the same
test file; they are what the GPU tests compare against at sizes the loops would take minutes for.
"""
from __future__ import annotations

import numpy as np

F = np.float32


# ------------------------------------------------------------------ KV cache ----
class StandardKVCache:
    """src/attention.rs:8-99.  k / v: [num_kv_heads, capacity, head_dim], `len` tokens used."""

    def __init__(self, num_kv_heads: int, head_dim: int):
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        self.k = np.zeros((num_kv_heads, 0, head_dim), F)
        self.v = np.zeros((num_kv_heads, 0, head_dim), F)
        self.len = 0
        self.capacity = 0

    def _ensure_capacity(self, needed: int) -> None:      # :31-62: at least double, or to `needed`
        if needed <= self.capacity:
            return
        new_cap = max(needed, max(self.capacity, 16) * 2)
        nk = np.zeros((self.num_kv_heads, new_cap, self.head_dim), F)
        nv = np.zeros_like(nk)
        nk[:, : self.len] = self.k[:, : self.len]
        nv[:, : self.len] = self.v[:, : self.len]
        self.k, self.v, self.capacity = nk, nv, new_cap

    def append(self, new_k, new_v, seq_len: int) -> None:  # :65-83: new_k [heads, seq_len, head_dim]
        new_k = np.asarray(new_k, F).reshape(self.num_kv_heads, seq_len, self.head_dim)
        new_v = np.asarray(new_v, F).reshape(self.num_kv_heads, seq_len, self.head_dim)
        self._ensure_capacity(self.len + seq_len)
        self.k[:, self.len : self.len + seq_len] = new_k
        self.v[:, self.len : self.len + seq_len] = new_v
        self.len += seq_len

    def rollback_to(self, new_len: int) -> None:           # :87-91
        assert new_len <= self.len, f"rollback_to: new_len {new_len} > current len {self.len}"
        self.len = new_len


# ----------------------------------------------------------------- attention ----
def _is_masked(mask, qt: int, kt: int) -> bool:
    """src/attention.rs:267-276 for the two masks the Llama path uses: None, ("causal", offset)."""
    if mask is None:
        return False
    kind, offset = mask
    assert kind == "causal"
    return kt > offset + qt


def gqa_attention_cpu(q, k_cache: StandardKVCache, v_cache: StandardKVCache, num_q_heads: int, num_kv_heads: int, seq_q: int,
                      head_dim: int, scale, mask=None):
    """src/attention.rs:141-265, scalar branch, statement by statement.  q: [num_q_heads, seq_q, head_dim] (rotated);
    returns [seq_q, num_q_heads * head_dim].  f32 throughout, sums in ascending index order."""
    q = np.asarray(q, F).reshape(num_q_heads, seq_q, head_dim)
    total_len = k_cache.len
    group = num_q_heads // num_kv_heads
    scale = F(scale)
    out = np.zeros((seq_q, num_q_heads * head_dim), F)
    for qh in range(num_q_heads):
        kvh = qh // group
        for qt in range(seq_q):
            scores = np.zeros(total_len, F)
            for kt in range(total_len):
                if _is_masked(mask, qt, kt):
                    scores[kt] = -np.inf
                else:
                    d = F(0.0)
                    kr = k_cache.k[kvh, kt]
                    for i in range(head_dim):
                        d = F(d + F(q[qh, qt, i] * kr[i]))
                    scores[kt] = F(d * scale)
            max_score = F(-np.inf)
            for s in scores:
                max_score = max(max_score, s)          # f32::max
            exp_sum = F(0.0)
            with np.errstate(invalid="ignore"):
                for kt in range(total_len):
                    scores[kt] = np.exp(F(scores[kt] - max_score), dtype=F)
                    exp_sum = F(exp_sum + scores[kt])
            if exp_sum > 0.0:
                inv_sum = F(F(1.0) / exp_sum)
                scores = (scores * inv_sum).astype(F)
            o = out[qt, qh * head_dim : (qh + 1) * head_dim]
            for kt in range(total_len):
                w = scores[kt]
                if w > 0.0:
                    vr = v_cache.v[kvh, kt]
                    for dd in range(head_dim):
                        o[dd] = F(o[dd] + F(w * vr[dd]))
    return out


def attention_decode(q, K, V, length: int, group: int):
    """One new token per sequence: q [B, Hq, hd] (rotated), K / V [B, Hkv, cap, hd] with the newest row already at
    position length - 1.  What gqa_attention_cpu computes with seq_q = 1 and mask Causal{offset = length - 1} (every
    cached position visible), vectorised: numpy's reductions add in another order than the reference's loops."""
    B, Hq, hd = q.shape
    out = np.zeros((B, Hq * hd), F)
    scale = F(1.0) / np.sqrt(F(hd))
    for b in range(B):
        for h in range(Hq):
            k = K[b, h // group, :length]
            s = ((k @ q[b, h]).astype(F) * scale).astype(F)
            p = np.exp(s - s.max(), dtype=F)
            p = (p * (F(1.0) / p.sum(dtype=F))).astype(F)
            out[b, h * hd : (h + 1) * hd] = (p[:, None] * V[b, h // group, :length]).sum(axis=0, dtype=F)
    return out


# ---------------------------------------------------------------- row kernels ----
def rmsnorm_rows(x, w, eps):
    """src/nn.rs:643-652 (scalar branch): ss = sum of squares in index order, inv_rms = 1 / sqrt(ss * (1/dim) + eps),
    out = x * inv_rms * w (two rounded products, left to right)."""
    x = np.asarray(x, F)
    rows, dim = x.shape
    inv_dim = F(F(1.0) / F(dim))
    out = np.zeros_like(x)
    for r in range(rows):
        ss = F(0.0)
        for v in x[r]:
            ss = F(ss + F(v * v))
        inv_rms = F(F(1.0) / np.sqrt(F(F(ss * inv_dim) + F(eps)), dtype=F))
        out[r] = ((x[r] * inv_rms).astype(F) * w).astype(F)
    return out


def rmsnorm(x, w, eps):
    """rmsnorm_rows with numpy reductions (sum of squares in another order)."""
    x = np.asarray(x, F)
    ss = (x * x).sum(axis=1, dtype=F)
    inv = (F(1.0) / np.sqrt(ss * F(F(1.0) / F(x.shape[1])) + F(eps), dtype=F)).astype(F)
    return ((x * inv[:, None]).astype(F) * np.asarray(w, F)[None, :]).astype(F)


def rope_tables(head_dim: int, max_pos: int, base):
    """RoPE::new (src/nn.rs:1258-1283): theta = pos / base^(2i / head_dim) in f32; cos, sin [max_pos, head_dim / 2]
    (the reference stores each row twice over; the second half repeats the first)."""
    half = head_dim // 2
    i = np.arange(half, dtype=F)
    inv = np.power(F(base), F(2.0) * i / F(head_dim)).astype(F)
    theta = (np.arange(max_pos, dtype=F)[:, None] / inv[None, :]).astype(F)
    return np.cos(theta).astype(F), np.sin(theta).astype(F)


def rope_apply(v, cos_row, sin_row):
    """RoPE::apply_one (src/nn.rs:1322-1338) on the last axis: [x0 c - x1 s | x0 s + x1 c]."""
    v = np.asarray(v, F)
    half = v.shape[-1] // 2
    x0, x1 = v[..., :half], v[..., half:]
    return np.concatenate([(x0 * cos_row).astype(F) - (x1 * sin_row).astype(F), (x0 * sin_row).astype(F) + (x1 * cos_row).astype(F)],
                          axis=-1).astype(F)


def silu_mul(gate, up):
    """src/models/llama/decoder.rs:143-150: g / (1 + exp(-g)) * up."""
    gate, up = np.asarray(gate, F), np.asarray(up, F)
    return ((gate / (F(1.0) + np.exp(-gate, dtype=F))).astype(F) * up).astype(F)


def greedy_decode(logits_row) -> int:
    """examples/llama/main.rs:15-26: strict '>' from -inf, so the first maximum wins and an all-NaN row gives 0."""
    best_idx, best_val = 0, F(-np.inf)
    for i, v in enumerate(np.asarray(logits_row, F)):
        if v > best_val:
            best_val, best_idx = v, i
    return best_idx


def embedding(table, tokens):
    """Embedding::forward (src/nn.rs:217-227)."""
    return np.asarray(table, F)[np.asarray(tokens, np.int64)]


# ------------------------------------------------------------- weight layout ----
def load_transposed_weight(w_out_in):
    """src/models/llama/model.rs:243-257: GGUF [out, in] row-major -> [in, out]."""
    return np.ascontiguousarray(np.asarray(w_out_in, F).T)


def fuse_qkv(q_proj, k_proj, v_proj):
    """src/models/llama/attention.rs:51-71: columns [Q | K | V] of [model_dim, q_dim + 2 kv_dim]."""
    return np.ascontiguousarray(np.concatenate([q_proj, k_proj, v_proj], axis=1), F)


def fuse_gate_up(gate_proj, up_proj):
    """src/models/llama/decoder.rs:49-67: columns [gate | up] of [model_dim, 2 ffn_dim]."""
    return np.ascontiguousarray(np.concatenate([gate_proj, up_proj], axis=1), F)


# ---------------------------------------------------------------- decode step ----
def decode_step(orc, cfg, W, Q, x, K, V, pos: int, cos, sin, trace=None):
    """One decode step for `cfg.batch` independent sequences at position `pos`.

    W: f32 norm weights; Q: oracle QuantizedTensors of the five linears per layer ("l{i}.qkv", "l{i}.o",
    "l{i}.gate_up", "l{i}.down", "lm_head", all [in, out]); x [B, hidden] embedded tokens; K, V per layer
    [B, Hkv, cap, hd] (updated in place at `pos`).  Returns the logits [B, vocab].  `trace` (a dict) receives the f32
    inputs of every quantised linear, keyed like Q."""
    B, H, Hq, Hkv, hd = cfg.batch, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    x = np.asarray(x, F)
    delta = None

    def note(key, a):
        if trace is not None:
            trace[key] = a

    for i in range(cfg.layers):
        if delta is not None:
            x = (x + delta).astype(F)
        n = rmsnorm(x, W[f"l{i}.attn_norm"], cfg.eps)
        note(f"l{i}.qkv", n)
        qkv = orc.matmul_quantized(n, B, H, Q[f"l{i}.qkv"]).reshape(B, Hq + 2 * Hkv, hd)
        q = rope_apply(qkv[:, :Hq], cos[pos], sin[pos])
        K[i][:, :, pos] = rope_apply(qkv[:, Hq : Hq + Hkv], cos[pos], sin[pos])
        V[i][:, :, pos] = qkv[:, Hq + Hkv :]
        a = attention_decode(q, K[i], V[i], pos + 1, Hq // Hkv)
        note(f"l{i}.o", a)
        o = orc.matmul_quantized(a, B, Hq * hd, Q[f"l{i}.o"])
        x = (x + o).astype(F)
        n = rmsnorm(x, W[f"l{i}.ffn_norm"], cfg.eps)
        note(f"l{i}.gate_up", n)
        gu = orc.matmul_quantized(n, B, H, Q[f"l{i}.gate_up"])
        act = silu_mul(gu[:, : cfg.ffn], gu[:, cfg.ffn :])
        note(f"l{i}.down", act)
        delta = orc.matmul_quantized(act, B, cfg.ffn, Q[f"l{i}.down"])
    if delta is not None:
        x = (x + delta).astype(F)
    n = rmsnorm(x, W["final_norm"], cfg.eps)
    note("lm_head", n)
    return orc.matmul_quantized(n, B, H, Q["lm_head"])
