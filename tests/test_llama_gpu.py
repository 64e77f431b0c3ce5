"""The Llama decode glue (csrc/pg_llama.cu) and the int8 decode step built from it
(peregrine_b200/llama.py), against oracle/llama_oracle.py: the CPU restatement of the reference's host code
(src/nn.rs RMSNorm / RoPE, src/attention.rs gqa_attention_cpu, src/models/llama/{attention,decoder,model}.rs), which
tests/test_llama_oracle_cpu.py pins to the reference's own tests, with the C oracle's matmul_quantized for the linears.

Bars: RoPE, KV append, embedding, argmax: bit-exact.  RMSNorm, SwiGLU, attention: f32 sums in another
order, 1e-5 of the row maximum.  Whole step (teacher-forced tokens): the quantised rows that enter every linear are
compared with the oracle's element by element; a sequence none of whose quantised elements differs must give
bit-identical logits, and the logits of every other sequence must lie within what the differing elements of the
last quantiser can move them (elements x one quantisation step x the largest weight)."""
import ctypes as C

import numpy as np
import pytest

from _inputs import normal, rng
from oracle import llama_oracle as lo

pytestmark = pytest.mark.gpu


def _t(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


rmsnorm_ref = lo.rmsnorm
rope_ref = lo.rope_apply
attention_ref = lo.attention_decode


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
        ref = lo.silu_mul(gate, up)
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
    _lib.check(lib.pg_argmax_advance(gpu.handle, tl.data_ptr(), 3, 5000, picks.data_ptr(), p.data_ptr(), 0))
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
    _lib.check(lib.pg_argmax_advance(gpu.handle, tb.data_ptr(), 5, 128256, picks.data_ptr(), p.data_ptr(), 0))
    gpu.sync()
    assert picks.cpu().numpy().tolist() == [100, 128255, 16031, 0, int(np.argmax(big[4]))] and int(p.item()) == 7


LINEAR_IN_DIM = {"qkv": "hidden", "o": "attn", "gate_up": "hidden", "down": "ffn", "lm_head": "hidden"}


def run_step_with_taps(model, gpu):
    """One eager, unsharded step of `model`, stopping after every launch that a linear follows or makes:
    name + ".in"  -> (i8 rows [B, dim], scales [B], residual stream x [B, hidden]) as the linear `name` received them,
    name + ".out" -> the linear's f32 output."""
    c = model.cfg
    dims = {"hidden": c.hidden, "attn": c.n_q_heads * c.head_dim, "ffn": c.ffn}
    outs = {"qkv": lambda: model.qkv, "o": lambda: model.o, "gate_up": lambda: model.gate_up, "down": lambda: model.down,
            "lm_head": lambda: model.logits}
    taps = {}
    for label in model.step_ops():
        name, _, kind = label.rpartition(".")
        if kind == "in":
            dim = dims[LINEAR_IN_DIM[name.split(".")[-1]]]
            gpu.sync()
            taps[label] = (model.q8[: c.batch * dim].cpu().numpy().reshape(c.batch, dim).copy(), model.q8s.cpu().numpy().copy(),
                           model.x.cpu().numpy().copy())
        elif kind == "out":
            gpu.sync()
            taps[label] = outs[name.split(".")[-1]]().cpu().numpy().copy()
    gpu.sync()
    return taps


def check_stages(orc, cfg, W, Q, taps, x, K, V, pos, cos, sin, what=""):
    """Walks the step stage by stage, every stage fed with what the GPU itself produced before it:
      * a linear given the GPU's quantised rows must reproduce the GPU's output bit for bit (integer sums);
      * the residual stream must be the exact f32 sum of the GPU's own linear outputs;
      * the oracle's glue (RMSNorm, RoPE + attention over the cache, SiLU(g) u) applied to the GPU's inputs, then the
        oracle's quantiser, is compared element by element with the quantised rows the GPU's fused kernel produced:
        f32 sums in another order can move an activation across a rounding boundary, nothing else can differ.  The count
        of such elements is the measurement; it must stay at the level of rounding ties (each off by one step, at most
        two per thousand, scales within 1e-5).
    K, V (host copies of the caches) are advanced with the GPU's own appended rows.  Returns {linear: (differing
    elements, largest scale distance in ulps)} and the GPU's logits."""
    B, H, Hq, Hkv, hd = cfg.batch, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    stats = {}

    def compare_q(name, rows):
        q_ref, s_ref = orc.quantize_activations(np.ascontiguousarray(rows, np.float32), B, rows.shape[1])
        q_gpu, s_gpu, _ = taps[name + ".in"]
        d = np.abs(q_gpu.astype(np.int32) - q_ref.astype(np.int32))
        ulps = np.abs(s_gpu.view(np.int32).astype(np.int64) - s_ref.view(np.int32).astype(np.int64))
        stats[name] = (int((d != 0).sum()), int(ulps.max()))
        assert d.max() <= 1, f"{what} {name}: a quantised element differs by {d.max()} steps"
        # 1e-5 of the row maximum (the bar of the glue kernels) is 84 ulps of the scale
        assert ulps.max() <= 128, f"{what} {name}: row scale {ulps.max()} ulps from the oracle's"
        assert (d != 0).sum() <= max(3, 2e-3 * d.size), f"{what} {name}: {(d != 0).sum()} of {d.size} quantised elements differ"

    def linear(name, k):
        q_gpu, s_gpu, _ = taps[name + ".in"]
        qt = Q[name]
        y_ref, _ = orc.gemm_i8(q_gpu, s_gpu, qt.data_i8_t, qt.scales, B, qt.cols, k)
        y_gpu = taps[name + ".out"]
        assert np.array_equal(y_gpu.view(np.uint32), y_ref.view(np.uint32)), f"{what} {name}: product differs from the integer oracle on the GPU's own rows"
        return y_gpu

    x = np.asarray(x, np.float32)
    delta = None
    for i in range(cfg.layers):
        if delta is not None:
            x = (x + delta).astype(np.float32)
        assert np.array_equal(x.view(np.uint32), taps[f"l{i}.qkv.in"][2].view(np.uint32)), f"{what} l{i}: residual stream before attention"
        compare_q(f"l{i}.qkv", lo.rmsnorm(x, W[f"l{i}.attn_norm"], cfg.eps))
        heads = linear(f"l{i}.qkv", H).reshape(B, Hq + 2 * Hkv, hd)
        q = lo.rope_apply(heads[:, :Hq], cos[pos], sin[pos])
        K[i][:, :, pos] = lo.rope_apply(heads[:, Hq:Hq + Hkv], cos[pos], sin[pos])
        V[i][:, :, pos] = heads[:, Hq + Hkv:]
        compare_q(f"l{i}.o", lo.attention_decode(q, K[i], V[i], pos + 1, Hq // Hkv))
        o = linear(f"l{i}.o", Hq * hd)
        x = (x + o).astype(np.float32)
        assert np.array_equal(x.view(np.uint32), taps[f"l{i}.gate_up.in"][2].view(np.uint32)), f"{what} l{i}: residual stream before the FFN"
        compare_q(f"l{i}.gate_up", lo.rmsnorm(x, W[f"l{i}.ffn_norm"], cfg.eps))
        gu = linear(f"l{i}.gate_up", H)
        compare_q(f"l{i}.down", lo.silu_mul(gu[:, :cfg.ffn], gu[:, cfg.ffn:]))
        delta = linear(f"l{i}.down", cfg.ffn)
    if delta is not None:
        x = (x + delta).astype(np.float32)
    assert np.array_equal(x.view(np.uint32), taps["lm_head.in"][2].view(np.uint32)), f"{what}: residual stream before the output head"
    compare_q("lm_head", lo.rmsnorm(x, W["final_norm"], cfg.eps))
    return stats, linear("lm_head", H)


def check_free_running_oracle(orc, cfg, Q, taps, trace, got_logits, ref_logits, what=""):
    """Against the oracle running on its own (its own caches, its own activations all the way): a sequence none of
    whose quantised elements differs anywhere must give bit-identical logits; for the others the logit error is bounded
    by what the differing elements of the last quantiser can move the output head:
    |y_gpu - y_ref| <= max|w| * (s_gpu * sum|dq| + |ds| * sum|q_ref|)."""
    B = cfg.batch
    differing = np.zeros(B, np.int64)
    last = None
    for name, a_ref in trace.items():
        q_ref, s_ref = orc.quantize_activations(a_ref, B, a_ref.shape[1])
        q_gpu, s_gpu, _ = taps[name + ".in"]
        dq = np.abs(q_gpu.astype(np.int32) - q_ref.astype(np.int32)).sum(axis=1)
        differing += (q_gpu != q_ref).sum(axis=1) + (s_gpu.view(np.uint32) != s_ref.view(np.uint32))
        last = (dq, q_ref, s_ref, s_gpu)
    scale = np.abs(ref_logits).max()
    rows_err = np.abs(got_logits - ref_logits).max(axis=1)
    clean = differing == 0
    assert np.array_equal(got_logits[clean].view(np.uint32), ref_logits[clean].view(np.uint32)), \
        f"{what}: sequences without a single differing quantised element must give identical logits"
    dq, q_ref, s_ref, s_gpu = last
    wmax = float(Q["lm_head"].scales.max()) * 127.0
    bound = wmax * (s_gpu.astype(np.float64) * dq + np.abs(s_gpu.astype(np.float64) - s_ref) * np.abs(q_ref.astype(np.int32)).sum(axis=1))
    assert np.all(rows_err <= bound * (1 + 1e-5) + 1e-5 * scale), \
        f"{what}: logit error {np.array2string(rows_err, precision=3)} above the bound {np.array2string(bound, precision=3)}"
    # and nothing drifts far: a few quantisation steps of one activation at most
    assert rows_err.max() <= 2e-2 * scale, f"{what}: {np.array2string(rows_err, precision=3)} vs max|logit| {scale}"
    return int(clean.sum())


def make_weights(cfg, g, sigma=0.05):
    W = {"embedding": normal(g, (cfg.vocab, cfg.hidden), 0.5), "final_norm": (1 + normal(g, (cfg.hidden,), 0.1)).astype(np.float32),
         "lm_head": normal(g, (cfg.hidden, cfg.vocab), 0.02)}
    for i in range(cfg.layers):
        W[f"l{i}.attn_norm"] = (1 + normal(g, (cfg.hidden,), 0.1)).astype(np.float32)
        W[f"l{i}.ffn_norm"] = (1 + normal(g, (cfg.hidden,), 0.1)).astype(np.float32)
        W[f"l{i}.qkv"] = normal(g, (cfg.hidden, cfg.qkv_dim), sigma)
        W[f"l{i}.o"] = normal(g, (cfg.n_q_heads * cfg.head_dim, cfg.hidden), sigma)
        W[f"l{i}.gate_up"] = normal(g, (cfg.hidden, 2 * cfg.ffn), sigma)
        W[f"l{i}.down"] = normal(g, (cfg.ffn, cfg.hidden), sigma)
    return W


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
    W = make_weights(cfg, g)
    Q = {k: oracle_mt.quantize_weights(v, v.shape[0], v.shape[1]) for k, v in W.items() if v.ndim == 2 and k != "embedding"}
    model = LlamaInt8Decoder(cfg, gpu, W)
    # a short synthetic history in the cache
    start = 5
    K = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    V = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    for i in range(cfg.layers):
        model.load_cache(i, K[i], V[i])
    Kg, Vg = [k.copy() for k in K], [v.copy() for v in V]      # host copies that follow the GPU's caches
    cos, sin = rope_tables(cfg.head_dim, cfg.capacity, cfg.rope_base)
    tokens = g.integers(0, cfg.vocab, cfg.batch).astype(np.int32)
    tokens[0] = cfg.vocab - 1
    model.set_position(start)
    model.set_tokens(tokens)
    torch.cuda.synchronize()
    model.embed()
    gpu.sync()
    graph = None
    for step in range(3):
        x = W["embedding"][tokens]
        trace = {}
        ref_logits = lo.decode_step(oracle_mt, cfg, W, Q, x, K, V, start + step, cos, sin, trace)
        if step == 0:
            taps = run_step_with_taps(model, gpu)      # eager, launch by launch
        else:
            # the recorded step must do the same: its quantised rows are read back from a second, eager pass below
            if graph is None:
                graph = model.record()
            x0, t0 = model.x.clone(), model.tokens.clone()
            graph.launch()
            gpu.sync()
            logits_graph = model.logits.cpu().numpy().copy()
            k_graph = model.kcache[0][:, :, start + step].cpu().numpy().copy()
            model.set_position(start + step)
            model.x.copy_(x0)
            model.tokens.copy_(t0)
            torch.cuda.synchronize()
            taps = run_step_with_taps(model, gpu)
            assert np.array_equal(model.logits.cpu().numpy().view(np.uint32), logits_graph.view(np.uint32)), "graph replay differs from eager launches"
            assert np.array_equal(model.kcache[0][:, :, start + step].cpu().numpy(), k_graph)
        assert gpu.device_status() == 0
        got = model.logits.cpu().numpy()
        stats, staged_logits = check_stages(oracle_mt, cfg, W, Q, taps, x, Kg, Vg, start + step, cos, sin, f"step {step}")
        assert np.array_equal(staged_logits, got)
        for i in range(cfg.layers):             # the GPU's caches hold exactly the rows its own projections gave
            assert np.array_equal(model.kcache[i].cpu().numpy()[:, :, :start + step + 1], Kg[i][:, :, :start + step + 1])
            assert np.array_equal(model.vcache[i].cpu().numpy()[:, :, :start + step + 1], Vg[i][:, :, :start + step + 1])
        clean = check_free_running_oracle(oracle_mt, cfg, Q, taps, trace, got, ref_logits, f"step {step}")
        print(f"step {step}: quantised elements that differ from the oracle's, per linear (elements, scale ulps): {stats}; "
              f"{clean} of {cfg.batch} sequences identical to the free-running oracle")
        assert int(model.pos.item()) == start + step + 1
        picked = model.tokens.cpu().numpy()
        tol = 2e-2 * np.abs(ref_logits).max()
        srt = np.sort(ref_logits, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 2 * tol
        assert np.array_equal(picked[clear], np.argmax(ref_logits, axis=1)[clear])
        # teacher forcing: continue from the oracle's greedy choice on both sides
        tokens = np.array([lo.greedy_decode(r) for r in ref_logits], np.int32)
        model.set_tokens(tokens)
        model.embed()
        gpu.sync()
        # the caches must agree too (same rounding path for k, v up to the f32 tolerance of their inputs)
        assert np.abs(model.kcache[0][:, :, start + step].cpu().numpy() - K[0][:, :, start + step]).max() <= 1e-2
    if graph is not None:
        graph.free()
    model.free()


def test_llama8b_shape_layer_teacher_forced(pg, gpu, oracle_mt):
    """One whole layer at the Llama-3-8B shape of the benchmark (hidden 4096, 32 query / 8 KV heads of 128, SwiGLU
    14336, 16 sequences, 2048 cached positions of N(0,1) keys and values) plus a small output head, against the oracle
    with the accounting above."""
    import torch
    from peregrine_b200.llama import LlamaConfig, LlamaInt8Decoder, rope_tables

    cfg = LlamaConfig(layers=1, vocab=2048, batch=16, capacity=2176)
    g = rng(4000)
    W = make_weights(cfg, g, 0.02)
    Q = {k: oracle_mt.quantize_weights(v, v.shape[0], v.shape[1]) for k, v in W.items() if v.ndim == 2 and k != "embedding"}
    model = LlamaInt8Decoder(cfg, gpu, W)
    ctx0 = 2048
    K = [np.zeros((cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim), np.float32)]
    V = [np.zeros_like(K[0])]
    K[0][:, :, :ctx0] = normal(g, (cfg.batch, cfg.n_kv_heads, ctx0, cfg.head_dim))
    V[0][:, :, :ctx0] = normal(g, (cfg.batch, cfg.n_kv_heads, ctx0, cfg.head_dim))
    model.load_cache(0, K[0], V[0])
    cos, sin = rope_tables(cfg.head_dim, cfg.capacity, cfg.rope_base)
    tokens = g.integers(0, cfg.vocab, cfg.batch).astype(np.int32)
    model.set_position(ctx0)
    model.set_tokens(tokens)
    torch.cuda.synchronize()
    model.embed()
    gpu.sync()
    trace = {}
    Kg, Vg = [K[0].copy()], [V[0].copy()]
    x = W["embedding"][tokens]
    ref_logits = lo.decode_step(oracle_mt, cfg, W, Q, x, K, V, ctx0, cos, sin, trace)
    taps = run_step_with_taps(model, gpu)
    assert gpu.device_status() == 0
    got = model.logits.cpu().numpy()
    stats, staged_logits = check_stages(oracle_mt, cfg, W, Q, taps, x, Kg, Vg, ctx0, cos, sin, "8B-shape layer")
    assert np.array_equal(staged_logits, got)
    clean = check_free_running_oracle(oracle_mt, cfg, Q, taps, trace, got, ref_logits, "8B-shape layer")
    print(f"8B-shape layer: differing quantised elements per linear (elements, scale ulps): {stats}; {clean} of 16 sequences "
          "identical to the free-running oracle")
    # appended rows of the cache: exactly the GPU's own projection, rotated
    assert np.array_equal(model.kcache[0][:, :, ctx0].cpu().numpy(), Kg[0][:, :, ctx0])
    assert np.array_equal(model.vcache[0][:, :, ctx0].cpu().numpy(), Vg[0][:, :, ctx0])
    assert np.abs(Kg[0][:, :, ctx0] - K[0][:, :, ctx0]).max() <= 1e-4
    assert int(model.pos.item()) == ctx0 + 1
    model.free()


def test_lm_head_product_at_full_vocabulary(pg, gpu, oracle_mt):
    """The output head of the benchmark's stack, [4096, 128256] at 16 rows: weights drawn and quantised on the device;
    2048 sampled columns of the quantised weights and of the product are held to the oracle bit for bit."""
    import torch
    from peregrine_b200 import _lib

    lib = gpu.lib
    k, n, m = 4096, 128256, 16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4001)
    w = torch.randn(k, n, generator=gen, device="cuda") * 0.02
    h = C.c_void_p()
    torch.cuda.synchronize()
    _lib.check(lib.pg_qtensor_from_f32(gpu.handle, w.data_ptr(), k, n, 0, C.byref(h)))
    gpu.sync()
    g = rng(4002)
    cols = np.sort(g.choice(n, 2048, replace=False))
    cols[:3] = (0, 1, 2)
    cols[-2:] = (n - 2, n - 1)
    cols = np.unique(cols)
    w_cols = w[:, torch.from_numpy(cols).cuda()].cpu().numpy()
    del w
    torch.cuda.empty_cache()
    x = normal(g, (m, k))
    ch = g.choice(k, 41, replace=False)
    x[:, ch] *= np.float32(20.0)
    tx = _t(x)
    y = torch.empty(m, n, device="cuda")
    q8 = torch.empty(m * k + 64, dtype=torch.int8, device="cuda")
    q8s = torch.empty(m, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.pg_matmul_quantized_ex(gpu.handle, tx.data_ptr(), m, k, h, y.data_ptr(), None, q8.data_ptr(), q8s.data_ptr(), _lib.ALGO_AUTO))
    gpu.sync()
    wt = np.empty((n, k), np.int8)
    ws = np.empty(n, np.float32)
    _lib.check(lib.pg_qtensor_download(gpu.handle, h, None, wt.ctypes.data_as(C.c_void_p), ws.ctypes.data_as(C.c_void_p)))
    ref_q = oracle_mt.quantize_weights(np.ascontiguousarray(w_cols), k, len(cols))
    assert np.array_equal(wt[cols], ref_q.data_i8_t) and np.array_equal(ws[cols].view(np.uint32), ref_q.scales.view(np.uint32))
    ref_y = oracle_mt.matmul_quantized(x, m, k, ref_q)
    assert np.array_equal(y.cpu().numpy()[:, cols].view(np.uint32), ref_y.view(np.uint32))
    lib.pg_qtensor_free(gpu.handle, h)


def test_position_outside_the_cache_is_reported_not_written(pg, gpu):
    """A decode loop that runs past its KV capacity: the kernels that read the position must leave the caches alone,
    record PG_ERR_INVALID in the status word, and the position must stop advancing at the capacity."""
    import torch
    from peregrine_b200 import _lib
    from peregrine_b200.llama import rope_tables

    lib = gpu.lib
    hd, cap = 128, 96
    g = rng(77)
    for B, Hq, Hkv in ((2, 8, 2), (2, 2, 2)):          # streaming (fused) kernel and the chunked one
        cos, sin = rope_tables(hd, cap, 500000.0)
        tc, ts = _t(cos), _t(sin)
        qkv = _t(normal(g, (B, (Hq + 2 * Hkv) * hd)))
        # guard rows behind the caches: one allocation, the caches in front, a canary behind
        cache_elems = B * Hkv * cap * hd
        Kbuf = torch.full((cache_elems + 4096,), 7.0, device="cuda")
        Vbuf = torch.full((cache_elems + 4096,), 9.0, device="cuda")
        for bad in (cap, cap + 5, -1):
            tpos = torch.tensor([bad], dtype=torch.int32, device="cuda")
            qrot = torch.zeros(B, Hq, hd, device="cuda")
            S = lib.pg_gqa_decode_splits(gpu.handle, B, Hq, Hkv, cap)
            work = torch.zeros(B * Hq * S * 130, device="cuda")
            out = torch.zeros(B, Hq * hd, device="cuda")
            torch.cuda.synchronize()
            _lib.check(lib.pg_rope_kv_append(gpu.handle, qkv.data_ptr(), tpos.data_ptr(), tc.data_ptr(), ts.data_ptr(), B, Hq, Hkv, hd, cap,
                                             qrot.data_ptr(), Kbuf.data_ptr(), Vbuf.data_ptr()))
            assert gpu.device_status() == _lib.PG_ERR_INVALID
            _lib.check(lib.pg_gqa_attention_decode(gpu.handle, qrot.data_ptr(), Kbuf.data_ptr(), Vbuf.data_ptr(), tpos.data_ptr(), B, Hq, Hkv, hd,
                                                   cap, work.data_ptr(), out.data_ptr(), None, None))
            assert gpu.device_status() == _lib.PG_ERR_INVALID
            if Hq // Hkv in (4, 8):
                _lib.check(lib.pg_gqa_attention_decode_fused(gpu.handle, qkv.data_ptr(), tpos.data_ptr(), tc.data_ptr(), ts.data_ptr(),
                                                             Kbuf.data_ptr(), Vbuf.data_ptr(), B, Hq, Hkv, hd, cap, work.data_ptr(), out.data_ptr(),
                                                             None, None))
                assert gpu.device_status() == _lib.PG_ERR_INVALID
            gpu.sync()
            assert bool((Kbuf == 7.0).all()) and bool((Vbuf == 9.0).all()), f"cache or canary written at position {bad}"
            assert gpu.device_status() == 0           # reading the status cleared it; the context is still usable
    # the position stops at the limit
    logits = _t(normal(g, (2, 300)))
    picks = torch.zeros(2, dtype=torch.int32, device="cuda")
    p = torch.tensor([cap - 1], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for expect in (cap, cap, cap):
        _lib.check(lib.pg_argmax_advance(gpu.handle, logits.data_ptr(), 2, 300, picks.data_ptr(), p.data_ptr(), cap))
        gpu.sync()
        assert int(p.item()) == expect


def _emulated_ranks(pg, gpu, cfg, W, world, attn_splits):
    from peregrine_b200.llama import LlamaInt8Decoder

    ranks = [LlamaInt8Decoder(cfg, gpu, W, rank=r, world=world, attn_splits=attn_splits, connect=False) for r in range(world)]
    LlamaInt8Decoder.connect_local(ranks)
    return ranks


def _step_all(ranks):
    """The ranks share this process, this GPU and one stream: advance them in turn, launch by launch.  A launch that
    waits for the other ranks' flags is then always enqueued behind the launches that raise them."""
    for _ in zip(*[r.step_ops() for r in ranks]):
        pass


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_sharded_step_equals_single_gpu_step(pg, gpu, world):
    """The column-sharded decode step (heads, gate/up channels, O / down / vocabulary columns split over `world` ranks,
    exchanges stored by the producing kernels and awaited by the consuming ones), with all ranks played on this one GPU:
    logits, chosen tokens, residual stream and caches must be bit-identical to the unsharded step when the attention
    slices are cut as on one GPU, and within f32 summation noise of it when every rank cuts for itself."""
    import torch
    from peregrine_b200.llama import LlamaConfig, LlamaInt8Decoder

    cfg = LlamaConfig(layers=2, hidden=8 * 128, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=2048, vocab=4096, batch=5, capacity=300)
    cfg.hidden = 1024
    g = rng(600 + world)
    W = make_weights(cfg, g)
    start = 130
    K = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    V = [normal(g, (cfg.batch, cfg.n_kv_heads, cfg.capacity, cfg.head_dim)) for _ in range(cfg.layers)]
    tokens = g.integers(0, cfg.vocab, cfg.batch).astype(np.int32)

    def prime(models):
        for m in models:
            for i in range(cfg.layers):
                m.load_cache(i, K[i], V[i])
            m.set_position(start)
            m.set_tokens(tokens)
            torch.cuda.synchronize()
            m.embed()
        gpu.sync()

    one = LlamaInt8Decoder(cfg, gpu, W)
    prime([one])
    ref = []
    for _ in range(3):
        one.enqueue_step()
        gpu.sync()
        ref.append((one.logits.cpu().numpy().copy(), one.tokens.cpu().numpy().copy(), one.x.cpu().numpy().copy()))
    ref_k = one.kcache.cpu().numpy().copy()
    one.free()
    for mode in ("match", "auto"):
        ranks = _emulated_ranks(pg, gpu, cfg, W, world, mode)
        prime(ranks)
        for step in range(3):
            _step_all(ranks)
            gpu.sync()
            assert gpu.device_status() == 0
            logits = np.concatenate([r.logits.cpu().numpy() for r in ranks], axis=1)
            ref_logits, ref_tok, ref_x = ref[step]
            if mode == "match":
                assert np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32)), f"step {step}"
                for r in ranks:
                    assert np.array_equal(r.tokens.cpu().numpy(), ref_tok) and np.array_equal(r.x.cpu().numpy().view(np.uint32), ref_x.view(np.uint32))
            else:
                assert np.abs(logits - ref_logits).max() <= 2e-2 * np.abs(ref_logits).max()
                for r in ranks[1:]:
                    assert np.array_equal(r.tokens.cpu().numpy(), ranks[0].tokens.cpu().numpy())      # every rank picks the same token
            assert all(int(r.pos.item()) == start + step + 1 for r in ranks)
        if mode == "match":
            got_k = np.concatenate([r.kcache.cpu().numpy() for r in ranks], axis=2)
            assert np.array_equal(got_k, ref_k)
        for r in ranks:
            r.free()


def test_sharded_vocabulary_argmax_ties_and_nan(pg, gpu):
    """pg_argmax_exchange + pg_pick_embed over four emulated ranks: the first maximum over the whole vocabulary wins, a
    tie across two ranks' ranges goes to the lower index, NaN never wins, an all-NaN row gives token 0."""
    import torch
    from peregrine_b200 import _lib
    from peregrine_b200.sharded import Exchange

    lib = gpu.lib
    world, B, V, dim = 4, 5, 4096, 64
    vl = V // world
    g = rng(91)
    logits = normal(g, (B, V))
    logits[0, 100] = logits[0, 3000] = 9.0             # tie across ranks 0 and 2
    logits[1, V - 1] = 12.0                            # maximum in the last rank's last column
    logits[2, :] = np.nan                              # all NaN
    logits[3, :vl] = np.nan                            # rank 0's slice all NaN
    logits[3, 2 * vl + 7] = 50.0
    logits[4, :] = -np.inf
    table = normal(g, (V, dim))
    exs = [Exchange(gpu, r, world, B * world * 8) for r in range(world)]
    Exchange.connect_local(exs)
    parts = [_t(logits[:, r * vl:(r + 1) * vl]) for r in range(world)]
    tt = _t(table)
    toks = [torch.full((B,), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.zeros(B, dim, device="cuda") for _ in range(world)]
    poss = [torch.tensor([10], dtype=torch.int32, device="cuda") for _ in range(world)]
    torch.cuda.synchronize()
    for rep in range(2):                               # twice: the exchange counters advance
        for r in range(world):
            _lib.check(lib.pg_argmax_exchange(gpu.handle, parts[r].data_ptr(), B, vl, r * vl, exs[r].handle))
        for r in range(world):
            _lib.check(lib.pg_pick_embed(gpu.handle, exs[r].handle, B, toks[r].data_ptr(), poss[r].data_ptr(), 0, tt.data_ptr(), dim, outs[r].data_ptr()))
        gpu.sync()
        assert gpu.device_status() == 0
        expect = [100, V - 1, 0, 2 * vl + 7, 0]
        for r in range(world):
            assert toks[r].cpu().numpy().tolist() == expect
            assert np.array_equal(outs[r].cpu().numpy(), table[expect])
            assert int(poss[r].item()) == 11 + rep
    for e in exs:
        e.destroy()
