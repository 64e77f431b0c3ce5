"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.
One generator (numpy PCG64) feeds the oracle and the GPU alike."""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def normal(g, shape, sigma=1.0):
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def linear_inputs(m, k, n, seed, outliers=False):
    """X ~ N(0,1) [m,k] (optionally 1 % of the channels scaled x20), W ~ N(0,0.02) [k,n]."""
    g = rng(seed)
    x = normal(g, (m, k))
    if outliers:
        ch = g.choice(k, size=int(np.ceil(0.01 * k)), replace=False)
        x[:, ch] *= np.float32(20.0)
    w = normal(g, (k, n), 0.02)
    return x, w


def bits_equal(a, b):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def lcg(n, seed):
    """The LCG stream of tests/huffman_parity.rs:9-21 (f32 arithmetic as in the reference)."""
    out = np.empty(n, np.float32)
    state = seed
    for i in range(n):
        state = (state * 1103515245 + 12345) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(state) / np.float32(0xFFFFFFFF)) * np.float32(2.0) - np.float32(1.0)
    return out
