"""Seeded synthetic inputs of the five benchmark configurations.

No dataset is involved: the reference path is exercised with tensors of the stated shapes and
distributions, drawn with numpy's PCG64 (``default_rng(seed)``) and cast to fp32 once, so the
CPU oracle, the fp64 ground truth and the GPU all see identical buffers.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def gemm_square(n: int = 512, seed: int = 0):
    """Config 1: C = A.B, row-major, no transpose; A, B ~ U[-1,1)."""
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, (n, n)).astype(F32)
    b = rng.uniform(-1.0, 1.0, (n, n)).astype(F32)
    return a, b


def xavier_uniform(rng, fan_out: int, fan_in: int):
    """U(-sqrt(6/(fan_in+fan_out)), +...): the reference's `normalized_xavier` initialiser
    (api_objects/vmodule.cpp:1391); weights are stored [out, in]."""
    lim = np.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-lim, lim, (fan_out, fan_in)).astype(F32)


def mlp(batch: int = 128, d_in: int = 784, d_hidden: int = 512, n_class: int = 10, seed: int = 0):
    """Config 2: Linear(784->512)+ReLU -> Linear(512->10), softmax cross-entropy on int labels."""
    rng = np.random.default_rng(seed)
    return {
        "x": rng.uniform(0.0, 1.0, (batch, d_in)).astype(F32),
        "w1": xavier_uniform(rng, d_hidden, d_in),
        "b1": np.zeros(d_hidden, F32),
        "w2": xavier_uniform(rng, n_class, d_hidden),
        "b2": np.zeros(n_class, F32),
        "labels": rng.integers(0, n_class, batch).astype(np.int32),
    }


def attention(nbat: int = 32, ntimes: int = 512, nhead: int = 8, npiece: int = 64, seed: int = 0):
    """Config 3: Q, K, V ~ N(0,1), [nbat, ntimes, nhead*npiece] head-interleaved; coef = 1/sqrt(npiece)."""
    rng = np.random.default_rng(seed)
    shape = (nbat, ntimes, nhead * npiece)
    q = rng.standard_normal(shape, dtype=F32)
    k = rng.standard_normal(shape, dtype=F32)
    v = rng.standard_normal(shape, dtype=F32)
    return q, k, v, float(1.0 / np.sqrt(npiece))


def gemm_large(m: int = 8192, n: int = 8192, k: int = 8192, seed: int = 0):
    """Config 4: Y = X.W^T, X [m,k] row-major, W [n,k] (B 'column-major'); U[-1,1)."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, (m, k)).astype(F32)
    w = rng.uniform(-1.0, 1.0, (n, k)).astype(F32)
    return x, w


def linear_step(tokens: int = 8192, d_in: int = 4096, d_out: int = 4096, seed: int = 0):
    """Config 5: X ~ N(0,1), W ~ N(0, 1/d_in), dY ~ N(0,1), b ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    return {
        "x": rng.standard_normal((tokens, d_in), dtype=F32),
        "w": (rng.standard_normal((d_out, d_in), dtype=F32) / np.sqrt(d_in)).astype(F32),
        "dy": rng.standard_normal((tokens, d_out), dtype=F32),
        "b": rng.standard_normal(d_out, dtype=F32),
    }
