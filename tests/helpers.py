"""Shared helpers of the GPU parity tests."""
from __future__ import annotations

import numpy as np


def to_dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_host(t):
    return t.detach().cpu().numpy()


def rel_fro(got, truth64) -> float:
    t = np.asarray(truth64, np.float64)
    d = np.asarray(got, np.float64) - t
    den = np.linalg.norm(t.ravel())
    return float(np.linalg.norm(d.ravel()) / (den if den > 0 else 1.0))


def gemm_truth(layout: int, a, b):
    """fp64 ground truth of the three reference layouts (0 NT, 1 NN, 2 TN)."""
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    if layout == 0:
        return a64 @ b64.T
    if layout == 1:
        return a64 @ b64
    return a64.T @ b64


def check_gemm_error(err_gpu: float, err_ref: float, K: int, what: str = ""):
    """The acceptance rule of the path: relative Frobenius error against fp64
    <= 1e-5 * sqrt(K), and no worse than 2x the reference CPU path's own error."""
    assert err_gpu <= 1e-5 * np.sqrt(max(K, 1)), f"{what}: {err_gpu:.3e} > 1e-5*sqrt(K)"
    # An exact reference result (tiny K) has error 0; allow fp32 rounding of the output then.
    assert err_gpu <= 2.0 * err_ref + 6e-8, f"{what}: gpu {err_gpu:.3e} vs 2 x reference {err_ref:.3e}"
