"""GPU parity of layernorm / layernorm_backward (support/vmath.cu:5977-6087) against the CPU oracle.

The GPU sums a row lane-wise and then over the warp, the reference serially, so results agree to
fp32 rounding of the sums, not bit for bit; the statistics are compared against fp64 as well."""
import numpy as np
import pytest

from helpers import to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 1), (3, 7), (16, 64), (33, 128), (64, 512), (128, 1024), (9, 2048),
                                   (5, 513), (4, 4096), (2, 10000), (8192, 512)])
def test_layernorm_forward_backward(torch_cuda, vm, port, shape):
    torch = torch_cuda
    nrow, ncol = shape
    rng = np.random.default_rng(nrow * 31 + ncol)
    x = (rng.standard_normal((nrow, ncol)) * 3 + 1).astype(np.float32)
    gy = rng.standard_normal((nrow, ncol)).astype(np.float32)
    scale = 1.25
    want_y, want_s = port.layernorm(x, scale)
    want_g = port.layernorm_backward(gy, want_s, scale)
    dx, dgy = to_dev(torch, x), to_dev(torch, gy)
    dscale = torch.tensor([scale], device="cuda")
    y = torch.full((nrow, ncol), float("nan"), device="cuda")
    st = torch.full((nrow, 2), float("nan"), device="cuda")
    gx = torch.full((nrow, ncol), float("nan"), device="cuda")
    vm.layernorm(0, y, dx, st, nrow, ncol, dscale)
    vm.layernorm_backward(0, gx, dgy, st, nrow, ncol, dscale)
    torch.cuda.synchronize()
    x64 = x.astype(np.float64)
    avg64 = x64.mean(axis=1)
    std64 = np.sqrt(((x64 - avg64[:, None]) ** 2).mean(axis=1) + 1e-10)
    got_s = to_host(st)
    # the statistics: at least as close to fp64 as the reference's serial sums (plus rounding of the result)
    err_ref = np.abs(want_s[:, 0] - avg64).max(), np.abs(want_s[:, 1] - std64).max()
    assert np.abs(got_s[:, 0] - avg64).max() <= 2 * err_ref[0] + 1e-6
    assert np.abs(got_s[:, 1] - std64).max() <= 2 * err_ref[1] + 1e-6
    np.testing.assert_allclose(to_host(y), want_y, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(to_host(gx), want_g, rtol=2e-5, atol=2e-5)


def test_layernorm_null_scale_and_unaligned(torch_cuda, vm, port):
    torch = torch_cuda
    rng = np.random.default_rng(4)
    x = rng.standard_normal((6, 40)).astype(np.float32)
    buf = torch.zeros(6 * 40 + 1, device="cuda")
    buf[1:] = to_dev(torch, x).flatten()          # 4-byte aligned interior pointer: generic kernel
    y = torch.full((6, 40), float("nan"), device="cuda")
    st = torch.empty((6, 2), device="cuda")
    vm.layernorm(0, y, buf.data_ptr() + 4, st, 6, 40, torch.tensor([2.0], device="cuda"))
    torch.cuda.synchronize()
    np.testing.assert_allclose(to_host(y), port.layernorm(x, 2.0)[0], rtol=2e-5, atol=2e-5)
    vm.layernorm(0, y, to_dev(torch, x), st, 6, 40, None)       # NULL HYPER reads as 0
    torch.cuda.synchronize()
    assert float(y.abs().max()) == 0.0
    vm.layernorm(0, y, y, st, 0, 40, None)                      # nothing to do
