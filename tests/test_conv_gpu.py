"""GPU parity of conv2d / conv2d_backward_x / conv2d_backward_k (NCHW, stride 1, zero padding) against the
CPU restatement of the reference loops, on the tensor-core path (large cases), the CUDA-core GEMM path
(small cases) and the per-output kernels (group != 1)."""
import numpy as np
import pytest

from helpers import rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

CASES = [  # ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, yh, yw, group
    (1, 1, 1, 1, 1, 1, 1, 0, 0, 1, 1, 1),
    (2, 3, 4, 6, 5, 3, 3, 1, 1, 6, 5, 1),
    (1, 4, 2, 5, 7, 5, 3, 2, 1, 5, 7, 1),
    (3, 5, 7, 9, 11, 3, 3, 0, 0, 7, 9, 1),         # "valid": output smaller than input
    (2, 8, 6, 8, 8, 1, 1, 0, 0, 8, 8, 1),          # 1 x 1
    (2, 4, 3, 4, 4, 3, 3, 1, 1, 4, 4, 2),          # group 2: per-output kernels
    (1, 6, 4, 5, 5, 3, 3, 1, 1, 5, 5, 3),
    (4, 32, 64, 28, 28, 3, 3, 1, 1, 28, 28, 1),    # tensor-core GEMMs
    (1, 64, 48, 30, 34, 3, 3, 1, 1, 30, 34, 1),    # one image: no layout permutation
    (2, 16, 40, 21, 19, 5, 5, 2, 2, 21, 19, 1),    # pixel count not a multiple of 4
    (3, 56, 100, 9, 30, 5, 3, 2, 1, 9, 30, 1),     # channels-last tiles: channels padded to 64, 100 outputs, ragged last tile
    (4, 96, 128, 13, 13, 3, 3, 1, 1, 13, 13, 1),   # nine short rows per tile, both directions on the channels-last kernel
    (2, 32, 32, 20, 20, 3, 3, 0, 0, 18, 18, 1),    # "valid" on the channels-last kernel
]


def _truth_conv(x, k, yh, yw, ph, pw):
    ndat, xchn, xh, xw = x.shape
    ychn, _, kh, kw = k.shape
    xp = np.zeros((ndat, xchn, xh + 2 * kh, xw + 2 * kw), np.float64)
    xp[:, :, kh:kh + xh, kw:kw + xw] = x
    y = np.zeros((ndat, ychn, yh, yw), np.float64)
    for kr in range(kh):
        for kc in range(kw):
            r0, c0 = kh + kr - ph, kw + kc - pw
            patch = xp[:, :, r0:r0 + yh, c0:c0 + yw]
            y += np.einsum("ncrs,oc->nors", patch, k[:, :, kr, kc].astype(np.float64))
    return y


@pytest.mark.parametrize("case", CASES)
def test_conv2d_trio(torch_cuda, vm, port, case):
    torch = torch_cuda
    ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, yh, yw, group = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
    k = (rng.standard_normal((ychn, xchn // group, kh, kw)) / np.sqrt(xchn * kh * kw)).astype(np.float32)
    gy = rng.standard_normal((ndat, ychn, yh, yw)).astype(np.float32)
    dx, dk, dgy = (to_dev(torch, t) for t in (x, k, gy))

    y = torch.full((ndat, ychn, yh, yw), float("nan"), device="cuda")
    vm.conv2d(0, y, dx, dk, ndat, ychn, yh, yw, xchn, xh, xw, kh, kw, group, ph, pw)
    gx = torch.full((ndat, xchn, xh, xw), float("nan"), device="cuda")
    vm.conv2d_backward_x(0, gx, dgy, dk, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw)
    gk = torch.full((ychn, xchn // group, kh, kw), float("nan"), device="cuda")
    vm.conv2d_backward_k(0, gk, dgy, dx, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw)
    torch.cuda.synchronize()

    want_y = port.conv2d(x, k, yh, yw, ph, pw, group)
    want_gx = port.conv2d_backward_x(gy, k, xh, xw, ph, pw, group)
    want_gk = port.conv2d_backward_k(gy, x, kh, kw, ph, pw, group)
    for name, got, want in (("y", y, want_y), ("gx", gx, want_gx), ("gk", gk, want_gk)):
        g = to_host(got)
        assert np.isfinite(g).all(), name
        assert rel_fro(g, want) < 5e-6, f"{name}: {rel_fro(g, want):.3e}"
    if group == 1:   # the accuracy rule of the GEMM path: no worse than twice the reference loop's own error
        truth = _truth_conv(x, k, yh, yw, ph, pw)
        assert rel_fro(to_host(y), truth) <= 2 * rel_fro(want_y, truth) + 1e-7


def test_conv2d_rejects_other_padding_modes(vm, pkg, torch_cuda):
    torch = torch_cuda
    t = torch.zeros((1, 1, 2, 2), device="cuda")
    with pytest.raises(pkg.capi.KaiError) as ei:
        vm.conv2d(0, t, t, t, 1, 1, 2, 2, 1, 2, 2, 1, 1, 1, 0, 0, pmode=1)
    assert ei.value.code == pkg.capi.E_INVALID_ARG


VARIANT_CASES = [  # ndat, xchn, ychn, xh, xw, kh, kw, p0, p1
    (1, 1, 1, 1, 1, 1, 1, 1, 1), (2, 3, 4, 6, 5, 3, 3, 2, 2), (1, 2, 3, 4, 7, 5, 3, 3, 1), (2, 4, 2, 5, 5, 1, 1, 1, 2),
    (1, 3, 2, 6, 6, 4, 2, 2, 3), (3, 8, 16, 12, 10, 3, 3, 2, 2), (2, 32, 48, 24, 20, 3, 3, 2, 2),
]


@pytest.mark.parametrize("case", VARIANT_CASES)
def test_conv2d_transposed_and_dilated(torch_cuda, vm, port, case):
    """The transposed family reproduces the reference's loops bit for bit (same index rules, same summation
    order, unfused multiply-add); the dilated family runs on the GEMM kernels and is compared by norm."""
    torch = torch_cuda
    ndat, xchn, ychn, xh, xw, kh, kw, p0, p1 = case
    rng = np.random.default_rng(sum(case) + 1)
    x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
    k = (rng.standard_normal((ychn, xchn, kh, kw)) / np.sqrt(xchn * kh * kw)).astype(np.float32)
    gy_t = rng.standard_normal((ndat, ychn, xh * p0, xw * p1)).astype(np.float32)
    gy_d = rng.standard_normal((ndat, ychn, xh, xw)).astype(np.float32)
    dims = (ndat, xchn, xh, xw, ychn, kh, kw, p0, p1)
    jobs = (("transposed", gy_t.shape, x, k, True), ("transposed_backward_x", x.shape, gy_t, k, True),
            ("transposed_backward_k", k.shape, gy_t, x, True), ("dilated", gy_d.shape, x, k, False),
            ("dilated_backward_x", x.shape, gy_d, k, False), ("dilated_backward_k", k.shape, gy_d, x, False))
    for which, shape, a, b, exact in jobs:
        out = torch.full(shape, float("nan"), device="cuda")
        getattr(vm, "conv2d_" + which)(0, out, to_dev(torch, a), to_dev(torch, b), *dims)
        torch.cuda.synchronize()
        got = to_host(out)
        want = port.conv2d_variant(which, shape, a, b, *dims)
        if exact:
            np.testing.assert_array_equal(got, want, err_msg=which)
        else:
            assert np.isfinite(got).all(), which
            assert rel_fro(got, want) < 5e-6 or np.abs(got - want).max() < 1e-6, f"{which}: {rel_fro(got, want):.3e}"
