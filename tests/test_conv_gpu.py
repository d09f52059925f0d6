"""GPU parity of conv2d / conv2d_backward_x / conv2d_backward_k (NCHW, stride 1, zero padding) and of the
transposed and dilated families against the CPU restatement of the reference loops: on the tensor-core
kernels (large cases), the CUDA-core GEMM path (small cases), and -- behind the "conv_direct" option -- the
one-thread-per-output kernels that repeat the reference's loops bit for bit."""
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
    (2, 4, 3, 4, 4, 3, 3, 1, 1, 4, 4, 2),          # group 2: channel-group sums, then the group-1 path
    (1, 6, 4, 5, 5, 3, 3, 1, 1, 5, 5, 3),
    (4, 64, 48, 28, 28, 3, 3, 1, 1, 28, 28, 2),    # group 2 at a size the tensor-core kernels take
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
def test_conv2d_trio(torch_cuda, pkg, vm, port, case):
    torch = torch_cuda
    ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, yh, yw, group = case
    tc0 = pkg.load().kai_tc_launch_count()
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
    # the accuracy rule of the GEMM path: no worse than twice the reference loop's own error
    k_full = np.repeat(k, group, axis=1)       # kernel channel xn / group for input channel xn
    truth = _truth_conv(x, k_full, yh, yw, ph, pw)
    assert rel_fro(to_host(y), truth) <= 2 * rel_fro(want_y, truth) + 1e-7
    if ndat * ychn * yh * yw * xchn * kh * kw >= 1 << 28:     # large cases: all three calls ran tcgen05 kernels
        assert pkg.load().kai_tc_launch_count() - tc0 >= 3


def test_conv2d_group_direct_kernels_equal_the_gemm_path(torch_cuda, pkg, vm, port):
    """Option conv_direct = 1 keeps the one-thread-per-output kernels for group != 1; both paths agree with the oracle."""
    torch = torch_cuda
    ndat, xchn, ychn, hh, ww, group = 2, 6, 5, 7, 6, 3
    rng = np.random.default_rng(12)
    x = rng.standard_normal((ndat, xchn, hh, ww)).astype(np.float32)
    k = rng.standard_normal((ychn, xchn // group, 3, 3)).astype(np.float32)
    gy = rng.standard_normal((ndat, ychn, hh, ww)).astype(np.float32)
    dx, dk, dgy = (to_dev(torch, t) for t in (x, k, gy))
    outs = {}
    for direct in (1, 0):
        pkg.capi.call("kai_set_option", b"conv_direct", direct)
        try:
            y = torch.empty((ndat, ychn, hh, ww), device="cuda")
            gx = torch.empty((ndat, xchn, hh, ww), device="cuda")
            gk = torch.empty((ychn, xchn // group, 3, 3), device="cuda")
            vm.conv2d(0, y, dx, dk, ndat, ychn, hh, ww, xchn, hh, ww, 3, 3, group, 1, 1)
            vm.conv2d_backward_x(0, gx, dgy, dk, ndat, xchn, hh, ww, ychn, hh, ww, 3, 3, group, 1, 1)
            vm.conv2d_backward_k(0, gk, dgy, dx, ndat, xchn, hh, ww, ychn, hh, ww, 3, 3, group, 1, 1)
            torch.cuda.synchronize()
            outs[direct] = [to_host(t) for t in (y, gx, gk)]
        finally:
            pkg.capi.call("kai_set_option", b"conv_direct", 0)
    wants = (port.conv2d(x, k, hh, ww, 1, 1, group), port.conv2d_backward_x(gy, k, hh, ww, 1, 1, group),
             port.conv2d_backward_k(gy, x, 3, 3, 1, 1, group))
    for got_d, got_g, want in zip(outs[1], outs[0], wants):
        assert rel_fro(got_d, want) < 5e-6 and rel_fro(got_g, want) < 5e-6


def test_conv2d_treats_every_padding_mode_as_zero_padding(vm, pkg, torch_cuda, port):
    """The reference skips out-of-range taps whatever pmode says (support/vmath.cu:3509-3512, 3552-3555)."""
    torch = torch_cuda
    rng = np.random.default_rng(2)
    x = rng.standard_normal((1, 2, 4, 4)).astype(np.float32)
    k = rng.standard_normal((3, 2, 3, 3)).astype(np.float32)
    want = port.conv2d(x, k, 4, 4, 1, 1)
    for pmode in (0, 1, 2):
        y = torch.empty((1, 3, 4, 4), device="cuda")
        vm.conv2d(0, y, to_dev(torch, x), to_dev(torch, k), 1, 3, 4, 4, 2, 4, 4, 3, 3, 1, 1, 1, pmode=pmode)
        torch.cuda.synchronize()
        assert rel_fro(to_host(y), want) < 5e-6


VARIANT_CASES = [  # ndat, xchn, ychn, xh, xw, kh, kw, p0, p1
    (1, 1, 1, 1, 1, 1, 1, 1, 1), (2, 3, 4, 6, 5, 3, 3, 2, 2), (1, 2, 3, 4, 7, 5, 3, 3, 1), (2, 4, 2, 5, 5, 1, 1, 1, 2),
    (1, 3, 2, 6, 6, 4, 2, 2, 3), (3, 8, 16, 12, 10, 3, 3, 2, 2), (2, 32, 48, 24, 20, 3, 3, 2, 2),
    (1, 4, 4, 5, 6, 1, 1, 3, 2), (2, 4, 8, 7, 5, 2, 5, 3, 3), (8, 128, 128, 16, 16, 3, 3, 2, 2),
]


@pytest.mark.parametrize("direct", [1, 0])
@pytest.mark.parametrize("case", VARIANT_CASES)
def test_conv2d_transposed_and_dilated(torch_cuda, pkg, vm, port, case, direct):
    """conv_direct = 1: the transposed family reproduces the reference's loops bit for bit (same index rules, same
    summation order, unfused multiply-add).  conv_direct = 0 (default): it runs on the GEMM kernels -- the forward as
    a plain convolution of the row / column-repeated image, the gradients through a strided unfolding -- and is
    compared by norm, like the dilated family."""
    torch = torch_cuda
    ndat, xchn, ychn, xh, xw, kh, kw, p0, p1 = case
    pkg.capi.call("kai_set_option", b"conv_direct", direct)
    try:
        _variants(torch, pkg, vm, port, case, bool(direct))
    finally:
        pkg.capi.call("kai_set_option", b"conv_direct", 0)


def _variants(torch, pkg, vm, port, case, direct):
    ndat, xchn, ychn, xh, xw, kh, kw, p0, p1 = case
    rng = np.random.default_rng(sum(case) + 1)
    x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
    k = (rng.standard_normal((ychn, xchn, kh, kw)) / np.sqrt(xchn * kh * kw)).astype(np.float32)
    gy_t = rng.standard_normal((ndat, ychn, xh * p0, xw * p1)).astype(np.float32)
    gy_d = rng.standard_normal((ndat, ychn, xh, xw)).astype(np.float32)
    dims = (ndat, xchn, xh, xw, ychn, kh, kw, p0, p1)
    jobs = (("transposed", gy_t.shape, x, k, direct), ("transposed_backward_x", x.shape, gy_t, k, direct),
            ("transposed_backward_k", k.shape, gy_t, x, direct), ("dilated", gy_d.shape, x, k, False),
            ("dilated_backward_x", x.shape, gy_d, k, False), ("dilated_backward_k", k.shape, gy_d, x, False))
    big = ndat * xchn * ychn * xh * xw * kh * kw >= 1 << 28
    for which, shape, a, b, exact in jobs:
        out = torch.full(shape, float("nan"), device="cuda")
        tc0 = pkg.load().kai_tc_launch_count()
        getattr(vm, "conv2d_" + which)(0, out, to_dev(torch, a), to_dev(torch, b), *dims)
        torch.cuda.synchronize()
        if big and not direct:      # the large case runs a tcgen05 kernel in every one of the six calls
            assert pkg.load().kai_tc_launch_count() > tc0, which
        got = to_host(out)
        want = port.conv2d_variant(which, shape, a, b, *dims)
        if exact:
            np.testing.assert_array_equal(got, want, err_msg=which)
        else:
            assert np.isfinite(got).all(), which
            assert rel_fro(got, want) < 5e-6 or np.abs(got - want).max() < 1e-6, f"{which}: {rel_fro(got, want):.3e}"


WGRAD_CASES = [  # ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, yh, yw, gh, gw
    (2, 8, 16, 6, 5, 3, 3, 1, 1, 6, 5, 1, 1),          # width 5 -> padded to 8
    (3, 24, 40, 9, 12, 3, 3, 1, 1, 9, 12, 1, 1),
    (2, 70, 130, 8, 8, 3, 3, 1, 1, 8, 8, 1, 1),        # two channel blocks, two tiles of output channels
    (2, 16, 32, 10, 11, 1, 1, 0, 0, 10, 11, 1, 1),     # 1 x 1
    (2, 16, 16, 9, 9, 2, 2, 0, 0, 8, 8, 1, 1),         # even kernel, "valid"
    (1, 12, 20, 12, 10, 4, 5, 1, 2, 11, 10, 1, 1),     # kh = 4, kw = 5
    (2, 16, 24, 12, 12, 3, 3, 1, 1, 12, 12, 2, 2),     # gaps of 2 (the dilated family: taps centred, same-size output)
    (2, 9, 17, 7, 7, 3, 3, 0, 0, 5, 5, 1, 1),          # "valid", odd channel counts
    (8, 64, 64, 32, 32, 3, 3, 1, 1, 32, 32, 1, 1),     # large enough for the default dispatch
]


@pytest.mark.parametrize("case", WGRAD_CASES)
def test_conv2d_kernel_gradient_from_shifted_planes(torch_cuda, pkg, vm, port, case):
    """conv2d_backward_k on the tap-row form of the tensor-core GEMM (no unfolded matrix): forced for small shapes by
    dropping the size threshold, compared with the reference loop and with fp64."""
    torch = torch_cuda
    ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, yh, yw, gh, gw = case
    rng = np.random.default_rng(sum(case) + 7)
    x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
    gy = rng.standard_normal((ndat, ychn, yh, yw)).astype(np.float32)
    lib = pkg.load()
    old = lib.kai_get_option(b"tc_min_flops")
    pkg.capi.call("kai_set_option", b"tc_min_flops", 0)
    try:
        gk = torch.full((ychn, xchn, kh, kw), float("nan"), device="cuda")
        tc0 = lib.kai_tc_launch_count()
        if gh == 1 and gw == 1:
            vm.conv2d_backward_k(0, gk, to_dev(torch, gy), to_dev(torch, x), ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, 1, ph, pw)
        else:
            vm.conv2d_dilated_backward_k(0, gk, to_dev(torch, gy), to_dev(torch, x), ndat, xchn, xh, xw, ychn, kh, kw, gh, gw)
        torch.cuda.synchronize()
        assert lib.kai_tc_launch_count() > tc0          # the tcgen05 kernel ran
    finally:
        pkg.capi.call("kai_set_option", b"tc_min_flops", old)
    got = to_host(gk)
    assert np.isfinite(got).all()
    # fp64 truth: gk[yn,xn,kr,kc] = sum gy[nd,yn,r,c] x[nd,xn,r+(kr-ph)gh,c+(kc-pw)gw]
    xp = np.zeros((ndat, xchn, xh + 2 * kh * gh, xw + 2 * kw * gw), np.float64)
    xp[:, :, kh * gh:kh * gh + xh, kw * gw:kw * gw + xw] = x
    truth = np.zeros((ychn, xchn, kh, kw))
    for kr in range(kh):
        for kc in range(kw):
            r0, c0 = kh * gh + (kr - ph) * gh, kw * gw + (kc - pw) * gw
            truth[:, :, kr, kc] = np.einsum("nors,ncrs->oc", gy.astype(np.float64), xp[:, :, r0:r0 + yh, c0:c0 + yw])
    if gh == 1 and gw == 1:
        want = port.conv2d_backward_k(gy, x, kh, kw, ph, pw)
    else:
        want = port.conv2d_variant("dilated_backward_k", (ychn, xchn, kh, kw), gy, x, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw)
    assert rel_fro(want, truth) < 1e-5          # the oracle and this test's truth mean the same map
    assert rel_fro(got, truth) <= 2 * rel_fro(want, truth) + 2e-7, f"{rel_fro(got, truth):.3e} vs {rel_fro(want, truth):.3e}"


@pytest.mark.parametrize("case", [
    (4, 32, 64, 28, 28, 3, 3, 1, 1, 28, 28),      # four output rows of 30 positions per tile
    (2, 64, 48, 30, 34, 3, 3, 1, 1, 30, 34),      # three rows of 36
    (2, 32, 32, 20, 20, 3, 3, 0, 0, 18, 18),      # "valid"
    (2, 32, 40, 24, 24, 2, 2, 0, 0, 23, 23),      # two kernel columns
])
def test_one_box_per_kernel_row_equals_one_box_per_tap(torch_cuda, pkg, vm, port, case):
    """The TMA-fed implicit-GEMM kernel in both forms (option conv_wide): one operand box per kernel row with the
    row's taps read through shifted descriptors (default), and one box per tap.  Same products, same promotion
    interval: the results agree to fp32 rounding of differently ordered sums, and both match the reference loop."""
    torch = torch_cuda
    ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, yh, yw = case
    rng = np.random.default_rng(sum(case) + 3)
    x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
    k = (rng.standard_normal((ychn, xchn, kh, kw)) / np.sqrt(xchn * kh * kw)).astype(np.float32)
    gy = rng.standard_normal((ndat, ychn, yh, yw)).astype(np.float32)
    dx, dk, dgy = (to_dev(torch, t) for t in (x, k, gy))
    lib = pkg.load()
    old_flops = lib.kai_get_option(b"tc_min_flops")
    outs = {}
    try:
        pkg.capi.call("kai_set_option", b"tc_min_flops", 0)
        for wide in (1, 0):
            pkg.capi.call("kai_set_option", b"conv_wide", wide)
            y = torch.full((ndat, ychn, yh, yw), float("nan"), device="cuda")
            gx = torch.full((ndat, xchn, xh, xw), float("nan"), device="cuda")
            tc0 = lib.kai_tc_launch_count()
            vm.conv2d(0, y, dx, dk, ndat, ychn, yh, yw, xchn, xh, xw, kh, kw, 1, ph, pw)
            vm.conv2d_backward_x(0, gx, dgy, dk, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, 1, ph, pw)
            torch.cuda.synchronize()
            assert lib.kai_tc_launch_count() - tc0 >= 2
            outs[wide] = (to_host(y), to_host(gx))
    finally:
        pkg.capi.call("kai_set_option", b"conv_wide", 1)
        pkg.capi.call("kai_set_option", b"tc_min_flops", old_flops)
    want_y = port.conv2d(x, k, yh, yw, ph, pw, 1)
    want_gx = port.conv2d_backward_x(gy, k, xh, xw, ph, pw, 1)
    for wide in (1, 0):
        assert rel_fro(outs[wide][0], want_y) < 5e-6 and rel_fro(outs[wide][1], want_gx) < 5e-6, wide
    assert rel_fro(outs[1][0], outs[0][0].astype(np.float64)) < 5e-7
    assert rel_fro(outs[1][1], outs[0][1].astype(np.float64)) < 5e-7
