"""kai_linear_forward_static: the Linear forward for hosts that cannot allocate device memory
while they run (a replayed call list with fixed pointers, a process whose own pool owns all of
HBM).  Its scratch is a fixed array inside the library instead of a cudaMalloc'ed workspace, so
the test checks three things through the C ABI: it returns what kai_linear_forward returns, it
still does so on a second call that reuses the array with another shape, and it refuses problems
that do not fit.  The file name sorts last on purpose: a run that stops at the first failure has
then already been through every other test."""
import ctypes

import numpy as np
import pytest

from helpers import to_dev, to_host

pytestmark = pytest.mark.gpu

TC = 1


def _case(torch, vm, ndat, xvec, yvec, act, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((ndat, xvec), dtype=np.float32)
    w = (rng.standard_normal((yvec, xvec), dtype=np.float32) / np.sqrt(xvec)).astype(np.float32)
    b = rng.standard_normal(yvec, dtype=np.float32)
    dx, dw, db = to_dev(torch, x), to_dev(torch, w), to_dev(torch, b)
    alpha = to_dev(torch, np.array([0.1], np.float32))
    want = torch.empty((ndat, yvec), device="cuda")
    vm.sgemm(0, 0, want, dx, dw, ndat, yvec, xvec, bias=db, act=act, leaky_alpha=alpha, path=TC)
    got = torch.full((ndat, yvec), float("nan"), device="cuda")
    vm.linear_forward_static(0, got, dw, dx, db, yvec, ndat, xvec, act=act, leaky_alpha=alpha)
    torch.cuda.synchronize()
    return to_host(got), to_host(want)


def test_static_scratch_matches_regular_path_twice(torch_cuda, vm):
    torch = torch_cuda
    # Two calls in a row with different shapes: the second one finds the first one's planes in the array.
    for ndat, xvec, yvec, act, seed in [(300, 500, 200, "relu", 0), (130, 1030, 520, "leaky", 1),
                                        (300, 500, 200, "relu", 0)]:
        got, want = _case(torch, vm, ndat, xvec, yvec, act, seed)
        assert np.isfinite(got).all()
        # Same kernel; only the K-split of the regular path can change the summation order.
        np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5)


def test_static_scratch_same_bits_without_split_k(torch_cuda, pkg, vm):
    torch = torch_cuda
    pkg.capi.call("kai_set_option", b"split_k", 1)
    pkg.capi.call("kai_set_option", b"tc_raw_hi", 2)   # the regular path may read small operands as their own hi plane
    try:
        for _ in range(2):
            got, want = _case(torch, vm, 256, 768, 384, "none", 2)
            np.testing.assert_array_equal(got, want)
    finally:
        pkg.capi.call("kai_set_option", b"split_k", 0)
        pkg.capi.call("kai_set_option", b"tc_raw_hi", 0)


def test_static_scratch_refuses_what_does_not_fit(torch_cuda, pkg, vm):
    torch = torch_cuda
    t = torch.zeros(16, device="cuda")
    with pytest.raises(pkg.KaiError) as e:
        vm.linear_forward_static(0, t, t, t, None, 4096, 4096, 4096)   # 256 MiB of planes
    assert e.value.code == pkg.capi.E_TOO_LARGE
    assert "33554432" in e.value.message
    # the largest documented case fits: ndat = yvec = 1024, xvec = 2048 -> exactly 32 MiB
    rng = np.random.default_rng(3)
    x = to_dev(torch, rng.standard_normal((1024, 2048), dtype=np.float32))
    w = to_dev(torch, rng.standard_normal((1024, 2048), dtype=np.float32))
    y = torch.empty((1024, 1024), device="cuda")
    vm.linear_forward_static(0, y, w, x, None, 1024, 1024, 2048)
    torch.cuda.synchronize()
    ref = x.double() @ w.double().T
    assert float((y.double() - ref).norm() / ref.norm()) < 2e-6


def _driver_allocs(pkg) -> int:
    n = ctypes.c_int64(0)
    pkg.capi.call("kai_mem_stats", 0, None, None, ctypes.byref(n))
    return n.value


def test_static_scratch_allocates_nothing_and_replays(torch_cuda, pkg, vm):
    """Free device memory and the library's own allocation count are the same before and after the calls, and
    the call can sit in a recorded list that is replayed with fixed pointers (the host it was written for)."""
    torch = torch_cuda
    rng = np.random.default_rng(5)
    ndat, xvec, yvec = 384, 640, 512
    x = to_dev(torch, rng.standard_normal((ndat, xvec), dtype=np.float32))
    w = to_dev(torch, (rng.standard_normal((yvec, xvec), dtype=np.float32) / 25).astype(np.float32))
    b = to_dev(torch, rng.standard_normal(yvec, dtype=np.float32))
    want = torch.empty((ndat, yvec), device="cuda")
    got = torch.full((ndat, yvec), float("nan"), device="cuda")
    vm.linear_forward(0, want, w, x, b, yvec, ndat, xvec, act="tanh")
    vm.linear_forward_static(0, got, w, x, b, yvec, ndat, xvec, act="tanh")     # first call: set-up happens here
    torch.cuda.synchronize()
    free0, allocs0 = torch.cuda.mem_get_info()[0], _driver_allocs(pkg)
    for _ in range(3):
        got.fill_(float("nan"))
        vm.linear_forward_static(0, got, w, x, b, yvec, ndat, xvec, act="tanh")
        torch.cuda.synchronize()
        np.testing.assert_allclose(to_host(got), to_host(want), rtol=2e-5, atol=2e-5)
    assert torch.cuda.mem_get_info()[0] == free0
    assert _driver_allocs(pkg) == allocs0
    # recorded once, replayed twice
    with vm.Replay(0) as rp:
        vm.linear_forward_static(0, got, w, x, b, yvec, ndat, xvec, act="tanh", stream=rp.stream)
    try:
        for _ in range(2):
            got.fill_(float("nan"))
            torch.cuda.synchronize()
            rp.launch()
            torch.cuda.synchronize()
            np.testing.assert_allclose(to_host(got), to_host(want), rtol=2e-5, atol=2e-5)
        assert pkg.load().kai_device_status(0, None) == 0
    finally:
        rp.close()
    assert _driver_allocs(pkg) == allocs0
