"""Failure detection on the device: every wait inside the kernels of this library is bounded; on expiry
the kernel records KAI_E_DEVICE_WAIT with a location code in a host-visible status word and returns by
itself.  Here the wait is made to run out in the allowed form -- a barrier that nothing arrives at, with a
limit of one millisecond -- so nothing faults, traps or hangs; the status is read, cleared, and the next
GEMM runs normally."""
import ctypes

import numpy as np
import pytest

from helpers import to_host

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_reports_and_clears(torch_cuda, pkg, vm):
    torch = torch_cuda
    lib = pkg.load()
    assert lib.kai_device_status(0, None) == 0
    a = torch.randn((256, 256), device="cuda")
    c = torch.empty((256, 256), device="cuda")
    try:
        pkg.capi.call("kai_selftest_bounded_wait", 0, 1_000_000, None)     # 1 ms
        detail = ctypes.c_int(0)
        rc = lib.kai_device_status(0, ctypes.byref(detail))
        assert rc == pkg.capi.E_DEVICE_WAIT
        assert detail.value == 99
        assert b"bounded wait" in lib.kai_last_error_string()
        # while the word is set, the tensor-core path refuses to pretend all is well
        with pytest.raises(pkg.KaiError) as e:
            vm.sgemm(0, 0, c, a, a, 256, 256, 256, path=1)
        assert e.value.code == pkg.capi.E_DEVICE_WAIT
    finally:
        # clear: the context is intact and the same call now succeeds
        pkg.capi.call("kai_device_status_clear", 0)
    assert lib.kai_device_status(0, None) == 0
    vm.sgemm(0, 0, c, a, a, 256, 256, 256, path=1)
    torch.cuda.synchronize()
    want = a.double() @ a.double().T
    assert float((c.double() - want).norm() / want.norm()) < 1e-6
    assert lib.kai_device_status(0, None) == 0


def test_selftest_rejects_unbounded_limits(torch_cuda, pkg):
    with pytest.raises(pkg.KaiError):
        pkg.capi.call("kai_selftest_bounded_wait", 0, 5_000_000_000, None)
    with pytest.raises(pkg.KaiError):
        pkg.capi.call("kai_selftest_bounded_wait", 0, 0, None)
