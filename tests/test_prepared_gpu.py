"""Prepared operands (kai_operand_prepare / kai_linear_forward_prepared / kai_sgemm_prepared): the hi/lo
planes of an operand that does not change between calls are written once.  Results must equal the plain
calls' -- bit for bit where both run the same kernel on the same planes."""
import numpy as np
import pytest

from helpers import check_gemm_error, rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

NT, NN, TN = 0, 1, 2
TC = 1


@pytest.mark.parametrize("shape", [(300, 200, 128), (1024, 512, 1030), (129, 257, 33), (2048, 1024, 2048)])
@pytest.mark.parametrize("raw_hi", [False, True])
def test_linear_forward_with_prepared_weight(torch_cuda, pkg, vm, port, shape, raw_hi):
    torch = torch_cuda
    M, N, K = shape
    if raw_hi and K % 4:
        pytest.skip("KAI_PREP_RAW_HI needs k % 4 == 0")
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    dx, dw, db = to_dev(torch, x), to_dev(torch, w), to_dev(torch, b)
    wp = vm.PreparedOperand(0, dw, N, K, raw_hi=raw_hi)
    try:
        y = torch.full((M, N), float("nan"), device="cuda")
        vm.linear_forward_prepared(0, y, wp, dx, db, M, act="relu")
        want = torch.empty((M, N), device="cuda")
        vm.sgemm(0, NT, want, dx, dw, M, N, K, bias=db, act="relu", path=TC)
        torch.cuda.synchronize()
        truth = np.maximum(x.astype(np.float64) @ w.astype(np.float64).T + b, 0)
        rows = slice(0, min(M, 32))
        ref = port.activate(port.add_bias(port.matmul(w, np.ascontiguousarray(x[rows])), b), 1)
        check_gemm_error(rel_fro(to_host(y), truth), rel_fro(ref, truth[rows]), K, f"prepared W {shape}")
        assert rel_fro(to_host(y), to_host(want).astype(np.float64)) < 1e-6
        # new weights of the same shape: refresh, not a new handle
        if not raw_hi:
            w2 = (w * 0.5 + 0.25).astype(np.float32)
            wp.refresh(to_dev(torch, w2))
            vm.linear_forward_prepared(0, y, wp, dx, None, M)
            torch.cuda.synchronize()
            truth2 = x.astype(np.float64) @ w2.astype(np.float64).T
            assert rel_fro(to_host(y), truth2) < 1e-5 * np.sqrt(K)
    finally:
        wp.release()


def test_sgemm_prepared_row_slabs_equal_the_whole(torch_cuda, pkg, vm, port):
    """dW = dY^T . X computed in four row slabs of dW from two prepared (transposed) operands: every slab is
    the same tiles the whole call computes, so the assembled result has the whole call's bits."""
    torch = torch_cuda
    tokens, N, K = 1024, 1024, 768           # dW [N, K]
    rng = np.random.default_rng(9)
    dy = rng.standard_normal((tokens, N), dtype=np.float32)
    x = rng.standard_normal((tokens, K), dtype=np.float32)
    ddy, dx = to_dev(torch, dy), to_dev(torch, x)
    a = vm.PreparedOperand(0, ddy, N, tokens, transpose=True)     # A' = dY^T: [N][tokens]
    b = vm.PreparedOperand(0, dx, K, tokens, transpose=True)      # B' = X^T : [K][tokens]
    try:
        whole = torch.empty((N, K), device="cuda")
        vm.sgemm_prepared(0, whole, a, 0, N, b, 0, K)
        slabs = torch.full((N, K), float("nan"), device="cuda")
        for r0 in range(0, N, 256):
            vm.sgemm_prepared(0, slabs.data_ptr() + 4 * r0 * K, a, r0, 256, b, 0, K, ldc=K)
        plain = torch.empty((N, K), device="cuda")
        vm.matmul_backward_w(0, plain, ddy, dx, N, tokens, K, False)
        torch.cuda.synchronize()
        truth = dy.astype(np.float64).T @ x.astype(np.float64)
        ref = port.matmul_backward_w(np.ascontiguousarray(dy[:, :8]), x, 8, K)
        check_gemm_error(rel_fro(to_host(whole), truth), rel_fro(ref, truth[:8]), tokens, "prepared dW")
        check_gemm_error(rel_fro(to_host(slabs), truth), rel_fro(ref, truth[:8]), tokens, "prepared dW in slabs")
        assert rel_fro(to_host(plain), to_host(whole).astype(np.float64)) < 1e-6
        # column slabs of the second operand and accumulation
        acc = torch.ones((N, K), device="cuda")
        vm.sgemm_prepared(0, acc.data_ptr() + 4 * 256, a, 0, N, b, 256, 128, ldc=K, accumulate=True)
        torch.cuda.synchronize()
        got = to_host(acc)
        np.testing.assert_allclose(got[:, 256:384], 1.0 + truth[:, 256:384], rtol=1e-4, atol=1e-3)
        assert (got[:, :256] == 1.0).all() and (got[:, 384:] == 1.0).all()
    finally:
        a.release()
        b.release()


def test_prepared_argument_checks(torch_cuda, pkg, vm):
    torch = torch_cuda
    t = torch.zeros((64, 64), device="cuda")
    a = vm.PreparedOperand(0, t, 64, 64)
    b = vm.PreparedOperand(0, t[:, :32].contiguous(), 64, 32)
    try:
        with pytest.raises(pkg.KaiError) as e:
            vm.sgemm_prepared(0, t, a, 0, 64, b, 0, 64)           # reduction lengths differ
        assert e.value.code == pkg.capi.E_INVALID_ARG
        with pytest.raises(pkg.KaiError):
            vm.sgemm_prepared(0, t, a, 32, 64, a, 0, 64)          # rows outside the operand
        with pytest.raises(pkg.KaiError):
            pkg.capi.call("kai_operand_refresh", t.data_ptr(), t.data_ptr(), None)   # not a handle
    finally:
        a.release()
        b.release()
    with pytest.raises(pkg.KaiError):
        vm.PreparedOperand(0, t.data_ptr() + 4, 63, 63, ld=64, raw_hi=True)          # raw hi needs a dense aligned matrix
