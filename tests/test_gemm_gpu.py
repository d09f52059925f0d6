"""GPU parity of the GEMM trio against the CPU oracle and an fp64 ground truth.

The path's acceptance rule: relative Frobenius error against fp64 <= 1e-5*sqrt(K) and <= 2x the error of
the reference's own fp32 CPU path on the same inputs.
"""
import numpy as np
import pytest

from helpers import check_gemm_error, gemm_truth, rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

NT, NN, TN = 0, 1, 2
TC, SIMT, SKINNY = 1, 2, 3


def _operands(layout, M, N, K, seed, dist="uniform"):
    rng = np.random.default_rng(seed)
    draw = (lambda s: rng.uniform(-1, 1, s).astype(np.float32)) if dist == "uniform" else (
        lambda s: rng.standard_normal(s, dtype=np.float32))
    a = draw((M, K)) if layout != TN else draw((K, M))
    b = draw((N, K)) if layout == NT else draw((K, N))
    return a, b


def _oracle_gemm(port, layout, a, b, M, N, K, acc_into=None):
    if layout == NT:
        return port.matmul(b, a, acc_into)
    if layout == NN:
        return port.matmul_backward_x(a, b, acc_into)  # pgy=a [M,K], pw=b [K,N]
    return port.matmul_backward_w(a, b, M, N, acc_into)  # pgy=a [K,M], px=b [K,N]


@pytest.mark.parametrize("path", [TC, SIMT])
@pytest.mark.parametrize("layout", [NT, NN, TN])
@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 300, 100), (129, 257, 33), (64, 48, 7), (512, 512, 512),
                                   (1, 5, 3), (257, 130, 1000), (128, 512, 784), (64, 2048, 512), (100, 10, 512)])
def test_gemm_matches_oracle(torch_cuda, vm, port, path, layout, shape):
    torch = torch_cuda
    M, N, K = shape
    a, b = _operands(layout, M, N, K, seed=M * 7 + N * 3 + K)
    truth = gemm_truth(layout, a, b)
    ref = _oracle_gemm(port, layout, a, b, M, N, K)
    c = torch.full((M, N), float("nan"), device="cuda")
    vm.sgemm(0, layout, c, to_dev(torch, a), to_dev(torch, b), M, N, K, path=path)
    torch.cuda.synchronize()
    got = to_host(c)
    assert np.isfinite(got).all()
    check_gemm_error(rel_fro(got, truth), rel_fro(ref, truth), K, f"layout={layout} path={path} {shape}")


@pytest.mark.parametrize("bn,bk", [(256, 16), (256, 32), (128, 16), (128, 32)])
def test_tc_tile_variants(torch_cuda, pkg, vm, port, bn, bk):
    torch = torch_cuda
    M, N, K = 384, 640, 328
    a, b = _operands(NT, M, N, K, seed=5)
    truth = gemm_truth(NT, a, b)
    ref = port.matmul(b, a)
    lib = pkg.load()
    old = lib.kai_get_option(b"tc_bn"), lib.kai_get_option(b"tc_bk")
    try:
        pkg.capi.call("kai_set_option", b"tc_bn", bn)
        pkg.capi.call("kai_set_option", b"tc_bk", bk)
        c = torch.zeros((M, N), device="cuda")
        vm.sgemm(0, NT, c, to_dev(torch, a), to_dev(torch, b), M, N, K, path=TC)
        torch.cuda.synchronize()
    finally:
        pkg.capi.call("kai_set_option", b"tc_bn", old[0])
        pkg.capi.call("kai_set_option", b"tc_bk", old[1])
    check_gemm_error(rel_fro(to_host(c), truth), rel_fro(ref, truth), K, f"bn={bn} bk={bk}")


@pytest.mark.parametrize("path", [TC, SIMT])
@pytest.mark.parametrize("layout", [NT, NN, TN])
def test_accumulate_bias_activation_ldc(torch_cuda, vm, port, path, layout):
    """acc=true reads the old output; bias and activation are applied after it; ldc > N leaves the
    columns outside the block untouched."""
    torch = torch_cuda
    M, N, K, ldc = 150, 200, 96, 264
    a, b = _operands(layout, M, N, K, seed=11, dist="normal")
    rng = np.random.default_rng(3)
    bias = rng.standard_normal(N, dtype=np.float32)
    old = rng.standard_normal((M, ldc), dtype=np.float32)
    alpha = np.array([0.1], np.float32)
    expect = _oracle_gemm(port, layout, a, b, M, N, K, acc_into=np.ascontiguousarray(old[:, :N]))
    expect = port.activate(port.add_bias(expect, bias), 2, 0.1)
    c = to_dev(torch, old)
    vm.sgemm(0, layout, c, to_dev(torch, a), to_dev(torch, b), M, N, K, ldc=ldc, accumulate=True,
             bias=to_dev(torch, bias), act="leaky", leaky_alpha=to_dev(torch, alpha), path=path)
    torch.cuda.synchronize()
    got = to_host(c)
    np.testing.assert_array_equal(got[:, N:], old[:, N:])
    np.testing.assert_allclose(got[:, :N], expect, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("regx", [1, 0])
@pytest.mark.parametrize("K", [1024, 1100, 256, 4096])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 7, 8, 9, 16])
def test_skinny_rows(torch_cuda, pkg, vm, port, M, K, regx):
    """M <= 4 streams W rows with X from L1; M = 5..16 keeps X in registers (regx = 1) or uses the
    streaming kernel as well (regx = 0)."""
    torch = torch_cuda
    N = 1030
    if regx == 0 and M <= 4:
        pytest.skip("same kernel as regx = 1")
    pkg.capi.call("kai_set_option", b"skinny_regx", regx)
    a, b = _operands(NT, M, N, K, seed=M, dist="normal")
    truth = gemm_truth(NT, a, b)
    ref = port.matmul(b, a)
    bias = np.random.default_rng(1).standard_normal(N, dtype=np.float32)
    c = torch.zeros((M, N), device="cuda")
    try:
        vm.sgemm(0, NT, c, to_dev(torch, a), to_dev(torch, b), M, N, K, bias=to_dev(torch, bias), act="relu",
                 path=SKINNY)
        torch.cuda.synchronize()
    finally:
        pkg.capi.call("kai_set_option", b"skinny_regx", 1)
    expect = np.maximum(truth + bias, 0)
    ref_full = port.activate(port.add_bias(ref, bias), 1)
    check_gemm_error(rel_fro(to_host(c), expect), rel_fro(ref_full, expect), K, f"skinny M={M}")


def test_split_k_is_deterministic(torch_cuda, pkg, vm, port):
    """Few tiles and a long reduction: the K-split path; two runs must agree bit for bit."""
    torch = torch_cuda
    M, N, K = 256, 256, 4096
    a, b = _operands(NT, M, N, K, seed=2)
    truth = gemm_truth(NT, a, b)
    ref = port.matmul(b, a)
    da, db = to_dev(torch, a), to_dev(torch, b)
    outs = []
    for _ in range(2):
        c = torch.zeros((M, N), device="cuda")
        vm.sgemm(0, NT, c, da, db, M, N, K, path=TC)
        torch.cuda.synchronize()
        outs.append(to_host(c))
    np.testing.assert_array_equal(outs[0], outs[1])
    check_gemm_error(rel_fro(outs[0], truth), rel_fro(ref, truth), K, "split-K")
    pkg.capi.call("kai_set_option", b"split_k", 1)
    try:
        c = torch.zeros((M, N), device="cuda")
        vm.sgemm(0, NT, c, da, db, M, N, K, path=TC)
        torch.cuda.synchronize()
    finally:
        pkg.capi.call("kai_set_option", b"split_k", 0)
    check_gemm_error(rel_fro(to_host(c), truth), rel_fro(ref, truth), K, "no split")


def test_reference_entry_points(torch_cuda, vm, port):
    """kai_matmul / _backward_x / _backward_w take the reference's argument order."""
    torch = torch_cuda
    ndat, xvec, yvec = 96, 160, 224
    rng = np.random.default_rng(9)
    x = rng.standard_normal((ndat, xvec), dtype=np.float32)
    w = rng.standard_normal((yvec, xvec), dtype=np.float32)
    gy = rng.standard_normal((ndat, yvec), dtype=np.float32)
    dx, dw, dgy = to_dev(torch, x), to_dev(torch, w), to_dev(torch, gy)
    y = torch.zeros((ndat, yvec), device="cuda")
    gx = torch.zeros((ndat, xvec), device="cuda")
    gw = torch.zeros((yvec, xvec), device="cuda")
    vm.matmul(0, y, dw, dx, yvec, ndat, xvec, False)
    vm.matmul_backward_x(0, gx, dgy, dw, yvec, ndat, xvec, False)
    vm.matmul_backward_w(0, gw, dgy, dx, yvec, ndat, xvec, False)
    torch.cuda.synchronize()
    np.testing.assert_allclose(to_host(y), port.matmul(w, x), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(to_host(gx), port.matmul_backward_x(gy, w), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(to_host(gw), port.matmul_backward_w(gy, x, yvec, xvec), rtol=1e-4, atol=1e-4)


def test_interior_pointers(torch_cuda, vm, port):
    """Operands 4-byte but not 16-byte aligned (the RNN path passes interior pointers)."""
    torch = torch_cuda
    M, N, K = 130, 70, 50
    rng = np.random.default_rng(4)
    a = rng.standard_normal(M * K + 3, dtype=np.float32)
    b = rng.standard_normal(N * K + 1, dtype=np.float32)
    da, db = to_dev(torch, a), to_dev(torch, b)
    dc = torch.zeros(M * N + 1, device="cuda")
    A, B = a[3:].reshape(M, K), b[1:].reshape(N, K)
    for path in (TC, SIMT):
        dc.zero_()
        vm.sgemm(0, NT, dc.data_ptr() + 4, da.data_ptr() + 12, db.data_ptr() + 4, M, N, K, path=path)
        torch.cuda.synchronize()
        got = to_host(dc)[1:].reshape(M, N)
        np.testing.assert_allclose(got, port.matmul(np.ascontiguousarray(B), np.ascontiguousarray(A)), rtol=1e-4,
                                   atol=1e-4)


@pytest.mark.parametrize("K", [2048, 8192])
def test_long_reduction_accuracy(torch_cuda, vm, port, K):
    """The 2x clause at long K, where tensor-core accumulation order matters.  The oracle is run on
    a 16-row slab (rows are independent in the reference loop) to keep the CPU time in seconds."""
    torch = torch_cuda
    M, N = 256, 512
    a, b = _operands(NT, M, N, K, seed=K)
    truth = gemm_truth(NT, a, b)
    ref_slab = port.matmul(b, np.ascontiguousarray(a[:16]))
    err_ref = rel_fro(ref_slab, truth[:16])
    c = torch.zeros((M, N), device="cuda")
    vm.sgemm(0, NT, c, to_dev(torch, a), to_dev(torch, b), M, N, K, path=TC)
    torch.cuda.synchronize()
    err = rel_fro(to_host(c), truth)
    print(f"K={K}: gpu {err:.3e} reference {err_ref:.3e}")
    check_gemm_error(err, err_ref, K, f"K={K}")


def test_edge_sizes(torch_cuda, vm):
    torch = torch_cuda
    c = torch.full((4, 4), 7.0, device="cuda")
    a = torch.zeros(16, device="cuda")
    vm.sgemm(0, NT, c, a, a, 0, 4, 4)        # M = 0: nothing happens
    vm.sgemm(0, NT, c, a, a, 4, 4, 0)        # K = 0: C = 0
    torch.cuda.synchronize()
    assert float(c.abs().sum()) == 0.0
    c.fill_(7.0)
    vm.sgemm(0, NT, c, a, a, 4, 4, 0, accumulate=True)  # K = 0 with acc: C unchanged
    torch.cuda.synchronize()
    assert float(c.min()) == 7.0


@pytest.mark.parametrize("shape", [(70, 50, 33), (300, 200, 128), (5000, 1100, 1028), (4096, 512, 2048),
                                   (4500, 2048, 2048), (4608, 1024, 4096)])   # the last two run in row chunks (ragged / even)
def test_matmul_on_host_buffers(torch_cuda, vm, port, shape):
    """kai_matmul_host: operands and result in (pinned) host memory, rows processed in pipelined chunks."""
    torch = torch_cuda
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    x = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    w = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    hx, hw, hb = (torch.from_numpy(t).pin_memory() for t in (x, w, bias))
    hy = torch.full((M, N), float("nan")).pin_memory()
    vm.matmul_host(0, hy, hw, hx, N, M, K, hb, act="relu")
    got = hy.numpy()
    rows = slice(0, min(M, 64))                      # the CPU loop on a slab of rows (rows are independent)
    want = port.activate(port.add_bias(port.matmul(w, np.ascontiguousarray(x[rows])), bias), 1)
    truth = np.maximum(x.astype(np.float64) @ w.astype(np.float64).T + bias, 0.0)
    assert np.isfinite(got).all()
    check_gemm_error(rel_fro(got, truth), rel_fro(want, truth[rows]), K, f"matmul_host {shape}")
    # a second call reuses the cached device blocks and gives the same bits
    hy2 = torch.empty((M, N)).pin_memory()
    vm.matmul_host(0, hy2, hw, hx, N, M, K, hb, act="relu")
    assert torch.equal(hy, hy2)
