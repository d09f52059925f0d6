"""Parity at the full sizes of the five benchmark configurations.

The other GPU tests sweep shapes the CPU oracle finishes in seconds; the launches that the benchmark
times (8192^3 with its 2048-tile persistent schedule, the 8192 x 4096 x 4096 Linear step in all three
layouts, the skinny sweep at N = K = 4096, attention at 32 batch items) are checked here.

fp64 ground truth is computed on the GPU with torch (float64 matmul); the reference's own fp32 loop
(the oracle) runs on a slab of output rows -- rows are independent in all three reference loops
(support/vmath.cu:2962, 3008, 3052) and batch items in the attention loops (:6729-6750) -- which
gives the "no worse than 2x the reference CPU path's error" clause of the acceptance rule.
"""
import importlib

import numpy as np
import pytest

from helpers import check_gemm_error, rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

NT, NN, TN = 0, 1, 2
TC = 1
wl = importlib.import_module("deep-learning-framework_b200.workloads")


def _rel_fro_dev(torch, got32, truth64) -> float:
    d = got32.double() - truth64
    return float(torch.linalg.norm(d.flatten()) / torch.linalg.norm(truth64.flatten()))


@pytest.fixture(scope="module")
def cfg4(torch_cuda):
    torch = torch_cuda
    x, w = wl.gemm_large()
    dx, dw = to_dev(torch, x), to_dev(torch, w)
    truth = dx.double() @ dw.double().T
    yield x, w, dx, dw, truth
    del dx, dw, truth
    torch.cuda.empty_cache()


def test_config4_whole_8192_cubed(torch_cuda, vm, port, cfg4):
    """The benchmarked launch itself: matmul(d, Y, W, X, 8192, 8192, 8192, false)."""
    torch = torch_cuda
    x, w, dx, dw, truth = cfg4
    y = torch.full((8192, 8192), float("nan"), device="cuda")
    vm.matmul(0, y, dw, dx, 8192, 8192, 8192, False)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(y).all())
    err = _rel_fro_dev(torch, y, truth)
    rows = slice(4096, 4112)            # a slab in the middle of the tile grid
    ref = port.matmul(w, np.ascontiguousarray(x[rows]))
    t_slab = to_host(truth[rows])
    err_ref = rel_fro(ref, t_slab)
    err_slab = rel_fro(to_host(y[rows]), t_slab)
    print(f"8192^3: gpu {err:.3e} (slab {err_slab:.3e}) reference slab {err_ref:.3e}")
    check_gemm_error(err, err_ref, 8192, "config 4 whole")
    check_gemm_error(err_slab, err_ref, 8192, "config 4 slab")
    # a second run gives the same bits (fixed tile schedule, fixed promotion order)
    y2 = torch.empty_like(y)
    vm.matmul(0, y2, dw, dx, 8192, 8192, 8192, False)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)


@pytest.mark.parametrize("grid", [(1, 8), (2, 4), (1, 2), (2, 2)])
def test_config4_rank_shapes_write_into_full_width_output(torch_cuda, vm, cfg4, grid):
    """Every rank's call of the column-slab (1 x G) and block (pr x pc) partitions, written with ldc = 8192
    into one full-width Y; the assembled Y must equal the single-call result's accuracy."""
    torch = torch_cuda
    x, w, dx, dw, truth = cfg4
    pr, pc = grid
    y = torch.full((8192, 8192), float("nan"), device="cuda")
    mrows, ncols = 8192 // pr, 8192 // pc
    ranks = [(0, 0), (pr - 1, pc - 1)] if pr * pc > 4 else [(i, j) for i in range(pr) for j in range(pc)]
    for i, j in ranks:
        m0, n0 = i * mrows, j * ncols
        vm.sgemm(0, NT, y.data_ptr() + 4 * (m0 * 8192 + n0), dx.data_ptr() + 4 * m0 * 8192,
                 dw.data_ptr() + 4 * n0 * 8192, mrows, ncols, 8192, ldc=8192)
    torch.cuda.synchronize()
    for i, j in ranks:
        blk = (slice(i * mrows, (i + 1) * mrows), slice(j * ncols, (j + 1) * ncols))
        assert bool(torch.isfinite(y[blk]).all())
        err = _rel_fro_dev(torch, y[blk], truth[blk])
        assert err <= 2.0e-6, f"grid {grid} rank {(i, j)}: {err:.3e}"      # the whole-call figure is ~9e-7
    if pr * pc > 4:   # untouched blocks stay untouched
        assert bool(torch.isnan(y[:mrows, ncols:2 * ncols]).all())


@pytest.fixture(scope="module")
def cfg5(torch_cuda):
    torch = torch_cuda
    d = wl.linear_step()
    t = {k: to_dev(torch, v) for k, v in d.items()}
    yield d, t
    del t
    torch.cuda.empty_cache()


def test_config5_linear_forward_with_bias(torch_cuda, vm, port, cfg5):
    torch = torch_cuda
    d, t = cfg5
    M, N, K = 8192, 4096, 4096
    y = torch.full((M, N), float("nan"), device="cuda")
    vm.linear_forward(0, y, t["w"], t["x"], t["b"], N, M, K)
    torch.cuda.synchronize()
    truth = t["x"].double() @ t["w"].double().T + t["b"].double()
    err = _rel_fro_dev(torch, y, truth)
    rows = slice(8176, 8192)
    ref = port.add_bias(port.matmul(d["w"], np.ascontiguousarray(d["x"][rows])), d["b"])
    err_ref = rel_fro(ref, to_host(truth[rows]))
    print(f"config 5 forward: gpu {err:.3e} reference slab {err_ref:.3e}")
    check_gemm_error(err, err_ref, K, "config 5 Y = X.W^T + b")


def test_config5_backward_x(torch_cuda, vm, port, cfg5):
    torch = torch_cuda
    d, t = cfg5
    M, N, K = 8192, 4096, 4096      # ndat, yvec, xvec
    gx = torch.full((M, K), float("nan"), device="cuda")
    vm.matmul_backward_x(0, gx, t["dy"], t["w"], N, M, K, False)
    torch.cuda.synchronize()
    truth = t["dy"].double() @ t["w"].double()
    err = _rel_fro_dev(torch, gx, truth)
    rows = slice(100, 108)
    ref = port.matmul_backward_x(np.ascontiguousarray(d["dy"][rows]), d["w"])
    err_ref = rel_fro(ref, to_host(truth[rows]))
    print(f"config 5 dX: gpu {err:.3e} reference slab {err_ref:.3e}")
    check_gemm_error(err, err_ref, N, "config 5 dX = dY.W")


def test_config5_backward_w_and_token_shards(torch_cuda, vm, port, cfg5):
    """dW = dY^T.X over all 8192 tokens, and as the sum of 8 token shards (the K-split whose partials the
    multi-GPU step all-reduces) -- the shards use acc into one buffer here."""
    torch = torch_cuda
    d, t = cfg5
    M, N, K = 8192, 4096, 4096
    gw = torch.full((N, K), float("nan"), device="cuda")
    vm.matmul_backward_w(0, gw, t["dy"], t["x"], N, M, K, False)
    torch.cuda.synchronize()
    truth = t["dy"].double().T @ t["x"].double()
    err = _rel_fro_dev(torch, gw, truth)
    # reference loop on 4 output rows: dW[n, :] needs column n of dY only
    cols = slice(2048, 2052)
    ref = port.matmul_backward_w(np.ascontiguousarray(d["dy"][:, cols]), d["x"], 4, K)
    err_ref = rel_fro(ref, to_host(truth[cols]))
    print(f"config 5 dW: gpu {err:.3e} reference slab {err_ref:.3e}")
    check_gemm_error(err, err_ref, M, "config 5 dW = dY^T.X")
    acc = torch.zeros((N, K), device="cuda")
    for g in range(8):
        r0 = g * 1024
        vm.matmul_backward_w(0, acc, t["dy"].data_ptr() + 4 * r0 * N, t["x"].data_ptr() + 4 * r0 * K, N, 1024, K,
                             True)
    torch.cuda.synchronize()
    check_gemm_error(_rel_fro_dev(torch, acc, truth), err_ref, M, "config 5 dW as 8 token shards")


@pytest.mark.parametrize("M", [1, 4, 8, 16])
def test_config5_skinny_sweep(torch_cuda, vm, port, cfg5, M):
    torch = torch_cuda
    d, t = cfg5
    N = K = 4096
    x = np.ascontiguousarray(d["x"][:M])
    y = torch.full((M, N), float("nan"), device="cuda")
    vm.matmul(0, y, t["w"], to_dev(torch, x), N, M, K, False)
    torch.cuda.synchronize()
    truth = x.astype(np.float64) @ d["w"].astype(np.float64).T
    ref = port.matmul(d["w"], x)
    got = to_host(y)
    assert np.isfinite(got).all()
    check_gemm_error(rel_fro(got, truth), rel_fro(ref, truth), K, f"skinny M={M}")


def _attention_truth(torch, q, k, v, H, P, coef):
    nb, T, _ = q.shape
    q4, k4, v4 = (t.double().view(nb, T, H, P).permute(0, 2, 1, 3) for t in (q, k, v))   # [b,h,t,p]
    s = (q4 @ k4.transpose(-1, -2)) * coef                                                  # [b,h,q,k]
    pr = torch.softmax(s, dim=-1)
    o = pr @ v4                                                                             # [b,h,q,p]
    return pr.permute(0, 2, 3, 1).contiguous(), o.permute(0, 2, 1, 3).contiguous()          # [b,q,k,h], [b,q,h,p]


def test_config3_attention_nbat32_separate_and_fused(torch_cuda, vm, port):
    torch = torch_cuda
    nb, T, H, P = 32, 512, 8, 64
    q, k, v, coef = wl.attention()
    dq, dk, dv = (to_dev(torch, t) for t in (q, k, v))
    dcoef = torch.tensor([coef], device="cuda")
    probs = torch.full((nb, T, T, H), float("nan"), device="cuda")
    out = torch.full((nb, T, H, P), float("nan"), device="cuda")
    fused = torch.full((nb, T, H, P), float("nan"), device="cuda")
    vm.mult_on_heads(0, probs, dk, dq, nb, T, H * P, H, P, dcoef)
    vm.softmax_direct_on_axis(0, probs, nb * T, T, H)
    vm.mix_values(0, out, probs, dv, nb, T, H * P, H, P)
    vm.mh_attention_forward(0, fused, dk, dq, dv, nb, T, H * P, H, P, dcoef)
    torch.cuda.synchronize()
    errs_p, errs_o, errs_f = [], [], []
    for b0 in range(0, nb, 8):      # fp64 truth in groups of 8 batch items (probs in fp64 is 134 MB per group)
        tp, to = _attention_truth(torch, dq[b0:b0 + 8], dk[b0:b0 + 8], dv[b0:b0 + 8], H, P, coef)
        errs_p.append(_rel_fro_dev(torch, probs[b0:b0 + 8], tp))
        errs_o.append(_rel_fro_dev(torch, out[b0:b0 + 8], to))
        errs_f.append(_rel_fro_dev(torch, fused[b0:b0 + 8], to))
        if b0 == 24:
            t_last = to_host(to[7:8])
    # the reference's three loops on the last batch item
    ref = port.mix_values(port.softmax_direct_on_axis(port.mult_on_heads(k[31:], q[31:], H, coef)), v[31:], H)
    err_ref = rel_fro(ref, t_last)
    print(f"attention nbat=32: probs {max(errs_p):.3e} out {max(errs_o):.3e} fused {max(errs_f):.3e} "
          f"reference (one item) {err_ref:.3e}")
    assert bool(torch.isfinite(out).all()) and bool(torch.isfinite(fused).all())
    for name, e in (("probs", max(errs_p)), ("out", max(errs_o)), ("fused", max(errs_f))):
        check_gemm_error(e, err_ref, T, f"config 3 {name}")
    check_gemm_error(rel_fro(to_host(out[31:]), t_last), err_ref, T, "config 3 out, last item")
    check_gemm_error(rel_fro(to_host(fused[31:]), t_last), err_ref, T, "config 3 fused, last item")


@pytest.mark.parametrize("dist", ["normal", "full_mantissa"])
def test_raw_hi_operand_equals_rounded_hi_within_the_rule(torch_cuda, pkg, vm, port, dist):
    """The tensor core is fed the caller's fp32 matrix as the hi operand where the layout allows
    (option tc_raw_hi: 1 = always, 2 = never); the lo plane is then taken against the truncated high
    part.  Both forms must satisfy the acceptance rule and agree closely -- also on values whose low 13
    mantissa bits are all set, where truncation and rounding differ most."""
    torch = torch_cuda
    M, N, K = 512, 768, 1536      # below 2048: reductions from there on never read an operand as its own hi plane
    rng = np.random.default_rng(77)
    a = rng.standard_normal((M, K), dtype=np.float32)
    b = rng.standard_normal((N, K), dtype=np.float32)
    if dist == "full_mantissa":
        a = (a.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
        b = (b.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    truth = a.astype(np.float64) @ b.astype(np.float64).T
    ref = port.matmul(b, np.ascontiguousarray(a[:16]))
    err_ref = rel_fro(ref, truth[:16])
    da, db = to_dev(torch, a), to_dev(torch, b)
    lib = pkg.load()
    old = lib.kai_get_option(b"tc_raw_hi")
    outs = {}
    try:
        for mode in (1, 2):
            pkg.capi.call("kai_set_option", b"tc_raw_hi", mode)
            c = torch.full((M, N), float("nan"), device="cuda")
            vm.sgemm(0, NT, c, da, db, M, N, K, path=TC)
            torch.cuda.synchronize()
            outs[mode] = to_host(c)
    finally:
        pkg.capi.call("kai_set_option", b"tc_raw_hi", old)
    e1, e2 = rel_fro(outs[1], truth), rel_fro(outs[2], truth)
    print(f"{dist}: raw hi {e1:.3e} rounded hi {e2:.3e} reference {err_ref:.3e}")
    check_gemm_error(e1, err_ref, K, f"raw hi, {dist}")
    check_gemm_error(e2, err_ref, K, f"rounded hi, {dist}")
    assert rel_fro(outs[1], outs[2].astype(np.float64)) <= 1e-6
