"""The two MMA schemes of the tensor-core GEMM and the CTA-pair form of its kernel.

Reductions of 2048 values and more (K % 8 == 0) form the two cross terms hi.lo + lo.hi of every K step
with one BF16 MMA instead of two TF32 MMAs (option tc_cross_bf16, default 1).  The BF16 rounding of the
cross terms adds a K-independent ~5.6e-7 (relative, Frobenius) -- below the error of the reference's own
sequential fp32 sum (support/vmath.cu:2961-2977) from K = 2048 on -- so both schemes must pass the
acceptance rule, for all three reference layouts, on normal values and on values whose low mantissa bits
are all set.  The CTA-pair kernel (option tc_pair) computes 256 x 256 tiles with cta_group::2 MMAs and
must give results of the same accuracy.
"""
import numpy as np
import pytest

from helpers import check_gemm_error, rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

NT, NN, TN = 0, 1, 2
TC = 1


def _set(pkg, **opts):
    lib = pkg.load()
    old = {k: lib.kai_get_option(k.encode()) for k in opts}
    for k, v in opts.items():
        pkg.capi.call("kai_set_option", k.encode(), v)
    return old


def _restore(pkg, old):
    for k, v in old.items():
        pkg.capi.call("kai_set_option", k.encode(), v)


def _inputs(dist, M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32)
    b = rng.standard_normal((N, K), dtype=np.float32)
    if dist == "full_mantissa":
        a = (a.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
        b = (b.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    return a, b


@pytest.mark.parametrize("dist", ["normal", "full_mantissa"])
@pytest.mark.parametrize("K", [2048, 4096])
def test_both_schemes_pass_the_rule_in_all_layouts(torch_cuda, pkg, vm, port, K, dist):
    torch = torch_cuda
    M, N = 640, 896
    a, b = _inputs(dist, M, N, K, 5 + K)
    truth = a.astype(np.float64) @ b.astype(np.float64).T
    err_ref = rel_fro(port.matmul(b, np.ascontiguousarray(a[:16])), truth[:16])
    da, db = to_dev(torch, a), to_dev(torch, b)
    dat, dbt = da.T.contiguous(), db.T.contiguous()
    outs = {}
    old = _set(pkg, tc_cross_bf16=1)
    try:
        for cross in (0, 1):
            pkg.capi.call("kai_set_option", b"tc_cross_bf16", cross)
            for layout, (pa, pb) in ((NT, (da, db)), (NN, (da, dbt)), (TN, (dat, dbt))):
                c = torch.full((M, N), float("nan"), device="cuda")
                vm.sgemm(0, layout, c, pa, pb, M, N, K, path=TC)
                torch.cuda.synchronize()
                outs[(cross, layout)] = to_host(c)
    finally:
        _restore(pkg, old)
    for (cross, layout), got in outs.items():
        err = rel_fro(got, truth)
        print(f"K={K} {dist} cross={cross} layout={layout}: {err:.3e} (reference slab {err_ref:.3e})")
        check_gemm_error(err, err_ref, K, f"cross={cross} layout={layout} {dist}")
    for layout in (NT, NN, TN):
        # the schemes differ by the bf16 rounding of the cross terms only
        assert rel_fro(outs[(1, layout)], outs[(0, layout)].astype(np.float64)) <= 1.5e-6
        assert not np.array_equal(outs[(1, layout)], outs[(0, layout)])      # the option does select another scheme


def test_short_or_odd_reductions_keep_three_tf32_products(torch_cuda, pkg, vm):
    """Below 2048, or with K % 8 != 0, the option changes nothing: bit-identical results."""
    torch = torch_cuda
    for (M, N, K) in [(256, 512, 1024), (256, 384, 2052)]:
        a, b = _inputs("normal", M, N, K, 11)
        da, db = to_dev(torch, a), to_dev(torch, b)
        got = []
        old = _set(pkg, tc_cross_bf16=1)
        try:
            for cross in (0, 1):
                pkg.capi.call("kai_set_option", b"tc_cross_bf16", cross)
                c = torch.empty((M, N), device="cuda")
                vm.sgemm(0, NT, c, da, db, M, N, K, path=TC)
                torch.cuda.synchronize()
                got.append(to_host(c))
        finally:
            _restore(pkg, old)
        assert np.array_equal(got[0], got[1]), (M, N, K)


@pytest.mark.parametrize("shape", [(2560, 2048, 2048), (2432, 2100, 520), (4096, 2304, 1024)])
@pytest.mark.parametrize("cross", [0, 1])
def test_cta_pair_kernel_matches_fp64_and_the_single_cta_kernel(torch_cuda, pkg, vm, port, shape, cross):
    """tc_pair = 1: 256 x 256 tiles on pairs of CTAs (cta_group::2), with the fused epilogue, a row tail
    (M not a multiple of 256) and a column tail."""
    torch = torch_cuda
    M, N, K = shape
    a, b = _inputs("normal", M, N, K, 3)
    bias = np.random.default_rng(4).standard_normal(N).astype(np.float32)
    truth = np.maximum(a.astype(np.float64) @ b.astype(np.float64).T + bias, 0.0)
    err_ref = rel_fro(np.maximum(port.matmul(b, np.ascontiguousarray(a[:16])) + bias, 0.0), truth[:16])
    da, db, dbias = to_dev(torch, a), to_dev(torch, b), to_dev(torch, bias)
    lib = pkg.load()
    got = {}
    old = _set(pkg, tc_pair=0, tc_cross_bf16=cross)
    try:
        for pair in (0, 1):
            pkg.capi.call("kai_set_option", b"tc_pair", pair)
            n0, p0 = lib.kai_tc_launch_count(), lib.kai_tc_pair_launch_count()
            c = torch.full((M, N + 8), float("nan"), device="cuda")
            vm.sgemm(0, NT, c, da, db, M, N, K, ldc=N + 8, bias=dbias, act="relu", path=TC)
            torch.cuda.synchronize()
            assert lib.kai_tc_launch_count() == n0 + 1
            assert lib.kai_tc_pair_launch_count() == p0 + pair        # the pair kernel took the call, or did not
            out = to_host(c)
            assert np.isnan(out[:, N:]).all()          # the padding columns of the pitched output stay untouched
            got[pair] = out[:, :N]
    finally:
        _restore(pkg, old)
    for pair in (0, 1):
        err = rel_fro(got[pair], truth)
        print(f"{shape} cross={cross} pair={pair}: {err:.3e} (reference slab {err_ref:.3e})")
        check_gemm_error(err, err_ref, K, f"pair={pair} {shape}")
    # same products, same promotion interval; only the K-block width differs (32 vs 16 per stage)
    assert rel_fro(got[1], got[0].astype(np.float64)) <= 3e-7


def test_prepared_operands_are_written_for_one_side(torch_cuda, pkg, vm):
    """A handle with a reduction of 2048 or more carries the bf16 cross-term plane of a right operand unless
    KAI_PREP_LEFT is given; the other side is refused; KAI_PREP_TF32_LO handles work on either side."""
    torch = torch_cuda
    M, N, K = 384, 512, 2048
    a, b = _inputs("normal", M, N, K, 21)
    truth = a.astype(np.float64) @ b.astype(np.float64).T
    da, db = to_dev(torch, a), to_dev(torch, b)
    c = torch.empty((M, N), device="cuda")
    right = vm.PreparedOperand(0, db, N, K)
    left = vm.PreparedOperand(0, da, M, K, left=True)
    plain_a = vm.PreparedOperand(0, da, M, K, tf32_lo=True)
    plain_b = vm.PreparedOperand(0, db, N, K, tf32_lo=True)
    try:
        vm.sgemm_prepared(0, c, left, 0, M, right, 0, N)
        torch.cuda.synchronize()
        e_mixed = rel_fro(to_host(c), truth)
        vm.sgemm_prepared(0, c, plain_a, 0, M, plain_b, 0, N)
        torch.cuda.synchronize()
        e_pure = rel_fro(to_host(c), truth)
        vm.linear_forward_prepared(0, c, right, da, None, M)
        torch.cuda.synchronize()
        e_fwd = rel_fro(to_host(c), truth)
        print(f"prepared: mixed {e_mixed:.3e} pure {e_pure:.3e} forward {e_fwd:.3e}")
        assert e_mixed < 1.2e-6 and e_pure < 1.0e-6 and e_fwd < 1.2e-6
        with pytest.raises(pkg.KaiError):
            vm.sgemm_prepared(0, c, right, 0, N, right, 0, N)       # a right-side handle as the left operand
        with pytest.raises(pkg.KaiError):
            vm.sgemm_prepared(0, c, left, 0, M, left, 0, M)         # a left-side handle as the right operand
        with pytest.raises(pkg.KaiError):
            vm.linear_forward_prepared(0, c, left, da, None, M)
        with pytest.raises(pkg.KaiError):
            vm.sgemm_prepared(0, c, left, 0, M, plain_b, 0, N)      # cross-term plane against TF32 lo values
    finally:
        for h in (right, left, plain_a, plain_b):
            h.release()


def test_cta_pair_kernel_in_a_recorded_call_list(torch_cuda, pkg, vm):
    """The cluster launch of the pair kernel is captured and replayed like any other call: the replay
    gives the bits of the direct call, twice."""
    torch = torch_cuda
    M, N, K = 2560, 2048, 2048
    a, b = _inputs("normal", M, N, K, 31)
    da, db = to_dev(torch, a), to_dev(torch, b)
    lib = pkg.load()
    old = _set(pkg, tc_pair=1)
    try:
        direct = torch.empty((M, N), device="cuda")
        p0 = lib.kai_tc_pair_launch_count()
        vm.sgemm(0, NT, direct, da, db, M, N, K, path=TC)      # also sizes the workspace before the capture
        torch.cuda.synchronize()
        assert lib.kai_tc_pair_launch_count() == p0 + 1
        out = torch.full((M, N), float("nan"), device="cuda")
        with vm.Replay(0) as rp:
            vm.sgemm(0, NT, out, da, db, M, N, K, path=TC, stream=rp.stream)
        try:
            for _ in range(2):
                out.fill_(float("nan"))
                rp.launch()
                torch.cuda.synchronize()
                assert torch.equal(out, direct)
        finally:
            rp.close()
    finally:
        _restore(pkg, old)
