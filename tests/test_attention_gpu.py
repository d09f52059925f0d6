"""GPU parity of the attention contractions (mult_on_heads, mask, softmax over the key axis,
mix_values) in the reference's head-interleaved / head-minor layouts."""
import numpy as np
import pytest

from helpers import rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

SHAPES = [  # nbat, ntimes, nhead, npiece
    (1, 1, 1, 1), (2, 7, 3, 4), (2, 64, 8, 64), (1, 130, 8, 16), (3, 50, 5, 12), (2, 96, 16, 8), (1, 33, 2, 6),
    (2, 512, 8, 64), (1, 100, 3, 24), (1, 70, 12, 32), (2, 40, 8, 128), (2, 200, 12, 64), (1, 64, 3, 64),
]


@pytest.fixture(params=[0, 2, 1], ids=["tcgen05", "warp_mma", "cuda_core"], autouse=True)
def attn_path(request, pkg):
    """Every test runs on the tensor-core kernels (when the shape allows) and on the CUDA-core ones."""
    pkg.capi.call("kai_set_option", b"attn_path", request.param)
    yield request.param
    pkg.capi.call("kai_set_option", b"attn_path", 0)


def _qkv(shape, seed=0):
    nbat, ntimes, nhead, npiece = shape
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((nbat, ntimes, nhead * npiece), dtype=np.float32) for _ in range(3)]


@pytest.mark.parametrize("shape", SHAPES)
def test_attention_forward_trio(torch_cuda, vm, port, shape):
    torch = torch_cuda
    nbat, ntimes, nhead, npiece = shape
    nvec = nhead * npiece
    q, k, v = _qkv(shape)
    coef = float(1.0 / np.sqrt(npiece))
    dq, dk, dv = (to_dev(torch, t) for t in (q, k, v))
    dcoef = to_dev(torch, np.array([coef], np.float32))
    pp = torch.full((nbat, ntimes, ntimes, nhead), float("nan"), device="cuda")
    out = torch.full((nbat, ntimes, nhead, npiece), float("nan"), device="cuda")

    vm.mult_on_heads(0, pp, dk, dq, nbat, ntimes, nvec, nhead, npiece, dcoef)
    torch.cuda.synchronize()
    want_pp = port.mult_on_heads(k, q, nhead, coef)
    np.testing.assert_allclose(to_host(pp), want_pp, rtol=1e-5, atol=1e-5)
    truth_pp = np.einsum("bqhp,bkhp->bqkh", q.reshape(nbat, ntimes, nhead, npiece).astype(np.float64),
                         k.reshape(nbat, ntimes, nhead, npiece).astype(np.float64)) * coef
    # the GEMM acceptance rule: no worse than twice the reference loop's own error against fp64
    assert rel_fro(to_host(pp), truth_pp) <= 2 * rel_fro(want_pp, truth_pp) + 6e-8

    vm.softmax_direct_on_axis(0, pp, nbat * ntimes, ntimes, nhead)
    torch.cuda.synchronize()
    want_sm = port.softmax_direct_on_axis(want_pp)
    np.testing.assert_allclose(to_host(pp), want_sm, rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(to_host(pp).sum(axis=2), 1.0, rtol=1e-5)

    vm.mix_values(0, out, pp, dv, nbat, ntimes, nvec, nhead, npiece)
    torch.cuda.synchronize()
    want_out = port.mix_values(want_sm, v, nhead)
    assert rel_fro(to_host(out), want_out) < 1e-5
    truth_out = np.einsum("bqkh,bkhp->bqhp", want_sm.astype(np.float64),
                          v.reshape(nbat, ntimes, nhead, npiece).astype(np.float64))
    got_on_same_probs = torch.empty_like(out)
    vm.mix_values(0, got_on_same_probs, to_dev(torch, want_sm), dv, nbat, ntimes, nvec, nhead, npiece)
    torch.cuda.synchronize()
    assert rel_fro(to_host(got_on_same_probs), truth_out) <= 2 * rel_fro(want_out, truth_out) + 6e-8


@pytest.mark.parametrize("shape", [(2, 7, 3, 4), (1, 64, 8, 8), (2, 33, 5, 4)])
def test_causal_mask_then_softmax(torch_cuda, vm, port, shape):
    torch = torch_cuda
    nbat, ntimes, nhead, npiece = shape
    q, k, _ = _qkv(shape, seed=1)
    pp = port.mult_on_heads(k, q, nhead, 0.5)
    d = to_dev(torch, pp)
    vm.set_mh_attention_mask(0, d, nbat, ntimes, nhead, True)
    torch.cuda.synchronize()
    want = port.set_mh_attention_mask(pp, True)
    np.testing.assert_array_equal(to_host(d), want)
    vm.softmax_direct_on_axis(0, d, nbat * ntimes, ntimes, nhead)
    torch.cuda.synchronize()
    np.testing.assert_allclose(to_host(d), port.softmax_direct_on_axis(want), rtol=1e-4, atol=1e-7)
    d2 = to_dev(torch, pp)
    vm.set_mh_attention_mask(0, d2, nbat, ntimes, nhead, False)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(to_host(d2), port.set_mh_attention_mask(pp, False))


def test_coef_null_reads_zero(torch_cuda, vm):
    torch = torch_cuda
    q = torch.randn((1, 4, 8), device="cuda")
    pp = torch.full((1, 4, 4, 2), 5.0, device="cuda")
    vm.mult_on_heads(0, pp, q, q, 1, 4, 8, 2, 4, None)
    torch.cuda.synchronize()
    assert float(pp.abs().max()) == 0.0


def test_batch_sharding_is_a_pointer_offset(torch_cuda, vm, port):
    """A rank's share of the batch is a contiguous slab of every tensor: running two half-batches
    through offset pointers gives exactly the full-batch result."""
    torch = torch_cuda
    shape = (4, 32, 4, 8)
    nbat, ntimes, nhead, npiece = shape
    nvec = nhead * npiece
    q, k, v = _qkv(shape, seed=2)
    dq, dk, dv = (to_dev(torch, t) for t in (q, k, v))
    coef = to_dev(torch, np.array([0.35], np.float32))

    def run(b0, b1):
        pp = torch.empty((b1 - b0, ntimes, ntimes, nhead), device="cuda")
        out = torch.empty((b1 - b0, ntimes, nhead, npiece), device="cuda")
        vm.mult_on_heads(0, pp, dk[b0:b1], dq[b0:b1], b1 - b0, ntimes, nvec, nhead, npiece, coef)
        vm.softmax_direct_on_axis(0, pp, (b1 - b0) * ntimes, ntimes, nhead)
        vm.mix_values(0, out, pp, dv[b0:b1], b1 - b0, ntimes, nvec, nhead, npiece)
        torch.cuda.synchronize()
        return to_host(out)

    full = run(0, 4)
    np.testing.assert_array_equal(np.concatenate([run(0, 2), run(2, 4)]), full)


@pytest.mark.parametrize("shape", SHAPES)
def test_attention_backward_chain(torch_cuda, vm, port, shape):
    """The engine's backward order (api_objects/vtensor.cpp:3145-3154): value gradient and score
    gradient from gy, softmax backward in place, then one mult_on_heads_backward per operand."""
    torch = torch_cuda
    nbat, ntimes, nhead, npiece = shape
    nvec = nhead * npiece
    q, k, v = _qkv(shape, seed=3)
    coef = float(1.0 / np.sqrt(npiece))
    gy = np.random.default_rng(4).standard_normal((nbat, ntimes, nhead, npiece), dtype=np.float32)
    probs = port.softmax_direct_on_axis(port.mult_on_heads(k, q, nhead, coef))
    dq, dk, dv, dgy, dprobs = (to_dev(torch, t) for t in (q, k, v, gy, probs))
    dcoef = to_dev(torch, np.array([coef], np.float32))
    f64 = np.float64
    q4, k4, v4 = (t.reshape(nbat, ntimes, nhead, npiece).astype(f64) for t in (q, k, v))

    gv = torch.full((nbat, ntimes, nvec), float("nan"), device="cuda")
    vm.mix_values_backward_value(0, gv, dgy, dprobs, nbat, ntimes, nvec, nhead, npiece)
    torch.cuda.synchronize()
    want_gv = port.mix_values_backward_value(gy, probs, nhead)
    truth_gv = np.einsum("bqkh,bqhp->bkhp", probs.astype(f64), gy.astype(f64)).reshape(nbat, ntimes, nvec)
    assert rel_fro(to_host(gv), want_gv) < 1e-5
    assert rel_fro(to_host(gv), truth_gv) <= 2 * rel_fro(want_gv, truth_gv) + 6e-8

    gp = torch.full((nbat, ntimes, ntimes, nhead), float("nan"), device="cuda")
    vm.mix_values_backward_prop(0, gp, dgy, dv, nbat, ntimes, nvec, nhead, npiece)
    torch.cuda.synchronize()
    want_gp = port.mix_values_backward_prop(gy, v, nhead)
    truth_gp = np.einsum("bqhp,bkhp->bqkh", gy.astype(f64), v4)
    np.testing.assert_allclose(to_host(gp), want_gp, rtol=1e-5, atol=2e-5)
    assert rel_fro(to_host(gp), truth_gp) <= 2 * rel_fro(want_gp, truth_gp) + 6e-8

    # softmax backward, in place, on the oracle's gp so that the comparison isolates this op
    gs = to_dev(torch, want_gp)
    vm.softmax_direct_on_axis_backward(0, gs, dprobs, nbat, ntimes, nhead, dcoef)
    torch.cuda.synchronize()
    want_gs = port.softmax_direct_on_axis_backward(want_gp, probs, coef)
    p64, g64 = probs.astype(f64), want_gp.astype(f64)
    truth_gs = coef * p64 * (g64 - (p64 * g64).sum(axis=2, keepdims=True))
    assert rel_fro(to_host(gs), want_gs) < 2e-6
    assert rel_fro(to_host(gs), truth_gs) <= 2 * rel_fro(want_gs, truth_gs) + 1e-7

    # The function contracts the score gradient's LAST time axis with the given operand: that is the
    # gradient of Q when the operand is K.  (The engine passes the same score gradient for its K
    # call too, vtensor.cpp:3153; the function itself is what is checked here.)
    dgs = to_dev(torch, want_gs)
    gq = torch.full((nbat, ntimes, nvec), float("nan"), device="cuda")
    vm.mult_on_heads_backward(0, gq, dgs, dk, nbat, ntimes, nvec, nhead, npiece)
    torch.cuda.synchronize()
    want_gq = port.mult_on_heads_backward(want_gs, k, nhead)
    truth_gq = np.einsum("bqkh,bkhp->bqhp", want_gs.astype(f64), k4).reshape(nbat, ntimes, nvec)
    assert rel_fro(to_host(gq), want_gq) < 1e-5
    assert rel_fro(to_host(gq), truth_gq) <= 2 * rel_fro(want_gq, truth_gq) + 6e-8


def test_attention_backward_matches_autograd_identity(torch_cuda, vm):
    """End to end against an fp64 autograd of softmax(coef * Q K^T) V on one small case."""
    torch = torch_cuda
    nbat, ntimes, nhead, npiece = 2, 24, 4, 8
    nvec = nhead * npiece
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn((nbat, ntimes, nvec), device="cuda", generator=g) for _ in range(3))
    gy = torch.randn((nbat, ntimes, nhead, npiece), device="cuda", generator=g)
    coef = torch.tensor([npiece ** -0.5], device="cuda")
    pp = torch.empty((nbat, ntimes, ntimes, nhead), device="cuda")
    vm.mult_on_heads(0, pp, k, q, nbat, ntimes, nvec, nhead, npiece, coef)
    vm.softmax_direct_on_axis(0, pp, nbat * ntimes, ntimes, nhead)
    gv, gq, gk = (torch.empty_like(q) for _ in range(3))
    gp = torch.empty_like(pp)
    vm.mix_values_backward_value(0, gv, gy, pp, nbat, ntimes, nvec, nhead, npiece)
    vm.mix_values_backward_prop(0, gp, gy, v, nbat, ntimes, nvec, nhead, npiece)
    vm.softmax_direct_on_axis_backward(0, gp, pp, nbat, ntimes, nhead, coef)
    vm.mult_on_heads_backward(0, gq, gp, k, nbat, ntimes, nvec, nhead, npiece)
    gpt = gp.transpose(1, 2).contiguous()
    vm.mult_on_heads_backward(0, gk, gpt, q, nbat, ntimes, nvec, nhead, npiece)
    torch.cuda.synchronize()

    q64, k64, v64 = (t.double().reshape(nbat, ntimes, nhead, npiece).requires_grad_() for t in (q, k, v))
    s = torch.einsum("bqhp,bkhp->bqkh", q64, k64) * float(coef)
    y = torch.einsum("bqkh,bkhp->bqhp", torch.softmax(s, dim=2), v64)
    y.backward(gy.double())
    for got, want in ((gq, q64.grad), (gk, k64.grad), (gv, v64.grad)):
        err = (got.double().reshape(want.shape) - want).norm() / want.norm()
        assert float(err) < 5e-6


FUSED_SHAPES = [  # nbat, ntimes, nhead, npiece, causal
    (2, 64, 2, 64, False), (1, 128, 4, 64, False), (2, 512, 8, 64, False), (1, 200, 3, 64, False),
    (3, 70, 5, 64, False), (1, 130, 8, 64, True), (2, 512, 8, 64, True), (1, 100, 3, 64, True),
    (2, 640, 4, 64, False),
    # shapes outside the fused kernel: served by the separate steps
    (2, 50, 4, 16, False), (1, 33, 2, 6, True), (1, 40, 8, 128, False),
]


@pytest.mark.parametrize("shape", FUSED_SHAPES)
def test_fused_attention_forward(torch_cuda, vm, port, shape):
    """kai_mh_attention_forward against the reference's three steps (mask, when asked, in between)."""
    torch = torch_cuda
    nbat, ntimes, nhead, npiece, causal = shape
    nvec = nhead * npiece
    q, k, v = _qkv(shape[:4], seed=7)
    coef = float(1.0 / np.sqrt(npiece))
    scores = port.mult_on_heads(k, q, nhead, coef)
    if causal:
        scores = port.set_mh_attention_mask(scores, True)
    probs = port.softmax_direct_on_axis(scores)
    want = port.mix_values(probs, v, nhead)
    f64 = np.float64
    q4, k4, v4 = (t.reshape(nbat, ntimes, nhead, npiece).astype(f64) for t in (q, k, v))
    s64 = np.einsum("bqhp,bkhp->bqkh", q4, k4) * coef
    if causal:
        s64 = np.where(np.arange(ntimes)[None, :, None, None] < np.arange(ntimes)[None, None, :, None], -np.inf, s64)
    p64 = np.exp(s64 - s64.max(axis=2, keepdims=True))
    p64 /= p64.sum(axis=2, keepdims=True)
    truth = np.einsum("bqkh,bkhp->bqhp", p64, v4)

    dq, dk, dv = (to_dev(torch, t) for t in (q, k, v))
    dcoef = to_dev(torch, np.array([coef], np.float32))
    out = torch.full((nbat, ntimes, nhead, npiece), float("nan"), device="cuda")
    vm.mh_attention_forward(0, out, dk, dq, dv, nbat, ntimes, nvec, nhead, npiece, dcoef, causal)
    torch.cuda.synchronize()
    got = to_host(out)
    assert np.isfinite(got).all()
    assert rel_fro(got, want) < 5e-6
    assert rel_fro(got, truth) <= 2 * rel_fro(want, truth) + 1e-7


def test_fused_attention_twice_and_batch_split(torch_cuda, vm):
    """Same inputs, same bits on a second call; a batch split through offset pointers changes nothing."""
    torch = torch_cuda
    nbat, ntimes, nhead, npiece = 4, 256, 4, 64
    nvec = nhead * npiece
    g = torch.Generator(device="cuda").manual_seed(11)
    q, k, v = (torch.randn((nbat, ntimes, nvec), device="cuda", generator=g) for _ in range(3))
    coef = torch.tensor([0.125], device="cuda")
    a, b, c = (torch.empty((nbat, ntimes, nhead, npiece), device="cuda") for _ in range(3))
    vm.mh_attention_forward(0, a, k, q, v, nbat, ntimes, nvec, nhead, npiece, coef)
    vm.mh_attention_forward(0, b, k, q, v, nbat, ntimes, nvec, nhead, npiece, coef)
    vm.mh_attention_forward(0, c[:2], k[:2], q[:2], v[:2], 2, ntimes, nvec, nhead, npiece, coef)
    vm.mh_attention_forward(0, c[2:], k[2:], q[2:], v[2:], 2, ntimes, nvec, nhead, npiece, coef)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(a, c)
