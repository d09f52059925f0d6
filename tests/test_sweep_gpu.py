"""Seeded random shape sweeps through the automatic dispatch, against fp64 results computed by torch: GEMM in
all three layouts with and without accumulation, the attention steps (separate and fused, with and without the
causal mask) and the convolution trio.  Complements the fixed-shape oracle tests with odd sizes."""
import random

import pytest

pytestmark = pytest.mark.gpu


def _rel(got, want):
    return float((got.double() - want).norm() / (want.norm() + 1e-30))


def test_gemm_shape_sweep(torch_cuda, vm):
    torch = torch_cuda
    rnd = random.Random(11)
    g = torch.Generator(device="cuda").manual_seed(11)
    ms = [1, 2, 3, 5, 8, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 200, 255, 256, 300, 511, 513, 700, 1000, 1500, 2049]
    ns = [1, 2, 7, 10, 16, 31, 32, 33, 64, 65, 100, 128, 129, 255, 257, 384, 500, 512, 1000, 1025, 2048]
    ks = [1, 2, 3, 4, 7, 8, 15, 16, 17, 32, 33, 63, 64, 100, 128, 129, 255, 256, 257, 500, 512, 784, 1000, 1024, 2048, 4100]
    for _ in range(120):
        layout, M, N, K, acc = rnd.choice([0, 1, 2]), rnd.choice(ms), rnd.choice(ns), rnd.choice(ks), rnd.random() < 0.3
        a = torch.randn((M, K) if layout != 2 else (K, M), device="cuda", generator=g)
        b = torch.randn((N, K) if layout == 0 else (K, N), device="cuda", generator=g)
        c0 = torch.randn((M, N), device="cuda", generator=g)
        c = c0.clone()
        vm.sgemm(0, layout, c, a, b, M, N, K, accumulate=acc)
        A = a.double() if layout != 2 else a.double().t()
        B = b.double().t() if layout == 0 else b.double()
        want = A @ B + (c0.double() if acc else 0)
        assert bool(torch.isfinite(c).all())
        assert _rel(c, want) < 3e-6 * max(1, K) ** 0.5, (layout, M, N, K, acc)


def test_attention_shape_sweep(torch_cuda, vm):
    torch = torch_cuda
    rnd = random.Random(12)
    g = torch.Generator(device="cuda").manual_seed(12)
    for _ in range(16):
        nb, T = rnd.choice([1, 2, 3]), rnd.choice([64, 65, 100, 128, 130, 200, 256, 300, 512])
        H, P, causal = rnd.choice([1, 2, 3, 4, 8, 12]), rnd.choice([64, 64, 64, 16, 32, 8, 128]), rnd.random() < 0.4
        q, k, v = (torch.randn((nb, T, H * P), device="cuda", generator=g) for _ in range(3))
        coef = torch.tensor([P ** -0.5], device="cuda")
        out = torch.empty((nb, T, H, P), device="cuda")
        fused = torch.empty_like(out)
        pp = torch.empty((nb, T, T, H), device="cuda")
        vm.mult_on_heads(0, pp, k, q, nb, T, H * P, H, P, coef)
        if causal:
            vm.set_mh_attention_mask(0, pp, nb, T, H, True)
        vm.softmax_direct_on_axis(0, pp, nb * T, T, H)
        vm.mix_values(0, out, pp, v, nb, T, H * P, H, P)
        vm.mh_attention_forward(0, fused, k, q, v, nb, T, H * P, H, P, coef, causal)
        q4, k4, v4 = (t.double().reshape(nb, T, H, P) for t in (q, k, v))
        s = torch.einsum("bqhp,bkhp->bqkh", q4, k4) * float(coef)
        if causal:
            ar = torch.arange(T, device="cuda")
            s = s.masked_fill(ar[None, :, None, None] < ar[None, None, :, None], float("-inf"))
        ref = torch.einsum("bqkh,bkhp->bqhp", torch.softmax(s, dim=2), v4)
        assert _rel(out, ref) < 3e-6 and _rel(fused, ref) < 3e-6, (nb, T, H, P, causal)


def test_convolution_shape_sweep(torch_cuda, vm):
    torch = torch_cuda
    F = torch.nn.functional
    rnd = random.Random(13)
    g = torch.Generator(device="cuda").manual_seed(13)
    for _ in range(16):
        nd, cx, cy = rnd.choice([1, 2, 3]), rnd.choice([1, 3, 4, 8, 16, 33]), rnd.choice([1, 2, 8, 16, 40])
        h, w, kh, kw = rnd.choice([5, 8, 14, 17, 28]), rnd.choice([5, 8, 13, 28]), rnd.choice([1, 3, 5]), rnd.choice([1, 3, 5])
        ph, pw = kh // 2, kw // 2
        x = torch.randn((nd, cx, h, w), device="cuda", generator=g)
        kk = torch.randn((cy, cx, kh, kw), device="cuda", generator=g)
        gy = torch.randn((nd, cy, h, w), device="cuda", generator=g)
        y, gx, gk = torch.empty_like(gy), torch.empty_like(x), torch.empty_like(kk)
        vm.conv2d(0, y, x, kk, nd, cy, h, w, cx, h, w, kh, kw, 1, ph, pw)
        vm.conv2d_backward_x(0, gx, gy, kk, nd, cx, h, w, cy, h, w, kh, kw, 1, ph, pw)
        vm.conv2d_backward_k(0, gk, gy, x, nd, cx, h, w, cy, h, w, kh, kw, 1, ph, pw)
        xd, kd = x.double().requires_grad_(), kk.double().requires_grad_()
        yd = F.conv2d(xd, kd, padding=(ph, pw))
        yd.backward(gy.double())
        for name, got, want in (("y", y, yd.detach()), ("gx", gx, xd.grad), ("gk", gk, kd.grad)):
            assert _rel(got, want) < 3e-6, (name, nd, cx, cy, h, w, kh, kw)
