"""Recorded call lists (kai_replay_*): the config-2 MLP step and the config-1 GEMM recorded once and
replayed as one launch must reproduce the call-by-call results bit for bit."""
import importlib

import numpy as np
import pytest

from helpers import to_dev, to_host

pytestmark = pytest.mark.gpu


def test_recording_refuses_to_grow_scratch(torch_cuda, vm, pkg):
    """Scratch memory may not move while a list is being recorded: the call fails with KAI_E_ALLOC, the
    library stays usable, and after one un-recorded pass the same list records and replays.
    (Runs before any other recording in this file: kai_mem_trim keeps scratch a recording points into.)"""
    torch = torch_cuda
    lib = pkg.capi.load()
    n = 1024
    a = torch.randn((n, n), device="cuda")
    c = torch.empty((n, n), device="cuda")
    torch.cuda.synchronize()
    assert lib.kai_mem_trim(0) == 0              # also drops the scratch workspace
    rp = vm.Replay(0)
    rp.__enter__()
    try:
        with pytest.raises(pkg.capi.KaiError) as ei:
            vm.matmul(0, c, a, a, n, n, n, False, stream=rp.stream)
        assert ei.value.code == pkg.capi.E_ALLOC
    finally:
        rp.close()
    vm.matmul(0, c, a, a, n, n, n, False)
    torch.cuda.synchronize()
    want = to_host(c).copy()
    with vm.Replay(0) as rp2:
        vm.matmul(0, c, a, a, n, n, n, False, stream=rp2.stream)
    c.zero_()
    rp2.launch()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(to_host(c), want)
    rp2.close()


def _mlp_buffers(torch, d):
    B, D = d["x"].shape
    H, C = d["w1"].shape[0], d["w2"].shape[0]
    t = {k: to_dev(torch, v) for k, v in d.items()}
    t["alpha"] = to_dev(torch, np.array([0.1], np.float32))
    shapes = dict(h0=(B, H), h1=(B, H), h2=(B, H), l0=(B, C), l1=(B, C), ce=(B,), loss=(1,), gce=(B,), gl=(B, C),
                  gb2=(C,), gh2=(B, H), gw2=(C, H), gh1=(B, H), gb1=(H,), gw1=(H, D))
    for k, s in shapes.items():
        t[k] = torch.zeros(s, device="cuda")
    return t, (B, D, H, C)


def _mlp_calls(vm, t, dims, stream):
    """The reference's 15 math calls of one training step of the 2-layer MLP."""
    B, D, H, C = dims
    vm.matmul(0, t["h0"], t["w1"], t["x"], H, B, D, False, stream=stream)
    vm.add_bias(0, t["h1"], t["h0"], t["b1"], B, H, stream=stream)
    vm.activate(0, t["h2"], t["h1"], B, H, 1, t["alpha"], stream=stream)
    vm.matmul(0, t["l0"], t["w2"], t["h2"], C, B, H, False, stream=stream)
    vm.add_bias(0, t["l1"], t["l0"], t["b2"], B, C, stream=stream)
    vm.softmax_idx_crossentropy(0, t["ce"], t["l1"], t["labels"], B, C, stream=stream)
    vm.sum(0, t["loss"], t["ce"], B, stream=stream)
    vm.sum_backward(0, t["gce"], None, B, stream=stream)
    vm.softmax_idx_crossentropy_backward_x(0, t["gl"], t["gce"], t["l1"], t["labels"], B, C, stream=stream)
    vm.add_bias_backward_b(0, t["gb2"], t["gl"], B, C, False, stream=stream)
    vm.matmul_backward_x(0, t["gh2"], t["gl"], t["w2"], C, B, H, False, stream=stream)
    vm.matmul_backward_w(0, t["gw2"], t["gl"], t["h2"], C, B, H, False, stream=stream)
    vm.activate_backward(0, t["gh1"], t["gh2"], t["h1"], B, H, 1, t["alpha"], stream=stream)
    vm.add_bias_backward_b(0, t["gb1"], t["gh1"], B, H, False, stream=stream)
    vm.matmul_backward_w(0, t["gw1"], t["gh1"], t["x"], H, B, D, False, stream=stream)


OUTS = ("loss", "l1", "h2", "gw1", "gb1", "gw2", "gb2")


def test_mlp_step_replayed_matches_call_by_call(torch_cuda, vm, pkg):
    torch = torch_cuda
    wl = importlib.import_module("deep-learning-framework_b200.workloads")
    d = wl.mlp(seed=3)
    t, dims = _mlp_buffers(torch, d)
    _mlp_calls(vm, t, dims, None)            # first pass, call by call (also sizes the scratch memory)
    torch.cuda.synchronize()
    want = {k: to_host(t[k]).copy() for k in OUTS}
    before = pkg.capi.load().kai_launch_count()
    with vm.Replay(0) as rp:
        _mlp_calls(vm, t, dims, rp.stream)
    recorded = pkg.capi.load().kai_launch_count() - before
    assert recorded >= 15
    for rounds in range(2):
        for k in OUTS:
            t[k].fill_(float("nan"))
        torch.cuda.synchronize()
        rp.launch()
        torch.cuda.synchronize()
        for k in OUTS:
            np.testing.assert_array_equal(to_host(t[k]), want[k], err_msg=f"{k} (replay {rounds})")
    # new inputs behind the same pointers: the replay computes on the current contents
    d2 = wl.mlp(seed=4)
    t["x"].copy_(to_dev(torch, d2["x"]))
    _mlp_calls(vm, t, dims, None)
    torch.cuda.synchronize()
    want2 = {k: to_host(t[k]).copy() for k in OUTS}
    for k in OUTS:
        t[k].fill_(float("nan"))
    rp.launch()
    torch.cuda.synchronize()
    for k in OUTS:
        np.testing.assert_array_equal(to_host(t[k]), want2[k])
    assert pkg.capi.load().kai_device_status(0, None) == 0
    rp.close()


def test_tensor_core_gemm_and_attention_replayed(torch_cuda, vm):
    torch = torch_cuda
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.rand((512, 512), device="cuda", generator=g) * 2 - 1
    b = torch.rand((512, 512), device="cuda", generator=g) * 2 - 1
    c = torch.empty((512, 512), device="cuda")
    nb, T, H, P = 2, 128, 4, 64
    q, k, v = (torch.randn((nb, T, H * P), device="cuda", generator=g) for _ in range(3))
    pp = torch.empty((nb, T, T, H), device="cuda")
    out = torch.empty((nb, T, H, P), device="cuda")
    coef = torch.tensor([0.125], device="cuda")

    def calls(stream):
        vm.matmul_backward_x(0, c, a, b, 512, 512, 512, False, stream=stream)   # config 1: C = A . B
        vm.mult_on_heads(0, pp, k, q, nb, T, H * P, H, P, coef, stream=stream)
        vm.softmax_direct_on_axis(0, pp, nb * T, T, H, stream=stream)
        vm.mix_values(0, out, pp, v, nb, T, H * P, H, P, stream=stream)

    calls(None)
    torch.cuda.synchronize()
    want = [to_host(x).copy() for x in (c, pp, out)]
    with vm.Replay(0) as rp:
        calls(rp.stream)
    for x in (c, pp, out):
        x.fill_(float("nan"))
    rp.launch()
    torch.cuda.synchronize()
    for got, w in zip((c, pp, out), want):
        np.testing.assert_array_equal(to_host(got), w)
    rp.close()


def test_convolution_and_attention_training_calls_replayed(torch_cuda, vm):
    """The convolution trio (workspace shared between the unfolded matrix and the GEMM planes), the fused
    attention forward and the attention gradients recorded once and replayed: same bits as call by call."""
    torch = torch_cuda
    g = torch.Generator(device="cuda").manual_seed(2)
    nd, cx, cy, hh, ww = 2, 16, 24, 12, 12
    x = torch.randn((nd, cx, hh, ww), device="cuda", generator=g)
    kk = torch.randn((cy, cx, 3, 3), device="cuda", generator=g) * 0.1
    gy = torch.randn((nd, cy, hh, ww), device="cuda", generator=g)
    y, gx, gk = torch.empty_like(gy), torch.empty_like(x), torch.empty_like(kk)
    nb, T, H, P = 2, 128, 4, 64
    q, k, v = (torch.randn((nb, T, H * P), device="cuda", generator=g) for _ in range(3))
    ga = torch.randn((nb, T, H, P), device="cuda", generator=g)
    coef = torch.tensor([0.125], device="cuda")
    fused = torch.empty((nb, T, H, P), device="cuda")
    pp = torch.empty((nb, T, T, H), device="cuda")
    gp = torch.empty_like(pp)
    gq, gv = torch.empty_like(q), torch.empty_like(q)
    outs = (y, gx, gk, fused, gp, gq, gv)

    def calls(s):
        vm.conv2d(0, y, x, kk, nd, cy, hh, ww, cx, hh, ww, 3, 3, 1, 1, 1, stream=s)
        vm.conv2d_backward_x(0, gx, gy, kk, nd, cx, hh, ww, cy, hh, ww, 3, 3, 1, 1, 1, stream=s)
        vm.conv2d_backward_k(0, gk, gy, x, nd, cx, hh, ww, cy, hh, ww, 3, 3, 1, 1, 1, stream=s)
        vm.mh_attention_forward(0, fused, k, q, v, nb, T, H * P, H, P, coef, stream=s)
        vm.mult_on_heads(0, pp, k, q, nb, T, H * P, H, P, coef, stream=s)
        vm.softmax_direct_on_axis(0, pp, nb * T, T, H, stream=s)
        vm.mix_values_backward_prop(0, gp, ga, v, nb, T, H * P, H, P, stream=s)
        vm.mix_values_backward_value(0, gv, ga, pp, nb, T, H * P, H, P, stream=s)
        vm.softmax_direct_on_axis_backward(0, gp, pp, nb, T, H, coef, stream=s)
        vm.mult_on_heads_backward(0, gq, gp, k, nb, T, H * P, H, P, stream=s)

    calls(None)
    torch.cuda.synchronize()
    want = [to_host(t).copy() for t in outs]
    with vm.Replay(0) as rp:
        calls(rp.stream)
    for t in outs:
        t.fill_(float("nan"))
    rp.launch()
    torch.cuda.synchronize()
    for got, w in zip(outs, want):
        np.testing.assert_array_equal(to_host(got), w)
    rp.close()
