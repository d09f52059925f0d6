"""Config 2 end to end: the 2-layer MLP training step replayed op by op in the reference's call
order (matmul, add_bias, activate, ..., softmax cross-entropy, sum, and the backward list), on the
GPU through the C ABI and on the CPU oracle, from the same seeded inputs."""
import importlib

import numpy as np
import pytest

from helpers import rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu


def oracle_step(orc, d):
    h0 = orc.matmul(d["w1"], d["x"])
    h1 = orc.add_bias(h0, d["b1"])
    h2 = orc.activate(h1, 1, 0.1)
    l0 = orc.matmul(d["w2"], h2)
    l1 = orc.add_bias(l0, d["b2"])
    ce = orc.softmax_idx_crossentropy(l1, d["labels"])
    loss = orc.sum(ce)
    gce = orc.sum_backward(ce.size)
    gl = orc.softmax_idx_crossentropy_backward_x(gce, l1, d["labels"])
    gb2 = orc.add_bias_backward_b(gl)
    gh2 = orc.matmul_backward_x(gl, d["w2"])
    gw2 = orc.matmul_backward_w(gl, h2, *d["w2"].shape)
    gh1 = orc.activate_backward(gh2, h1, 1, 0.1)
    gb1 = orc.add_bias_backward_b(gh1)
    gw1 = orc.matmul_backward_w(gh1, d["x"], *d["w1"].shape)
    return dict(loss=loss, l1=l1, gw1=gw1, gb1=gb1, gw2=gw2, gb2=gb2, h2=h2)


def gpu_step(torch, vm, d, fused):
    B, D = d["x"].shape
    H, C = d["w1"].shape[0], d["w2"].shape[0]
    t = {k: to_dev(torch, v) for k, v in d.items()}
    alpha = to_dev(torch, np.array([0.1], np.float32))
    z = lambda *s: torch.empty(s, device="cuda")  # noqa: E731
    h1, h2, l1 = z(B, H), z(B, H), z(B, C)
    if fused:  # `dense` as one launch; pre-activation recomputed for the backward mask below
        vm.linear_forward(0, h1, t["w1"], t["x"], t["b1"], H, B, D)
        vm.linear_forward(0, h2, t["w1"], t["x"], t["b1"], H, B, D, act="relu", leaky_alpha=alpha)
        vm.linear_forward(0, l1, t["w2"], h2, t["b2"], C, B, H)
    else:
        h0, l0 = z(B, H), z(B, C)
        vm.matmul(0, h0, t["w1"], t["x"], H, B, D, False)
        vm.add_bias(0, h1, h0, t["b1"], B, H)
        vm.activate(0, h2, h1, B, H, 1, alpha)
        vm.matmul(0, l0, t["w2"], h2, C, B, H, False)
        vm.add_bias(0, l1, l0, t["b2"], B, C)
    ce, loss, gce, gl = z(B), z(1), z(B), z(B, C)
    vm.softmax_idx_crossentropy(0, ce, l1, t["labels"], B, C)
    vm.sum(0, loss, ce, B)
    vm.sum_backward(0, gce, None, B)
    vm.softmax_idx_crossentropy_backward_x(0, gl, gce, l1, t["labels"], B, C)
    gb2, gh2, gw2, gh1, gb1, gw1 = z(C), z(B, H), z(C, H), z(B, H), z(H), z(H, D)
    vm.add_bias_backward_b(0, gb2, gl, B, C, False)
    vm.matmul_backward_x(0, gh2, gl, t["w2"], C, B, H, False)
    vm.matmul_backward_w(0, gw2, gl, h2, C, B, H, False)
    vm.activate_backward(0, gh1, gh2, h1, B, H, 1, alpha)
    vm.add_bias_backward_b(0, gb1, gh1, B, H, False)
    vm.matmul_backward_w(0, gw1, gh1, t["x"], H, B, D, False)
    torch.cuda.synchronize()
    return {k: to_host(v) for k, v in dict(loss=loss, l1=l1, gw1=gw1, gb1=gb1, gw2=gw2, gb2=gb2, h2=h2).items()}


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("seed", [0, 1])
def test_mlp_training_step(torch_cuda, vm, port, fused, seed):
    wl = importlib.import_module("deep-learning-framework_b200.workloads")
    d = wl.mlp(seed=seed)
    d["b1"] = np.random.default_rng(seed).standard_normal(512).astype(np.float32) * 0.1  # exercise the bias path
    want = oracle_step(port, d)
    got = gpu_step(torch_cuda, vm, d, fused)
    for name in ("l1", "h2", "gw1", "gb1", "gw2", "gb2"):
        err = rel_fro(got[name], want[name])
        assert err < 5e-6, f"{name}: {err:.3e}"
    np.testing.assert_allclose(got["loss"], want["loss"], rtol=2e-6)
