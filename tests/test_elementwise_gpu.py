"""GPU parity of the bias / activation / loss kernels against the CPU oracle."""
import numpy as np
import pytest

from helpers import to_dev, to_host

pytestmark = pytest.mark.gpu

ACTS = {"none": 0, "relu": 1, "leaky": 2, "sigmoid": 3, "tanh": 4, "gelu": 5, "selu": 6, "mish": 7, "swish": 8}
# The device's expf/erff/logf differ from glibc's by a few ulp; mish chains four of them.
TOL = dict(rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("shape", [(1, 1), (7, 13), (128, 512), (130, 10), (33, 1000)])
def test_add_bias_and_inplace(torch_cuda, vm, port, shape):
    torch = torch_cuda
    rng = np.random.default_rng(0)
    a = rng.standard_normal(shape, dtype=np.float32)
    b = rng.standard_normal(shape[1], dtype=np.float32)
    da, db = to_dev(torch, a), to_dev(torch, b)
    y = torch.empty_like(da)
    vm.add_bias(0, y, da, db, *shape)
    vm.add_bias(0, da, da, db, *shape)  # in place, as the attention layer calls it
    torch.cuda.synchronize()
    want = port.add_bias(a, b)
    np.testing.assert_array_equal(to_host(y), want)
    np.testing.assert_array_equal(to_host(da), want)


@pytest.mark.parametrize("shape", [(1, 1), (5, 3), (128, 512), (128, 10), (8192, 96), (1000, 33), (70, 4096)])
@pytest.mark.parametrize("acc", [False, True])
def test_add_bias_backward_b(torch_cuda, vm, port, shape, acc):
    torch = torch_cuda
    rng = np.random.default_rng(1)
    gy = rng.standard_normal(shape, dtype=np.float32)
    old = rng.standard_normal(shape[1], dtype=np.float32)
    gb = to_dev(torch, old)
    vm.add_bias_backward_b(0, gb, to_dev(torch, gy), shape[0], shape[1], acc)
    torch.cuda.synchronize()
    want = port.add_bias_backward_b(gy, old if acc else None)
    truth = gy.astype(np.float64).sum(axis=0) + (old if acc else 0)
    scale = np.abs(gy).astype(np.float64).sum(axis=0) + 1
    # both are fp32 summations of the same numbers in different orders: compare each with fp64
    assert np.max(np.abs(to_host(gb) - truth) / scale) <= max(2e-7, 2 * np.max(np.abs(want - truth) / scale))


@pytest.mark.parametrize("name", list(ACTS))
def test_activate_forward_backward(torch_cuda, vm, port, name):
    torch = torch_cuda
    act = ACTS[name]
    rng = np.random.default_rng(act)
    x = (rng.standard_normal((37, 129)) * 3).astype(np.float32)
    x[0, :6] = [0.0, -0.0, 1e-30, -1e-30, 30.0, -30.0]
    gy = rng.standard_normal(x.shape, dtype=np.float32)
    alpha = to_dev(torch, np.array([0.1], np.float32))
    dx, dgy = to_dev(torch, x), to_dev(torch, gy)
    y, gx, gxy = torch.empty_like(dx), torch.empty_like(dx), torch.empty_like(dx)
    vm.activate(0, y, dx, *x.shape, act, alpha)
    vm.activate_backward(0, gx, dgy, dx, *x.shape, act, alpha)
    torch.cuda.synchronize()
    np.testing.assert_allclose(to_host(y), port.activate(x, act, 0.1), **TOL)
    np.testing.assert_allclose(to_host(gx), port.activate_backward(gy, x, act, 0.1), **TOL)
    if act <= 4:
        vm.activate_backward_with_y(0, gxy, dgy, y, *x.shape, act, alpha)
        torch.cuda.synchronize()
        np.testing.assert_allclose(to_host(gxy), port.activate_backward_with_y(gy, to_host(y), act, 0.1), **TOL)
    # in place (the RNN path does activate(pr, pr, ...))
    vm.activate(0, dx, dx, *x.shape, act, alpha)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(to_host(dx), to_host(y))


def test_leaky_alpha_null_reads_zero(torch_cuda, vm, port):
    torch = torch_cuda
    x = np.array([[-2.0, 3.0]], np.float32)
    y = torch.empty((1, 2), device="cuda")
    vm.activate(0, y, to_dev(torch, x), 1, 2, 2, None)
    torch.cuda.synchronize()
    assert to_host(y).tolist() == [[-0.0, 3.0]] or to_host(y).tolist() == [[0.0, 3.0]]


@pytest.mark.parametrize("shape", [(1, 1), (9, 10), (64, 1000), (5, 33)])
def test_softmax_activation(torch_cuda, vm, port, shape):
    torch = torch_cuda
    x = (np.random.default_rng(2).standard_normal(shape) * 4).astype(np.float32)
    dx = to_dev(torch, x)
    y = torch.empty_like(dx)
    vm.activate(0, y, dx, *shape, 9)
    vm.activate(0, dx, dx, *shape, 9)
    torch.cuda.synchronize()
    np.testing.assert_allclose(to_host(y), port.activate(x, 9), rtol=2e-5, atol=1e-7)
    np.testing.assert_array_equal(to_host(dx), to_host(y))


def test_unknown_activation_is_rejected(torch_cuda, pkg, vm):
    torch = torch_cuda
    t = torch.zeros((2, 2), device="cuda")
    with pytest.raises(pkg.KaiError):
        vm.activate(0, t, t, 2, 2, 17)
    with pytest.raises(pkg.KaiError):
        vm.activate_backward(0, t, t, t, 2, 2, 9)       # no softmax case in the reference either
    with pytest.raises(pkg.KaiError):
        vm.activate_backward_with_y(0, t, t, t, 2, 2, 5)


@pytest.mark.parametrize("shape", [(1, 2), (128, 10), (300, 1000), (7, 33)])
def test_crossentropy_and_sum(torch_cuda, vm, port, shape):
    torch = torch_cuda
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    lab = rng.integers(0, shape[1], shape[0]).astype(np.int32)
    dx, dl = to_dev(torch, x), to_dev(torch, lab)
    ce = torch.empty(shape[0], device="cuda")
    loss = torch.empty(1, device="cuda")
    gce = torch.empty(shape[0], device="cuda")
    gx = torch.empty_like(dx)
    vm.softmax_idx_crossentropy(0, ce, dx, dl, *shape)
    vm.sum(0, loss, ce, shape[0])
    vm.sum_backward(0, gce, None, shape[0])
    vm.softmax_idx_crossentropy_backward_x(0, gx, gce, dx, dl, *shape)
    torch.cuda.synchronize()
    want_ce = port.softmax_idx_crossentropy(x, lab)
    np.testing.assert_allclose(to_host(ce), want_ce, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(to_host(loss), port.sum(want_ce), rtol=1e-5)
    np.testing.assert_array_equal(to_host(gce), np.ones(shape[0], np.float32))
    np.testing.assert_allclose(to_host(gx), port.softmax_idx_crossentropy_backward_x(port.sum_backward(shape[0]), x, lab),
                               rtol=2e-5, atol=2e-7)
    two = to_dev(torch, np.array([2.5], np.float32))
    vm.sum_backward(0, gce, two, shape[0])
    torch.cuda.synchronize()
    assert (to_host(gce) == 2.5).all()


def test_crossentropy_label_out_of_range(torch_cuda, pkg, vm):
    torch = torch_cuda
    x = torch.zeros((2, 3), device="cuda")
    lab = to_dev(torch, np.array([0, 3], np.int32))
    ce = torch.zeros(2, device="cuda")
    with pytest.raises(pkg.KaiError) as e:
        vm.softmax_idx_crossentropy(0, ce, x, lab, 2, 3)
    assert e.value.code == pkg.capi.E_OUT_OF_RANGE
