"""Pins the CPU oracle: the C port must reproduce, bit for bit, (a) the committed vectors that
tests/golden/make_golden.py generated from the unmodified reference and (b) the compiled reference
itself whenever oracle/_ref is present.  Also records the reference path's own error against fp64,
which the GPU tests use for the "no worse than 2x" rule."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_vectors.npz"


def _load_make_golden():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN.parent / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_port_reproduces_reference_vectors(port):
    mg = _load_make_golden()
    got = mg.compute(port)
    want = np.load(GOLDEN)
    assert set(got) == set(want.files)
    for name in want.files:
        np.testing.assert_array_equal(got[name], want[name], err_msg=name)


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference (oracle/_ref) not built on this machine")
def test_port_matches_compiled_reference_on_random_shapes(port):
    ref = oracle.Oracle("ref")
    rng = np.random.default_rng(1)
    for ndat, xvec, yvec in [(1, 1, 1), (3, 5, 2), (17, 64, 33), (40, 100, 10), (128, 48, 96)]:
        x = rng.standard_normal((ndat, xvec)).astype(np.float32)
        w = rng.standard_normal((yvec, xvec)).astype(np.float32)
        gy = rng.standard_normal((ndat, yvec)).astype(np.float32)
        np.testing.assert_array_equal(port.matmul(w, x), ref.matmul(w, x))
        np.testing.assert_array_equal(port.matmul_backward_x(gy, w), ref.matmul_backward_x(gy, w))
        np.testing.assert_array_equal(port.matmul_backward_w(gy, x, yvec, xvec),
                                      ref.matmul_backward_w(gy, x, yvec, xvec))
        np.testing.assert_array_equal(port.add_bias_backward_b(gy), ref.add_bias_backward_b(gy))
    q, k, v = (rng.standard_normal((3, 20, 32)).astype(np.float32) for _ in range(3))
    pp, pr = port.mult_on_heads(k, q, 4, 0.25), ref.mult_on_heads(k, q, 4, 0.25)
    np.testing.assert_array_equal(pp, pr)
    np.testing.assert_array_equal(port.softmax_direct_on_axis(pp), ref.softmax_direct_on_axis(pr))
    sp = port.softmax_direct_on_axis(pp)
    np.testing.assert_array_equal(port.mix_values(sp, v, 4), ref.mix_values(ref.softmax_direct_on_axis(pr), v, 4))
    gy = rng.standard_normal((3, 20, 4, 8)).astype(np.float32)
    np.testing.assert_array_equal(port.mix_values_backward_value(gy, sp, 4), ref.mix_values_backward_value(gy, sp, 4))
    gp = port.mix_values_backward_prop(gy, v, 4)
    np.testing.assert_array_equal(gp, ref.mix_values_backward_prop(gy, v, 4))
    gs = port.softmax_direct_on_axis_backward(gp, sp, 0.25)
    np.testing.assert_array_equal(gs, ref.softmax_direct_on_axis_backward(gp, sp, 0.25))
    np.testing.assert_array_equal(port.mult_on_heads_backward(gs, k, 4), ref.mult_on_heads_backward(gs, k, 4))


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference (oracle/_ref) not built on this machine")
def test_conv2d_port_matches_compiled_reference(port):
    ref = oracle.Oracle("ref")
    rng = np.random.default_rng(5)
    for (ndat, xchn, ychn, xh, xw, kh, kw, ph, pw, group) in [(2, 3, 4, 6, 5, 3, 3, 1, 1, 1), (1, 4, 2, 5, 7, 5, 3, 2, 1, 1),
                                                              (2, 4, 3, 4, 4, 3, 3, 1, 1, 2), (1, 2, 2, 3, 3, 1, 1, 0, 0, 1)]:
        x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
        k = rng.standard_normal((ychn, xchn // group, kh, kw)).astype(np.float32)
        gy = rng.standard_normal((ndat, ychn, xh, xw)).astype(np.float32)
        np.testing.assert_array_equal(port.conv2d(x, k, xh, xw, ph, pw, group), ref.conv2d(x, k, xh, xw, ph, pw, group))
        np.testing.assert_array_equal(port.conv2d_backward_x(gy, k, xh, xw, ph, pw, group),
                                      ref.conv2d_backward_x(gy, k, xh, xw, ph, pw, group))
    # kernel gradient: the compiled host loop is only comparable where yw == pw (see kai_oracle.c)
    x = rng.standard_normal((2, 3, 5, 1)).astype(np.float32)
    gy = rng.standard_normal((2, 4, 5, 1)).astype(np.float32)
    np.testing.assert_array_equal(port.conv2d_backward_k(gy, x, 3, 3, 1, 1), ref.conv2d_backward_k(gy, x, 3, 3, 1, 1))
    # and everywhere it is the adjoint of the forward map: <conv(x, k), gy> = <k, backward_k(gy, x)>
    x = rng.standard_normal((2, 3, 6, 5)).astype(np.float64)
    k = rng.standard_normal((4, 3, 3, 3)).astype(np.float64)
    gy = rng.standard_normal((2, 4, 6, 5)).astype(np.float64)
    y = port.conv2d(x.astype(np.float32), k.astype(np.float32), 6, 5, 1, 1)
    gk = port.conv2d_backward_k(gy.astype(np.float32), x.astype(np.float32), 3, 3, 1, 1)
    gx = port.conv2d_backward_x(gy.astype(np.float32), k.astype(np.float32), 6, 5, 1, 1)
    lhs = float((y.astype(np.float64) * gy).sum())
    assert abs(lhs - float((gk.astype(np.float64) * k).sum())) < 1e-3 * abs(lhs) + 1e-3
    assert abs(lhs - float((gx.astype(np.float64) * x).sum())) < 1e-3 * abs(lhs) + 1e-3


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference (oracle/_ref) not built on this machine")
def test_conv2d_variants_port_matches_compiled_reference(port):
    ref = oracle.Oracle("ref")
    rng = np.random.default_rng(6)
    for (ndat, xchn, ychn, xh, xw, kh, kw, p0, p1) in [(2, 3, 4, 6, 5, 3, 3, 2, 2), (1, 2, 3, 4, 7, 5, 3, 3, 1),
                                                        (2, 4, 2, 5, 5, 1, 1, 1, 2), (1, 3, 2, 6, 6, 4, 2, 2, 3)]:
        x = rng.standard_normal((ndat, xchn, xh, xw)).astype(np.float32)
        k = rng.standard_normal((ychn, xchn, kh, kw)).astype(np.float32)
        gy_t = rng.standard_normal((ndat, ychn, xh * p0, xw * p1)).astype(np.float32)
        gy_d = rng.standard_normal((ndat, ychn, xh, xw)).astype(np.float32)
        dims = (ndat, xchn, xh, xw, ychn, kh, kw, p0, p1)
        for which, shape, a, b in (("transposed", gy_t.shape, x, k), ("transposed_backward_x", x.shape, gy_t, k),
                                   ("transposed_backward_k", k.shape, gy_t, x), ("dilated", gy_d.shape, x, k),
                                   ("dilated_backward_x", x.shape, gy_d, k), ("dilated_backward_k", k.shape, gy_d, x)):
            np.testing.assert_array_equal(port.conv2d_variant(which, shape, a, b, *dims),
                                          ref.conv2d_variant(which, shape, a, b, *dims), err_msg=f"{which} {dims}")


def test_empty_and_degenerate_inputs(port):
    z = np.zeros((0, 5), np.float32)
    w = np.ones((3, 5), np.float32)
    assert port.matmul(w, z).shape == (0, 3)
    assert port.add_bias_backward_b(np.zeros((0, 4), np.float32)).tolist() == [0, 0, 0, 0]
    one = port.matmul(np.array([[2.0]], np.float32), np.array([[3.0]], np.float32))
    assert one.tolist() == [[6.0]]
    assert port.sum(np.zeros(0, np.float32)).tolist() == [0.0]
    # a label outside [0, ncol) is an error in the reference (VERR_OUT_OF_RANGE, vmath.cu:8918)
    rc = port._call("softmax_idx_crossentropy", oracle._ptr(np.zeros(1, np.float32)),
                    oracle._ptr(np.zeros((1, 3), np.float32)), oracle._ptr(np.array([3], np.int32)),
                    oracle._I64(1), oracle._I64(3))
    assert rc == -1


def test_softmax_activation_is_row_softmax(port):
    """ActFunc::softmax in the port uses the intended row base (the reference's pointer arithmetic
    reads in front of the array, see oracle/kai_oracle.c)."""
    x = np.random.default_rng(0).standard_normal((5, 7)).astype(np.float32)
    y = port.activate(x, 9)
    e = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    np.testing.assert_allclose(y, e / e.sum(axis=1, keepdims=True), rtol=1e-6)


@pytest.mark.parametrize("K", [64, 512, 2048])
def test_reference_error_model(port, K):
    """The reference's sequential fp32 accumulation errs by about 1.8e-8*sqrt(K) (relative Frobenius,
    U[-1,1) inputs): the yardstick of the 2x rule."""
    rng = np.random.default_rng(K)
    x = rng.uniform(-1, 1, (32, K)).astype(np.float32)
    w = rng.uniform(-1, 1, (64, K)).astype(np.float32)
    err = oracle.rel_fro(port.matmul(w, x), x.astype(np.float64) @ w.astype(np.float64).T)
    assert 0.5e-8 * np.sqrt(K) < err < 4e-8 * np.sqrt(K)


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference (oracle/_ref) not built on this machine")
def test_layernorm_port_matches_compiled_reference(port):
    ref = oracle.Oracle("ref")
    rng = np.random.default_rng(6)
    for nrow, ncol in [(1, 1), (3, 7), (16, 64), (5, 513), (2, 4096)]:
        x = (rng.standard_normal((nrow, ncol)) * 3 + 1).astype(np.float32)
        gy = rng.standard_normal((nrow, ncol)).astype(np.float32)
        for scale in (1.0, 0.37, None):          # a NULL HYPER reads as 0 (local_objects/vhypermanager.h:9)
            yp, sp = port.layernorm(x, scale)
            yr, sr = ref.layernorm(x, scale)
            np.testing.assert_array_equal(yp, yr)
            np.testing.assert_array_equal(sp, sr)
            np.testing.assert_array_equal(port.layernorm_backward(gy, sp, scale), ref.layernorm_backward(gy, sr, scale))
