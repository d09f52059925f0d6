"""TEST INFRASTRUCTURE -- the CPU oracle of the matmul / Linear path.

Two interchangeable back ends with one numpy API:

* ``Oracle("port")``  -- oracle/kai_oracle.c, the C restatement of the reference's host loops
  (built by ``make -C oracle``).
* ``Oracle("ref")``   -- oracle/_ref/libkonan_ref.so, the UNMODIFIED reference math layer
  compiled from a reference checkout by oracle/build_ref.sh; its ``VMath::*`` static methods
  are called by their mangled names with ``device = -1`` (the reference's host branch).

Only tests/, the smoke check and bench.py's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "liboracle_port.so"
REF_LIB = HERE / "_ref" / "libkonan_ref.so"

_f = np.float32
_P, _I64, _I, _B = C.c_void_p, C.c_int64, C.c_int, C.c_bool


def build_port(force: bool = False) -> Path:
    if force or not PORT_LIB.exists() or PORT_LIB.stat().st_mtime < (HERE / "kai_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B" if force else "-s", "liboracle_port.so"], check=True,
                       capture_output=True)
    return PORT_LIB


def have_ref() -> bool:
    return REF_LIB.exists()


def _ptr(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"], "oracle arguments must be contiguous numpy arrays"
    return C.c_void_p(a.ctypes.data)


# port symbol, reference mangled symbol (itanium ABI of `static void VMath::f(int, ...)`)
_SYMS = {
    "matmul": ("orc_matmul", "_ZN5VMath6matmulEiPfS0_S0_lllb"),
    "matmul_backward_x": ("orc_matmul_backward_x", "_ZN5VMath17matmul_backward_xEiPfS0_S0_lllb"),
    "matmul_backward_w": ("orc_matmul_backward_w", "_ZN5VMath17matmul_backward_wEiPfS0_S0_lllb"),
    "add_bias": ("orc_add_bias", "_ZN5VMath8add_biasEiPfS0_S0_ll"),
    "add_bias_backward_b": ("orc_add_bias_backward_b", "_ZN5VMath19add_bias_backward_bEiPfS0_llb"),
    "activate": ("orc_activate", "_ZN5VMath8activateEiPfS0_lliS0_"),
    "activate_backward": ("orc_activate_backward", "_ZN5VMath17activate_backwardEiPfS0_S0_lliS0_"),
    "activate_backward_with_y": ("orc_activate_backward_with_y", "_ZN5VMath24activate_backward_with_yEiPfS0_S0_lliS0_"),
    "mult_on_heads": ("orc_mult_on_heads", "_ZN5VMath13mult_on_headsEiPfS0_S0_lllllS0_"),
    "set_mh_attention_mask": ("orc_set_mh_attention_mask", "_ZN5VMath21set_mh_attention_maskEiPflllb"),
    "softmax_direct_on_axis": ("orc_softmax_direct_on_axis", "_ZN5VMath22softmax_direct_on_axisEiPflll"),
    "mix_values": ("orc_mix_values", "_ZN5VMath10mix_valuesEiPfS0_S0_lllll"),
    "mult_on_heads_backward": ("orc_mult_on_heads_backward", "_ZN5VMath22mult_on_heads_backwardEiPfS0_S0_lllll"),
    "softmax_direct_on_axis_backward": ("orc_softmax_direct_on_axis_backward",
                                        "_ZN5VMath31softmax_direct_on_axis_backwardEiPfS0_lllS0_"),
    "mix_values_backward_prop": ("orc_mix_values_backward_prop", "_ZN5VMath24mix_values_backward_propEiPfS0_S0_lllll"),
    "mix_values_backward_value": ("orc_mix_values_backward_value",
                                  "_ZN5VMath25mix_values_backward_valueEiPfS0_S0_lllll"),
    "conv2d": ("orc_conv2d", "_ZN5VMath6conv2dEiPfS0_S0_lllllllllllli"),
    "conv2d_backward_x": ("orc_conv2d_backward_x", "_ZN5VMath17conv2d_backward_xEiPfS0_S0_llllllllllll"),
    "conv2d_backward_k": ("orc_conv2d_backward_k", "_ZN5VMath17conv2d_backward_kEiPfS0_S0_llllllllllll"),
    "conv2d_transposed": ("orc_conv2d_transposed", "_ZN5VMath17conv2d_transposedEiPfS0_S0_lllllllll"),
    "conv2d_transposed_backward_x": ("orc_conv2d_transposed_backward_x",
                                     "_ZN5VMath28conv2d_transposed_backward_xEiPfS0_S0_lllllllll"),
    "conv2d_transposed_backward_k": ("orc_conv2d_transposed_backward_k",
                                     "_ZN5VMath28conv2d_transposed_backward_kEiPfS0_S0_lllllllll"),
    "conv2d_dilated": ("orc_conv2d_dilated", "_ZN5VMath14conv2d_dilatedEiPfS0_S0_lllllllll"),
    "conv2d_dilated_backward_x": ("orc_conv2d_dilated_backward_x", "_ZN5VMath25conv2d_dilated_backward_xEiPfS0_S0_lllllllll"),
    "conv2d_dilated_backward_k": ("orc_conv2d_dilated_backward_k", "_ZN5VMath25conv2d_dilated_backward_kEiPfS0_S0_lllllllll"),
    "softmax_idx_crossentropy": ("orc_softmax_idx_crossentropy", "_ZN5VMath24softmax_idx_crossentropyEiPfS0_Pill"),
    "softmax_idx_crossentropy_backward_x": ("orc_softmax_idx_crossentropy_backward_x",
                                            "_ZN5VMath35softmax_idx_crossentropy_backward_xEiPfS0_S0_Pill"),
    "sum": ("orc_sum", "_ZN5VMath3sumEiPfS0_l"),
    "sum_backward": ("orc_sum_backward", "_ZN5VMath12sum_backwardEiPfS0_l"),
    "layernorm": ("orc_layernorm", "_ZN5VMath9layernormEiPfS0_S0_llS0_"),
    "layernorm_backward": ("orc_layernorm_backward", "_ZN5VMath18layernorm_backwardEiPfS0_S0_llS0_"),
}


class Oracle:
    """numpy front end; every method returns freshly allocated outputs."""

    def __init__(self, kind: str = "port"):
        assert kind in ("port", "ref")
        self.kind = kind
        if kind == "port":
            self.lib = C.CDLL(str(build_port()))
        else:
            if not have_ref():
                raise FileNotFoundError(f"{REF_LIB} missing: run oracle/build_ref.sh where the reference is mounted")
            self.lib = C.CDLL(str(REF_LIB))

    def _call(self, name, *args):
        port, ref = _SYMS[name]
        if self.kind == "port":
            fn = getattr(self.lib, port)
            fn.restype = C.c_int
            return fn(*args)
        fn = getattr(self.lib, ref)
        fn.restype = None
        return fn(C.c_int(-1), *args)

    # --- GEMM trio (raw form: writes into `out`, which also carries the old value for acc) ---
    def matmul_into(self, py, pw, px, yvec, ndat, xvec, acc=False):
        self._call("matmul", _ptr(py), _ptr(pw), _ptr(px), _I64(yvec), _I64(ndat), _I64(xvec), _B(acc))

    def matmul(self, w, x, acc_into=None):
        yvec, xvec = w.shape
        ndat = x.size // xvec
        y = np.zeros((ndat, yvec), _f) if acc_into is None else acc_into.copy()
        self.matmul_into(y, w, x, yvec, ndat, xvec, acc_into is not None)
        return y

    def matmul_backward_x(self, gy, w, acc_into=None):
        yvec, xvec = w.shape
        ndat = gy.size // yvec
        gx = np.zeros((ndat, xvec), _f) if acc_into is None else acc_into.copy()
        self._call("matmul_backward_x", _ptr(gx), _ptr(gy), _ptr(w), _I64(yvec), _I64(ndat), _I64(xvec),
                   _B(acc_into is not None))
        return gx

    def matmul_backward_w(self, gy, x, yvec, xvec, acc_into=None):
        ndat = x.size // xvec
        gw = np.zeros((yvec, xvec), _f) if acc_into is None else acc_into.copy()
        self._call("matmul_backward_w", _ptr(gw), _ptr(gy), _ptr(x), _I64(yvec), _I64(ndat), _I64(xvec),
                   _B(acc_into is not None))
        return gw

    # --- bias / activation ---
    def add_bias(self, a, b):
        nrow, ncol = a.shape
        y = np.empty_like(a)
        self._call("add_bias", _ptr(y), _ptr(a), _ptr(b), _I64(nrow), _I64(ncol))
        return y

    def add_bias_backward_b(self, gy, acc_into=None):
        nrow, ncol = gy.shape
        gb = np.zeros(ncol, _f) if acc_into is None else acc_into.copy()
        self._call("add_bias_backward_b", _ptr(gb), _ptr(gy), _I64(nrow), _I64(ncol), _B(acc_into is not None))
        return gb

    def _alpha(self, alpha):
        return None if alpha is None else np.array([alpha], _f)

    def activate(self, x, act, alpha=None):
        if act == 9 and self.kind == "ref":
            raise ValueError("the reference's softmax activation reads in front of its input (vmath.cu:3145)")
        nrow, ncol = x.shape
        y = np.empty_like(x)
        a = self._alpha(alpha)
        self._call("activate", _ptr(y), _ptr(x), _I64(nrow), _I64(ncol), _I(act), _ptr(a))
        return y

    def activate_backward(self, gy, x, act, alpha=None):
        nrow, ncol = x.shape
        gx = np.empty_like(x)
        a = self._alpha(alpha)
        self._call("activate_backward", _ptr(gx), _ptr(gy), _ptr(x), _I64(nrow), _I64(ncol), _I(act), _ptr(a))
        return gx

    def activate_backward_with_y(self, gy, y, act, alpha=None):
        nrow, ncol = y.shape
        gx = np.empty_like(y)
        a = self._alpha(alpha)
        self._call("activate_backward_with_y", _ptr(gx), _ptr(gy), _ptr(y), _I64(nrow), _I64(ncol), _I(act), _ptr(a))
        return gx

    # --- attention ---
    def mult_on_heads(self, K, Q, nhead, coef):
        nbat, ntimes, nvec = Q.shape
        npiece = nvec // nhead
        pp = np.empty((nbat, ntimes, ntimes, nhead), _f)
        c = np.array([coef], _f)
        self._call("mult_on_heads", _ptr(pp), _ptr(K), _ptr(Q), _I64(nbat), _I64(ntimes), _I64(nvec), _I64(nhead),
                   _I64(npiece), _ptr(c))
        return pp

    def set_mh_attention_mask(self, pp, forward=True):
        ndat, ntimes, _, nhead = pp.shape
        out = pp.copy()
        self._call("set_mh_attention_mask", _ptr(out), _I64(ndat), _I64(ntimes), _I64(nhead), _B(forward))
        return out

    def softmax_direct_on_axis(self, pp):
        """pp: [..., nvec, ncol]; softmax over the next-to-last axis."""
        nvec, ncol = pp.shape[-2:]
        nrow = pp.size // (nvec * ncol)
        out = pp.copy()
        self._call("softmax_direct_on_axis", _ptr(out), _I64(nrow), _I64(nvec), _I64(ncol))
        return out

    def mix_values(self, pp, V, nhead):
        nbat, ntimes, nvec = V.shape
        npiece = nvec // nhead
        y = np.empty((nbat, ntimes, nhead, npiece), _f)
        self._call("mix_values", _ptr(y), _ptr(pp), _ptr(V), _I64(nbat), _I64(ntimes), _I64(nvec), _I64(nhead),
                   _I64(npiece))
        return y

    def mult_on_heads_backward(self, gp, KQ, nhead):
        """Gradient of one operand of mult_on_heads given the other one (KQ) and the score gradient gp."""
        nbat, ntimes, nvec = KQ.shape
        npiece = nvec // nhead
        g = np.empty((nbat, ntimes, nvec), _f)
        self._call("mult_on_heads_backward", _ptr(g), _ptr(gp), _ptr(KQ), _I64(nbat), _I64(ntimes), _I64(nvec),
                   _I64(nhead), _I64(npiece))
        return g

    def softmax_direct_on_axis_backward(self, gp, pp, coef):
        nbat, ntimes, _, nhead = pp.shape
        out = gp.copy()
        c = np.array([coef], _f)
        self._call("softmax_direct_on_axis_backward", _ptr(out), _ptr(pp), _I64(nbat), _I64(ntimes), _I64(nhead),
                   _ptr(c))
        return out

    def mix_values_backward_prop(self, gy, V, nhead):
        nbat, ntimes, nvec = V.shape
        npiece = nvec // nhead
        gp = np.empty((nbat, ntimes, ntimes, nhead), _f)
        self._call("mix_values_backward_prop", _ptr(gp), _ptr(gy), _ptr(V), _I64(nbat), _I64(ntimes), _I64(nvec),
                   _I64(nhead), _I64(npiece))
        return gp

    def mix_values_backward_value(self, gy, pp, nhead):
        nbat, ntimes, _, _ = pp.shape
        nvec = gy.size // (nbat * ntimes)
        npiece = nvec // nhead
        gV = np.empty((nbat, ntimes, nvec), _f)
        self._call("mix_values_backward_value", _ptr(gV), _ptr(gy), _ptr(pp), _I64(nbat), _I64(ntimes), _I64(nvec),
                   _I64(nhead), _I64(npiece))
        return gV

    # --- convolution (NCHW, stride 1, zero padding) ---
    def conv2d(self, x, k, yh, yw, ph, pw, group=1):
        ndat, xchn, xh, xw = x.shape
        ychn, _, kh, kw = k.shape
        y = np.empty((ndat, ychn, yh, yw), _f)
        args = [_ptr(y), _ptr(x), _ptr(k), _I64(ndat), _I64(ychn), _I64(yh), _I64(yw), _I64(xchn), _I64(xh), _I64(xw),
                _I64(kh), _I64(kw), _I64(group), _I64(ph), _I64(pw)]
        if self.kind == "ref":
            args.append(_I(0))           # pmode: zero padding (the only mode the reference implements)
        self._call("conv2d", *args)
        return y

    def conv2d_backward_x(self, gy, k, xh, xw, ph, pw, group=1):
        ndat, ychn, yh, yw = gy.shape
        _, kchn, kh, kw = k.shape
        xchn = kchn * group
        gx = np.empty((ndat, xchn, xh, xw), _f)
        self._call("conv2d_backward_x", _ptr(gx), _ptr(gy), _ptr(k), _I64(ndat), _I64(xchn), _I64(xh), _I64(xw),
                   _I64(ychn), _I64(yh), _I64(yw), _I64(kh), _I64(kw), _I64(group), _I64(ph), _I64(pw))
        return gx

    def conv2d_backward_k(self, gy, x, kh, kw, ph, pw, group=1):
        ndat, ychn, yh, yw = gy.shape
        _, xchn, xh, xw = x.shape
        gk = np.empty((ychn, xchn // group, kh, kw), _f)
        self._call("conv2d_backward_k", _ptr(gk), _ptr(gy), _ptr(x), _I64(ndat), _I64(xchn), _I64(xh), _I64(xw),
                   _I64(ychn), _I64(yh), _I64(yw), _I64(kh), _I64(kw), _I64(group), _I64(ph), _I64(pw))
        return gk

    def conv2d_variant(self, which, out_shape, first, second, ndat, xchn, xh, xw, ychn, kh, kw, p0, p1):
        """The transposed / dilated family: `which` in {transposed, dilated}[_backward_x|_backward_k]; all six take
        (out, in1, in2, ndat, xchn, xh, xw, ychn, kh, kw, stride-or-gap h, w)."""
        out = np.empty(out_shape, _f)
        self._call("conv2d_" + which, _ptr(out), _ptr(first), _ptr(second), _I64(ndat), _I64(xchn), _I64(xh), _I64(xw),
                   _I64(ychn), _I64(kh), _I64(kw), _I64(p0), _I64(p1))
        return out

    # --- loss ---
    def softmax_idx_crossentropy(self, x, labels):
        nrow, ncol = x.shape
        y = np.empty(nrow, _f)
        self._call("softmax_idx_crossentropy", _ptr(y), _ptr(x), _ptr(labels), _I64(nrow), _I64(ncol))
        return y

    def softmax_idx_crossentropy_backward_x(self, gy, x, labels):
        nrow, ncol = x.shape
        gx = np.empty_like(x)
        self._call("softmax_idx_crossentropy_backward_x", _ptr(gx), _ptr(gy), _ptr(x), _ptr(labels), _I64(nrow),
                   _I64(ncol))
        return gx

    def sum(self, x):
        y = np.empty(1, _f)
        self._call("sum", _ptr(y), _ptr(x), _I64(x.size))
        return y

    def sum_backward(self, n, gy=None):
        gx = np.empty(n, _f)
        self._call("sum_backward", _ptr(gx), _ptr(gy), _I64(n))
        return gx


    # --- layernorm (support/vmath.cu:5977-6085) ---
    def layernorm(self, x, scale):
        """Returns (y, stat) with stat[r] = (avg, std) of row r."""
        nrow, ncol = x.shape
        y = np.empty_like(x)
        stat = np.empty((nrow, 2), _f)
        self._call("layernorm", _ptr(y), _ptr(x), _ptr(stat), _I64(nrow), _I64(ncol), _ptr(self._alpha(scale)))
        return y, stat

    def layernorm_backward(self, gy, stat, scale):
        nrow, ncol = gy.shape
        gx = np.empty_like(gy)
        self._call("layernorm_backward", _ptr(gx), _ptr(gy), _ptr(stat), _I64(nrow), _I64(ncol),
                   _ptr(self._alpha(scale)))
        return gx


def rel_fro(got, truth64) -> float:
    """Relative Frobenius error against an fp64 ground truth."""
    t = np.asarray(truth64, np.float64)
    d = np.asarray(got, np.float64) - t
    den = np.linalg.norm(t.ravel())
    return float(np.linalg.norm(d.ravel()) / (den if den > 0 else 1.0))
