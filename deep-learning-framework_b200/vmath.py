"""Python mirror of the reference's ``class VMath`` for the matmul / Linear path.

Same function names, argument order and meaning as source/engine/support/vmath.h
(lines 18-19, 65-66, 137-143, 234-241, 299-301, 325-326); ``device`` is a CUDA ordinal.
Arguments that are pointers in C++ may be torch CUDA tensors (their ``data_ptr()`` is used),
raw integer addresses, or None.  Errors raise ``KaiError`` carrying the text the reference
would throw with VERR_CUDA_ERROR ("cuda:<message>").
"""
from __future__ import annotations

import ctypes as C

from . import capi


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return C.c_void_p(x)
    if hasattr(x, "data_ptr"):
        if not x.is_contiguous():
            raise ValueError("tensor arguments must be contiguous (the reference has no strides)")
        return C.c_void_p(x.data_ptr())
    raise TypeError(f"cannot take the address of {type(x)!r}")


def _act(a) -> int:
    return capi.ACT[a] if isinstance(a, str) else int(a)


def mem_alloc(device: int, size: int) -> int:
    out = C.c_void_p()
    capi.call("kai_mem_alloc", device, size, C.byref(out))
    return out.value or 0


def mem_free(device: int, ptr: int) -> None:
    capi.call("kai_mem_free", device, C.c_void_p(ptr))


def matmul(device, py, pw, px, yvec, ndat, xvec, acc=False, stream=None):
    capi.call("kai_matmul", device, _ptr(py), _ptr(pw), _ptr(px), yvec, ndat, xvec, int(bool(acc)), _ptr(stream))


def matmul_backward_x(device, pgx, pgy, pw, yvec, ndat, xvec, acc=False, stream=None):
    capi.call("kai_matmul_backward_x", device, _ptr(pgx), _ptr(pgy), _ptr(pw), yvec, ndat, xvec, int(bool(acc)),
              _ptr(stream))


def matmul_backward_w(device, pgw, pgy, px, yvec, ndat, xvec, acc=False, stream=None):
    capi.call("kai_matmul_backward_w", device, _ptr(pgw), _ptr(pgy), _ptr(px), yvec, ndat, xvec, int(bool(acc)),
              _ptr(stream))


def linear_forward(device, py, pw, px, pb, yvec, ndat, xvec, ldy=None, act="none", leaky_alpha=None, stream=None):
    """Fused matmul + add_bias + activate (the `linear` / `dense` layer formulas)."""
    capi.call("kai_linear_forward", device, _ptr(py), _ptr(pw), _ptr(px), _ptr(pb), yvec, ndat, xvec,
              yvec if ldy is None else ldy, _act(act), _ptr(leaky_alpha), _ptr(stream))


def linear_forward_static(device, py, pw, px, pb, yvec, ndat, xvec, ldy=None, act="none", leaky_alpha=None,
                          stream=None):
    """linear_forward without any device allocation: the kernel's scratch is a fixed 32 MiB array inside the
    library, so (ndat + yvec) * xvec is limited (KaiError with code E_TOO_LARGE beyond it).  For callers that
    cannot allocate while they run; calls on one device must not overlap on the GPU."""
    capi.call("kai_linear_forward_static", device, _ptr(py), _ptr(pw), _ptr(px), _ptr(pb), yvec, ndat, xvec,
              yvec if ldy is None else ldy, _act(act), _ptr(leaky_alpha), _ptr(stream))


def matmul_host(device, py_host, pw_host, px_host, yvec, ndat, xvec, pb_host=None, act="none", leaky_alpha=0.0):
    """py = act(px . pw^T + pb) on host tensors (pinned for asynchronous copies); returns when py_host is written."""
    capi.call("kai_matmul_host", device, _ptr(py_host), _ptr(pw_host), _ptr(px_host), yvec, ndat, xvec, _ptr(pb_host),
              _act(act), float(leaky_alpha))


def sgemm(device, layout, c, a, b, M, N, K, ldc=None, accumulate=False, bias=None, act="none", leaky_alpha=None,
          path=capi.PATH_AUTO, stream=None):
    capi.call("kai_sgemm", device, layout, _ptr(c), _ptr(a), _ptr(b), M, N, K, N if ldc is None else ldc,
              int(bool(accumulate)), _ptr(bias), _act(act), _ptr(leaky_alpha), path, _ptr(stream))


class PreparedOperand:
    """K-major hi/lo planes of one GEMM operand, written once (kai_operand_prepare) -- e.g. a Linear layer's
    weight, which changes only at the optimiser step.  ``src`` is [rows, k] (``transpose=False``) or [k, rows]."""

    def __init__(self, device, src, rows, k, ld=None, transpose=False, raw_hi=False, left=False, tf32_lo=False,
                 stream=None):
        self.device, self.rows, self.k = device, rows, k
        h = C.c_void_p()
        capi.call("kai_operand_prepare", device, _ptr(src), rows, k, (rows if transpose else k) if ld is None else ld,
                  int(bool(transpose)),
                  (capi.PREP_RAW_HI if raw_hi else 0) | (capi.PREP_LEFT if left else 0) |
                  (capi.PREP_TF32_LO if tf32_lo else 0), C.byref(h), _ptr(stream))
        self.handle = h.value

    def refresh(self, src, stream=None):
        capi.call("kai_operand_refresh", C.c_void_p(self.handle), _ptr(src), _ptr(stream))

    def release(self):
        if self.handle is not None:
            capi.call("kai_operand_release", C.c_void_p(self.handle))
            self.handle = None


def linear_forward_prepared(device, py, w_prep, px, pb, ndat, ldy=None, act="none", leaky_alpha=None, stream=None):
    """linear_forward with the weight given as a PreparedOperand (yvec = its rows, xvec = its k)."""
    capi.call("kai_linear_forward_prepared", device, _ptr(py), C.c_void_p(w_prep.handle), _ptr(px), _ptr(pb), ndat,
              w_prep.rows if ldy is None else ldy, _act(act), _ptr(leaky_alpha), _ptr(stream))


def linear_forward_host(device, py_host, w_prep, px_host, ndat, pb_host=None, act="none", leaky_alpha=0.0):
    """matmul_host with the weight device-resident as a PreparedOperand: only px goes up and py comes down."""
    capi.call("kai_linear_forward_host", device, _ptr(py_host), C.c_void_p(w_prep.handle), _ptr(px_host), ndat,
              _ptr(pb_host), _act(act), float(leaky_alpha))


def sgemm_prepared(device, c, a_prep, a_row0, M, b_prep, b_row0, N, ldc=None, accumulate=False, bias=None, act="none",
                   leaky_alpha=None, stream=None):
    """C[M,N] (+)= A'[a_row0:a_row0+M] . B'[b_row0:b_row0+N]^T on two PreparedOperands."""
    capi.call("kai_sgemm_prepared", device, _ptr(c), C.c_void_p(a_prep.handle), a_row0, M, C.c_void_p(b_prep.handle),
              b_row0, N, N if ldc is None else ldc, int(bool(accumulate)), _ptr(bias), _act(act), _ptr(leaky_alpha),
              _ptr(stream))


def sgemm_grouped(device, layout, cs, as_, bs, M, N, K, ldc=None, accumulate=False, bias=None, act="none",
                  leaky_alpha=None, stream=None):
    """len(cs) products of one shape in one launch; cs / as_ / bs are lists of tensors or addresses."""
    n = len(cs)
    arr = lambda xs: (C.c_void_p * n)(*[_ptr(x) for x in xs])  # noqa: E731
    capi.call("kai_sgemm_grouped", device, layout, n, arr(cs), arr(as_), arr(bs), M, N, K, N if ldc is None else ldc,
              int(bool(accumulate)), _ptr(bias), _act(act), _ptr(leaky_alpha), _ptr(stream))


def layernorm(device, py, px, ps, nrow, ncol, hScale, stream=None):
    capi.call("kai_layernorm", device, _ptr(py), _ptr(px), _ptr(ps), nrow, ncol, _ptr(hScale), _ptr(stream))


def layernorm_backward(device, pgx, pgy, ps, nrow, ncol, hScale, stream=None):
    capi.call("kai_layernorm_backward", device, _ptr(pgx), _ptr(pgy), _ptr(ps), nrow, ncol, _ptr(hScale), _ptr(stream))


def add_bias(device, py, pa, pb, nrow, ncol, stream=None):
    capi.call("kai_add_bias", device, _ptr(py), _ptr(pa), _ptr(pb), nrow, ncol, _ptr(stream))


def add_bias_backward_b(device, pgb, pgy, nrow, ncol, acc=False, stream=None):
    capi.call("kai_add_bias_backward_b", device, _ptr(pgb), _ptr(pgy), nrow, ncol, int(bool(acc)), _ptr(stream))


def activate(device, py, px, nrow, ncol, actFunc, hLeakyAlpha=None, stream=None):
    capi.call("kai_activate", device, _ptr(py), _ptr(px), nrow, ncol, _act(actFunc), _ptr(hLeakyAlpha), _ptr(stream))


def activate_backward(device, pgx, pgy, px, nrow, ncol, actFunc, hLeakyAlpha=None, stream=None):
    capi.call("kai_activate_backward", device, _ptr(pgx), _ptr(pgy), _ptr(px), nrow, ncol, _act(actFunc),
              _ptr(hLeakyAlpha), _ptr(stream))


def activate_backward_with_y(device, pgx, pgy, py, nrow, ncol, actFunc, hLeakyAlpha=None, stream=None):
    capi.call("kai_activate_backward_with_y", device, _ptr(pgx), _ptr(pgy), _ptr(py), nrow, ncol, _act(actFunc),
              _ptr(hLeakyAlpha), _ptr(stream))


def mult_on_heads(device, pp, pK, pQ, nbat, ntimes, nvec, nhead, npiece, hCoef, stream=None):
    capi.call("kai_mult_on_heads", device, _ptr(pp), _ptr(pK), _ptr(pQ), nbat, ntimes, nvec, nhead, npiece,
              _ptr(hCoef), _ptr(stream))


def set_mh_attention_mask(device, pp, ndat, ntimes, nhead, forward=True, stream=None):
    capi.call("kai_set_mh_attention_mask", device, _ptr(pp), ndat, ntimes, nhead, int(bool(forward)), _ptr(stream))


def softmax_direct_on_axis(device, pp, nrow, nvec, ncol, stream=None):
    capi.call("kai_softmax_direct_on_axis", device, _ptr(pp), nrow, nvec, ncol, _ptr(stream))


def mix_values(device, py, pp, pV, nbat, ntimes, nvec, nhead, npiece, stream=None):
    capi.call("kai_mix_values", device, _ptr(py), _ptr(pp), _ptr(pV), nbat, ntimes, nvec, nhead, npiece,
              _ptr(stream))


def conv2d(device, py, px, pk, ndat, ychn, yh, yw, xchn, xh, xw, kh, kw, group, ph, pw, pmode=0, stream=None):
    capi.call("kai_conv2d", device, _ptr(py), _ptr(px), _ptr(pk), ndat, ychn, yh, yw, xchn, xh, xw, kh, kw, group, ph, pw,
              int(pmode), _ptr(stream))


def conv2d_backward_x(device, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw, stream=None):
    capi.call("kai_conv2d_backward_x", device, _ptr(pgx), _ptr(pgy), _ptr(pk), ndat, xchn, xh, xw, ychn, yh, yw, kh, kw,
              group, ph, pw, _ptr(stream))


def conv2d_backward_k(device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw, stream=None):
    capi.call("kai_conv2d_backward_k", device, _ptr(pgk), _ptr(pgy), _ptr(px), ndat, xchn, xh, xw, ychn, yh, yw, kh, kw,
              group, ph, pw, _ptr(stream))


def _conv_variant(name):
    def f(device, out, first, second, ndat, xchn, xh, xw, ychn, kh, kw, p0, p1, stream=None):
        capi.call("kai_" + name, device, _ptr(out), _ptr(first), _ptr(second), ndat, xchn, xh, xw, ychn, kh, kw, p0, p1,
                  _ptr(stream))
    f.__name__ = name
    f.__doc__ = f"VMath::{name}(device, out, in1, in2, ndat, xchn, xh, xw, ychn, kh, kw, stride-or-gap h, w)"
    return f


conv2d_transposed = _conv_variant("conv2d_transposed")
conv2d_transposed_backward_x = _conv_variant("conv2d_transposed_backward_x")
conv2d_transposed_backward_k = _conv_variant("conv2d_transposed_backward_k")
conv2d_dilated = _conv_variant("conv2d_dilated")
conv2d_dilated_backward_x = _conv_variant("conv2d_dilated_backward_x")
conv2d_dilated_backward_k = _conv_variant("conv2d_dilated_backward_k")


def mh_attention_forward(device, py, pK, pQ, pV, nbat, ntimes, nvec, nhead, npiece, hCoef, causal_mask=False,
                         stream=None):
    capi.call("kai_mh_attention_forward", device, _ptr(py), _ptr(pK), _ptr(pQ), _ptr(pV), nbat, ntimes, nvec, nhead,
              npiece, _ptr(hCoef), int(bool(causal_mask)), _ptr(stream))


def mult_on_heads_backward(device, pgQK, pgp, pKQ, nbat, ntimes, nvec, nhead, npiece, stream=None):
    capi.call("kai_mult_on_heads_backward", device, _ptr(pgQK), _ptr(pgp), _ptr(pKQ), nbat, ntimes, nvec, nhead, npiece,
              _ptr(stream))


def softmax_direct_on_axis_backward(device, pgp, pp, nbat, ntimes, nhead, hCoef, stream=None):
    capi.call("kai_softmax_direct_on_axis_backward", device, _ptr(pgp), _ptr(pp), nbat, ntimes, nhead, _ptr(hCoef),
              _ptr(stream))


def mix_values_backward_prop(device, pgp, pgy, pV, nbat, ntimes, nvec, nhead, npiece, stream=None):
    capi.call("kai_mix_values_backward_prop", device, _ptr(pgp), _ptr(pgy), _ptr(pV), nbat, ntimes, nvec, nhead, npiece,
              _ptr(stream))


def mix_values_backward_value(device, pgV, pgy, pp, nbat, ntimes, nvec, nhead, npiece, stream=None):
    capi.call("kai_mix_values_backward_value", device, _ptr(pgV), _ptr(pgy), _ptr(pp), nbat, ntimes, nvec, nhead,
              npiece, _ptr(stream))


def softmax_idx_crossentropy(device, py, px, pz, nrow, ncol, stream=None):
    capi.call("kai_softmax_idx_crossentropy", device, _ptr(py), _ptr(px), _ptr(pz), nrow, ncol, _ptr(stream))


def softmax_idx_crossentropy_backward_x(device, pgx, pgy, px, pz, nrow, ncol, stream=None):
    capi.call("kai_softmax_idx_crossentropy_backward_x", device, _ptr(pgx), _ptr(pgy), _ptr(px), _ptr(pz), nrow,
              ncol, _ptr(stream))


def sum(device, py, px, nrow, stream=None):  # noqa: A001 - the reference's name
    capi.call("kai_sum", device, _ptr(py), _ptr(px), nrow, _ptr(stream))


def sum_backward(device, pgx, pgy, nrow, stream=None):
    capi.call("kai_sum_backward", device, _ptr(pgx), _ptr(pgy), nrow, _ptr(stream))


class Replay:
    """A recorded list of calls replayed as one launch (kai_replay_* of the C ABI; the counterpart of the
    reference tracer's replay pass, local_objects/vexectracer.cpp:496-550).

        with Replay(0) as rp:
            matmul(0, y, w, x, N, M, K, stream=rp.stream)      # recorded, not executed
            add_bias(0, y, y, b, M, N, stream=rp.stream)
        rp.launch()                                            # runs both
    """

    def __init__(self, device: int):
        self.device = device
        self.handle = None
        self.stream = None

    def __enter__(self):
        import ctypes as C
        h, s = C.c_void_p(), C.c_void_p()
        capi.call("kai_replay_begin", self.device, C.byref(h), C.byref(s))
        self.handle, self.stream = h.value, s.value
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is not None:
            self.close()
            return False
        capi.call("kai_replay_end", self.handle)
        return False

    def launch(self, stream=None):
        capi.call("kai_replay_launch", self.handle, _ptr(stream))

    def close(self):
        if self.handle is not None:
            capi.call("kai_replay_destroy", self.handle)
            self.handle = None
