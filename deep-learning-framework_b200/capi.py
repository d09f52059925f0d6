"""ctypes declarations of the C ABI in include/kai_b200.h.

There is no fallback: if the shared library is missing, ``load()`` raises, and every
compute call on a machine without a B200 returns a CUDA error that is raised as KaiError.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "lib" / "libkai_b200.so"

# status codes / enums of kai_b200.h
OK = 0
E_INVALID_ARG, E_NO_HOST_PATH, E_NO_DRIVER, E_TENSOR_MAP = -1, -2, -3, -4
E_DEVICE_WAIT, E_OUT_OF_RANGE, E_TOO_LARGE, E_ALLOC = -5, -6, -7, -8
GEMM_NT, GEMM_NN, GEMM_TN = 0, 1, 2
ACT = {"none": 0, "relu": 1, "leaky": 2, "sigmoid": 3, "tanh": 4, "gelu": 5, "selu": 6, "mish": 7,
       "swish": 8, "softmax": 9}
PATH_AUTO, PATH_TC, PATH_SIMT, PATH_SKINNY = 0, 1, 2, 3
PREP_RAW_HI, PREP_LEFT, PREP_TF32_LO = 1, 2, 4

_i, _i64, _p, _s = C.c_int, C.c_int64, C.c_void_p, C.c_char_p

# name -> (restype, argtypes); one entry per declaration in include/kai_b200.h
SIGNATURES = {
    "kai_version": (_s, []),
    "kai_last_error_string": (_s, []),
    "kai_device_status": (_i, [_i, C.POINTER(_i)]),
    "kai_device_status_clear": (_i, [_i]),
    "kai_selftest_bounded_wait": (_i, [_i, _i64, _p]),
    "kai_set_option": (_i, [_s, _i64]),
    "kai_get_option": (_i64, [_s]),
    "kai_launch_count": (_i64, []),
    "kai_tc_launch_count": (_i64, []),
    "kai_tc_pair_launch_count": (_i64, []),
    "kai_profile_enable": (_i, [_i]),
    "kai_profile_read": (_i, [C.POINTER(C.c_double), C.POINTER(_i64)]),
    "kai_mem_alloc": (_i, [_i, _i64, C.POINTER(_p)]),
    "kai_mem_free": (_i, [_i, _p]),
    "kai_mem_alloc_pitched": (_i, [_i, _i64, _i64, C.POINTER(_p), C.POINTER(_i64)]),
    "kai_mem_trim": (_i, [_i]),
    "kai_mem_stats": (_i, [_i, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "kai_matmul": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i, _p]),
    "kai_matmul_backward_x": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i, _p]),
    "kai_matmul_backward_w": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i, _p]),
    "kai_linear_forward": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "kai_linear_forward_static": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "kai_matmul_host": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _p, _i, C.c_float]),
    "kai_operand_prepare": (_i, [_i, _p, _i64, _i64, _i64, _i, _i, C.POINTER(_p), _p]),
    "kai_operand_refresh": (_i, [_p, _p, _p]),
    "kai_operand_release": (_i, [_p]),
    "kai_linear_forward_prepared": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _i, _p, _p]),
    "kai_sgemm_prepared": (_i, [_i, _p, _p, _i64, _i64, _p, _i64, _i64, _i64, _i, _p, _i, _p, _p]),
    "kai_sgemm_grouped": (_i, [_i, _i, _i, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p), _i64, _i64, _i64, _i64, _i, _p,
                               _i, _p, _p]),
    "kai_layernorm": (_i, [_i, _p, _p, _p, _i64, _i64, _p, _p]),
    "kai_layernorm_backward": (_i, [_i, _p, _p, _p, _i64, _i64, _p, _p]),
    "kai_linear_forward_host": (_i, [_i, _p, _p, _p, _i64, _p, _i, C.c_float]),
    "kai_sgemm": (_i, [_i, _i, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _p, _i, _p, _i, _p]),
    "kai_add_bias": (_i, [_i, _p, _p, _p, _i64, _i64, _p]),
    "kai_add_bias_backward_b": (_i, [_i, _p, _p, _i64, _i64, _i, _p]),
    "kai_activate": (_i, [_i, _p, _p, _i64, _i64, _i, _p, _p]),
    "kai_activate_backward": (_i, [_i, _p, _p, _p, _i64, _i64, _i, _p, _p]),
    "kai_activate_backward_with_y": (_i, [_i, _p, _p, _p, _i64, _i64, _i, _p, _p]),
    "kai_mult_on_heads": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p, _p]),
    "kai_set_mh_attention_mask": (_i, [_i, _p, _i64, _i64, _i64, _i, _p]),
    "kai_softmax_direct_on_axis": (_i, [_i, _p, _i64, _i64, _i64, _p]),
    "kai_mix_values": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p]),
    "kai_conv2d": (_i, [_i, _p, _p, _p] + [_i64] * 12 + [_i, _p]),
    "kai_conv2d_backward_x": (_i, [_i, _p, _p, _p] + [_i64] * 12 + [_p]),
    "kai_conv2d_backward_k": (_i, [_i, _p, _p, _p] + [_i64] * 12 + [_p]),
    **{f"kai_conv2d_{v}{b}": (_i, [_i, _p, _p, _p] + [_i64] * 9 + [_p])
       for v in ("transposed", "dilated") for b in ("", "_backward_x", "_backward_k")},
    "kai_mh_attention_forward": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p, _i, _p]),
    "kai_replay_begin": (_i, [_i, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "kai_replay_end": (_i, [_p]),
    "kai_replay_launch": (_i, [_p, _p]),
    "kai_replay_destroy": (_i, [_p]),
    "kai_mult_on_heads_backward": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p]),
    "kai_softmax_direct_on_axis_backward": (_i, [_i, _p, _p, _i64, _i64, _i64, _p, _p]),
    "kai_mix_values_backward_prop": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p]),
    "kai_mix_values_backward_value": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p]),
    "kai_softmax_idx_crossentropy": (_i, [_i, _p, _p, _p, _i64, _i64, _p]),
    "kai_softmax_idx_crossentropy_backward_x": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _p]),
    "kai_sum": (_i, [_i, _p, _p, _i64, _p]),
    "kai_sum_backward": (_i, [_i, _p, _p, _i64, _p]),
}


class KaiError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"kai_b200 error {code}: {message}")
        self.code = code
        self.message = message


_lib = None


def load(path: str | Path | None = None) -> C.CDLL:
    """Loads libkai_b200.so (once) and attaches the prototypes."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else LIB_PATH
    if not p.exists():
        raise FileNotFoundError(
            f"{p} is missing: build it with `python deep-learning-framework_b200/build.py` "
            "(there is no non-CUDA fallback)")
    lib = C.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        if not hasattr(lib, name):
            continue  # optional symbols are checked by the tests against the header
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != OK:
        raise KaiError(rc, load().kai_last_error_string().decode("utf-8", "replace"))


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args))
