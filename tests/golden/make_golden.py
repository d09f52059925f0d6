"""Generates tests/golden/reference_vectors.npz from the UNMODIFIED reference math layer.

Run where the reference checkout is mounted and oracle/_ref/libkonan_ref.so has been built
(oracle/build_ref.sh).  Inputs are drawn from numpy's PCG64 with the seeds below; outputs are what
the reference's `VMath::*` host branch (device = -1) returns for them.  The reference ships no
golden vectors of its own, so these pin the CPU oracle port (and, through it, the GPU path) on
machines where the reference itself is not available.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402

OUT = Path(__file__).resolve().parent / "reference_vectors.npz"


def inputs():
    """Deterministic small inputs; shared by this script and tests/test_oracle.py."""
    rng = np.random.default_rng(20240917)
    f = np.float32
    d = {}
    d["x"] = rng.uniform(-1, 1, (9, 21)).astype(f)          # [ndat, xvec]
    d["w"] = rng.uniform(-1, 1, (13, 21)).astype(f)         # [yvec, xvec]
    d["gy"] = rng.standard_normal((9, 13)).astype(f)        # [ndat, yvec]
    d["acc_y"] = rng.standard_normal((9, 13)).astype(f)
    d["acc_x"] = rng.standard_normal((9, 21)).astype(f)
    d["acc_w"] = rng.standard_normal((13, 21)).astype(f)
    d["b"] = rng.standard_normal(13).astype(f)
    d["act_in"] = (rng.standard_normal((6, 11)) * 3).astype(f)
    d["act_gy"] = rng.standard_normal((6, 11)).astype(f)
    d["q"] = rng.standard_normal((2, 7, 12)).astype(f)      # [nbat, ntimes, nhead*npiece], 3 heads x 4
    d["k"] = rng.standard_normal((2, 7, 12)).astype(f)
    d["v"] = rng.standard_normal((2, 7, 12)).astype(f)
    d["logits"] = (rng.standard_normal((8, 10)) * 2).astype(f)
    d["labels"] = rng.integers(0, 10, 8).astype(np.int32)
    d["attn_gy"] = rng.standard_normal((2, 7, 3, 4)).astype(f)   # drawn last: earlier inputs keep their values
    d["conv_x"] = rng.standard_normal((2, 3, 6, 5)).astype(f)      # NCHW
    d["conv_k"] = rng.standard_normal((4, 3, 3, 3)).astype(f)      # [ychn, xchn, kh, kw]
    d["conv_gy"] = rng.standard_normal((2, 4, 6, 5)).astype(f)
    d["ln_x"] = (rng.standard_normal((5, 37)) * 2 + 0.5).astype(f)   # drawn after everything above: earlier inputs keep their values
    d["ln_gy"] = rng.standard_normal((5, 37)).astype(f)
    return d


def compute(orc):
    d = inputs()
    o = {}
    o["matmul"] = orc.matmul(d["w"], d["x"])
    o["matmul_acc"] = orc.matmul(d["w"], d["x"], d["acc_y"])
    o["matmul_backward_x"] = orc.matmul_backward_x(d["gy"], d["w"])
    o["matmul_backward_x_acc"] = orc.matmul_backward_x(d["gy"], d["w"], d["acc_x"])
    o["matmul_backward_w"] = orc.matmul_backward_w(d["gy"], d["x"], 13, 21)
    o["matmul_backward_w_acc"] = orc.matmul_backward_w(d["gy"], d["x"], 13, 21, d["acc_w"])
    o["add_bias"] = orc.add_bias(d["gy"], d["b"])
    o["add_bias_backward_b"] = orc.add_bias_backward_b(d["gy"])
    o["add_bias_backward_b_acc"] = orc.add_bias_backward_b(d["gy"], d["b"])
    for act in range(9):  # 9 = softmax: the reference reads out of bounds there (vmath.cu:3145)
        o[f"activate_{act}"] = orc.activate(d["act_in"], act, 0.1)
        o[f"activate_backward_{act}"] = orc.activate_backward(d["act_gy"], d["act_in"], act, 0.1)
        if act <= 4:
            o[f"activate_backward_with_y_{act}"] = orc.activate_backward_with_y(d["act_gy"], d["act_in"], act, 0.1)
    pp = orc.mult_on_heads(d["k"], d["q"], 3, 0.5)
    o["mult_on_heads"] = pp
    o["mask_forward"] = orc.set_mh_attention_mask(pp, True)
    o["mask_backward"] = orc.set_mh_attention_mask(pp, False)
    o["softmax_axis"] = orc.softmax_direct_on_axis(pp)
    o["softmax_axis_masked"] = orc.softmax_direct_on_axis(o["mask_forward"])
    o["mix_values"] = orc.mix_values(o["softmax_axis"], d["v"], 3)
    # attention backward, chained as the engine does (api_objects/vtensor.cpp:3145-3154)
    gy = d["attn_gy"]
    o["mix_values_backward_value"] = orc.mix_values_backward_value(gy, o["softmax_axis"], 3)
    gp = orc.mix_values_backward_prop(gy, d["v"], 3)
    o["mix_values_backward_prop"] = gp
    gs = orc.softmax_direct_on_axis_backward(gp, o["softmax_axis"], 0.5)
    o["softmax_axis_backward"] = gs
    o["mult_on_heads_backward_q"] = orc.mult_on_heads_backward(gs, d["k"], 3)
    o["conv2d"] = orc.conv2d(d["conv_x"], d["conv_k"], 6, 5, 1, 1)
    o["conv2d_backward_x"] = orc.conv2d_backward_x(d["conv_gy"], d["conv_k"], 6, 5, 1, 1)
    # The host loop of conv2d_backward_k offsets columns by the output width instead of the padding
    # (vmath.cu:3676); the vector below comes from a case where the two agree (yw == pw == 1).
    o["conv2d_backward_k_w1"] = orc.conv2d_backward_k(d["conv_gy"][:, :, :, :1].copy(), d["conv_x"][:, :, :, :1].copy(),
                                                      3, 3, 1, 1)
    # transposed (stride 2) and dilated (gap 2) variants on the same 2 x 3 x 6 x 5 input, kernel [4][3][3][3]
    x, k = d["conv_x"], d["conv_k"]
    gy2 = np.tile(d["conv_gy"], (1, 1, 2, 2))                      # [2, 4, 12, 10]
    o["conv2d_transposed"] = orc.conv2d_variant("transposed", (2, 4, 12, 10), x, k, 2, 3, 6, 5, 4, 3, 3, 2, 2)
    o["conv2d_transposed_backward_x"] = orc.conv2d_variant("transposed_backward_x", (2, 3, 6, 5), gy2, k, 2, 3, 6, 5, 4, 3, 3, 2, 2)
    o["conv2d_transposed_backward_k"] = orc.conv2d_variant("transposed_backward_k", (4, 3, 3, 3), gy2, x, 2, 3, 6, 5, 4, 3, 3, 2, 2)
    o["conv2d_dilated"] = orc.conv2d_variant("dilated", (2, 4, 6, 5), x, k, 2, 3, 6, 5, 4, 3, 3, 2, 2)
    o["conv2d_dilated_backward_x"] = orc.conv2d_variant("dilated_backward_x", (2, 3, 6, 5), d["conv_gy"], k, 2, 3, 6, 5, 4, 3, 3, 2, 2)
    o["conv2d_dilated_backward_k"] = orc.conv2d_variant("dilated_backward_k", (4, 3, 3, 3), d["conv_gy"], x, 2, 3, 6, 5, 4, 3, 3, 2, 2)
    o["ce"] = orc.softmax_idx_crossentropy(d["logits"], d["labels"])
    o["ce_backward"] = orc.softmax_idx_crossentropy_backward_x(orc.sum_backward(8), d["logits"], d["labels"])
    o["sum"] = orc.sum(o["ce"])
    o["sum_backward_null"] = orc.sum_backward(8)
    o["sum_backward_val"] = orc.sum_backward(8, np.array([2.5], np.float32))
    o["layernorm"], o["layernorm_stat"] = orc.layernorm(d["ln_x"], 1.25)
    o["layernorm_backward"] = orc.layernorm_backward(d["ln_gy"], o["layernorm_stat"], 1.25)
    return o


if __name__ == "__main__":
    ref = oracle.Oracle("ref")
    out = compute(ref)
    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(out)} vectors)")
