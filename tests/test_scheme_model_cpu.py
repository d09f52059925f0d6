"""The arithmetic of the tensor-core GEMM's two MMA schemes, modelled in numpy (no GPU).

The kernels split every fp32 operand value a into hi = TF32(a) and lo = a - hi and form
a.b ~= hi.hi + (hi.lo + lo.hi); the lo.lo term is dropped.  For reductions of 2048 values and more the two
cross terms are computed from bf16 roundings of hi and lo (one BF16 MMA instead of two TF32 MMAs).  This file
pins the error model the dispatch rules rest on, with exact (fp64) accumulation so that only the split shows:

  * three TF32 products: ~3e-8 .. 8e-8 relative (Frobenius) -- far below a sequential fp32 sum
    (support/vmath.cu:2961-2977), whose error grows like 1.8e-8 * sqrt(K);
  * bf16 cross terms, hi rounded to nearest: ~5.6e-7, independent of K -- below the reference's own error from
    K = 2048 on (8.1e-7), which is where the scheme starts;
  * bf16 cross terms with a TRUNCATED hi (an operand read as its own hi plane): the lo part is twice as large
    and so is its rounding error -- fine for one operand at K >= 4096 (reference 1.15e-6), not for both at 2048.
"""
import numpy as np


def tf32_round(x: np.ndarray) -> np.ndarray:
    b = x.view(np.uint32).astype(np.uint64)
    return ((b + 0x1000) & 0xFFFFE000).astype(np.uint32).view(np.float32)


def tf32_trunc(x: np.ndarray) -> np.ndarray:
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    b = b + 0x7FFF + ((b >> 16) & 1)            # round to nearest, ties to even
    return (b & 0xFFFF0000).astype(np.uint32).view(np.float32)


def rel_fro(c, ref):
    return float(np.linalg.norm(c - ref) / np.linalg.norm(ref))


def products(a, b, hi_a, hi_b, cross_bf16):
    """hi.hi + hi.lo + lo.hi with the given high parts, accumulated exactly."""
    ah, bh = hi_a(a), hi_b(b)
    al, bl = a - ah, b - bh                      # exact in fp32
    d = np.float64
    main = ah.astype(d) @ bh.astype(d).T
    if cross_bf16:
        cross = bf16_round(ah).astype(d) @ bf16_round(bl).astype(d).T + bf16_round(al).astype(d) @ bf16_round(bh).astype(d).T
    else:
        cross = ah.astype(d) @ tf32_round(bl).astype(d).T + tf32_round(al).astype(d) @ bh.astype(d).T
    return main + cross


def inputs(kind, M, N, K, seed):
    rng = np.random.default_rng(seed)
    if kind == "uniform":
        a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    else:
        a = rng.standard_normal((M, K), dtype=np.float32)
        b = rng.standard_normal((N, K), dtype=np.float32)
    if kind == "full_mantissa":
        a = (a.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
        b = (b.view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    return a, b


def reference_error(K):
    return 1.8e-8 * np.sqrt(K)


def test_three_tf32_products_are_far_below_a_sequential_fp32_sum():
    for kind in ("uniform", "normal", "full_mantissa"):
        a, b = inputs(kind, 48, 48, 2048, 1)
        ref = a.astype(np.float64) @ b.astype(np.float64).T
        e = rel_fro(products(a, b, tf32_round, tf32_round, False), ref)
        assert e < 1.5e-7, (kind, e)


def test_bf16_cross_terms_stay_below_the_reference_from_2048_on():
    for K in (2048, 8192):
        for kind in ("uniform", "normal", "full_mantissa"):
            a, b = inputs(kind, 48, 48, K, 2)
            ref = a.astype(np.float64) @ b.astype(np.float64).T
            e = rel_fro(products(a, b, tf32_round, tf32_round, True), ref)
            assert e < 7.5e-7, (K, kind, e)
            assert e < reference_error(K), (K, kind, e)          # below the reference loop's own error
    # ... and not below it for short reductions, which is why those keep three TF32 products
    a, b = inputs("normal", 48, 48, 256, 3)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    assert rel_fro(products(a, b, tf32_round, tf32_round, True), ref) > reference_error(256)


def test_a_truncated_hi_plane_doubles_the_cross_term_error():
    """One operand read as its own hi plane (the tensor core truncates it): acceptable from K = 4096 on, where twice
    the reference's error is 2.3e-6; both operands that way at K = 2048 are not (2 x 8.1e-7)."""
    a, b = inputs("full_mantissa", 48, 48, 4096, 4)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    one_raw = rel_fro(products(a, b, tf32_trunc, tf32_round, True), ref)
    assert 8e-7 < one_raw < 1.5e-6, one_raw
    assert one_raw < 2 * reference_error(4096) - 6e-7              # room for the accumulation error on top
    a, b = inputs("full_mantissa", 48, 48, 2048, 5)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    both_raw = rel_fro(products(a, b, tf32_trunc, tf32_trunc, True), ref)
    assert both_raw > 2 * reference_error(2048)                    # the case the dispatch rule excludes
    rounded = rel_fro(products(a, b, tf32_round, tf32_round, True), ref)
    assert rounded < 1e-8                                          # such values round to hi exactly: lo = -2^-13 ulp steps
