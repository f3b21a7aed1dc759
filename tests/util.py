"""Shared helpers of the parity tests: seeded inputs of the benchmark configurations and the
comparison rules (bit-exact for extrema / indices / top-k, float64-anchored tolerance for
sum / mean / var / std)."""
from __future__ import annotations

import numpy as np

# Tolerances (float32 results):
#   accuracy:   |gpu - truth64| <= REL * |truth64|                      (sum, mean, var, std)
#   agreement:  |gpu - reference| <= REL * |truth64| + COND * sum|x|   (sum, mean)
# The second form exists because the reference's own dim-sum accumulates sequentially in float32
# and itself misses REL on near-zero sums (its error is bounded by ~2e-7 * sum|x|).
REL = 1e-5
COND = 1e-6


def config1(rows=4096, cols=4096):
    return np.random.default_rng(0).standard_normal((rows, cols), dtype=np.float32)


def config2(rows=256, cols=151936):
    rng = np.random.default_rng(1)
    x = rng.normal(0.0, 2.0, (rows, cols)).astype(np.float32)
    for r in range(rows):
        x[r, rng.choice(cols, 64, replace=False)] = np.float32(8.0)
    return x


def config3(a=64, b=4096, c=512):
    return np.random.default_rng(2).uniform(-1.0, 1.0, (a, b, c)).astype(np.float32)


def config4(n=1 << 31, chunk=1 << 24):
    """Flat uniform(-1,1) with 1% of positions set to +-1e4, generated chunk by chunk."""
    rng = np.random.default_rng(3)
    out = np.empty(n, dtype=np.float32)
    for s in range(0, n, chunk):
        m = min(chunk, n - s)
        v = rng.uniform(-1.0, 1.0, m).astype(np.float32)
        pos = rng.choice(m, max(1, m // 100), replace=False)
        v[pos] = np.where(rng.integers(0, 2, pos.size) == 0, np.float32(1e4), np.float32(-1e4))
        out[s:s + m] = v
    return out


_config5_cache = {}


def config5(rows=512, cols=1 << 20):
    """Integers 0..999 as float (tie-heavy).  The full-size array (2 GiB) is kept for the second test
    that asks for it; generated block by block so that the int64 draw never exists whole."""
    key = (rows, cols)
    if key not in _config5_cache:
        rng = np.random.default_rng(4)
        if rows * cols <= (1 << 26):
            x = rng.integers(0, 1000, (rows, cols)).astype(np.float32)
        else:
            x = np.empty((rows, cols), dtype=np.float32)
            step = max(1, (1 << 26) // cols)
            for r in range(0, rows, step):
                x[r:r + step] = rng.integers(0, 1000, (min(step, rows - r), cols))
        _config5_cache.clear()
        _config5_cache[key] = x
    return _config5_cache[key]


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bits_equal(got: np.ndarray, want: np.ndarray, what=""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    g, w = bits(got), bits(want)
    if not np.array_equal(g, w):
        bad = np.flatnonzero(g.ravel() != w.ravel())
        i = bad[0]
        raise AssertionError(f"{what}: {bad.size} value(s) differ bitwise; first at {i}: "
                             f"{got.ravel()[i]!r} vs {want.ravel()[i]!r}")


def assert_index_equal(got: np.ndarray, want: np.ndarray, what=""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert got.dtype == np.int64
    if not np.array_equal(got, want):
        bad = np.flatnonzero(got.ravel() != want.ravel())
        i = bad[0]
        raise AssertionError(f"{what}: {bad.size} index(es) differ; first at {i}: {got.ravel()[i]} vs {want.ravel()[i]}")


def assert_close64(got: np.ndarray, truth: np.ndarray, what="", rel=REL):
    got = np.asarray(got, dtype=np.float64)
    truth = np.asarray(truth, dtype=np.float64)
    assert got.shape == truth.shape, f"{what}: shape {got.shape} != {truth.shape}"
    both_nan = np.isnan(got) & np.isnan(truth)
    same_inf = np.isinf(truth) & (got == truth)
    fin = ~(both_nan | same_inf)
    err = np.abs(got[fin] - truth[fin])
    tol = rel * np.abs(truth[fin]) + 1e-38
    if not np.all(err <= tol):
        j = int(np.argmax(err - tol))
        raise AssertionError(f"{what}: |gpu - float64| = {err[j]:.3e} > {tol[j]:.3e} "
                             f"(gpu {got[fin][j]!r}, float64 {truth[fin][j]!r})")


def assert_agrees(got, ref, truth, abs_sum, what=""):
    """Condition-aware agreement between the GPU and the reference for sum / mean."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    truth = np.asarray(truth, dtype=np.float64)
    abs_sum = np.asarray(abs_sum, dtype=np.float64)
    fin = np.isfinite(ref) & np.isfinite(got)
    assert np.array_equal(np.isnan(got), np.isnan(ref)), f"{what}: NaN pattern differs"
    err = np.abs(got - ref)[fin]
    tol = (REL * np.abs(truth) + COND * abs_sum)[fin] + 1e-38
    if not np.all(err <= tol):
        j = int(np.argmax(err - tol))
        raise AssertionError(f"{what}: |gpu - reference| = {err[j]:.3e} > {tol[j]:.3e}")
