"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations."""
import numpy as np


def make_inputs(rows, hidden, seed=0, x_std=1.0, gamma_std=0.02, outlier_frac=0.0, outlier_scale=100.0):
    """x ~ N(0, x_std), gamma = 1 + gamma_std*N(0,1), gy ~ N(0,1); independent streams per array.

    With outlier_frac > 0 a seeded fraction of rows of x is multiplied by outlier_scale.
    """
    sx, sg, sgy, so = np.random.SeedSequence(seed).spawn(4)
    x = (np.random.default_rng(sx).standard_normal((rows, hidden), dtype=np.float32) * np.float32(x_std))
    gamma = (1.0 + gamma_std * np.random.default_rng(sg).standard_normal(hidden)).astype(np.float32)
    gy = np.random.default_rng(sgy).standard_normal((rows, hidden), dtype=np.float32)
    if outlier_frac > 0:
        k = max(1, int(round(rows * outlier_frac)))
        idx = np.random.default_rng(so).choice(rows, size=k, replace=False)
        x[idx] *= np.float32(outlier_scale)
    return x, gamma, gy


def fp32_accum_dgamma_tol(rows):
    """(rtol, atol) for a dgamma whose column sums were ACCUMULATED IN FP32 (the 16-bit-I/O kernels).
    A column is a sum of `rows` products of O(1); each fp32 product and addition carries a relative
    rounding error of 2^-24, so the sum of a column that cancels to almost zero is still uncertain by
    about sqrt(rows) * 2^-24 * (a few): no relative bound can hold there, hence the floor grows like
    sqrt(rows).  Columns of typical size (~sqrt(rows)) are held to 1e-5 relative."""
    return 1e-5, 4e-6 * float(np.sqrt(max(rows, 1)))


def assert_close(a, b, rtol, atol, what=""):
    """|a-b| <= atol + rtol*|b| elementwise, with a readable failure."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    err = np.abs(a - b)
    tol = atol + rtol * np.abs(b)
    bad = err > tol
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), a.shape)
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{a.size} outside rtol={rtol} atol={atol}; worst at {i}: "
            f"got {a[i]!r} want {b[i]!r} err {err[i]:.3e} tol {tol[i]:.3e}")
