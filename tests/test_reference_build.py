"""The oracle against the REFERENCE'S OWN CODE.

oracle/_ref/libcgadimpl_ref.so is built from the reference's unmodified sources for this path
(rms_nodeops, mul_nodeops, add_nodeops, the reduction builders, backward / jvp and every VJP / JVP
rule -- cgadimpl/src/{core,ops,autodiff}) over a CPU stand-in for its absent tensor library.  Running
it pins the reference's composition: the oracle must reproduce it bit for bit when both use the same
reduction arithmetic.  What stays unpinned is the arithmetic inside the real OwnTensor library.
Skipped where the library has not been built (needs the reference tree)."""
import numpy as np
import pytest

import oracle_ffi as O
import ref_ffi as REF
from inputs import make_inputs

pytestmark = pytest.mark.skipif(not REF.available(), reason="reference build not available")


@pytest.mark.parametrize("fp64", [False, True])
@pytest.mark.parametrize("rows,hidden,with_gamma,gamma_2d", [(4, 10, False, False), (64, 1024, True, False),
                                                             (33, 1000, True, True), (256, 4096, True, False)])
def test_oracle_reproduces_reference_composition_bitwise(fp64, rows, hidden, with_gamma, gamma_2d):
    x, gamma, gy = make_inputs(rows, hidden, seed=rows + hidden)
    if not with_gamma:
        gamma = None
    REF.set_reduce_fp64(fp64)
    ref = REF.rmsnorm_fwd_bwd(x, gamma, gy, gamma_2d=gamma_2d)
    mine = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-5, O.RED_F64 if fp64 else O.RED_F32)
    for k in ("y", "rstd", "dx") + (("dgamma",) if with_gamma else ()):
        assert np.array_equal(ref[k], mine[k]), f"{k}: the restatement departs from the reference's own code"


def test_reference_parallel_backward_matches_sequential():
    x, gamma, gy = make_inputs(32, 256, seed=1)
    REF.set_reduce_fp64(True)
    a = REF.rmsnorm_fwd_bwd(x, gamma, gy, parallel=False)
    b = REF.rmsnorm_fwd_bwd(x, gamma, gy, parallel=True)
    for k in ("y", "dx", "dgamma"):
        assert np.array_equal(a[k], b[k]), k


@pytest.mark.parametrize("fp64", [False, True])
def test_oracle_residual_stack_matches_reference_graph(fp64):
    R, H, L = 24, 128, 4
    rng = np.random.default_rng(0)
    x, r, g = (rng.standard_normal((R, H)).astype(np.float32) for _ in range(3))
    gam = (1 + 0.02 * rng.standard_normal((L, H))).astype(np.float32)
    REF.set_reduce_fp64(fp64)
    ref = REF.residual_stack(x, r, gam, g)
    mine = O.residual_stack(x, r, gam, g, 1e-5, O.RED_F64 if fp64 else O.RED_F32)
    assert np.array_equal(ref["y"], mine["y"])
    assert np.array_equal(ref["dx0"], mine["dh0"]) and np.array_equal(ref["dr0"], mine["dh0"])
    assert np.array_equal(ref["dgammas"], mine["dgammas"])


def test_reference_jvp_is_the_literal_form_and_is_off_by_rstd_squared():
    rows, hidden = 16, 256
    x, _, _ = make_inputs(rows, hidden, seed=2)
    t = np.random.default_rng(3).standard_normal((rows, hidden)).astype(np.float32)
    REF.set_reduce_fp64(True)
    ref = REF.rms_jvp(x, t)
    # through ag::jvp the seed never reaches the rule: jvp_Leaf's "unused" empty tensor replaces it
    assert not np.any(REF.rms_jvp(x, t, via_engine=True))
    yhat, rstd = O.rmsnorm_fwd(x, None, 1e-5)
    assert np.array_equal(ref, O.jvp_rms(t, yhat, rstd, corrected=False))        # the oracle's literal form IS the reference's
    good = O.jvp_rms(t, yhat, rstd, corrected=True)
    ok = np.abs(good) > 1e-3
    ratio = (ref / good)[ok]
    want = np.broadcast_to((1.0 / rstd.astype(np.float64) ** 2)[:, None], ref.shape)[ok]
    assert np.allclose(ratio, want, rtol=1e-3)                                    # wrong by exactly 1/rstd^2 per row
    # and the correct form is the one that matches finite differences
    h = 1e-3
    fd = (O.rmsnorm_fwd(x + h * t, None, 1e-5)[0] - O.rmsnorm_fwd(x - h * t, None, 1e-5)[0]) / (2 * h)
    assert np.abs(fd - good).max() < 2e-3 < np.abs(fd - ref).max()


@pytest.mark.parametrize("fp64", [False, True])
def test_oracle_reductions_match_reference(fp64):
    x = np.random.default_rng(4).standard_normal((37, 1000)).astype(np.float32)
    REF.set_reduce_fp64(fp64)
    red = O.RED_F64 if fp64 else O.RED_F32
    out, dx = REF.reduction("rowsum", x)
    assert np.array_equal(out, O.rowsum(x, red)) and np.array_equal(dx, np.ones_like(x))
    out, _ = REF.reduction("rowmax", x)
    assert np.array_equal(out, O.rowmax(x))
    out, dx = REF.reduction("sum", x)
    assert out[0] == np.float32(O.total_sum(x, red)) and np.array_equal(dx, np.ones_like(x))
    out, dx = REF.reduction("mean_all", x)
    assert out[0] == np.float32(O.mean_all(x, red))
    assert np.array_equal(dx, np.full_like(x, np.float32(1.0) / np.float32(x.size)))


def test_oracle_optimizer_steps_match_reference_optim_cpp():
    rng = np.random.default_rng(5)
    n, steps = 1000, 7
    p0 = (1 + 0.02 * rng.standard_normal(n)).astype(np.float32)
    grads = rng.standard_normal((steps, n)).astype(np.float32)
    want = REF.optimizer("sgd", p0, grads, 1e-2)
    p = p0.copy()
    for g in grads:
        p = O.sgd_step(p, g, 1e-2)
    assert np.array_equal(p, want)
    want = REF.optimizer("adam", p0, grads, 1e-3)
    p, m, v = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t, g in enumerate(grads, 1):
        p, m, v = O.adam_step(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, t)
    assert np.array_equal(p, want)


@pytest.mark.parametrize("fp64", [False, True])
@pytest.mark.parametrize("rows,hidden", [(4, 10), (64, 1024), (33, 1000)])
def test_oracle_layernorm_matches_reference_bitwise(fp64, rows, hidden):
    x, _, gy = make_inputs(rows, hidden, seed=rows * 3 + hidden)
    x = x + np.float32(0.5)                      # a non-zero mean makes the mean path matter
    REF.set_reduce_fp64(fp64)
    ref = REF.layernorm_fwd_bwd(x, gy)
    mine = O.layernorm_fwd_bwd(x, gy, 1e-5, O.RED_F64 if fp64 else O.RED_F32)
    for k in ("y", "mean", "var", "dx"):
        assert np.array_equal(ref[k], mine[k]), k


def _logits(rows, hidden, seed):
    """Logit-like rows: N(0, 3) with a masked tail (-1e4) on some rows and one dominant entry on others."""
    rng = np.random.default_rng(seed)
    z = (3.0 * rng.standard_normal((rows, hidden))).astype(np.float32)
    z[::3, hidden // 2:] = np.float32(-1e4)
    z[1::5, 0] = np.float32(60.0)
    return z


@pytest.mark.parametrize("fp64", [False, True])
@pytest.mark.parametrize("rows,hidden", [(4, 10), (64, 1024), (33, 1000)])
def test_oracle_softmax_and_logsumexp_match_reference_bitwise(fp64, rows, hidden):
    z = _logits(rows, hidden, seed=rows + hidden)
    rng = np.random.default_rng(5)
    gy = rng.standard_normal((rows, hidden)).astype(np.float32)
    gy_row = rng.standard_normal(rows).astype(np.float32)
    t = rng.standard_normal((rows, hidden)).astype(np.float32)
    REF.set_reduce_fp64(fp64)
    red = O.RED_F64 if fp64 else O.RED_F32
    ref = REF.softmax_family("softmax", z, gy, t)
    y = O.softmax_row(z, red)
    assert np.array_equal(ref["y"], y)
    assert np.array_equal(ref["dz"], O.softmax_row_vjp(y, gy, red))
    assert np.array_equal(ref["ty"], O.softmax_row_vjp(y, t, red))
    ref = REF.softmax_family("logsumexp", z, gy_row, t)
    assert np.array_equal(ref["y"], O.logsumexp_row(z, red))
    assert np.array_equal(ref["dz"], O.logsumexp_row_vjp(z, gy_row, red))
    assert np.array_equal(ref["ty"], O.logsumexp_row_jvp(z, t, red))
    # sanity against a float64 computation
    z64 = z.astype(np.float64)
    e = np.exp(z64 - z64.max(-1, keepdims=True))
    np.testing.assert_allclose(y, e / e.sum(-1, keepdims=True), rtol=2e-6, atol=1e-9)
    np.testing.assert_allclose(ref["y"], np.log(e.sum(-1)) + z64.max(-1), rtol=1e-6, atol=1e-6)
