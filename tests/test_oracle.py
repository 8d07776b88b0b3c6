"""The CPU oracle against everything that can pin it without the (unbuildable) reference.

1. The reference's own numeric test of this path: central finite differences (h=1e-4 there),
   max-abs error <= 1e-3 on a random [4,10] input (cgadimpl/Tests/test_core_ops_gpu.cpp:15-84
   and :262-267 for rms, :198-205 for broadcast mul incl. the reduced gradient, :228-233 rowsum,
   :216-227 sum / mean_all).
2. An independent second opinion: torch autograd in fp64 on CPU.
3. Internal consistency: op-by-op vs row-fused restatement, fp32 vs fp64 reductions,
   adjoint identity <gy, JVP(t)> == <VJP(gy), t> for the corrected JVP, and the size of the
   reference's literal-JVP deviation.
"""
import numpy as np
import pytest
import torch

import oracle_ffi as O
from inputs import assert_close, make_inputs


def _numgrad(f, a, h=1e-2):
    """test_core_ops_gpu.cpp:38-84: perturb one element at a time in fp32, central difference.

    Two deviations keep the check's own noise below its 1e-3 tolerance: the step is 1e-2 instead
    of 1e-4 (fp32 outputs carry ~1e-7 of rounding, and 1e-7 / 2e-4 is already ~1e-3, while the
    truncation error at h=1e-2 is ~1e-4), and the loss is summed in fp64."""
    a = a.astype(np.float32).copy()
    g = np.zeros_like(a)
    flat = a.reshape(-1)
    for i in range(flat.size):
        orig = flat[i]
        flat[i] = np.float32(orig + h)
        l1 = float(f(a).sum(dtype=np.float64))
        flat[i] = np.float32(orig - h)
        l2 = float(f(a).sum(dtype=np.float64))
        flat[i] = orig
        g.reshape(-1)[i] = (l1 - l2) / (2.0 * h)
    return g


@pytest.mark.parametrize("red", [O.RED_F32, O.RED_F64])
def test_reference_finite_difference_rms(red):
    rng = np.random.default_rng(1234)
    a = rng.standard_normal((4, 10)).astype(np.float32)
    ones = np.ones_like(a)
    ana = O.rmsnorm_fwd_bwd(a, None, ones, 1e-5, red)["dx"]     # backward(sum(rms(a)))
    num = _numgrad(lambda v: O.rmsnorm_fwd(v, None, 1e-5, red)[0], a)
    assert np.abs(ana - num).max() <= 1e-3                      # check_grad tol, :15


def test_reference_finite_difference_scaled_rms_and_broadcast_mul():
    rng = np.random.default_rng(7)
    a = rng.standard_normal((4, 5)).astype(np.float32)
    b = rng.standard_normal((5,)).astype(np.float32)
    ones = np.ones_like(a)
    out = O.rmsnorm_fwd_bwd(a, b, ones, 1e-5)
    num_a = _numgrad(lambda v: O.rmsnorm_fwd(v, b, 1e-5)[0], a)
    num_b = _numgrad(lambda v: O.rmsnorm_fwd(a, v, 1e-5)[0], b)
    assert np.abs(out["dx"] - num_a).max() <= 1e-3
    assert np.abs(out["dgamma"] - num_b).max() <= 1e-3


def test_reference_finite_difference_reductions():
    rng = np.random.default_rng(9)
    a = rng.standard_normal((4, 5)).astype(np.float32)
    # d sum(rowsum(a)) / da == 1, d sum(a)/da == 1, d mean_all(a)/da == 1/N
    assert np.abs(_numgrad(lambda v: O.rowsum(v), a) - 1.0).max() <= 1e-3
    assert np.abs(_numgrad(lambda v: np.array([O.total_sum(v)], np.float32), a) - 1.0).max() <= 1e-3
    assert np.abs(_numgrad(lambda v: np.array([O.mean_all(v)], np.float32), a) - 1.0 / a.size).max() <= 1e-3


def _torch_ref(x, gamma, gy, eps):
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    gt = None if gamma is None else torch.tensor(gamma, dtype=torch.float64, requires_grad=True)
    rstd = torch.rsqrt((xt * xt).mean(-1, keepdim=True) + eps)
    y = xt * rstd
    if gt is not None:
        y = y * gt
    y.backward(torch.tensor(gy, dtype=torch.float64))
    return (y.detach().numpy(), rstd.detach().numpy()[:, 0], xt.grad.numpy(),
            None if gt is None else gt.grad.numpy())


@pytest.mark.parametrize("rows,hidden,eps,with_gamma", [
    (4096, 1024, 1e-6, True),      # benchmark configuration 1 (CPU-runnable)
    (33, 1000, 1e-6, True),
    (7, 4096, 1e-5, True),
    (5, 10, 1e-5, False),
    (1, 1, 1e-5, True),
])
def test_against_torch_fp64(rows, hidden, eps, with_gamma):
    x, gamma, gy = make_inputs(rows, hidden, seed=0)
    if not with_gamma:
        gamma = None
    out = O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F64)
    y, rstd, dx, dg = _torch_ref(x, gamma, gy, eps)
    # elementwise fp32 rounding noise only: a few 1e-7 relative
    assert_close(out["y"], y, 1e-6, 1e-7, "y")
    assert_close(out["rstd"], rstd, 1e-6, 0, "rstd")
    assert_close(out["dx"], dx, 2e-6, 2e-6, "dx")
    if with_gamma:
        # each product gy*yhat is rounded to fp32 before the (fp64) column sum: noise ~ sqrt(R)*6e-8
        scale = float(np.sqrt(rows))
        assert np.abs(out["dgamma"] - dg).max() <= 4e-7 * scale * 4 + 1e-6


def test_fused_restatement_matches_op_by_op_bitwise():
    x, gamma, gy = make_inputs(257, 1000, seed=3)
    a = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-6, O.RED_F64)
    b = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-6, fused=True)
    for k in ("y", "rstd", "dx"):
        assert np.array_equal(a[k], b[k]), k
    # dgamma: fused variant combines per-thread fp64 partials; may differ in the last fp32 bit
    assert np.abs(a["dgamma"].view(np.int32) - b["dgamma"].view(np.int32)).max() <= 1


def test_fp32_vs_fp64_reduction_modes_bound_the_reference():
    """How far apart two legitimate fp32 implementations can be: this is the noise floor that any
    comparison with the real (fp32, unknown summation order) reference would have."""
    x, gamma, gy = make_inputs(4096, 1024, seed=0)
    a = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-6, O.RED_F32)
    b = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-6, O.RED_F64)
    assert_close(a["y"], b["y"], 1e-5, 1e-6, "y")
    assert_close(a["dx"], b["dx"], 1e-5, 1e-6, "dx")
    # dgamma: an fp32 left-to-right sum over 4096 rows drifts by several 1e-4 absolute (values ~60),
    # i.e. far outside rel 1e-5 / abs 1e-6 -- two fp32 summation orders cannot agree elementwise to
    # that tolerance, which is why the fp64-reduced result is the arbiter.  Norm-wise they agree.
    d = np.abs(a["dgamma"] - b["dgamma"]).max()
    assert 1e-6 < d < 5e-3
    assert np.linalg.norm(a["dgamma"] - b["dgamma"]) / np.linalg.norm(b["dgamma"]) < 2e-5


def test_bf16_wrapper_rounds_once():
    x, gamma, gy = make_inputs(64, 1000, seed=5, x_std=3.0, gamma_std=0.1, outlier_frac=0.05)
    xb, gb, gyb = O.f32_to_bf16_bits(x), O.f32_to_bf16_bits(gamma), O.f32_to_bf16_bits(gy)
    out = O.rmsnorm_fwd_bwd_bf16(xb, gb, gyb, 1e-6)
    ref = O.rmsnorm_fwd_bwd(O.bf16_bits_to_f32(xb), O.bf16_bits_to_f32(gb), O.bf16_bits_to_f32(gyb), 1e-6)
    assert np.array_equal(out["y"], O.f32_to_bf16_bits(ref["y"]))
    assert np.array_equal(out["dx"], O.f32_to_bf16_bits(ref["dx"]))
    assert np.array_equal(out["rstd"], ref["rstd"])
    assert np.array_equal(out["dgamma"], ref["dgamma"])
    # bf16 helpers agree with torch's conversion
    t = torch.tensor(x).to(torch.bfloat16)
    assert np.array_equal(t.view(torch.int16).numpy().view(np.uint16), xb)


def test_corrected_jvp_adjoint_identity_and_literal_deviation():
    rows, hidden, eps = 16, 256, 1e-5
    x, gamma, gy = make_inputs(rows, hidden, seed=11)
    t = np.random.default_rng(5).standard_normal((rows, hidden)).astype(np.float32)
    yhat, rstd = O.rmsnorm_fwd(x, None, eps)
    jv = O.jvp_rms(t, yhat, rstd, corrected=True)
    vj = O.rmsnorm_fwd_bwd(x, None, gy, eps)["dx"]
    lhs = float((gy.astype(np.float64) * jv).sum())
    rhs = float((vj.astype(np.float64) * t).sum())
    assert abs(lhs - rhs) <= 1e-5 * max(1.0, abs(lhs))
    # directional finite difference
    h = 1e-3
    yp, _ = O.rmsnorm_fwd(x + h * t, None, eps)
    ym, _ = O.rmsnorm_fwd(x - h * t, None, eps)
    assert np.abs((yp - ym) / (2 * h) - jv).max() < 2e-3
    # the reference's literal formula is off by exactly 1/rstd^2 = mean(x^2)+eps per row
    lit = O.jvp_rms(t, yhat, rstd, corrected=False)
    ratio = lit / jv
    want = (1.0 / (rstd.astype(np.float64) ** 2))[:, None]
    ok = np.abs(jv) > 1e-3
    assert np.allclose(ratio[ok], np.broadcast_to(want, ratio.shape)[ok], rtol=1e-3)
    # with gamma: JVP of mul(rms(x), gamma)
    tg = np.random.default_rng(6).standard_normal(hidden).astype(np.float32)
    full = O.rmsnorm_jvp(x, gamma, t, tg, eps)
    want_full = jv * gamma + yhat * tg
    assert_close(full, want_full, 1e-6, 1e-6, "jvp with gamma")


def test_row_and_global_reductions():
    x = np.random.default_rng(2).standard_normal((37, 1000)).astype(np.float32)
    assert_close(O.rowsum(x), x.astype(np.float64).sum(-1), 1e-6, 1e-6, "rowsum")
    assert np.array_equal(O.rowmax(x), x.max(-1))
    assert abs(O.total_sum(x) - x.astype(np.float64).sum()) < 1e-3
    assert abs(O.mean_all(x) - x.astype(np.float64).mean()) < 1e-6
    assert_close(O.colsum(x), x.astype(np.float64).sum(0), 1e-6, 1e-6, "colsum")


def test_residual_stack_matches_torch_fp64():
    R, H, L, eps = 24, 128, 6, 1e-6
    rng = np.random.default_rng(0)
    x = rng.standard_normal((R, H)).astype(np.float32)
    r = rng.standard_normal((R, H)).astype(np.float32)
    g = rng.standard_normal((R, H)).astype(np.float32)
    gam = (1 + 0.02 * rng.standard_normal((L, H))).astype(np.float32)
    out = O.residual_stack(x, r, gam, g, eps)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    rt = torch.tensor(r, dtype=torch.float64, requires_grad=True)
    gt = torch.tensor(gam, dtype=torch.float64, requires_grad=True)
    xl, rl = xt, rt
    for l in range(L):
        h = xl + rl
        y = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * gt[l]
        xl, rl = h, y
    y.backward(torch.tensor(g, dtype=torch.float64))
    assert_close(out["y"], y.detach().numpy(), 1e-5, 1e-6, "y_last")
    assert_close(out["dh0"], xt.grad.numpy(), 1e-5, 1e-5, "dx0")
    assert_close(out["dh0"], rt.grad.numpy(), 1e-5, 1e-5, "dr0")
    assert_close(out["dgammas"], gt.grad.numpy(), 1e-4, 1e-5, "dgammas")


def test_layernorm_against_torch_fp64_and_finite_differences():
    rows, hidden, eps = 37, 1000, 1e-5
    x, _, gy = make_inputs(rows, hidden, seed=8)
    x = x * np.float32(1.5) + np.float32(0.3)
    out = O.layernorm_fwd_bwd(x, gy, eps)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    y = torch.nn.functional.layer_norm(xt, (hidden,), eps=eps)
    y.backward(torch.tensor(gy, dtype=torch.float64))
    assert_close(out["y"], y.detach().numpy(), 2e-6, 2e-6, "y")
    assert_close(out["dx"], xt.grad.numpy(), 1e-4, 2e-5, "dx")     # the reference's formula cancels heavily
    # the reference's own check: finite differences on [4,10] at 1e-3 (test_core_ops_gpu.cpp:256-261)
    a = np.random.default_rng(3).standard_normal((4, 10)).astype(np.float32)
    ana = O.layernorm_fwd_bwd(a, np.ones_like(a), eps)["dx"]
    num = _numgrad(lambda v: O.layernorm_fwd_bwd(v, np.ones_like(v), eps)["y"], a)
    assert np.abs(ana - num).max() <= 1e-3


def test_layernorm_jvp_definition_against_torch_fp64_and_the_adjoint_identity():
    """The reference's jvp_LayerNorm throws, so the JVP is this library's own definition: it must be the
    directional derivative of the pinned forward and the adjoint of the pinned VJP."""
    rows, hidden, eps = 29, 1000, 1e-5
    x, _, gy = make_inputs(rows, hidden, seed=12)
    x = x * np.float32(1.5) + np.float32(0.3)
    t = np.random.default_rng(13).standard_normal((rows, hidden)).astype(np.float32)
    out = O.layernorm_fwd_bwd(x, gy, eps)
    ty = O.layernorm_jvp(out["y"], t, out["var"], eps)
    xt = torch.tensor(x, dtype=torch.float64)
    _, want = torch.func.jvp(lambda v: torch.nn.functional.layer_norm(v, (hidden,), eps=eps), (xt,),
                             (torch.tensor(t, dtype=torch.float64),))
    assert_close(ty, want.numpy(), 1e-5, 2e-6, "ty")
    lhs = float((gy.astype(np.float64) * ty).sum())
    rhs = float((out["dx"].astype(np.float64) * t).sum())
    assert abs(lhs - rhs) <= 1e-4 * max(1.0, abs(lhs))
