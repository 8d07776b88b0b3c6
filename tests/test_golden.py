"""Golden vectors (tests/golden/*.npz, made by tests/golden/make_golden.py from the oracle).

CPU: the oracle still reproduces them bit for bit, and they agree with a torch fp64 computation.
GPU: the CUDA path, called through the C ABI, reproduces them within the stated tolerance
(fp32 rel 1e-5 / abs 1e-6, bf16 I/O rel 2e-2) -- in practice bit for bit."""
import glob
import os

import numpy as np
import pytest
import torch

import oracle_ffi as O
from inputs import assert_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def test_fixture_set_is_complete():
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "*.npz")))
    assert names == ["bf16_16x256_outliers", "fp32_4x10_plain", "fp32_5x1000", "fp32_8x64", "jvp_8x64",
                     "ref_layernorm_6x48", "ref_logsumexp_6x40", "ref_optim_64", "ref_rms_plain_6x48", "ref_rmsnorm_6x48",
                     "ref_softmax_6x40", "ref_stack_5x32x3", "stack_6x32x3"]


@pytest.mark.parametrize("name", ["fp32_8x64", "fp32_4x10_plain", "fp32_5x1000"])
def test_oracle_reproduces_fp32_golden_and_matches_fp64(name):
    c = load(name)
    gamma = c.get("gamma")
    out = O.rmsnorm_fwd_bwd(c["x"], gamma, c["gy"], float(c["eps"]))
    for k in ("y", "rstd", "dx") + (("dgamma",) if gamma is not None else ()):
        assert np.array_equal(out[k], c[k]), k
    x = torch.tensor(c["x"], dtype=torch.float64, requires_grad=True)
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + float(c["eps"]))
    if gamma is not None:
        y = y * torch.tensor(gamma, dtype=torch.float64)
    y.backward(torch.tensor(c["gy"], dtype=torch.float64))
    assert_close(c["y"], y.detach().numpy(), 1e-6, 1e-7, "y vs fp64")
    assert_close(c["dx"], x.grad.numpy(), 2e-6, 2e-6, "dx vs fp64")


def test_oracle_reproduces_other_golden():
    c = load("bf16_16x256_outliers")
    out = O.rmsnorm_fwd_bwd_bf16(c["x"], c["gamma"], c["gy"], float(c["eps"]))
    for k in ("y", "rstd", "dx", "dgamma"):
        assert np.array_equal(out[k], c[k]), k
    c = load("jvp_8x64")
    assert np.array_equal(O.rmsnorm_jvp(c["x"], c["gamma"], c["tx"], c["tgamma"], float(c["eps"])), c["ty"])
    c = load("stack_6x32x3")
    out = O.residual_stack(c["x"], c["r"], c["gammas"], c["g"], float(c["eps"]))
    assert np.array_equal(out["y"], c["y"]) and np.array_equal(out["dh0"], c["dh0"])
    assert np.array_equal(out["dgammas"], c["dgammas"])


def test_oracle_reproduces_the_reference_builds_vectors_bitwise():
    """ref_*.npz hold outputs of the reference's own code (tests/golden/make_reference_golden.py); they pin the
    oracle on machines without the reference tree."""
    eps = 1e-5
    c = load("ref_rmsnorm_6x48")
    out = O.rmsnorm_fwd_bwd(c["x"], c["gamma"], c["gy"], eps)
    for k in ("y", "rstd", "dx", "dgamma"):
        assert np.array_equal(out[k], c[k]), k
    c = load("ref_rms_plain_6x48")
    out = O.rmsnorm_fwd_bwd(c["x"], None, c["gy"], eps)
    for k in ("y", "rstd", "dx"):
        assert np.array_equal(out[k], c[k]), k
    c = load("ref_stack_5x32x3")
    out = O.residual_stack(c["x"], c["r"], c["gammas"], c["g"], eps)
    assert np.array_equal(out["y"], c["y"]) and np.array_equal(out["dgammas"], c["dgammas"])
    assert np.array_equal(out["dh0"], c["dx0"]) and np.array_equal(out["dh0"], c["dr0"])
    c = load("ref_layernorm_6x48")
    out = O.layernorm_fwd_bwd(c["x"], c["gy"], eps)
    for k in ("y", "mean", "var", "dx"):
        assert np.array_equal(out[k], c[k]), k
    c = load("ref_softmax_6x40")
    y = O.softmax_row(c["z"])
    assert np.array_equal(y, c["y"])
    assert np.array_equal(O.softmax_row_vjp(y, c["gy"]), c["dz"]) and np.array_equal(O.softmax_row_vjp(y, c["t"]), c["ty"])
    c = load("ref_logsumexp_6x40")
    assert np.array_equal(O.logsumexp_row(c["z"]), c["y"])
    assert np.array_equal(O.logsumexp_row_vjp(c["z"], c["gy"]), c["dz"])
    assert np.array_equal(O.logsumexp_row_jvp(c["z"], c["t"]), c["ty"])
    c = load("ref_optim_64")
    p = c["p0"].copy()
    for g in c["grads"]:
        p = O.sgd_step(p, g, 1e-2)
    assert np.array_equal(p, c["sgd"])
    p, m, v = c["p0"].copy(), np.zeros(64, np.float32), np.zeros(64, np.float32)
    for t, g in enumerate(c["grads"], 1):
        p, m, v = O.adam_step(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, t)
    assert np.array_equal(p, c["adam"])


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["fp32_8x64", "fp32_4x10_plain", "fp32_5x1000"])
def test_cuda_reproduces_fp32_golden(name):
    from cgadimpl_b200 import ops

    c = load(name)
    gamma = None if "gamma" not in c else _dev(c["gamma"])
    x, gy = _dev(c["x"]), _dev(c["gy"])
    y, rstd = ops.rmsnorm_fwd(x, gamma, float(c["eps"]))
    dx, dg = ops.rmsnorm_bwd(x, gamma, rstd, gy)
    for k, got in (("y", y), ("rstd", rstd), ("dx", dx)) + ((("dgamma", dg),) if gamma is not None else ()):
        assert_close(got.cpu().numpy(), c[k], 1e-5, 1e-6, k)
        assert np.array_equal(got.cpu().numpy(), c[k]), f"{k}: not bit-identical on a tiny case"


@pytest.mark.gpu
def test_cuda_reproduces_bf16_jvp_and_stack_golden():
    from cgadimpl_b200 import ops

    c = load("bf16_16x256_outliers")
    bf = torch.bfloat16
    x, gamma, gy = _dev(c["x"].view(np.int16), bf), _dev(c["gamma"].view(np.int16), bf), _dev(c["gy"].view(np.int16), bf)
    # default for 16-bit I/O: fp32 accumulation, held to the bf16 tolerance
    y, rstd = ops.rmsnorm_fwd(x, gamma, float(c["eps"]))
    dx, dg = ops.rmsnorm_bwd(x, gamma, rstd, gy)
    assert_close(y.float().cpu().numpy(), O.bf16_bits_to_f32(c["y"]), 2e-2, 1e-6, "y")
    assert_close(dx.float().cpu().numpy(), O.bf16_bits_to_f32(c["dx"]), 2e-2, 1e-6, "dx")
    assert_close(rstd.cpu().numpy(), c["rstd"], 1e-5, 0, "rstd")
    assert_close(dg.cpu().numpy(), c["dgamma"], 1e-5, 4e-6 * 4, "dgamma (fp32-accumulated over 16 rows)")
    # the strictly rounded kernels reproduce the stored bits
    ops.set_option("bf16_strict", 1)
    try:
        y, rstd = ops.rmsnorm_fwd(x, gamma, float(c["eps"]))
        dx, dg = ops.rmsnorm_bwd(x, gamma, rstd, gy)
    finally:
        ops.set_option("bf16_strict", 0)
    assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), c["y"])
    assert np.array_equal(rstd.cpu().numpy(), c["rstd"]) and np.array_equal(dg.cpu().numpy(), c["dgamma"])
    c = load("jvp_8x64")
    x, gamma = _dev(c["x"]), _dev(c["gamma"])
    _, rstd = ops.rmsnorm_fwd(x, gamma, float(c["eps"]))
    ty = ops.rmsnorm_jvp(x, gamma, rstd, _dev(c["tx"]), _dev(c["tgamma"]))
    assert_close(ty.cpu().numpy(), c["ty"], 1e-5, 1e-6, "ty")
    c = load("stack_6x32x3")
    xl, rl, gam = _dev(c["x"]), _dev(c["r"]), _dev(c["gammas"])
    hs, rs = [], []
    for l in range(gam.shape[0]):
        h, y, rstd = ops.add_rmsnorm_fwd(xl, rl, gam[l], float(c["eps"]))
        hs.append(h)
        rs.append(rstd)
        xl, rl = h, y
    assert_close(y.cpu().numpy(), c["y"], 1e-5, 1e-6, "y_last")
    gh = _dev(c["g"])
    dgs = torch.zeros_like(gam)
    L = gam.shape[0]
    for l in reversed(range(L)):
        gh, _ = ops.rmsnorm_bwd(hs[l], gam[l], rs[l], gh, dx_add=None if l == L - 1 else gh, dgamma=dgs[l])
    assert_close(gh.cpu().numpy(), c["dh0"], 1e-5, 1e-6, "dh0")
    assert_close(dgs.cpu().numpy(), c["dgammas"], 1e-5, 1e-6, "dgammas")


@pytest.mark.gpu
def test_cuda_reproduces_the_reference_builds_vectors():
    """The CUDA path against outputs of the reference's own code, carried here as fixtures."""
    from cgadimpl_b200 import ops

    eps = 1e-5
    host = lambda t: t.cpu().numpy()  # noqa: E731
    for name in ("ref_rmsnorm_6x48", "ref_rms_plain_6x48"):
        c = load(name)
        gamma = _dev(c["gamma"]) if "gamma" in c else None
        y, rstd = ops.rmsnorm_fwd(_dev(c["x"]), gamma, eps)
        dx, dg = ops.rmsnorm_bwd(_dev(c["x"]), gamma, rstd, _dev(c["gy"]))
        for k, got in (("y", y), ("rstd", rstd), ("dx", dx)) + ((("dgamma", dg),) if gamma is not None else ()):
            assert_close(host(got), c[k], 1e-5, 1e-6, f"{name} {k}")
            assert np.array_equal(host(got), c[k]), f"{name} {k}: not bit-identical on a tiny case"
    c = load("ref_layernorm_6x48")
    y, mean, var = ops.layernorm_fwd(_dev(c["x"]), eps)
    dx = ops.layernorm_bwd(_dev(c["x"]), mean, var, _dev(c["gy"]), eps)
    for k, got in (("y", y), ("mean", mean), ("var", var), ("dx", dx)):
        assert_close(host(got), c[k], 1e-5, 1e-6, f"layernorm {k}")
    c = load("ref_softmax_6x40")
    y = ops.softmax_row(_dev(c["z"]))
    assert_close(host(y), c["y"], 1e-5, 1e-30, "softmax")
    yd = _dev(c["y"])
    assert_close(host(ops.softmax_row_bwd(yd, _dev(c["gy"]))), c["dz"], 1e-5, 1e-6, "softmax vjp")
    assert_close(host(ops.softmax_row_bwd(yd, _dev(c["t"]))), c["ty"], 1e-5, 1e-6, "softmax jvp")
    c = load("ref_logsumexp_6x40")
    z = _dev(c["z"])
    assert_close(host(ops.logsumexp_row(z)), c["y"], 1e-5, 1e-6, "logsumexp")
    assert_close(host(ops.logsumexp_row_bwd(z, _dev(c["gy"]))), c["dz"], 1e-5, 1e-30, "logsumexp vjp")
    assert_close(host(ops.logsumexp_row_jvp(z, _dev(c["t"]))), c["ty"], 1e-5, 1e-6, "logsumexp jvp")
    c = load("ref_optim_64")
    p = _dev(c["p0"]).clone()
    for g in c["grads"]:
        ops.sgd_step(p, _dev(g), 1e-2)
    assert np.array_equal(host(p), c["sgd"])
    p, m, v = _dev(c["p0"]).clone(), torch.zeros(64, device="cuda"), torch.zeros(64, device="cuda")
    for t, g in enumerate(c["grads"], 1):
        a_eff, e_eff = O.adam_scalars(1e-3, 0.9, 0.999, 1e-8, t)
        ops.adam_step(p, _dev(g), m, v, 0.9, 0.999, a_eff, e_eff)
    assert np.array_equal(host(p), c["adam"])
