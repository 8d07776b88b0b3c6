"""Generates the ref_*.npz golden vectors in this directory from THE REFERENCE'S OWN CODE.

    python tests/golden/make_reference_golden.py        (needs the reference tree; development container only)

oracle/build_ref.py compiles the reference's op builders, autodiff engine and rules, unmodified, over a
CPU stand-in for its (absent) tensor library; tests/ref_ffi.py drives that build.  The outputs stored
here are therefore what the reference's composition of tensor calls produces for these inputs, with the
stand-in's fp64-accumulated reductions.  They travel to machines that have no reference tree:
tests/test_golden.py checks that the oracle reproduces them bit for bit (CPU) and that the CUDA path
matches them within the stated tolerance (GPU).  eps is the reference's hard-coded 1e-5 throughout.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import ref_ffi as REF  # noqa: E402


def main():
    if not REF.available():
        raise SystemExit("the reference build (oracle/_ref) is not available on this machine")
    REF.set_reduce_fp64(True)
    rng = np.random.default_rng(2024)
    f32 = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
    cases = {}

    x, gy = f32(6, 48), f32(6, 48)
    gamma = (1 + 0.02 * rng.standard_normal(48)).astype(np.float32)
    out = REF.rmsnorm_fwd_bwd(x, gamma, gy)
    cases["ref_rmsnorm_6x48"] = dict(x=x, gamma=gamma, gy=gy, **out)
    out = REF.rmsnorm_fwd_bwd(x, None, gy)
    cases["ref_rms_plain_6x48"] = dict(x=x, gy=gy, y=out["y"], rstd=out["rstd"], dx=out["dx"])

    x, r, g = f32(5, 32), f32(5, 32), f32(5, 32)
    gammas = (1 + 0.02 * rng.standard_normal((3, 32))).astype(np.float32)
    out = REF.residual_stack(x, r, gammas, g)
    cases["ref_stack_5x32x3"] = dict(x=x, r=r, g=g, gammas=gammas, **out)

    x, gy = (1.5 * f32(6, 48) + np.float32(0.3)), f32(6, 48)
    cases["ref_layernorm_6x48"] = dict(x=x, gy=gy, **REF.layernorm_fwd_bwd(x, gy))

    z = (3.0 * f32(6, 40)).astype(np.float32)
    z[1, 20:] = np.float32(-1e4)          # a masked tail
    z[4, 0] = np.float32(60.0)            # one dominant logit
    gy, gy_row, t = f32(6, 40), f32(6), f32(6, 40)
    o = REF.softmax_family("softmax", z, gy, t)
    cases["ref_softmax_6x40"] = dict(z=z, gy=gy, t=t, y=o["y"], dz=o["dz"], ty=o["ty"])
    o = REF.softmax_family("logsumexp", z, gy_row, t)
    cases["ref_logsumexp_6x40"] = dict(z=z, gy=gy_row, t=t, y=o["y"], dz=o["dz"], ty=o["ty"])

    p0, grads = f32(64), f32(4, 64)
    cases["ref_optim_64"] = dict(p0=p0, grads=grads, sgd=REF.optimizer("sgd", p0, grads, 1e-2),
                                 adam=REF.optimizer("adam", p0, grads, 1e-3))

    for name, c in cases.items():
        c = {k: v for k, v in c.items() if v is not None}
        np.savez(os.path.join(HERE, name + ".npz"), **c)
        print(name, sum(np.asarray(v).nbytes for v in c.values()), "bytes")


if __name__ == "__main__":
    main()
