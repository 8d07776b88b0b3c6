"""Generates the golden vectors in this directory from the CPU oracle (fp64-reduced mode).

    python tests/golden/make_golden.py

The reference ships no golden vectors.  These files pin the ORACLE at configurations the reference's own
code cannot run (eps 1e-6, bf16 I/O, the corrected JVP): a later change to the oracle or to the kernels
that alters any bit of these outputs fails tests/test_golden.py.  Vectors produced by the reference's
own code (eps 1e-5, fp32) are the ref_*.npz files made by make_reference_golden.py.  Inputs are seeded
numpy draws with the distributions of the benchmark configurations, kept tiny (R <= 64).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_ffi as O  # noqa: E402
from inputs import make_inputs  # noqa: E402


def main():
    cases = {}
    # fp32, with and without gamma, including the reference test's own [4,10] shape
    for name, rows, hidden, eps, with_gamma in (("fp32_8x64", 8, 64, 1e-6, True), ("fp32_4x10_plain", 4, 10, 1e-5, False),
                                                ("fp32_5x1000", 5, 1000, 1e-5, True)):
        x, gamma, gy = make_inputs(rows, hidden, seed=sum(map(ord, name)))
        if not with_gamma:
            gamma = None
        out = O.rmsnorm_fwd_bwd(x, gamma, gy, eps)
        c = dict(x=x, gy=gy, eps=np.float32(eps), y=out["y"], rstd=out["rstd"], dx=out["dx"])
        if with_gamma:
            c.update(gamma=gamma, dgamma=out["dgamma"])
        cases[name] = c
    # bf16 I/O with outlier rows
    x, gamma, gy = make_inputs(16, 256, seed=3, x_std=3.0, gamma_std=0.1, outlier_frac=0.1)
    xb, gb, gyb = O.f32_to_bf16_bits(x), O.f32_to_bf16_bits(gamma), O.f32_to_bf16_bits(gy)
    out = O.rmsnorm_fwd_bwd_bf16(xb, gb, gyb, 1e-6)
    cases["bf16_16x256_outliers"] = dict(x=xb, gamma=gb, gy=gyb, eps=np.float32(1e-6), y=out["y"], rstd=out["rstd"],
                                         dx=out["dx"], dgamma=out["dgamma"])
    # corrected JVP
    x, gamma, _ = make_inputs(8, 64, seed=5)
    rng = np.random.default_rng(6)
    tx = rng.standard_normal((8, 64)).astype(np.float32)
    tg = rng.standard_normal(64).astype(np.float32)
    cases["jvp_8x64"] = dict(x=x, gamma=gamma, tx=tx, tgamma=tg, eps=np.float32(1e-5), ty=O.rmsnorm_jvp(x, gamma, tx, tg, 1e-5))
    # residual stack
    rng = np.random.default_rng(7)
    R, H, L = 6, 32, 3
    x = rng.standard_normal((R, H)).astype(np.float32)
    r = rng.standard_normal((R, H)).astype(np.float32)
    g = rng.standard_normal((R, H)).astype(np.float32)
    gam = (1 + 0.02 * rng.standard_normal((L, H))).astype(np.float32)
    out = O.residual_stack(x, r, gam, g, 1e-6)
    cases["stack_6x32x3"] = dict(x=x, r=r, g=g, gammas=gam, eps=np.float32(1e-6), y=out["y"], dh0=out["dh0"],
                                 dgammas=out["dgammas"])
    for name, c in cases.items():
        np.savez(os.path.join(HERE, name + ".npz"), **c)
        print(name, sum(v.nbytes for v in c.values()), "bytes")


if __name__ == "__main__":
    main()
