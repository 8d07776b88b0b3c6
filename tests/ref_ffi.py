"""ctypes binding of oracle/_ref/libcgadimpl_ref.so: the reference's own op builders and autodiff
rules for the RMSNorm path, compiled from the reference tree over the CPU stand-in tensor library
(oracle/build_ref.py).  Test infrastructure.  `available()` is False where the library has not been
built (it needs the reference tree, which only the development container has)."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402

_lib = None


def available():
    return build_ref.available() or os.path.exists(build_ref.OUT)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_ref.build())
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def set_reduce_fp64(on):
    lib().cgadimpl_ref_set_reduce_fp64(C.c_int(1 if on else 0))


def rmsnorm_fwd_bwd(x, gamma, gy, gamma_2d=False, parallel=False):
    """mul(rms(x), gamma) and its backward through the reference's graph engine (eps = 1e-5)."""
    x, gamma, gy = _c(x), _c(gamma), _c(gy)
    R, H = x.shape
    y, dx = np.empty_like(x), np.empty_like(x)
    rstd = np.empty(R, np.float32)
    dg = None if gamma is None else np.empty(H, np.float32)
    rc = lib().cgadimpl_ref_rmsnorm_fwd_bwd(_p(x), _p(gamma), _p(gy), _p(y), _p(rstd), _p(dx), _p(dg), C.c_int64(R),
                                            C.c_int64(H), C.c_int(int(gamma_2d)), C.c_int(int(parallel)))
    assert rc == 0
    return dict(y=y, rstd=rstd, dx=dx, dgamma=dg)


def residual_stack(x, r, gammas, g):
    x, r, gammas, g = _c(x), _c(r), _c(gammas), _c(g)
    R, H = x.shape
    L = gammas.shape[0]
    y, dx0, dr0, dg = np.empty_like(x), np.empty_like(x), np.empty_like(x), np.empty_like(gammas)
    rc = lib().cgadimpl_ref_residual_stack(_p(x), _p(r), _p(gammas), _p(g), _p(y), _p(dx0), _p(dr0), _p(dg),
                                           C.c_int64(R), C.c_int64(H), C.c_int(L))
    assert rc == 0
    return dict(y=y, dx0=dx0, dr0=dr0, dgammas=dg)


def rms_jvp(x, tx, via_engine=False):
    """The reference's jvp_RMSNorm rule applied to tangent tx (via_engine: through ag::jvp instead)."""
    x, tx = _c(x), _c(tx)
    R, H = x.shape
    ty = np.empty_like(x)
    assert lib().cgadimpl_ref_rms_jvp(_p(x), _p(tx), _p(ty), C.c_int64(R), C.c_int64(H), C.c_int(int(via_engine))) == 0
    return ty


def reduction(which, x, want_grad=True):
    x = _c(x)
    R, H = x.shape
    code = {"rowsum": 0, "rowmax": 1, "sum": 2, "mean_all": 3}[which]
    out = np.empty(R if code < 2 else 1, np.float32)
    dx = np.empty_like(x) if want_grad and code != 1 else None
    assert lib().cgadimpl_ref_reduction(C.c_int(code), _p(x), _p(out), _p(dx), C.c_int64(R), C.c_int64(H)) == 0
    return out, dx


def use_all_cores():
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().cgadimpl_ref_set_num_threads(C.c_int(n))
    lib().cgadimpl_ref_num_threads.restype = C.c_int
    return int(lib().cgadimpl_ref_num_threads())


def time_fwd_bwd(rows, hidden, iters, warmup=1):
    """Seconds per forward + backward pass of the reference's own graph code (data resident in tensors)."""
    sec = C.c_double(0.0)
    assert lib().cgadimpl_ref_time_fwd_bwd(C.c_int64(rows), C.c_int64(hidden), C.c_int(iters), C.c_int(warmup), C.byref(sec)) == 0
    return sec.value


def optimizer(which, param, grads, lr_or_alpha):
    """`len(grads)` updates of `param` through the reference's own ag::SGD ('sgd') or ag::Adam ('adam')."""
    p = np.ascontiguousarray(param, np.float32).copy()
    g = np.ascontiguousarray(grads, np.float32)
    rc = lib().cgadimpl_ref_optimizer(C.c_int(0 if which == "sgd" else 1), _p(p), _p(g), C.c_int64(p.size),
                                      C.c_int(g.shape[0]), C.c_float(lr_or_alpha))
    assert rc == 0
    return p


def layernorm_fwd_bwd(x, gy):
    x, gy = _c(x), _c(gy)
    R, H = x.shape
    y, dx = np.empty_like(x), np.empty_like(x)
    mean, var = np.empty(R, np.float32), np.empty(R, np.float32)
    rc = lib().cgadimpl_ref_layernorm_fwd_bwd(_p(x), _p(gy), _p(y), _p(mean), _p(var), _p(dx), C.c_int64(R), C.c_int64(H))
    assert rc == 0
    return dict(y=y, mean=mean, var=var, dx=dx)


def softmax_family(which, z, gy, t):
    """softmax_row ('softmax') or logsumexp_row ('logsumexp') forward, VJP and JVP through the reference's
    own builders and rules.  gy is [R,H] / [R]; returns y, dz, ty."""
    z, gy, t = _c(z), _c(gy), _c(t)
    R, H = z.shape
    lse = which == "logsumexp"
    y = np.empty(R if lse else (R, H), np.float32)
    ty = np.empty(R if lse else (R, H), np.float32)
    dz = np.empty_like(z)
    rc = lib().cgadimpl_ref_softmax_family(C.c_int(1 if lse else 0), _p(z), _p(gy), _p(t), _p(y), _p(dz), _p(ty),
                                           C.c_int64(R), C.c_int64(H))
    assert rc == 0
    return dict(y=y, dz=dz, ty=ty)
