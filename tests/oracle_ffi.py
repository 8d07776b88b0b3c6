"""ctypes binding of oracle/liboracle.so for the tests (the checker, never the product)."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_oracle  # noqa: E402

RED_F32, RED_F64 = 0, 1

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_oracle.build())
        _lib.agb_oracle_sum.restype = C.c_float
        _lib.agb_oracle_mean_all.restype = C.c_float
        _lib.agb_oracle_num_threads.restype = C.c_int
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def f32_to_bf16_bits(a):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def rmsnorm_fwd_bwd(x, gamma, gy, eps, red=RED_F64, fused=False):
    """x,gy [R,H] fp32, gamma [H] or None -> dict(y, rstd, dx, dgamma)."""
    x, gy, gamma = _c32(x), _c32(gy), _c32(gamma)
    R, H = x.shape
    y = np.empty_like(x)
    dx = np.empty_like(x)
    rstd = np.empty(R, np.float32)
    dg = np.zeros(H, np.float32) if gamma is not None else None
    if fused:
        lib().agb_oracle_rmsnorm_fwd_bwd_fused(_f(x), _f(gamma), _f(gy), _f(y), _f(rstd), _f(dx), _f(dg),
                                               C.c_int64(R), C.c_int64(H), C.c_float(eps))
    else:
        lib().agb_oracle_rmsnorm_fwd_bwd(_f(x), _f(gamma), _f(gy), _f(y), _f(rstd), _f(dx), _f(dg),
                                         C.c_int64(R), C.c_int64(H), C.c_float(eps), C.c_int(red))
    return dict(y=y, rstd=rstd, dx=dx, dgamma=dg)


def rmsnorm_fwd(x, gamma, eps, red=RED_F64):
    x, gamma = _c32(x), _c32(gamma)
    R, H = x.shape
    y = np.empty_like(x)
    rstd = np.empty(R, np.float32)
    lib().agb_oracle_rmsnorm_fwd(_f(x), _f(gamma), _f(y), _f(rstd), C.c_int64(R), C.c_int64(H),
                                 C.c_float(eps), C.c_int(red))
    return y, rstd


def rmsnorm_fwd_bwd_bf16(x_bits, gamma_bits, gy_bits, eps, red=RED_F64):
    """uint16 bf16 bit patterns in, dict(y bits, rstd f32, dx bits, dgamma f32) out."""
    x = np.ascontiguousarray(x_bits, np.uint16)
    gy = np.ascontiguousarray(gy_bits, np.uint16)
    gamma = None if gamma_bits is None else np.ascontiguousarray(gamma_bits, np.uint16)
    R, H = x.shape
    y = np.empty_like(x)
    dx = np.empty_like(x)
    rstd = np.empty(R, np.float32)
    dg = np.zeros(H, np.float32) if gamma is not None else None
    lib().agb_oracle_rmsnorm_fwd_bwd_bf16(_f(x), _f(gamma), _f(gy), _f(y), _f(rstd), _f(dx), _f(dg),
                                          C.c_int64(R), C.c_int64(H), C.c_float(eps), C.c_int(red))
    return dict(y=y, rstd=rstd, dx=dx, dgamma=dg)


def jvp_rms(t, yhat, rstd, corrected=True, red=RED_F64):
    t, yhat, rstd = _c32(t), _c32(yhat), _c32(rstd)
    R, H = t.shape
    out = np.empty_like(t)
    fn = lib().agb_oracle_jvp_rms_corrected if corrected else lib().agb_oracle_jvp_rms_literal
    fn(_f(t), _f(yhat), _f(rstd), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def jvp_scale(tyhat, yhat, gamma, tgamma):
    tyhat, yhat, gamma, tgamma = _c32(tyhat), _c32(yhat), _c32(gamma), _c32(tgamma)
    R, H = tyhat.shape
    out = np.empty_like(tyhat)
    lib().agb_oracle_jvp_scale(_f(tyhat), _f(yhat), _f(gamma), _f(tgamma), _f(out), C.c_int64(R), C.c_int64(H))
    return out


def rmsnorm_jvp(x, gamma, tx, tgamma, eps, red=RED_F64):
    """Corrected JVP of y = mul(rms(x), gamma): returns ty [R,H]."""
    yhat, rstd = rmsnorm_fwd(x, None, eps, red)
    tyhat = jvp_rms(tx, yhat, rstd, True, red)
    if gamma is None:
        return tyhat
    return jvp_scale(tyhat, yhat, gamma, tgamma)


def add(a, b):
    a, b = _c32(a), _c32(b)
    out = np.empty_like(a)
    lib().agb_oracle_add_forward(_f(a), _f(b), _f(out), C.c_int64(a.size))
    return out


def rowsum(x, red=RED_F64):
    x = _c32(x)
    R, H = x.shape
    out = np.empty(R, np.float32)
    lib().agb_oracle_rowsum(_f(x), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def rowmean(x, red=RED_F64):
    x = _c32(x)
    R, H = x.shape
    out = np.empty(R, np.float32)
    lib().ot_reduce_mean_last(_f(x), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def rowmax(x):
    x = _c32(x)
    R, H = x.shape
    out = np.empty(R, np.float32)
    lib().agb_oracle_rowmax(_f(x), _f(out), C.c_int64(R), C.c_int64(H))
    return out


def total_sum(x, red=RED_F64):
    x = _c32(x)
    return float(lib().agb_oracle_sum(_f(x), C.c_int64(x.size), C.c_int(red)))


def mean_all(x, red=RED_F64):
    x = _c32(x)
    return float(lib().agb_oracle_mean_all(_f(x), C.c_int64(x.size), C.c_int(red)))


def colsum(x, red=RED_F64):
    x = _c32(x)
    R, H = x.shape
    out = np.empty(H, np.float32)
    lib().ot_reduce_sum_lead(_f(x), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def residual_stack(x, r, gammas, g, eps, red=RED_F64):
    x, r, gammas, g = _c32(x), _c32(r), _c32(gammas), _c32(g)
    R, H = x.shape
    L = gammas.shape[0]
    y = np.empty_like(x)
    dh0 = np.empty_like(x)
    dg = np.empty_like(gammas)
    lib().agb_oracle_residual_stack(_f(x), _f(r), _f(gammas), _f(g), _f(y), _f(dh0), _f(dg),
                                    C.c_int64(R), C.c_int64(H), C.c_int(L), C.c_float(eps), C.c_int(red))
    return dict(y=y, dh0=dh0, dgammas=dg)


def num_threads():
    return int(lib().agb_oracle_num_threads())


def use_all_cores():
    """Undo an inherited OMP_NUM_THREADS=1 (torchrun sets it): use every core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().agb_oracle_set_num_threads(n)
    return num_threads()


def sgd_step(param, grad, lr):
    p = np.ascontiguousarray(param, np.float32).copy()
    g = _c32(grad)
    lib().agb_oracle_sgd_step(_f(p), _f(g), C.c_int64(p.size), C.c_float(lr))
    return p


def adam_step(param, grad, m, v, alpha, beta1, beta2, epsilon, t):
    """Returns new (param, m, v) after step t (1-based)."""
    p, mm, vv = (np.ascontiguousarray(a, np.float32).copy() for a in (param, m, v))
    g = _c32(grad)
    lib().agb_oracle_adam_step(_f(p), _f(g), _f(mm), _f(vv), C.c_int64(p.size), C.c_float(alpha), C.c_float(beta1),
                               C.c_float(beta2), C.c_float(epsilon), C.c_int(t))
    return p, mm, vv


def adam_scalars(alpha, beta1, beta2, epsilon, t):
    a, e = C.c_float(0), C.c_float(0)
    lib().agb_oracle_adam_scalars(C.c_float(alpha), C.c_float(beta1), C.c_float(beta2), C.c_float(epsilon), C.c_int(t),
                                  C.byref(a), C.byref(e))
    return a.value, e.value


def layernorm_fwd_bwd(x, gy, eps, red=RED_F64):
    """laynor(x) and its VJP: dict(y, mean, var, dx)."""
    x, gy = _c32(x), _c32(gy)
    R, H = x.shape
    y, dx = np.empty_like(x), np.empty_like(x)
    mean, var = np.empty(R, np.float32), np.empty(R, np.float32)
    lib().agb_oracle_layernorm_forward(_f(x), _f(y), _f(mean), _f(var), C.c_int64(R), C.c_int64(H), C.c_float(eps), C.c_int(red))
    lib().agb_oracle_layernorm_vjp(_f(x), _f(mean), _f(var), _f(gy), _f(dx), C.c_int64(R), C.c_int64(H), C.c_float(eps), C.c_int(red))
    return dict(y=y, mean=mean, var=var, dx=dx)


def softmax_row(z, red=RED_F64):
    z = np.ascontiguousarray(z, np.float32)
    R, H = z.shape
    y = np.empty_like(z)
    lib().agb_oracle_softmax_row_forward(_f(z), _f(y), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return y


def logsumexp_row(z, red=RED_F64):
    z = np.ascontiguousarray(z, np.float32)
    R, H = z.shape
    out = np.empty(R, np.float32)
    lib().agb_oracle_logsumexp_row_forward(_f(z), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def softmax_row_vjp(y, g, red=RED_F64):
    """Also the JVP: the same expression with the tangent in place of gy."""
    y, g = np.ascontiguousarray(y, np.float32), np.ascontiguousarray(g, np.float32)
    R, H = y.shape
    out = np.empty_like(y)
    lib().agb_oracle_softmax_row_vjp(_f(y), _f(g), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def logsumexp_row_vjp(z, gy, red=RED_F64):
    z, gy = np.ascontiguousarray(z, np.float32), np.ascontiguousarray(gy, np.float32)
    R, H = z.shape
    dz = np.empty_like(z)
    lib().agb_oracle_logsumexp_row_vjp(_f(z), _f(gy), _f(dz), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return dz


def logsumexp_row_jvp(z, tz, red=RED_F64):
    z, tz = np.ascontiguousarray(z, np.float32), np.ascontiguousarray(tz, np.float32)
    R, H = z.shape
    out = np.empty(R, np.float32)
    lib().agb_oracle_logsumexp_row_jvp(_f(z), _f(tz), _f(out), C.c_int64(R), C.c_int64(H), C.c_int(red))
    return out


def layernorm_jvp(y, t, var, eps):
    y, t, var = (np.ascontiguousarray(a, np.float32) for a in (y, t, var))
    R, H = y.shape
    ty = np.empty_like(y)
    lib().agb_oracle_layernorm_jvp(_f(y), _f(t), _f(var), _f(ty), C.c_int64(R), C.c_int64(H), C.c_float(eps))
    return ty
