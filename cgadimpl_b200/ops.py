"""Thin wrappers that hand torch CUDA tensors to the C ABI (data_ptr + current stream).

torch is used for device memory and streams only; every computation below is one of the
library's own kernels.  Argument meaning follows include/agb/agb.h.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import AGB_BF16, AGB_F32, AGB_F64, check

_DT = {torch.float32: AGB_F32, torch.bfloat16: AGB_BF16}


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}: float32 or bfloat16 only") from None


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _rows_hidden(x):
    if not x.is_cuda:
        raise ValueError("tensor must live on a CUDA device (no CPU path exists)")
    if not x.is_contiguous():
        raise ValueError("tensor must be contiguous")
    hidden = x.shape[-1]
    return x.numel() // hidden if hidden else 0, hidden


def _same(x, *others):
    """Operands that must match x in shape, dtype and device and be contiguous (None is skipped)."""
    for t in others:
        if t is None:
            continue
        if t.shape != x.shape or t.dtype != x.dtype or t.device != x.device or not t.is_contiguous():
            raise ValueError(f"operand {tuple(t.shape)} {t.dtype} on {t.device} does not match "
                             f"{tuple(x.shape)} {x.dtype} on {x.device} (or is not contiguous)")


def _vec(x, n, dtype, *others):
    """Per-row or per-column vectors: n elements of dtype on x's device, contiguous (None is skipped)."""
    for t in others:
        if t is None:
            continue
        if t.numel() != n or t.dtype != dtype or t.device != x.device or not t.is_contiguous():
            raise ValueError(f"operand {tuple(t.shape)} {t.dtype} on {t.device}: expected {n} contiguous elements of "
                             f"{dtype} on {x.device}")


def rmsnorm_fwd(x, gamma=None, eps=1e-5, out=None, rstd=None):
    """y = (x * rstd) * gamma; returns (y, rstd[rows] fp32).  gamma=None is cgadimpl's `rms(x)`."""
    rows, hidden = _rows_hidden(x)
    y = torch.empty_like(x) if out is None else out
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if rstd is None else rstd
    _same(x, y)
    _vec(x, hidden, x.dtype, gamma)
    _vec(x, rows, torch.float32, rstd)
    check(_lib.lib().agb_rmsnorm_fwd(_p(x), _p(gamma), _p(y), _p(rstd), rows, hidden, eps, _dt(x), _stream()))
    return y, rstd


def add_rmsnorm_fwd(x, r, gamma=None, eps=1e-5, h=None, out=None, rstd=None):
    """h = x + r; y = rmsnorm(h) * gamma; returns (h, y, rstd)."""
    rows, hidden = _rows_hidden(x)
    h = torch.empty_like(x) if h is None else h
    y = torch.empty_like(x) if out is None else out
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if rstd is None else rstd
    _same(x, r, h, y)
    _vec(x, hidden, x.dtype, gamma)
    _vec(x, rows, torch.float32, rstd)
    check(_lib.lib().agb_add_rmsnorm_fwd(_p(x), _p(r), _p(gamma), _p(h), _p(y), _p(rstd), rows, hidden, eps,
                                         _dt(x), _stream()))
    return h, y, rstd


def bwd_workspace(x):
    rows, hidden = _rows_hidden(x)
    nbytes = _lib.lib().agb_rmsnorm_bwd_workspace_bytes(rows, hidden, _dt(x))
    return torch.empty(nbytes, dtype=torch.uint8, device=x.device)


def rmsnorm_bwd(x, gamma, rstd, gy, dx_add=None, dx=None, dgamma=None, accumulate_dgamma=False,
                workspace=None, dgamma_f64=False, dgamma_f64_ptr=None):
    """Returns (dx, dgamma).  dgamma is fp32 [hidden] (or the un-rounded fp64 sum when
    dgamma_f64), None when gamma is None.  dx_add is added to dx (may be gy or dx itself).
    dgamma_f64_ptr: a raw device address of `hidden` doubles that receives the un-rounded sums
    instead of a tensor (the buffer of a PeerExchange); dgamma is then returned as None."""
    rows, hidden = _rows_hidden(x)
    dx = torch.empty_like(x) if dx is None else dx
    dg_dtype = AGB_F32
    ws_bytes = 0
    if dgamma_f64_ptr is not None:
        if gamma is None or dgamma is not None:
            raise ValueError("dgamma_f64_ptr needs gamma and excludes dgamma")
        if workspace is None:
            workspace = bwd_workspace(x)
        _same(x, gy, dx_add, dx)
        _vec(x, hidden, x.dtype, gamma)
        _vec(x, rows, torch.float32, rstd)
        check(_lib.lib().agb_rmsnorm_bwd(_p(x), _p(gamma), _p(rstd), _p(gy), _p(dx_add), _p(dx),
                                         C.c_void_p(int(dgamma_f64_ptr)), AGB_F64, int(bool(accumulate_dgamma)),
                                         _p(workspace), workspace.numel() * workspace.element_size(), rows, hidden,
                                         _dt(x), _stream()))
        return dx, None
    if gamma is not None:
        if dgamma is None:
            dgamma = torch.zeros(hidden, dtype=torch.float64 if dgamma_f64 else torch.float32, device=x.device)
        dg_dtype = AGB_F64 if dgamma.dtype == torch.float64 else AGB_F32
        if workspace is None:
            workspace = bwd_workspace(x)
        ws_bytes = workspace.numel() * workspace.element_size()
    _same(x, gy, dx_add, dx)
    _vec(x, hidden, x.dtype, gamma)
    _vec(x, rows, torch.float32, rstd)
    if dgamma is not None and dgamma.numel() != hidden:
        raise ValueError("dgamma must have `hidden` elements")
    check(_lib.lib().agb_rmsnorm_bwd(_p(x), _p(gamma), _p(rstd), _p(gy), _p(dx_add), _p(dx), _p(dgamma), dg_dtype,
                                     int(bool(accumulate_dgamma)), _p(workspace), ws_bytes, rows, hidden, _dt(x),
                                     _stream()))
    return dx, dgamma


def rmsnorm_bwd_static(x, gamma, rstd, gy, dx_add=None, dx=None, dgamma=None, accumulate_dgamma=False):
    """agb_rmsnorm_bwd_static: the VJP with the library's built-in scratch array instead of a caller
    workspace (for callers that cannot allocate).  The output tensors are still the caller's; pass
    dx and dgamma to make this wrapper allocation-free as well."""
    rows, hidden = _rows_hidden(x)
    dx = torch.empty_like(x) if dx is None else dx
    if gamma is not None and dgamma is None:
        dgamma = torch.zeros(hidden, dtype=torch.float32, device=x.device)
    _same(x, gy, dx_add, dx)
    _vec(x, hidden, x.dtype, gamma)
    _vec(x, rows, torch.float32, rstd)
    _vec(x, hidden, torch.float32, dgamma)
    check(_lib.lib().agb_rmsnorm_bwd_static(_p(x), _p(gamma), _p(rstd), _p(gy), _p(dx_add), _p(dx), _p(dgamma),
                                            int(bool(accumulate_dgamma)), rows, hidden, _dt(x), _stream()))
    return dx, dgamma


def dgamma_finalize(sum_f64, dgamma=None, accumulate=False):
    hidden = sum_f64.numel()
    dgamma = torch.empty(hidden, dtype=torch.float32, device=sum_f64.device) if dgamma is None else dgamma
    check(_lib.lib().agb_dgamma_finalize(_p(sum_f64), _p(dgamma), hidden, int(bool(accumulate)), _stream()))
    return dgamma


def rmsnorm_jvp(x, gamma, rstd, tx, tgamma=None, out=None):
    rows, hidden = _rows_hidden(x)
    ty = torch.empty_like(x) if out is None else out
    _same(x, tx, ty)
    _vec(x, hidden, x.dtype, gamma, tgamma)
    _vec(x, rows, torch.float32, rstd)
    check(_lib.lib().agb_rmsnorm_jvp(_p(x), _p(gamma), _p(rstd), _p(tx), _p(tgamma), _p(ty), rows, hidden, _dt(x),
                                     _stream()))
    return ty


def residual_add(a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    _rows_hidden(a)
    _same(a, b, out)
    check(_lib.lib().agb_residual_add(_p(a), _p(b), _p(out), a.numel(), _dt(a), _stream()))
    return out


def vjp_add(ga, gb, gy):
    """ga += gy; gb += gy (either may be None)."""
    check(_lib.lib().agb_vjp_add(_p(ga), _p(gb), _p(gy), gy.numel(), _dt(gy), _stream()))


def scale_lastdim(a, g, out=None):
    rows, hidden = _rows_hidden(a)
    out = torch.empty_like(a) if out is None else out
    check(_lib.lib().agb_scale_lastdim(_p(a), _p(g), _p(out), rows, hidden, _dt(a), _stream()))
    return out


def layernorm_fwd(x, eps=1e-5, out=None):
    """cgadimpl's laynor: y = (x - mean) / sqrt(var + eps); returns (y, mean[rows], var[rows])."""
    rows, hidden = _rows_hidden(x)
    y = torch.empty_like(x) if out is None else out
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    var = torch.empty(rows, dtype=torch.float32, device=x.device)
    _same(x, y)
    check(_lib.lib().agb_layernorm_fwd(_p(x), _p(y), _p(mean), _p(var), rows, hidden, eps, _dt(x), _stream()))
    return y, mean, var


def layernorm_bwd(x, mean, var, gy, eps=1e-5, dx_add=None, dx=None):
    rows, hidden = _rows_hidden(x)
    dx = torch.empty_like(x) if dx is None else dx
    _same(x, gy, dx_add, dx)
    _vec(x, rows, torch.float32, mean, var)
    check(_lib.lib().agb_layernorm_bwd(_p(x), _p(mean), _p(var), _p(gy), _p(dx_add), _p(dx), rows, hidden, eps, _dt(x),
                                       _stream()))
    return dx


def layernorm_jvp(y, t, var, eps=1e-5, out=None):
    """Tangent of laynor's output for a tangent t of its input (y, var from layernorm_fwd)."""
    rows, hidden = _rows_hidden(y)
    ty = torch.empty_like(y) if out is None else out
    _same(y, t, ty)
    _vec(y, rows, torch.float32, var)
    check(_lib.lib().agb_layernorm_jvp(_p(y), _p(t), _p(var), _p(ty), rows, hidden, eps, _dt(y), _stream()))
    return ty


def softmax_row(z, out=None):
    """cgadimpl's softmax_row: softmax over the last axis."""
    rows, hidden = _rows_hidden(z)
    y = torch.empty_like(z) if out is None else out
    _same(z, y)
    check(_lib.lib().agb_softmax_row_fwd(_p(z), _p(y), rows, hidden, _dt(z), _stream()))
    return y


def logsumexp_row(z, out=None):
    """cgadimpl's logsumexp_row: [rows] (same dtype as z)."""
    rows, hidden = _rows_hidden(z)
    o = torch.empty(rows, dtype=z.dtype, device=z.device) if out is None else out
    _vec(z, rows, z.dtype, o)
    check(_lib.lib().agb_logsumexp_row_fwd(_p(z), _p(o), rows, hidden, _dt(z), _stream()))
    return o


def softmax_row_bwd(y, g, dz_add=None, dz=None):
    """y * (g - sum(y*g)) [+ dz_add]: the softmax VJP (g = gy) and JVP (g = tangent)."""
    rows, hidden = _rows_hidden(y)
    dz = torch.empty_like(y) if dz is None else dz
    _same(y, g, dz_add, dz)
    check(_lib.lib().agb_softmax_row_bwd(_p(y), _p(g), _p(dz_add), _p(dz), rows, hidden, _dt(y), _stream()))
    return dz


def logsumexp_row_bwd(z, gy, dz_add=None, dz=None):
    """gy[rows] * softmax(z) [+ dz_add]."""
    rows, hidden = _rows_hidden(z)
    dz = torch.empty_like(z) if dz is None else dz
    _same(z, dz_add, dz)
    _vec(z, rows, z.dtype, gy)
    check(_lib.lib().agb_logsumexp_row_bwd(_p(z), _p(gy), _p(dz_add), _p(dz), rows, hidden, _dt(z), _stream()))
    return dz


def logsumexp_row_jvp(z, tz, out=None):
    rows, hidden = _rows_hidden(z)
    o = torch.empty(rows, dtype=z.dtype, device=z.device) if out is None else out
    _same(z, tz)
    _vec(z, rows, z.dtype, o)
    check(_lib.lib().agb_logsumexp_row_jvp(_p(z), _p(tz), _p(o), rows, hidden, _dt(z), _stream()))
    return o


def sgd_step(param, grad, lr):
    """param += -lr * grad, as ag::SGD updates a leaf."""
    check(_lib.lib().agb_sgd_step(_p(param), _p(grad), param.numel(), float(lr), _dt(param), _stream()))


def adam_step(param, grad, m, v, beta1, beta2, alpha_eff, eps_eff):
    """One Adam update of one fp32 parameter (m, v in place); see agb_adam_step."""
    check(_lib.lib().agb_adam_step(_p(param), _p(grad), _p(m), _p(v), param.numel(), float(beta1), float(beta2),
                                   float(alpha_eff), float(eps_eff), _stream()))


def row_reduce(x, op):
    """op: 'sum' | 'mean' | 'max' over the last axis, keepdim; result has x's dtype."""
    rows, hidden = _rows_hidden(x)
    code = {"sum": _lib.REDUCE_SUM, "mean": _lib.REDUCE_MEAN, "max": _lib.REDUCE_MAX}[op]
    out = torch.empty(x.shape[:-1] + (1,), dtype=x.dtype, device=x.device)
    check(_lib.lib().agb_row_reduce(code, _p(x), _p(out), rows, hidden, _dt(x), _stream()))
    return out


def reduce_all(x, op):
    """op: 'sum' | 'mean' over all elements; one-element tensor of x's dtype."""
    code = {"sum": _lib.REDUCE_SUM, "mean": _lib.REDUCE_MEAN}[op]
    n = x.numel()
    ws = torch.empty(_lib.lib().agb_reduce_all_workspace_bytes(n), dtype=torch.uint8, device=x.device)
    out = torch.empty(1, dtype=x.dtype, device=x.device)
    check(_lib.lib().agb_reduce_all(code, _p(x), _p(out), n, _dt(x), _p(ws), ws.numel(), _stream()))
    return out


def device_status():
    """Raises AgbError(AGB_ERR_TIMEOUT) if a kernel's bounded wait ran out since the last call."""
    check(_lib.lib().agb_device_status())


def launch_count():
    return int(_lib.lib().agb_launch_count())


def set_option(key, value):
    check(_lib.lib().agb_set_option(key.encode(), int(value)))


def describe_launch(which, rows, hidden, dtype, fused_add=0):
    out = (C.c_int64 * 6)()
    code = {"fwd": 0, "bwd": 1, "jvp": 2, "ln_fwd": 3, "ln_bwd": 4, "ln_jvp": 5}[which]
    check(_lib.lib().agb_describe_launch(code, rows, hidden, _DT[dtype], fused_add, out))
    keys = ("grid", "block", "smem", "stages", "rows_per_tile", "generic")
    return dict(zip(keys, [int(v) for v in out]))
