"""agb_rmsnorm_bwd_static: the RMSNorm VJP for callers that cannot allocate device memory.

Some hosts of this library may not call cudaMalloc in their hot path at all: a service that got one
fixed device arena at start-up and has to stay inside it, a real-time loop that cannot afford the
device-wide synchronisation an allocation implies, a plugin that is handed raw tensor pointers but
no allocator.  For them the VJP's dgamma partial rows live in an array compiled into the library
instead of a caller workspace.  This test calls that entry point through the C ABI twice in a row
(the second call finds the first call's leftovers in the shared array) and compares each result
with the ordinary workspace-taking entry point, at the tolerance the fp32 parity tests use.

The file sorts last on purpose, so a run that stops at the first failure has already run everything
else; it also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from inputs import assert_close, make_inputs

pytestmark = pytest.mark.gpu

F32_RTOL, F32_ATOL = 1e-5, 1e-6


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _reference_call(lib, x, gamma, rstd, gy, dx_add, dtype_code):
    """The existing entry point, with a caller-provided workspace."""
    rows, hidden = x.shape
    ws_bytes = lib.agb_rmsnorm_bwd_workspace_bytes(rows, hidden, dtype_code)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    dx = torch.empty_like(x)
    dg = torch.empty(hidden, dtype=torch.float32, device="cuda")
    st = lib.agb_rmsnorm_bwd(_ptr(x), _ptr(gamma), _ptr(rstd), _ptr(gy), _ptr(dx_add), _ptr(dx), _ptr(dg), 0, 0,
                             _ptr(ws), ws_bytes, rows, hidden, dtype_code, _stream())
    assert st == 0, lib.agb_last_error()
    return dx, dg


@pytest.mark.parametrize("rows,hidden,dtype", [(1500, 4096, torch.float32), (700, 8192, torch.bfloat16),
                                               (33, 1000, torch.float32)])
def test_static_scratch_vjp_matches_workspace_vjp_twice_in_a_row(rows, hidden, dtype):
    from cgadimpl_b200 import _lib

    lib = _lib.lib()
    code = _lib.AGB_F32 if dtype == torch.float32 else _lib.AGB_BF16
    results = []
    for call in range(2):                       # different inputs each time, same shared scratch array
        x, gamma, gy = make_inputs(rows, hidden, seed=100 + call)
        xd = torch.from_numpy(x).cuda().to(dtype)
        gd = torch.from_numpy(gamma).cuda().to(dtype)
        gyd = torch.from_numpy(gy).cuda().to(dtype)
        y = torch.empty_like(xd)
        rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
        assert lib.agb_rmsnorm_fwd(_ptr(xd), _ptr(gd), _ptr(y), _ptr(rstd), rows, hidden, 1e-6, code, _stream()) == 0
        want_dx, want_dg = _reference_call(lib, xd, gd, rstd, gyd, gyd if call else None, code)
        # outputs are the caller's buffers; the entry point itself gets no workspace
        dx = torch.empty_like(xd)
        dg = torch.full((hidden,), float("nan"), dtype=torch.float32, device="cuda")
        st = lib.agb_rmsnorm_bwd_static(_ptr(xd), _ptr(gd), _ptr(rstd), _ptr(gyd), _ptr(gyd if call else None),
                                        _ptr(dx), _ptr(dg), 0, rows, hidden, code, _stream())
        assert st == 0, lib.agb_last_error()
        torch.cuda.synchronize()
        rtol = F32_RTOL if dtype == torch.float32 else 2e-2
        assert_close(dx.float().cpu().numpy(), want_dx.float().cpu().numpy(), rtol, F32_ATOL, f"dx call {call}")
        assert_close(dg.cpu().numpy(), want_dg.cpu().numpy(), F32_RTOL, F32_ATOL, f"dgamma call {call}")
        results.append(dg.clone())
    assert not torch.equal(results[0], results[1])          # the two calls really computed different things
    assert lib.agb_device_status() == 0


def test_static_scratch_accumulates_and_rejects_oversize():
    from cgadimpl_b200 import _lib

    lib = _lib.lib()
    rows, hidden = 64, 2048
    x, gamma, gy = make_inputs(rows, hidden, seed=5)
    xd, gd, gyd = (torch.from_numpy(a).cuda() for a in (x, gamma, gy))
    y = torch.empty_like(xd)
    rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
    assert lib.agb_rmsnorm_fwd(_ptr(xd), _ptr(gd), _ptr(y), _ptr(rstd), rows, hidden, 1e-6, 0, _stream()) == 0
    _, want_dg = _reference_call(lib, xd, gd, rstd, gyd, None, 0)
    dx = torch.empty_like(xd)
    old = torch.randn(hidden, device="cuda")
    dg = old.clone()
    assert lib.agb_rmsnorm_bwd_static(_ptr(xd), _ptr(gd), _ptr(rstd), _ptr(gyd), None, _ptr(dx), _ptr(dg), 1,
                                      rows, hidden, 0, _stream()) == 0
    assert torch.equal(dg, old + want_dg)
    # a hidden size whose partial rows do not fit the built-in array is refused before any launch
    before = lib.agb_launch_count()
    big = 1 << 16
    st = lib.agb_rmsnorm_bwd_static(_ptr(xd), _ptr(gd), _ptr(rstd), _ptr(gyd), None, _ptr(dx), _ptr(dg), 0,
                                    1, big, 0, _stream())
    assert st == 5 and b"built-in array" in lib.agb_last_error()
    assert lib.agb_launch_count() == before
    # without dgamma no scratch is needed, so any size goes through
    assert lib.agb_rmsnorm_bwd_static(_ptr(xd), None, _ptr(rstd), _ptr(gyd), None, _ptr(dx), None, 0,
                                      rows, hidden, 0, _stream()) == 0
    torch.cuda.synchronize()
    assert lib.agb_device_status() == 0
