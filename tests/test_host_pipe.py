"""The host-buffer entry point of include/agb/agb_host.h, called through the C ABI with page-locked host
buffers: chunked copies in, kernels, copies out on three streams.  Results must be the device-resident
calls' results; dgamma is accumulated over the chunks in fp64 and rounded once, so it does not depend on
the chunking."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_ffi as O
from inputs import assert_close, fp32_accum_dgamma_tol, make_inputs

pytestmark = pytest.mark.gpu


def _hp(t):
    return None if t is None else C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("rows,hidden,dtype,chunk", [(1000, 1024, torch.float32, 96), (257, 4096, torch.float32, 0),
                                                     (700, 2048, torch.bfloat16, 128), (0, 512, torch.float32, 0)])
def test_host_pipe_matches_the_device_calls(rows, hidden, dtype, chunk):
    from cgadimpl_b200 import _lib, ops

    lib = _lib.lib()
    code = _lib.AGB_F32 if dtype == torch.float32 else _lib.AGB_BF16
    x, gamma, gy = make_inputs(max(rows, 1), hidden, seed=rows + hidden)
    x, gy = x[:rows], gy[:rows]
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    gyh = torch.from_numpy(gy).to(dtype).pin_memory()
    gh = torch.from_numpy(gamma).to(dtype).pin_memory()
    yh, dxh = torch.empty_like(xh).pin_memory(), torch.empty_like(xh).pin_memory()
    dgh = torch.full((hidden,), float("nan")).pin_memory()
    rstdh = torch.empty(rows).pin_memory()
    pipe = C.c_void_p()
    assert lib.agb_host_pipe_create(hidden, code, chunk, C.byref(pipe)) == 0, lib.agb_last_error()
    try:
        if chunk:
            assert lib.agb_host_pipe_chunk_rows(pipe) == chunk
        for _ in range(2):      # twice: the slots and events are reused across calls
            st = lib.agb_host_pipe_fwd_bwd(pipe, _hp(xh), _hp(gyh), _hp(gh), _hp(yh), _hp(dxh), _hp(dgh), _hp(rstdh), rows, 1e-6, None)
            assert st == 0, lib.agb_last_error()
    finally:
        assert lib.agb_host_pipe_destroy(pipe) == 0
    ops.device_status()
    if rows == 0:
        assert bool((dgh == 0).all())
        return
    xd, gyd, gd = xh.cuda(), gyh.cuda(), gh.cuda()
    y, rstd = ops.rmsnorm_fwd(xd, gd, 1e-6)
    dx, dg = ops.rmsnorm_bwd(xd, gd, rstd, gyd)
    assert torch.equal(yh.cuda(), y) and torch.equal(dxh.cuda(), dx) and torch.equal(rstdh.cuda(), rstd)
    if dtype == torch.float32:
        assert int((dgh.cuda().view(torch.int32) - dg.view(torch.int32)).abs().max()) <= 1   # fp64 sums, rounded once
        ref = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-6, O.RED_F64)
        assert_close(dgh.numpy(), ref["dgamma"], 1e-5, 1e-6, "dgamma vs oracle")
    else:
        assert_close(dgh.numpy(), dg.cpu().numpy(), *fp32_accum_dgamma_tol(rows), "dgamma")


def test_executor_host_entry_goes_through_the_pipe():
    from cgadimpl_b200 import ops
    from cgadimpl_b200.executor import RowShardedRMSNorm

    rows, hidden = 300, 1024
    x, gamma, gy = make_inputs(rows, hidden, seed=2)
    xh, gyh, gh = (torch.from_numpy(a).pin_memory() for a in (x, gy, gamma))
    yh, dxh, dgh = torch.empty_like(xh).pin_memory(), torch.empty_like(xh).pin_memory(), torch.empty(hidden).pin_memory()
    ex = RowShardedRMSNorm(hidden, torch.float32, 1e-5, chunk_rows=64)
    before = ops.launch_count()
    ex.fwd_bwd_host(xh, gyh, gh, yh, dxh, dgh)
    assert ops.launch_count() - before == 5 * 3 + 1      # 5 chunks x (forward, backward, reduction) + the final rounding
    ref = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-5, O.RED_F64)
    assert_close(yh.numpy(), ref["y"], 1e-5, 1e-6, "y")
    assert_close(dxh.numpy(), ref["dx"], 1e-5, 1e-6, "dx")
    assert_close(dgh.numpy(), ref["dgamma"], 1e-5, 1e-6, "dgamma")
    ex.close()
