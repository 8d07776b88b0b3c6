"""The cross-rank dgamma exchange of include/agb/agb_shard.h (agb_peer_*) on ONE GPU: two ranks as two
objects of one process, connected by address (agb_peer_connect_local).  Both ranks publish before either
sums, so no kernel ever waits for a later launch on its own GPU; the wait that runs out is tested with a
counter nobody advances and a small poll limit, and must leave the context usable.  The IPC path between
processes needs two GPUs (tests/test_multigpu.py)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_ffi as O
from inputs import assert_close, make_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cgadimpl_b200 import ops as _ops

    yield _ops
    _ops.device_status()


def _make_ranks(world, hidden):
    from cgadimpl_b200 import _lib
    from cgadimpl_b200._lib import check

    lib = _lib.lib()
    peers, bases = [], (C.c_void_p * world)()
    for r in range(world):
        h = C.c_void_p()
        check(lib.agb_peer_create(r, world, hidden, C.byref(h), None))
        base = C.c_void_p()
        check(lib.agb_peer_block(h, C.byref(base)))
        peers.append(h)
        bases[r] = base.value
    for h in peers:
        check(lib.agb_peer_connect_local(h, bases))
    return lib, peers


def _destroy(lib, peers):
    torch.cuda.synchronize()
    for h in peers:
        assert lib.agb_peer_destroy(h) == 0


def test_two_ranks_in_one_process_sum_in_rank_order(ops):
    from cgadimpl_b200._lib import check

    hidden, eps, world, steps = 2048, 1e-5, 2, 19     # 19 steps: all eight buffers reused twice, acks consulted from step 9
    x, gamma, gy = make_inputs(1000, hidden, seed=4)
    cut = 600
    xs = [torch.from_numpy(x[:cut]).cuda(), torch.from_numpy(x[cut:]).cuda()]
    gys = [torch.from_numpy(gy[:cut]).cuda(), torch.from_numpy(gy[cut:]).cuda()]
    gd = torch.from_numpy(gamma).cuda()
    lib, peers = _make_ranks(world, hidden)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        rstds = [ops.rmsnorm_fwd(xs[r], gd, eps)[1] for r in range(world)]
        outs = [torch.zeros(hidden, device="cuda") for _ in range(world)]
        for k in range(steps):
            scale = float(k + 1)
            for r in range(world):                       # every rank: acquire, backward, publish
                buf = C.c_void_p()
                check(lib.agb_peer_acquire(peers[r], stream, C.byref(buf)))
                ops.rmsnorm_bwd(xs[r], gd, rstds[r], gys[r] * scale, dgamma_f64_ptr=buf.value)
                check(lib.agb_peer_publish(peers[r], stream))
            for r in range(world):                       # only then: sum (all counters already advanced)
                check(lib.agb_peer_sum(peers[r], C.c_void_p(outs[r].data_ptr()), hidden, 0, stream))
            torch.cuda.synchronize()
            ref = O.rmsnorm_fwd_bwd(x, gamma, (gy * np.float32(scale)).astype(np.float32), eps, O.RED_F64)
            assert torch.equal(outs[0], outs[1]), f"step {k}: ranks disagree"
            assert_close(outs[0].cpu().numpy(), ref["dgamma"], 1e-5, 1e-6, f"dgamma step {k}")
        ops.device_status()
    finally:
        _destroy(lib, peers)


def test_fused_backward_publishes_and_matches_the_unfused_sequence(ops):
    """agb_peer_rmsnorm_bwd (wait + publish inside the backward's column reduction) against acquire /
    backward / publish: same dx, same dgamma bits, over enough steps to reuse both buffers."""
    from cgadimpl_b200 import ops as O2
    from cgadimpl_b200._lib import check

    hidden, eps, world, steps = 1024, 1e-6, 2, 19
    x, gamma, gy = make_inputs(777, hidden, seed=12)
    cut = 300
    xs = [torch.from_numpy(x[:cut]).cuda(), torch.from_numpy(x[cut:]).cuda()]
    gys = [torch.from_numpy(gy[:cut]).cuda(), torch.from_numpy(gy[cut:]).cuda()]
    gd = torch.from_numpy(gamma).cuda()
    lib, peers = _make_ranks(world, hidden)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = O2._p
    try:
        rstds = [ops.rmsnorm_fwd(xs[r], gd, eps)[1] for r in range(world)]
        ws = ops.bwd_workspace(xs[1])
        outs = [torch.zeros(hidden, device="cuda") for _ in range(world)]
        for k in range(steps):
            scale = float(k + 1)
            dxs = []
            for r in range(world):
                g = gys[r] * scale
                dx = torch.empty_like(xs[r])
                check(lib.agb_peer_rmsnorm_bwd(peers[r], p(xs[r]), p(gd), p(rstds[r]), p(g), None, p(dx), p(ws),
                                               ws.numel(), xs[r].shape[0], hidden, 0, stream))
                dxs.append(dx)
            for r in range(world):
                check(lib.agb_peer_sum(peers[r], C.c_void_p(outs[r].data_ptr()), hidden, 0, stream))
            torch.cuda.synchronize()
            xd, gyd = torch.cat(xs), torch.cat(gys) * scale
            dx1, dg1 = ops.rmsnorm_bwd(xd, gd, torch.cat(rstds), gyd)
            assert torch.equal(torch.cat(dxs), dx1)
            assert torch.equal(outs[0], outs[1])
            assert int((outs[0].view(torch.int32) - dg1.view(torch.int32)).abs().max()) <= 1, f"step {k}"
        ops.device_status()
    finally:
        _destroy(lib, peers)


def test_wait_that_runs_out_reports_timeout_and_leaves_dgamma_untouched(ops):
    from cgadimpl_b200._lib import AgbError, check

    hidden, world = 512, 2
    lib, peers = _make_ranks(world, hidden)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ops.set_option("peer_poll_limit", 2000)              # ~1 ms instead of ~2 s
    try:
        buf = C.c_void_p()
        check(lib.agb_peer_acquire(peers[0], stream, C.byref(buf)))
        torch.cuda.synchronize()
        check(lib.agb_peer_publish(peers[0], stream))    # rank 1 never publishes step 1
        out = torch.full((hidden,), 7.0, device="cuda")
        check(lib.agb_peer_sum(peers[0], C.c_void_p(out.data_ptr()), hidden, 0, stream))
        torch.cuda.synchronize()
        with pytest.raises(AgbError) as e:
            ops.device_status()
        assert e.value.status == 6                       # AGB_ERR_TIMEOUT
        assert bool((out == 7.0).all())
        ops.device_status()                              # the status word was cleared by the read
        y, _ = ops.rmsnorm_fwd(torch.ones(4, 64, device="cuda"), None, 1e-5)   # the context still works
        assert torch.isfinite(y).all()
    finally:
        ops.set_option("peer_poll_limit", 0)
        _destroy(lib, peers)


def test_fused_reduce_whose_ack_wait_runs_out_publishes_nothing_and_leaves_its_counter_at_zero(ops):
    """agb_peer_rmsnorm_bwd waits, inside the backward's column reduction, for every rank's acknowledgement of the
    step eight steps back (eight buffers are used in turn).  Here that acknowledgement is wiped (a rank that fell behind), the wait runs out after a small
    poll limit, and the kernel must report AGB_ERR_TIMEOUT, publish nothing, write no sums, and leave the
    "last CTA" counter of its block at zero -- a counter left part-way would make a later launch publish early."""
    cudart = pytest.importorskip("cuda.bindings.runtime")
    from cgadimpl_b200 import ops as O2
    from cgadimpl_b200._lib import AgbError, check

    hidden, eps, world = 1024, 1e-6, 2
    x, gamma, gy = make_inputs(512, hidden, seed=5)
    xs = [torch.from_numpy(x[:256]).cuda(), torch.from_numpy(x[256:]).cuda()]
    gys = [torch.from_numpy(gy[:256]).cuda(), torch.from_numpy(gy[256:]).cuda()]
    gd = torch.from_numpy(gamma).cuda()
    lib, peers = _make_ranks(world, hidden)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = O2._p

    def words(base, offset, n, dtype):
        host = np.zeros(n, dtype)
        (err,) = cudart.cudaMemcpy(host.ctypes.data, base + offset, host.nbytes, cudart.cudaMemcpyKind.cudaMemcpyDeviceToHost)
        assert int(err) == 0
        return host

    try:
        rstds = [ops.rmsnorm_fwd(xs[r], gd, eps)[1] for r in range(world)]
        ws = ops.bwd_workspace(xs[0])
        outs = [torch.zeros(hidden, device="cuda") for _ in range(world)]
        dxs = [torch.empty_like(t) for t in xs]

        def fused_bwd(r):
            return lib.agb_peer_rmsnorm_bwd(peers[r], p(xs[r]), p(gd), p(rstds[r]), p(gys[r]), None, p(dxs[r]), p(ws),
                                            ws.numel(), xs[r].shape[0], hidden, 0, stream)

        for _ in range(8):                                  # steps 1..8: everybody publishes, sums, acknowledges; every buffer used once
            for r in range(world):
                check(fused_bwd(r))
            for r in range(world):
                check(lib.agb_peer_sum(peers[r], C.c_void_p(outs[r].data_ptr()), hidden, 0, stream))
        torch.cuda.synchronize()
        ops.device_status()
        base0, base1 = C.c_void_p(), C.c_void_p()
        check(lib.agb_peer_block(peers[0], C.byref(base0)))
        check(lib.agb_peer_block(peers[1], C.byref(base1)))
        # rank 0's block after eight steps (buffer b = step mod 8): ready[s][b] of both sources, ack[r][b] of both readers
        after8 = [8, 1, 2, 3, 4, 5, 6, 7]
        assert list(words(base0.value, 0, 16, np.uint64)) == after8 + after8
        assert list(words(base0.value, 1024, 16, np.uint64)) == after8 + after8
        (err,) = cudart.cudaMemset(base0.value + 1024 + 64, 0, 64)              # reader 1 "has not acknowledged" anything
        assert int(err) == 0
        slot = 4096 + (0 * 8 + 1) * hidden * 8                                  # rank 0's slot of buffer 1 (step 9's buffer)
        sums_before = words(base0.value, slot, hidden, np.float64)
        remote_before = words(base1.value, slot, hidden, np.float64)            # and its copy in rank 1's block
        ops.set_option("peer_poll_limit", 2000)
        check(fused_bwd(0))                                                     # step 9 of rank 0: needs ack >= 1 of reader 1
        torch.cuda.synchronize()
        with pytest.raises(AgbError) as e:
            ops.device_status()
        assert e.value.status == 6
        assert list(words(base0.value, 0, 8, np.uint64)) == after8              # step 9 was published nowhere
        assert list(words(base1.value, 0, 8, np.uint64)) == after8
        assert list(words(base0.value, 2048, 2, np.uint32)) == [0, 0]           # counter and expired-CTA count back at zero
        assert np.array_equal(words(base0.value, slot, hidden, np.float64), sums_before)      # no sums stored, here or there
        assert np.array_equal(words(base1.value, slot, hidden, np.float64), remote_before)
        y, _ = ops.rmsnorm_fwd(torch.ones(4, 64, device="cuda"), None, 1e-5)    # the context still works
        assert torch.isfinite(y).all()
    finally:
        ops.set_option("peer_poll_limit", 0)
        _destroy(lib, peers)


def test_call_order_is_checked(ops):
    lib, peers = _make_ranks(1, 256)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        out = torch.zeros(256, device="cuda")
        assert lib.agb_peer_publish(peers[0], stream) == 1                      # no acquire yet
        assert lib.agb_peer_sum(peers[0], C.c_void_p(out.data_ptr()), 256, 0, stream) == 1
        buf = C.c_void_p()
        assert lib.agb_peer_acquire(peers[0], stream, C.byref(buf)) == 0
        assert lib.agb_peer_acquire(peers[0], stream, C.byref(buf)) == 1        # twice
        assert lib.agb_peer_sum(peers[0], C.c_void_p(out.data_ptr()), 256, 0, stream) == 1   # not published
        # a world of one: the exchange degenerates to rounding the rank's own sums (the block starts zeroed)
        assert lib.agb_peer_publish(peers[0], stream) == 0
        assert lib.agb_peer_publish(peers[0], stream) == 1                      # twice
        assert lib.agb_peer_sum(peers[0], C.c_void_p(out.data_ptr()), 4096, 0, stream) == 5   # hidden > max_hidden
        out.fill_(3.0)
        assert lib.agb_peer_sum(peers[0], C.c_void_p(out.data_ptr()), 256, 0, stream) == 0
        torch.cuda.synchronize()
        assert bool((out == 0).all())
    finally:
        _destroy(lib, peers)
