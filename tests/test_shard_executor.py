"""The single-process multi-GPU executor (include/agb/agb_shard.h) against the single-device calls
and the CPU oracle.  Shards may share a GPU, so the sharding logic, the event ordering and the peer-sum
kernel are exercised on a one-GPU machine too; the cases over two distinct devices run where there
are two."""
import numpy as np
import pytest
import torch

import oracle_ffi as O
from inputs import assert_close, fp32_accum_dgamma_tol, make_inputs

pytestmark = pytest.mark.gpu

F32_RTOL, F32_ATOL = 1e-5, 1e-6


@pytest.fixture(scope="module")
def ops():
    from cgadimpl_b200 import ops as _ops

    yield _ops
    _ops.device_status()


def _split(a, bounds, devices, dtype=None):
    out = []
    for (lo, hi), d in zip(bounds, devices):
        t = torch.from_numpy(np.ascontiguousarray(a[lo:hi])).to(f"cuda:{d}")
        out.append(t if dtype is None else t.to(dtype))
    return out


def _bounds(rows_per_shard):
    edges = np.concatenate([[0], np.cumsum(rows_per_shard)])
    return [(int(edges[i]), int(edges[i + 1])) for i in range(len(rows_per_shard))]


def _run_sharded(devices, rows_per_shard, hidden, eps, seed, dtype=torch.float32, steps=1, accumulate=False,
                 deferred=False):
    from cgadimpl_b200.shard_executor import ShardExecutor

    rows = int(sum(rows_per_shard))
    x, gamma, gy = make_inputs(rows, hidden, seed=seed)
    bounds = _bounds(rows_per_shard)
    xs, gys = _split(x, bounds, devices, dtype), _split(gy, bounds, devices, dtype)
    gammas = [torch.from_numpy(gamma).to(f"cuda:{d}").to(dtype) for d in devices]
    dgammas = [torch.full((hidden,), 0.5, dtype=torch.float32, device=f"cuda:{d}") for d in devices]
    for d in set(devices):
        torch.cuda.synchronize(d)
    with ShardExecutor(devices, hidden) as ex:
        assert len(ex) == len(devices)
        ex.set_deferred_exchange(deferred)
        for _ in range(steps):   # repeated runs reuse the executor's fp64 buffers: the done-event path
            ys, rstds, dxs, dgs = ex.fwd_bwd(xs, gammas, gys, eps, dgammas=dgammas, accumulate_dgamma=accumulate)
        ex.synchronize()
    cat = lambda ts: torch.cat([t.to("cuda:0") for t in ts])
    return (x, gamma, gy), cat(ys), cat(rstds), cat(dxs), [d.to("cuda:0") for d in dgs]


@pytest.mark.parametrize("rows_per_shard", [(600, 424), (1, 1023), (512, 0, 512), (100, 200, 300, 424)])
def test_shards_on_one_gpu_equal_the_single_call_and_the_oracle(ops, rows_per_shard):
    hidden, eps = 4096, 1e-5
    devices = [0] * len(rows_per_shard)
    (x, gamma, gy), y, rstd, dx, dgs = _run_sharded(devices, rows_per_shard, hidden, eps, seed=11)
    xd, gd, gyd = (torch.from_numpy(a).cuda() for a in (x, gamma, gy))
    y1, rstd1 = ops.rmsnorm_fwd(xd, gd, eps)
    dx1, dg1 = ops.rmsnorm_bwd(xd, gd, rstd1, gyd)
    # rows are independent: sharding must not change a single bit of y, rstd, dx
    assert torch.equal(y, y1) and torch.equal(rstd, rstd1) and torch.equal(dx, dx1)
    # every shard holds the same dgamma bits; against the unsharded call only the fp64 summation order differs
    for d in dgs[1:]:
        assert torch.equal(d, dgs[0])
    assert_close(dgs[0].cpu().numpy(), dg1.cpu().numpy(), 1e-6, 1e-7, "dgamma sharded vs single call")
    ref = O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F64)
    assert_close(dgs[0].cpu().numpy(), ref["dgamma"], F32_RTOL, F32_ATOL, "dgamma vs oracle")
    assert_close(dx.cpu().numpy(), ref["dx"], F32_RTOL, F32_ATOL, "dx vs oracle")


@pytest.mark.parametrize("deferred", [False, True])
def test_repeated_runs_and_accumulation(ops, deferred):
    """Several runs through one executor: the sum buffers are reused (one in the immediate mode, two in turn
    with the exchange deferred to the side streams), guarded by the done events."""
    hidden, eps, steps = 1024, 1e-6, 5
    (x, gamma, gy), y, rstd, dx, dgs = _run_sharded([0, 0, 0], (300, 112, 100), hidden, eps, seed=5, steps=steps,
                                                    accumulate=True, deferred=deferred)
    ref = O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F64)
    want = np.float32(0.5)
    for _ in range(steps):   # dgamma started at 0.5 and received the same sum `steps` times, rounded each time
        want = (want + ref["dgamma"]).astype(np.float32)
    assert_close(dgs[0].cpu().numpy(), want, F32_RTOL, 2e-6, "accumulated dgamma")
    assert torch.equal(dgs[0], dgs[1]) and torch.equal(dgs[0], dgs[2])


def test_deferred_exchange_is_ordered_by_wait_dgamma(ops):
    """With the exchange on the side streams, a reader on a shard's own stream is ordered after it by
    wait_dgamma(): copy dgamma on that stream right after, without a host synchronisation in between."""
    from cgadimpl_b200.shard_executor import ShardExecutor

    hidden, eps = 2048, 1e-5
    x, gamma, gy = make_inputs(4096, hidden, seed=8)
    xs, gys = _split(x, [(0, 3000), (3000, 4096)], [0, 0]), _split(gy, [(0, 3000), (3000, 4096)], [0, 0])
    gammas = [torch.from_numpy(gamma).cuda() for _ in range(2)]
    dgs = [torch.zeros(hidden, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    with ShardExecutor([0, 0], hidden) as ex:
        ex.set_deferred_exchange(True)
        ex.fwd_bwd(xs, gammas, gys, eps, dgammas=dgs)
        ex.wait_dgamma()
        with torch.cuda.stream(ex.stream(1)):
            seen = dgs[1].clone()
        ex.synchronize()
        ex.set_deferred_exchange(False)      # and back: the immediate mode gives the same bits
        again = [torch.zeros(hidden, device="cuda") for _ in range(2)]
        ex.fwd_bwd(xs, gammas, gys, eps, dgammas=again)
        ex.synchronize()
    ref = O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F64)
    assert_close(seen.cpu().numpy(), ref["dgamma"], F32_RTOL, F32_ATOL, "dgamma read on the shard stream")
    assert torch.equal(seen, dgs[0]) and torch.equal(seen, again[0]) and torch.equal(seen, again[1])


def test_bf16_shards(ops):
    hidden, eps = 1000, 1e-6
    (x, gamma, gy), y, rstd, dx, dgs = _run_sharded([0, 0, 0], (100, 57, 99), hidden, eps, seed=3, dtype=torch.bfloat16)
    xd, gd, gyd = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in (x, gamma, gy))
    y1, rstd1 = ops.rmsnorm_fwd(xd, gd, eps)
    dx1, dg1 = ops.rmsnorm_bwd(xd, gd, rstd1, gyd)
    assert torch.equal(y, y1) and torch.equal(rstd, rstd1) and torch.equal(dx, dx1)
    # fp32-accumulated column sums: three shards add up in another order than one call over all rows
    assert_close(dgs[0].cpu().numpy(), dg1.cpu().numpy(), *fp32_accum_dgamma_tol(256), "bf16 dgamma sharded vs single call")


def test_without_gamma_and_argument_errors(ops):
    from cgadimpl_b200._lib import AgbError
    from cgadimpl_b200.shard_executor import ShardExecutor

    x = torch.randn(64, 512, device="cuda")
    gy = torch.randn(64, 512, device="cuda")
    gamma = torch.ones(512, device="cuda")
    with ShardExecutor([0, 0], 512) as ex:
        ys, rstds, dxs, dgs = ex.fwd_bwd([x[:40], x[40:]], [None, None], [gy[:40], gy[40:]])
        ex.synchronize()
        assert dgs == [None, None]
        y1, rstd1 = ops.rmsnorm_fwd(x, None, 1e-5)
        dx1, _ = ops.rmsnorm_bwd(x, None, rstd1, gy)
        assert torch.equal(torch.cat(ys), y1) and torch.equal(torch.cat(dxs), dx1)
        with pytest.raises(AgbError) as e:   # dgamma for one shard only
            ex.fwd_bwd([x[:40], x[40:]], [gamma, gamma], [gy[:40], gy[40:]],
                       dgammas=[torch.empty(512, device="cuda"), None])
        assert e.value.status == 1
        with pytest.raises(ValueError):      # wrong number of shards
            ex.fwd_bwd([x], [gamma], [gy])
    wide = torch.randn(8, 1024, device="cuda")
    with ShardExecutor([0], 512) as ex:
        with pytest.raises(AgbError) as e:   # wider than the executor was created for
            ex.fwd_bwd([wide], [torch.ones(1024, device="cuda")], [wide])
        assert e.value.status == 5
    with pytest.raises(AgbError):
        ShardExecutor([torch.cuda.device_count()], 512)   # no such device


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("deferred", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_devices_exchange_over_peer_mappings(ops, dtype, deferred):
    hidden, eps = 4096, 1e-5
    n = min(torch.cuda.device_count(), 4)
    rows_per_shard = [1000 + 13 * i for i in range(n)]
    (x, gamma, gy), y, rstd, dx, dgs = _run_sharded(list(range(n)), rows_per_shard, hidden, eps, seed=21, dtype=dtype, steps=4,
                                                    deferred=deferred)
    xd, gd, gyd = (torch.from_numpy(a).cuda().to(dtype) for a in (x, gamma, gy))
    y1, rstd1 = ops.rmsnorm_fwd(xd, gd, eps)
    dx1, dg1 = ops.rmsnorm_bwd(xd, gd, rstd1, gyd)
    assert torch.equal(y, y1) and torch.equal(rstd, rstd1) and torch.equal(dx, dx1)
    for d in dgs[1:]:
        assert torch.equal(d, dgs[0])
    tol = (1e-6, 1e-7) if dtype == torch.float32 else fp32_accum_dgamma_tol(sum(rows_per_shard))
    assert_close(dgs[0].cpu().numpy(), dg1.cpu().numpy(), *tol, "dgamma over peers vs single device")
