"""The N > 1 host logic on CPU: two gloo ranks shard the rows, each forms the fp64 dgamma partial of
its shard, the partials are summed by the executor's exchange step and rounded once -- and the result
equals the single-rank dgamma.  (The kernels themselves need a GPU; here the per-shard arithmetic is
the oracle's, so only the partition and the exchange are under test.)"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_ffi as O
from inputs import make_inputs


def test_shard_rows_partition():
    from cgadimpl_b200.executor import shard_rows

    for total in (0, 1, 7, 64, 524288, 1000003):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))          # contiguous, no gaps
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1                                  # near-equal
    assert [shard_rows(524288, 8, r) for r in (0, 7)] == [(0, 65536), (458752, 524288)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, rows, hidden, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cgadimpl_b200.executor import allreduce_dgamma_f64, shard_rows

        x, gamma, gy = make_inputs(rows, hidden, seed=0)
        a, b = shard_rows(rows, world, rank)
        yhat, _ = O.rmsnorm_fwd(x[a:b], None, 1e-6)
        prod = (gy[a:b] * yhat).astype(np.float32)                # rounded to fp32 like the kernel does
        part = torch.from_numpy(prod.astype(np.float64).sum(0))   # fp64 partial of this shard
        allreduce_dgamma_f64(part)
        dgamma = part.numpy().astype(np.float32)                   # rounded once, after the exchange
        with pytest.raises(TypeError):
            allreduce_dgamma_f64(torch.zeros(4))                   # fp32 partials are refused
        if rank == 0:
            q.put(dgamma)
    finally:
        dist.destroy_process_group()


def _late_rank_main(rank, world, port, q):
    """Rank 1 never enters the all-reduce; rank 0's exchange must give up after its host deadline."""
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cgadimpl_b200.executor import ExchangeTimeout, allreduce_dgamma_f64

    part = torch.ones(64, dtype=torch.float64)
    if rank == 0:
        t0 = time.monotonic()
        try:
            allreduce_dgamma_f64(part, timeout_s=1.0)
            q.put(("no error", time.monotonic() - t0))
        except ExchangeTimeout as e:
            q.put(("timeout", time.monotonic() - t0, str(e)))
    else:
        time.sleep(4.0)          # the failure is made on the host: this rank simply does not show up
    # no destroy_process_group: a collective is still pending on rank 0; the processes just exit
    os._exit(0)


def test_a_rank_that_never_arrives_ends_the_exchange_with_an_error_after_the_deadline():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_late_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        if p.is_alive():
            p.terminate()
    assert not q.empty(), "rank 0 reported nothing"
    got = q.get()
    assert got[0] == "timeout", got
    assert 0.9 <= got[1] < 3.5, f"gave up after {got[1]:.2f} s, deadline was 1 s"


def test_two_rank_dgamma_exchange_matches_single_rank():
    rows, hidden, world = 1000, 256, 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, rows, hidden, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    x, gamma, gy = make_inputs(rows, hidden, seed=0)
    want = O.rmsnorm_fwd_bwd(x, gamma, gy, 1e-6)["dgamma"]
    # identical up to fp64 summation order, i.e. the same fp32 bits except on rare rounding ties
    assert np.abs(got.view(np.int32) - want.view(np.int32)).max() <= 1
    assert (got == want).mean() > 0.99
