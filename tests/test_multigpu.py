"""Row-sharded forward + VJP on 2 GPUs (one process per GPU): every rank's y and dx equal the
rows of the single-GPU result bit for bit, and the exchanged dgamma equals the single-GPU dgamma
(the partials are exchanged in fp64 and rounded once) -- with the library's own exchange over
CUDA-IPC peer mappings ("peer") and with the NCCL all-reduce ("collective").  Skipped with fewer
than 2 GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

from inputs import fp32_accum_dgamma_tol

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, rows, hidden, dtype_name, exchange, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cgadimpl_b200 import ops
        from cgadimpl_b200.executor import RowShardedRMSNorm, shard_rows

        dtype = getattr(torch, dtype_name)

        def close(a, b, scale=1.0):
            """fp32 I/O: fp64 sums exchanged and rounded once, so at most one ulp apart.  bf16 I/O: the column
            sums are accumulated in fp32, and two shards add up in another order than one call over all rows."""
            if dtype == torch.float32:
                return int((a.view(torch.int32) - b.view(torch.int32)).abs().max()) <= 1
            rt, at = fp32_accum_dgamma_tol(rows)
            return bool(((a - b).abs() <= at * scale + rt * b.abs()).all())

        g = torch.Generator().manual_seed(0)                      # same full problem on every rank
        x = torch.randn(rows, hidden, generator=g).to(dtype)
        gy = torch.randn(rows, hidden, generator=g).to(dtype)
        gamma = (1 + 0.02 * torch.randn(hidden, generator=g)).to(dtype)
        a, b = shard_rows(rows, world, rank)
        ex = RowShardedRMSNorm(hidden, dtype, 1e-6, exchange=exchange)
        assert ex.exchange == exchange, f"asked for {exchange}, got {ex.exchange}"
        y, rstd, dx, dg = ex.fwd_bwd(x[a:b].cuda().contiguous(), gy[a:b].cuda().contiguous(), gamma.cuda())
        torch.cuda.synchronize()
        ops.device_status()
        # single-GPU result of the whole problem, computed on this rank's own GPU
        ys, rs = ops.rmsnorm_fwd(x.cuda(), gamma.cuda(), 1e-6)
        dxs, dgs = ops.rmsnorm_bwd(x.cuda(), gamma.cuda(), rs, gy.cuda())
        ok = bool(torch.equal(y, ys[a:b]) and torch.equal(dx, dxs[a:b]) and torch.equal(rstd, rs[a:b]))
        same = float((dg == dgs).float().mean())
        maxulp = int((dg.view(torch.int32) - dgs.view(torch.int32)).abs().max())
        # overlapped exchange: several steps back to back with alternating upstream gradients, the
        # all-reduce of step k running beside the kernels of step k+1; every dgamma must be its own step's
        xs, gs, gam = x[a:b].cuda().contiguous(), gy[a:b].cuda().contiguous(), gamma.cuda()
        outs = [torch.empty(hidden, device="cuda") for _ in range(12)]
        for k in range(12):
            ex.fwd_bwd(xs, gs * float(k + 1), gam, dgamma=outs[k], wait=False)
        ex.wait_dgamma()
        torch.cuda.synchronize()
        for k in range(12):
            _, want = ops.rmsnorm_bwd(x.cuda(), gam, rs, gy.cuda() * float(k + 1))
            ok = ok and close(outs[k], want, float(k + 1))
        # the prepared step (operands validated once, bare C-ABI calls per step)
        st = ex.prepare_step(xs, gs, gam, torch.empty_like(xs), torch.empty(xs.shape[0], device="cuda"),
                             torch.empty_like(xs), outs[0])
        for k in range(3):
            st.fwd()
            st.bwd()
        ex.wait_dgamma()
        torch.cuda.synchronize()
        ok = ok and close(outs[0], dgs)
        # the exchange without the side stream (every step waits for its dgamma), accumulating over steps
        ex2 = RowShardedRMSNorm(hidden, dtype, 1e-6, overlap=False, exchange=exchange)
        for k in range(4):
            _, _, _, dg2 = ex2.fwd_bwd(xs, gs, gam)
        torch.cuda.synchronize()
        ok = ok and close(dg2, dgs)
        if dtype != torch.float32:          # bit statistics only mean something for the fp64-reduced fp32 path
            same, maxulp = (1.0, 0) if close(dg, dgs) else (0.0, 1 << 30)
        ops.device_status()
        ex2.close()
        ex.close()
        q.put((rank, ok, same, maxulp))
    except BaseException:
        import traceback

        q.put((rank, False, 0.0, -1, traceback.format_exc()))      # the parent must never wait for a dead rank
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["peer", "collective"])
@pytest.mark.parametrize("dtype_name,rows,hidden", [("float32", 3001, 4096), ("bfloat16", 2048, 8192)])
def test_two_gpu_sharded_fwd_bwd(dtype_name, rows, hidden, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, rows, hidden, dtype_name, exchange, q)) for r in range(world)]
    for p in procs:
        p.start()
    import time

    results, deadline = [], time.time() + 600
    while len(results) < world and time.time() < deadline:
        if not q.empty():
            results.append(q.get())
        elif all(not p.is_alive() for p in procs) and q.empty():
            break                                                   # every rank is gone and nothing is queued
        else:
            time.sleep(0.2)
    for p in procs:
        p.join(60)
        if p.is_alive():
            p.terminate()
    failures = [r[4] for r in results if len(r) > 4]
    assert not failures, "a rank raised:\n" + "\n".join(failures)
    assert len(results) == world, f"only {len(results)} of {world} ranks reported (exit codes {[p.exitcode for p in procs]})"
    assert all(p.exitcode == 0 for p in procs)
    for rank, ok, same, maxulp in results:
        assert ok, f"rank {rank}: shard outputs differ from the single-GPU rows"
        assert same > 0.99 and maxulp <= 1, f"rank {rank}: dgamma {same:.4f} equal, max ulp {maxulp}"
