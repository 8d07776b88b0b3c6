"""Row-sharded executor for the RMSNorm forward + VJP path.

Rows are independent in the forward and in dx; only dgamma couples them.  So each rank (one
process per GPU) owns a contiguous block of rows, runs the same two kernels on it, and the
ranks exchange exactly one thing: the [hidden] fp64 column sum of dgamma, all-reduced over
NCCL (NVLink / NVSwitch) and rounded to fp32 once afterwards.  Reducing in fp64 keeps the
N-GPU dgamma equal to the 1-GPU result up to fp64 rounding, i.e. the same fp32 bits in all
but rare tie cases.

The all-reduce carries 8 * hidden bytes and is latency-bound, so with overlap=True (default) it
runs on a side stream and overlaps whatever the caller enqueues next (the next step's kernels);
`wait_dgamma()` makes the current stream wait for the newest dgamma before it is read.

Two entry points:
  fwd_bwd(x, gy, gamma)           device tensors of this rank's shard
  fwd_bwd_host(...)               pinned HOST buffers; chunks of rows are copied in, processed
                                  and copied out on three streams so PCIe transfers in both
                                  directions overlap the kernels
"""
import torch

from . import ops


def shard_rows(total_rows, world_size, rank):
    """Contiguous, near-equal split: first (total % world) ranks get one extra row."""
    base, extra = divmod(total_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class ExchangeTimeout(RuntimeError):
    """The dgamma exchange did not complete within the caller's deadline: a rank is late, has left, or never
    entered the collective.  The collective may still be pending; the caller decides whether to wait on or
    tear the process group down (its buffers must not be reused before then)."""


def allreduce_dgamma_f64(dg64, group=None, timeout_s=None):
    """The path's only exchange: sum the [hidden] fp64 dgamma partials of all ranks in place.
    Works on CUDA tensors (NCCL) and CPU tensors (gloo); a no-op without a process group.

    timeout_s: a host-side deadline.  The collective is started asynchronously and waited for at most that
    long; on expiry ExchangeTimeout is raised instead of blocking forever on a rank that never arrives
    (the reference's only failure handling is print-and-exit, cgadimpl/src/runtime/cuda_graphs.cpp:12-19).
    On CPU tensors the wait is the work handle's own; on CUDA tensors, where a collective is stream-ordered
    and its handle's wait returns at once, the deadline applies to an event recorded behind the collective."""
    if dg64.dtype != torch.float64:
        raise TypeError("dgamma partials are exchanged in fp64 so that the N-rank result rounds like the 1-rank one")
    dist = torch.distributed
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        return dg64
    if timeout_s is None:
        dist.all_reduce(dg64, op=dist.ReduceOp.SUM, group=group)
        return dg64
    import datetime
    import time

    work = dist.all_reduce(dg64, op=dist.ReduceOp.SUM, group=group, async_op=True)
    if dg64.is_cuda:
        work.wait()                                   # stream-ordered: returns once the collective is enqueued
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(dg64.device))
        deadline = time.monotonic() + float(timeout_s)
        while not done.query():
            if time.monotonic() > deadline:
                raise ExchangeTimeout(f"dgamma all-reduce not complete after {timeout_s} s")
            time.sleep(0.0005)
        return dg64
    try:
        ok = work.wait(timeout=datetime.timedelta(seconds=float(timeout_s)))
    except RuntimeError as e:                         # gloo reports an expired wait as a RuntimeError
        raise ExchangeTimeout(f"dgamma all-reduce not complete after {timeout_s} s: {e}") from None
    if ok is False:
        raise ExchangeTimeout(f"dgamma all-reduce not complete after {timeout_s} s")
    return dg64


class RowShardedRMSNorm:
    def __init__(self, hidden, dtype=torch.float32, eps=1e-5, device=None, group=None, chunk_rows=None, overlap=True,
                 exchange="auto", exchange_timeout_s=None):
        """exchange_timeout_s: host-side deadline of every BLOCKING dgamma exchange of this executor
        (fwd_bwd with overlap off, fwd_bwd_host, and wait_dgamma(timeout_s=...) for the overlapped one);
        ExchangeTimeout is raised when it runs out.  None waits as long as the process group does."""
        self.exchange_timeout_s = exchange_timeout_s
        self.hidden = int(hidden)
        self.dtype = dtype
        self.eps = float(eps)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.group = group
        self.world = 1
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            self.world = torch.distributed.get_world_size(group)
        self._ws = None
        self._dg64 = torch.zeros(self.hidden, dtype=torch.float64, device=self.device)
        # overlapped exchange: two fp64 buffers used in turn, a side stream, one "reduced" event per buffer
        self.overlap = bool(overlap) and self.world > 1
        self._dg64_ring = [self._dg64, torch.zeros_like(self._dg64)] if self.overlap else [self._dg64]
        self._side = torch.cuda.Stream(self.device) if self.overlap else None
        self._reduced = [None, None]
        self._newest = None
        self._turn = 0
        self._chunk_rows = chunk_rows
        self._slots = None
        self._streams = None
        # How the fp64 dgamma sums cross the ranks: "collective" = torch.distributed all-reduce (NCCL, or gloo
        # on CPU); "peer" = the library's own kernels over CUDA-IPC peer mappings (PeerExchange; CUDA ranks of
        # one node): the backward's last kernel stores this rank's sums into every rank's block, one small
        # kernel per rank adds the local copies.  "auto" takes the peer exchange on CUDA ranks with the
        # overlapped mode -- measured on the row-sharded bf16 configuration (65536 x 8192 rows per rank):
        # 8 GPUs 0.946-0.948 ms per step against 0.952-0.956 with the NCCL all-reduce, 2 GPUs 0.923 against
        # 0.925-0.929, and with a smaller spread between blocks -- and falls back to the collective if the
        # blocks cannot be mapped (ranks on different nodes, no peer access).
        if exchange not in ("auto", "peer", "collective"):
            raise ValueError("exchange must be 'auto', 'peer' or 'collective'")
        self._peer = None
        want_peer = exchange == "peer" or (exchange == "auto" and self.device.type == "cuda" and self.overlap)
        if self.world > 1 and want_peer:
            if self.device.type != "cuda":
                raise ValueError("exchange='peer' needs CUDA ranks")
            from .peer_exchange import PeerExchange

            try:
                self._peer = PeerExchange(self.hidden, group=group, device=self.device)
            except RuntimeError:
                if exchange == "peer":
                    raise
                self._peer = None      # every rank fails together (the constructor agrees on it): use the collective
        self.exchange = "peer" if self._peer is not None else ("collective" if self.world > 1 else "none")

    def close(self):
        """Collective when the peer exchange is in use: every rank must call it (before the process group goes)."""
        if getattr(self, "_pipe", None) is not None:
            from . import _lib

            _lib.lib().agb_host_pipe_destroy(self._pipe)
            self._pipe = None
        if self._peer is not None:
            self._peer.close()
            self._peer = None

    # ------------------------------------------------------------------ device-resident path
    def _workspace(self, x):
        if self._ws is None:
            self._ws = ops.bwd_workspace(x)
        return self._ws

    def fwd_bwd(self, x, gy, gamma, y=None, rstd=None, dx=None, dgamma=None, wait=True):
        """One pass over this rank's rows.  Returns (y, rstd, dx, dgamma); dgamma is the sum over
        ALL ranks' rows (fp32 [hidden]).  wait=False leaves the exchange running on the side stream
        (call wait_dgamma() before dgamma is read) so that it overlaps the next step."""
        y, rstd = ops.rmsnorm_fwd(x, gamma, self.eps, out=y, rstd=rstd)
        if gamma is None:
            dx, _ = ops.rmsnorm_bwd(x, None, rstd, gy, dx=dx)
            return y, rstd, dx, None
        if self.world == 1:
            dx, dgamma = ops.rmsnorm_bwd(x, gamma, rstd, gy, dx=dx, dgamma=dgamma, workspace=self._workspace(x))
            return y, rstd, dx, dgamma
        if dgamma is None:
            dgamma = torch.empty(self.hidden, dtype=torch.float32, device=self.device)
        if self._peer is not None and not self.overlap:
            dx = torch.empty_like(x) if dx is None else dx
            self._peer.rmsnorm_bwd(x, gamma, rstd, gy, dx, self._workspace(x))
            self._peer.exchange(dgamma, self.hidden)
            return y, rstd, dx, dgamma
        if not self.overlap:
            dx, _ = ops.rmsnorm_bwd(x, gamma, rstd, gy, dx=dx, dgamma=self._dg64, workspace=self._workspace(x))
            allreduce_dgamma_f64(self._dg64, self.group, self.exchange_timeout_s)
            ops.dgamma_finalize(self._dg64, dgamma)
            return y, rstd, dx, dgamma
        dx = self.bwd_and_exchange(x, gamma, rstd, gy, dx, dgamma)
        if wait:
            self.wait_dgamma()
        return y, rstd, dx, dgamma

    def bwd_and_exchange(self, x, gamma, rstd, gy, dx, dgamma):
        """Backward on the current stream; all-reduce + rounding of dgamma on the side stream.  The
        caller's stream does not wait for the exchange: call wait_dgamma() before reading dgamma."""
        cur = torch.cuda.current_stream(self.device)
        if self._peer is not None:
            # the library's own exchange: the backward's column reduction waits for the buffer (eight steps old)
            # and publishes the sums -- on the side stream, like the summing kernel that waits for the other
            # ranks, so that the caller's stream carries the backward kernel only
            dx = torch.empty_like(x) if dx is None else dx
            self._peer.rmsnorm_bwd(x, gamma, rstd, gy, dx, self._workspace(x), stream=cur, side_stream=self._side)
            self._peer.exchange(dgamma, self.hidden, stream=cur, sum_stream=self._side)
            return dx
        slot = self._turn
        self._turn ^= 1
        buf = self._dg64_ring[slot]
        if self._reduced[slot] is not None:
            cur.wait_event(self._reduced[slot])          # the exchange that last used this buffer
        dx, _ = ops.rmsnorm_bwd(x, gamma, rstd, gy, dx=dx, dgamma=buf, workspace=self._workspace(x))
        self._side.wait_stream(cur)
        with torch.cuda.stream(self._side):
            allreduce_dgamma_f64(buf, self.group)
            ops.dgamma_finalize(buf, dgamma)
            ev = torch.cuda.Event()
            ev.record()
        self._reduced[slot] = ev
        self._newest = ev
        return dx

    def wait_dgamma(self, timeout_s=None):
        """Orders the current stream after the newest dgamma exchange (no-op without overlap).  With timeout_s
        the HOST also waits, at most that long, for the exchange to have completed, and raises ExchangeTimeout
        otherwise (a rank that never arrived)."""
        if not self.overlap:
            return
        if self._peer is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._side)
            ev = torch.cuda.Event()
            ev.record(self._side)
        else:
            if self._newest is None:
                return
            torch.cuda.current_stream(self.device).wait_event(self._newest)
            ev = self._newest
        if timeout_s is not None:
            import time

            deadline = time.monotonic() + float(timeout_s)
            while not ev.query():
                if time.monotonic() > deadline:
                    raise ExchangeTimeout(f"dgamma exchange not complete after {timeout_s} s")
                time.sleep(0.0005)

    def prepare_step(self, x, gy, gamma, y, rstd, dx, dgamma):
        """For loops that repeat a step over the same buffers: validates the operands once and returns an
        object whose fwd() and bwd() enqueue the forward, and the VJP with the dgamma exchange, with the
        fewest host calls.  With the peer exchange these are three bare C-ABI calls with prebuilt arguments
        (the host work per step matters once eight ranks share the host's cores); otherwise they call
        rmsnorm_fwd / bwd_and_exchange.  dgamma is final after wait_dgamma()."""
        import ctypes as C

        from . import _lib

        ex = self
        rows, hidden = ops._rows_hidden(x)
        ops._same(x, gy, y, dx)
        ops._vec(x, hidden, x.dtype, gamma)
        ops._vec(x, hidden, torch.float32, dgamma)
        ops._vec(x, rows, torch.float32, rstd)
        if hidden != self.hidden or x.dtype != self.dtype:
            raise ValueError("operands do not match the executor's hidden / dtype")

        class _Slow:
            def fwd(self_inner):
                ops.rmsnorm_fwd(x, gamma, ex.eps, out=y, rstd=rstd)

            def bwd(self_inner):
                if ex.world == 1:
                    ops.rmsnorm_bwd(x, gamma, rstd, gy, dx=dx, dgamma=dgamma, workspace=ex._workspace(x))
                elif ex.overlap:
                    ex.bwd_and_exchange(x, gamma, rstd, gy, dx, dgamma)
                else:
                    ex.fwd_bwd(x, gy, gamma, y=y, rstd=rstd, dx=dx, dgamma=dgamma)

        if self._peer is None or not self.overlap:
            return _Slow()
        lib, p, vp = _lib.lib(), ops._p, C.c_void_p
        ws = self._workspace(x)
        cur = torch.cuda.current_stream(self.device)
        main, side = vp(cur.cuda_stream), vp(self._side.cuda_stream)
        fwd_args = (p(x), p(gamma), p(y), p(rstd), rows, hidden, C.c_float(self.eps), ops._dt(x), main)
        bwd_args = (self._peer._h, p(x), p(gamma), p(rstd), p(gy), None, p(dx), p(ws), ws.numel() * ws.element_size(),
                    rows, hidden, ops._dt(x), main, side)
        exc_args = (self._peer._h, p(dgamma), hidden, 0, main, side)
        keep = (x, gy, gamma, y, rstd, dx, dgamma, ws)     # the prebuilt pointers must stay valid

        class _Fast:
            _keep = keep

            def fwd(self_inner):
                _lib.check(lib.agb_rmsnorm_fwd(*fwd_args))

            def bwd(self_inner):
                _lib.check(lib.agb_peer_rmsnorm_bwd_overlapped(*bwd_args))
                _lib.check(lib.agb_peer_exchange(*exc_args))

        return _Fast()

    # ------------------------------------------------------------------ host-buffer path
    def _ensure_slots(self, chunk_rows, nslots=3):
        if self._slots is not None and self._slots[0]["x"].shape[0] >= chunk_rows:
            return
        mk = lambda: torch.empty(chunk_rows, self.hidden, dtype=self.dtype, device=self.device)  # noqa: E731
        self._slots = []
        for _ in range(nslots):
            s = dict(x=mk(), gy=mk(), y=mk(), dx=mk(),
                     rstd=torch.empty(chunk_rows, dtype=torch.float32, device=self.device),
                     in_ready=torch.cuda.Event(), done=torch.cuda.Event(), out_done=torch.cuda.Event())
            self._slots.append(s)
        self._streams = dict(h2d=torch.cuda.Stream(self.device), compute=torch.cuda.Stream(self.device),
                             d2h=torch.cuda.Stream(self.device))
        self._gamma_dev = torch.empty(self.hidden, dtype=self.dtype, device=self.device)
        self._dg32 = torch.empty(self.hidden, dtype=torch.float32, device=self.device)

    def default_chunk_rows(self, rows):
        if self._chunk_rows:
            return min(rows, self._chunk_rows)
        # ~64 MB per array and chunk: long enough to run PCIe at full rate, short enough to overlap
        per_row = self.hidden * torch.empty((), dtype=self.dtype).element_size()
        return max(1, min(rows, (64 << 20) // per_row))

    def _host_pipe(self):
        """The library's own host-buffer pipe (include/agb/agb_host.h), created on first use."""
        import ctypes as C

        from . import _lib

        if getattr(self, "_pipe", None) is None:
            h = C.c_void_p()
            with torch.cuda.device(self.device):
                _lib.check(_lib.lib().agb_host_pipe_create(self.hidden, ops._DT[self.dtype], int(self._chunk_rows or 0), C.byref(h)))
            self._pipe = h
        return self._pipe

    def fwd_bwd_host(self, x_host, gy_host, gamma_host, y_host, dx_host, dgamma_host, rstd_host=None):
        """x_host, gy_host [rows, hidden] and gamma_host [hidden] are pinned host tensors; y_host,
        dx_host, dgamma_host (fp32 [hidden]) and optionally rstd_host receive the results.
        Returns when everything has landed in host memory.  A single rank goes through the library's own
        host-buffer entry point (agb_host_pipe_fwd_bwd: the call a C or C++ user makes); with several ranks the
        same pipeline runs here, around the all-reduce of the dgamma sums."""
        rows = x_host.shape[0]
        if self.world == 1:
            import ctypes as C

            from . import _lib

            for t in (x_host, gy_host, y_host, dx_host):
                if t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype or t.shape != x_host.shape:
                    raise ValueError("fwd_bwd_host: contiguous host tensors of the executor's dtype and one shape, please")
            hp = lambda t: None if t is None else C.c_void_p(t.data_ptr())  # noqa: E731
            with torch.cuda.device(self.device):
                _lib.check(_lib.lib().agb_host_pipe_fwd_bwd(self._host_pipe(), hp(x_host), hp(gy_host), hp(gamma_host), hp(y_host),
                                                            hp(dx_host), hp(dgamma_host), hp(rstd_host), rows, self.eps, None))
            return y_host, dx_host, dgamma_host
        chunk = self.default_chunk_rows(rows)
        self._ensure_slots(chunk)
        st = self._streams
        cur = torch.cuda.current_stream(self.device)
        for s in st.values():
            s.wait_stream(cur)
        with torch.cuda.stream(st["h2d"]):
            self._gamma_dev.copy_(gamma_host, non_blocking=True)
            gamma_ready = torch.cuda.Event()
            gamma_ready.record()
        nchunks = (rows + chunk - 1) // chunk
        if nchunks == 0:
            # an empty shard (more ranks than rows) contributes zeros, not the sums of an earlier call
            with torch.cuda.stream(st["compute"]):
                self._dg64.zero_()
        first = True
        for c in range(nchunks):
            r0, r1 = c * chunk, min(rows, (c + 1) * chunk)
            n = r1 - r0
            s = self._slots[c % len(self._slots)]
            with torch.cuda.stream(st["h2d"]):
                if c >= len(self._slots):
                    st["h2d"].wait_event(s["done"])      # kernels of the chunk that used this slot
                s["x"][:n].copy_(x_host[r0:r1], non_blocking=True)
                s["gy"][:n].copy_(gy_host[r0:r1], non_blocking=True)
                s["in_ready"].record()
            with torch.cuda.stream(st["compute"]):
                st["compute"].wait_event(s["in_ready"])
                if first:
                    st["compute"].wait_event(gamma_ready)
                if c >= len(self._slots):
                    st["compute"].wait_event(s["out_done"])  # outputs of the previous user copied out
                x, gy = s["x"][:n], s["gy"][:n]
                y, rstd = ops.rmsnorm_fwd(x, self._gamma_dev, self.eps, out=s["y"][:n], rstd=s["rstd"][:n])
                ops.rmsnorm_bwd(x, self._gamma_dev, rstd, gy, dx=s["dx"][:n], dgamma=self._dg64,
                                accumulate_dgamma=not first, workspace=self._workspace(x))
                s["done"].record()
                first = False
            with torch.cuda.stream(st["d2h"]):
                st["d2h"].wait_event(s["done"])
                y_host[r0:r1].copy_(s["y"][:n], non_blocking=True)
                dx_host[r0:r1].copy_(s["dx"][:n], non_blocking=True)
                if rstd_host is not None:
                    rstd_host[r0:r1].copy_(s["rstd"][:n], non_blocking=True)
                s["out_done"].record()
        with torch.cuda.stream(st["compute"]):
            allreduce_dgamma_f64(self._dg64, self.group, self.exchange_timeout_s)
            ops.dgamma_finalize(self._dg64, self._dg32)
            dgamma_host.copy_(self._dg32, non_blocking=True)
        for s in st.values():
            cur.wait_stream(s)
        cur.synchronize()
        return y_host, dx_host, dgamma_host
