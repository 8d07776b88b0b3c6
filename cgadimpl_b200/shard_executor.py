"""ctypes front end of the single-process, multi-GPU executor (include/agb/agb_shard.h).

One host process drives several GPUs: every shard runs the forward and the VJP on its own device
and stream, and the [hidden] fp64 dgamma sums are added across shards by one small kernel per shard
that reads the others' sums through NVLink peer mappings.  `RowShardedRMSNorm` (executor.py) is the
one-process-per-GPU counterpart with an NCCL all-reduce in the same place.

torch supplies device memory only.  The executor runs on streams of its own: `run` makes those
streams wait for the work already enqueued on torch's current stream of each device, and
`synchronize` waits for the executor before results are read.
"""
import ctypes as C

import torch

from . import _lib, ops
from ._lib import check


class ShardExecutor:
    def __init__(self, devices, max_hidden):
        self.devices = [int(d) for d in devices]
        self.max_hidden = int(max_hidden)
        self._h = C.c_void_p()
        arr = (C.c_int * len(self.devices))(*self.devices)
        check(_lib.lib().agb_shard_create(arr, len(self.devices), self.max_hidden, C.byref(self._h)))
        self._streams = []
        for i in range(len(self.devices)):
            s = C.c_void_p()
            check(_lib.lib().agb_shard_stream(self._h, i, C.byref(s)))
            self._streams.append(torch.cuda.ExternalStream(s.value, device=torch.device("cuda", self.devices[i])))

    def __len__(self):
        return int(_lib.lib().agb_shard_count(self._h))

    def stream(self, i):
        return self._streams[i]

    def _io(self, xs, gammas, gys, ys, rstds, dxs, dgammas, dx_adds):
        n = len(self.devices)
        for name, seq in (("x", xs), ("gamma", gammas), ("gy", gys), ("y", ys), ("rstd", rstds), ("dx", dxs),
                          ("dgamma", dgammas), ("dx_add", dx_adds)):
            if len(seq) != n:
                raise ValueError(f"{name}: {len(seq)} entries for {n} shards")
        io = (_lib.ShardIO * n)()
        hidden, dtype = xs[0].shape[-1], xs[0].dtype
        for i in range(n):
            x = xs[i]
            dev = torch.device("cuda", self.devices[i])
            if x.device != dev:
                raise ValueError(f"shard {i}: x on {x.device}, executor shard on {dev}")
            if x.shape[-1] != hidden or x.dtype != dtype:
                raise ValueError("all shards must share hidden and dtype")
            rows, _ = ops._rows_hidden(x)
            ops._same(x, gys[i], ys[i], dxs[i], dx_adds[i])
            ops._vec(x, hidden, dtype, gammas[i])
            ops._vec(x, hidden, torch.float32, dgammas[i])
            ops._vec(x, rows, torch.float32, rstds[i])
            p = lambda t: None if t is None else t.data_ptr()
            io[i] = _lib.ShardIO(p(x), p(gammas[i]), p(gys[i]), p(dx_adds[i]), p(ys[i]), p(rstds[i]), p(dxs[i]),
                                 p(dgammas[i]), rows)
        return io, hidden, ops._dt(xs[0])

    def _after_current_streams(self):
        for i, d in enumerate(self.devices):
            self._streams[i].wait_stream(torch.cuda.current_stream(torch.device("cuda", d)))

    def fwd_bwd(self, xs, gammas, gys, eps=1e-5, ys=None, rstds=None, dxs=None, dgammas=None, dx_adds=None,
                accumulate_dgamma=False):
        """Enqueues forward + VJP + dgamma exchange on every shard; returns (ys, rstds, dxs, dgammas).
        Outputs that are not passed in are allocated here.  Call synchronize() before reading them."""
        n = len(self.devices)
        ys = [torch.empty_like(x) for x in xs] if ys is None else ys
        dxs = [torch.empty_like(x) for x in xs] if dxs is None else dxs
        rstds = [torch.empty(ops._rows_hidden(x)[0], dtype=torch.float32, device=x.device) for x in xs] \
            if rstds is None else rstds
        if dgammas is None:
            dgammas = [None if g is None else torch.empty(x.shape[-1], dtype=torch.float32, device=x.device)
                       for x, g in zip(xs, gammas)]
        dx_adds = [None] * n if dx_adds is None else dx_adds
        io, hidden, dt = self._io(xs, gammas, gys, ys, rstds, dxs, dgammas, dx_adds)
        self._after_current_streams()
        check(_lib.lib().agb_shard_run_fwd_bwd(self._h, io, hidden, float(eps), dt, int(bool(accumulate_dgamma))))
        return ys, rstds, dxs, dgammas

    def run_prepared(self, io, hidden, eps, dt, accumulate_dgamma=False):
        """The bare call with a prepared io array (from prepare()): what a timing loop repeats."""
        check(_lib.lib().agb_shard_run_fwd_bwd(self._h, io, hidden, float(eps), dt, int(bool(accumulate_dgamma))))

    def prepare(self, xs, gammas, gys, ys, rstds, dxs, dgammas, dx_adds=None):
        return self._io(xs, gammas, gys, ys, rstds, dxs, dgammas, [None] * len(self.devices) if dx_adds is None else dx_adds)

    def set_deferred_exchange(self, on):
        """Run the dgamma exchange on side streams (see agb_shard_set_deferred_exchange)."""
        check(_lib.lib().agb_shard_set_deferred_exchange(self._h, int(bool(on))))

    def wait_dgamma(self):
        check(_lib.lib().agb_shard_wait_dgamma(self._h))

    def synchronize(self):
        check(_lib.lib().agb_shard_synchronize(self._h))

    def close(self):
        if self._h:
            check(_lib.lib().agb_shard_destroy(self._h))
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
