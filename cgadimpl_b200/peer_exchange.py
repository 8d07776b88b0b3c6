"""The dgamma exchange between ranks that are separate processes (agb_peer_* of include/agb/agb_shard.h).

Every rank owns a small device block (two fp64 [hidden] sum buffers, a ready and an ack counter each)
and maps the blocks of the other ranks through CUDA IPC; one kernel per rank then adds all ranks' sums
in rank order over NVLink peer loads.  torch.distributed is used at set-up, to collect the 64-byte IPC
handles of all ranks, and at close, for the barriers that must precede unmapping and freeing the blocks.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import check

HANDLE_BYTES = 64


class PeerExchange:
    """One per rank.  Collective constructor (all ranks of `group` must call it) and close()."""

    def __init__(self, max_hidden, group=None, device=None):
        import torch.distributed as dist

        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_hidden = int(max_hidden)
        self._h = C.c_void_p()
        lib = _lib.lib()

        def all_ok(ok):   # every collective below is entered by every rank, whatever happened locally
            t = torch.tensor([1 if ok else 0], device=self.device, dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return bool(t.item())

        handle = C.create_string_buffer(HANDLE_BYTES)
        with torch.cuda.device(self.device):
            st = lib.agb_peer_create(self.rank, self.world, self.max_hidden, C.byref(self._h), handle)
            err = lib.agb_last_error().decode() if st != 0 else ""
            if not all_ok(st == 0):
                self._drop_local()
                raise RuntimeError(f"peer exchange: creating the device block failed on some rank ({err or 'not here'})")
            # gather the handles with a SUM all-reduce of a [world, 64] table that is zero outside this rank's
            # row: unlike all_gather it exists for every algorithm a caller may have pinned NCCL to
            table = torch.zeros(self.world, HANDLE_BYTES, dtype=torch.int32, device=self.device)
            table[self.rank] = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).to(self.device, torch.int32)
            dist.all_reduce(table, op=dist.ReduceOp.SUM, group=group)
            blob = table.to(torch.uint8).cpu().numpy().tobytes()
            st = lib.agb_peer_connect(self._h, blob)
            err = lib.agb_last_error().decode() if st != 0 else ""
            torch.cuda.synchronize(self.device)
            if not all_ok(st == 0):      # (the MIN all-reduce is also the barrier: everybody has mapped everybody)
                lib.agb_peer_disconnect(self._h)
                dist.barrier(group)
                self._drop_local()
                raise RuntimeError(f"peer exchange: mapping the other ranks' blocks failed on some rank ({err or 'not here'})")

    def _drop_local(self):
        if self._h:
            with torch.cuda.device(self.device):
                _lib.lib().agb_peer_destroy(self._h)
            self._h = C.c_void_p()

    def acquire(self, stream=None):
        """Enqueues the wait for this step's sum buffer and returns its device address (int): where the
        backward must leave its fp64 sums (ops.rmsnorm_bwd(..., dgamma_f64_ptr=address))."""
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        out = C.c_void_p()
        check(_lib.lib().agb_peer_acquire(self._h, C.c_void_p(s.cuda_stream), C.byref(out)))
        return out.value

    def rmsnorm_bwd(self, x, gamma, rstd, gy, dx, workspace, dx_add=None, stream=None, side_stream=None):
        """The VJP of this rank's rows with the exchange's bookkeeping fused into its last kernel
        (agb_peer_rmsnorm_bwd): no extra launch on the backward's stream.  With side_stream that last kernel,
        the publishing column reduction, runs there (agb_peer_rmsnorm_bwd_overlapped).  Follow with exchange()
        (with sum_stream=side_stream in the second case)."""
        from . import ops

        rows, hidden = ops._rows_hidden(x)
        ops._same(x, gy, dx_add, dx)
        ops._vec(x, hidden, x.dtype, gamma)
        ops._vec(x, rows, torch.float32, rstd)
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        p = ops._p
        if side_stream is not None:
            check(_lib.lib().agb_peer_rmsnorm_bwd_overlapped(self._h, p(x), p(gamma), p(rstd), p(gy), p(dx_add), p(dx),
                                                             p(workspace), workspace.numel() * workspace.element_size(),
                                                             rows, hidden, ops._dt(x), C.c_void_p(s.cuda_stream),
                                                             C.c_void_p(side_stream.cuda_stream)))
            return dx
        check(_lib.lib().agb_peer_rmsnorm_bwd(self._h, p(x), p(gamma), p(rstd), p(gy), p(dx_add), p(dx), p(workspace),
                                              workspace.numel() * workspace.element_size(), rows, hidden, ops._dt(x),
                                              C.c_void_p(s.cuda_stream)))
        return dx

    def exchange(self, dgamma, hidden, accumulate=False, stream=None, sum_stream=None):
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        q = s if sum_stream is None else sum_stream
        check(_lib.lib().agb_peer_exchange(self._h, C.c_void_p(dgamma.data_ptr()), int(hidden), int(bool(accumulate)),
                                           C.c_void_p(s.cuda_stream), C.c_void_p(q.cuda_stream)))

    def close(self):
        """Collective: synchronise, barrier, then unmap and free."""
        if not self._h:
            return
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)                 # no kernel of any rank still reads a peer's block
        with torch.cuda.device(self.device):
            check(_lib.lib().agb_peer_disconnect(self._h))
        dist.barrier(self.group)                 # nobody has anybody's block mapped any more
        with torch.cuda.device(self.device):
            check(_lib.lib().agb_peer_destroy(self._h))
        self._h = C.c_void_p()
