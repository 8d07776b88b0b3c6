"""ctypes binding of libagb_cuda.so -- the same entry points a C++ or cgo caller binds.

There is no fallback: if the library is missing this raises, and without a CUDA device every
compute call returns AGB_ERR_CUDA, which is raised as AgbError.
"""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libagb_cuda.so")

AGB_OK = 0
AGB_F32, AGB_BF16, AGB_F64 = 0, 1, 2
REDUCE_SUM, REDUCE_MEAN, REDUCE_MAX = 0, 1, 2

# name -> (restype, argtypes); must list every symbol include/agb/agb.h declares
_vp, _i64, _i, _f, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t
SIGNATURES = {
    "agb_version": (_i, []),
    "agb_status_string": (C.c_char_p, [_i]),
    "agb_last_error": (C.c_char_p, []),
    "agb_launch_count": (C.c_uint64, []),
    "agb_device_status": (_i, []),
    "agb_selftest_bounded_wait": (_i, [_i, _vp, _vp]),
    "agb_set_option": (_i, [C.c_char_p, _i64]),
    "agb_describe_launch": (_i, [_i, _i64, _i64, _i, _i, C.POINTER(_i64)]),
    "agb_rmsnorm_fwd": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _vp]),
    "agb_add_rmsnorm_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _vp]),
    "agb_rmsnorm_bwd_workspace_bytes": (_sz, [_i64, _i64, _i]),
    "agb_rmsnorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _sz, _i64, _i64, _i, _vp]),
    "agb_rmsnorm_bwd_partials": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i, _vp, C.POINTER(_i)]),
    "agb_dgamma_reduce": (_i, [_vp, _i, _i64, _vp, _i, _i, _vp]),
    "agb_rmsnorm_bwd_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _vp]),
    "agb_dgamma_finalize": (_i, [_vp, _vp, _i64, _i, _vp]),
    "agb_rmsnorm_jvp": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "agb_residual_add": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "agb_vjp_add": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "agb_scale_lastdim": (_i, [_vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "agb_binary_broadcast": (_i, [_i, _vp, _vp, _vp, _i64, _i64, _i, _i, _vp]),
    "agb_accumulate_broadcast": (_i, [_vp, _vp, _i64, _i64, _i, _f, _i, _vp]),
    "agb_mul_reduce_workspace_bytes": (_sz, [_i64, _i64]),
    "agb_mul_reduce": (_i, [_vp, _vp, _vp, _i64, _i64, _i, _i, _vp, _sz, _i, _vp]),
    "agb_layernorm_fwd": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _vp]),
    "agb_layernorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _vp]),
    "agb_layernorm_jvp": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _vp]),
    "agb_softmax_row_fwd": (_i, [_vp, _vp, _i64, _i64, _i, _vp]),
    "agb_logsumexp_row_fwd": (_i, [_vp, _vp, _i64, _i64, _i, _vp]),
    "agb_softmax_row_bwd": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "agb_logsumexp_row_bwd": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "agb_logsumexp_row_jvp": (_i, [_vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "agb_sgd_step": (_i, [_vp, _vp, _i64, _f, _i, _vp]),
    "agb_adam_step": (_i, [_vp, _vp, _vp, _vp, _i64, _f, _f, _f, _f, _vp]),
    "agb_row_reduce": (_i, [_i, _vp, _vp, _i64, _i64, _i, _vp]),
    "agb_reduce_all_workspace_bytes": (_sz, [_i64]),
    "agb_reduce_all": (_i, [_i, _vp, _vp, _i64, _i, _vp, _sz, _vp]),
}


class ShardIO(C.Structure):
    """agb_shard_io_t of include/agb/agb_shard.h."""
    _fields_ = [("x", _vp), ("gamma", _vp), ("gy", _vp), ("dx_add", _vp), ("y", _vp), ("rstd", _vp), ("dx", _vp),
                ("dgamma", _vp), ("rows", _i64)]


# every symbol include/agb/agb_shard.h declares (same library)
SHARD_SIGNATURES = {
    "agb_shard_create": (_i, [C.POINTER(_i), _i, _i64, C.POINTER(_vp)]),
    "agb_shard_count": (_i, [_vp]),
    "agb_shard_stream": (_i, [_vp, _i, C.POINTER(_vp)]),
    "agb_shard_run_fwd_bwd": (_i, [_vp, C.POINTER(ShardIO), _i64, _f, _i, _i]),
    "agb_shard_run_fwd": (_i, [_vp, C.POINTER(ShardIO), _i64, _f, _i]),
    "agb_shard_run_bwd": (_i, [_vp, C.POINTER(ShardIO), _i64, _i, _i]),
    "agb_shard_set_deferred_exchange": (_i, [_vp, _i]),
    "agb_shard_wait_dgamma": (_i, [_vp]),
    "agb_shard_synchronize": (_i, [_vp]),
    "agb_shard_destroy": (_i, [_vp]),
    "agb_peer_create": (_i, [_i, _i, _i64, C.POINTER(_vp), C.c_char_p]),
    "agb_peer_connect": (_i, [_vp, C.c_char_p]),
    "agb_peer_acquire": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "agb_peer_exchange": (_i, [_vp, _vp, _i64, _i, _vp, _vp]),
    "agb_peer_rmsnorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i, _vp]),
    "agb_peer_rmsnorm_bwd_overlapped": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i, _vp, _vp]),
    "agb_peer_publish": (_i, [_vp, _vp]),
    "agb_peer_sum": (_i, [_vp, _vp, _i64, _i, _vp]),
    "agb_peer_block": (_i, [_vp, C.POINTER(_vp)]),
    "agb_peer_connect_local": (_i, [_vp, C.POINTER(_vp)]),
    "agb_peer_disconnect": (_i, [_vp]),
    "agb_peer_destroy": (_i, [_vp]),
}


# every symbol include/agb/agb_host.h declares (same library)
HOST_SIGNATURES = {
    "agb_host_pipe_create": (_i, [_i64, _i, _i64, C.POINTER(_vp)]),
    "agb_host_pipe_chunk_rows": (_i64, [_vp]),
    "agb_host_pipe_fwd_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _f, _vp]),
    "agb_host_pipe_destroy": (_i, [_vp]),
}


class AgbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"agb status {status}: {message}")
        self.status = status


_lib = None


def lib():
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cgadimpl_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in list(SIGNATURES.items()) + list(SHARD_SIGNATURES.items()) + list(HOST_SIGNATURES.items()):
            fn = getattr(h, name)
            fn.restype = res
            fn.argtypes = args
        _lib = h
    return _lib


def check(status):
    if status != AGB_OK:
        raise AgbError(status, lib().agb_last_error().decode())
