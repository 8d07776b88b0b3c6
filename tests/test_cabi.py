"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and
rejects bad arguments before touching CUDA.  No compute call is made here."""
import ctypes as C
import os
import re

import pytest

from cgadimpl_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def _declared_symbols(header="agb.h"):
    text = open(os.path.join(ROOT, "include", "agb", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(agb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    declared = _declared_symbols()
    assert declared, "no declarations found"
    assert sorted(_lib.SIGNATURES) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in agb.h but not exported"


def test_shard_header_and_binding_agree(lib):
    declared = _declared_symbols("agb_shard.h")
    assert sorted(_lib.SHARD_SIGNATURES) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in agb_shard.h but not exported"


def test_host_header_and_binding_agree(lib):
    declared = _declared_symbols("agb_host.h")
    assert sorted(_lib.HOST_SIGNATURES) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in agb_host.h but not exported"
    out = C.c_void_p()
    assert lib.agb_host_pipe_create(0, 0, 0, C.byref(out)) == 1          # hidden must be positive
    assert lib.agb_host_pipe_create(4096, 7, 0, C.byref(out)) == 2       # unknown dtype
    assert lib.agb_host_pipe_create(4096, 0, 0, None) == 1
    assert lib.agb_host_pipe_fwd_bwd(None, None, None, None, None, None, None, None, 0, 1e-5, None) == 1
    assert lib.agb_host_pipe_destroy(None) == 0 and lib.agb_host_pipe_chunk_rows(None) == 0


def test_shard_argument_validation_needs_no_device(lib):
    out = C.c_void_p()
    devs = (C.c_int * 2)(0, 0)
    assert lib.agb_shard_create(None, 2, 4096, C.byref(out)) == 1
    assert lib.agb_shard_create(devs, 0, 4096, C.byref(out)) == 1
    assert lib.agb_shard_create(devs, 17, 4096, C.byref(out)) == 1
    assert lib.agb_shard_create(devs, 2, 0, C.byref(out)) == 1
    assert lib.agb_shard_create(devs, 2, 4096, None) == 1
    assert out.value is None
    assert lib.agb_shard_count(None) == 0
    assert lib.agb_shard_destroy(None) == 0
    assert lib.agb_shard_synchronize(None) == 1
    io = (_lib.ShardIO * 1)()
    assert lib.agb_shard_run_fwd_bwd(None, io, 4096, 1e-5, 0, 0) == 1


def test_peer_argument_validation_needs_no_device(lib):
    out = C.c_void_p()
    handle = C.create_string_buffer(64)
    assert lib.agb_peer_create(0, 0, 4096, C.byref(out), handle) == 1        # world must be >= 1
    assert lib.agb_peer_create(2, 2, 4096, C.byref(out), handle) == 1        # rank outside the world
    assert lib.agb_peer_create(0, 17, 4096, C.byref(out), handle) == 1       # more ranks than AGB_SHARD_MAX
    assert lib.agb_peer_create(0, 2, 0, C.byref(out), handle) == 1           # max_hidden must be positive
    assert lib.agb_peer_create(0, 2, 4096, None, handle) == 1
    assert out.value is None
    one = C.c_void_p(16)
    for fn, extra in ((lib.agb_peer_rmsnorm_bwd, ()), (lib.agb_peer_rmsnorm_bwd_overlapped, (one,))):
        assert fn(None, one, one, one, one, None, one, one, 1 << 20, 8, 64, 0, None, *extra) == 1   # no exchange object
    assert lib.agb_peer_exchange(None, one, 64, 0, None, None) == 1
    assert lib.agb_peer_sum(None, one, 64, 0, None) == 1 and lib.agb_peer_publish(None, None) == 1
    assert lib.agb_peer_destroy(None) == 0 and lib.agb_peer_disconnect(None) == 0


def test_version_and_strings(lib):
    assert lib.agb_version() >= 100
    assert lib.agb_status_string(0) == b"ok"
    assert b"workspace" in lib.agb_status_string(5)
    assert lib.agb_last_error() is not None


def test_argument_validation_needs_no_device(lib):
    one = C.c_void_p(0x1000)
    # negative rows / zero hidden
    assert lib.agb_rmsnorm_fwd(one, None, one, one, -1, 8, 1e-5, 0, None) == 1
    assert lib.agb_rmsnorm_fwd(one, None, one, one, 4, 0, 1e-5, 0, None) == 1
    # unknown dtype
    assert lib.agb_rmsnorm_fwd(one, None, one, one, 4, 8, 1e-5, 7, None) == 2
    # null x
    assert lib.agb_rmsnorm_fwd(None, None, one, one, 4, 8, 1e-5, 0, None) == 1
    assert b"x is NULL" in lib.agb_last_error()
    # misaligned fp32 pointer
    assert lib.agb_rmsnorm_fwd(C.c_void_p(0x1002), None, one, one, 4, 8, 1e-5, 0, None) == 3
    # dgamma without gamma, bad dgamma dtype
    assert lib.agb_rmsnorm_bwd(one, None, one, one, None, one, one, 0, 0, None, 0, 4, 8, 0, None) == 1
    assert lib.agb_rmsnorm_bwd(one, one, one, one, None, one, one, 1, 0, None, 0, 4, 8, 0, None) == 1
    # tgamma without gamma
    assert lib.agb_rmsnorm_jvp(one, None, one, one, one, one, 4, 8, 0, None) == 1
    # rows == 0 is a no-op that succeeds without a device
    assert lib.agb_rmsnorm_fwd(None, None, None, None, 0, 8, 1e-5, 0, None) == 0
    assert lib.agb_set_option(b"no_such_option", 1) == 1
    assert lib.agb_set_option(b"stages", 0) == 0
    assert lib.agb_reduce_all(2, one, one, 8, 0, one, 8192, None) == 1  # max is not a global op


def test_no_cpu_fallback_without_device(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    one = C.c_void_p(0x1000)
    assert lib.agb_rmsnorm_fwd(one, None, one, one, 4, 8, 1e-5, 0, None) == 4  # AGB_ERR_CUDA
