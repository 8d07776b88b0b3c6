"""The allocator's C ABI (include/agb/agb_alloc.h, exported by libagb_host.so): the host-side behaviour
without a GPU, the caching behaviour with one."""
import ctypes as C
import os
import re

import pytest

from cgadimpl_b200.host import build as host_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    so = host_build.build()
    L = C.CDLL(so)
    L.agb_alloc_last_error.restype = C.c_char_p
    L.agb_malloc_async.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.c_void_p]
    L.agb_free_async.argtypes = [C.c_void_p]
    L.agb_arena_reserve.argtypes = [C.c_size_t, C.c_int, C.c_void_p]
    L.agb_alloc_set_limit.argtypes = [C.c_size_t]
    L.agb_alloc_stats.argtypes = [C.POINTER(C.c_size_t)]
    return L


def _stats(lib):
    out = (C.c_size_t * 5)()
    assert lib.agb_alloc_stats(out) == 0
    return dict(zip(("in_use", "cached", "device_allocs", "cache_hits", "peak"), out))


def test_every_declared_symbol_is_exported(lib):
    text = open(os.path.join(ROOT, "include", "agb", "agb_alloc.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(agb_[a-z0-9_]+)\s*\(", text)))
    assert names == ["agb_alloc_empty_cache", "agb_alloc_last_error", "agb_alloc_set_limit", "agb_alloc_stats",
                     "agb_arena_reserve", "agb_free_async", "agb_malloc_async"]
    for n in names:
        assert hasattr(lib, n), n


def test_host_side_failures_need_no_device(lib):
    p = C.c_void_p()
    assert lib.agb_alloc_set_limit(1 << 20) == 0
    try:
        assert lib.agb_malloc_async(C.byref(p), 8 << 20, 0, None) == 1          # refused before any CUDA call
        assert b"out of memory" in lib.agb_alloc_last_error() and not p.value
    finally:
        assert lib.agb_alloc_set_limit(0) == 0
    assert lib.agb_malloc_async(None, 16, 0, None) == 1
    assert lib.agb_free_async(None) == 0                                          # like free(NULL)
    assert lib.agb_free_async(C.c_void_p(0x1000)) == 1                            # not ours
    assert b"not handed out" in lib.agb_alloc_last_error()
    assert lib.agb_alloc_stats(None) == 1
    assert _stats(lib)["device_allocs"] == 0


@pytest.mark.gpu
def test_blocks_are_reused_per_stream(lib):
    import torch

    s0 = _stats(lib)
    a, b = C.c_void_p(), C.c_void_p()
    assert lib.agb_malloc_async(C.byref(a), 3 << 20, 0, None) == 0 and a.value
    s1 = _stats(lib)
    assert s1["in_use"] - s0["in_use"] >= 3 << 20
    assert lib.agb_free_async(a) == 0
    assert lib.agb_free_async(a) == 1                                             # double free is reported
    assert lib.agb_malloc_async(C.byref(b), 3 << 20, 0, None) == 0
    assert b.value == a.value                                                     # same stream: the cached block comes back
    assert _stats(lib)["cache_hits"] == s1["cache_hits"] + 1
    # another stream does not get that block while it is in use, nor after it was freed on the first stream
    st = torch.cuda.Stream()
    c = C.c_void_p()
    assert lib.agb_free_async(b) == 0
    assert lib.agb_malloc_async(C.byref(c), 3 << 20, 0, C.c_void_p(st.cuda_stream)) == 0
    assert c.value != a.value
    assert lib.agb_free_async(c) == 0
    # reserve pre-populates: the next request on that stream is a hit, with no cudaMalloc
    assert lib.agb_arena_reserve(5 << 20, 0, C.c_void_p(st.cuda_stream)) == 0
    before = _stats(lib)
    d = C.c_void_p()
    assert lib.agb_malloc_async(C.byref(d), 5 << 20, 0, C.c_void_p(st.cuda_stream)) == 0
    after = _stats(lib)
    assert after["cache_hits"] == before["cache_hits"] + 1 and after["device_allocs"] == before["device_allocs"]
    assert lib.agb_free_async(d) == 0
    assert lib.agb_alloc_empty_cache() == 0
    assert _stats(lib)["cached"] == 0
