/*
 * agb_alloc.h -- C ABI of the stream-ordered caching device allocator (libagb_host.so).
 *
 * The reference takes its device memory from its tensor library (OwnTensor; every op result and every
 * gradient is one allocation, e.g. cgadimpl/src/core/graph.cpp:36, cgadimpl/src/ops/normalization.cpp:24-27,
 * and its graph runner relies on that library's pool being warm, cgadimpl/src/runtime/cuda_graphs.cpp:37-38).
 * That library is not part of the reference tree; these entry points are what a pointer-only caller of
 * libagb_cuda.so binds instead.  The C++ host layer (namespace OwnTensor, TensorLib.h) sits on the same
 * allocator.
 *
 * Semantics: a block freed on stream S is handed out again only to requests made on S, so stream order
 * makes the reuse safe without events.  A request that misses the cache calls cudaMalloc, except while S
 * is being captured into a CUDA graph, where it fails: warm the cache first (run once, or reserve).
 * All functions return 0 on success, non-zero on failure with a message in agb_alloc_last_error()
 * (thread-local); none of them calls exit().
 */
#ifndef AGB_ALLOC_H
#define AGB_ALLOC_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* agb_alloc_stream_t; /* == cudaStream_t */

int agb_malloc_async(void** ptr, size_t bytes, int device, agb_alloc_stream_t stream);
int agb_free_async(void* ptr);                  /* back to the cache of the stream it was allocated on */
int agb_arena_reserve(size_t bytes, int device, agb_alloc_stream_t stream); /* pre-populates the cache with one block */
int agb_alloc_empty_cache(void);                /* cudaFree of every cached block that is not in use */
int agb_alloc_set_limit(size_t bytes);          /* 0 = unlimited; a request beyond it fails on the host, no cudaMalloc */
/* out: bytes in use, bytes cached, cudaMalloc calls, cache hits, peak bytes in use */
int agb_alloc_stats(size_t out[5]);
const char* agb_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
