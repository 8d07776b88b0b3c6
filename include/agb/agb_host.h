/*
 * agb_host.h -- RMSNorm forward + VJP over HOST buffers (exported by libagb_cuda.so).
 *
 * The entry points of agb.h take device pointers.  A caller whose activations live in host memory (the
 * reference's tensors start on the CPU and move with Tensor::to, cgadimpl/include/tensor.hpp:6-15) uses this
 * pipe instead: rows are cut into chunks, and chunk k's host-to-device copy, kernels and device-to-host copy
 * run on three streams over three sets of device buffers, so transfers in both directions overlap the
 * kernels and the whole pass runs at the speed of the PCIe link.  dgamma is accumulated over the chunks as
 * an un-rounded fp64 column sum and rounded once at the end, so it does not depend on the chunking
 * (fp32 I/O: the bits of one agb_rmsnorm_bwd call over all rows, up to fp64 rounding).
 *
 * agb_host_pipe_create / _destroy allocate and free device memory, streams and events on the current
 * device; agb_host_pipe_fwd_bwd only enqueues and waits.  Host buffers should be page-locked
 * (cudaHostAlloc / cudaHostRegister): with pageable memory the copies are staged by the driver and do not
 * overlap.  A pipe is not thread-safe: one host thread drives it at a time.
 */
#ifndef AGB_AGB_HOST_H
#define AGB_AGB_HOST_H

#include "agb/agb.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct agb_host_pipe agb_host_pipe_t;

/* hidden and dtype (AGB_F32 / AGB_BF16) are fixed for the pipe's life.  chunk_rows = 0 picks chunks of
 * about 64 MB per array (long enough to run the link at full rate, short enough to overlap). */
int agb_host_pipe_create(int64_t hidden, int dtype, int64_t chunk_rows, agb_host_pipe_t** out);
int64_t agb_host_pipe_chunk_rows(const agb_host_pipe_t* p);

/* y = rmsnorm(x) * gamma; dx, dgamma = its VJP for the upstream gradient gy.  All pointers are HOST memory:
 * x, gy, y, dx [rows, hidden] of the pipe's dtype; gamma [hidden] of the pipe's dtype; dgamma [hidden] fp32;
 * rstd [rows] fp32, nullable.  Returns when every result is in host memory.
 * dgamma_sum (nullable, [hidden] doubles, DEVICE memory): if given, the un-rounded column sums are ALSO left
 * there before the rounding, for a caller that all-reduces them across ranks itself. */
int agb_host_pipe_fwd_bwd(agb_host_pipe_t* p, const void* x, const void* gy, const void* gamma, void* y, void* dx,
                          float* dgamma, float* rstd, int64_t rows, float eps, double* dgamma_sum);

/* Synchronises the pipe's streams, then frees everything it owns.  NULL is accepted. */
int agb_host_pipe_destroy(agb_host_pipe_t* p);

#ifdef __cplusplus
}
#endif
#endif /* AGB_AGB_HOST_H */
