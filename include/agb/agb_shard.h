/*
 * agb_shard.h -- row-sharded RMSNorm forward + VJP over several GPUs of one node, driven from ONE
 * host process (exported by libagb_cuda.so).
 *
 * The path shards by rows: the forward and dx need nothing from other rows; only dgamma, the column
 * sum of gy * xhat over ALL rows, couples the shards (in cgadimpl it is reduce_for_broadcast inside
 * vjp_Mul, cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:15-35 and :54-59, over the whole tensor).
 * Each shard runs agb_rmsnorm_fwd / agb_rmsnorm_bwd on its own device and stream and leaves its
 * un-rounded fp64 [hidden] column sums in a buffer of the executor.  The exchange is ONE small kernel
 * per shard that reads every shard's sums with ordinary loads -- over NVLink peer mappings when the
 * shards sit on different GPUs -- adds them in shard order in fp64 and rounds once to fp32, so every
 * shard ends with the bit-identical dgamma and the result does not depend on timing.  The kernels are
 * ordered by CUDA events recorded and waited on from the calling host thread; no kernel waits on
 * another kernel, nothing spins, there is no multicast load.
 *
 * A caller with one process per GPU (torch.distributed, MPI) does not need this header: it calls
 * agb_rmsnorm_bwd with dgamma_dtype = AGB_F64, all-reduces the [hidden] doubles with its own
 * collective and finishes with agb_dgamma_finalize.
 *
 * Unlike the entry points of agb.h, agb_shard_create / agb_shard_destroy allocate and free device
 * memory (streams, events, the backward workspace and two fp64 vectors per shard); the run calls
 * only enqueue work.  An executor is not thread-safe: one host thread drives it at a time.
 */
#ifndef AGB_AGB_SHARD_H
#define AGB_AGB_SHARD_H

#include "agb/agb.h"

#ifdef __cplusplus
extern "C" {
#endif

#define AGB_SHARD_MAX 16

typedef struct agb_shard agb_shard_t;

/* What one shard works on; every pointer is device memory of that shard's device.
 *   x, gy, y, dx [rows, hidden]; rstd [rows] fp32; gamma [hidden] (a replica per device; NULL = the
 *   gamma-less rms(x), then dgamma must be NULL); dx_add nullable, same meaning as in
 *   agb_rmsnorm_bwd; dgamma [hidden] fp32 receives the sum over ALL shards (nullable).
 *   rows may differ between shards and may be 0 (the shard then contributes zeros). */
typedef struct {
    const void* x;
    const void* gamma;
    const void* gy;
    const void* dx_add;
    void* y;
    float* rstd;
    void* dx;
    float* dgamma;
    int64_t rows;
} agb_shard_io_t;

/* Creates an executor with one shard per entry of `devices` (CUDA ordinals).  An ordinal may be
 * listed more than once: those shards share the GPU, each on its own stream (useful on a one-GPU
 * machine and in tests).  Distinct devices must be able to map each other's memory
 * (cudaDeviceCanAccessPeer), otherwise AGB_ERR_UNSUPPORTED.  max_hidden bounds the `hidden` of later
 * runs and sizes the workspaces.  The caller's current device is restored before returning. */
int agb_shard_create(const int* devices, int n, int64_t max_hidden, agb_shard_t** out);
int agb_shard_count(const agb_shard_t* s);
/* The stream shard i runs on (a cudaStream_t of devices[i]), so that a caller can order its own
 * copies and kernels before and after a run with events. */
int agb_shard_stream(const agb_shard_t* s, int i, agb_stream_t* stream);

/* Enqueues, on every shard: forward, VJP, then the dgamma exchange.  io[i] belongs to shard i.
 * With accumulate_dgamma the summed dgamma is added to the old contents of each io[i].dgamma.
 * Returns as soon as everything is enqueued. */
int agb_shard_run_fwd_bwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, float eps, int dtype,
                          int accumulate_dgamma);
/* The two halves, for callers that run other work in between (the forward uses x, gamma, y, rstd;
 * the backward x, gamma, rstd, gy, dx_add, dx, dgamma). */
int agb_shard_run_fwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, float eps, int dtype);
int agb_shard_run_bwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, int dtype, int accumulate_dgamma);

/* Deferred exchange (off by default).  In the default mode the dgamma exchange runs on the shard streams,
 * so after a run each shard's stream holds its final dgamma -- and every shard waits, in every run, for
 * the slowest one.  With on != 0 the exchange runs on a second stream per shard with two alternating sum
 * buffers: a shard's stream goes straight on to the next run and only waits, before its backward, until
 * the sums it wrote two runs ago have been read.  dgamma is then final on the shard streams only after
 * agb_shard_wait_dgamma (which makes every shard stream wait for the latest exchange; enqueue-only) or
 * after agb_shard_synchronize.  Switching modes synchronises the executor. */
int agb_shard_set_deferred_exchange(agb_shard_t* s, int on);
int agb_shard_wait_dgamma(agb_shard_t* s);

/* Waits for every shard's stream and returns the worst device status (see agb_device_status). */
int agb_shard_synchronize(agb_shard_t* s);
/* Synchronises, then frees everything the executor owns.  NULL is accepted. */
int agb_shard_destroy(agb_shard_t* s);

/* ---- the same exchange between PROCESSES (one process per GPU, all on one node) ----
 * Each rank owns one device block with, for every rank, two fp64 [max_hidden] slots used in turn plus a
 * "ready" and an "ack" counter per slot, and maps the blocks of all other ranks through CUDA IPC.  The
 * exchange PUSHES: a rank stores its sums and its counters into every rank's block (plain peer stores over
 * NVLink), so every wait polls the waiting GPU's own memory and every read of sums is local.  Per step:
 *   agb_peer_acquire   enqueues, on `stream`, a wait until every rank has read what this rank pushed
 *                      two steps ago, and returns where this step's backward must leave its
 *                      sums (pass it to agb_rmsnorm_bwd as dgamma with dgamma_dtype = AGB_F64);
 *   agb_peer_exchange  enqueues, on `stream`, the publication of those sums (they are stored into every
 *                      rank's block, then the step number with release semantics) and, on `sum_stream`
 *                      (may be the same stream; a second one keeps the caller's stream from waiting for the
 *                      slowest rank), one kernel that waits for every rank's publication of this step, adds
 *                      all ranks' sums in rank order in fp64, rounds once to fp32 into `dgamma` (+= with
 *                      accumulate) and acknowledges the read.  Every rank gets the same bits.
 * Processes cannot order each other's streams with events, so these kernels wait on counters in
 * device memory that kernels on OTHER GPUs write.  Every such wait is bounded (about two seconds);
 * when it runs out the kernel raises the device status word (agb_device_status -> AGB_ERR_TIMEOUT),
 * leaves dgamma untouched and returns.  Never run two ranks on the same GPU.
 * Setup is collective: every rank calls agb_peer_create, the 64-byte handles are all-gathered by the
 * caller's own means (rank order), then every rank calls agb_peer_connect.  Before agb_peer_destroy
 * every rank must have synchronised its device and passed a barrier, so that nobody still reads a
 * block that is being freed. */
#define AGB_PEER_HANDLE_BYTES 64
typedef struct agb_peer agb_peer_t;
int agb_peer_create(int rank, int world, int64_t max_hidden, agb_peer_t** out, unsigned char handle[AGB_PEER_HANDLE_BYTES]);
int agb_peer_connect(agb_peer_t* p, const unsigned char* all_handles /* world * AGB_PEER_HANDLE_BYTES */);
int agb_peer_acquire(agb_peer_t* p, agb_stream_t stream, double** sums);
int agb_peer_exchange(agb_peer_t* p, float* dgamma, int64_t hidden, int accumulate, agb_stream_t stream,
                      agb_stream_t sum_stream);
/* agb_peer_acquire + agb_rmsnorm_bwd + agb_peer_publish in one call and WITHOUT extra kernels: the
 * backward's final column reduction itself waits for the acknowledgements before it overwrites the sum
 * buffer and publishes the step when its last CTA has written.  Follow it with agb_peer_exchange (which
 * then only orders the streams and enqueues the summing kernel) or agb_peer_sum.  Arguments as in
 * agb_rmsnorm_bwd; gamma is required. */
int agb_peer_rmsnorm_bwd(agb_peer_t* p, const void* x, const void* gamma, const float* rstd, const void* gy,
                         const void* dx_add, void* dx, void* workspace, size_t workspace_bytes, int64_t rows,
                         int64_t hidden, int dtype, agb_stream_t stream);
/* The same with the column reduction -- and with it the stores into the peers' blocks and their system-scope
 * fences -- on `side_stream`: `stream` carries only the backward kernel, so the kernels that follow on it do not
 * wait for the publication (among eight ranks about 40 us of a 0.9 ms step).  The partial rows in `workspace`
 * are then read on the side stream; the next call orders `stream` after that reader before its backward
 * overwrites them.  Follow with agb_peer_exchange(p, ..., stream, side_stream) with the SAME side stream (the
 * summing kernel simply follows the reduction there).  side_stream == stream, or rows == 0: agb_peer_rmsnorm_bwd. */
int agb_peer_rmsnorm_bwd_overlapped(agb_peer_t* p, const void* x, const void* gamma, const float* rstd, const void* gy,
                                    const void* dx_add, void* dx, void* workspace, size_t workspace_bytes, int64_t rows,
                                    int64_t hidden, int dtype, agb_stream_t stream, agb_stream_t side_stream);
/* agb_peer_exchange is these two, with an event between them when the streams differ. */
int agb_peer_publish(agb_peer_t* p, agb_stream_t stream);
int agb_peer_sum(agb_peer_t* p, float* dgamma, int64_t hidden, int accumulate, agb_stream_t stream);
/* Ranks that are threads of ONE process (CUDA IPC cannot map a block into the process that made it):
 * every rank reads its block's address with agb_peer_block and all of them connect with the array of
 * addresses instead of handles.  Ranks on the same GPU must publish before any of them sums, so that
 * no kernel waits for a later launch on its own GPU. */
int agb_peer_block(agb_peer_t* p, void** base);
int agb_peer_connect_local(agb_peer_t* p, void* const* bases /* world addresses, rank order */);
/* Tear-down in two collective phases: every rank unmaps the others' blocks (agb_peer_disconnect, which
 * synchronises the device first), a barrier, then every rank frees its own (agb_peer_destroy) -- a block
 * must not be freed while another process still has it mapped. */
int agb_peer_disconnect(agb_peer_t* p);
int agb_peer_destroy(agb_peer_t* p);

#ifdef __cplusplus
}
#endif
#endif /* AGB_AGB_SHARD_H */
