/*
 * agb.h -- C ABI of libagb_cuda.so: the RMSNorm forward / VJP / JVP path of cgadimpl,
 * hand-written for NVIDIA B200 (sm_100a).
 *
 * Style follows cgadimpl's own raw-pointer kernel plugin (`ag::kernels::cuda()` loaded with
 * `load_cuda_plugin("./libagkernels_cuda.so")`, cgadimpl/Tests/test_kernels_gpu.cpp:39-148):
 * plain device pointers, element counts and a stream; the caller owns every buffer.
 * Each entry point below names the reference code it replaces (paths inside the cgadimpl
 * project).
 *
 * Conventions
 *   - All tensors are row-major and contiguous: [rows, hidden]; `rows` is the product of all
 *     leading dimensions, `hidden` the last one.  rows == 0 is a no-op.
 *   - `dtype` is the storage type of x / y / gy / dx / gamma (AGB_F32 or AGB_BF16).  Statistics
 *     (rstd) and dgamma are always fp32.  AGB_F32: all arithmetic is fp32 with fp64 reductions, rounded
 *     exactly where the reference materialises a tensor.  AGB_BF16 (RMSNorm forward and VJP): values are
 *     widened once, sums are carried in fp32 with fused multiply-adds, outputs are rounded once; the
 *     "bf16_strict" option selects the fp32 arithmetic above for 16-bit I/O as well.
 *   - `stream` is a cudaStream_t (NULL = the legacy default stream).  Calls only enqueue work;
 *     they never synchronise, allocate or free.
 *   - Return value: AGB_OK or an agb_status_t; agb_last_error() gives a message for the
 *     calling thread.  Nothing here calls exit() (the reference's CUDA_CHECK does,
 *     cgadimpl/src/runtime/cuda_graphs.cpp:12-19).
 *   - Re-entrant: every entry point may be called from many threads at once (cgadimpl's parallel
 *     backward calls VJP rules from many threads, cgadimpl/src/core/autodiff.cpp:155-159).  The
 *     process-wide state is: the launch counter and the tuning options of agb_set_option (atomics), the
 *     per-device properties cache and the per-device address of the built-in scratch array (each under
 *     a mutex), the device status word that bounded waits raise (one per device, in device memory), and
 *     the built-in scratch array itself, which calls of agb_rmsnorm_bwd_static share.
 *   - There is no CPU fallback: without a CUDA device every compute entry point returns
 *     AGB_ERR_CUDA.
 */
#ifndef AGB_AGB_H
#define AGB_AGB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    AGB_OK = 0,
    AGB_ERR_INVALID_ARG = 1,   /* null pointer, negative size, bad enum */
    AGB_ERR_UNSUPPORTED = 2,   /* dtype / shape outside what the kernels handle */
    AGB_ERR_MISALIGNED = 3,    /* a pointer is not aligned to its element size */
    AGB_ERR_CUDA = 4,          /* a CUDA runtime call failed (message has the CUDA error) */
    AGB_ERR_WORKSPACE = 5,     /* workspace too small or missing */
    AGB_ERR_TIMEOUT = 6        /* a bounded device-side wait gave up (see agb_device_status) */
} agb_status_t;

typedef enum { AGB_F32 = 0, AGB_BF16 = 1, AGB_F64 = 2 } agb_dtype_t;
typedef enum { AGB_REDUCE_SUM = 0, AGB_REDUCE_MEAN = 1, AGB_REDUCE_MAX = 2 } agb_reduce_op_t;

typedef void* agb_stream_t; /* cudaStream_t */

/* ---- library ---- */
int         agb_version(void);                 /* major*10000 + minor*100 + patch */
const char* agb_status_string(int status);
const char* agb_last_error(void);              /* thread-local, never NULL */

/* Number of kernels this library has launched since load (all threads, all devices). */
uint64_t agb_launch_count(void);

/* Reads (and clears) the device-side status word of the current device: 0, or AGB_ERR_TIMEOUT
 * if a kernel's bounded wait on a shared-memory barrier ran out (the kernel then skipped the
 * rest of its work and returned; its outputs are undefined).  Synchronises the device. */
int agb_device_status(void);

/* Exercises the failure path without any fault: launches one warp that waits, for at most
 * `poll_limit` polls (each up to 10 us), on a shared-memory barrier nobody completes, then raises the
 * device status word exactly as a kernel whose bulk copy never arrived would.  The next
 * agb_device_status() returns AGB_ERR_TIMEOUT and the context stays usable.  polls_done (device
 * pointer, nullable) receives the number of polls made. */
int agb_selftest_bounded_wait(int poll_limit, int* polls_done, agb_stream_t stream);

/* Process-wide options; value 0 restores the built-in behaviour unless stated.  Unknown key:
 * AGB_ERR_INVALID_ARG.
 *   launch-plan knobs for sweeps: "stages", "ctas_per_sm", "threads", "ept" (elements per thread of the
 *     strict backward), "rows_per_warp" (strict backward, one-warp rows), "bwd_keep" (16-bit backward:
 *     1 keep x/gy in registers, 2 re-read the tile, 3 64 elements per thread re-reading the tile, 4 64 elements
 *     per thread with x/gy kept where 256 resident threads allow it), "lone_ring" (2: a single
 *     CTA per SM may run a two-slot ring), "reserve_sms" (SMs the persistent grids leave free),
 *     "bwd_refill" (16-bit backward: 1 thread 0 refills a ring slot after the mid-tile barrier, 2 the
 *     last warp out of the slot does wherever that form is built), "softmax_two_pass" (approximate softmax / logsumexp forward:
 *     1 maximum first, then exp; 2 always the one-pass kernel), "free_rows" (1: the 16-bit forward keeps a
 *     block-wide barrier per tile also for rows that one warp owns), "force_generic" (1: the unstaged kernels);
 *   "bf16_strict"  1: 16-bit I/O through the strictly rounded, fp64-reducing kernels (the fp32 path's
 *                  arithmetic) instead of the fp32-accumulating ones;
 *   "softmax_strict"  1: softmax / logsumexp forward with the reference composition's rounding points
 *                  (exp to 2^-33, fp64 sums, exact division; reproduces the CPU composition's bits) instead
 *                  of the default approximate exp (2e-7 relative; the terms of a logsumexp sum 2.4e-7 +
 *                  1.2e-7 per unit below the row maximum) with fp32 sums;
 *   "pdl"          programmatic dependent launch between the library's kernels: 1 (default) a kernel's CTAs
 *                  are placed while the previous one drains, 2 as soon as it has started, 0 off;
 *   "peer_poll_limit"  polls (up to 2 us each) before a wait on another rank's counter gives up
 *                  (0 = default, about two seconds); process-wide, applies on every device. */
int agb_set_option(const char* key, int64_t value);

/* Describes the launch the heuristic would make: out[0]=grid, out[1]=block, out[2]=dynamic
 * shared bytes, out[3]=pipeline stages, out[4]=rows per tile, out[5]=1 if the generic
 * (unstaged) kernel is used.  `which`: 0 = forward, 1 = backward, 2 = jvp of the RMSNorm layer;
 * 3, 4, 5 = the same three of LayerNorm. */
int agb_describe_launch(int which, int64_t rows, int64_t hidden, int dtype, int fused_add, int64_t out[6]);

/* ---- RMSNorm forward ----
 * Replaces rms_nodeops (cgadimpl/src/ops/normalization.cpp:23-35: x*x, reduce_mean, +eps, sqrt,
 * 1/., x*rsqrt_var -- six tensor calls) followed, when gamma != NULL, by mul_nodeops with a
 * [hidden] right operand (cgadimpl/src/ops/arithmetic.cpp:31-39).
 *   y[r,j]  = (x[r,j] * rstd[r]) * gamma[j]        rstd[r] = 1 / sqrt(mean_j(x[r,j]^2) + eps)
 * gamma == NULL gives the reference's gamma-less `rms(x)`.  rstd [rows] fp32 is tape[0]. */
int agb_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd,
                    int64_t rows, int64_t hidden, float eps, int dtype, agb_stream_t stream);

/* ---- residual add + RMSNorm forward, fused ----
 * Replaces add_nodeops (cgadimpl/src/ops/arithmetic.cpp:11-19) followed by the two calls above.
 *   h = x + r;  y = rmsnorm(h) * gamma.   Writes h (the saved input of the norm), y and rstd. */
int agb_add_rmsnorm_fwd(const void* x, const void* r, const void* gamma, void* h, void* y, float* rstd,
                        int64_t rows, int64_t hidden, float eps, int dtype, agb_stream_t stream);

/* ---- RMSNorm VJP ----
 * Replaces vjp_Mul for the gamma product (cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:54-59, with
 * the column reduction of reduce_for_broadcast :15-35) and vjp_RMSNorm (:368-377):
 *   dy   = gy * gamma                                  (gy itself when gamma == NULL)
 *   dot  = sum_j dy[r,j] * x[r,j]
 *   dx   = rstd * (dy - x * (rstd*rstd) * dot / hidden)   [+ dx_add]
 *   dgamma[j] = sum_r gy[r,j] * (x[r,j] * rstd[r])
 * dx_add (nullable) is added to dx: it fuses Node::accumulate_grad's `grad +=`
 * (cgadimpl/src/core/graph.cpp:44-47) and the second parent of vjp_Add (:40-45).  dx_add may
 * alias gy or dx (in-place accumulation).
 * dgamma is produced in two deterministic stages: per-CTA fp64 partials in `workspace`, then a
 * fixed-order column reduction.  The workspace must hold at least 2 * SMs rows of `hidden` doubles;
 * agb_rmsnorm_bwd_workspace_bytes returns the 4 * SMs rows the largest launch uses, and a smaller
 * workspace only means fewer CTAs (one partial row each).  For a given workspace size the result is
 * bit-reproducible.  `dgamma_dtype`:
 * AGB_F32 writes the final fp32 [hidden]; AGB_F64 writes the un-rounded fp64 [hidden] sum, for
 * a cross-device all-reduce or for accumulation over row chunks, to be finished with
 * agb_dgamma_finalize.  With accumulate_dgamma the result is added to the old contents.
 * dgamma == NULL skips it (then workspace may be NULL). */
size_t agb_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t hidden, int dtype);
int agb_rmsnorm_bwd(const void* x, const void* gamma, const float* rstd, const void* gy,
                    const void* dx_add, void* dx, void* dgamma, int dgamma_dtype, int accumulate_dgamma,
                    void* workspace, size_t workspace_bytes,
                    int64_t rows, int64_t hidden, int dtype, agb_stream_t stream);

/* The two stages of agb_rmsnorm_bwd as separate calls, for callers that overlap the column reduction of one
 * layer with the backward of the next (two workspaces used in turn, the reduction on a second stream
 * behind an event): the VJP kernel alone, which leaves one fp64 [hidden] partial row per CTA in `workspace`
 * and reports how many in *n_partials (gamma is required), and the fixed-order reduction of those rows
 * (the second half of reduce_for_broadcast, cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:15-35).  Calling
 * them back to back on one stream gives the bits of agb_rmsnorm_bwd. */
int agb_rmsnorm_bwd_partials(const void* x, const void* gamma, const float* rstd, const void* gy,
                             const void* dx_add, void* dx, void* workspace, size_t workspace_bytes,
                             int64_t rows, int64_t hidden, int dtype, agb_stream_t stream, int* n_partials);
int agb_dgamma_reduce(const void* partials, int n_partials, int64_t hidden, void* dgamma, int dgamma_dtype,
                      int accumulate, agb_stream_t stream);

/* ---- RMSNorm VJP without a caller workspace ----
 * No counterpart in the reference.  Same computation and same results as agb_rmsnorm_bwd with an
 * fp32 dgamma, for callers that cannot hand over scratch memory because they cannot allocate any:
 * a host that was given one fixed device arena at start-up and may not grow it (a real-time loop,
 * an inference service running under a memory budget), or a plugin that receives raw tensor
 * pointers but no allocator handle -- for them cudaMalloc in the hot path is off limits (it
 * synchronises the device, can fail late and fragments the budget).
 * The per-CTA dgamma partial rows go into an array of AGB_STATIC_SCRATCH_BYTES built into the
 * library (every GPU that loads the library holds it until the process exits).  Consequences:
 *   - limit: partial_rows * hidden * 8 <= AGB_STATIC_SCRATCH_BYTES, partial_rows = 2 * SM count;
 *     on a 148-SM B200 that is hidden <= 8856.  Larger sizes are refused with AGB_ERR_WORKSPACE
 *     and nothing is launched.
 *   - the first call on each device looks up the array's device address (one CUDA runtime query,
 *     no allocation); make that first call outside any stream capture.
 *   - all calls share the one array.  It keeps the previous call's partials, which is harmless:
 *     every partial row that is read has been fully rewritten by the same call, so nothing needs
 *     clearing.  Two calls that overlap on the GPU (different streams, no dependency) race on it
 *     and corrupt each other's dgamma; order them on one stream or with an event.
 * The entry point itself calls no cudaMalloc, cudaFree or any allocating routine. */
#define AGB_STATIC_SCRATCH_BYTES (20u << 20)
int agb_rmsnorm_bwd_static(const void* x, const void* gamma, const float* rstd, const void* gy,
                           const void* dx_add, void* dx, float* dgamma, int accumulate_dgamma,
                           int64_t rows, int64_t hidden, int dtype, agb_stream_t stream);

/* Rounds an fp64 [hidden] column sum to fp32 (dgamma = (float)sum, or += when accumulate). */
int agb_dgamma_finalize(const double* sum, float* dgamma, int64_t hidden, int accumulate, agb_stream_t stream);

/* ---- RMSNorm JVP ----
 * Replaces jvp_RMSNorm (cgadimpl/src/autodiff/autodiff_jvp_ops.cpp:366-379) and jvp_Mul (:24-31).
 * The reference divides by tape[0] as if it held rms, but the forward stores rstd there, so its
 * result is off by 1/rstd^2 per row; this entry point computes the mathematically correct
 *   tyhat = tx*rstd - (yhat*dot)*(rstd/hidden),  dot = sum_j tx*yhat,  yhat = x*rstd
 *   ty    = tyhat*gamma + yhat*tgamma            (tgamma may be NULL; gamma NULL -> ty = tyhat) */
int agb_rmsnorm_jvp(const void* x, const void* gamma, const float* rstd, const void* tx, const void* tgamma,
                    void* ty, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream);

/* ---- residual add and its VJP ----
 * add_nodeops (arithmetic.cpp:11-19): out = a + b over n elements.
 * vjp_Add (autodiff_vjp_ops.cpp:40-45) with accumulate_grad: ga += gy; gb += gy (either may be
 * NULL).  Same shape as the legacy plugin's vjp_add(ga, gb, gy, n, stream)
 * (cgadimpl/Tests/test_kernels_gpu.cpp:90). */
int agb_residual_add(const void* a, const void* b, void* out, int64_t n, int dtype, agb_stream_t stream);
int agb_vjp_add(void* ga, void* gb, const void* gy, int64_t n, int dtype, agb_stream_t stream);

/* ---- broadcast scale and its VJP (the unfused gamma product) ----
 * mul_nodeops with a [hidden] operand: out[r,j] = a[r,j] * g[j].
 * vjp_Mul: da += gy*g (da nullable); dg += sum_r gy*a (dg fp32 [hidden], nullable, needs the
 * same workspace as agb_rmsnorm_bwd). */
int agb_scale_lastdim(const void* a, const void* g, void* out, int64_t rows, int64_t hidden, int dtype,
                      agb_stream_t stream);

/* ---- general broadcast forms of add / mul and of their VJPs ----
 * What add_nodeops / mul_nodeops (arithmetic.cpp:11-39), Node::accumulate_grad (graph.cpp:44-47) and
 * reduce_for_broadcast (autodiff_vjp_ops.cpp:15-35) do for the operand shapes that occur on this
 * path.  `b_mode` says how the second operand broadcasts against [rows, hidden]:
 *   AGB_BCAST_FULL [rows,hidden], AGB_BCAST_LASTVEC [hidden] or [1,hidden],
 *   AGB_BCAST_ROWSTAT [rows,1], AGB_BCAST_SCALAR [1].
 * agb_binary_broadcast: out = a (+|*) broadcast(b); op 0 = add, 1 = mul.
 * agb_accumulate_broadcast: dst += broadcast(src) * scale (scale == 1 adds src unchanged; otherwise
 *   the product is rounded first, like the separate `gy * scale` tensor of vjp_MeanAll :405-408).
 * agb_mul_reduce: out (+)= sum of g*a (a NULL: of g) over the axes that `out_mode` broadcasts, i.e.
 *   the gradient of a broadcast operand: LASTVEC -> out[hidden] summed over rows, ROWSTAT ->
 *   out[rows] summed over hidden, SCALAR -> out[1].  fp64 accumulation in a fixed order; each
 *   product rounded to the tensor dtype first.  Workspace: agb_mul_reduce_workspace_bytes. */
typedef enum { AGB_BCAST_FULL = 0, AGB_BCAST_LASTVEC = 1, AGB_BCAST_ROWSTAT = 2, AGB_BCAST_SCALAR = 3 } agb_bcast_t;
int agb_binary_broadcast(int op, const void* a, const void* b, void* out, int64_t rows, int64_t hidden, int b_mode,
                         int dtype, agb_stream_t stream);
int agb_accumulate_broadcast(void* dst, const void* src, int64_t rows, int64_t hidden, int src_mode, float scale,
                             int dtype, agb_stream_t stream);
size_t agb_mul_reduce_workspace_bytes(int64_t rows, int64_t hidden);
int agb_mul_reduce(const void* g, const void* a, void* out, int64_t rows, int64_t hidden, int out_mode,
                   int accumulate, void* workspace, size_t workspace_bytes, int dtype, agb_stream_t stream);

/* ---- LayerNorm without affine parameters (cgadimpl's `laynor`) ----
 * Forward replaces laynor_nodeops (cgadimpl/src/ops/normalization.cpp:10-22):
 *   mean = mean_j x; xm = x - mean; var = mean_j xm^2; y = xm / sqrt(var + eps)
 * and saves var and mean ([rows] fp32: tape[0], tape[1]).  eps is 1e-5 in the reference.
 * Backward replaces vjp_LayerNorm (cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:351-365), with the
 * same dx_add convention as agb_rmsnorm_bwd.  (The reference's jvp_LayerNorm throws.) */
int agb_layernorm_fwd(const void* x, void* y, float* mean, float* var, int64_t rows, int64_t hidden, float eps,
                      int dtype, agb_stream_t stream);
int agb_layernorm_bwd(const void* x, const float* mean, const float* var, const void* gy, const void* dx_add,
                      void* dx, int64_t rows, int64_t hidden, float eps, int dtype, agb_stream_t stream);
/* The JVP the reference leaves unimplemented (jvp_LayerNorm throws, autodiff_jvp_ops.cpp:361-363).
 * y is the forward's output, t the tangent of x, var the saved variance:
 *   tmean = mean_j t;  d = mean_j y*(t - tmean);  ty = (1/sqrt(var+eps)) * ((t - tmean) - y*d). */
int agb_layernorm_jvp(const void* y, const void* t, const float* var, void* ty, int64_t rows, int64_t hidden, float eps,
                      int dtype, agb_stream_t stream);

/* ---- row softmax / logsumexp over the last axis and their rules ----
 * agb_softmax_row_fwd replaces softmax_row_nodeops (cgadimpl/src/ops/reduction.cpp:42-53):
 *   m = max_j z; e = exp(z - m); s = sum_j e; y = e / s.
 * agb_logsumexp_row_fwd replaces logsumexp_row_nodeops (reduction.cpp:54-66): out[rows] = log(s) + m.
 * agb_softmax_row_bwd is vjp_SoftmaxRow (autodiff_vjp_ops.cpp:421-428) with g = gy AND jvp_SoftmaxRow
 *   (autodiff_jvp_ops.cpp:411-420) with g = the tangent of z -- the same expression:
 *   dz = y * (g - sum_j y*g)  [+ dz_add; dz_add may alias dz: gradient accumulation in place].
 * agb_logsumexp_row_bwd replaces vjp_LogSumExpRow (autodiff_vjp_ops.cpp:430-440): softmax(z) is
 *   recomputed; dz = gy[rows] * softmax(z) [+ dz_add].
 * agb_logsumexp_row_jvp replaces jvp_LogSumExpRow (autodiff_jvp_ops.cpp:421-434):
 *   out[rows] = sum_j softmax(z) * tz.
 * Row statistics ([rows] arrays: out, gy) have the element type of z.  exp and log are evaluated in
 * fp64 and rounded to fp32 once; every other step rounds where the reference materialises a tensor,
 * and the sums are carried in fp64. */
int agb_softmax_row_fwd(const void* z, void* y, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream);
int agb_logsumexp_row_fwd(const void* z, void* out, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream);
int agb_softmax_row_bwd(const void* y, const void* g, const void* dz_add, void* dz, int64_t rows, int64_t hidden,
                        int dtype, agb_stream_t stream);
int agb_logsumexp_row_bwd(const void* z, const void* gy, const void* dz_add, void* dz, int64_t rows, int64_t hidden,
                          int dtype, agb_stream_t stream);
int agb_logsumexp_row_jvp(const void* z, const void* tz, void* out, int64_t rows, int64_t hidden, int dtype,
                          agb_stream_t stream);

/* ---- optimiser steps on the layer's parameters ----
 * agb_sgd_step: ag::SGD's update of one leaf, `value += -learning_rate * grad`
 *   (cgadimpl/src/optimizer/optim.cpp:12-19).
 * agb_adam_step: one Adam::step() for one parameter (optim.cpp:33-72), fp32: the caller passes
 *   alpha_eff = alpha*sqrt(1-beta2^t)/(1-beta1^t) and eps_eff = epsilon*sqrt(1-beta2^t) as the
 *   reference computes them on the host.  m and v are updated in place. */
int agb_sgd_step(void* param, const void* grad, int64_t n, float learning_rate, int dtype, agb_stream_t stream);
int agb_adam_step(float* param, const float* grad, float* m, float* v, int64_t n, float beta1, float beta2,
                  float alpha_eff, float eps_eff, agb_stream_t stream);

/* ---- row and global reductions ----
 * rowsum / rowmax (cgadimpl/src/ops/reduction.cpp:25-40) and the reduce_sum / reduce_mean
 * (., {-1}, keepdim) primitive inside the norm: out[r] = op_j x[r,j], out has x's dtype.
 * sum / mean_all (reduction.cpp:9-24): out[0] = op over all n elements, fp64 accumulation in a
 * fixed order; workspace from agb_reduce_all_workspace_bytes. */
int agb_row_reduce(int op, const void* x, void* out, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream);
size_t agb_reduce_all_workspace_bytes(int64_t n);
int agb_reduce_all(int op, const void* x, void* out, int64_t n, int dtype,
                   void* workspace, size_t workspace_bytes, agb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AGB_AGB_H */
