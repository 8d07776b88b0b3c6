/*
 * agb_oracle.h -- CPU restatement of cgadimpl's RMSNorm path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is the checker the CUDA kernels are compared against and the CPU arm of the
 * benchmark.  Nothing in the shipped library links, loads or calls it.
 *
 * What pins it.  The reference cannot be built by its own build system (its tensor library
 * OwnTensor -- git submodule `tensor`, url kathir-23s/Tensor-Implementations, pinned commit
 * unknown -- is an empty directory in the reference checkout, and MLIR / Nova are required too)
 * and it ships no golden vectors.  But its op builders, autodiff engine and rules for this path
 * compile unmodified over a small stand-in for that library (oracle/ref_shim, oracle/build_ref.py
 * -> oracle/_ref/libcgadimpl_ref.so), and tests/test_reference_build.py checks that this file
 * reproduces THAT bit for bit (forward, VJP, the residual stack through the reference's graph
 * engine, the literal JVP rule, the reductions) in both reduction modes.  So the reference's
 * COMPOSITION is pinned: which tensor calls are made, in which order, where an fp32 temporary is
 * materialised.  PARITY REMAINS UNPINNED at one place only: the arithmetic inside the real
 * OwnTensor (summation order, accumulator width), which no file in the reference shows.
 * The reference's own numeric test of this path, a central finite-difference check on a random
 * [4,10] input at max-abs 1e-3 (cgadimpl/Tests/test_core_ops_gpu.cpp:15-84, 262-267), is re-run
 * against this oracle as well.
 *
 * Reduction modes.  OwnTensor's summation order and accumulator width are unknown, so every
 * reduction exists twice:
 *   AGB_RED_F32  fp32 accumulator, left to right  (one plausible reference result)
 *   AGB_RED_F64  fp64 accumulator, left to right, rounded once to fp32 (the arbiter: any
 *                fp32 summation order agrees with it to within its own rounding noise)
 * All elementwise steps round to fp32 exactly where the reference materialises a Tensor.
 * Build with -ffp-contract=off so the compiler cannot fuse a multiply into an add.
 *
 * bf16 I/O: inputs are widened to fp32 once, all maths as above, outputs rounded to bf16
 * once (round-to-nearest-even); rstd and dgamma stay fp32.
 */
#ifndef AGB_ORACLE_H
#define AGB_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { AGB_RED_F32 = 0, AGB_RED_F64 = 1 };

/* ---- OwnTensor stand-ins (each = one reference tensor call = one pass over memory) ---- */
void ot_mul(const float* a, const float* b, float* out, int64_t n);            /* a * b, same shape      */
void ot_add(const float* a, const float* b, float* out, int64_t n);            /* a + b                  */
void ot_sub(const float* a, const float* b, float* out, int64_t n);            /* a - b                  */
void ot_mul_rowstat(const float* a, const float* s, float* out, int64_t R, int64_t H); /* [R,H]*[R,1]   */
void ot_mul_lastvec(const float* a, const float* g, float* out, int64_t R, int64_t H); /* [R,H]*[H]     */
void ot_div_scalar(const float* a, float d, float* out, int64_t n);            /* a / d                  */
void ot_mul_scalar(const float* a, float d, float* out, int64_t n);            /* a * d                  */
void ot_add_scalar(const float* a, float d, float* out, int64_t n);            /* a + d                  */
void ot_sqrt(const float* a, float* out, int64_t n);
void ot_rdiv_scalar(float d, const float* a, float* out, int64_t n);           /* d / a                  */
void ot_reduce_sum_last(const float* a, float* out, int64_t R, int64_t H, int red);   /* sum over -1, keepdim  */
void ot_reduce_mean_last(const float* a, float* out, int64_t R, int64_t H, int red);  /* mean over -1, keepdim */
void ot_reduce_max_last(const float* a, float* out, int64_t R, int64_t H);
void ot_reduce_sum_lead(const float* a, float* out, int64_t R, int64_t H, int red);   /* sum over leading axes */
float ot_reduce_sum_all(const float* a, int64_t n, int red);
float ot_reduce_mean_all(const float* a, int64_t n, int red);

/* ---- reference compositions ---- */

/* rms_nodeops, cgadimpl/src/ops/normalization.cpp:23-35 (eps is 1e-5f there; a parameter here).
 * Writes rstd[R] (tape[0]) and yhat[R,H] (node value == tape[1]). */
void agb_oracle_rms_forward(const float* x, float* yhat, float* rstd,
                            int64_t R, int64_t H, float eps, int red);

/* mul_nodeops with a [H] (or [1,H]) right operand, cgadimpl/src/ops/arithmetic.cpp:31-39 */
void agb_oracle_scale_forward(const float* yhat, const float* gamma, float* y, int64_t R, int64_t H);

/* vjp_Mul for y = yhat * gamma: cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:54-59 with
 * reduce_for_broadcast :15-35.  dyhat[R,H] = gy*gamma; dgamma[H] = sum_rows(gy*yhat). */
void agb_oracle_vjp_scale(const float* gy, const float* yhat, const float* gamma,
                          float* dyhat, float* dgamma, int64_t R, int64_t H, int red);

/* vjp_RMSNorm, cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:368-377:
 * dot = sum(gy*x,-1); dx = rstd * (gy - x*(rstd*rstd)*dot/D). */
void agb_oracle_vjp_rms(const float* x, const float* rstd, const float* gy, float* dx,
                        int64_t R, int64_t H, int red);

/* add_nodeops / vjp_Add, cgadimpl/src/ops/arithmetic.cpp:11-19, autodiff_vjp_ops.cpp:40-45 */
void agb_oracle_add_forward(const float* a, const float* b, float* out, int64_t n);

/* Whole layer y = mul(rms(x), gamma) forward + VJP, fp32.  gamma may be NULL (plain rms).
 * Outputs: y[R,H], rstd[R], dx[R,H], dgamma[H] (untouched if gamma NULL).
 * Allocates the same [R,H] temporaries the reference does. */
void agb_oracle_rmsnorm_fwd_bwd(const float* x, const float* gamma, const float* gy,
                                float* y, float* rstd, float* dx, float* dgamma,
                                int64_t R, int64_t H, float eps, int red);
void agb_oracle_rmsnorm_fwd(const float* x, const float* gamma, float* y, float* rstd,
                            int64_t R, int64_t H, float eps, int red);

/* A single-pass, row-fused CPU variant of the same arithmetic (identical results, one read of
 * each input per pass).  Timed separately so the GPU/CPU ratio is not flattered by the
 * reference's extra memory passes. */
void agb_oracle_rmsnorm_fwd_bwd_fused(const float* x, const float* gamma, const float* gy,
                                      float* y, float* rstd, float* dx, float* dgamma,
                                      int64_t R, int64_t H, float eps);

/* bf16 I/O wrappers (uint16_t = raw bf16 bits). */
void agb_oracle_rmsnorm_fwd_bwd_bf16(const uint16_t* x, const uint16_t* gamma, const uint16_t* gy,
                                     uint16_t* y, float* rstd, uint16_t* dx, float* dgamma,
                                     int64_t R, int64_t H, float eps, int red);

/* jvp_RMSNorm.  `literal` follows cgadimpl/src/autodiff/autodiff_jvp_ops.cpp:366-379 to the
 * letter (it divides by tape[0], which holds rstd, so it is off by 1/rstd^2).  `corrected`
 * multiplies by rstd instead: ty = t*rstd - yhat*dot*(rstd/N), dot = sum(t*yhat,-1). */
void agb_oracle_jvp_rms_literal(const float* t, const float* yhat, const float* rstd, float* ty,
                                int64_t R, int64_t H, int red);
void agb_oracle_jvp_rms_corrected(const float* t, const float* yhat, const float* rstd, float* ty,
                                  int64_t R, int64_t H, int red);
/* jvp_Mul, autodiff_jvp_ops.cpp:24-31: t_out = tyhat*gamma + yhat*tgamma (tgamma may be NULL) */
void agb_oracle_jvp_scale(const float* tyhat, const float* yhat, const float* gamma,
                          const float* tgamma, float* tout, int64_t R, int64_t H);

/* Row / global reductions: cgadimpl/src/ops/reduction.cpp:9-40 */
void agb_oracle_rowsum(const float* x, float* out, int64_t R, int64_t H, int red);
void agb_oracle_rowmax(const float* x, float* out, int64_t R, int64_t H);
float agb_oracle_sum(const float* x, int64_t n, int red);
float agb_oracle_mean_all(const float* x, int64_t n, int red);

/* Residual stack (pre-norm residual stream), L layers:
 *   x_0=x, r_0=r; h_l=x_l+r_l; y_l=mul(rms(h_l),gamma_l); x_{l+1}=h_l; r_{l+1}=y_l
 *   backward from g on y_{L-1}; dh_l = vjp(h_l) accumulated exactly as accumulate_grad does.
 * gammas is [L,H]; outputs y_last[R,H], dh0[R,H] (= dx_0 = dr_0), dgammas[L,H].
 * Composition of add_nodeops + rms_nodeops + mul_nodeops and their VJPs as cited above. */
void agb_oracle_residual_stack(const float* x, const float* r, const float* gammas, const float* g,
                               float* y_last, float* dh0, float* dgammas,
                               int64_t R, int64_t H, int L, float eps, int red);

/* LayerNorm without affine parameters: laynor_nodeops cgadimpl/src/ops/normalization.cpp:10-22 and
 * vjp_LayerNorm cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:351-365 (its JVP throws in the reference). */
void agb_oracle_layernorm_forward(const float* x, float* y, float* mean, float* var,
                                  int64_t R, int64_t H, float eps, int red);
void agb_oracle_layernorm_vjp(const float* x, const float* mean, const float* var, const float* gy, float* dx,
                              int64_t R, int64_t H, float eps, int red);

/* JVP of laynor: a definition of this library (the reference's rule throws); y, var from the forward. */
void agb_oracle_layernorm_jvp(const float* y, const float* t, const float* var, float* ty, int64_t R, int64_t H, float eps);

/* Row softmax / logsumexp over the last axis: cgadimpl/src/ops/reduction.cpp:42-66, rules
 * autodiff_vjp_ops.cpp:421-440 and autodiff_jvp_ops.cpp:411-434.  exp / log are the C library's expf /
 * logf, as in the stand-in tensor library the reference is compiled over.  softmax_row_vjp is also
 * the JVP (same expression with the tangent in place of gy).  gy / out of the logsumexp rules are [R]. */
void ot_exp(const float* a, float* out, int64_t n);
void ot_log(const float* a, float* out, int64_t n);
void ot_sub_rowstat(const float* a, const float* s, float* out, int64_t R, int64_t H);
void ot_div_rowstat(const float* a, const float* s, float* out, int64_t R, int64_t H);
void agb_oracle_softmax_row_forward(const float* z, float* y, int64_t R, int64_t H, int red);
void agb_oracle_logsumexp_row_forward(const float* z, float* out, int64_t R, int64_t H, int red);
void agb_oracle_softmax_row_vjp(const float* y, const float* g, float* out, int64_t R, int64_t H, int red);
void agb_oracle_logsumexp_row_vjp(const float* z, const float* gy, float* dz, int64_t R, int64_t H, int red);
void agb_oracle_logsumexp_row_jvp(const float* z, const float* tz, float* out, int64_t R, int64_t H, int red);

/* Optimiser steps on a parameter: cgadimpl/src/optimizer/optim.cpp:12-19 (SGD), :33-72 (Adam). */
void agb_oracle_sgd_step(float* param, const float* grad, int64_t n, float lr);
void agb_oracle_adam_step(float* param, const float* grad, float* m, float* v, int64_t n, float alpha, float beta1,
                          float beta2, float epsilon, int t);
void agb_oracle_adam_scalars(float alpha, float beta1, float beta2, float epsilon, int t, float* alpha_eff, float* eps_eff);

/* helpers */
float    agb_bf16_to_f32(uint16_t b);
uint16_t agb_f32_to_bf16(float f);
int      agb_oracle_num_threads(void);
void     agb_oracle_set_num_threads(int n);   /* launchers such as torchrun export OMP_NUM_THREADS=1 */

#ifdef __cplusplus
}
#endif
#endif
