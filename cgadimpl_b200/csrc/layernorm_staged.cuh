// layernorm_staged.cuh -- LayerNorm without affine parameters (cgadimpl's `laynor`) on the same
// skeleton as the RMSNorm kernels: persistent CTAs, bulk-copy ring, 16-byte vectors, fp64
// reductions, packed fp32 arithmetic, every rounding point of the reference's composition kept.
//   forward  (cgadimpl/src/ops/normalization.cpp:10-22):
//     mean = mean(x); xm = x - mean; var = mean(xm*xm); y = xm / sqrt(var + eps)
//   backward (cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:351-365):
//     std_inv = 1/sqrt(var+eps); d_var = sum(gy*xm*-0.5*std_inv^3);
//     d_mean = sum(gy*-std_inv) + d_var*sum(xm*-2)/D;
//     dx = gy*std_inv + d_var*xm*(2/D) + d_mean/D
// `y = xm / s` is a true division in the reference; here it is the exact three-instruction
// division by the per-row constant s (quotient estimate, FMA residual, one correction; checked
// against IEEE division on 1.5e9 random operand pairs).
// FAST (16-bit I/O unless "bf16_strict"): sums carried in fp32 with fused multiply-adds, y = xm * (1/s), and the
// backward's three row sums reduced to A = sum(gy*xm), B = sum(gy), C = sum(xm) -- the same algebra, a third
// of the instructions, outputs rounded to the 16-bit type once (rel 2e-2).
#pragma once
#include "rmsnorm_fast.cuh"

namespace agb {

struct LnFwdArgs {
    PipeGeom g;
    const void* x;
    void* y;
    float* mean;
    float* var;
    float eps;
};

template <typename T, int VPT, bool FULL, bool FAST = false>
__global__ void __launch_bounds__(1024, 1) layernorm_fwd_staged(const __grid_constant__ LnFwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);  // [2 phases][2 sums][nwarps]
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();

    const unsigned char* const src1[1] = {reinterpret_cast<const unsigned char*>(a.x)};
    const long long first = blockIdx.x, stride = gridDim.x;
    const long long my_tiles = g.ntiles > first ? (g.ntiles - first + stride - 1) / stride : 0;
    long long issued = 0;
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued)
            issue_tile<1>(g, ring, s_full, src1, first + issued * stride, static_cast<int>(issued));

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
        const uint4* sx = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(slot) * g.stage_stride +
                                                         static_cast<size_t>(grp) * g.row_bytes);
        double* red_sum = s_red + (k & 1) * 2 * nwarps;
        double* red_sq = red_sum + nwarps;

        // pass 1: sum of x; the vectors stay in registers
        uint4 keep[VPT];
        double s0 = 0.0, s1 = 0.0;
        float2 fs0 = make_float2(0.f, 0.f), fs1 = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    keep[i] = sx[v];
                    float2 xv[NP];
                    Pairs<T>::unpack(keep[i], xv);
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        if constexpr (FAST) {
                            if (e & 1) fs1 = add2(fs1, xv[e]);
                            else fs0 = add2(fs0, xv[e]);
                        } else {
                            s0 += static_cast<double>(xv[e].x);
                            s1 += static_cast<double>(xv[e].y);
                        }
                    }
                }
            }
        }
        const double wsum = FAST ? static_cast<double>(warp_sum_f32((fs0.x + fs0.y) + (fs1.x + fs1.y))) : warp_sum(s0 + s1);
        if (lane == 0) red_sum[warp] = wsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && issued < my_tiles) {  // every thread holds its vectors in registers
            issue_tile<1>(g, ring, s_full, src1, first + issued * stride, slot);
            ++issued;
        }
        const float mean = static_cast<float>(group_total(red_sum + grp * wpr, wpr, lane) / static_cast<double>(g.hidden));
        const float2 mean2 = splat(mean);

        // pass 2: variance of the centred values
        double q0 = 0.0, q1 = 0.0;
        float2 fq0 = make_float2(0.f, 0.f), fq1 = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP];
                    Pairs<T>::unpack(keep[i], xv);
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 xm = sub2(xv[e], mean2);
                        if constexpr (FAST) {
                            if (e & 1) fq1 = fma2(xm, xm, fq1);
                            else fq0 = fma2(xm, xm, fq0);
                        } else {
                            const float2 q = mul2(xm, xm);
                            q0 += static_cast<double>(q.x);
                            q1 += static_cast<double>(q.y);
                        }
                    }
                }
            }
        }
        const double wsq = FAST ? static_cast<double>(warp_sum_f32((fq0.x + fq0.y) + (fq1.x + fq1.y))) : warp_sum(q0 + q1);
        if (lane == 0) red_sq[warp] = wsq;
        __syncthreads();
        const float var = static_cast<float>(group_total(red_sq + grp * wpr, wpr, lane) / static_cast<double>(g.hidden));
        const float s = __fsqrt_rn(__fadd_rn(var, a.eps));
        const DivConst2 div_s{splat(s), splat(__fdiv_rn(1.0f, s))};

        // pass 3: y = xm / s
        if (valid) {
            if (tig == 0) {
                a.mean[row] = mean;
                a.var[row] = var;
            }
            uint4* gy = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.y) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP];
                    Pairs<T>::unpack(keep[i], xv);
#pragma unroll
                    for (int e = 0; e < NP; ++e) xv[e] = FAST ? mul2(sub2(xv[e], mean2), div_s.dinv) : div_s(sub2(xv[e], mean2));
                    store_vec_streaming(gy + v, Pairs<T>::pack(xv));
                }
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

struct LnBwdArgs {
    PipeGeom g;
    const void* x;
    const void* gy;
    const void* add;   // add_mode 1
    const float* mean;
    const float* var;
    void* dx;
    int add_mode;      // 0 none, 1 third staged array, 2 the addend is gy itself
    float eps, hidden_f, two_over_h;
};

template <typename T, int VPT, bool FULL, bool FAST = false>
__global__ void __launch_bounds__(1024, 1) layernorm_bwd_staged(const __grid_constant__ LnBwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);  // [2 phases][3 sums][nwarps]
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;
    const bool staged_add = a.add_mode == 1;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();

    const unsigned char* const src3[3] = {reinterpret_cast<const unsigned char*>(a.x),
                                          reinterpret_cast<const unsigned char*>(a.gy),
                                          reinterpret_cast<const unsigned char*>(a.add)};
    auto issue = [&](long long tile, int slot) {
        if (staged_add)
            issue_tile<3>(g, ring, s_full, src3, tile, slot);
        else
            issue_tile<2>(g, ring, s_full, reinterpret_cast<const unsigned char* const(&)[2]>(src3), tile, slot);
    };
    const long long first = blockIdx.x, stride = gridDim.x;
    const long long my_tiles = g.ntiles > first ? (g.ntiles - first + stride - 1) / stride : 0;
    long long issued = 0;
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued) issue(first + issued * stride, static_cast<int>(issued));

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        const float mean = valid ? a.mean[row] : 0.0f;
        const float var = valid ? a.var[row] : 1.0f;
        // per-row scalars, rounded as the reference's [R,1] tensors are
        const float std_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
        const float c3 = mul_rn(mul_rn(std_inv, std_inv), std_inv);
        const float2 mean2 = splat(mean), c32 = splat(c3), nsi2 = splat(-std_inv);
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;

        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sx = reinterpret_cast<const uint4*>(base);
        const uint4* sg = reinterpret_cast<const uint4*>(base + g.tile_stride);
        const uint4* sa = reinterpret_cast<const uint4*>(base + 2 * static_cast<size_t>(g.tile_stride));
        double* red = s_red + (k & 1) * 3 * nwarps;

        // pass 1: the three row sums
        double a0 = 0.0, a1 = 0.0, b0 = 0.0, b1 = 0.0, c0 = 0.0, c1 = 0.0;
        float2 fa = make_float2(0.f, 0.f), fb = make_float2(0.f, 0.f), fc = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP], gv[NP];
                    Pairs<T>::unpack(sx[v], xv);
                    Pairs<T>::unpack(sg[v], gv);
                    if constexpr (FAST) {
#pragma unroll
                        for (int e = 0; e < NP; ++e) {
                            const float2 xm = sub2(xv[e], mean2);
                            fa = fma2(gv[e], xm, fa);   // A = sum gy*xm
                            fb = add2(fb, gv[e]);       // B = sum gy
                            fc = add2(fc, xm);          // C = sum xm
                        }
                        continue;
                    }
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 xm = sub2(xv[e], mean2);
                        float2 t = mul2(gv[e], xm);            // gy * (x - mean)
                        t = mul2(t, splat(-0.5f));             // * -0.5f  (exact)
                        t = mul2(t, c32);                      // * std_inv^3
                        a0 += static_cast<double>(t.x);
                        a1 += static_cast<double>(t.y);
                        const float2 u = mul2(gv[e], nsi2);    // gy * (std_inv * -1)
                        b0 += static_cast<double>(u.x);
                        b1 += static_cast<double>(u.y);
                        const float2 w = mul2(xm, splat(-2.0f));  // (x - mean) * -2  (exact)
                        c0 += static_cast<double>(w.x);
                        c1 += static_cast<double>(w.y);
                    }
                }
            }
        }
        // FAST: d_var = -0.5 std_inv^3 A, sum1 = -std_inv B, sum2 = -2 C: the same three quantities the strict
        // form accumulates term by term
        const double ra = FAST ? static_cast<double>(-0.5f * c3 * warp_sum_f32(fa.x + fa.y)) : warp_sum(a0 + a1);
        const double rb = FAST ? static_cast<double>(-std_inv * warp_sum_f32(fb.x + fb.y)) : warp_sum(b0 + b1);
        const double rc = FAST ? static_cast<double>(-2.0f * warp_sum_f32(fc.x + fc.y)) : warp_sum(c0 + c1);
        if (lane == 0) {
            red[warp] = ra;
            red[nwarps + warp] = rb;
            red[2 * nwarps + warp] = rc;
        }
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue(first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        const float d_var = static_cast<float>(group_total(red + grp * wpr, wpr, lane));
        const float sum1 = static_cast<float>(group_total(red + nwarps + grp * wpr, wpr, lane));
        const float sum2 = static_cast<float>(group_total(red + 2 * nwarps + grp * wpr, wpr, lane));
        const float d_mean = add_rn(sum1, __fdiv_rn(mul_rn(d_var, sum2), a.hidden_f));
        const float2 md2 = splat(__fdiv_rn(d_mean, a.hidden_f)), dvar2 = splat(d_var), si2 = splat(std_inv),
                     k22 = splat(a.two_over_h);

        // pass 2: dx = gy*std_inv + d_var*xm*(2/D) + d_mean/D
        if (valid) {
            uint4* gdx = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.dx) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP], gv[NP], ov[NP];
                    Pairs<T>::unpack(sx[v], xv);
                    Pairs<T>::unpack(sg[v], gv);
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 xm = sub2(xv[e], mean2);
                        if constexpr (FAST) {
                            ov[e] = fma2(gv[e], si2, fma2(xm, splat(d_var * a.two_over_h), md2));
                        } else {
                            const float2 dxh = mul2(gv[e], si2);
                            float2 u = mul2(dvar2, xm);
                            u = mul2(u, k22);
                            ov[e] = add2_after_mul(add2_after_mul(dxh, u), md2);
                        }
                    }
                    if (a.add_mode == 2) {
#pragma unroll
                        for (int e = 0; e < NP; ++e) ov[e] = add2(ov[e], gv[e]);   // neither operand is a product
                    } else if (staged_add) {
                        float2 av[NP];
                        Pairs<T>::unpack(sa[v], av);
#pragma unroll
                        for (int e = 0; e < NP; ++e) ov[e] = add2(ov[e], av[e]);
                    }
                    store_vec_streaming(gdx + v, Pairs<T>::pack(ov));
                }
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

// ---------------------------------------------------------------- unstaged versions (any shape)
template <typename T>
__global__ void __launch_bounds__(kGenericThreads) layernorm_fwd_generic(const T* __restrict__ x, T* __restrict__ y,
                                                                         float* __restrict__ mean_out,
                                                                         float* __restrict__ var_out, long long rows,
                                                                         int hidden, float eps) {
    __shared__ double scratch[16];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * hidden;
        double s = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) s += static_cast<double>(Vec<T>::load1(xr + j));
        const float mean = static_cast<float>(block_sum_256(s, scratch, phase++) / static_cast<double>(hidden));
        double q = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float xm = sub_rn(Vec<T>::load1(xr + j), mean);
            q += static_cast<double>(mul_rn(xm, xm));
        }
        const float var = static_cast<float>(block_sum_256(q, scratch, phase++) / static_cast<double>(hidden));
        const float sd = __fsqrt_rn(__fadd_rn(var, eps));
        if (threadIdx.x == 0) {
            mean_out[row] = mean;
            var_out[row] = var;
        }
        T* yr = y + row * hidden;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads)
            Vec<T>::store1(yr + j, __fdiv_rn(sub_rn(Vec<T>::load1(xr + j), mean), sd));
    }
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads) layernorm_bwd_generic(const T* __restrict__ x,
                                                                         const float* __restrict__ mean_in,
                                                                         const float* __restrict__ var_in,
                                                                         const T* __restrict__ gy, const T* add, T* dx,
                                                                         long long rows, int hidden, float eps,
                                                                         float hidden_f, float two_over_h) {
    __shared__ double scratch[16];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * hidden;
        const T* gr = gy + row * hidden;
        const T* ar = add ? add + row * hidden : nullptr;
        T* dr = dx + row * hidden;
        const float mean = mean_in[row];
        const float std_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var_in[row], eps)));
        const float c3 = mul_rn(mul_rn(std_inv, std_inv), std_inv);
        const float nsi = -std_inv;
        double sa = 0.0, sb = 0.0, sc = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float xm = sub_rn(Vec<T>::load1(xr + j), mean);
            const float g = Vec<T>::load1(gr + j);
            sa += static_cast<double>(mul_rn(mul_rn(mul_rn(g, xm), -0.5f), c3));
            sb += static_cast<double>(mul_rn(g, nsi));
            sc += static_cast<double>(mul_rn(xm, -2.0f));
        }
        const float d_var = static_cast<float>(block_sum_256(sa, scratch, phase++));
        const float sum1 = static_cast<float>(block_sum_256(sb, scratch, phase++));
        const float sum2 = static_cast<float>(block_sum_256(sc, scratch, phase++));
        const float d_mean = add_rn(sum1, __fdiv_rn(mul_rn(d_var, sum2), hidden_f));
        const float md = __fdiv_rn(d_mean, hidden_f);
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float xm = sub_rn(Vec<T>::load1(xr + j), mean);
            const float g = Vec<T>::load1(gr + j);
            float o = add_rn(add_rn(mul_rn(g, std_inv), mul_rn(mul_rn(d_var, xm), two_over_h)), md);
            if (ar) o = add_rn(o, Vec<T>::load1(ar + j));
            Vec<T>::store1(dr + j, o);
        }
    }
}

// ------------------------------------------------------------------------------------------
// JVP of laynor (the reference's jvp_LayerNorm throws, cgadimpl/src/autodiff/autodiff_jvp_ops.cpp:361-363).
// With y = (x - mean) / sqrt(var + eps) saved by the forward and t the tangent of x:
//   tmean = sum(t) / H ;  d = (sum(y*t) - tmean * sum(y)) / H      (= mean(y * (t - tmean)); fp64, rounded once)
//   ty = std_inv * ((t - tmean) - y * d) ,  std_inv = 1 / sqrt(var + eps)
// Every elementwise step rounds to fp32 once, like the other rules of this library.
// ------------------------------------------------------------------------------------------
struct LnJvpArgs {
    PipeGeom g;
    const void* y;
    const void* t;
    const float* var;
    void* ty;
    float eps;
};

__device__ __forceinline__ void ln_jvp_stats(double st, double sy, double syt, int hidden, float* tmean, float* d) {
    const double tm = st / static_cast<double>(hidden);
    *tmean = static_cast<float>(tm);
    *d = static_cast<float>((syt - tm * sy) / static_cast<double>(hidden));
}

// FAST (16-bit I/O): the three row sums in fp32, ty = std_inv*t - std_inv*mean(t) - y*(std_inv*d) as two fused
// multiply-adds per pair.
template <typename T, bool FAST = false>
__global__ void __launch_bounds__(1024, 1) layernorm_jvp_staged(const __grid_constant__ LnJvpArgs a) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();

    const unsigned char* const src2[2] = {reinterpret_cast<const unsigned char*>(a.y),
                                          reinterpret_cast<const unsigned char*>(a.t)};
    const long long first = blockIdx.x, stride = gridDim.x;
    const long long my_tiles = g.ntiles > first ? (g.ntiles - first + stride - 1) / stride : 0;
    long long issued = 0;
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued)
            issue_tile<2>(g, ring, s_full, src2, first + issued * stride, static_cast<int>(issued));

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        const float var = valid ? a.var[row] : 1.0f;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sy = reinterpret_cast<const uint4*>(base);
        const uint4* st = reinterpret_cast<const uint4*>(base + g.tile_stride);

        double at = 0.0, ay = 0.0, ayt0 = 0.0, ayt1 = 0.0;
        float2 ft = make_float2(0.f, 0.f), fy = make_float2(0.f, 0.f), fyt = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float2 yv[NP], tv[NP];
                Pairs<T>::unpack(sy[v], yv);
                Pairs<T>::unpack(st[v], tv);
#pragma unroll
                for (int e = 0; e < NP; ++e) {
                    if constexpr (FAST) {
                        ft = add2(ft, tv[e]);
                        fy = add2(fy, yv[e]);
                        fyt = __ffma2_rn(yv[e], tv[e], fyt);
                    } else {
                        const float2 p = mul2(yv[e], tv[e]);
                        at += static_cast<double>(tv[e].x) + static_cast<double>(tv[e].y);
                        ay += static_cast<double>(yv[e].x) + static_cast<double>(yv[e].y);
                        ayt0 += static_cast<double>(p.x);
                        ayt1 += static_cast<double>(p.y);
                    }
                }
            }
        }
        if constexpr (FAST) {   // the per-lane fp32 sums join the shared fp64 reduction path
            at = static_cast<double>(ft.x + ft.y);
            ay = static_cast<double>(fy.x + fy.y);
            ayt0 = static_cast<double>(fyt.x + fyt.y);
        }
        double* red = s_red + (k & 1) * 3 * nwarps;
        const double wt = warp_sum(at), wy = warp_sum(ay), wyt = warp_sum(ayt0 + ayt1);
        if (lane == 0) {
            red[warp] = wt;
            red[nwarps + warp] = wy;
            red[2 * nwarps + warp] = wyt;
        }
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue_tile<2>(g, ring, s_full, src2, first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        float tmean, d;
        ln_jvp_stats(group_total(red + grp * wpr, wpr, lane), group_total(red + nwarps + grp * wpr, wpr, lane),
                     group_total(red + 2 * nwarps + grp * wpr, wpr, lane), g.hidden, &tmean, &d);
        const float std_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
        const float2 tm2 = splat(tmean), d2 = splat(d), si2 = splat(std_inv);
        const float2 c02 = splat(-std_inv * tmean), nsd2 = splat(-std_inv * d);   // FAST

        if (valid) {
            uint4* gout = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.ty) + row * g.row_bytes);
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float2 yv[NP], tv[NP];
                Pairs<T>::unpack(sy[v], yv);
                Pairs<T>::unpack(st[v], tv);
#pragma unroll
                for (int e = 0; e < NP; ++e) {
                    if constexpr (FAST) {
                        yv[e] = __ffma2_rn(yv[e], nsd2, __ffma2_rn(tv[e], si2, c02));
                    } else {
                        const float2 tc = sub2(tv[e], tm2);                  // neither operand is a product
                        yv[e] = mul2(si2, sub2_after_mul(tc, mul2(yv[e], d2)));
                    }
                }
                store_vec_streaming(gout + v, Pairs<T>::pack(yv));
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads) layernorm_jvp_generic(const T* __restrict__ y, const T* __restrict__ t,
                                                                         const float* __restrict__ var_in, T* __restrict__ ty,
                                                                         long long rows, int hidden, float eps) {
    __shared__ double scratch[16];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* yr = y + row * hidden;
        const T* tr = t + row * hidden;
        double at = 0.0, ay = 0.0, ayt = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float yv = Vec<T>::load1(yr + j), tv = Vec<T>::load1(tr + j);
            at += static_cast<double>(tv);
            ay += static_cast<double>(yv);
            ayt += static_cast<double>(mul_rn(yv, tv));
        }
        const double st = block_sum_256(at, scratch, phase++);
        const double sy = block_sum_256(ay, scratch, phase++);
        const double syt = block_sum_256(ayt, scratch, phase++);
        float tmean, d;
        ln_jvp_stats(st, sy, syt, hidden, &tmean, &d);
        const float std_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var_in[row], eps)));
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float yv = Vec<T>::load1(yr + j);
            const float tc = sub_rn(Vec<T>::load1(tr + j), tmean);
            Vec<T>::store1(ty + row * hidden + j, mul_rn(std_inv, sub_rn(tc, mul_rn(yv, d))));
        }
    }
}

}  // namespace agb
