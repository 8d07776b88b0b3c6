// rmsnorm_generic.cuh -- the unstaged kernels: same arithmetic and rounding points as the
// staged ones, but with ordinary element loads, so they take any hidden size and any
// element-aligned pointer (rows whose byte length is not a multiple of 16, rows too wide for
// the shared-memory ring).  One CTA of 256 threads per row, grid-stride over rows; inputs are
// read twice (the second read normally hits L1/L2).  Correctness path, not the fast path.
#pragma once
#include "agb_device.cuh"

namespace agb {

constexpr int kGenericThreads = 256;

// Sum over the CTA, identical in every thread, fixed order.  `scratch` holds >= 2*8 doubles and is
// double-buffered by `phase` so one __syncthreads per call suffices.
__device__ __forceinline__ double block_sum_256(double v, double* scratch, int phase) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    double* s = scratch + (phase & 1) * 8;
    if (lane == 0) s[warp] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < kGenericThreads / 32; ++w) t += s[w];
    return t;
}

template <typename T, bool FUSE_ADD>
__global__ void __launch_bounds__(kGenericThreads) rmsnorm_fwd_generic(const T* __restrict__ x, const T* __restrict__ r,
                                                                       const T* __restrict__ gamma, T* __restrict__ h,
                                                                       T* __restrict__ y, float* __restrict__ rstd,
                                                                       long long rows, int hidden, float eps) {
    __shared__ double scratch[16];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++phase) {
        const T* xr = x + row * hidden;
        const T* rr = FUSE_ADD ? r + row * hidden : nullptr;
        T* hr = FUSE_ADD ? h + row * hidden : nullptr;
        double ss = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            float v = Vec<T>::load1(xr + j);
            if (FUSE_ADD) {
                v = add_rn(v, Vec<T>::load1(rr + j));
                Vec<T>::store1(hr + j, v);
                v = Vec<T>::load1(hr + j);  // the norm sees h as stored
            }
            ss += static_cast<double>(mul_rn(v, v));
        }
        const double tot = block_sum_256(ss, scratch, phase);
        const float rs = rstd_from_sumsq(tot, hidden, eps);
        if (threadIdx.x == 0) rstd[row] = rs;
        const T* in = FUSE_ADD ? hr : xr;
        T* yr = y + row * hidden;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float yh = mul_rn(Vec<T>::load1(in + j), rs);
            Vec<T>::store1(yr + j, gamma ? mul_rn(yh, Vec<T>::load1(gamma + j)) : yh);
        }
    }
}

// dx only; dgamma comes from dgamma_generic_partial below.
template <typename T>
__global__ void __launch_bounds__(kGenericThreads) rmsnorm_bwd_generic(const T* __restrict__ x, const T* __restrict__ gamma,
                                                                       const float* __restrict__ rstd,
                                                                       const T* __restrict__ gy, const T* add, T* dx,
                                                                       long long rows, int hidden, float hidden_f,
                                                                       float hidden_inv) {
    __shared__ double scratch[16];
    const DivConst div_h{hidden_f, hidden_inv};
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++phase) {
        const T* xr = x + row * hidden;
        const T* gr = gy + row * hidden;
        const T* ar = add ? add + row * hidden : nullptr;
        T* dr = dx + row * hidden;
        const float rs = rstd[row];
        double d = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            float dy = Vec<T>::load1(gr + j);
            if (gamma) dy = mul_rn(dy, Vec<T>::load1(gamma + j));
            d += static_cast<double>(mul_rn(dy, Vec<T>::load1(xr + j)));
        }
        const float dot = static_cast<float>(block_sum_256(d, scratch, phase));
        const float r2 = mul_rn(rs, rs);
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float xv = Vec<T>::load1(xr + j);
            float dy = Vec<T>::load1(gr + j);
            if (gamma) dy = mul_rn(dy, Vec<T>::load1(gamma + j));
            float t = mul_rn(xv, r2);
            t = mul_rn(t, dot);
            t = div_h(t);
            t = sub_rn(dy, t);
            t = mul_rn(rs, t);
            if (ar) t = add_rn(t, Vec<T>::load1(ar + j));  // may alias dx or gy: read before the write below
            Vec<T>::store1(dr + j, t);
        }
    }
}

// partials[p, c] = sum over the p-th chunk of rows of gy*(x*rstd), fp64, rows in order.
// grid (ceil(hidden/256), P).  Must run BEFORE a dx that aliases gy is written.
template <typename T>
__global__ void __launch_bounds__(kGenericThreads) dgamma_generic_partial(const T* __restrict__ x,
                                                                          const T* __restrict__ gy,
                                                                          const float* __restrict__ rstd,
                                                                          double* __restrict__ partials, long long rows,
                                                                          int hidden, long long rows_per_chunk) {
    const int c = blockIdx.x * kGenericThreads + threadIdx.x;
    const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_chunk;
    long long r1 = r0 + rows_per_chunk;
    if (r1 > rows) r1 = rows;
    if (c >= hidden) return;
    double acc = 0.0;
    for (long long row = r0; row < r1; ++row) {
        const float yh = mul_rn(Vec<T>::load1(x + row * hidden + c), rstd[row]);
        acc += static_cast<double>(mul_rn(Vec<T>::load1(gy + row * hidden + c), yh));
    }
    partials[static_cast<size_t>(blockIdx.y) * hidden + c] = acc;
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads) rmsnorm_jvp_generic(const T* __restrict__ x, const T* __restrict__ gamma,
                                                                       const float* __restrict__ rstd,
                                                                       const T* __restrict__ tx,
                                                                       const T* __restrict__ tgamma, T* __restrict__ ty,
                                                                       long long rows, int hidden, float hidden_f) {
    __shared__ double scratch[16];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++phase) {
        const T* xr = x + row * hidden;
        const T* tr = tx + row * hidden;
        T* out = ty + row * hidden;
        const float rs = rstd[row];
        double d = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads)
            d += static_cast<double>(mul_rn(Vec<T>::load1(tr + j), mul_rn(Vec<T>::load1(xr + j), rs)));
        const float dot = static_cast<float>(block_sum_256(d, scratch, phase));
        const float c = __fdiv_rn(rs, hidden_f);
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            const float yh = mul_rn(Vec<T>::load1(xr + j), rs);
            const float q = mul_rn(Vec<T>::load1(tr + j), rs);
            float p = mul_rn(yh, dot);
            p = mul_rn(p, c);
            float o = sub_rn(q, p);
            if (gamma) {
                o = mul_rn(o, Vec<T>::load1(gamma + j));
                if (tgamma) o = add_rn(o, mul_rn(yh, Vec<T>::load1(tgamma + j)));
            }
            Vec<T>::store1(out + j, o);
        }
    }
}

}  // namespace agb
