// elementwise.cuh -- the small kernels either side of the norm: residual add and its VJP, the
// broadcast gamma product, row reductions and the deterministic global sum / mean.
#pragma once
#include "agb_device.cuh"

namespace agb {

// out = a + b.  16-byte vectors when `vec` (all pointers 16-byte aligned), scalar tail otherwise.
template <typename T>
__global__ void __launch_bounds__(256) residual_add_kernel(const T* a, const T* b, T* out, long long n, int vec) {
    constexpr int EPV = Vec<T>::EPV;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long nv = vec ? n / EPV : 0;
    for (long long v = tid; v < nv; v += nthreads) {
        float av[EPV], bv[EPV];
        Vec<T>::unpack(reinterpret_cast<const uint4*>(a)[v], av);
        Vec<T>::unpack(reinterpret_cast<const uint4*>(b)[v], bv);
#pragma unroll
        for (int e = 0; e < EPV; ++e) av[e] = add_rn(av[e], bv[e]);
        reinterpret_cast<uint4*>(out)[v] = Vec<T>::pack(av);
    }
    for (long long i = nv * EPV + tid; i < n; i += nthreads)
        Vec<T>::store1(out + i, add_rn(Vec<T>::load1(a + i), Vec<T>::load1(b + i)));
}

// ga += gy; gb += gy (either may be null).
template <typename T>
__global__ void __launch_bounds__(256) vjp_add_kernel(T* ga, T* gb, const T* gy, long long n, int vec) {
    constexpr int EPV = Vec<T>::EPV;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long nv = vec ? n / EPV : 0;
    for (long long v = tid; v < nv; v += nthreads) {
        float gv[EPV], t[EPV];
        Vec<T>::unpack(reinterpret_cast<const uint4*>(gy)[v], gv);
        if (ga) {
            Vec<T>::unpack(reinterpret_cast<const uint4*>(ga)[v], t);
#pragma unroll
            for (int e = 0; e < EPV; ++e) t[e] = add_rn(t[e], gv[e]);
            reinterpret_cast<uint4*>(ga)[v] = Vec<T>::pack(t);
        }
        if (gb) {
            Vec<T>::unpack(reinterpret_cast<const uint4*>(gb)[v], t);
#pragma unroll
            for (int e = 0; e < EPV; ++e) t[e] = add_rn(t[e], gv[e]);
            reinterpret_cast<uint4*>(gb)[v] = Vec<T>::pack(t);
        }
    }
    for (long long i = nv * EPV + tid; i < n; i += nthreads) {
        const float g = Vec<T>::load1(gy + i);
        if (ga) Vec<T>::store1(ga + i, add_rn(Vec<T>::load1(ga + i), g));
        if (gb) Vec<T>::store1(gb + i, add_rn(Vec<T>::load1(gb + i), g));
    }
}

// out[r, j] = a[r, j] * g[j]
template <typename T>
__global__ void __launch_bounds__(256) scale_lastdim_kernel(const T* a, const T* g, T* out, long long rows, int hidden,
                                                            int vec) {
    constexpr int EPV = Vec<T>::EPV;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    if (vec) {
        const int nvec = hidden / EPV;
        const long long total = rows * nvec;
        for (long long v = tid; v < total; v += nthreads) {
            const int cv = static_cast<int>(v % nvec);
            float av[EPV], gv[EPV];
            Vec<T>::unpack(reinterpret_cast<const uint4*>(a)[v], av);
            Vec<T>::unpack(reinterpret_cast<const uint4*>(g)[cv], gv);
#pragma unroll
            for (int e = 0; e < EPV; ++e) av[e] = mul_rn(av[e], gv[e]);
            reinterpret_cast<uint4*>(out)[v] = Vec<T>::pack(av);
        }
    } else {
        const long long total = rows * hidden;
        for (long long i = tid; i < total; i += nthreads)
            Vec<T>::store1(out + i, mul_rn(Vec<T>::load1(a + i), Vec<T>::load1(g + (i % hidden))));
    }
}

// out[r] = op_j x[r, j]; TPR threads per row (32 or 256), 256 threads per CTA.
// op: 0 sum, 1 mean, 2 max.  Sums in fp64, rounded once (mean: divided in fp64 first).
template <typename T, int TPR>
__global__ void __launch_bounds__(256) row_reduce_kernel(const T* __restrict__ x, T* __restrict__ out, long long rows,
                                                         int hidden, int op) {
    __shared__ double s_sum[2][8];
    __shared__ float s_max[2][8];
    constexpr int RPC = 256 / TPR;
    const int grp = threadIdx.x / TPR, tig = threadIdx.x % TPR;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int phase = 0;
    for (long long row0 = static_cast<long long>(blockIdx.x) * RPC; row0 < rows;
         row0 += static_cast<long long>(gridDim.x) * RPC, phase ^= 1) {
        const long long row = row0 + grp;
        double s = 0.0;
        float m = -INFINITY;
        if (row < rows) {
            const T* xr = x + row * hidden;
            for (int j = tig; j < hidden; j += TPR) {
                const float v = Vec<T>::load1(xr + j);
                s += static_cast<double>(v);
                m = fmaxf(m, v);
            }
        }
        s = warp_sum(s);
        m = warp_max(m);
        if (TPR > 32) {
            if (lane == 0) {
                s_sum[phase][warp] = s;
                s_max[phase][warp] = m;
            }
            __syncthreads();
            s = 0.0;
            m = -INFINITY;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                s += s_sum[phase][w];
                m = fmaxf(m, s_max[phase][w]);
            }
        }
        if (row < rows && tig == 0) {
            float r;
            if (op == 0) r = static_cast<float>(s);
            else if (op == 1) r = static_cast<float>(s / static_cast<double>(hidden));
            else r = m;
            Vec<T>::store1(out + row, r);
        }
    }
}

// The same for rows that are whole 16-byte vectors at a 16-byte aligned base: one 16-byte load per thread and
// step, only the asked-for reduction is computed (MAXOP), and 16-bit values are pre-added in fp32 eight at a time
// (bf16 has 8 significant bits: such a partial sum is exact unless the eight span more than 2^13 in magnitude)
// before the fp64 accumulation, so the conversion and the fp64 addition are paid once per vector.
template <typename T, int TPR, bool MAXOP>
__global__ void __launch_bounds__(256) row_reduce_vec_kernel(const T* __restrict__ x, T* __restrict__ out, long long rows,
                                                             int hidden, int op) {
    __shared__ double s_sum[2][8];
    __shared__ float s_max[2][8];
    constexpr int RPC = 256 / TPR;
    constexpr int EPV = Vec<T>::EPV;
    const int nvec = hidden / EPV;
    const int grp = threadIdx.x / TPR, tig = threadIdx.x % TPR;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int phase = 0;
    for (long long row0 = static_cast<long long>(blockIdx.x) * RPC; row0 < rows;
         row0 += static_cast<long long>(gridDim.x) * RPC, phase ^= 1) {
        const long long row = row0 + grp;
        double s0 = 0.0, s1 = 0.0;
        float m = -INFINITY;
        if (row < rows) {
            const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
#pragma unroll 4
            for (int v = tig; v < nvec; v += TPR) {
                float f[EPV];
                Vec<T>::unpack(__ldg(xr + v), f);
                if constexpr (MAXOP) {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) m = fmaxf(m, f[e]);
                } else if constexpr (sizeof(T) == 2) {
                    s0 += static_cast<double>(((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7])));
                } else {
                    s0 += static_cast<double>(f[0]) + static_cast<double>(f[1]);
                    s1 += static_cast<double>(f[2]) + static_cast<double>(f[3]);
                }
            }
        }
        double s = MAXOP ? 0.0 : warp_sum(s0 + s1);
        if (MAXOP) m = warp_max(m);
        if (TPR > 32) {
            if (lane == 0) {
                s_sum[phase][warp] = s;
                s_max[phase][warp] = m;
            }
            __syncthreads();
            s = 0.0;
            m = -INFINITY;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                s += s_sum[phase][w];
                m = fmaxf(m, s_max[phase][w]);
            }
        }
        if (row < rows && tig == 0) {
            float r;
            if (MAXOP) r = m;
            else if (op == 1) r = static_cast<float>(s / static_cast<double>(hidden));
            else r = static_cast<float>(s);
            Vec<T>::store1(out + row, r);
        }
    }
}

// Global sum, stage 1: block b reduces elements [b*chunk, (b+1)*chunk) to partial[b].
template <typename T>
__global__ void __launch_bounds__(256) reduce_all_stage1(const T* __restrict__ x, double* __restrict__ partial,
                                                         long long n, long long chunk) {
    __shared__ double s[8];
    const long long i0 = static_cast<long long>(blockIdx.x) * chunk;
    long long i1 = i0 + chunk;
    if (i1 > n) i1 = n;
    double v = 0.0;
    constexpr int EPV = Vec<T>::EPV;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0 && chunk % EPV == 0) {
        // whole 16-byte vectors (every chunk starts on one): vector loads, 16-bit values pre-added in fp32 per vector
        const long long nv = (i1 - i0) / EPV;
        const uint4* xv = reinterpret_cast<const uint4*>(x + i0);
        double v1 = 0.0;
#pragma unroll 4
        for (long long q = threadIdx.x; q < nv; q += 256) {
            float f[EPV];
            Vec<T>::unpack(__ldg(xv + q), f);
            if constexpr (sizeof(T) == 2) {
                v += static_cast<double>(((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7])));
            } else {
                v += static_cast<double>(f[0]) + static_cast<double>(f[1]);
                v1 += static_cast<double>(f[2]) + static_cast<double>(f[3]);
            }
        }
        v += v1;
        for (long long i = i0 + nv * EPV + threadIdx.x; i < i1; i += 256) v += static_cast<double>(Vec<T>::load1(x + i));
    } else {
        for (long long i = i0 + threadIdx.x; i < i1; i += 256) v += static_cast<double>(Vec<T>::load1(x + i));
    }
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += s[w];
        partial[blockIdx.x] = t;
    }
}
// Stage 2: one warp adds the partials in index order (lane-strided, then a fixed shuffle tree).
template <typename T>
__global__ void __launch_bounds__(32) reduce_all_stage2(const double* __restrict__ partial, int nblocks, T* out,
                                                        long long n, int op) {
    double v = 0.0;
    for (int i = threadIdx.x; i < nblocks; i += 32) v += partial[i];
    v = warp_sum(v);
    if (threadIdx.x == 0) {
        const float r = op == 1 ? static_cast<float>(v / static_cast<double>(n)) : static_cast<float>(v);
        Vec<T>::store1(out, r);
    }
}

// Broadcast modes of the second operand of a [rows, hidden] elementwise op.
enum BcastMode { kBcastFull = 0, kBcastLastVec = 1, kBcastRowStat = 2, kBcastScalar = 3 };

template <typename T>
__device__ __forceinline__ float bcast_load(const T* b, int mode, long long row, int col, long long idx) {
    switch (mode) {
        case kBcastFull: return Vec<T>::load1(b + idx);
        case kBcastLastVec: return Vec<T>::load1(b + col);
        case kBcastRowStat: return Vec<T>::load1(b + row);
        default: return Vec<T>::load1(b);
    }
}
// The value a tensor of type T would hold after storing v (identity for fp32, one rounding for bf16).
template <typename T>
__device__ __forceinline__ float as_stored(float v);
template <>
__device__ __forceinline__ float as_stored<float>(float v) { return v; }
template <>
__device__ __forceinline__ float as_stored<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// out = a (op) broadcast(b);  op 0 add, 1 mul.  One rounding, like one tensor call.
template <typename T>
__global__ void __launch_bounds__(256) binary_broadcast_kernel(const T* a, const T* b, T* out, long long rows, int hidden,
                                                               int mode, int op) {
    const long long total = rows * hidden;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += nthreads) {
        const long long row = i / hidden;
        const int col = static_cast<int>(i - row * hidden);
        const float av = Vec<T>::load1(a + i);
        const float bv = bcast_load(b, mode, row, col, i);
        Vec<T>::store1(out + i, op == 0 ? add_rn(av, bv) : mul_rn(av, bv));
    }
}

// dst += broadcast(src) [* scale].  With use_scale the product is rounded first, as the separate
// tensor call `gy * scale` of the reference would, then the accumulation rounds once more.
template <typename T>
__global__ void __launch_bounds__(256) accumulate_broadcast_kernel(T* dst, const T* src, long long rows, int hidden,
                                                                   int mode, float scale, int use_scale) {
    const long long total = rows * hidden;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += nthreads) {
        const long long row = i / hidden;
        const int col = static_cast<int>(i - row * hidden);
        float sv = bcast_load(src, mode, row, col, i);
        if (use_scale) sv = as_stored<T>(mul_rn(sv, scale));
        Vec<T>::store1(dst + i, add_rn(Vec<T>::load1(dst + i), sv));
    }
}

// Column sums of a product, stage 1: partials[p, c] = sum over the p-th chunk of rows of g*a
// (a may be null: plain column sum).  grid (ceil(hidden/256), P); rows in order, fp64.
template <typename T>
__global__ void __launch_bounds__(256) mul_colsum_partial_kernel(const T* __restrict__ g, const T* __restrict__ a,
                                                                 double* __restrict__ partials, long long rows,
                                                                 int hidden, long long rows_per_chunk) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_chunk;
    long long r1 = r0 + rows_per_chunk;
    if (r1 > rows) r1 = rows;
    if (c >= hidden) return;
    double acc = 0.0;
    for (long long row = r0; row < r1; ++row) {
        float v = Vec<T>::load1(g + row * hidden + c);
        if (a) v = as_stored<T>(mul_rn(v, Vec<T>::load1(a + row * hidden + c)));
        acc += static_cast<double>(v);
    }
    partials[static_cast<size_t>(blockIdx.y) * hidden + c] = acc;
}
// Stage 2 for a T-typed destination: out[c] (+)= (T) sum_p partials[p, c], p in order.
template <typename T>
__global__ void __launch_bounds__(256) colsum_finish_kernel(const double* __restrict__ partials, int P, int hidden,
                                                            T* out, int accumulate) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= hidden) return;
    double t = 0.0;
    for (int p = 0; p < P; ++p) t += partials[static_cast<size_t>(p) * hidden + c];
    const float v = as_stored<T>(static_cast<float>(t));
    Vec<T>::store1(out + c, accumulate ? add_rn(Vec<T>::load1(out + c), v) : v);
}

// Row sums of a product: out[r] (+)= (T) sum_j g[r,j]*a[r,j]; one CTA of 256 threads per row.
template <typename T>
__global__ void __launch_bounds__(256) mul_rowsum_kernel(const T* __restrict__ g, const T* __restrict__ a, T* out,
                                                         long long rows, int hidden, int accumulate) {
    __shared__ double s[2][8];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, phase ^= 1) {
        double acc = 0.0;
        for (int j = threadIdx.x; j < hidden; j += 256) {
            float v = Vec<T>::load1(g + row * hidden + j);
            if (a) v = as_stored<T>(mul_rn(v, Vec<T>::load1(a + row * hidden + j)));
            acc += static_cast<double>(v);
        }
        acc = warp_sum(acc);
        if ((threadIdx.x & 31) == 0) s[phase][threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += s[phase][w];
            const float v = as_stored<T>(static_cast<float>(t));
            Vec<T>::store1(out + row, accumulate ? add_rn(Vec<T>::load1(out + row), v) : v);
        }
    }
}

// Global sum of a product, stage 1 (same chunking as reduce_all_stage1); stage 2 below.
template <typename T>
__global__ void __launch_bounds__(256) mul_sumall_stage1(const T* __restrict__ g, const T* __restrict__ a,
                                                         double* __restrict__ partial, long long n, long long chunk) {
    __shared__ double s[8];
    const long long i0 = static_cast<long long>(blockIdx.x) * chunk;
    long long i1 = i0 + chunk;
    if (i1 > n) i1 = n;
    double v = 0.0;
    for (long long i = i0 + threadIdx.x; i < i1; i += 256) {
        float t = Vec<T>::load1(g + i);
        if (a) t = as_stored<T>(mul_rn(t, Vec<T>::load1(a + i)));
        v += static_cast<double>(t);
    }
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += s[w];
        partial[blockIdx.x] = t;
    }
}
template <typename T>
__global__ void __launch_bounds__(32) sumall_finish_kernel(const double* __restrict__ partial, int nblocks, T* out,
                                                           int accumulate) {
    double v = 0.0;
    for (int i = threadIdx.x; i < nblocks; i += 32) v += partial[i];
    v = warp_sum(v);
    if (threadIdx.x == 0) {
        const float r = as_stored<T>(static_cast<float>(v));
        Vec<T>::store1(out, accumulate ? add_rn(Vec<T>::load1(out), r) : r);
    }
}

// ---------------------------------------------------------------- optimiser steps on parameters
// SGD as the reference writes it (cgadimpl/src/optimizer/optim.cpp:12-19):
//   value += -learning_rate * grad      -> t = (-lr)*g rounded, then p + t rounded
template <typename T>
__global__ void __launch_bounds__(256) sgd_step_kernel(T* p, const T* g, long long n, float neg_lr) {
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += nthreads) {
        const float t = as_stored<T>(mul_rn(neg_lr, Vec<T>::load1(g + i)));
        Vec<T>::store1(p + i, add_rn(Vec<T>::load1(p + i), t));
    }
}

// Adam as the reference writes it (optim.cpp:33-72), one rounding per tensor operation:
//   m *= b1;  m += (1-b1)*g;  v *= b2;  v += (1-b2)*square(g);
//   value -= alpha_eff * m / (sqrt(v) + eps_eff)
__global__ void __launch_bounds__(256) adam_step_kernel(float* p, const float* g, float* m, float* v, long long n,
                                                        float b1, float b2, float omb1, float omb2, float alpha_eff,
                                                        float eps_eff) {
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += nthreads) {
        const float gi = g[i];
        const float mi = add_rn(mul_rn(m[i], b1), mul_rn(omb1, gi));
        const float vi = add_rn(mul_rn(v[i], b2), mul_rn(omb2, mul_rn(gi, gi)));
        m[i] = mi;
        v[i] = vi;
        const float num = mul_rn(alpha_eff, mi);
        const float den = add_rn(__fsqrt_rn(vi), eps_eff);
        p[i] = sub_rn(p[i], __fdiv_rn(num, den));
    }
}

}  // namespace agb
