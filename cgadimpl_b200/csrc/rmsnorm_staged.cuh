// rmsnorm_staged.cuh -- the bandwidth-bound RMSNorm kernels for B200.
//
// One persistent CTA per SM slot walks over tiles of consecutive rows.  A tile of every input
// array is brought into a shared-memory ring by the bulk asynchronous copy engine
// (cp.async.bulk, untiled, no multicast) and signalled on an mbarrier, so the bytes in flight
// are bounded by shared memory (up to ~200 KB per SM), not by registers or occupancy.  A group
// of `group_threads` threads owns one row of the tile; each thread reads 16-byte vectors
// (conflict-free, consecutive threads -> consecutive vectors), reduces in fp64 with warp
// shuffles plus one shared-memory step, and writes its outputs with 16-byte streaming stores.
// gamma sits in shared memory for the life of the CTA.  The backward kernel keeps its
// per-column dgamma sums in fp64 registers across all its rows and writes one partial row per
// CTA; a second, fixed-order kernel reduces the partials, so dgamma is bit-reproducible.
//
// Rounding follows the reference's op-by-op composition: every elementwise product / sum that
// the reference materialises as an fp32 tensor is rounded to fp32 here (no FMA contraction),
// and every reduction is carried in fp64 and rounded once.
#pragma once
#include "agb_device.cuh"

namespace agb {

struct PipeGeom {
    long long rows;
    long long ntiles;
    int hidden;
    int nvec;           // 16-byte vectors per row
    int row_bytes;
    int rows_per_tile;  // row groups per CTA
    int group_threads;  // threads per row, multiple of 32
    int stages;
    int tile_stride;    // bytes between the staged arrays inside one stage
    int stage_stride;   // bytes between stages
    int off_gamma;      // shared-memory offsets
    int off_gamma2;
    int off_red;
    int off_bar;
    int off_flag;
};

// Issues the bulk copies of one tile into a ring slot.  Called by one thread.
template <int NARR>
__device__ __forceinline__ void issue_tile(const PipeGeom& g, unsigned char* ring, uint64_t* full,
                                           const unsigned char* const (&src)[NARR], long long tile, int slot) {
    const long long row0 = tile * g.rows_per_tile;
    long long nrows = g.rows - row0;
    if (nrows > g.rows_per_tile) nrows = g.rows_per_tile;
    const uint32_t bytes = static_cast<uint32_t>(nrows) * static_cast<uint32_t>(g.row_bytes);
    mbar_arrive_expect_tx(&full[slot], bytes * NARR);
#pragma unroll
    for (int a = 0; a < NARR; ++a)
        bulk_load(ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(a) * g.tile_stride,
                  src[a] + row0 * g.row_bytes, bytes, &full[slot]);
}

// After a bounded wait ran out: wait (bounded again) for the copies this CTA still has in
// flight so none lands after the CTA has gone, then publish the status.
__device__ __forceinline__ void drain_after_abort(const PipeGeom& g, uint64_t* full, long long next_to_wait,
                                                  long long issued) {
    for (long long k = next_to_wait; k < issued; ++k)
        mbar_wait_bounded(&full[k % g.stages], static_cast<uint32_t>((k / g.stages) & 1));
    atomicExch(&g_device_status, 6 /* AGB_ERR_TIMEOUT */);
}

// ------------------------------------------------------------------------------------------
// Forward.  y = (x*rstd)*gamma, rstd saved.  FUSE_ADD: h = x + r is formed first, written out
// and normalised instead of x.
// ------------------------------------------------------------------------------------------
struct FwdArgs {
    PipeGeom g;
    const void* x;
    const void* r;      // FUSE_ADD only
    const void* gamma;  // HAS_GAMMA only
    void* h;            // FUSE_ADD only
    void* y;
    float* rstd;
    float eps;
};

template <typename T, bool HAS_GAMMA, bool FUSE_ADD>
__global__ void __launch_bounds__(1024, 1) rmsnorm_fwd_staged(const __grid_constant__ FwdArgs a) {
    constexpr int EPV = Vec<T>::EPV;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    const uint4* s_gamma = reinterpret_cast<const uint4*>(smem + g.off_gamma);
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
    if (HAS_GAMMA) {
        uint4* dst = reinterpret_cast<uint4*>(smem + g.off_gamma);
        const uint4* src = reinterpret_cast<const uint4*>(a.gamma);
        for (int v = tid; v < g.nvec; v += blockDim.x) dst[v] = src[v];
    }
    __syncthreads();

    const unsigned char* const src2[2] = {reinterpret_cast<const unsigned char*>(a.x),
                                          reinterpret_cast<const unsigned char*>(a.r)};
    auto issue = [&](long long tile, int slot) {
        if (FUSE_ADD)
            issue_tile<2>(g, ring, s_full, src2, tile, slot);
        else
            issue_tile<1>(g, ring, s_full, reinterpret_cast<const unsigned char* const(&)[1]>(src2), tile, slot);
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
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;

        const uint4* sx = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(slot) * g.stage_stride +
                                                         static_cast<size_t>(grp) * g.row_bytes);
        const uint4* sr = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sx) + g.tile_stride);
        uint4* gh = FUSE_ADD ? reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.h) + row * g.row_bytes) : nullptr;

        // pass 1: sum of squares (each square rounded to fp32, summed in fp64)
        double ss0 = 0.0, ss1 = 0.0;
        if (valid) {
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float xv[EPV];
                Vec<T>::unpack(sx[v], xv);
                if (FUSE_ADD) {
                    float rv[EPV];
                    Vec<T>::unpack(sr[v], rv);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) xv[e] = add_rn(xv[e], rv[e]);
                    const uint4 hp = Vec<T>::pack(xv);
                    store_vec_streaming(gh + v, hp);
                    Vec<T>::unpack(hp, xv);  // the norm sees h as stored (bf16: after rounding)
                }
#pragma unroll
                for (int e = 0; e < EPV; e += 2) {
                    ss0 += static_cast<double>(mul_rn(xv[e], xv[e]));
                    ss1 += static_cast<double>(mul_rn(xv[e + 1], xv[e + 1]));
                }
            }
        }
        double ss = warp_sum(ss0 + ss1);
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = ss;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        // every thread has finished with the slot of the previous iteration: refill it
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue(first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        double tot = 0.0;
        for (int w = 0; w < wpr; ++w) tot += s_red[(k & 1) * nwarps + grp * wpr + w];
        const float rs = rstd_from_sumsq(tot, g.hidden, a.eps);

        // pass 2: y = (x*rstd)*gamma
        if (valid) {
            if (tig == 0) a.rstd[row] = rs;
            uint4* gy = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.y) + row * g.row_bytes);
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float xv[EPV];
                Vec<T>::unpack(sx[v], xv);
                if (FUSE_ADD) {
                    float rv[EPV];
                    Vec<T>::unpack(sr[v], rv);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) xv[e] = add_rn(xv[e], rv[e]);
                    const uint4 hp = Vec<T>::pack(xv);
                    Vec<T>::unpack(hp, xv);
                }
                float gv[EPV];
                if (HAS_GAMMA) Vec<T>::unpack(s_gamma[v], gv);
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    float yh = mul_rn(xv[e], rs);
                    xv[e] = HAS_GAMMA ? mul_rn(yh, gv[e]) : yh;
                }
                store_vec_streaming(gy + v, Vec<T>::pack(xv));
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

// ------------------------------------------------------------------------------------------
// Backward.  dx = rstd*(dy - x*rstd^2*dot/H) [+ add], dy = gy*gamma; dgamma partial per CTA.
// add_mode: 0 none, 1 a third staged array, 2 the addend is gy itself (read once).
// ------------------------------------------------------------------------------------------
struct BwdArgs {
    PipeGeom g;
    const void* x;
    const void* gy;
    const void* add;    // add_mode 1
    const void* gamma;  // HAS_GAMMA
    const float* rstd;
    void* dx;
    double* partials;   // [gridDim.x, hidden], HAS_GAMMA and non-null
    int add_mode;
    float hidden_f, hidden_inv;
};

template <typename T, int VPT, bool HAS_GAMMA>
__global__ void __launch_bounds__(512, 1) rmsnorm_bwd_staged(const __grid_constant__ BwdArgs a) {
    constexpr int EPV = Vec<T>::EPV;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    const uint4* s_gamma = reinterpret_cast<const uint4*>(smem + g.off_gamma);
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;
    const bool staged_add = a.add_mode == 1;
    const DivConst div_h{a.hidden_f, a.hidden_inv};

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    if (HAS_GAMMA) {
        uint4* dst = reinterpret_cast<uint4*>(smem + g.off_gamma);
        const uint4* src = reinterpret_cast<const uint4*>(a.gamma);
        for (int v = tid; v < g.nvec; v += blockDim.x) dst[v] = src[v];
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

    double acc[HAS_GAMMA ? VPT * EPV : 1];
#pragma unroll
    for (int i = 0; i < (HAS_GAMMA ? VPT * EPV : 1); ++i) acc[i] = 0.0;

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        const float rs = valid ? a.rstd[row] : 0.0f;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;

        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sx = reinterpret_cast<const uint4*>(base);
        const uint4* sg = reinterpret_cast<const uint4*>(base + g.tile_stride);
        const uint4* sa = reinterpret_cast<const uint4*>(base + 2 * static_cast<size_t>(g.tile_stride));

        // pass 1: dot = sum(dy*x), products rounded to fp32, summed in fp64
        double d0 = 0.0, d1 = 0.0;
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (v < g.nvec) {
                    float xv[EPV], gv[EPV];
                    Vec<T>::unpack(sx[v], xv);
                    Vec<T>::unpack(sg[v], gv);
                    if (HAS_GAMMA) {
                        float wv[EPV];
                        Vec<T>::unpack(s_gamma[v], wv);
#pragma unroll
                        for (int e = 0; e < EPV; ++e) gv[e] = mul_rn(gv[e], wv[e]);
                    }
#pragma unroll
                    for (int e = 0; e < EPV; e += 2) {
                        d0 += static_cast<double>(mul_rn(gv[e], xv[e]));
                        d1 += static_cast<double>(mul_rn(gv[e + 1], xv[e + 1]));
                    }
                }
            }
        }
        double dsum = warp_sum(d0 + d1);
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = dsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue(first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        double tot = 0.0;
        for (int w = 0; w < wpr; ++w) tot += s_red[(k & 1) * nwarps + grp * wpr + w];
        const float dot = static_cast<float>(tot);
        const float r2 = mul_rn(rs, rs);

        // pass 2: dx and the dgamma terms
        if (valid) {
            uint4* gdx = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.dx) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (v < g.nvec) {
                    float xv[EPV], gv[EPV], ov[EPV];
                    Vec<T>::unpack(sx[v], xv);
                    Vec<T>::unpack(sg[v], gv);
                    float wv[EPV];
                    if (HAS_GAMMA) Vec<T>::unpack(s_gamma[v], wv);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        const float dy = HAS_GAMMA ? mul_rn(gv[e], wv[e]) : gv[e];
                        float t = mul_rn(xv[e], r2);
                        t = mul_rn(t, dot);
                        t = div_h(t);
                        t = sub_rn(dy, t);
                        ov[e] = mul_rn(rs, t);
                        if (HAS_GAMMA) {
                            const float yh = mul_rn(xv[e], rs);
                            acc[i * EPV + e] += static_cast<double>(mul_rn(gv[e], yh));
                        }
                    }
                    if (a.add_mode == 2) {
#pragma unroll
                        for (int e = 0; e < EPV; ++e) ov[e] = add_rn(ov[e], gv[e]);
                    } else if (staged_add) {
                        float av[EPV];
                        Vec<T>::unpack(sa[v], av);
#pragma unroll
                        for (int e = 0; e < EPV; ++e) ov[e] = add_rn(ov[e], av[e]);
                    }
                    store_vec_streaming(gdx + v, Vec<T>::pack(ov));
                }
            }
        }
    }
    if (aborted) {
        if (tid == 0) drain_after_abort(g, s_full, k, issued);
        return;
    }

    if (HAS_GAMMA && a.partials != nullptr) {
        double* prow = a.partials + static_cast<size_t>(blockIdx.x) * g.hidden;
        if (g.rows_per_tile == 1) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (v < g.nvec) {
#pragma unroll
                    for (int e = 0; e < EPV; e += 2)
                        *reinterpret_cast<double2*>(prow + static_cast<size_t>(v) * EPV + e) =
                            make_double2(acc[i * EPV + e], acc[i * EPV + e + 1]);
                }
            }
        } else {
            // combine the row groups of this CTA in group order, through the (now idle) ring
            __syncthreads();
            double* s_acc = reinterpret_cast<double*>(ring);
            for (int gi = 0; gi < g.rows_per_tile; ++gi) {
                if (grp == gi) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        const int v = tig + i * G;
                        if (v < g.nvec) {
#pragma unroll
                            for (int e = 0; e < EPV; ++e) {
                                const int c = v * EPV + e;
                                s_acc[c] = gi == 0 ? acc[i * EPV + e] : s_acc[c] + acc[i * EPV + e];
                            }
                        }
                    }
                }
                __syncthreads();
            }
            for (int c = tid; c < g.hidden; c += blockDim.x) prow[c] = s_acc[c];
        }
    }
}

// Stage 2: dgamma[c] = sum over partial rows p = 0..P-1, fixed order, fp64.
// Block (32, 8): thread (cx, py) sums rows py, py+8, ... of column c, then the 8 sub-sums are
// added in py order.  out_mode 0: fp32 store, 1: fp32 accumulate, 2: fp64 store, 3: fp64 accumulate.
__global__ void __launch_bounds__(256) dgamma_reduce_kernel(const double* __restrict__ partials, int P, int hidden,
                                                            void* out, int out_mode) {
    __shared__ double s[8][33];
    const int cx = threadIdx.x, py = threadIdx.y;
    const int c = blockIdx.x * 32 + cx;
    double v = 0.0;
    if (c < hidden)
        for (int p = py; p < P; p += 8) v += partials[static_cast<size_t>(p) * hidden + c];
    s[py][cx] = v;
    __syncthreads();
    if (py == 0 && c < hidden) {
        double t = s[0][cx];
#pragma unroll
        for (int j = 1; j < 8; ++j) t += s[j][cx];
        if (out_mode == 2)
            static_cast<double*>(out)[c] = t;
        else if (out_mode == 3)
            static_cast<double*>(out)[c] += t;
        else if (out_mode == 1)
            static_cast<float*>(out)[c] = add_rn(static_cast<float*>(out)[c], static_cast<float>(t));
        else
            static_cast<float*>(out)[c] = static_cast<float>(t);
    }
}

__global__ void dgamma_finalize_kernel(const double* __restrict__ sum, float* __restrict__ dgamma, int hidden,
                                       int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < hidden) {
        const float v = static_cast<float>(sum[c]);
        dgamma[c] = accumulate ? add_rn(dgamma[c], v) : v;
    }
}

// ------------------------------------------------------------------------------------------
// JVP (corrected form).  ty = (tx*rstd - (yhat*dot)*(rstd/H)) * gamma + yhat*tgamma
// ------------------------------------------------------------------------------------------
struct JvpArgs {
    PipeGeom g;
    const void* x;
    const void* tx;
    const void* gamma;   // nullable
    const void* tgamma;  // nullable (needs gamma)
    const float* rstd;
    void* ty;
    float hidden_f;
};

template <typename T>
__global__ void __launch_bounds__(1024, 1) rmsnorm_jvp_staged(const __grid_constant__ JvpArgs a) {
    constexpr int EPV = Vec<T>::EPV;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    const uint4* s_gamma = reinterpret_cast<const uint4*>(smem + g.off_gamma);
    const uint4* s_tgamma = reinterpret_cast<const uint4*>(smem + g.off_gamma2);
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);
    const bool has_gamma = a.gamma != nullptr, has_tgamma = a.tgamma != nullptr;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    for (int v = tid; v < g.nvec; v += blockDim.x) {
        if (has_gamma) reinterpret_cast<uint4*>(smem + g.off_gamma)[v] = reinterpret_cast<const uint4*>(a.gamma)[v];
        if (has_tgamma) reinterpret_cast<uint4*>(smem + g.off_gamma2)[v] = reinterpret_cast<const uint4*>(a.tgamma)[v];
    }
    __syncthreads();

    const unsigned char* const src2[2] = {reinterpret_cast<const unsigned char*>(a.x),
                                          reinterpret_cast<const unsigned char*>(a.tx)};
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
        const float rs = valid ? a.rstd[row] : 0.0f;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sx = reinterpret_cast<const uint4*>(base);
        const uint4* st = reinterpret_cast<const uint4*>(base + g.tile_stride);

        double d0 = 0.0, d1 = 0.0;
        if (valid) {
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float xv[EPV], tv[EPV];
                Vec<T>::unpack(sx[v], xv);
                Vec<T>::unpack(st[v], tv);
#pragma unroll
                for (int e = 0; e < EPV; e += 2) {
                    d0 += static_cast<double>(mul_rn(tv[e], mul_rn(xv[e], rs)));
                    d1 += static_cast<double>(mul_rn(tv[e + 1], mul_rn(xv[e + 1], rs)));
                }
            }
        }
        double dsum = warp_sum(d0 + d1);
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = dsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue_tile<2>(g, ring, s_full, src2, first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        double tot = 0.0;
        for (int w = 0; w < wpr; ++w) tot += s_red[(k & 1) * nwarps + grp * wpr + w];
        const float dot = static_cast<float>(tot);
        const float c = __fdiv_rn(rs, a.hidden_f);

        if (valid) {
            uint4* gout = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.ty) + row * g.row_bytes);
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float xv[EPV], tv[EPV], wv[EPV], twv[EPV];
                Vec<T>::unpack(sx[v], xv);
                Vec<T>::unpack(st[v], tv);
                if (has_gamma) Vec<T>::unpack(s_gamma[v], wv);
                if (has_tgamma) Vec<T>::unpack(s_tgamma[v], twv);
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    const float yh = mul_rn(xv[e], rs);
                    const float q = mul_rn(tv[e], rs);
                    float p = mul_rn(yh, dot);
                    p = mul_rn(p, c);
                    float o = sub_rn(q, p);
                    if (has_gamma) {
                        o = mul_rn(o, wv[e]);
                        if (has_tgamma) o = add_rn(o, mul_rn(yh, twv[e]));
                    }
                    xv[e] = o;
                }
                store_vec_streaming(gout + v, Vec<T>::pack(xv));
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

}  // namespace agb
