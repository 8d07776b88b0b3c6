// rmsnorm_staged.cuh -- the bandwidth-bound RMSNorm kernels for B200.
//
// One persistent CTA per SM slot walks over tiles of consecutive rows.  A tile of every input
// array is brought into a shared-memory ring by the bulk asynchronous copy engine
// (cp.async.bulk, untiled, no multicast) and signalled on an mbarrier, so the bytes in flight
// are bounded by shared memory, not by registers or occupancy.  A group of `group_threads`
// threads owns one row of the tile; each thread reads 16-byte vectors (conflict-free, consecutive
// threads -> consecutive vectors), reduces in fp64 with warp shuffles plus one shared-memory
// step, and writes its outputs with 16-byte streaming stores.  gamma sits in shared memory, already
// widened to fp32, for the life of the CTA.  The backward kernel keeps its per-column dgamma sums
// in fp64 registers across all its rows and writes one partial row per CTA; a second, fixed-order
// kernel reduces the partials, so dgamma is bit-reproducible.
//
// Rounding follows the reference's op-by-op composition: every elementwise product / sum that
// the reference materialises as an fp32 tensor is rounded to fp32 here (no FMA contraction),
// and every reduction is carried in fp64 and rounded once.  The elementwise arithmetic uses the
// packed two-lane fp32 instructions of sm_100 (__fmul2_rn / __ffma2_rn): same IEEE result per
// lane, half the issue slots -- these kernels are limited by instruction issue, not by DRAM, as
// soon as the data type is 16 bits wide.
#pragma once
#include "agb_device.cuh"

namespace agb {

struct PipeGeom {
    long long rows;
    long long ntiles;
    int hidden;
    int nvec;           // 16-byte vectors per row
    int row_bytes;
    int rows_per_tile;  // rows per tile (= row groups per CTA, times rows_per_warp)
    int rows_per_warp;  // > 1 only in the backward with one-warp rows: rows a warp handles per tile (else 1)
    int group_threads;  // threads per row, multiple of 32
    int stages;
    int tile_stride;    // bytes between the staged arrays inside one stage
    int stage_stride;   // bytes between stages
    int off_gamma;      // shared-memory offsets; gamma is stored as fp32, hidden*4 bytes
    int off_gamma2;
    int off_red;
    int off_bar;
    int off_flag;
    int pdl_early;      // 1: let the next kernel's CTAs be placed as soon as this one has started (else: when it drains)
    int early_refill;   // backward (fp32-accumulating): the last warp to leave a ring slot refills it at once
};

// ---------------------------------------------------------------- packed fp32 helpers
// CAUTION.  The packed intrinsics are documented to behave per lane like __fmul_rn / __fadd_rn, but
// unlike those a __fmul2_rn feeding a __fadd2_rn WAS observed to become one FFMA2 (measured: 24 % of
// the results off by one rounding; neither --fmad=false nor an optimisation barrier between the two
// prevents it).  Rule in these kernels: add2 / sub2 only where NO operand is a product; an addition
// or subtraction that consumes a product uses add2_after_mul / sub2_after_mul, built from the scalar
// intrinsics, which are never fused.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 add2_after_mul(float2 a, float2 b) {
    return make_float2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
}
__device__ __forceinline__ float2 sub2_after_mul(float2 a, float2 b) {
    return make_float2(__fsub_rn(a.x, b.x), __fsub_rn(a.y, b.y));
}
// a - b, one rounding (an FMA with multiplier -1 is exact up to that rounding)
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a); }
__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }
struct DivConst2 {
    float2 d, dinv;
    __device__ __forceinline__ float2 operator()(float2 a) const {
        const float2 q0 = __fmul2_rn(a, dinv);
        const float2 r = __ffma2_rn(make_float2(-q0.x, -q0.y), d, a);
        return __ffma2_rn(r, dinv, q0);
    }
};

// 16-byte vector <-> NP pairs of floats
template <typename T>
struct Pairs;
template <>
struct Pairs<float> {
    static constexpr int NP = 2;
    __device__ __forceinline__ static void unpack(const uint4& u, float2 (&p)[2]) {
        p[0] = make_float2(__uint_as_float(u.x), __uint_as_float(u.y));
        p[1] = make_float2(__uint_as_float(u.z), __uint_as_float(u.w));
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&p)[2]) {
        return make_uint4(__float_as_uint(p[0].x), __float_as_uint(p[0].y), __float_as_uint(p[1].x), __float_as_uint(p[1].y));
    }
};
template <>
struct Pairs<__nv_bfloat16> {
    static constexpr int NP = 4;
    __device__ __forceinline__ static void unpack(const uint4& u, float2 (&p)[4]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&p)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 b = __floats2bfloat162_rn(p[i].x, p[i].y);
            w[i] = *reinterpret_cast<uint32_t*>(&b);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// gamma in shared memory: fp32, laid out in NP/2 planes of [nvec] float4 so that every 16-byte read
// of a warp is conflict-free.  Plane q of vector v holds pairs 2q and 2q+1 of that vector.
template <typename T>
__device__ __forceinline__ void stage_gamma(float4* s_gamma, const void* gamma, int nvec) {
    constexpr int NP = Pairs<T>::NP;
    const uint4* src = reinterpret_cast<const uint4*>(gamma);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float2 p[NP];
        Pairs<T>::unpack(src[v], p);
#pragma unroll
        for (int q = 0; q < NP / 2; ++q) s_gamma[q * nvec + v] = make_float4(p[2 * q].x, p[2 * q].y, p[2 * q + 1].x, p[2 * q + 1].y);
    }
}
template <typename T>
__device__ __forceinline__ void load_gamma(const float4* s_gamma, int nvec, int v, float2 (&w)[Pairs<T>::NP]) {
#pragma unroll
    for (int q = 0; q < Pairs<T>::NP / 2; ++q) {
        const float4 f = s_gamma[q * nvec + v];
        w[2 * q] = make_float2(f.x, f.y);
        w[2 * q + 1] = make_float2(f.z, f.w);
    }
}

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

// Sum of the `wpr` per-warp partials of this row group, identical in every thread of the group.
__device__ __forceinline__ double group_total(const double* s_red, int wpr, int lane) {
    double v = lane < wpr ? s_red[lane] : 0.0;
    return warp_sum(v);
}

// ------------------------------------------------------------------------------------------
// Forward.  y = (x*rstd)*gamma, rstd saved.  FUSE_ADD: h = x + r is formed first, written out
// and normalised instead of x.  Each thread owns vectors tig, tig+G, ... (VPT of them; FULL means
// every one of them exists, so no bounds checks) and keeps them in registers between the passes.
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

template <typename T, int VPT, bool HAS_GAMMA, bool FUSE_ADD, bool FULL>
__global__ void __launch_bounds__(1024, 1) rmsnorm_fwd_staged(const __grid_constant__ FwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    float4* s_gamma = reinterpret_cast<float4*>(smem + g.off_gamma);
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;

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
    // The first tiles are requested before gamma is staged, so that their latency overlaps it.  The thread
    // that initialised the barriers issues the copies itself (program order + the init fence suffice); the
    // others touch the barriers only after the __syncthreads below.
    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    pdl_wait();      // the inputs may be the output of the kernel before this one in the stream
    if (g.pdl_early) pdl_trigger();
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued) issue(first + issued * stride, static_cast<int>(issued));
    if (HAS_GAMMA) stage_gamma<T>(s_gamma, a.gamma, g.nvec);
    __syncthreads();

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

        // pass 1: sum of squares (each square rounded to fp32, summed in fp64); the (x+r) vectors
        // stay in registers for pass 2
        uint4 keep[VPT];
        double ss[4] = {0.0, 0.0, 0.0, 0.0};
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    uint4 raw = sx[v];
                    float2 xv[NP];
                    Pairs<T>::unpack(raw, xv);
                    if (FUSE_ADD) {
                        float2 rv[NP];
                        Pairs<T>::unpack(sr[v], rv);
#pragma unroll
                        for (int e = 0; e < NP; ++e) xv[e] = add2(xv[e], rv[e]);
                        raw = Pairs<T>::pack(xv);
                        store_vec_streaming(gh + v, raw);
                        Pairs<T>::unpack(raw, xv);  // the norm sees h as stored (bf16: after rounding)
                    }
                    keep[i] = raw;
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 q = mul2(xv[e], xv[e]);
                        ss[(2 * e) & 3] += static_cast<double>(q.x);
                        ss[(2 * e + 1) & 3] += static_cast<double>(q.y);
                    }
                }
            }
        }
        const double ssum = warp_sum((ss[0] + ss[1]) + (ss[2] + ss[3]));
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = ssum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        // every thread has its vectors in registers: the slot can be refilled right away
        if (tid == 0 && issued < my_tiles) {
            issue(first + issued * stride, slot);
            ++issued;
        }
        // a row owned by one warp needs no second step: the shuffle sum is already the row's total
        const double tot = wpr == 1 ? ssum : group_total(s_red + (k & 1) * nwarps + grp * wpr, wpr, lane);
        const float rs = rstd_from_sumsq(tot, g.hidden, a.eps);
        const float2 rs2 = splat(rs);

        // pass 2: y = (x*rstd)*gamma
        if (valid) {
            if (tig == 0) a.rstd[row] = rs;
            uint4* gy = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.y) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP];
                    Pairs<T>::unpack(keep[i], xv);
                    if (HAS_GAMMA) {
                        float2 wv[NP];
                        load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                        for (int e = 0; e < NP; ++e) xv[e] = mul2(mul2(xv[e], rs2), wv[e]);
                    } else {
#pragma unroll
                        for (int e = 0; e < NP; ++e) xv[e] = mul2(xv[e], rs2);
                    }
                    store_vec_streaming(gy + v, Pairs<T>::pack(xv));
                }
            }
        }
    }
    pdl_trigger();   // this CTA has no tiles left: the next kernel's CTAs may take the room it frees
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

// POW2: hidden is a power of two, so `/ hidden` is an exact multiplication by 2^-k (one
// instruction instead of the three of the general exact division).
// MULTI: the rows-per-warp form for short rows (see the first loop below); a separate instantiation, because
// two loop bodies in one kernel cost the main one its registers (measured: 800 bytes of spills).
template <typename T, int VPT, bool HAS_GAMMA, bool FULL, int MAXT, bool POW2, bool MULTI = false>
__global__ void __launch_bounds__(MAXT, 1) rmsnorm_bwd_staged(const __grid_constant__ BwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    constexpr int EPV = 2 * NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    float4* s_gamma = reinterpret_cast<float4*>(smem + g.off_gamma);
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;
    const bool staged_add = a.add_mode == 1;
    const DivConst2 div_h{splat(a.hidden_f), splat(a.hidden_inv)};

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
    // first tiles requested before gamma is staged (see the forward kernel)
    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    pdl_wait();      // the inputs may be the output of the kernel before this one in the stream
    if (g.pdl_early) pdl_trigger();
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued) issue(first + issued * stride, static_cast<int>(issued));
    if (HAS_GAMMA) stage_gamma<T>(s_gamma, a.gamma, g.nvec);
    __syncthreads();

    double acc[HAS_GAMMA ? VPT * EPV : 1];
#pragma unroll
    for (int i = 0; i < (HAS_GAMMA ? VPT * EPV : 1); ++i) acc[i] = 0.0;

    long long k = 0;
    bool aborted = false;
    const int RW = MULTI ? g.rows_per_warp : 1;
    if constexpr (MULTI) {
        // Short rows owned by ONE warp each (G == 32): a warp takes RW consecutive rows of the tile one after
        // the other with no block-wide step in between -- its shuffle sum is already the row's total -- so the
        // barrier, the wait and the refill are paid once per tile of nwarps * RW rows instead of once per row.
        for (; k < my_tiles; ++k) {
            const int slot = static_cast<int>(k % S);
            const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
            if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
            const long long row0 = (first + k * stride) * g.rows_per_tile + static_cast<long long>(warp) * RW;
            const unsigned char* tile_base = ring + static_cast<size_t>(slot) * g.stage_stride +
                                             static_cast<size_t>(warp) * RW * g.row_bytes;
            for (int j = 0; j < RW; ++j) {
                const long long row = row0 + j;
                if (row >= g.rows) break;
                const float rs = a.rstd[row];
                const uint4* sx = reinterpret_cast<const uint4*>(tile_base + static_cast<size_t>(j) * g.row_bytes);
                const uint4* sg = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sx) + g.tile_stride);
                const uint4* sa = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sx) + 2 * static_cast<size_t>(g.tile_stride));
                double d[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = lane + i * 32;
                    if (FULL || v < g.nvec) {
                        float2 xv[NP], gv[NP];
                        Pairs<T>::unpack(sx[v], xv);
                        Pairs<T>::unpack(sg[v], gv);
                        if (HAS_GAMMA) {
                            float2 wv[NP];
                            load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                            for (int e = 0; e < NP; ++e) gv[e] = mul2(gv[e], wv[e]);
                        }
#pragma unroll
                        for (int e = 0; e < NP; ++e) {
                            const float2 p = mul2(gv[e], xv[e]);
                            d[(2 * e) & 3] += static_cast<double>(p.x);
                            d[(2 * e + 1) & 3] += static_cast<double>(p.y);
                        }
                    }
                }
                const float dot = static_cast<float>(warp_sum((d[0] + d[1]) + (d[2] + d[3])));
                const float2 dot2 = splat(dot), rs2 = splat(rs), r22 = splat(mul_rn(rs, rs));
                uint4* gdx = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.dx) + row * g.row_bytes);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = lane + i * 32;
                    if (FULL || v < g.nvec) {
                        float2 xv[NP], gv[NP], ov[NP], wv[NP];
                        Pairs<T>::unpack(sx[v], xv);
                        Pairs<T>::unpack(sg[v], gv);
                        if (HAS_GAMMA) load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                        for (int e = 0; e < NP; ++e) {
                            const float2 dy = HAS_GAMMA ? mul2(gv[e], wv[e]) : gv[e];
                            float2 t = mul2(xv[e], r22);
                            t = mul2(t, dot2);
                            t = POW2 ? mul2(t, div_h.dinv) : div_h(t);
                            t = sub2_after_mul(dy, t);
                            ov[e] = mul2(rs2, t);
                            if (HAS_GAMMA) {
                                const float2 q = mul2(gv[e], mul2(xv[e], rs2));
                                acc[i * EPV + 2 * e] += static_cast<double>(q.x);
                                acc[i * EPV + 2 * e + 1] += static_cast<double>(q.y);
                            }
                        }
                        if (a.add_mode == 2) {
#pragma unroll
                            for (int e = 0; e < NP; ++e) ov[e] = add2_after_mul(ov[e], gv[e]);
                        } else if (staged_add) {
                            float2 av[NP];
                            Pairs<T>::unpack(sa[v], av);
#pragma unroll
                            for (int e = 0; e < NP; ++e) ov[e] = add2_after_mul(ov[e], av[e]);
                        }
                        store_vec_streaming(gdx + v, Pairs<T>::pack(ov));
                    }
                }
            }
            __syncthreads();   // every warp is done with the slot
            if (*s_abort) { aborted = true; break; }
            if (tid == 0 && issued < my_tiles) {
                issue(first + issued * stride, slot);
                ++issued;
            }
        }
    }
    for (; !MULTI && k < my_tiles; ++k) {
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
        // (four independent fp64 chains: a dependent DADD chain of 16 would cost more than the loads)
        double d[4] = {0.0, 0.0, 0.0, 0.0};
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP], gv[NP];
                    Pairs<T>::unpack(sx[v], xv);
                    Pairs<T>::unpack(sg[v], gv);
                    if (HAS_GAMMA) {
                        float2 wv[NP];
                        load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                        for (int e = 0; e < NP; ++e) gv[e] = mul2(gv[e], wv[e]);
                    }
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 p = mul2(gv[e], xv[e]);
                        d[(2 * e) & 3] += static_cast<double>(p.x);
                        d[(2 * e + 1) & 3] += static_cast<double>(p.y);
                    }
                }
            }
        }
        const double dsum = warp_sum((d[0] + d[1]) + (d[2] + d[3]));
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = dsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        // all threads are past pass 2 of the previous tile: its slot can be refilled
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue(first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        const float dot = static_cast<float>(wpr == 1 ? dsum : group_total(s_red + (k & 1) * nwarps + grp * wpr, wpr, lane));
        const float2 dot2 = splat(dot), rs2 = splat(rs), r22 = splat(mul_rn(rs, rs));

        // pass 2: dx and the dgamma terms
        if (valid) {
            uint4* gdx = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.dx) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
                    float2 xv[NP], gv[NP], ov[NP], wv[NP];
                    Pairs<T>::unpack(sx[v], xv);
                    Pairs<T>::unpack(sg[v], gv);
                    if (HAS_GAMMA) load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 dy = HAS_GAMMA ? mul2(gv[e], wv[e]) : gv[e];
                        float2 t = mul2(xv[e], r22);
                        t = mul2(t, dot2);
                        t = POW2 ? mul2(t, div_h.dinv) : div_h(t);
                        t = sub2_after_mul(dy, t);
                        ov[e] = mul2(rs2, t);
                        if (HAS_GAMMA) {
                            const float2 q = mul2(gv[e], mul2(xv[e], rs2));
                            acc[i * EPV + 2 * e] += static_cast<double>(q.x);
                            acc[i * EPV + 2 * e + 1] += static_cast<double>(q.y);
                        }
                    }
                    if (a.add_mode == 2) {
#pragma unroll
                        for (int e = 0; e < NP; ++e) ov[e] = add2_after_mul(ov[e], gv[e]);
                    } else if (staged_add) {
                        float2 av[NP];
                        Pairs<T>::unpack(sa[v], av);
#pragma unroll
                        for (int e = 0; e < NP; ++e) ov[e] = add2_after_mul(ov[e], av[e]);
                    }
                    store_vec_streaming(gdx + v, Pairs<T>::pack(ov));
                }
            }
        }
    }
    pdl_trigger();   // this CTA has no tiles left: the next kernel's CTAs may take the room it frees
    if (aborted) {
        if (tid == 0) drain_after_abort(g, s_full, k, issued);
        return;
    }

    if (HAS_GAMMA && a.partials != nullptr) {
        double* prow = a.partials + static_cast<size_t>(blockIdx.x) * g.hidden;
        const int ngroups = blockDim.x / G;   // row groups of this CTA, each with its own column sums
        if (ngroups == 1) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = tig + i * G;
                if (FULL || v < g.nvec) {
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
            for (int gi = 0; gi < ngroups; ++gi) {
                if (grp == gi) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        const int v = tig + i * G;
                        if (FULL || v < g.nvec) {
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

// Self-test of the failure path: one CTA waits on a barrier that nothing will ever complete, with a
// caller-chosen poll limit, and then does exactly what the real kernels do when a wait runs out:
// raise the status word and return.  Bounded by poll_limit * kWaitSuspendNs; nothing hangs or traps.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int poll_limit, int* polls_done) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        int i = 0;
        bool done = false;
        for (; i < poll_limit && !done; ++i) done = mbar_try_wait(&bar, 0);
        if (polls_done) *polls_done = i;
        if (!done) atomicExch(&g_device_status, 6 /* AGB_ERR_TIMEOUT */);
    }
}

// Stage 2: dgamma[c] = sum over partial rows p = 0..P-1, fixed order, fp64.
// Block (kReduceCols, kReduceLanes): thread (cx, py) sums rows py, py+32, ... of column c with four
// independent chains, then the 32 sub-sums are added in py order.  16 columns (128 bytes of every partial
// row) per CTA make hidden/16 CTAs: more than one per SM from hidden = 4096 on, and the partial rows come
// out of L2 in a few microseconds.
constexpr int kReduceCols = 16, kReduceLanes = 32;
// out_mode 0: fp32 store, 1: fp32 accumulate, 2: fp64 store, 3: fp64 accumulate.
__global__ void __launch_bounds__(512) dgamma_reduce_kernel(const double* __restrict__ partials, int P, int hidden,
                                                            void* out, int out_mode) {
    __shared__ double s[kReduceLanes][kReduceCols + 1];
    const int cx = threadIdx.x, py = threadIdx.y;
    const int c = blockIdx.x * kReduceCols + cx;
    pdl_wait();   // the partial rows are written by the backward kernel launched just before
    pdl_trigger();
    double v0 = 0.0, v1 = 0.0, v2 = 0.0, v3 = 0.0;
    if (c < hidden) {
        int p = py;
        for (; p + 3 * kReduceLanes < P; p += 4 * kReduceLanes) {
            v0 += partials[static_cast<size_t>(p) * hidden + c];
            v1 += partials[static_cast<size_t>(p + kReduceLanes) * hidden + c];
            v2 += partials[static_cast<size_t>(p + 2 * kReduceLanes) * hidden + c];
            v3 += partials[static_cast<size_t>(p + 3 * kReduceLanes) * hidden + c];
        }
        for (; p < P; p += kReduceLanes) v0 += partials[static_cast<size_t>(p) * hidden + c];
    }
    s[py][cx] = (v0 + v1) + (v2 + v3);
    __syncthreads();
    if (py == 0 && c < hidden) {
        double t = s[0][cx];
#pragma unroll
        for (int j = 1; j < kReduceLanes; ++j) t += s[j][cx];
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

// FAST (16-bit I/O): fp32 sums and fused multiply-adds, ty = (rstd*t + x*k)*gamma [+ x*rstd*tgamma] with
// k = -rstd^3 * sum(t*x) / H per row -- the same algebra as the fp32-accumulating backward (rmsnorm_fast.cuh).
template <typename T, bool FAST = false>
__global__ void __launch_bounds__(1024, 1) rmsnorm_jvp_staged(const __grid_constant__ JvpArgs a) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    float4* s_gamma = reinterpret_cast<float4*>(smem + g.off_gamma);
    float4* s_tgamma = reinterpret_cast<float4*>(smem + g.off_gamma2);
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
    if (has_gamma) stage_gamma<T>(s_gamma, a.gamma, g.nvec);
    if (has_tgamma) stage_gamma<T>(s_tgamma, a.tgamma, g.nvec);
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
        const float2 rs2 = splat(rs);
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sx = reinterpret_cast<const uint4*>(base);
        const uint4* st = reinterpret_cast<const uint4*>(base + g.tile_stride);

        double d0 = 0.0, d1 = 0.0;
        float2 f0 = make_float2(0.f, 0.f), f1 = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float2 xv[NP], tv[NP];
                Pairs<T>::unpack(sx[v], xv);
                Pairs<T>::unpack(st[v], tv);
#pragma unroll
                for (int e = 0; e < NP; ++e) {
                    if constexpr (FAST) {
                        if (e & 1) f1 = __ffma2_rn(tv[e], xv[e], f1);
                        else f0 = __ffma2_rn(tv[e], xv[e], f0);
                    } else {
                        const float2 p = mul2(tv[e], mul2(xv[e], rs2));
                        d0 += static_cast<double>(p.x);
                        d1 += static_cast<double>(p.y);
                    }
                }
            }
        }
        // (FAST: the per-lane fp32 sums, widened only for the shared reduction path; rstd is applied after the sum)
        const double dsum = FAST ? warp_sum(static_cast<double>((f0.x + f0.y) + (f1.x + f1.y))) : warp_sum(d0 + d1);
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = dsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue_tile<2>(g, ring, s_full, src2, first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        const float dot = static_cast<float>(wpr == 1 ? dsum : group_total(s_red + (k & 1) * nwarps + grp * wpr, wpr, lane));
        const float2 dot2 = splat(dot), c2 = splat(__fdiv_rn(rs, a.hidden_f));
        const float2 k2 = splat(-(rs * rs) * (rs * dot) / a.hidden_f);   // FAST (dot = sum(t*x) there)

        if (valid) {
            uint4* gout = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.ty) + row * g.row_bytes);
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float2 xv[NP], tv[NP], wv[NP], twv[NP];
                Pairs<T>::unpack(sx[v], xv);
                Pairs<T>::unpack(st[v], tv);
                if (has_gamma) load_gamma<T>(s_gamma, g.nvec, v, wv);
                if (has_tgamma) load_gamma<T>(s_tgamma, g.nvec, v, twv);
#pragma unroll
                for (int e = 0; e < NP; ++e) {
                    float2 o;
                    if constexpr (FAST) {
                        o = __ffma2_rn(tv[e], rs2, mul2(xv[e], k2));
                        if (has_gamma) {
                            o = mul2(o, wv[e]);
                            if (has_tgamma) o = __ffma2_rn(mul2(xv[e], rs2), twv[e], o);
                        }
                    } else {
                        const float2 yh = mul2(xv[e], rs2);
                        const float2 q = mul2(tv[e], rs2);
                        float2 p = mul2(yh, dot2);
                        p = mul2(p, c2);
                        o = sub2_after_mul(q, p);
                        if (has_gamma) {
                            o = mul2(o, wv[e]);
                            if (has_tgamma) o = add2_after_mul(o, mul2(yh, twv[e]));
                        }
                    }
                    xv[e] = o;
                }
                store_vec_streaming(gout + v, Pairs<T>::pack(xv));
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

}  // namespace agb
