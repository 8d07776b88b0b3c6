// rmsnorm_fast.cuh -- RMSNorm forward / VJP for 16-bit I/O with fp32 accumulation.
//
// Same pipeline as rmsnorm_staged.cuh (persistent CTAs, bulk-copy ring signalled on mbarriers, a
// group of threads per row, 16-byte conflict-free shared-memory reads, streaming 16-byte stores;
// only the assignment of a row's vectors to the group's threads differs, see v0 below),
// different arithmetic: every sum is carried in fp32 (packed two-lane FMA chains, fp32 warp
// shuffles), multiply-adds are fused, and no value passes through fp64 until the per-CTA dgamma
// partial row is written.  That is what "bf16 I/O with fp32 accumulation" asks for, and it is what
// takes these kernels from 0.6-0.8 to 0.9-1.0 of the copy bandwidth: the strictly rounded backward
// spends two fp32->fp64 conversions and two fp64 additions per element (23 instructions per element,
// the conversion unit alone 40 % busy), this one 13, the forward 11, with no fp64 at all.
//
// Results differ from the strictly rounded kernels in the last bits of fp32 intermediates (fused
// multiply-adds, fp32 sums); outputs are rounded to the 16-bit type once.  The fp32 kernels of
// rmsnorm_staged.cuh stay as they are: their bit-identity with the reference's composition is what
// pins parity.  agb_set_option("bf16_strict", 1) selects them for 16-bit I/O too.
//
// Backward algebra (one multiply-add per output element and one per dgamma term):
//   gr = gy*rstd ;  dx = gr*gamma + x*kk,  kk = -rstd^3 * dot / H,  dot = sum_j gy_j*gamma_j*x_j
//   dgamma_j += gr_j * x_j
#pragma once
#include "rmsnorm_staged.cuh"

namespace agb {

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

__device__ __forceinline__ float warp_sum_f32(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Sum of the `wpr` per-warp partials of a row group, identical in every thread of the group.
__device__ __forceinline__ float group_total_f32(const float* s_red, int wpr, int lane) {
    return warp_sum_f32(lane < wpr ? s_red[lane] : 0.0f);
}
__device__ __forceinline__ float rstd_from_sumsq_f32(float sumsq, float hidden_inv, float eps) {
    return __fdiv_rn(1.0f, __fsqrt_rn(fmaf(sumsq, hidden_inv, eps)));
}

// Slot release by count: every warp calls this when it has read all it needs from ring slot `slot` (tile k of
// the CTA); the LAST warp to arrive refills the slot with tile k + stages.  Words behind the abort flag:
// flag[1] = tiles issued so far (for the drain after an abort), flag[4 + slot] = arrivals.
template <typename Issue>
__device__ __forceinline__ void release_slot(volatile int* flag, int slot, int nwarps, long long k, int stages,
                                             long long my_tiles, int lane, Issue&& issue) {
    __syncwarp();   // this warp's shared-memory reads of the slot are complete (their values were consumed)
    if (lane == 0) {
        int* cnt = const_cast<int*>(flag) + 4 + slot;
        __threadfence_block();
        if (atomicAdd(cnt, 1) == nwarps - 1) {
            __threadfence_block();
            *cnt = 0;   // nobody counts on this slot again before the refill below has been consumed
            if (k + stages < my_tiles) {
                issue(k + stages, slot);
                atomicMax(const_cast<int*>(flag) + 1, static_cast<int>(k + stages + 1));
            }
        }
    }
}
// After an abort in a kernel that releases by count: wait (bounded) for the last `stages` tiles issued.
__device__ __forceinline__ void drain_counted(const PipeGeom& g, uint64_t* full, volatile int* flag) {
    const long long issued = flag[1];
    drain_after_abort(g, full, issued > g.stages ? issued - g.stages : 0, issued);
}

// ------------------------------------------------------------------------------------------
// Forward.  Arguments as rmsnorm_fwd_staged (FwdArgs); hidden_inv = 1/H.
// FREE (rows that one warp owns): no block-wide barrier in the tile loop at all -- a warp needs nothing from
// the others, takes its row into registers, counts itself out of the slot and goes on; warps drift apart by
// up to the ring's depth, which hides the fixed latencies of a row (wait, reduction, statistics) that a
// barrier per tile would line up in every warp at once.
// ------------------------------------------------------------------------------------------
template <typename T, int VPT, bool HAS_GAMMA, bool FUSE_ADD, bool FULL, bool FREE = false>
__global__ void __launch_bounds__(1024, 1) rmsnorm_fwd_fast(const __grid_constant__ FwdArgs a, const float hidden_inv) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    float4* s_gamma = reinterpret_cast<float4*>(smem + g.off_gamma);
    float* s_red = reinterpret_cast<float*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    // Vector i of this thread: each warp of a row group owns VPT*32 consecutive vectors, lane-interleaved, so the
    // stride between a thread's vectors is a compile-time 512 bytes (immediate offsets, no address arithmetic
    // per access) and a warp's 16-byte accesses stay consecutive (conflict-free, coalesced).
    const int v0 = (tig >> 5) * (VPT * 32) + lane;
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
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&s_full[s], 1); s_abort[4 + s] = 0; }
        *s_abort = 0;
        mbar_fence_init();
    }
    pdl_wait();      // the inputs may be the output of the kernel before this one in the stream
    if (g.pdl_early) pdl_trigger();
    if (tid == 0) {
        for (; issued < my_tiles && issued < S; ++issued) issue(first + issued * stride, static_cast<int>(issued));
        s_abort[1] = static_cast<int>(issued);
    }
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
        if (FREE && *s_abort) break;

        const uint4* sx = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(slot) * g.stage_stride +
                                                         static_cast<size_t>(grp) * g.row_bytes);
        const uint4* sr = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sx) + g.tile_stride);
        uint4* gh = FUSE_ADD ? reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.h) + row * g.row_bytes) : nullptr;

        uint4 keep[VPT];
        float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = v0 + i * 32;
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
                        Pairs<T>::unpack(raw, xv);  // the norm sees h as stored
                    }
                    keep[i] = raw;
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        if (e & 1) s1 = fma2(xv[e], xv[e], s1);
                        else s0 = fma2(xv[e], xv[e], s0);
                    }
                }
            }
        }
        const float ssum = warp_sum_f32((s0.x + s0.y) + (s1.x + s1.y));
        float tot;
        if constexpr (FREE) {
            // this warp holds its row in registers: it is done with the slot
            release_slot(s_abort, slot, nwarps, k, S, my_tiles, lane,
                         [&](long long kk, int sl) { issue(first + kk * stride, sl); });
            tot = ssum;
        } else {
            if (wpr > 1 && lane == 0) s_red[(k & 1) * nwarps + warp] = ssum;
            __syncthreads();
            if (*s_abort) { aborted = true; break; }
            if (tid == 0 && issued < my_tiles) {   // every thread holds its vectors in registers: refill now
                issue(first + issued * stride, slot);
                ++issued;
            }
            tot = wpr == 1 ? ssum : group_total_f32(s_red + (k & 1) * nwarps + grp * wpr, wpr, lane);
        }
        const float rs = rstd_from_sumsq_f32(tot, hidden_inv, a.eps);
        const float2 rs2 = splat(rs);

        if (valid) {
            if (tig == 0) a.rstd[row] = rs;
            uint4* gy = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.y) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = v0 + i * 32;
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
    if constexpr (FREE) {
        __syncthreads();
        if (*s_abort && tid == 0) drain_counted(g, s_full, s_abort);
    } else {
        if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
    }
}

// ------------------------------------------------------------------------------------------
// Backward.  Arguments as rmsnorm_bwd_staged (BwdArgs).  KEEP: x (unpacked) and gy (as loaded) stay in
// registers between the two passes (fewer instructions and shared-memory reads, ~110 registers);
// otherwise the tile is read and unpacked again (~80 registers, more resident threads).
// The per-column dgamma sums are fp32 registers, one chain per thread over the rows it owns; at the
// end the row groups of the CTA are added in group order in fp64 and the CTA writes one fp64
// partial row, exactly the layout dgamma_reduce_kernel expects.
// ------------------------------------------------------------------------------------------
template <typename T, int VPT, bool HAS_GAMMA, bool FULL, int MAXT, bool KEEP, int REL = 0>
__global__ void __launch_bounds__(MAXT, 1) rmsnorm_bwd_fast(const __grid_constant__ BwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    constexpr int EPV = 2 * NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    float4* s_gamma = reinterpret_cast<float4*>(smem + g.off_gamma);
    float* s_red = reinterpret_cast<float*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    // Vector i of this thread: each warp of a row group owns VPT*32 consecutive vectors, lane-interleaved, so the
    // stride between a thread's vectors is a compile-time 512 bytes (immediate offsets, no address arithmetic
    // per access) and a warp's 16-byte accesses stay consecutive (conflict-free, coalesced).
    const int v0 = (tig >> 5) * (VPT * 32) + lane;
    const int S = g.stages;
    const bool staged_add = a.add_mode == 1;
    // Slot release.  REL 0: thread 0 refills the slot of tile k-1 after the block-wide barrier in the middle of
    // tile k.  REL 1 (EARLY): every warp counts itself out of a slot when its pass 2 is done and the LAST one
    // refills the slot at once, so a copy has a whole tile's time to arrive instead of half, and rstd is fetched
    // one tile ahead.  Measured at 65536 x 8192 bf16 (one row per tile, two CTAs per SM): 6053 against 5735 GB/s;
    // with three rows per tile (4096 columns) it is 4 % behind, and its extra state spills in the 32-element
    // variants, so it is a template parameter used where the plan asks for it.  (A third form for rows that one
    // warp owns, release by count and no block-wide barrier at all as in the forward, measured 5-8 % BEHIND the
    // barrier form here -- 4941 against 5192 GB/s at 1000 columns, 4606 against 4969 at 1024 -- and was dropped.)
    static_assert(REL == 0 || REL == 1, "late or early refill");

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
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&s_full[s], 1); s_abort[4 + s] = 0; }
        *s_abort = 0;
        mbar_fence_init();
    }
    pdl_wait();      // the inputs may be the output of the kernel before this one in the stream
    if (g.pdl_early) pdl_trigger();
    if (tid == 0) {
        for (; issued < my_tiles && issued < S; ++issued) issue(first + issued * stride, static_cast<int>(issued));
        s_abort[1] = static_cast<int>(issued);
    }
    if (HAS_GAMMA) stage_gamma<T>(s_gamma, a.gamma, g.nvec);
    __syncthreads();

    float2 acc[HAS_GAMMA ? VPT * NP : 1];
#pragma unroll
    for (int i = 0; i < (HAS_GAMMA ? VPT * NP : 1); ++i) acc[i] = make_float2(0.f, 0.f);

    long long k = 0;
    bool aborted = false;
    float rs_ahead = 0.0f;
    if constexpr (REL != 0) {
        const long long row0 = first * g.rows_per_tile + grp;
        if (my_tiles > 0 && row0 < g.rows) rs_ahead = a.rstd[row0];
    }
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        float rs;
        if constexpr (REL != 0) {
            rs = rs_ahead;
            const long long nrow = row + stride * g.rows_per_tile;
            rs_ahead = (k + 1 < my_tiles && nrow < g.rows) ? a.rstd[nrow] : 0.0f;
        } else {
            rs = valid ? a.rstd[row] : 0.0f;
        }
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;

        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sx = reinterpret_cast<const uint4*>(base);
        const uint4* sg = reinterpret_cast<const uint4*>(base + g.tile_stride);
        const uint4* sa = reinterpret_cast<const uint4*>(base + 2 * static_cast<size_t>(g.tile_stride));

        // pass 1: dot = sum(gy*gamma*x), four independent fp32 chains per thread
        float2 kx[KEEP ? VPT * NP : 1];
        uint4 kg[KEEP ? VPT : 1];
        float2 d0 = make_float2(0.f, 0.f), d1 = make_float2(0.f, 0.f);
        if (valid) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = v0 + i * 32;
                if (FULL || v < g.nvec) {
                    float2 xv[NP], gv[NP];
                    const uint4 graw = sg[v];
                    Pairs<T>::unpack(sx[v], xv);
                    Pairs<T>::unpack(graw, gv);
                    if (KEEP) {
                        kg[i] = graw;
#pragma unroll
                        for (int e = 0; e < NP; ++e) kx[i * NP + e] = xv[e];
                    }
                    if (HAS_GAMMA) {
                        float2 wv[NP];
                        load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                        for (int e = 0; e < NP; ++e) gv[e] = mul2(gv[e], wv[e]);
                    }
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        if (e & 1) d1 = fma2(gv[e], xv[e], d1);
                        else d0 = fma2(gv[e], xv[e], d0);
                    }
                }
            }
        }
        const float dsum = warp_sum_f32((d0.x + d0.y) + (d1.x + d1.y));
        if (wpr > 1 && lane == 0) s_red[(k & 1) * nwarps + warp] = dsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        // all threads are past pass 2 of the previous tile: its slot can be refilled
        if (REL == 0 && tid == 0 && k >= 1 && issued < my_tiles) {
            issue(first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        const float dot = wpr == 1 ? dsum : group_total_f32(s_red + (k & 1) * nwarps + grp * wpr, wpr, lane);
        const float2 rs2 = splat(rs);
        const float2 kk2 = splat(-(rs * rs) * (rs * dot) * a.hidden_inv);

        // pass 2: dx and the dgamma terms
        if (valid) {
            uint4* gdx = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.dx) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = v0 + i * 32;
                if (FULL || v < g.nvec) {
                    float2 xv[NP], gv[NP], ov[NP], wv[NP];
                    if (KEEP) {
#pragma unroll
                        for (int e = 0; e < NP; ++e) xv[e] = kx[i * NP + e];
                        Pairs<T>::unpack(kg[i], gv);
                    } else {
                        Pairs<T>::unpack(sx[v], xv);
                        Pairs<T>::unpack(sg[v], gv);
                    }
                    if (HAS_GAMMA) load_gamma<T>(s_gamma, g.nvec, v, wv);
#pragma unroll
                    for (int e = 0; e < NP; ++e) {
                        const float2 gr = mul2(gv[e], rs2);
                        const float2 u = mul2(xv[e], kk2);
                        if (HAS_GAMMA) {
                            acc[i * NP + e] = fma2(gr, xv[e], acc[i * NP + e]);
                            ov[e] = fma2(gr, wv[e], u);
                        } else {
                            ov[e] = add2(gr, u);
                        }
                    }
                    if (a.add_mode == 2) {
#pragma unroll
                        for (int e = 0; e < NP; ++e) ov[e] = add2(ov[e], gv[e]);
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
        if constexpr (REL != 0)
            release_slot(s_abort, slot, nwarps, k, S, my_tiles, lane, [&](long long kk, int sl) { issue(first + kk * stride, sl); });
    }
    pdl_trigger();   // this CTA has no tiles left: the next kernel's CTAs may take the room it frees
    if (aborted) {
        if (tid == 0) {
            if (REL != 0) drain_counted(g, s_full, s_abort);
            else drain_after_abort(g, s_full, k, issued);
        }
        return;
    }

    if (HAS_GAMMA && a.partials != nullptr) {
        double* prow = a.partials + static_cast<size_t>(blockIdx.x) * g.hidden;
        const int ngroups = blockDim.x / G;
        if (ngroups == 1) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = v0 + i * 32;
                if (FULL || v < g.nvec) {
#pragma unroll
                    for (int e = 0; e < NP; ++e)
                        *reinterpret_cast<double2*>(prow + static_cast<size_t>(v) * EPV + 2 * e) =
                            make_double2(static_cast<double>(acc[i * NP + e].x), static_cast<double>(acc[i * NP + e].y));
                }
            }
        } else {
            // combine the row groups of this CTA in group order, in fp64, through the (now idle) ring
            __syncthreads();
            double* s_acc = reinterpret_cast<double*>(ring);
            for (int gi = 0; gi < ngroups; ++gi) {
                if (grp == gi) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        const int v = v0 + i * 32;
                        if (FULL || v < g.nvec) {
#pragma unroll
                            for (int e = 0; e < NP; ++e) {
                                const int c = v * EPV + 2 * e;
                                const double ax = static_cast<double>(acc[i * NP + e].x), ay = static_cast<double>(acc[i * NP + e].y);
                                s_acc[c] = gi == 0 ? ax : s_acc[c] + ax;
                                s_acc[c + 1] = gi == 0 ? ay : s_acc[c + 1] + ay;
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

}  // namespace agb
