// agb_peer_device.cuh -- device side of the cross-process dgamma exchange (host side: agb_peer.cuh;
// block layout and protocol are described there).
#pragma once
#include "agb/agb_shard.h"
#include "agb_device.cuh"
#include "rmsnorm_staged.cuh"   // kReduceCols / kReduceLanes: the column reduction's block shape

namespace agb {

constexpr int kPeerHeaderBytes = 128;
constexpr int kPeerCounterOffset = 32;   // an unsigned int used by the fused reduce kernel to find its last CTA
constexpr int kPeerTimeoutsOffset = 36;  // an unsigned int: CTAs of the current fused reduce whose ack wait ran out
// The bound of every wait below (polls; each sleeps up to 2 us) is a kernel argument taken from the
// process-wide "peer_poll_limit" option at launch, so that it holds on every device a process drives.

struct PeerBlocks {
    unsigned char* base[AGB_SHARD_MAX];
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Polls with RELAXED loads and a growing sleep (0.2 -> 2 us), and pays for the acquire once, with a fence,
// when the value has arrived.  A rank that runs ahead of the others waits here for most of a step, beside
// the CTAs of the next forward and backward: an acquire load every half microsecond (each one invalidates
// the SM's L1) slowed the co-resident forward CTA, and with it the whole statically partitioned kernel,
// by tens of microseconds.
__device__ __forceinline__ bool poll_until_at_least(const unsigned long long* p, unsigned long long want, int limit) {
    unsigned int ns = 200;
    for (int i = 0; i < limit; ++i) {
        if (ld_relaxed_sys(p) >= want) {
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            return true;
        }
        __nanosleep(ns);
        if (ns < 2000) ns *= 2;
    }
    return false;
}
__device__ __forceinline__ unsigned long long* peer_ready(unsigned char* base, int b) {
    return reinterpret_cast<unsigned long long*>(base) + b;
}
__device__ __forceinline__ unsigned long long* peer_ack(unsigned char* base, int b) {
    return reinterpret_cast<unsigned long long*>(base) + 2 + b;
}

// One warp: lane j waits until rank j has acknowledged step `need` on buffer b.
__global__ void peer_wait_ack_kernel(PeerBlocks blk, int n, int b, unsigned long long need, int poll_limit) {
    const int j = threadIdx.x;
    if (j < n && !poll_until_at_least(peer_ack(blk.base[j], b), need, poll_limit)) atomicExch(&g_device_status, AGB_ERR_TIMEOUT);
}

// The sums of step t are complete in this rank's buffer b (written by earlier kernels of the same
// stream): make them visible system-wide, then publish the step number.
__global__ void peer_publish_kernel(unsigned char* own, int b, unsigned long long t) {
    __threadfence_system();
    st_release_sys(peer_ready(own, b), t);
}

// One small CTA (256 threads, few registers: it must fit beside a resident CTA of the persistent forward
// or backward kernel instead of taking an SM from it -- a 1024-thread version delayed the next forward by
// ~10 us per step): wait for every rank's publication of step t, add the sums in rank order, round
// once, acknowledge.  On a timeout nothing is written and nothing is acknowledged.
constexpr int kPeerSumThreads = 256;
__global__ void __launch_bounds__(kPeerSumThreads) peer_sum_kernel(PeerBlocks blk, int n, int self, int b,
                                                                   unsigned long long t, long long max_hidden, int hidden,
                                                                   float* __restrict__ dgamma, int accumulate,
                                                                   int poll_limit) {
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    if (threadIdx.x < n && !poll_until_at_least(peer_ready(blk.base[threadIdx.x], b), t, poll_limit)) timed_out = 1;
    __syncthreads();
    if (timed_out) {
        if (threadIdx.x == 0) atomicExch(&g_device_status, AGB_ERR_TIMEOUT);
        return;
    }
    const size_t off = kPeerHeaderBytes + static_cast<size_t>(b) * static_cast<size_t>(max_hidden) * sizeof(double);
    // two columns per thread and pass (16-byte loads) when the buffers are 16-byte aligned: max_hidden even
    const int pairs = (max_hidden % 2 == 0) ? hidden / 2 : 0;
    for (int q = threadIdx.x; q < pairs; q += blockDim.x) {
        double2 s = __ldcg(reinterpret_cast<const double2*>(blk.base[0] + off) + q);
        for (int r = 1; r < n; ++r) {
            const double2 v = __ldcg(reinterpret_cast<const double2*>(blk.base[r] + off) + q);
            s.x += v.x;
            s.y += v.y;
        }
        const float v0 = static_cast<float>(s.x), v1 = static_cast<float>(s.y);
        dgamma[2 * q] = accumulate ? add_rn(dgamma[2 * q], v0) : v0;
        dgamma[2 * q + 1] = accumulate ? add_rn(dgamma[2 * q + 1], v1) : v1;
    }
    for (int c = 2 * pairs + threadIdx.x; c < hidden; c += blockDim.x) {
        double s = __ldcg(reinterpret_cast<const double*>(blk.base[0] + off) + c);
        for (int r = 1; r < n; ++r) s += __ldcg(reinterpret_cast<const double*>(blk.base[r] + off) + c);
        const float v = static_cast<float>(s);
        dgamma[c] = accumulate ? add_rn(dgamma[c], v) : v;
    }
    __syncthreads();   // every load of this CTA has returned (its value was used above)
    if (threadIdx.x == 0) {
        __threadfence_system();
        st_release_sys(peer_ack(blk.base[self], b), t);
    }
}

// What the backward's final column reduction needs to do the exchange's bookkeeping itself: wait until
// every rank has acknowledged step need_ack (0: nothing to wait for) before it overwrites the sums, and
// publish step t once the last CTA has written its columns.
struct PeerHook {
    PeerBlocks blk;
    int n, self, b;
    unsigned long long need_ack, t;
    int poll_limit;
};

// dgamma_reduce_kernel (fp64 store form) with the wait in front and the publication behind, so that the
// exchange adds no kernel to the backward's stream.  Same summation order, same bits.
__global__ void __launch_bounds__(512) dgamma_reduce_publish_kernel(const double* __restrict__ partials, int P, int hidden,
                                                                    double* __restrict__ out, PeerHook h) {
    __shared__ double s[kReduceLanes][kReduceCols + 1];
    __shared__ int timed_out;
    const int cx = threadIdx.x, py = threadIdx.y;
    const int c = blockIdx.x * kReduceCols + cx;
    if (cx == 0 && py == 0) timed_out = 0;
    __syncthreads();
    static_assert(AGB_SHARD_MAX <= kReduceCols * kReduceLanes, "one thread per rank polls");
    const int tid = py * kReduceCols + cx;
    if (h.need_ack > 0 && tid < h.n && !poll_until_at_least(peer_ack(h.blk.base[tid], h.b), h.need_ack, h.poll_limit))
        timed_out = 1;
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
    // Every CTA polls on its own, so an acknowledgement that lands near the limit can leave some CTAs timed
    // out and others not.  A CTA whose wait ran out writes nothing (somebody may still be reading the old
    // sums) but still counts itself, so the "last CTA" counter always returns to zero; the step is published
    // only if NO CTA of this launch timed out.
    const bool expired = timed_out != 0;
    if (!expired && py == 0 && c < hidden) {
        double t = s[0][cx];
#pragma unroll
        for (int j = 1; j < kReduceLanes; ++j) t += s[j][cx];
        out[c] = t;
        __threadfence();
    }
    __syncthreads();
    if (cx == 0 && py == 0) {
        unsigned int* counter = reinterpret_cast<unsigned int*>(h.blk.base[h.self] + kPeerCounterOffset);
        unsigned int* expired_ctas = reinterpret_cast<unsigned int*>(h.blk.base[h.self] + kPeerTimeoutsOffset);
        if (expired) {
            atomicExch(&g_device_status, AGB_ERR_TIMEOUT);
            atomicAdd(expired_ctas, 1u);
            __threadfence();
        }
        if (atomicAdd(counter, 1u) == gridDim.x - 1) {   // the last CTA of this launch
            __threadfence();
            const unsigned int bad = atomicExch(expired_ctas, 0u);
            atomicExch(counter, 0u);
            if (bad == 0) {                              // every column is written: publish the step
                __threadfence_system();
                st_release_sys(peer_ready(h.blk.base[h.self], h.b), h.t);
            }
        }
    }
}

}  // namespace agb
