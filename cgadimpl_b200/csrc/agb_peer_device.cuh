// agb_peer_device.cuh -- device side of the cross-process dgamma exchange (host side: agb_peer.cuh).
#pragma once
#include "agb/agb_shard.h"
#include "agb_device.cuh"
#include "rmsnorm_staged.cuh"   // kReduceCols / kReduceLanes: the column reduction's block shape

namespace agb {

// Block layout (one block per rank, in that rank's memory; N = world size, MH = max_hidden, NB = kPeerBuffers):
//   [0, 1024)     ready[s][b]  u64, s < 16, b < NB: step whose sums rank s has STORED INTO THIS BLOCK (written by s)
//   [1024, 2048)  ack[r][b]    u64: step up to which reader r has consumed THIS rank's sums (written by r)
//   [2048, 2052)  counter      u32: the fused reduce kernel's "last CTA" ticket
//   [2052, 2056)  expired      u32: CTAs of the current fused reduce whose ack wait ran out
//   [4096, ...)   sums[s][b][MH] fp64, s < N: rank s's column sums of the step that uses buffer b = t mod NB
// NB buffers in turn: a rank may run up to NB steps ahead of the slowest reader before it has to wait, so the
// ranks are coupled over windows of NB steps instead of step by step (a GPU under its power cap does not run
// every step at the same speed, and a step-by-step lock step runs at the slowest GPU OF EACH STEP).
// Push protocol: a producer STORES its sums and its ready counter into every rank's block (plain peer stores
// over NVLink, no multicast) and a reader stores its ack into every producer's block, so every WAIT polls the
// waiting GPU's own memory and every read of sums is local; nothing but fire-and-forget stores crosses NVLink.
constexpr int kPeerBuffers = 8;
constexpr int kPeerReadyOffset = 0;
constexpr int kPeerAckOffset = 1024;
constexpr int kPeerCounterOffset = 2048;
constexpr int kPeerTimeoutsOffset = 2052;
constexpr int kPeerHeaderBytes = 4096;
static_assert(AGB_SHARD_MAX * kPeerBuffers * 8 <= 1024, "counter tables");
// The bound of every wait below (polls; each sleeps up to 2 us) is a kernel argument taken from the
// process-wide "peer_poll_limit" option at launch, so that it holds on every device a process drives.

struct PeerBlocks {
    unsigned char* base[AGB_SHARD_MAX];
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Polls with RELAXED loads and a growing sleep (0.2 -> 2 us), and pays for the acquire once, with a fence,
// when the value has arrived.  The polled word always lives in the polling GPU's own memory.
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
// ready counter of source rank s / ack counter of reader r, buffer b, in the block at `base`
__device__ __forceinline__ unsigned long long* peer_ready(unsigned char* base, int s, int b) {
    return reinterpret_cast<unsigned long long*>(base + kPeerReadyOffset) + kPeerBuffers * s + b;
}
__device__ __forceinline__ unsigned long long* peer_ack(unsigned char* base, int r, int b) {
    return reinterpret_cast<unsigned long long*>(base + kPeerAckOffset) + kPeerBuffers * r + b;
}
// where rank s's sums of buffer b live inside a block
__device__ __host__ __forceinline__ size_t peer_sums_offset(int s, int b, long long max_hidden) {
    return kPeerHeaderBytes +
           (static_cast<size_t>(s) * kPeerBuffers + static_cast<size_t>(b)) * static_cast<size_t>(max_hidden) * sizeof(double);
}

// One warp: lane r waits (in this rank's own block) until reader r has acknowledged step `need` on buffer b.
__global__ void peer_wait_ack_kernel(unsigned char* own, int n, int b, unsigned long long need, int poll_limit) {
    const int r = threadIdx.x;
    if (r < n && !poll_until_at_least(peer_ack(own, r, b), need, poll_limit)) atomicExch(&g_device_status, AGB_ERR_TIMEOUT);
}

// The sums of step t are complete in this rank's own slot of its own block (written by earlier kernels of the
// same stream): copy them into this rank's slot of every other rank's block, then store the step number
// into every block.  One CTA.
constexpr int kPeerPublishThreads = 1024;
__global__ void __launch_bounds__(kPeerPublishThreads) peer_publish_kernel(PeerBlocks blk, int n, int self, int b,
                                                                           unsigned long long t, long long max_hidden,
                                                                           int hidden) {
    const size_t off = peer_sums_offset(self, b, max_hidden);
    const double* src = reinterpret_cast<const double*>(blk.base[self] + off);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const double v = src[c];
        for (int r = 0; r < n; ++r)
            if (r != self) reinterpret_cast<double*>(blk.base[r] + off)[c] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < n) st_release_sys(peer_ready(blk.base[threadIdx.x], self, b), t);
}

// One small CTA (256 threads, few registers: it must fit beside a resident CTA of the persistent forward
// or backward kernel instead of taking an SM from it): wait, in this rank's own block, for every rank's
// publication of step t, add the sums in rank order (all local reads), round once, and store the
// acknowledgement into every producer's block.  On a timeout nothing is written and nothing is acknowledged.
constexpr int kPeerSumThreads = 256;
__global__ void __launch_bounds__(kPeerSumThreads) peer_sum_kernel(PeerBlocks blk, int n, int self, int b,
                                                                   unsigned long long t, long long max_hidden, int hidden,
                                                                   float* __restrict__ dgamma, int accumulate,
                                                                   int poll_limit) {
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    unsigned char* own = blk.base[self];
    if (threadIdx.x < n && !poll_until_at_least(peer_ready(own, threadIdx.x, b), t, poll_limit)) timed_out = 1;
    __syncthreads();
    if (timed_out) {
        if (threadIdx.x == 0) atomicExch(&g_device_status, AGB_ERR_TIMEOUT);
        return;
    }
    const size_t stride = kPeerBuffers * static_cast<size_t>(max_hidden);   // doubles between consecutive ranks' slots
    const double* base = reinterpret_cast<const double*>(own + peer_sums_offset(0, b, max_hidden));
    // two columns per thread and pass (16-byte loads) when the slots are 16-byte aligned: max_hidden even
    const int pairs = (max_hidden % 2 == 0) ? hidden / 2 : 0;
    for (int q = threadIdx.x; q < pairs; q += blockDim.x) {
        double2 s = __ldcg(reinterpret_cast<const double2*>(base) + q);
        for (int r = 1; r < n; ++r) {
            const double2 v = __ldcg(reinterpret_cast<const double2*>(base + r * stride) + q);
            s.x += v.x;
            s.y += v.y;
        }
        const float v0 = static_cast<float>(s.x), v1 = static_cast<float>(s.y);
        dgamma[2 * q] = accumulate ? add_rn(dgamma[2 * q], v0) : v0;
        dgamma[2 * q + 1] = accumulate ? add_rn(dgamma[2 * q + 1], v1) : v1;
    }
    for (int c = 2 * pairs + threadIdx.x; c < hidden; c += blockDim.x) {
        double s = __ldcg(base + c);
        for (int r = 1; r < n; ++r) s += __ldcg(base + r * stride + c);
        const float v = static_cast<float>(s);
        dgamma[c] = accumulate ? add_rn(dgamma[c], v) : v;
    }
    __syncthreads();   // every load of this CTA has returned (its value was used above)
    if (threadIdx.x < n) {
        __threadfence_system();
        st_release_sys(peer_ack(blk.base[threadIdx.x], self, b), t);   // producer threadIdx.x: your slot b here is free
    }
}

// What the backward's final column reduction needs to do the exchange's bookkeeping itself: wait until
// every reader has acknowledged step need_ack (0: nothing to wait for) before it overwrites the sums, and
// publish step t once the last CTA has stored its columns.
struct PeerHook {
    PeerBlocks blk;
    int n, self, b;
    unsigned long long need_ack, t;
    long long max_hidden;
    int poll_limit;
};

// dgamma_reduce_kernel (fp64 store form) with the wait in front and the publication behind, so that the
// exchange adds no kernel to the backward's stream.  Same summation order, same bits; every column sum is
// stored into this rank's slot of EVERY rank's block (row lane py stores to rank py).
__global__ void __launch_bounds__(512) dgamma_reduce_publish_kernel(const double* __restrict__ partials, int P, int hidden,
                                                                    PeerHook h) {
    __shared__ double s[kReduceLanes][kReduceCols + 1];
    __shared__ double total[kReduceCols];
    __shared__ int timed_out;
    const int cx = threadIdx.x, py = threadIdx.y;
    const int c = blockIdx.x * kReduceCols + cx;
    if (cx == 0 && py == 0) timed_out = 0;
    __syncthreads();
    static_assert(AGB_SHARD_MAX <= kReduceLanes, "row lane py stores to rank py");
    const int tid = py * kReduceCols + cx;
    unsigned char* own = h.blk.base[h.self];
    if (h.need_ack > 0 && tid < h.n && !poll_until_at_least(peer_ack(own, tid, h.b), h.need_ack, h.poll_limit))
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
    // out and others not.  A CTA whose wait ran out stores nothing (somebody may still be reading the old
    // sums) but still counts itself, so the "last CTA" counter always returns to zero; the step is published
    // only if NO CTA of this launch timed out.
    const bool expired = timed_out != 0;
    if (!expired && py == 0 && c < hidden) {
        double t = s[0][cx];
#pragma unroll
        for (int j = 1; j < kReduceLanes; ++j) t += s[j][cx];
        total[cx] = t;
    }
    __syncthreads();
    if (!expired && py < h.n && c < hidden)
        reinterpret_cast<double*>(h.blk.base[py] + peer_sums_offset(h.self, h.b, h.max_hidden))[c] = total[cx];
    __syncthreads();
    if (cx == 0 && py == 0) {
        // ONE system-scope fence per CTA, after the barrier: it is cumulative over the stores the barrier has
        // ordered before it (the CTA's 16 columns in every rank's block), so the count below, and the flags the
        // last CTA writes after its own fence, cannot overtake them.
        __threadfence_system();
        unsigned int* counter = reinterpret_cast<unsigned int*>(own + kPeerCounterOffset);
        unsigned int* expired_ctas = reinterpret_cast<unsigned int*>(own + kPeerTimeoutsOffset);
        if (expired) {
            atomicExch(&g_device_status, AGB_ERR_TIMEOUT);
            atomicAdd(expired_ctas, 1u);
            __threadfence();
        }
        if (atomicAdd(counter, 1u) == gridDim.x - 1) {   // the last CTA of this launch
            __threadfence();
            const unsigned int bad = atomicExch(expired_ctas, 0u);
            atomicExch(counter, 0u);
            if (bad == 0) {                              // every column is stored everywhere: publish the step
                __threadfence_system();
                for (int r = 0; r < h.n; ++r) st_release_sys(peer_ready(h.blk.base[r], h.self, h.b), h.t);
            }
        }
    }
}

}  // namespace agb
