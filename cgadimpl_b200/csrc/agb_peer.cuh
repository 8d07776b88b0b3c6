// agb_peer.cuh -- the dgamma exchange between ranks that are separate PROCESSES (one per GPU, one
// node), declared in include/agb/agb_shard.h.  Included at the end of agb_cuda.cu.
//
// Each rank owns one device block (layout in agb_peer_device.cuh): for every source rank s and buffer b a
// ready counter and an fp64 [max_hidden] slot that s STORES into, and for every reader r an ack counter that
// r stores into.  Every rank maps every other rank's block through CUDA IPC; only plain peer STORES cross
// NVLink (no multicast, no remote load).  Step t uses buffer b = t mod 8.  Rank p may overwrite its slot b in
// the blocks at step t once every reader has acknowledged step t-8 (polled in p's own block); it publishes
// by storing t into ready[p][b] of every block with release semantics; a reader polls ready[s][b] >= t for all
// s in ITS OWN block, sums the local slots in rank order, and stores its ack into every producer's block.
// All waits are bounded polls of local memory.
#pragma once
#include "agb/agb_shard.h"
#include "agb_peer_device.cuh"


struct agb_peer {
    int rank = 0, world = 1, dev = 0;
    int64_t max_hidden = 0;
    unsigned long long step = 0;    // steps completed (exchange enqueued)
    bool connected = false, acquired = false, published = false;
    bool ipc_opened[AGB_SHARD_MAX] = {};
    agb::PeerBlocks blk{};          // blk.base[rank] is this rank's own allocation
    cudaEvent_t ev_pub = nullptr;
    // agb_peer_rmsnorm_bwd_overlapped: the stream the publishing reduction of the open step was put on, and the
    // event behind the last kernel that read the caller's partial rows there
    cudaStream_t pub_stream = nullptr;
    bool pub_on_side = false, side_pending = false;
    cudaEvent_t ev_side = nullptr;
};

namespace {

size_t peer_block_bytes(int world, int64_t max_hidden) {
    return agb::peer_sums_offset(world, 0, max_hidden);
}

int peer_check(const agb_peer_t* p, bool need_connected) {
    if (!p) return fail(AGB_ERR_INVALID_ARG, "exchange is NULL");
    if (need_connected && !p->connected) return fail(AGB_ERR_INVALID_ARG, "agb_peer_connect has not been called");
    int dev = -1;
    AGB_CUDA(cudaGetDevice(&dev));
    if (dev != p->dev) return fail(AGB_ERR_INVALID_ARG, "current device %d, exchange created on %d", dev, p->dev);
    return AGB_OK;
}

}  // namespace

extern "C" {

int agb_peer_create(int rank, int world, int64_t max_hidden, agb_peer_t** out, unsigned char handle[AGB_PEER_HANDLE_BYTES]) {
    if (!out) return fail(AGB_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (world < 1 || world > AGB_SHARD_MAX || rank < 0 || rank >= world)
        return fail(AGB_ERR_INVALID_ARG, "rank %d of %d (at most %d ranks)", rank, world, AGB_SHARD_MAX);
    if (max_hidden <= 0 || max_hidden > (1LL << 30)) return fail(AGB_ERR_INVALID_ARG, "max_hidden=%lld", (long long)max_hidden);
    static_assert(sizeof(cudaIpcMemHandle_t) <= AGB_PEER_HANDLE_BYTES, "handle does not fit");
    agb_peer_t* p = new agb_peer();
    p->rank = rank;
    p->world = world;
    p->max_hidden = max_hidden;
    cudaError_t e = cudaGetDevice(&p->dev);
    void* mem = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&mem, peer_block_bytes(world, max_hidden));
    if (e == cudaSuccess) e = cudaMemset(mem, 0, peer_block_bytes(world, max_hidden));
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_pub, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_side, cudaEventDisableTiming);
    if (e == cudaSuccess && handle) {
        cudaIpcMemHandle_t h;
        memset(handle, 0, AGB_PEER_HANDLE_BYTES);
        e = cudaIpcGetMemHandle(&h, mem);
        if (e == cudaSuccess) memcpy(handle, &h, sizeof(h));
    }
    if (e != cudaSuccess) {
        if (mem) cudaFree(mem);
        if (p->ev_pub) cudaEventDestroy(p->ev_pub);
        if (p->ev_side) cudaEventDestroy(p->ev_side);
        delete p;
        return cuda_fail(e, "agb_peer_create");
    }
    p->blk.base[rank] = static_cast<unsigned char*>(mem);
    *out = p;
    return AGB_OK;
}

int agb_peer_connect(agb_peer_t* p, const unsigned char* all_handles) {
    AGB_TRY(peer_check(p, false));
    if (p->connected) return fail(AGB_ERR_INVALID_ARG, "already connected");
    if (!all_handles && p->world > 1) return fail(AGB_ERR_INVALID_ARG, "all_handles is NULL");
    for (int r = 0; r < p->world; ++r) {
        if (r == p->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, all_handles + static_cast<size_t>(r) * AGB_PEER_HANDLE_BYTES, sizeof(h));
        void* ptr = nullptr;
        AGB_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        p->blk.base[r] = static_cast<unsigned char*>(ptr);
        p->ipc_opened[r] = true;
    }
    p->connected = true;
    return AGB_OK;
}

int agb_peer_block(agb_peer_t* p, void** base) {
    if (!p || !base) return fail(AGB_ERR_INVALID_ARG, "exchange or output is NULL");
    *base = p->blk.base[p->rank];
    return AGB_OK;
}

int agb_peer_connect_local(agb_peer_t* p, void* const* bases) {
    AGB_TRY(peer_check(p, false));
    if (p->connected) return fail(AGB_ERR_INVALID_ARG, "already connected");
    if (!bases) return fail(AGB_ERR_INVALID_ARG, "bases is NULL");
    for (int r = 0; r < p->world; ++r) {
        if (r == p->rank) continue;
        if (!bases[r]) return fail(AGB_ERR_INVALID_ARG, "bases[%d] is NULL", r);
        p->blk.base[r] = static_cast<unsigned char*>(bases[r]);
    }
    p->connected = true;
    return AGB_OK;
}

int agb_peer_acquire(agb_peer_t* p, agb_stream_t stream, double** sums) {
    AGB_TRY(peer_check(p, true));
    if (!sums) return fail(AGB_ERR_INVALID_ARG, "sums is NULL");
    if (p->acquired) return fail(AGB_ERR_INVALID_ARG, "agb_peer_acquire called twice without agb_peer_sum in between");
    const unsigned long long t = p->step + 1;
    const int b = static_cast<int>(t % agb::kPeerBuffers);
    if (p->world > 1 && t > agb::kPeerBuffers) {   // everybody must have read what this rank wrote into buffer b kPeerBuffers steps ago
        agb::peer_wait_ack_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p->blk.base[p->rank], p->world, b, t - agb::kPeerBuffers,
                                                                                  peer_poll_limit());
        AGB_TRY(after_launch("peer_wait_ack"));
    }
    *sums = reinterpret_cast<double*>(p->blk.base[p->rank] + agb::peer_sums_offset(p->rank, b, p->max_hidden));
    p->acquired = true;
    p->published = false;
    return AGB_OK;
}

int agb_peer_rmsnorm_bwd(agb_peer_t* p, const void* x, const void* gamma, const float* rstd, const void* gy,
                         const void* dx_add, void* dx, void* workspace, size_t workspace_bytes, int64_t rows,
                         int64_t hidden, int dtype, agb_stream_t stream) {
    AGB_TRY(peer_check(p, true));
    if (p->acquired) return fail(AGB_ERR_INVALID_ARG, "a step is already open (agb_peer_acquire without agb_peer_sum)");
    if (!gamma) return fail(AGB_ERR_INVALID_ARG, "gamma is NULL: without gamma there is no dgamma to exchange");
    if (hidden <= 0 || hidden > p->max_hidden)
        return fail(AGB_ERR_WORKSPACE, "hidden %lld outside (0, max_hidden %lld]", (long long)hidden, (long long)p->max_hidden);
    if (p->side_pending && rows > 0) {
        // an earlier agb_peer_rmsnorm_bwd_overlapped may still be reading the partial rows on its side stream
        AGB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), p->ev_side, 0));
        p->side_pending = false;
    }
    if (rows == 0) {   // no reduction kernel runs for an empty shard: the plain sequence
        double* sums = nullptr;
        AGB_TRY(agb_peer_acquire(p, stream, &sums));
        AGB_TRY(agb_rmsnorm_bwd(x, gamma, rstd, gy, dx_add, dx, sums, AGB_F64, 0, workspace, workspace_bytes, rows, hidden,
                                dtype, stream));
        return agb_peer_publish(p, stream);
    }
    const unsigned long long t = p->step + 1;
    const int b = static_cast<int>(t % agb::kPeerBuffers);
    agb::PeerHook hook{p->blk, p->world, p->rank, b, (p->world > 1 && t > agb::kPeerBuffers) ? t - agb::kPeerBuffers : 0ull, t,
                       static_cast<long long>(p->max_hidden), peer_poll_limit()};
    double* sums = reinterpret_cast<double*>(p->blk.base[p->rank] + agb::peer_sums_offset(p->rank, b, p->max_hidden));
    t_reduce_hook = &hook;
    t_reduce_hook_used = false;
    const int st = agb_rmsnorm_bwd(x, gamma, rstd, gy, dx_add, dx, sums, AGB_F64, 0, workspace, workspace_bytes, rows, hidden,
                                   dtype, stream);
    t_reduce_hook = nullptr;
    if (st != AGB_OK) return st;
    if (!t_reduce_hook_used) return fail(AGB_ERR_CUDA, "internal: the backward did not run its column reduction");
    p->acquired = true;
    p->published = true;
    return AGB_OK;
}

// The same step with the column reduction, and with it the stores into the peers' blocks and their system-scope
// fences, on `side_stream`: `stream` carries only the backward kernel, so the next forward does not wait for
// the publication (among eight ranks that wait is about 40 us of a 0.9 ms step).  The partial rows in
// `workspace` are read on the side stream; the next call makes `stream` wait for that reader before its
// backward overwrites them.  agb_peer_exchange must then be given the same side stream.
int agb_peer_rmsnorm_bwd_overlapped(agb_peer_t* p, const void* x, const void* gamma, const float* rstd, const void* gy,
                                    const void* dx_add, void* dx, void* workspace, size_t workspace_bytes, int64_t rows,
                                    int64_t hidden, int dtype, agb_stream_t stream, agb_stream_t side_stream) {
    if (rows == 0 || side_stream == stream)
        return agb_peer_rmsnorm_bwd(p, x, gamma, rstd, gy, dx_add, dx, workspace, workspace_bytes, rows, hidden, dtype, stream);
    AGB_TRY(peer_check(p, true));
    if (p->acquired) return fail(AGB_ERR_INVALID_ARG, "a step is already open (agb_peer_acquire without agb_peer_sum)");
    if (!gamma) return fail(AGB_ERR_INVALID_ARG, "gamma is NULL: without gamma there is no dgamma to exchange");
    if (hidden <= 0 || hidden > p->max_hidden)
        return fail(AGB_ERR_WORKSPACE, "hidden %lld outside (0, max_hidden %lld]", (long long)hidden, (long long)p->max_hidden);
    cudaStream_t st = static_cast<cudaStream_t>(stream), sd = static_cast<cudaStream_t>(side_stream);
    if (p->side_pending) AGB_CUDA(cudaStreamWaitEvent(st, p->ev_side, 0));   // the last reader of the partial rows
    int P = 0;
    AGB_TRY(agb_rmsnorm_bwd_partials(x, gamma, rstd, gy, dx_add, dx, workspace, workspace_bytes, rows, hidden, dtype, stream, &P));
    AGB_CUDA(cudaEventRecord(p->ev_pub, st));
    AGB_CUDA(cudaStreamWaitEvent(sd, p->ev_pub, 0));
    const unsigned long long t = p->step + 1;
    const int b = static_cast<int>(t % agb::kPeerBuffers);
    agb::PeerHook hook{p->blk, p->world, p->rank, b, (p->world > 1 && t > agb::kPeerBuffers) ? t - agb::kPeerBuffers : 0ull, t,
                       static_cast<long long>(p->max_hidden), peer_poll_limit()};
    double* sums = reinterpret_cast<double*>(p->blk.base[p->rank] + agb::peer_sums_offset(p->rank, b, p->max_hidden));
    t_reduce_hook = &hook;
    t_reduce_hook_used = false;
    const int rc = agb_dgamma_reduce(workspace, P, hidden, sums, AGB_F64, 0, side_stream);
    t_reduce_hook = nullptr;
    if (rc != AGB_OK) return rc;
    if (!t_reduce_hook_used) return fail(AGB_ERR_CUDA, "internal: the column reduction did not publish");
    AGB_CUDA(cudaEventRecord(p->ev_side, sd));
    p->side_pending = true;
    p->acquired = true;
    p->published = true;
    p->pub_on_side = true;
    p->pub_stream = sd;
    return AGB_OK;
}

int agb_peer_publish(agb_peer_t* p, agb_stream_t stream) {
    AGB_TRY(peer_check(p, true));
    if (!p->acquired || p->published) return fail(AGB_ERR_INVALID_ARG, "agb_peer_publish needs one agb_peer_acquire before it");
    const unsigned long long t = p->step + 1;
    // the whole slot is pushed: the width of the step's sums is not known here, and max_hidden doubles are 8 * max_hidden bytes
    agb::peer_publish_kernel<<<1, agb::kPeerPublishThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        p->blk, p->world, p->rank, static_cast<int>(t % agb::kPeerBuffers), t, static_cast<long long>(p->max_hidden),
        static_cast<int>(p->max_hidden));
    AGB_TRY(after_launch("peer_publish"));
    p->published = true;
    return AGB_OK;
}

int agb_peer_sum(agb_peer_t* p, float* dgamma, int64_t hidden, int accumulate, agb_stream_t stream) {
    AGB_TRY(peer_check(p, true));
    if (!p->published) return fail(AGB_ERR_INVALID_ARG, "agb_peer_sum needs agb_peer_publish before it");
    if (hidden <= 0 || hidden > p->max_hidden)
        return fail(AGB_ERR_WORKSPACE, "hidden %lld outside (0, max_hidden %lld]", (long long)hidden, (long long)p->max_hidden);
    AGB_TRY(check_ptr(dgamma, "dgamma", 4));
    const unsigned long long t = p->step + 1;
    agb::peer_sum_kernel<<<1, agb::kPeerSumThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        p->blk, p->world, p->rank, static_cast<int>(t % agb::kPeerBuffers), t, static_cast<long long>(p->max_hidden),
        static_cast<int>(hidden), dgamma, accumulate, peer_poll_limit());
    AGB_TRY(after_launch("peer_sum"));
    p->step = t;
    p->acquired = p->published = false;
    return AGB_OK;
}

int agb_peer_exchange(agb_peer_t* p, float* dgamma, int64_t hidden, int accumulate, agb_stream_t stream,
                      agb_stream_t sum_stream) {
    if (!p || !p->published) AGB_TRY(agb_peer_publish(p, stream));   // (agb_peer_rmsnorm_bwd has published already)
    if (p->pub_on_side) {
        // the publishing reduction already runs on a side stream: the sum follows it there, no event needed
        p->pub_on_side = false;
        if (static_cast<cudaStream_t>(sum_stream) != p->pub_stream)
            return fail(AGB_ERR_INVALID_ARG, "agb_peer_exchange: sum_stream must be the side stream given to agb_peer_rmsnorm_bwd_overlapped");
        return agb_peer_sum(p, dgamma, hidden, accumulate, sum_stream);
    }
    if (sum_stream != stream) {
        AGB_CUDA(cudaEventRecord(p->ev_pub, static_cast<cudaStream_t>(stream)));
        AGB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(sum_stream), p->ev_pub, 0));
    }
    return agb_peer_sum(p, dgamma, hidden, accumulate, sum_stream);
}

int agb_peer_disconnect(agb_peer_t* p) {
    if (!p) return AGB_OK;
    DeviceRestore restore;
    AGB_CUDA(cudaSetDevice(p->dev));
    AGB_CUDA(cudaDeviceSynchronize());
    for (int r = 0; r < p->world; ++r)
        if (p->ipc_opened[r]) {
            AGB_CUDA(cudaIpcCloseMemHandle(p->blk.base[r]));
            p->ipc_opened[r] = false;
            p->blk.base[r] = nullptr;
        }
    p->connected = false;
    return AGB_OK;
}

int agb_peer_destroy(agb_peer_t* p) {
    if (!p) return AGB_OK;
    DeviceRestore restore;
    cudaSetDevice(p->dev);
    cudaDeviceSynchronize();
    for (int r = 0; r < p->world; ++r)
        if (p->ipc_opened[r]) cudaIpcCloseMemHandle(p->blk.base[r]);
    if (p->blk.base[p->rank]) cudaFree(p->blk.base[p->rank]);
    if (p->ev_pub) cudaEventDestroy(p->ev_pub);
    if (p->ev_side) cudaEventDestroy(p->ev_side);
    delete p;
    return AGB_OK;
}

}  // extern "C"
