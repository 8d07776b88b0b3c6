// agb_shard.cuh -- the single-process, multi-GPU executor declared in include/agb/agb_shard.h.
// Included at the end of agb_cuda.cu (same translation unit: it uses that file's error helpers
// and calls the public entry points for the per-shard work).
//
// Ordering is by CUDA events only, all recorded and waited on from the calling host thread:
//   stream i:  forward | wait done[j] of the previous run | backward -> record bwd[i]
//              | wait bwd[j] for all j | peer-sum kernel -> record done[i]
// A wait always follows, in host program order, the record it refers to, so it can never see a
// stale record.  No kernel polls memory that another kernel writes.
// Deferred mode moves the last line to a second stream per shard and alternates two sum buffers, so
// that a shard's main stream goes on with the next step without waiting for the slowest shard; it
// only waits (for the sums it wrote two runs ago to have been read) before overwriting a buffer.
#pragma once
#include "agb/agb_shard.h"

namespace agb {

struct PeerSums {
    const double* p[AGB_SHARD_MAX];
};

// dgamma[c] = (float)(sums_0[c] + sums_1[c] + ... ) in shard order: the same additions in the same
// order on every shard, so all of them hold the same bits.  The sums of other shards are read through
// peer mappings (plain loads over NVLink); .cg keeps them out of L1, which is not coherent with a peer.
__global__ void dgamma_peer_sum_kernel(PeerSums src, int n, int hidden, float* __restrict__ dgamma, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    double s = __ldcg(src.p[0] + c);
    for (int r = 1; r < n; ++r) s += __ldcg(src.p[r] + c);
    const float v = static_cast<float>(s);
    dgamma[c] = accumulate ? add_rn(dgamma[c], v) : v;
}

}  // namespace agb

struct agb_shard {
    int n = 0;
    int64_t max_hidden = 0;
    size_t ws_bytes = 0;
    bool deferred = false;       // exchange on the side streams, two sum buffers in turn
    bool done_recorded[2] = {false, false};   // the done[][b] events have been recorded by an earlier run
    int turn = 0, newest = -1;   // buffer of the next run / of the latest exchange
    int dev[AGB_SHARD_MAX] = {};
    cudaStream_t st[AGB_SHARD_MAX] = {}, side[AGB_SHARD_MAX] = {};
    cudaEvent_t ev_bwd[AGB_SHARD_MAX] = {}, ev_done[AGB_SHARD_MAX][2] = {};
    void* ws[AGB_SHARD_MAX] = {};
    double* sums[AGB_SHARD_MAX][2] = {};
};

namespace {

// Restores the caller's current device on every exit path.
struct DeviceRestore {
    int saved = -1;
    DeviceRestore() { if (cudaGetDevice(&saved) != cudaSuccess) saved = -1; }
    ~DeviceRestore() { if (saved >= 0) cudaSetDevice(saved); }
};

int shard_check(const agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, int dtype) {
    if (!s) return fail(AGB_ERR_INVALID_ARG, "executor is NULL");
    if (!io) return fail(AGB_ERR_INVALID_ARG, "io is NULL");
    AGB_TRY(check_common(0, hidden, dtype));
    if (hidden > s->max_hidden)
        return fail(AGB_ERR_WORKSPACE, "hidden %lld exceeds the executor's max_hidden %lld", (long long)hidden,
                    (long long)s->max_hidden);
    for (int i = 0; i < s->n; ++i)
        if (io[i].rows < 0) return fail(AGB_ERR_INVALID_ARG, "shard %d: rows=%lld", i, (long long)io[i].rows);
    return AGB_OK;
}

void shard_free(agb_shard_t* s) {
    for (int i = 0; i < s->n; ++i) {
        if (cudaSetDevice(s->dev[i]) != cudaSuccess) continue;
        if (s->st[i]) cudaStreamSynchronize(s->st[i]);
        if (s->side[i]) cudaStreamSynchronize(s->side[i]);
    }
    for (int i = 0; i < s->n; ++i) {
        if (cudaSetDevice(s->dev[i]) != cudaSuccess) continue;
        if (s->ws[i]) cudaFree(s->ws[i]);
        if (s->ev_bwd[i]) cudaEventDestroy(s->ev_bwd[i]);
        for (int b = 0; b < 2; ++b) {
            if (s->sums[i][b]) cudaFree(s->sums[i][b]);
            if (s->ev_done[i][b]) cudaEventDestroy(s->ev_done[i][b]);
        }
        if (s->st[i]) cudaStreamDestroy(s->st[i]);
        if (s->side[i]) cudaStreamDestroy(s->side[i]);
    }
    delete s;
}

int shard_create(const int* devices, int n, int64_t max_hidden, agb_shard_t* s) {
    int ndev = 0;
    AGB_CUDA(cudaGetDeviceCount(&ndev));
    for (int i = 0; i < n; ++i)
        if (devices[i] < 0 || devices[i] >= ndev)
            return fail(AGB_ERR_INVALID_ARG, "devices[%d]=%d but the machine has %d", i, devices[i], ndev);
    for (int a = 0; a < n; ++a)
        for (int b = 0; b < n; ++b) {
            if (devices[a] == devices[b]) continue;
            int ok = 0;
            AGB_CUDA(cudaDeviceCanAccessPeer(&ok, devices[a], devices[b]));
            if (!ok) return fail(AGB_ERR_UNSUPPORTED, "device %d cannot map the memory of device %d", devices[a], devices[b]);
            AGB_CUDA(cudaSetDevice(devices[a]));
            cudaError_t e = cudaDeviceEnablePeerAccess(devices[b], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();   // not an error: clear it
            else if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
        }
    s->max_hidden = max_hidden;
    for (int i = 0; i < n; ++i) {
        s->dev[i] = devices[i];
        s->n = i + 1;   // shard_free releases what exists so far
        AGB_CUDA(cudaSetDevice(devices[i]));
        AGB_CUDA(cudaStreamCreateWithFlags(&s->st[i], cudaStreamNonBlocking));
        AGB_CUDA(cudaStreamCreateWithFlags(&s->side[i], cudaStreamNonBlocking));
        AGB_CUDA(cudaEventCreateWithFlags(&s->ev_bwd[i], cudaEventDisableTiming));
        for (int b = 0; b < 2; ++b) AGB_CUDA(cudaEventCreateWithFlags(&s->ev_done[i][b], cudaEventDisableTiming));
        const size_t wb = agb_rmsnorm_bwd_workspace_bytes(1, max_hidden, AGB_F32);
        if (wb == 0) return fail(AGB_ERR_CUDA, "no workspace size for device %d: %s", devices[i], t_err);
        if (i == 0 || wb < s->ws_bytes) s->ws_bytes = wb;
        AGB_CUDA(cudaMalloc(&s->ws[i], wb));
        for (int b = 0; b < 2; ++b)
            AGB_CUDA(cudaMalloc(reinterpret_cast<void**>(&s->sums[i][b]), static_cast<size_t>(max_hidden) * sizeof(double)));
    }
    return AGB_OK;
}

int shard_fwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, float eps, int dtype) {
    for (int i = 0; i < s->n; ++i) {
        if (io[i].rows == 0) continue;
        AGB_CUDA(cudaSetDevice(s->dev[i]));
        int st = agb_rmsnorm_fwd(io[i].x, io[i].gamma, io[i].y, io[i].rstd, io[i].rows, hidden, eps, dtype, s->st[i]);
        if (st != AGB_OK) return st;
    }
    return AGB_OK;
}

int shard_bwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, int dtype, int accumulate) {
    const bool want_dg = io[0].dgamma != nullptr;
    for (int i = 0; i < s->n; ++i) {
        if ((io[i].dgamma != nullptr) != want_dg)
            return fail(AGB_ERR_INVALID_ARG, "dgamma must be given for every shard or for none (shard %d differs)", i);
        if (want_dg && !io[i].gamma) return fail(AGB_ERR_INVALID_ARG, "shard %d: dgamma without gamma", i);
        if (want_dg) AGB_TRY(check_ptr(io[i].dgamma, "dgamma", 4));
    }
    const int b = s->deferred ? (s->turn & 1) : 0;   // the sum buffer of this run
    for (int i = 0; i < s->n; ++i) {
        AGB_CUDA(cudaSetDevice(s->dev[i]));
        if (want_dg && s->done_recorded[b])   // shards may still be reading what this shard last wrote into buffer b
            for (int j = 0; j < s->n; ++j)
                if (j != i || s->deferred) AGB_CUDA(cudaStreamWaitEvent(s->st[i], s->ev_done[j][b], 0));
        if (io[i].rows > 0) {
            int st = agb_rmsnorm_bwd(io[i].x, io[i].gamma, io[i].rstd, io[i].gy, io[i].dx_add, io[i].dx,
                                     want_dg ? s->sums[i][b] : nullptr, AGB_F64, 0, want_dg ? s->ws[i] : nullptr,
                                     want_dg ? s->ws_bytes : 0, io[i].rows, hidden, dtype, s->st[i]);
            if (st != AGB_OK) return st;
        } else if (want_dg) {
            AGB_CUDA(cudaMemsetAsync(s->sums[i][b], 0, static_cast<size_t>(hidden) * sizeof(double), s->st[i]));
        }
        if (want_dg) AGB_CUDA(cudaEventRecord(s->ev_bwd[i], s->st[i]));
    }
    if (!want_dg) return AGB_OK;
    agb::PeerSums src{};
    for (int j = 0; j < s->n; ++j) src.p[j] = s->sums[j][b];
    for (int i = 0; i < s->n; ++i) {
        AGB_CUDA(cudaSetDevice(s->dev[i]));
        cudaStream_t q = s->deferred ? s->side[i] : s->st[i];
        for (int j = 0; j < s->n; ++j)
            if (j != i || s->deferred) AGB_CUDA(cudaStreamWaitEvent(q, s->ev_bwd[j], 0));
        agb::dgamma_peer_sum_kernel<<<static_cast<unsigned>((hidden + 255) / 256), 256, 0, q>>>(
            src, s->n, static_cast<int>(hidden), io[i].dgamma, accumulate);
        AGB_TRY(after_launch("dgamma_peer_sum"));
        AGB_CUDA(cudaEventRecord(s->ev_done[i][b], q));
    }
    s->done_recorded[b] = true;
    s->newest = b;
    if (s->deferred) ++s->turn;
    return AGB_OK;
}

}  // namespace

extern "C" {

int agb_shard_create(const int* devices, int n, int64_t max_hidden, agb_shard_t** out) {
    if (!out) return fail(AGB_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (!devices || n < 1 || n > AGB_SHARD_MAX) return fail(AGB_ERR_INVALID_ARG, "n=%d outside [1, %d] or devices NULL", n, AGB_SHARD_MAX);
    if (max_hidden <= 0 || max_hidden > (1LL << 30)) return fail(AGB_ERR_INVALID_ARG, "max_hidden=%lld", (long long)max_hidden);
    DeviceRestore restore;
    agb_shard_t* s = new agb_shard();
    const int st = shard_create(devices, n, max_hidden, s);
    if (st != AGB_OK) {
        shard_free(s);
        return st;
    }
    *out = s;
    return AGB_OK;
}

int agb_shard_count(const agb_shard_t* s) { return s ? s->n : 0; }

int agb_shard_stream(const agb_shard_t* s, int i, agb_stream_t* stream) {
    if (!s || !stream || i < 0 || i >= s->n) return fail(AGB_ERR_INVALID_ARG, "bad executor, index or output");
    *stream = s->st[i];
    return AGB_OK;
}

int agb_shard_run_fwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, float eps, int dtype) {
    AGB_TRY(shard_check(s, io, hidden, dtype));
    DeviceRestore restore;
    return shard_fwd(s, io, hidden, eps, dtype);
}

int agb_shard_run_bwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, int dtype, int accumulate_dgamma) {
    AGB_TRY(shard_check(s, io, hidden, dtype));
    DeviceRestore restore;
    return shard_bwd(s, io, hidden, dtype, accumulate_dgamma);
}

int agb_shard_run_fwd_bwd(agb_shard_t* s, const agb_shard_io_t* io, int64_t hidden, float eps, int dtype,
                          int accumulate_dgamma) {
    AGB_TRY(shard_check(s, io, hidden, dtype));
    DeviceRestore restore;
    AGB_TRY(shard_fwd(s, io, hidden, eps, dtype));
    return shard_bwd(s, io, hidden, dtype, accumulate_dgamma);
}

int agb_shard_set_deferred_exchange(agb_shard_t* s, int on) {
    if (!s) return fail(AGB_ERR_INVALID_ARG, "executor is NULL");
    if ((on != 0) == s->deferred) return AGB_OK;
    // switching modes changes which stream owns the exchange: settle everything in flight first
    AGB_TRY(agb_shard_synchronize(s));
    s->deferred = on != 0;
    s->done_recorded[0] = s->done_recorded[1] = false;
    s->turn = 0;
    s->newest = -1;
    return AGB_OK;
}

int agb_shard_wait_dgamma(agb_shard_t* s) {
    if (!s) return fail(AGB_ERR_INVALID_ARG, "executor is NULL");
    if (!s->deferred || s->newest < 0) return AGB_OK;   // immediate mode: the shard streams already hold it
    DeviceRestore restore;
    for (int i = 0; i < s->n; ++i) {
        AGB_CUDA(cudaSetDevice(s->dev[i]));
        AGB_CUDA(cudaStreamWaitEvent(s->st[i], s->ev_done[i][s->newest], 0));
    }
    return AGB_OK;
}

int agb_shard_synchronize(agb_shard_t* s) {
    if (!s) return fail(AGB_ERR_INVALID_ARG, "executor is NULL");
    DeviceRestore restore;
    for (int i = 0; i < s->n; ++i) {
        AGB_CUDA(cudaSetDevice(s->dev[i]));
        AGB_CUDA(cudaStreamSynchronize(s->st[i]));
        AGB_CUDA(cudaStreamSynchronize(s->side[i]));
    }
    int worst = AGB_OK;
    for (int i = 0; i < s->n; ++i) {
        bool seen = false;
        for (int j = 0; j < i; ++j) seen = seen || s->dev[j] == s->dev[i];
        if (seen) continue;
        AGB_CUDA(cudaSetDevice(s->dev[i]));
        const int st = agb_device_status();
        if (st != AGB_OK) worst = st;
    }
    return worst;
}

int agb_shard_destroy(agb_shard_t* s) {
    if (!s) return AGB_OK;
    DeviceRestore restore;
    shard_free(s);
    return AGB_OK;
}

}  // extern "C"
