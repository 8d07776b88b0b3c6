// agb_host.cuh -- the host-buffer pipe of include/agb/agb_host.h.  Included at the end of agb_cuda.cu.
#pragma once
#include "agb/agb_host.h"

struct agb_host_pipe {
    static constexpr int kSlots = 3;
    int dev = 0, dtype = AGB_F32;
    int64_t hidden = 0, chunk = 0;
    size_t elem = 4, ws_bytes = 0;
    cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
    struct Slot {
        void *x = nullptr, *gy = nullptr, *y = nullptr, *dx = nullptr;
        float* rstd = nullptr;
        cudaEvent_t in_ready = nullptr, done = nullptr, out_done = nullptr;
    } slot[kSlots];
    void *gamma = nullptr, *ws = nullptr;
    double* sums = nullptr;
    float* dg32 = nullptr;
    cudaEvent_t gamma_ready = nullptr;
};

namespace {

void host_pipe_free(agb_host_pipe_t* p) {
    if (!p) return;
    for (cudaStream_t s : {p->h2d, p->compute, p->d2h})
        if (s) cudaStreamSynchronize(s);
    for (auto& s : p->slot) {
        for (void* q : {s.x, s.gy, s.y, s.dx, static_cast<void*>(s.rstd)})
            if (q) cudaFree(q);
        for (cudaEvent_t e : {s.in_ready, s.done, s.out_done})
            if (e) cudaEventDestroy(e);
    }
    for (void* q : {p->gamma, p->ws, static_cast<void*>(p->sums), static_cast<void*>(p->dg32)})
        if (q) cudaFree(q);
    if (p->gamma_ready) cudaEventDestroy(p->gamma_ready);
    for (cudaStream_t s : {p->h2d, p->compute, p->d2h})
        if (s) cudaStreamDestroy(s);
    delete p;
}

}  // namespace

extern "C" {

int agb_host_pipe_create(int64_t hidden, int dtype, int64_t chunk_rows, agb_host_pipe_t** out) {
    if (!out) return fail(AGB_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    AGB_TRY(check_common(0, hidden, dtype));
    if (chunk_rows < 0) return fail(AGB_ERR_INVALID_ARG, "chunk_rows=%lld", (long long)chunk_rows);
    agb_host_pipe_t* p = new agb_host_pipe();
    p->dtype = dtype;
    p->hidden = hidden;
    p->elem = dtype == AGB_F32 ? 4 : 2;
    const int64_t row_bytes = hidden * static_cast<int64_t>(p->elem);
    p->chunk = chunk_rows > 0 ? chunk_rows : (row_bytes >= (64 << 20) ? 1 : (64 << 20) / row_bytes);
    cudaError_t e = cudaGetDevice(&p->dev);
    auto ok = [&](cudaError_t r) { if (e == cudaSuccess) e = r; return e == cudaSuccess; };
    const size_t arr = static_cast<size_t>(p->chunk) * row_bytes;
    for (cudaStream_t* s : {&p->h2d, &p->compute, &p->d2h}) ok(cudaStreamCreateWithFlags(s, cudaStreamNonBlocking));
    for (auto& s : p->slot) {
        for (void** q : {&s.x, &s.gy, &s.y, &s.dx}) ok(cudaMalloc(q, arr));
        ok(cudaMalloc(reinterpret_cast<void**>(&s.rstd), static_cast<size_t>(p->chunk) * sizeof(float)));
        for (cudaEvent_t* ev : {&s.in_ready, &s.done, &s.out_done}) ok(cudaEventCreateWithFlags(ev, cudaEventDisableTiming));
    }
    p->ws_bytes = agb_rmsnorm_bwd_workspace_bytes(p->chunk, hidden, dtype);
    ok(cudaMalloc(&p->gamma, static_cast<size_t>(row_bytes)));
    ok(cudaMalloc(&p->ws, p->ws_bytes ? p->ws_bytes : 8));
    ok(cudaMalloc(reinterpret_cast<void**>(&p->sums), static_cast<size_t>(hidden) * sizeof(double)));
    ok(cudaMalloc(reinterpret_cast<void**>(&p->dg32), static_cast<size_t>(hidden) * sizeof(float)));
    ok(cudaEventCreateWithFlags(&p->gamma_ready, cudaEventDisableTiming));
    if (e != cudaSuccess || p->ws_bytes == 0) {
        host_pipe_free(p);
        return e != cudaSuccess ? cuda_fail(e, "agb_host_pipe_create") : fail(AGB_ERR_CUDA, "no CUDA device");
    }
    *out = p;
    return AGB_OK;
}

int64_t agb_host_pipe_chunk_rows(const agb_host_pipe_t* p) { return p ? p->chunk : 0; }

int agb_host_pipe_fwd_bwd(agb_host_pipe_t* p, const void* x, const void* gy, const void* gamma, void* y, void* dx,
                          float* dgamma, float* rstd, int64_t rows, float eps, double* dgamma_sum) {
    AGB_RANGE();
    if (!p) return fail(AGB_ERR_INVALID_ARG, "pipe is NULL");
    if (rows < 0) return fail(AGB_ERR_INVALID_ARG, "rows=%lld", (long long)rows);
    if (!gamma || !dgamma) return fail(AGB_ERR_INVALID_ARG, "gamma and dgamma are required");
    if (rows > 0 && (!x || !gy || !y || !dx)) return fail(AGB_ERR_INVALID_ARG, "a host buffer is NULL");
    int dev = -1;
    AGB_CUDA(cudaGetDevice(&dev));
    if (dev != p->dev) return fail(AGB_ERR_INVALID_ARG, "current device %d, pipe created on %d", dev, p->dev);
    const size_t row_bytes = static_cast<size_t>(p->hidden) * p->elem;
    AGB_CUDA(cudaMemcpyAsync(p->gamma, gamma, row_bytes, cudaMemcpyHostToDevice, p->h2d));
    AGB_CUDA(cudaEventRecord(p->gamma_ready, p->h2d));
    AGB_CUDA(cudaStreamWaitEvent(p->compute, p->gamma_ready, 0));
    const int64_t nchunks = (rows + p->chunk - 1) / p->chunk;
    if (nchunks == 0) AGB_CUDA(cudaMemsetAsync(p->sums, 0, static_cast<size_t>(p->hidden) * sizeof(double), p->compute));
    for (int64_t c = 0; c < nchunks; ++c) {
        const int64_t r0 = c * p->chunk, n = (rows - r0 < p->chunk ? rows - r0 : p->chunk);
        const size_t off = static_cast<size_t>(r0) * row_bytes, bytes = static_cast<size_t>(n) * row_bytes;
        agb_host_pipe::Slot& s = p->slot[c % agb_host_pipe::kSlots];
        const bool reused = c >= agb_host_pipe::kSlots;
        if (reused) AGB_CUDA(cudaStreamWaitEvent(p->h2d, s.done, 0));          // kernels of the chunk that used this slot
        AGB_CUDA(cudaMemcpyAsync(s.x, static_cast<const char*>(x) + off, bytes, cudaMemcpyHostToDevice, p->h2d));
        AGB_CUDA(cudaMemcpyAsync(s.gy, static_cast<const char*>(gy) + off, bytes, cudaMemcpyHostToDevice, p->h2d));
        AGB_CUDA(cudaEventRecord(s.in_ready, p->h2d));
        AGB_CUDA(cudaStreamWaitEvent(p->compute, s.in_ready, 0));
        if (reused) AGB_CUDA(cudaStreamWaitEvent(p->compute, s.out_done, 0));   // outputs of the previous user copied out
        AGB_TRY(agb_rmsnorm_fwd(s.x, p->gamma, s.y, s.rstd, n, p->hidden, eps, p->dtype, p->compute));
        AGB_TRY(agb_rmsnorm_bwd(s.x, p->gamma, s.rstd, s.gy, nullptr, s.dx, p->sums, AGB_F64, /*accumulate=*/c > 0, p->ws,
                                p->ws_bytes, n, p->hidden, p->dtype, p->compute));
        AGB_CUDA(cudaEventRecord(s.done, p->compute));
        AGB_CUDA(cudaStreamWaitEvent(p->d2h, s.done, 0));
        AGB_CUDA(cudaMemcpyAsync(static_cast<char*>(y) + off, s.y, bytes, cudaMemcpyDeviceToHost, p->d2h));
        AGB_CUDA(cudaMemcpyAsync(static_cast<char*>(dx) + off, s.dx, bytes, cudaMemcpyDeviceToHost, p->d2h));
        if (rstd) AGB_CUDA(cudaMemcpyAsync(rstd + r0, s.rstd, static_cast<size_t>(n) * sizeof(float), cudaMemcpyDeviceToHost, p->d2h));
        AGB_CUDA(cudaEventRecord(s.out_done, p->d2h));
    }
    if (dgamma_sum)
        AGB_CUDA(cudaMemcpyAsync(dgamma_sum, p->sums, static_cast<size_t>(p->hidden) * sizeof(double), cudaMemcpyDeviceToDevice, p->compute));
    AGB_TRY(agb_dgamma_finalize(p->sums, p->dg32, p->hidden, 0, p->compute));
    AGB_CUDA(cudaMemcpyAsync(dgamma, p->dg32, static_cast<size_t>(p->hidden) * sizeof(float), cudaMemcpyDeviceToHost, p->compute));
    AGB_CUDA(cudaStreamSynchronize(p->h2d));
    AGB_CUDA(cudaStreamSynchronize(p->compute));
    AGB_CUDA(cudaStreamSynchronize(p->d2h));
    return AGB_OK;
}

int agb_host_pipe_destroy(agb_host_pipe_t* p) {
    if (!p) return AGB_OK;
    DeviceRestore restore;
    cudaSetDevice(p->dev);
    host_pipe_free(p);
    return AGB_OK;
}

}  // extern "C"
