// rmsnorm_stack.hpp -- a stack of L fused residual-add + RMSNorm layers (pre-norm residual stream):
//     x_0 = x, r_0 = r;   h_l = x_l + r_l;   y_l = rmsnorm(h_l) * gamma_l;   x_{l+1} = h_l, r_{l+1} = y_l
// forward() and backward() make exactly one library call per layer each way (the add is fused into
// the norm forward, and `dh_l = vjp(h_l) + dh_{l+1}` into the norm backward, whose incoming
// gradient IS dh_{l+1}, so it is read once).  Every buffer is allocated in the constructor, so
// forward + backward can be captured into one CUDA graph with ag::CudaGraphRunner: 2L kernel
// launches plus L dgamma reductions, no allocation, no host work between layers.
// The column reduction of layer l's dgamma does not sit between the backward kernels of layers l and l-1:
// it runs on a second stream behind an event (a forked branch of the captured graph), over two partial-row
// workspaces used in turn, so that it overlaps the next layer's backward instead of adding its few
// microseconds to every layer; the branch is joined before backward() returns.
// The reference has no such class; it would run this as 3L graph nodes and ~25 tensor calls per
// layer (add_nodeops, rms_nodeops, mul_nodeops and their VJPs).
#pragma once
#include <vector>

#include "ad/runtime/cuda_graphs.hpp"
#include "tensor.hpp"

namespace ag::nn {

class ResidualRMSNormStack {
public:
    ResidualRMSNormStack(int layers, int64_t rows, int64_t hidden, Dtype dtype, float eps, DeviceIndex device);
    ~ResidualRMSNormStack();
    ResidualRMSNormStack(const ResidualRMSNormStack&) = delete;
    ResidualRMSNormStack& operator=(const ResidualRMSNormStack&) = delete;

    int layers() const { return layers_; }
    Tensor& gammas() { return gammas_; }            // [L, hidden], dtype of the stack; fill before use
    const Tensor& dgammas() const { return dgammas_; }  // [L, hidden] fp32, overwritten by backward()
    const Tensor& y_last() const { return y_[(layers_ - 1) & 1]; }
    const Tensor& dh0() const { return dh_[dh_final_]; }  // gradient of x_0 (== gradient of r_0)

    // Enqueue on ag::current_stream().  x, r, g: [rows, hidden], same dtype and device as the stack.
    void forward(const Tensor& x, const Tensor& r);
    void backward(const Tensor& g);

    // Captures forward(x, r) followed by backward(g) into `runner` (the tensors must stay alive and
    // keep their addresses; replay re-reads their current contents).
    void capture(CudaGraphRunner& runner, const Tensor& x, const Tensor& r, const Tensor& g);

    size_t saved_bytes() const;  // activations kept for the backward: L * (h + rstd)

private:
    int layers_;
    int64_t rows_, hidden_;
    Dtype dtype_;
    float eps_;
    DeviceIndex device_;
    Tensor gammas_, dgammas_, workspace_[2];
    void* side_stream_ = nullptr;         // cudaStream_t of the dgamma reductions
    void* ev_bwd_[2] = {nullptr, nullptr};     // cudaEvent_t: layer's backward kernel done (per workspace)
    void* ev_reduce_[2] = {nullptr, nullptr};  // cudaEvent_t: the reduction that read the workspace done
    std::vector<Tensor> h_, rstd_;
    Tensor y_[2], dh_[2];
    int dh_final_ = 0;
};

}  // namespace ag::nn
