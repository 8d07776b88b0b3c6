// rmsnorm_stack.cpp -- see nn/rmsnorm_stack.hpp.
#include "nn/rmsnorm_stack.hpp"

#include "ad/detail/host_util.hpp"

namespace ag::nn {

using detail::check_status;

ResidualRMSNormStack::ResidualRMSNormStack(int layers, int64_t rows, int64_t hidden, Dtype dtype, float eps,
                                           DeviceIndex device)
    : layers_(layers), rows_(rows), hidden_(hidden), dtype_(dtype), eps_(eps), device_(device) {
    if (layers < 1 || rows < 1 || hidden < 1) throw std::invalid_argument("ResidualRMSNormStack: bad sizes");
    if (!device.is_cuda()) throw std::invalid_argument("ResidualRMSNormStack: CUDA device required");
    const TensorOptions act = TensorOptions().with_dtype(dtype).with_device(device);
    const TensorOptions f32 = TensorOptions().with_dtype(Dtype::Float32).with_device(device);
    gammas_ = Tensor::ones(Shape{{layers, hidden}}, act);
    dgammas_ = Tensor::zeros(Shape{{layers, hidden}}, f32);
    for (int l = 0; l < layers; ++l) {
        h_.emplace_back(Shape{{rows, hidden}}, act);
        rstd_.emplace_back(Shape{{rows, 1}}, f32);
    }
    for (auto& t : y_) t = Tensor(Shape{{rows, hidden}}, act);
    for (auto& t : dh_) t = Tensor(Shape{{rows, hidden}}, act);
    const int code = dtype == Dtype::Float32 ? AGB_F32 : AGB_BF16;
    const size_t wsb = agb_rmsnorm_bwd_workspace_bytes(rows, hidden, code);
    for (auto& w : workspace_)
        w = Tensor(Shape{{static_cast<int64_t>((wsb + 7) / 8)}}, TensorOptions().with_dtype(Dtype::Float64).with_device(device));
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess)
        throw std::runtime_error("ResidualRMSNormStack: cannot create the reduction stream");
    side_stream_ = s;
    for (int i = 0; i < 2; ++i) {
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess)
            throw std::runtime_error("ResidualRMSNormStack: cannot create events");
        ev_bwd_[i] = a;
        ev_reduce_[i] = b;
    }
}

ResidualRMSNormStack::~ResidualRMSNormStack() {
    if (side_stream_) cudaStreamSynchronize(static_cast<cudaStream_t>(side_stream_));
    for (int i = 0; i < 2; ++i) {
        if (ev_bwd_[i]) cudaEventDestroy(static_cast<cudaEvent_t>(ev_bwd_[i]));
        if (ev_reduce_[i]) cudaEventDestroy(static_cast<cudaEvent_t>(ev_reduce_[i]));
    }
    if (side_stream_) cudaStreamDestroy(static_cast<cudaStream_t>(side_stream_));
}

size_t ResidualRMSNormStack::saved_bytes() const {
    return static_cast<size_t>(layers_) * (h_[0].nbytes() + rstd_[0].nbytes());
}

void ResidualRMSNormStack::forward(const Tensor& x, const Tensor& r) {
    if (x.numel() != rows_ * hidden_ || r.numel() != x.numel() || x.dtype() != dtype_ || r.dtype() != dtype_)
        throw std::invalid_argument("ResidualRMSNormStack::forward: x / r do not match the stack");
    const int code = detail::agb_dtype(x);
    const size_t esz = dtype_size(dtype_);
    const void* xl = x.raw();
    const void* rl = r.raw();
    for (int l = 0; l < layers_; ++l) {
        const char* gamma = static_cast<const char*>(gammas_.raw()) + static_cast<size_t>(l) * hidden_ * esz;
        Tensor& y = y_[l & 1];
        check_status(agb_add_rmsnorm_fwd(xl, rl, gamma, h_[l].raw(), y.raw(), rstd_[l].data<float>(), rows_, hidden_, eps_,
                                         code, current_stream()),
                     "stack forward");
        xl = h_[l].raw();
        rl = y.raw();
    }
}

void ResidualRMSNormStack::backward(const Tensor& g) {
    if (g.numel() != rows_ * hidden_ || g.dtype() != dtype_)
        throw std::invalid_argument("ResidualRMSNormStack::backward: g does not match the stack");
    const int code = detail::agb_dtype(g);
    const size_t esz = dtype_size(dtype_);
    const void* gy = g.raw();
    int out = 0;
    cudaStream_t main = reinterpret_cast<cudaStream_t>(current_stream());
    cudaStream_t side = static_cast<cudaStream_t>(side_stream_);
    auto cuda_ok = [](cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("stack backward: ") + what + ": " + cudaGetErrorString(e));
    };
    int step = 0;
    for (int l = layers_ - 1; l >= 0; --l, ++step) {
        const char* gamma = static_cast<const char*>(gammas_.raw()) + static_cast<size_t>(l) * hidden_ * esz;
        float* dg = dgammas_.data<float>() + static_cast<size_t>(l) * hidden_;
        const int w = step & 1;
        // this workspace was last read by the reduction of two layers ago
        if (step >= 2) cuda_ok(cudaStreamWaitEvent(main, static_cast<cudaEvent_t>(ev_reduce_[w]), 0), "wait for the reduction");
        // top layer: dh = vjp(g).  Below: dh_l = vjp(dh_{l+1}) + dh_{l+1}; the addend is gy itself.
        const void* add = l == layers_ - 1 ? nullptr : gy;
        int partials = 0;
        check_status(agb_rmsnorm_bwd_partials(h_[l].raw(), gamma, rstd_[l].data<float>(), gy, add, dh_[out].raw(),
                                              workspace_[w].raw(), workspace_[w].nbytes(), rows_, hidden_, code,
                                              current_stream(), &partials),
                     "stack backward");
        // the column reduction: on the second stream, behind this layer's backward, beside the next layer's
        cuda_ok(cudaEventRecord(static_cast<cudaEvent_t>(ev_bwd_[w]), main), "record");
        cuda_ok(cudaStreamWaitEvent(side, static_cast<cudaEvent_t>(ev_bwd_[w]), 0), "wait for the backward");
        check_status(agb_dgamma_reduce(workspace_[w].raw(), partials, hidden_, dg, AGB_F32, /*accumulate=*/0,
                                       reinterpret_cast<agb_stream_t>(side)),
                     "stack dgamma reduction");
        cuda_ok(cudaEventRecord(static_cast<cudaEvent_t>(ev_reduce_[w]), side), "record");
        gy = dh_[out].raw();
        dh_final_ = out;
        out ^= 1;
    }
    // join: the caller's stream holds every dgamma when backward() returns (and a capture sees the branch closed)
    for (int w = 0; w < 2 && w < layers_; ++w)
        cuda_ok(cudaStreamWaitEvent(main, static_cast<cudaEvent_t>(ev_reduce_[w]), 0), "join");
}

void ResidualRMSNormStack::capture(CudaGraphRunner& runner, const Tensor& x, const Tensor& r, const Tensor& g) {
    runner.begin_capture();
    try {
        forward(x, r);
        backward(g);
    } catch (...) {
        runner.end_capture();
        throw;
    }
    runner.end_capture();
}

}  // namespace ag::nn
