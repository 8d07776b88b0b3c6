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
    workspace_ = Tensor(Shape{{static_cast<int64_t>((wsb + 7) / 8)}}, TensorOptions().with_dtype(Dtype::Float64).with_device(device));
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
    for (int l = layers_ - 1; l >= 0; --l) {
        const char* gamma = static_cast<const char*>(gammas_.raw()) + static_cast<size_t>(l) * hidden_ * esz;
        float* dg = dgammas_.data<float>() + static_cast<size_t>(l) * hidden_;
        // top layer: dh = vjp(g).  Below: dh_l = vjp(dh_{l+1}) + dh_{l+1}; the addend is gy itself.
        const void* add = l == layers_ - 1 ? nullptr : gy;
        check_status(agb_rmsnorm_bwd(h_[l].raw(), gamma, rstd_[l].data<float>(), gy, add, dh_[out].raw(), dg, AGB_F32,
                                     /*accumulate_dgamma=*/0, workspace_.raw(), workspace_.nbytes(), rows_, hidden_, code,
                                     current_stream()),
                     "stack backward");
        gy = dh_[out].raw();
        dh_final_ = out;
        out ^= 1;
    }
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
