// nn.cpp -- see nn/nn.hpp (cgadimpl/src/nn/nn.cpp:8-23, 43-56 for Module and Sequential).
#include "nn/nn.hpp"

#include "ad/detail/host_util.hpp"

namespace ag::nn {

void Module::to(DeviceIndex dev) {
    for (Value& p : params_)
        if (p.node) {
            p.node->value = p.node->value.to(dev);
            p.node->grad = Tensor();          // allocated on the new device by the first contribution
            p.node->grad_live = false;
            p.node->creation_context.device = dev;
        }
}

void Module::zero_grad() {
    for (Value& p : params_)
        if (p.node && p.node->requires_grad()) {
            std::lock_guard<std::mutex> lock(p.node->grad_mutex);
            p.node->grad_live = false;        // reads as zeros; the next backward overwrites the buffer
        }
}

RMSNorm::RMSNorm(int64_t hidden, float eps, DeviceIndex dev, Dtype dtype) : eps_(eps) {
    if (hidden < 1) throw std::invalid_argument("RMSNorm: hidden must be positive");
    Tensor g = Tensor::ones(Shape{{hidden}}, TensorOptions().with_device(dev).with_dtype(dtype).with_req_grad(true));
    params_.push_back(make_tensor(g, "gamma"));
}
Value RMSNorm::operator()(Value input) { return ag::rmsnorm(input, params_[0], eps_); }
Value RMSNorm::operator()(Value x, Value residual) { return ag::add_rmsnorm(x, residual, params_[0], eps_); }

Sequential::Sequential(const std::vector<Module*>& modules) : layers_(modules) {
    for (auto* m : layers_)
        for (auto& p : m->parameters()) params_.push_back(p);
}
Value Sequential::operator()(Value x) {
    for (auto* layer : layers_) x = (*layer)(x);
    return x;
}

}  // namespace ag::nn
