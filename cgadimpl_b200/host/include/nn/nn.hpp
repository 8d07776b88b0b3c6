// nn.hpp -- Module API of cgadimpl/include/nn/nn.hpp:9-54 for the layer on this path.  Module and
// Sequential keep the reference's members and signatures; RMSNorm is the layer the reference lacks
// as a module (it only has the gamma-less `rms` op): a per-channel gamma parameter of shape
// [hidden] and a call operator that builds the fused RMSNormAffine node.  ResidualRMSNorm is the
// pre-norm residual block h = x + r, y = RMSNorm(h) built with one forward kernel.
#pragma once
#include <vector>

#include "ad/core/graph.hpp"
#include "ad/ops/ops.hpp"

namespace ag::nn {

class Module {
public:
    virtual ~Module() = default;
    virtual Value operator()(Value input) = 0;
    Value operator()(const Tensor& input) { return this->operator()(ag::make_tensor(input)); }

    std::vector<Value>& parameters() { return params_; }
    void to(DeviceIndex dev);   // moves parameters and gives them fresh zero gradients
    void to(Device dev) { to(DeviceIndex(dev)); }
    void zero_grad();
    void register_backward_hook(HookFn hook) {
        for (auto& p : params_) p.register_hook(hook);
    }

protected:
    std::vector<Value> params_;
};

class RMSNorm : public Module {
public:
    RMSNorm(int64_t hidden, float eps = 1e-5f, DeviceIndex dev = DeviceIndex(Device::CUDA), Dtype dtype = Dtype::Float32);
    using Module::operator();
    Value operator()(Value input) override;             // y = rmsnorm(x) * gamma
    Value operator()(Value x, Value residual);          // y = rmsnorm(x + residual) * gamma; residual_of(y) is x + residual
    Value& gamma() { return params_[0]; }
    float eps() const { return eps_; }

private:
    float eps_;
};

class Sequential : public Module {
public:
    explicit Sequential(const std::vector<Module*>& modules);
    using Module::operator();
    Value operator()(Value x) override;
    const std::vector<Module*>& get_layers() const { return layers_; }

private:
    std::vector<Module*> layers_;
};

}  // namespace ag::nn
