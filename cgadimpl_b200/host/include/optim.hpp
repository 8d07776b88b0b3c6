// optim.hpp -- ag::SGD and ag::Adam with the interface of cgadimpl/include/optim.hpp:18-37.  Each
// parameter is updated by one library kernel that keeps the reference's rounding points
// (cgadimpl/src/optimizer/optim.cpp:12-19 and :33-72).
#pragma once
#include <unordered_map>
#include <vector>

#include "ad/autodiff/autodiff.hpp"
#include "tensor.hpp"

namespace ag {

// Updates every leaf that requires grad under `root`: value += -learning_rate * grad.
// (grad_seed is unused, as in the reference; the default learning rate is the reference's.)
void SGD(const Value& root, const Tensor* grad_seed = nullptr, float learning_rate = 100);

class Adam {
public:
    Adam(const std::vector<Value>& params, float alpha = 0.001, float beta1 = 0.9, float beta2 = 0.999,
         float epsilon = 1e-8);
    void step();
    void zero_grad();
    int steps() const { return t_; }

private:
    std::vector<Value> params_;
    float alpha_, beta1_, beta2_, epsilon_;
    int t_;
    std::unordered_map<Node*, Tensor> m_, v_;
};

}  // namespace ag
