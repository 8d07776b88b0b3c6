// optim.cpp -- see optim.hpp.
#include "optim.hpp"

#include <cmath>

#include "ad/detail/host_util.hpp"

namespace ag {

void SGD(const Value& root, const Tensor*, float learning_rate) {
    for (Node* n : topo_from(root.node.get())) {
        if (n->op != Op::Leaf || !n->requires_grad()) continue;
        detail::require_cuda(n->value, "SGD");
        detail::check_status(agb_sgd_step(n->value.raw(), n->materialized_grad().raw(), n->value.numel(), learning_rate,
                                          detail::agb_dtype(n->value), n->creation_context.stream),
                             "SGD");
    }
}

Adam::Adam(const std::vector<Value>& params, float alpha, float beta1, float beta2, float epsilon)
    : params_(params), alpha_(alpha), beta1_(beta1), beta2_(beta2), epsilon_(epsilon), t_(0) {
    for (const auto& p : params_) {
        Node* n = p.node.get();
        if (!n->requires_grad()) continue;
        if (n->value.dtype() != Dtype::Float32) throw std::runtime_error("Adam: fp32 parameters only");
        detail::StreamGuard g(n->creation_context.stream);
        m_[n] = Tensor::zeros(n->value.shape(), ag::options(n->value).with_req_grad(false));
        v_[n] = Tensor::zeros(n->value.shape(), ag::options(n->value).with_req_grad(false));
    }
}

void Adam::step() {
    t_++;
    // the reference's host-side scalars, optim.cpp:34-36, 64
    const float bias_corr1 = 1.0f - std::pow(beta1_, t_);
    const float bias_corr2 = 1.0f - std::pow(beta2_, t_);
    const float alpha_eff = alpha_ * std::sqrt(bias_corr2) / bias_corr1;
    const float eps_eff = epsilon_ * std::sqrt(bias_corr2);
    for (const auto& p : params_) {
        Node* n = p.node.get();
        if (!n->requires_grad()) continue;
        detail::require_cuda(n->value, "Adam");
        detail::check_status(agb_adam_step(n->value.data<float>(), n->materialized_grad().data<float>(), m_[n].data<float>(),
                                           v_[n].data<float>(), n->value.numel(), beta1_, beta2_, alpha_eff, eps_eff,
                                           n->creation_context.stream),
                             "Adam::step");
    }
}

void Adam::zero_grad() {
    for (const auto& p : params_) {
        Node* n = p.node.get();
        if (n->requires_grad()) {
            std::lock_guard<std::mutex> lock(n->grad_mutex);
            n->grad_live = false;
        }
    }
}

}  // namespace ag
