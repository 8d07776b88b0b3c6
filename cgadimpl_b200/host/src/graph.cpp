// graph.cpp -- Node / Value / topological order (cgadimpl/src/core/graph.cpp:17-121).
#include "ad/core/graph.hpp"

#include <unordered_set>

#include "ad/detail/host_util.hpp"

namespace ag {

Node::Node(const Tensor& v, Op op_, bool req_grad, const char* nm)
    : value(v), debug_name(nm), op(op_), is_leaf(op_ == Op::Leaf), requires_grad_flag_(req_grad) {
    creation_context.stream = current_stream();
    creation_context.device = v.device();
    // No gradient buffer yet: see "Lazy gradients" in graph.hpp (the reference zero-fills one here, graph.cpp:36).
}

Tensor& Node::open_grad(bool* first) {
    const bool gone = value_released && value.numel() == 0;  // activation dropped by careful deletion
    const Shape& want = gone ? released_shape : value.shape();
    if (!grad.defined() || grad.numel() != want.numel()) {
        grad = Tensor(want, (gone ? released_options : ag::options(value)).with_req_grad(false));
        grad_live = false;
    }
    *first = !grad_live;
    grad_live = true;
    return grad;
}

Tensor& Node::materialized_grad() {
    std::lock_guard<std::mutex> lock(grad_mutex);
    if (!requires_grad_flag_) return grad;
    detail::StreamGuard g(creation_context.stream);
    bool first = false;
    Tensor& out = open_grad(&first);
    if (first) out.zero_();
    return out;
}

void Node::accumulate_grad(const Tensor& c) {
    std::lock_guard<std::mutex> lock(grad_mutex);
    bool first = false;
    open_grad(&first);
    if (c.numel() == 0) {
        if (first) grad.zero_();
        return;
    }
    if (!grad.is_cuda()) {
        // CPU nodes are scalar literals and tiny test inputs: plain loop, fp32 only
        if (grad.dtype() != Dtype::Float32 || c.is_cuda() || (c.numel() != grad.numel() && c.numel() != 1))
            throw std::runtime_error("accumulate_grad: unsupported CPU gradient");
        float* g = grad.data<float>();
        const float* s = c.data<float>();
        for (int64_t i = 0; i < grad.numel(); ++i) g[i] = (first ? 0.0f : g[i]) + s[c.numel() == 1 ? 0 : i];
        return;
    }
    const Tensor src = detail::on_device_of(c, grad);
    const auto rh = detail::rows_hidden(grad);
    const int mode = detail::classify_broadcast(grad, src);
    ag_cuda_stream_t st = reinterpret_cast<ag_cuda_stream_t>(OwnTensor::cuda::getCurrentStream());
    if (first && mode == AGB_BCAST_FULL && src.dtype() == grad.dtype()) {
        grad.copy_(src);        // the first contribution is the gradient
        return;
    }
    if (first) grad.zero_();    // a broadcast first contribution: clear, then add as below
    if (mode == AGB_BCAST_FULL)
        detail::check_status(agb_vjp_add(grad.raw(), nullptr, src.raw(), grad.numel(), detail::agb_dtype(grad), st),
                             "accumulate_grad");
    else
        detail::check_status(agb_accumulate_broadcast(grad.raw(), src.raw(), rh.rows, rh.hidden, mode, 1.0f,
                                                      detail::agb_dtype(grad), st),
                             "accumulate_grad");
}

Tensor& Value::val() { return node->value; }
const Tensor& Value::val() const { return node->value; }
Tensor& Value::grad() { return node->materialized_grad(); }
const Tensor& Value::grad() const { return node->materialized_grad(); }
Value::Value() = default;
Value::Value(std::shared_ptr<Node> n) : node(std::move(n)) {}
Value::Value(float v) {
    node = std::make_shared<Node>(Tensor::full(Shape{{1}}, TensorOptions(), v), Op::Leaf, false, "scalar_literal");
}
const std::vector<int64_t>& Value::shape() const { return node->shape(); }
std::pair<int, int> Value::shape_2d() const {
    const auto& d = node->shape();
    if (d.empty()) return {0, 0};
    if (d.size() == 1) return {1, static_cast<int>(d[0])};
    return {static_cast<int>(d[0]), static_cast<int>(d[1])};
}

// Iterative post-order DFS (the reference recurses through a std::function, graph.cpp:77-83, which
// overflows the stack on graphs a few tens of thousands of nodes deep).
std::vector<Node*> topo_from(Node* root) {
    std::vector<Node*> order;
    if (!root) return order;
    std::unordered_set<Node*> seen;
    std::vector<std::pair<Node*, size_t>> stack;
    stack.emplace_back(root, 0);
    seen.insert(root);
    while (!stack.empty()) {
        auto& [n, i] = stack.back();
        if (i < n->inputs.size()) {
            Node* p = n->inputs[i++].get();
            if (p && seen.insert(p).second) stack.emplace_back(p, 0);
        } else {
            order.push_back(n);
            stack.pop_back();
        }
    }
    return order;
}

}  // namespace ag
