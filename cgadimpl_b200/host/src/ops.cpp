// ops.cpp -- forward node builders of the RMSNorm path and their Value-level wrappers.
// Each builder makes ONE library call where the reference composes several tensor operations;
// node bookkeeping (inputs, tape, child_grad_count, on_node_created) follows the reference.
#include "ad/ops/ops.hpp"

#include <map>
#include <vector>

#include "ad/detail/host_util.hpp"

namespace ag {
namespace detail {

int classify_broadcast(const Tensor& full, const Tensor& b) {
    const auto& fd = full.shape().dims;
    const auto& bd = b.shape().dims;
    if (fd == bd) return AGB_BCAST_FULL;
    if (b.numel() == 1) return AGB_BCAST_SCALAR;
    const int64_t hidden = fd.empty() ? 1 : fd.back();
    // [hidden], [1, hidden], [1, 1, hidden] ...
    if (!bd.empty() && bd.back() == hidden && b.numel() == hidden) return AGB_BCAST_LASTVEC;
    // [..., 1] with the leading dims of `full`
    if (bd.size() == fd.size() && bd.back() == 1 && b.numel() * hidden == full.numel()) {
        bool same = true;
        for (size_t i = 0; i + 1 < fd.size(); ++i) same = same && fd[i] == bd[i];
        if (same) return AGB_BCAST_ROWSTAT;
    }
    throw std::runtime_error("broadcast of these shapes is outside the RMSNorm path "
                             "(supported: same shape, [hidden], [..., 1], scalar)");
}

void* workspace(size_t bytes, const Tensor& like, ag_cuda_stream_t stream) {
    thread_local std::map<std::pair<int, ag_cuda_stream_t>, Tensor> pool;
    // a workspace that is outgrown is retired, not freed: a captured CUDA graph may still point at it
    thread_local std::vector<Tensor> retired;
    Tensor& t = pool[{like.device().index, stream}];
    if (!t.defined() || t.nbytes() < bytes) {
        if (t.defined()) retired.push_back(t);
        StreamGuard g(stream);
        t = Tensor(Shape{{static_cast<int64_t>((bytes + 7) / 8)}},
                   TensorOptions().with_dtype(Dtype::Float64).with_device(like.device()));
    }
    return t.raw();
}

Tensor on_device_of(const Tensor& t, const Tensor& like) {
    if (t.device() == like.device()) return t;
    if (t.numel() != 1) throw std::runtime_error("operands live on different devices");
    return t.to(like.device());
}

namespace {

// Picks the full-shaped operand first; add and mul commute.
struct BinaryPlan {
    const Tensor* full;
    Tensor other;
    int mode;
};
BinaryPlan plan_binary(const Tensor& a, const Tensor& b) {
    const Tensor& full = a.numel() >= b.numel() ? a : b;
    const Tensor& small = a.numel() >= b.numel() ? b : a;
    require_cuda(full, "binary op");
    BinaryPlan p{&full, on_device_of(small, full), 0};
    p.mode = classify_broadcast(full, p.other);
    return p;
}

}  // namespace

Tensor binary_op(int op, const Tensor& a, const Tensor& b, ag_cuda_stream_t stream) {
    StreamGuard g(stream);
    BinaryPlan p = plan_binary(a, b);
    Tensor out(p.full->shape(), ag::options(*p.full).with_req_grad(false));
    const auto rh = rows_hidden(*p.full);
    if (p.mode == AGB_BCAST_FULL && op == 0)
        check_status(agb_residual_add(p.full->raw(), p.other.raw(), out.raw(), out.numel(), agb_dtype(out), stream), "add");
    else if (p.mode == AGB_BCAST_LASTVEC && op == 1)
        check_status(agb_scale_lastdim(p.full->raw(), p.other.raw(), out.raw(), rh.rows, rh.hidden, agb_dtype(out), stream), "mul");
    else
        check_status(agb_binary_broadcast(op, p.full->raw(), p.other.raw(), out.raw(), rh.rows, rh.hidden, p.mode,
                                          agb_dtype(out), stream),
                     op == 0 ? "add" : "mul");
    return out;
}

namespace {
Tensor binary(int op, const Tensor& a, const Tensor& b) { return binary_op(op, a, b, current_stream()); }

void link(const std::shared_ptr<Node>& n, std::initializer_list<std::shared_ptr<Node>> inputs) {
    n->inputs.assign(inputs.begin(), inputs.end());
    for (auto& p : n->inputs)
        if (p) p->child_grad_count++;
    ag::debug::on_node_created(n);
}

}  // namespace

// arithmetic.cpp:11-19
std::shared_ptr<Node> add_nodeops(const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b) {
    auto n = std::make_shared<Node>(binary(0, a->value, b->value), Op::Add, a->requires_grad() || b->requires_grad(), "+");
    link(n, {a, b});
    return n;
}
// arithmetic.cpp:31-39
std::shared_ptr<Node> mul_nodeops(const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b) {
    auto n = std::make_shared<Node>(binary(1, a->value, b->value), Op::Mul, a->requires_grad() || b->requires_grad(), "*");
    link(n, {a, b});
    return n;
}

namespace {
// Forward of the norm into fresh tensors; rstd has the leading dims of x and a trailing 1.
struct NormOut {
    Tensor y, rstd;
};
NormOut norm_forward(const Tensor& x, const Tensor* gamma, float eps) {
    require_cuda(x, "rms");
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(x);
    NormOut o;
    o.y = Tensor(x.shape(), ag::options(x).with_req_grad(false));
    Shape rs = x.shape();
    if (rs.dims.empty()) rs.dims.push_back(1);
    rs.dims.back() = 1;
    o.rstd = Tensor(rs, TensorOptions().with_dtype(Dtype::Float32).with_device(x.device()));
    check_status(agb_rmsnorm_fwd(x.raw(), gamma ? gamma->raw() : nullptr, o.y.raw(), o.rstd.data<float>(), rh.rows,
                                 rh.hidden, eps, agb_dtype(x), current_stream()),
                 "rms forward");
    return o;
}
void check_gamma(const Tensor& x, const Tensor& gamma) {
    const auto rh = rows_hidden(x);
    if (gamma.numel() != rh.hidden || gamma.shape().dims.back() != rh.hidden)
        throw std::runtime_error("rmsnorm: gamma must have shape [hidden] (or [1, hidden])");
    if (gamma.dtype() != x.dtype()) throw std::runtime_error("rmsnorm: gamma and x must have the same dtype");
    require_cuda(gamma, "rmsnorm gamma");
}
}  // namespace

namespace {
struct LayerNormOut {
    Tensor y, mean, var;
};
LayerNormOut layernorm_forward(const Tensor& xv, float eps) {
    require_cuda(xv, "laynor");
    const auto rh = rows_hidden(xv);
    StreamGuard g(current_stream());
    LayerNormOut o;
    o.y = Tensor(xv.shape(), ag::options(xv).with_req_grad(false));
    Shape rs = xv.shape();
    if (rs.dims.empty()) rs.dims.push_back(1);
    rs.dims.back() = 1;
    const auto f32 = TensorOptions().with_dtype(Dtype::Float32).with_device(xv.device());
    o.mean = Tensor(rs, f32);
    o.var = Tensor(rs, f32);
    check_status(agb_layernorm_fwd(xv.raw(), o.y.raw(), o.mean.data<float>(), o.var.data<float>(), rh.rows, rh.hidden, eps,
                                   agb_dtype(xv), current_stream()),
                 "laynor forward");
    return o;
}
}  // namespace

// normalization.cpp:10-22 -- tape = {variance, mean}, both [.., 1] fp32.
std::shared_ptr<Node> laynor_nodeops(const std::shared_ptr<Node>& x) {
    LayerNormOut o = layernorm_forward(x->value, 1e-5f);
    auto n = std::make_shared<Node>(o.y, Op::LayerNorm, x->requires_grad(), "layernor");
    n->eps = 1e-5f;
    n->tape.push_back(std::make_shared<Tensor>(o.var));
    n->tape.push_back(std::make_shared<Tensor>(o.mean));
    link(n, {x});
    return n;
}

// normalization.cpp:23-35 -- eps is fixed at 1e-5 there; tape = {rstd, y}.
std::shared_ptr<Node> rms_nodeops(const std::shared_ptr<Node>& x) {
    NormOut o = norm_forward(x->value, nullptr, 1e-5f);
    auto n = std::make_shared<Node>(o.y, Op::RMSNorm, x->requires_grad(), "rmsnorm");
    n->eps = 1e-5f;
    n->tape.push_back(std::make_shared<Tensor>(o.rstd));
    n->tape.push_back(std::make_shared<Tensor>(o.y));
    link(n, {x});
    return n;
}

// normalization.cpp:36-60 -- scalar gain G, a [1,1] leaf that requires grad, cached per value.
// inputs = {x, G}; tape = {rstd, y_normalized}.  (The reference's VJP / JVP for this op throw; the
// rules here are implemented.)
std::shared_ptr<Node> realrms_nodeops(const std::shared_ptr<Node>& x, float& g_val) {
    static std::mutex mu;
    static std::map<std::pair<float, int>, std::shared_ptr<Node>> cache;
    std::shared_ptr<Node> G;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto key = std::make_pair(g_val, x->value.device().index);
        auto it = cache.find(key);
        if (it != cache.end()) {
            G = it->second;
        } else {
            StreamGuard g(current_stream());
            Tensor gt = Tensor::full(Shape{{1, 1}}, ag::options(x->value).with_req_grad(true), g_val);
            G = std::make_shared<Node>(gt, Op::Leaf, true, "rms_gain");
            cache[key] = G;
        }
    }
    NormOut o = norm_forward(x->value, nullptr, 1e-5f);
    Tensor scaled = binary(1, o.y, G->value);
    auto n = std::make_shared<Node>(scaled, Op::RealRMSNorm, x->requires_grad() || G->requires_grad(), "realrmsnorm");
    n->eps = 1e-5f;
    n->tape.push_back(std::make_shared<Tensor>(o.rstd));
    n->tape.push_back(std::make_shared<Tensor>(o.y));
    link(n, {x, G});
    return n;
}

std::shared_ptr<Node> rmsnorm_nodeops(const std::shared_ptr<Node>& x, const std::shared_ptr<Node>& gamma, float eps) {
    check_gamma(x->value, gamma->value);
    NormOut o = norm_forward(x->value, &gamma->value, eps);
    auto n = std::make_shared<Node>(o.y, Op::RMSNormAffine, x->requires_grad() || gamma->requires_grad(), "rmsnorm_affine");
    n->eps = eps;
    n->tape.push_back(std::make_shared<Tensor>(o.rstd));
    link(n, {x, gamma});
    return n;
}

std::shared_ptr<Node> add_rmsnorm_nodeops(const std::shared_ptr<Node>& x, const std::shared_ptr<Node>& r,
                                          const std::shared_ptr<Node>& gamma, float eps) {
    if (x->value.shape().dims != r->value.shape().dims) throw std::runtime_error("add_rmsnorm: x and r must have the same shape");
    check_gamma(x->value, gamma->value);
    require_cuda(x->value, "add_rmsnorm");
    require_cuda(r->value, "add_rmsnorm");
    const Tensor& xv = x->value;
    const auto rh = rows_hidden(xv);
    Tensor h, y, rstd;
    {
        StreamGuard g(current_stream());
        h = Tensor(xv.shape(), ag::options(xv).with_req_grad(false));
        y = Tensor(xv.shape(), ag::options(xv).with_req_grad(false));
        Shape rs = xv.shape();
        rs.dims.back() = 1;
        rstd = Tensor(rs, TensorOptions().with_dtype(Dtype::Float32).with_device(xv.device()));
        check_status(agb_add_rmsnorm_fwd(xv.raw(), r->value.raw(), gamma->value.raw(), h.raw(), y.raw(), rstd.data<float>(),
                                         rh.rows, rh.hidden, eps, agb_dtype(xv), current_stream()),
                     "add_rmsnorm forward");
    }
    auto hn = std::make_shared<Node>(h, Op::Add, x->requires_grad() || r->requires_grad(), "+");
    link(hn, {x, r});
    auto n = std::make_shared<Node>(y, Op::RMSNormAffine, hn->requires_grad() || gamma->requires_grad(), "rmsnorm_affine");
    n->eps = eps;
    n->tape.push_back(std::make_shared<Tensor>(rstd));
    link(n, {hn, gamma});
    return n;
}

namespace {
Tensor reduce_all(const Tensor& x, int op) {
    require_cuda(x, "reduction");
    StreamGuard g(current_stream());
    Tensor out(Shape{{1}}, ag::options(x).with_req_grad(false));
    const size_t wsb = agb_reduce_all_workspace_bytes(x.numel());
    check_status(agb_reduce_all(op, x.raw(), out.raw(), x.numel(), agb_dtype(x), workspace(wsb, x, current_stream()), wsb,
                                current_stream()),
                 "reduce_all");
    return out;
}
Tensor reduce_axis1(const Tensor& x, int op) {
    require_cuda(x, "row reduction");
    const auto& d = x.shape().dims;
    if (d.size() != 2) throw std::runtime_error("rowsum / rowmax expect a [B, C] tensor (they reduce axis 1)");
    StreamGuard g(current_stream());
    Tensor out(Shape{{d[0], 1}}, ag::options(x).with_req_grad(false));
    check_status(agb_row_reduce(op, x.raw(), out.raw(), d[0], d[1], agb_dtype(x), current_stream()), "row_reduce");
    return out;
}
}  // namespace

// reduction.cpp:9-16
std::shared_ptr<Node> sum_nodeops(const std::shared_ptr<Node>& x) {
    auto n = std::make_shared<Node>(reduce_all(x->value, AGB_REDUCE_SUM), Op::Sum, x->requires_grad(), "sum");
    link(n, {x});
    return n;
}
// reduction.cpp:17-24
std::shared_ptr<Node> mean_all_nodeops(const std::shared_ptr<Node>& x) {
    auto n = std::make_shared<Node>(reduce_all(x->value, AGB_REDUCE_MEAN), Op::MeanAll, x->requires_grad(), "meanall");
    link(n, {x});
    return n;
}
// reduction.cpp:25-32 (axis 1, keepdim)
std::shared_ptr<Node> rowsum_nodeops(const std::shared_ptr<Node>& x) {
    auto n = std::make_shared<Node>(reduce_axis1(x->value, AGB_REDUCE_SUM), Op::RowSum, x->requires_grad(), "rowsum");
    link(n, {x});
    return n;
}
// reduction.cpp:33-40
std::shared_ptr<Node> rowmax_nodeops(const std::shared_ptr<Node>& x) {
    auto n = std::make_shared<Node>(reduce_axis1(x->value, AGB_REDUCE_MAX), Op::RowMax, x->requires_grad(), "rowmax");
    link(n, {x});
    return n;
}

namespace {
Tensor softmax_family_forward(const Tensor& z, bool lse) {
    require_cuda(z, lse ? "logsumexp_row" : "softmax_row");
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(z);
    Shape os = z.shape();
    if (lse) {
        if (os.dims.empty()) os.dims.push_back(1);
        os.dims.back() = 1;
    }
    Tensor out(os, ag::options(z).with_req_grad(false));
    if (lse) check_status(agb_logsumexp_row_fwd(z.raw(), out.raw(), rh.rows, rh.hidden, agb_dtype(z), current_stream()), "logsumexp_row");
    else check_status(agb_softmax_row_fwd(z.raw(), out.raw(), rh.rows, rh.hidden, agb_dtype(z), current_stream()), "softmax_row");
    return out;
}
}  // namespace

// reduction.cpp:42-53
std::shared_ptr<Node> softmax_row_nodeops(const std::shared_ptr<Node>& z) {
    auto n = std::make_shared<Node>(softmax_family_forward(z->value, false), Op::SoftmaxRow, z->requires_grad(), "softmax_row");
    link(n, {z});
    return n;
}
// reduction.cpp:54-66: [.., 1]
std::shared_ptr<Node> logsumexp_row_nodeops(const std::shared_ptr<Node>& z) {
    auto n = std::make_shared<Node>(softmax_family_forward(z->value, true), Op::LogSumExpRow, z->requires_grad(), "logsumexp_row");
    link(n, {z});
    return n;
}

}  // namespace detail

// Recomputes a node's value from its inputs' values -- and its tape, which the rules of the norm
// ops read -- with the same kernels and the same stream the forward used, so the recomputed bits
// equal the originals.  Covers every op of this library's path; cgadimpl/src/ops/ops.cpp:300-386
// covers the elementwise ops and MatMul / Linear and throws for the normalisation ops.
Tensor forward_eval_node(Node* node) {
    using namespace detail;
    if (!node) throw std::runtime_error("forward_eval_node: null node");
    if (node->op == Op::Leaf) return node->value;
    for (auto& p : node->inputs)
        if (!p || p->value.numel() == 0) throw std::runtime_error("forward_eval_node: an input of the node has no value");
    // the builders launch on the thread's current stream: make that the node's stream for the call
    struct CurrentStreamGuard {
        ag_cuda_stream_t prev;
        explicit CurrentStreamGuard(ag_cuda_stream_t s) : prev(current_stream()) { set_current_stream(s); }
        ~CurrentStreamGuard() { set_current_stream(prev); }
    } cs(node->creation_context.stream);
    StreamGuard g(node->creation_context.stream);
    auto in = [&](size_t i) -> const Tensor& { return node->inputs.at(i)->value; };
    auto set_tape = [&](std::initializer_list<Tensor> ts) {
        node->tape.clear();
        for (auto& t : ts) node->tape.push_back(std::make_shared<Tensor>(t));
    };
    switch (node->op) {
        case Op::Add: return binary(0, in(0), in(1));
        case Op::Mul: return binary(1, in(0), in(1));
        case Op::RMSNorm: {
            NormOut o = norm_forward(in(0), nullptr, node->eps);
            set_tape({o.rstd, o.y});
            return o.y;
        }
        case Op::RealRMSNorm: {
            NormOut o = norm_forward(in(0), nullptr, node->eps);
            set_tape({o.rstd, o.y});
            return binary(1, o.y, in(1));
        }
        case Op::RMSNormAffine: {
            NormOut o = norm_forward(in(0), &in(1), node->eps);
            set_tape({o.rstd});
            return o.y;
        }
        case Op::LayerNorm: {
            LayerNormOut o = layernorm_forward(in(0), node->eps);
            set_tape({o.var, o.mean});
            return o.y;
        }
        case Op::SoftmaxRow: return softmax_family_forward(in(0), false);
        case Op::LogSumExpRow: return softmax_family_forward(in(0), true);
        case Op::Sum: return reduce_all(in(0), AGB_REDUCE_SUM);
        case Op::MeanAll: return reduce_all(in(0), AGB_REDUCE_MEAN);
        case Op::RowSum: return reduce_axis1(in(0), AGB_REDUCE_SUM);
        case Op::RowMax: return reduce_axis1(in(0), AGB_REDUCE_MAX);
        default:
            throw std::runtime_error(std::string("forward_eval_node: unsupported op for recompute: ") + op_name(node->op));
    }
}
Tensor forward_eval_node(const std::shared_ptr<Node>& node) { return forward_eval_node(node.get()); }

Value add(const Value& a, const Value& b) { return Value(detail::add_nodeops(a.node, b.node)); }
Value mul(const Value& a, const Value& b) { return Value(detail::mul_nodeops(a.node, b.node)); }
Value laynor(const Value& x) { return Value(detail::laynor_nodeops(x.node)); }
Value rms(const Value& x) { return Value(detail::rms_nodeops(x.node)); }
Value realrms(const Value& x, float g) { return Value(detail::realrms_nodeops(x.node, g)); }
Value sum(const Value& x) { return Value(detail::sum_nodeops(x.node)); }
Value mean_all(const Value& x) { return Value(detail::mean_all_nodeops(x.node)); }
Value rowsum(const Value& x) { return Value(detail::rowsum_nodeops(x.node)); }
Value rowmax(const Value& x) { return Value(detail::rowmax_nodeops(x.node)); }
Value softmax_row(const Value& z) { return Value(detail::softmax_row_nodeops(z.node)); }
Value logsumexp_row(const Value& z) { return Value(detail::logsumexp_row_nodeops(z.node)); }
Value rmsnorm(const Value& x, const Value& gamma, float eps) { return Value(detail::rmsnorm_nodeops(x.node, gamma.node, eps)); }
Value add_rmsnorm(const Value& x, const Value& r, const Value& gamma, float eps) {
    return Value(detail::add_rmsnorm_nodeops(x.node, r.node, gamma.node, eps));
}
Value residual_of(const Value& y) {
    if (!y.node || y.node->op != Op::RMSNormAffine || y.node->inputs.empty() || y.node->inputs[0]->op != Op::Add)
        throw std::runtime_error("residual_of: not the result of add_rmsnorm");
    return Value(y.node->inputs[0]);
}

}  // namespace ag
