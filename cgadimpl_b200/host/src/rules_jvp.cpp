// rules_jvp.cpp -- JVP rules of the RMSNorm path (cgadimpl/src/autodiff/autodiff_jvp_ops.cpp) and
// the jvp_lookup table (:501-508).  jvp_RMSNorm is the CORRECTED form: the reference divides by
// tape[0] as if it held rms, while the forward stores rstd there (normalization.cpp:26,29 against
// autodiff_jvp_ops.cpp:370,378), which makes its result wrong by 1/rstd^2 per row.
#define AG_EXPOSE_AUTODIFF_RULES
#include "ad/detail/autodiff_ops.hpp"
#include "ad/detail/host_util.hpp"

namespace ag {
namespace detail {
namespace {

using TangentOf = std::function<const Tensor&(Node*)>;

// Tangent of p, or zeros of p's shape when none was recorded (the engine records one per node, so
// this only happens when a rule is called by hand).
Tensor tangent(const TangentOf& t, Node* p) {
    const Tensor& v = t(p);
    if (v.defined() && v.numel() == p->value.numel()) return v;
    StreamGuard g(current_stream());
    return Tensor::zeros(p->value.shape(), ag::options(p->value).with_req_grad(false));
}

Tensor norm_jvp(Node* X, Node* G, const Tensor& rstd, const Tensor& tx, const Tensor* tgamma) {
    const Tensor& x = X->value;
    require_cuda(x, "rms jvp");
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(x);
    Tensor out(x.shape(), ag::options(x).with_req_grad(false));
    check_status(agb_rmsnorm_jvp(x.raw(), G ? G->value.raw() : nullptr, rstd.data<float>(), tx.raw(),
                                 tgamma ? tgamma->raw() : nullptr, out.raw(), rh.rows, rh.hidden, agb_dtype(x),
                                 current_stream()),
                 "rmsnorm jvp");
    return out;
}

Tensor reduce_tangent_all(const Tensor& t, int op) {
    StreamGuard g(current_stream());
    Tensor out(Shape{{1}}, ag::options(t).with_req_grad(false));
    const size_t wsb = agb_reduce_all_workspace_bytes(t.numel());
    check_status(agb_reduce_all(op, t.raw(), out.raw(), t.numel(), agb_dtype(t), workspace(wsb, t, current_stream()), wsb,
                                current_stream()),
                 "jvp reduce");
    return out;
}

[[noreturn]] Tensor not_on_path(const char* name) {
    throw std::runtime_error(std::string("JVP for op '") + name + "' is not part of the RMSNorm path of this library");
}

}  // namespace

Tensor jvp_Leaf(Node* n, const TangentOf& t) { return tangent(t, n); }

// autodiff_jvp_ops.cpp:16-19
Tensor jvp_Add(Node* n, const TangentOf& t) {
    return binary_op(0, tangent(t, n->inputs[0].get()), tangent(t, n->inputs[1].get()), current_stream());
}
// autodiff_jvp_ops.cpp:24-31: (T(A) * B) + (A * T(B))
Tensor jvp_Mul(Node* n, const TangentOf& t) {
    Node* A = n->inputs[0].get();
    Node* B = n->inputs[1].get();
    Tensor l = binary_op(1, tangent(t, A), B->value, current_stream());
    Tensor r = binary_op(1, A->value, tangent(t, B), current_stream());
    return binary_op(0, l, r, current_stream());
}
// The reference throws here (autodiff_jvp_ops.cpp:361-363).  ty = std_inv * ((t - mean t) - y * mean(y * (t - mean t)))
// from the node's own value y and tape[0] = variance.
Tensor jvp_LayerNorm(Node* n, const TangentOf& t) {
    const Tensor tx = tangent(t, n->inputs[0].get());
    require_cuda(n->value, "laynor jvp");
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(n->value);
    Tensor out(n->value.shape(), ag::options(n->value).with_req_grad(false));
    check_status(agb_layernorm_jvp(n->value.raw(), tx.raw(), n->tape[0]->data<float>(), out.raw(), rh.rows, rh.hidden, n->eps,
                                   agb_dtype(n->value), current_stream()),
                 "laynor jvp");
    return out;
}
// autodiff_jvp_ops.cpp:366-379, corrected
Tensor jvp_RMSNorm(Node* n, const TangentOf& t) {
    Node* X = n->inputs[0].get();
    return norm_jvp(X, nullptr, *n->tape[0], tangent(t, X), nullptr);
}
Tensor jvp_RMSNormAffine(Node* n, const TangentOf& t) {
    Node* X = n->inputs[0].get();
    Node* G = n->inputs[1].get();
    const Tensor tg = tangent(t, G);
    return norm_jvp(X, G, *n->tape[0], tangent(t, X), &tg);
}
// The reference throws (autodiff_jvp_ops.cpp:380-382).  ty = tyhat*G + yhat*tG.
Tensor jvp_RealRMSNorm(Node* n, const TangentOf& t) {
    Node* X = n->inputs[0].get();
    Node* G = n->inputs[1].get();
    Tensor tyhat = norm_jvp(X, nullptr, *n->tape[0], tangent(t, X), nullptr);
    Tensor l = binary_op(1, tyhat, G->value, current_stream());
    Tensor r = binary_op(1, *n->tape[1], tangent(t, G), current_stream());
    return binary_op(0, l, r, current_stream());
}
// autodiff_jvp_ops.cpp:390-397
Tensor jvp_Sum(Node* n, const TangentOf& t) { return reduce_tangent_all(tangent(t, n->inputs[0].get()), AGB_REDUCE_SUM); }
Tensor jvp_MeanAll(Node* n, const TangentOf& t) { return reduce_tangent_all(tangent(t, n->inputs[0].get()), AGB_REDUCE_MEAN); }
// autodiff_jvp_ops.cpp:400-403: sum over the last dimension, keepdim
Tensor jvp_RowSum(Node* n, const TangentOf& t) {
    const Tensor tx = tangent(t, n->inputs[0].get());
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(tx);
    Shape s = tx.shape();
    s.dims.back() = 1;
    Tensor out(s, ag::options(tx).with_req_grad(false));
    check_status(agb_row_reduce(AGB_REDUCE_SUM, tx.raw(), out.raw(), rh.rows, rh.hidden, agb_dtype(tx), current_stream()),
                 "jvp_RowSum");
    return out;
}
// autodiff_jvp_ops.cpp:404-409 throws as well
Tensor jvp_RowMax(Node*, const TangentOf&) {
    throw std::runtime_error("JVP for RowMax cannot be implemented without argmax or comparison ops in the tensor library.");
}

// autodiff_jvp_ops.cpp:411-420: y * (tZ - sum(y*tZ))
Tensor jvp_SoftmaxRow(Node* n, const TangentOf& t) {
    const Tensor tz = tangent(t, n->inputs[0].get());
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(n->value);
    Tensor out(n->value.shape(), ag::options(n->value).with_req_grad(false));
    check_status(agb_softmax_row_bwd(n->value.raw(), tz.raw(), nullptr, out.raw(), rh.rows, rh.hidden, agb_dtype(n->value),
                                     current_stream()),
                 "jvp_SoftmaxRow");
    return out;
}
// autodiff_jvp_ops.cpp:421-434: sum(softmax(z) * tZ) per row, [.., 1]
Tensor jvp_LogSumExpRow(Node* n, const TangentOf& t) {
    Node* Z = n->inputs[0].get();
    const Tensor tz = tangent(t, Z);
    StreamGuard g(current_stream());
    const auto rh = rows_hidden(Z->value);
    Tensor out(n->value.shape(), ag::options(Z->value).with_req_grad(false));
    check_status(agb_logsumexp_row_jvp(Z->value.raw(), tz.raw(), out.raw(), rh.rows, rh.hidden, agb_dtype(Z->value),
                                       current_stream()),
                 "jvp_LogSumExpRow");
    return out;
}

#define AG_NOT_ON_PATH(name) \
    Tensor jvp_##name(Node*, const TangentOf&) { not_on_path(#name); }
AG_NOT_ON_PATH(Sub) AG_NOT_ON_PATH(Div) AG_NOT_ON_PATH(Exp) AG_NOT_ON_PATH(Log) AG_NOT_ON_PATH(Sqrt)
AG_NOT_ON_PATH(Reciprocal) AG_NOT_ON_PATH(Sign) AG_NOT_ON_PATH(Abs) AG_NOT_ON_PATH(Pow) AG_NOT_ON_PATH(Sin)
AG_NOT_ON_PATH(Cos) AG_NOT_ON_PATH(Tan) AG_NOT_ON_PATH(Sinh) AG_NOT_ON_PATH(Cosh) AG_NOT_ON_PATH(Asin)
AG_NOT_ON_PATH(Acos) AG_NOT_ON_PATH(Atan) AG_NOT_ON_PATH(ASinh) AG_NOT_ON_PATH(ACosh) AG_NOT_ON_PATH(ATanh)
AG_NOT_ON_PATH(Relu) AG_NOT_ON_PATH(Sigmoid) AG_NOT_ON_PATH(Tanh) AG_NOT_ON_PATH(Softplus) AG_NOT_ON_PATH(GELU)
AG_NOT_ON_PATH(SiLU) AG_NOT_ON_PATH(Mish) AG_NOT_ON_PATH(LeakyRelu) AG_NOT_ON_PATH(Gaus) AG_NOT_ON_PATH(Parcon)
AG_NOT_ON_PATH(LiSHT) AG_NOT_ON_PATH(MatMul)
AG_NOT_ON_PATH(Transpose) AG_NOT_ON_PATH(Linear) AG_NOT_ON_PATH(FMA) AG_NOT_ON_PATH(Dyntanh)
AG_NOT_ON_PATH(Attention) AG_NOT_ON_PATH(SWIGLU) AG_NOT_ON_PATH(CeWithLogits) AG_NOT_ON_PATH(KLDivergence)
AG_NOT_ON_PATH(MSELoss) AG_NOT_ON_PATH(MAELoss)
#undef AG_NOT_ON_PATH

}  // namespace detail

JvpFn jvp_lookup(Op op) {
    switch (op) {
#define OP(name, arity, str) \
    case Op::name: return &detail::jvp_##name;
#include "ad/detail/ops.def"
#undef OP
        default: return nullptr;
    }
}

}  // namespace ag
