// rules_vjp.cpp -- VJP rules of the RMSNorm path, one `void vjp_X(Node*, const Tensor& gy)` per op
// as in cgadimpl/src/autodiff/autodiff_vjp_ops.cpp, and the vjp_lookup table (:506-513).
// Every rule launches on the node's creation stream (the reference's current_stream() is
// thread-local and therefore null in the worker threads of the parallel backward).
#define AG_EXPOSE_AUTODIFF_RULES
#include "ad/detail/autodiff_ops.hpp"
#include "ad/detail/host_util.hpp"

namespace ag {
namespace detail {
namespace {

ag_cuda_stream_t rule_stream(Node* n) { return n->creation_context.stream; }

// P.grad += reduce_for_broadcast(g * a, P.value)   (a may be null: plain g)
// autodiff_vjp_ops.cpp:15-35 picks the axes to sum from the shapes; here the shape class does.
void accumulate_reduced(Node* P, const Tensor& g, const Tensor* a, ag_cuda_stream_t st) {
    std::unique_lock<std::mutex> lock(P->grad_mutex);
    bool first = false;
    Tensor& G = P->open_grad(&first);   // has P's shape even when P's value has been dropped
    int mode;
    try {
        mode = classify_broadcast(g, G);
    } catch (...) {
        if (first) P->grad_live = false;
        throw;
    }
    if (mode == AGB_BCAST_FULL) {
        if (first) P->grad_live = false;  // accumulate_grad opens the slot itself
        lock.unlock();
        P->accumulate_grad(a ? binary_op(1, g, *a, st) : g);
        return;
    }
    require_cuda(G, "broadcast gradient");
    const auto rh = rows_hidden(g);
    const size_t wsb = agb_mul_reduce_workspace_bytes(rh.rows, rh.hidden);
    void* ws = workspace(wsb, g, st);
    check_status(agb_mul_reduce(g.raw(), a ? a->raw() : nullptr, G.raw(), rh.rows, rh.hidden, mode, /*accumulate=*/first ? 0 : 1,
                                ws, wsb, agb_dtype(g), st),
                 "reduce_for_broadcast");
}

// X.grad += rms_vjp(x, gamma, rstd, gy): dx_add == dx == X.grad fuses accumulate_grad's `+=`; the FIRST
// contribution to X.grad is written instead (dx_add = NULL), so the buffer is neither zero-filled nor read.
// dgamma (fp32) is written to / accumulates into G->grad when G is given.
void norm_backward(Node* X, Node* G, const Tensor& rstd, const Tensor& gy, ag_cuda_stream_t st) {
    const Tensor& x = X->value;
    const auto rh = rows_hidden(x);
    const bool want_dx = X->requires_grad();
    const bool want_dg = G && G->requires_grad();
    if (!want_dx && !want_dg) return;
    if (want_dg && G->value.dtype() != Dtype::Float32)
        throw std::runtime_error("rmsnorm backward: dgamma is produced in fp32; a non-fp32 gamma node cannot "
                                 "receive it through the graph API (use agb_rmsnorm_bwd directly)");
    size_t wsb = 0;
    void* ws = nullptr;
    if (want_dg) {
        wsb = agb_rmsnorm_bwd_workspace_bytes(rh.rows, rh.hidden, agb_dtype(x));
        ws = workspace(wsb, x, st);
    }
    Tensor scratch_dx;
    if (!want_dx) scratch_dx = Tensor(x.shape(), ag::options(x).with_req_grad(false));
    std::unique_lock<std::mutex> lx(X->grad_mutex, std::defer_lock), lg;
    if (want_dx) lx.lock();
    if (want_dg) lg = std::unique_lock<std::mutex>(G->grad_mutex);
    bool first_dx = false, first_dg = false;
    Tensor* gx = want_dx ? &X->open_grad(&first_dx) : nullptr;
    Tensor* gg = want_dg ? &G->open_grad(&first_dg) : nullptr;
    check_status(agb_rmsnorm_bwd(x.raw(), G ? G->value.raw() : nullptr, rstd.data<float>(), gy.raw(),
                                 want_dx && !first_dx ? gx->raw() : nullptr, want_dx ? gx->raw() : scratch_dx.raw(),
                                 want_dg ? gg->raw() : nullptr, AGB_F32, /*accumulate_dgamma=*/first_dg ? 0 : 1, ws, wsb,
                                 rh.rows, rh.hidden, agb_dtype(x), st),
                 "rmsnorm backward");
}

[[noreturn]] void not_on_path(const char* what, const char* name) {
    throw std::runtime_error(std::string(what) + " for op '" + name + "' is not part of the RMSNorm path of this library");
}

}  // namespace

void vjp_Leaf(Node*, const Tensor&) {}

// autodiff_vjp_ops.cpp:40-45
void vjp_Add(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    for (int i = 0; i < 2; ++i) {
        Node* P = n->inputs[i].get();
        if (P->requires_grad()) accumulate_reduced(P, gy, nullptr, rule_stream(n));
    }
}

// autodiff_vjp_ops.cpp:54-59
void vjp_Mul(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* A = n->inputs[0].get();
    Node* B = n->inputs[1].get();
    if (A->requires_grad()) {
        const Tensor b = on_device_of(B->value, gy);
        if (classify_broadcast(gy, A->value) == AGB_BCAST_FULL) A->accumulate_grad(binary_op(1, gy, b, rule_stream(n)));
        else accumulate_reduced(A, gy, &b, rule_stream(n));
    }
    if (B->requires_grad()) {
        const Tensor a = on_device_of(A->value, gy);
        if (classify_broadcast(gy, B->value) == AGB_BCAST_FULL) B->accumulate_grad(binary_op(1, gy, a, rule_stream(n)));
        else accumulate_reduced(B, gy, &a, rule_stream(n));
    }
}

// autodiff_vjp_ops.cpp:351-365; X.grad += dx fused through dx_add == dx == X.grad
void vjp_LayerNorm(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* X = n->inputs[0].get();
    if (!X->requires_grad()) return;
    const auto rh = rows_hidden(X->value);
    std::lock_guard<std::mutex> lock(X->grad_mutex);
    bool first = false;
    Tensor& G = X->open_grad(&first);
    check_status(agb_layernorm_bwd(X->value.raw(), n->tape[1]->data<float>(), n->tape[0]->data<float>(), gy.raw(),
                                   first ? nullptr : G.raw(), G.raw(), rh.rows, rh.hidden, n->eps, agb_dtype(X->value),
                                   rule_stream(n)),
                 "laynor backward");
}

// autodiff_vjp_ops.cpp:368-377
void vjp_RMSNorm(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    norm_backward(n->inputs[0].get(), nullptr, *n->tape[0], gy, rule_stream(n));
}

void vjp_RMSNormAffine(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    norm_backward(n->inputs[0].get(), n->inputs[1].get(), *n->tape[0], gy, rule_stream(n));
}

// The reference throws here (autodiff_vjp_ops.cpp:379-381).  y = yhat * G with a scalar G:
// dyhat = gy * G -> through the norm;  dG = sum(gy * yhat).
void vjp_RealRMSNorm(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* X = n->inputs[0].get();
    Node* G = n->inputs[1].get();
    if (X->requires_grad()) {
        Tensor dyhat = binary_op(1, gy, G->value, rule_stream(n));
        norm_backward(X, nullptr, *n->tape[0], dyhat, rule_stream(n));
    }
    if (G->requires_grad()) accumulate_reduced(G, gy, n->tape[1].get(), rule_stream(n));
}

// autodiff_vjp_ops.cpp:399-402: X.grad += gy (scalar broadcast)
void vjp_Sum(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* X = n->inputs[0].get();
    if (X->requires_grad()) X->accumulate_grad(gy);
}
// autodiff_vjp_ops.cpp:403-409: X.grad += gy * (1/numel)
void vjp_MeanAll(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* X = n->inputs[0].get();
    if (!X->requires_grad()) return;
    std::lock_guard<std::mutex> lock(X->grad_mutex);
    bool first = false;
    Tensor& G = X->open_grad(&first);
    if (first) G.zero_();
    const float scale = 1.0f / static_cast<float>(G.numel());
    const auto rh = rows_hidden(G);
    const Tensor src = on_device_of(gy, G);
    check_status(agb_accumulate_broadcast(G.raw(), src.raw(), rh.rows, rh.hidden, AGB_BCAST_SCALAR, scale,
                                          agb_dtype(G), rule_stream(n)),
                 "vjp_MeanAll");
}
// autodiff_vjp_ops.cpp:411-414: X.grad += gy ([B,1] broadcast)
void vjp_RowSum(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* X = n->inputs[0].get();
    if (X->requires_grad()) X->accumulate_grad(gy);
}
// autodiff_vjp_ops.cpp:416-418 throws as well
void vjp_RowMax(Node*, const Tensor&) { throw std::runtime_error("VJP for RowMax not implemented yet!"); }

// autodiff_vjp_ops.cpp:421-428: Z.grad += y * (gy - sum(y*gy)); the `+=` is fused (dz_add == dz == Z.grad)
void vjp_SoftmaxRow(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* Z = n->inputs[0].get();
    if (!Z->requires_grad()) return;
    const auto rh = rows_hidden(n->value);
    std::lock_guard<std::mutex> lock(Z->grad_mutex);
    bool first = false;
    Tensor& G = Z->open_grad(&first);
    check_status(agb_softmax_row_bwd(n->value.raw(), gy.raw(), first ? nullptr : G.raw(), G.raw(), rh.rows, rh.hidden,
                                     agb_dtype(n->value), rule_stream(n)),
                 "vjp_SoftmaxRow");
}
// autodiff_vjp_ops.cpp:430-440: softmax(z) recomputed from Z.value; Z.grad += gy[.., 1] * softmax(z)
void vjp_LogSumExpRow(Node* n, const Tensor& gy) {
    StreamGuard g(rule_stream(n));
    Node* Z = n->inputs[0].get();
    if (!Z->requires_grad()) return;
    const auto rh = rows_hidden(Z->value);
    if (gy.numel() != rh.rows) throw std::runtime_error("vjp_LogSumExpRow: gy must have one entry per row");
    std::lock_guard<std::mutex> lock(Z->grad_mutex);
    bool first = false;
    Tensor& G = Z->open_grad(&first);
    check_status(agb_logsumexp_row_bwd(Z->value.raw(), gy.raw(), first ? nullptr : G.raw(), G.raw(), rh.rows, rh.hidden,
                                       agb_dtype(Z->value), rule_stream(n)),
                 "vjp_LogSumExpRow");
}

#define AG_NOT_ON_PATH(name) \
    void vjp_##name(Node*, const Tensor&) { not_on_path("VJP", #name); }
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

VjpFn vjp_lookup(Op op) {
    switch (op) {
#define OP(name, arity, str) \
    case Op::name: return &detail::vjp_##name;
#include "ad/detail/ops.def"
#undef OP
        default: return nullptr;
    }
}

}  // namespace ag
