// ref_driver.cpp -- TEST INFRASTRUCTURE.  A C interface that drives the REFERENCE's own code for
// the RMSNorm path (its op builders in cgadimpl/src/ops, its autodiff engine and rules in
// cgadimpl/src/core and src/autodiff, compiled from the reference tree as they are) over the
// stand-in tensor library in this directory.  Used to validate oracle/agb_oracle.c and as the CPU
// arm of the benchmark.  Also defines the few symbols of the reference that live in files which
// are not compiled here (tracing hooks, checkpoint recompute).
#ifdef _OPENMP
#include <omp.h>
#endif
#include <chrono>
#include <cstring>
#include <unordered_map>

#include "ad/autodiff/autodiff.hpp"
#include "ad/autodiff/checkpoint.hpp"
#include "ad/detail/autodiff_ops.hpp"
#include "ad/ops/nodeops.hpp"
#include "ad/utils/debug.hpp"
#include "optim.hpp"

// ---- symbols of reference files that are not part of the path ------------------------------
namespace ag {
namespace debug {
void on_node_created(const std::shared_ptr<Node>&) {}   // cgadimpl/src/tools/debug.cpp:96 (tracing off)
void on_backprop_step(Node*, const Tensor&) {}
void on_jvp_step(Node*) {}
}  // namespace debug
namespace checkpoint_impl {
bool recompute_subgraph(const std::shared_ptr<Node>&) { return false; }  // no node here is a checkpoint
}
}  // namespace ag

namespace {
using namespace ag;

Tensor from_host(const float* p, std::vector<int64_t> dims, bool req) {
    Tensor t(Shape{dims}, TensorOptions().with_req_grad(req));
    if (t.numel()) std::memcpy(t.data<float>(), p, sizeof(float) * t.numel());
    return t;
}
void to_host(const Tensor& t, float* p) {
    if (p && t.numel()) std::memcpy(p, t.data<float>(), sizeof(float) * t.numel());
}
std::shared_ptr<Node> leaf(const Tensor& t, const char* name) {
    return std::make_shared<Node>(t, Op::Leaf, t.requires_grad(), name);
}
}  // namespace

extern "C" {

void cgadimpl_ref_set_reduce_fp64(int on) { OwnTensor::shim::reduce_in_fp64 = on != 0; }

// y = mul(rms(x), gamma) (gamma NULL: y = rms(x)); backward with seed gy.  eps is the reference's
// hard-coded 1e-5.  gamma_2d: give gamma the shape [1,H] (as the reference's tests do) or [H].
int cgadimpl_ref_rmsnorm_fwd_bwd(const float* x, const float* gamma, const float* gy, float* y, float* rstd, float* dx,
                                 float* dgamma, int64_t R, int64_t H, int gamma_2d, int parallel_backward) {
    try {
        auto X = leaf(from_host(x, {R, H}, true), "x");
        std::shared_ptr<Node> G, out;
        auto n = detail::rms_nodeops(X);
        out = n;
        if (gamma) {
            G = leaf(from_host(gamma, gamma_2d ? std::vector<int64_t>{1, H} : std::vector<int64_t>{H}, true), "gamma");
            out = detail::mul_nodeops(n, G);
        }
        Tensor seed = from_host(gy, {R, H}, false);
        backward(Value(out), &seed, parallel_backward != 0);
        to_host(out->value, y);
        to_host(*n->tape[0], rstd);
        to_host(X->grad, dx);
        if (G) to_host(G->grad, dgamma);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

// The residual stack of the benchmark's configuration 4 as the reference would run it:
// h_l = add(x_l, r_l); y_l = mul(rms(h_l), gamma_l); x_{l+1} = h_l; r_{l+1} = y_l; backward from g.
int cgadimpl_ref_residual_stack(const float* x, const float* r, const float* gammas, const float* g, float* y_last,
                                float* dx0, float* dr0, float* dgammas, int64_t R, int64_t H, int L) {
    try {
        auto X = leaf(from_host(x, {R, H}, true), "x"), Rr = leaf(from_host(r, {R, H}, true), "r");
        std::vector<std::shared_ptr<Node>> G;
        std::shared_ptr<Node> xl = X, rl = Rr, yl;
        for (int l = 0; l < L; ++l) {
            G.push_back(leaf(from_host(gammas + static_cast<int64_t>(l) * H, {H}, true), "gamma"));
            auto h = detail::add_nodeops(xl, rl);
            yl = detail::mul_nodeops(detail::rms_nodeops(h), G.back());
            xl = h;
            rl = yl;
        }
        Tensor seed = from_host(g, {R, H}, false);
        backward(Value(yl), &seed, false);
        to_host(yl->value, y_last);
        to_host(X->grad, dx0);
        to_host(Rr->grad, dr0);
        for (int l = 0; l < L; ++l) to_host(G[l]->grad, dgammas + static_cast<int64_t>(l) * H);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

// JVP of rms(x) with tangent tx, two ways.
//   via_engine = 1: ag::jvp(root, seed) as a user would call it.  The reference's engine asks
//     jvp_lookup(Op::Leaf) for EVERY node, and jvp_Leaf returns an empty tensor "unused"
//     (cgadimpl/src/autodiff/autodiff_jvp_ops.cpp:190-192, cgadimpl/src/core/autodiff.cpp:246-247),
//     so the seed placed on a leaf is overwritten before any rule reads it.
//   via_engine = 0: the rule jvp_RMSNorm itself (jvp_lookup(Op::RMSNorm)) with the tangent handed
//     to it directly -- the literal formula of autodiff_jvp_ops.cpp:366-379.
int cgadimpl_ref_rms_jvp(const float* x, const float* tx, float* ty, int64_t R, int64_t H, int via_engine) {
    try {
        auto X = leaf(from_host(x, {R, H}, true), "x");
        auto n = detail::rms_nodeops(X);
        Tensor tangent = from_host(tx, {R, H}, false);
        Tensor t;
        if (via_engine) {
            std::unordered_map<Node*, Tensor> seed{{X.get(), tangent}};
            t = jvp(Value(n), seed);
        } else {
            std::function<const Tensor&(Node*)> tangent_of = [&](Node*) -> const Tensor& { return tangent; };
            t = jvp_lookup(Op::RMSNorm)(n.get(), tangent_of);
        }
        if (t.numel() == R * H) to_host(t, ty);
        else for (int64_t i = 0; i < R * H; ++i) ty[i] = t.numel() ? t.data<float>()[0] : 0.0f;  // broadcast what came back
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

// Times `iters` forward + backward passes of mul(rms(x), gamma) with the data already in tensors
// (what a user of the reference has): each pass builds the three nodes and runs ag::backward.
// x ~ N(0,1), gamma = 1 + 0.02 N(0,1), seed ~ N(0,1) from the stand-in's generator.
int cgadimpl_ref_time_fwd_bwd(int64_t R, int64_t H, int iters, int warmup, double* seconds_per_pass) {
    try {
        OwnTensor::manual_seed(0);
        Tensor xt = Tensor::randn(Shape{{R, H}}, TensorOptions().with_req_grad(true));
        Tensor gt = Tensor::randn(Shape{{H}}, TensorOptions().with_req_grad(true)) * 0.02f + 1.0f;
        Tensor gamma(Shape{{H}}, TensorOptions().with_req_grad(true));
        gamma.copy_(gt);
        Tensor seed = Tensor::randn(Shape{{R, H}}, TensorOptions());
        auto one_pass = [&] {
            auto X = leaf(xt, "x"), G = leaf(gamma, "gamma");
            auto out = detail::mul_nodeops(detail::rms_nodeops(X), G);
            backward(Value(out), &seed, false);
        };
        for (int i = 0; i < warmup; ++i) one_pass();
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < iters; ++i) one_pass();
        const auto t1 = std::chrono::steady_clock::now();
        *seconds_per_pass = std::chrono::duration<double>(t1 - t0).count() / (iters > 0 ? iters : 1);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

int cgadimpl_ref_num_threads(void);
void cgadimpl_ref_set_num_threads(int n);

// rowsum / rowmax / sum / mean_all forward and the gradient of sum(op(x)) w.r.t. x where defined.
// which: 0 rowsum, 1 rowmax (forward only), 2 sum, 3 mean_all.  out has R (row ops) or 1 elements.
int cgadimpl_ref_reduction(int which, const float* x, float* out, float* dx, int64_t R, int64_t H) {
    try {
        auto X = leaf(from_host(x, {R, H}, true), "x");
        std::shared_ptr<Node> n;
        switch (which) {
            case 0: n = detail::rowsum_nodeops(X); break;
            case 1: n = detail::rowmax_nodeops(X); break;
            case 2: n = detail::sum_nodeops(X); break;
            default: n = detail::mean_all_nodeops(X); break;
        }
        to_host(n->value, out);
        if (dx && which != 1) {
            auto loss = which < 2 ? detail::sum_nodeops(n) : n;
            backward(Value(loss), nullptr, false);
            to_host(X->grad, dx);
        }
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

// laynor(x) and its backward through the reference's own laynor_nodeops / vjp_LayerNorm (eps 1e-5).
int cgadimpl_ref_layernorm_fwd_bwd(const float* x, const float* gy, float* y, float* mean, float* var, float* dx,
                                   int64_t R, int64_t H) {
    try {
        auto X = leaf(from_host(x, {R, H}, true), "x");
        auto n = detail::laynor_nodeops(X);
        Tensor seed = from_host(gy, {R, H}, false);
        backward(Value(n), &seed, false);
        to_host(n->value, y);
        to_host(*n->tape[0], var);
        to_host(*n->tape[1], mean);
        to_host(X->grad, dx);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

// softmax_row (which 0) / logsumexp_row (which 1) through the reference's own builders and rules.
// gy and t are [R,H] for softmax and [R] / [R,H] for logsumexp; y, ty are [R,H] or [R] accordingly.
// The JVP rule is called directly (the engine overwrites leaf seeds, see cgadimpl_ref_rms_jvp).
int cgadimpl_ref_softmax_family(int which, const float* z, const float* gy, const float* t, float* y, float* dz, float* ty,
                                int64_t R, int64_t H) {
    try {
        auto Z = leaf(from_host(z, {R, H}, true), "z");
        auto n = which == 0 ? detail::softmax_row_nodeops(Z) : detail::logsumexp_row_nodeops(Z);
        Tensor seed = which == 0 ? from_host(gy, {R, H}, false) : from_host(gy, {R, 1}, false);
        backward(Value(n), &seed, false);
        to_host(n->value, y);
        to_host(Z->grad, dz);
        Tensor tangent = from_host(t, {R, H}, false);
        std::function<const Tensor&(Node*)> tangent_of = [&](Node*) -> const Tensor& { return tangent; };
        Tensor tv = jvp_lookup(which == 0 ? Op::SoftmaxRow : Op::LogSumExpRow)(n.get(), tangent_of);
        to_host(tv, ty);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

// `steps` optimiser updates of one parameter vector with given gradients grads[steps, n], through
// the reference's own ag::SGD / ag::Adam (cgadimpl/src/optimizer/optim.cpp).  which: 0 SGD, 1 Adam.
int cgadimpl_ref_optimizer(int which, float* param, const float* grads, int64_t n, int steps, float lr_or_alpha) {
    try {
        auto P = leaf(from_host(param, {n}, true), "p");
        auto root = detail::sum_nodeops(P);
        Adam adam({Value(P)}, lr_or_alpha);
        for (int s = 0; s < steps; ++s) {
            std::memcpy(P->grad.data<float>(), grads + static_cast<int64_t>(s) * n, sizeof(float) * n);
            if (which == 0) SGD(Value(root), nullptr, lr_or_alpha);
            else adam.step();
        }
        to_host(P->value, param);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cgadimpl_ref: %s\n", e.what());
        return 1;
    }
}

int cgadimpl_ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void cgadimpl_ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
