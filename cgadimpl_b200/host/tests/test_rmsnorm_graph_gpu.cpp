// test_rmsnorm_graph_gpu.cpp -- the graph API on the RMSNorm path against the CPU oracle and
// against itself: fused node vs the reference's composition mul(rms(x), gamma), sequential vs
// parallel backward (cgadimpl/Tests/dependency_counter_correctness, tolerance 1e-4 there), hooks
// (Tests/autograd_hooks_testing/test_hooks.cpp), creation context (Tests/test_phase1_metadata.cpp
// :201-232), the corrected JVP, and a small residual stack through add_rmsnorm / residual_of.
#include "ad/ag_all.hpp"
#include "agb_oracle.h"
#include "check.hpp"

using namespace ag;

static const auto kDev = DeviceIndex(Device::CUDA);

static Value leaf(const std::vector<float>& v, std::vector<int64_t> dims, bool req = true) {
    return make_tensor(Tensor::from_host(v.data(), Shape{dims}, TensorOptions().with_device(kDev).with_req_grad(req)));
}
static std::vector<float> randv(size_t n, unsigned seed, float scale = 1.f, float shift = 0.f) {
    std::vector<float> v(n);
    uint64_t s = seed * 0x9E3779B97F4A7C15ull + 1;
    for (auto& x : v) {  // sum of 4 uniforms, roughly normal
        double acc = 0;
        for (int k = 0; k < 4; ++k) { s = s * 6364136223846793005ull + 1442695040888963407ull; acc += double(s >> 11) / 9007199254740992.0; }
        x = shift + scale * float((acc - 2.0) * 1.7320508);
    }
    return v;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 2; }
    const int64_t R = 96, H = 1024;
    const float eps = 1e-5f;
    const auto xv = randv(R * H, 1), gv = randv(H, 2, 0.02f, 1.0f), gyv = randv(R * H, 3);

    // oracle, fp64-reduced arbiter
    std::vector<float> oy(R * H), orstd(R), odx(R * H), odg(H);
    agb_oracle_rmsnorm_fwd_bwd(xv.data(), gv.data(), gyv.data(), oy.data(), orstd.data(), odx.data(), odg.data(), R, H, eps, AGB_RED_F64);

    run_test("fused rmsnorm node vs oracle (rel 1e-5 / abs 1e-6)", [&] {
        Value x = leaf(xv, {R, H}), g = leaf(gv, {H});
        Value y = rmsnorm(x, g, eps);
        Tensor seed = Tensor::from_host(gyv.data(), Shape{{R, H}}, TensorOptions().with_device(kDev));
        backward(y, &seed);
        CHECK(all_close(y.val().to_vector(), oy, 1e-5, 1e-6, "y"));
        CHECK(all_close(y.node->tape[0]->to_vector(), orstd, 1e-5, 1e-6, "rstd"));
        CHECK(all_close(x.grad().to_vector(), odx, 1e-5, 1e-6, "dx"));
        CHECK(all_close(g.grad().to_vector(), odg, 1e-5, 1e-6, "dgamma"));
        CHECK(frac_equal(x.grad().to_vector(), odx) >= 0.999 && frac_equal(y.val().to_vector(), oy) >= 0.999);
        CHECK(y.node->op == Op::RMSNormAffine && y.node->inputs.size() == 2 && y.node->tape.size() == 1);
    });

    run_test("reference composition mul(rms(x), gamma) == fused node", [&] {
        Value x1 = leaf(xv, {R, H}), g1 = leaf(gv, {1, H});
        Value y1 = mul(rms(x1), g1);                      // three nodes, like the reference
        Value x2 = leaf(xv, {R, H}), g2 = leaf(gv, {H});
        Value y2 = rmsnorm(x2, g2, 1e-5f);                // one node
        Tensor seed = Tensor::from_host(gyv.data(), Shape{{R, H}}, TensorOptions().with_device(kDev));
        backward(y1, &seed);
        backward(y2, &seed);
        CHECK(y1.val().to_vector() == y2.val().to_vector());
        CHECK(x1.grad().to_vector() == x2.grad().to_vector());
        CHECK(all_close(g1.grad().to_vector(), g2.grad().to_vector(), 1e-6, 1e-7, "dgamma"));
        CHECK(g1.grad().shape().dims == std::vector<int64_t>({1, H}));   // reduce_for_broadcast keeps the operand's shape
        CHECK(y1.node->op == Op::Mul && y1.node->inputs[0]->op == Op::RMSNorm && y1.node->inputs[0]->tape.size() == 2);
    });

    run_test("accumulate: two backward passes add up; zero_grad resets", [&] {
        Value x = leaf(xv, {R, H}), g = leaf(gv, {H});
        Value y = rmsnorm(x, g, eps);
        Tensor seed = Tensor::from_host(gyv.data(), Shape{{R, H}}, TensorOptions().with_device(kDev));
        backward(y, &seed);
        auto once = x.grad().to_vector();
        auto dg_once = g.grad().to_vector();
        backward(y, &seed);
        auto twice = x.grad().to_vector(), dg_twice = g.grad().to_vector();
        bool ok = true;
        for (size_t i = 0; i < once.size(); ++i) ok = ok && twice[i] == once[i] + once[i];
        for (size_t i = 0; i < dg_once.size(); ++i) ok = ok && dg_twice[i] == dg_once[i] + dg_once[i];
        CHECK(ok);
        zero_grad(y);
        CHECK(x.grad().to_vector() == std::vector<float>(R * H, 0.f));
    });

    run_test("sequential vs parallel backward on a diamond", [&] {
        auto build = [&](Value& x, Value& g) {
            Value a = rms(x);
            Value b = rmsnorm(x, g, eps);
            Value c = a + b;              // x feeds two branches
            Value d = c * a;              // a is used twice
            return sum(rowsum(d));
        };
        Value x1 = leaf(xv, {R, H}), g1 = leaf(gv, {H});
        Value x2 = leaf(xv, {R, H}), g2 = leaf(gv, {H});
        backward(build(x1, g1), nullptr, false);
        backward(build(x2, g2), nullptr, true);
        cudaDeviceSynchronize();
        CHECK(all_close(x2.grad().to_vector(), x1.grad().to_vector(), 1e-4, 1e-4, "dx seq vs par"));
        CHECK(all_close(g2.grad().to_vector(), g1.grad().to_vector(), 1e-4, 1e-4, "dgamma seq vs par"));
    });

    run_test("post-accumulate hooks fire once per parameter (both modes)", [&] {
        for (bool par : {false, true}) {
            Value x = leaf(xv, {R, H}), g = leaf(gv, {H});
            int hx = 0, hg = 0;
            x.register_hook([&](Node*) { ++hx; });
            g.register_hook([&](Node*) { ++hg; });
            Value y = rmsnorm(x, g, eps) + rms(x);
            backward(sum(y), nullptr, par);
            CHECK(hx == 1 && hg == 1);
        }
    });

    run_test("creation context and explicit streams", [&] {
        cudaStream_t s;
        cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
        set_current_stream(reinterpret_cast<ag_cuda_stream_t>(s));
        Value x = leaf(xv, {R, H}), g = leaf(gv, {H});
        Value y = rmsnorm(x, g, eps);
        CHECK(y.node->creation_context.stream == reinterpret_cast<ag_cuda_stream_t>(s));
        CHECK(y.node->creation_context.device.is_cuda());
        set_current_stream(nullptr);       // the rules must still use the node's stream
        Tensor seed = Tensor::from_host(gyv.data(), Shape{{R, H}}, TensorOptions().with_device(kDev));
        cudaDeviceSynchronize();
        backward(y, &seed);
        cudaStreamSynchronize(s);
        CHECK(all_close(x.grad().to_vector(), odx, 1e-5, 1e-6, "dx on a side stream"));
        cudaStreamDestroy(s);
    });

    run_test("jvp: corrected form vs oracle, adjoint identity", [&] {
        const auto tv = randv(R * H, 5), tgv = randv(H, 6);
        Value x = leaf(xv, {R, H}), g = leaf(gv, {H});
        Value y = rmsnorm(x, g, eps);
        Tensor tx = Tensor::from_host(tv.data(), Shape{{R, H}}, TensorOptions().with_device(kDev));
        Tensor tg = Tensor::from_host(tgv.data(), Shape{{H}}, TensorOptions().with_device(kDev));
        Tensor ty = jvp(y, {{x.node.get(), tx}, {g.node.get(), tg}});
        // oracle: yhat, corrected jvp of rms, then jvp of the gamma product
        std::vector<float> yhat(R * H), rs(R), tyhat(R * H), want(R * H);
        agb_oracle_rms_forward(xv.data(), yhat.data(), rs.data(), R, H, eps, AGB_RED_F64);
        agb_oracle_jvp_rms_corrected(tv.data(), yhat.data(), rs.data(), tyhat.data(), R, H, AGB_RED_F64);
        agb_oracle_jvp_scale(tyhat.data(), yhat.data(), gv.data(), tgv.data(), want.data(), R, H);
        CHECK(all_close(ty.to_vector(), want, 1e-5, 1e-6, "jvp"));
        // composition through three nodes gives the same tangent
        Value x2 = leaf(xv, {R, H}), g2 = leaf(gv, {H});
        Value y2 = mul(rms(x2), g2);
        Tensor ty2 = jvp(y2, {{x2.node.get(), tx}, {g2.node.get(), tg}});
        CHECK(all_close(ty2.to_vector(), want, 1e-5, 1e-6, "jvp via composition"));
        // <gy, J tx> == <J^T gy, tx> with a zero gamma tangent
        Tensor ty0 = jvp(y, {{x.node.get(), tx}});
        auto t0 = ty0.to_vector();
        double lhs = 0, rhs = 0;
        for (size_t i = 0; i < t0.size(); ++i) { lhs += double(gyv[i]) * t0[i]; rhs += double(odx[i]) * tv[i]; }
        CHECK(std::fabs(lhs - rhs) <= 1e-5 * std::max(1.0, std::fabs(lhs)));
        // reductions
        Tensor ts = jvp(sum(y), {{x.node.get(), tx}});
        double want_s = 0;
        for (float f : t0) want_s += f;
        CHECK(std::fabs(ts.to_vector()[0] - want_s) <= 1e-4 * std::max(1.0, std::fabs(want_s)));
    });

    run_test("residual stack through add_rmsnorm / residual_of vs oracle", [&] {
        const int L = 3;
        const int64_t r2 = 24, h2 = 256;
        const auto x0 = randv(r2 * h2, 11), r0 = randv(r2 * h2, 12), gg = randv(r2 * h2, 13), gam = randv(L * h2, 14, 0.02f, 1.f);
        std::vector<float> wy(r2 * h2), wdh(r2 * h2), wdg(L * h2);
        agb_oracle_residual_stack(x0.data(), r0.data(), gam.data(), gg.data(), wy.data(), wdh.data(), wdg.data(), r2, h2, L, 1e-6f, AGB_RED_F64);
        Value x = leaf(x0, {r2, h2}), r = leaf(r0, {r2, h2});
        std::vector<Value> gammas;
        Value xl = x, rl = r, y;
        for (int l = 0; l < L; ++l) {
            gammas.push_back(leaf(std::vector<float>(gam.begin() + l * h2, gam.begin() + (l + 1) * h2), {h2}));
            y = add_rmsnorm(xl, rl, gammas[l], 1e-6f);
            xl = residual_of(y);
            rl = y;
        }
        Tensor seed = Tensor::from_host(gg.data(), Shape{{r2, h2}}, TensorOptions().with_device(kDev));
        backward(y, &seed);
        CHECK(all_close(y.val().to_vector(), wy, 1e-5, 1e-6, "y_last"));
        CHECK(all_close(x.grad().to_vector(), wdh, 1e-5, 1e-6, "dx0"));
        CHECK(all_close(r.grad().to_vector(), wdh, 1e-5, 1e-6, "dr0"));
        for (int l = 0; l < L; ++l)
            CHECK(all_close(gammas[l].grad().to_vector(), std::vector<float>(wdg.begin() + l * h2, wdg.begin() + (l + 1) * h2), 1e-5, 1e-6, "dgamma_l"));
    });

    run_test("bf16 tensors through the graph API", [&] {
        const auto bopts = TensorOptions().with_device(kDev).with_dtype(Dtype::Bfloat16);
        Value x = make_tensor(Tensor::from_host(xv.data(), Shape{{R, H}}, bopts.with_req_grad(true)));
        Value y = rms(x);
        Tensor seed = Tensor::from_host(gyv.data(), Shape{{R, H}}, bopts);
        backward(y, &seed);
        // oracle on the bf16-rounded inputs
        auto xr = x.val().to_vector(), gr = seed.to_vector();
        std::vector<float> wy(R * H), wr(R), wdx(R * H);
        agb_oracle_rmsnorm_fwd_bwd(xr.data(), nullptr, gr.data(), wy.data(), wr.data(), wdx.data(), nullptr, R, H, 1e-5f, AGB_RED_F64);
        CHECK(all_close(y.val().to_vector(), wy, 2e-2, 1e-6, "y bf16"));
        CHECK(all_close(x.grad().to_vector(), wdx, 2e-2, 1e-6, "dx bf16"));
    });

    cudaDeviceSynchronize();
    return finish("test_rmsnorm_graph_gpu");
}
