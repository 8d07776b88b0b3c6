// test_nn_optim_gpu.cpp -- the nn::RMSNorm module and the SGD / Adam updates of its gamma.
// Mirrors the reference's training smoke tests (cgadimpl/Tests/test_kitchen_sink_mlp.cpp:24,112-113:
// a model that uses rms, loss after training < loss before, no NaN) and checks every optimiser step
// against the CPU restatement of cgadimpl/src/optimizer/optim.cpp bit for bit.
#include "ad/ag_all.hpp"
#include "agb_oracle.h"
#include "check.hpp"

using namespace ag;
static const auto kDev = DeviceIndex(Device::CUDA);

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 2; }
    OwnTensor::manual_seed(3);
    const int64_t R = 64, H = 512;
    const auto opt = TensorOptions().with_device(kDev);

    run_test("module: parameters, to(), zero_grad, hooks", [&] {
        nn::RMSNorm norm(H, 1e-6f);
        CHECK(norm.parameters().size() == 1 && norm.gamma().val().numel() == H && norm.gamma().node->requires_grad());
        CHECK(norm.gamma().val().to_vector() == std::vector<float>(H, 1.0f));
        int fired = 0;
        norm.register_backward_hook([&](Node*) { ++fired; });
        Value x = make_tensor(Tensor::randn(Shape{{R, H}}, opt.with_req_grad(true)));
        Value y = norm(x);
        CHECK(y.node->op == Op::RMSNormAffine);
        backward(sum(y));
        CHECK(fired == 1);
        bool nonzero = false;
        for (float f : norm.gamma().grad().to_vector()) nonzero = nonzero || f != 0.f;
        CHECK(nonzero);
        norm.zero_grad();
        CHECK(norm.gamma().grad().to_vector() == std::vector<float>(H, 0.f));
        nn::RMSNorm a(H), b(H);
        nn::Sequential seq({&a, &b});
        CHECK(seq.parameters().size() == 2 && seq.get_layers().size() == 2);
        Value z = seq(x);
        CHECK(z.node->inputs[0]->op == Op::RMSNormAffine);
        // residual form
        Value r = make_tensor(Tensor::randn(Shape{{R, H}}, opt));
        Value yr = norm(x, r);
        CHECK(residual_of(yr).node->op == Op::Add);
    });

    // loss = sum(norm(x) * target): linear in gamma, so the gradient is known and both optimisers must lower it
    auto loss_of = [&](nn::RMSNorm& norm, const Value& x, const Value& target) { return sum(norm(x) * target); };

    run_test("SGD lowers the loss; each step equals the reference's update", [&] {
        nn::RMSNorm norm(H, 1e-6f);
        Value x = make_tensor(Tensor::randn(Shape{{R, H}}, opt)), target = make_tensor(Tensor::randn(Shape{{R, H}}, opt));
        float first = 0, last = 0;
        for (int it = 0; it < 5; ++it) {
            norm.zero_grad();
            Value loss = loss_of(norm, x, target);
            backward(loss);
            const float l = loss.val().to_vector()[0];
            if (it == 0) first = l;
            last = l;
            CHECK(std::isfinite(l));
            std::vector<float> p = norm.gamma().val().to_vector(), g = norm.gamma().grad().to_vector();
            SGD(loss, nullptr, 1e-3f);
            agb_oracle_sgd_step(p.data(), g.data(), H, 1e-3f);
            CHECK(norm.gamma().val().to_vector() == p);
        }
        CHECK(last < first);
    });

    run_test("Adam lowers the loss; m, v and the parameter match the reference's arithmetic", [&] {
        nn::RMSNorm norm(H, 1e-6f);
        Value x = make_tensor(Tensor::randn(Shape{{R, H}}, opt)), target = make_tensor(Tensor::randn(Shape{{R, H}}, opt));
        Adam adam(norm.parameters(), 1e-2f);
        std::vector<float> p = norm.gamma().val().to_vector(), m(H, 0.f), v(H, 0.f);
        float first = 0, last = 0;
        for (int it = 1; it <= 6; ++it) {
            adam.zero_grad();
            Value loss = loss_of(norm, x, target);
            backward(loss);
            const float l = loss.val().to_vector()[0];
            if (it == 1) first = l;
            last = l;
            std::vector<float> g = norm.gamma().grad().to_vector();
            adam.step();
            agb_oracle_adam_step(p.data(), g.data(), m.data(), v.data(), H, 1e-2f, 0.9f, 0.999f, 1e-8f, it);
            CHECK(norm.gamma().val().to_vector() == p);
        }
        CHECK(adam.steps() == 6 && last < first);
    });

    cudaDeviceSynchronize();
    return finish("test_nn_optim_gpu");
}
