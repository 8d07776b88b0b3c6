// test_graph_capture_gpu.cpp -- CUDA-graph capture of the layer stack.  The reference captures a
// forward MLP only, after three warm-up passes that fill its allocator pool, and checks nothing
// numerically (cgadimpl/Tests/test_graph_gpu.cpp:207-255).  Here forward AND backward of a stack of
// fused residual-add + RMSNorm layers go into one graph; the replay is checked against the eager
// run and the CPU oracle, and re-run with new input contents at the same addresses.
#include "ad/ag_all.hpp"
#include "agb/agb.h"
#include "agb_oracle.h"
#include "check.hpp"
#include "nn/rmsnorm_stack.hpp"

using namespace ag;

static const auto kDev = DeviceIndex(Device::CUDA);
static std::vector<float> randv(size_t n, unsigned seed, float scale = 1.f, float shift = 0.f) {
    std::vector<float> v(n);
    uint64_t s = seed * 0x9E3779B97F4A7C15ull + 1;
    for (auto& x : v) {
        double acc = 0;
        for (int k = 0; k < 4; ++k) { s = s * 6364136223846793005ull + 1442695040888963407ull; acc += double(s >> 11) / 9007199254740992.0; }
        x = shift + scale * float((acc - 2.0) * 1.7320508);
    }
    return v;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 2; }
    const int L = 6;
    const int64_t R = 200, H = 2048;
    const float eps = 1e-6f;
    const auto opt = TensorOptions().with_device(kDev);

    run_test("stack: eager == oracle, graph replay == eager, replay follows new inputs", [&] {
        auto x0 = randv(R * H, 1), r0 = randv(R * H, 2), g0 = randv(R * H, 3), gam = randv(L * H, 4, 0.02f, 1.f);
        std::vector<float> wy(R * H), wdh(R * H), wdg(L * H);
        agb_oracle_residual_stack(x0.data(), r0.data(), gam.data(), g0.data(), wy.data(), wdh.data(), wdg.data(), R, H, L, eps, AGB_RED_F64);

        nn::ResidualRMSNormStack stack(L, R, H, Dtype::Float32, eps, kDev);
        stack.gammas().copy_(Tensor::from_host(gam.data(), Shape{{L, H}}, opt));
        Tensor x = Tensor::from_host(x0.data(), Shape{{R, H}}, opt), r = Tensor::from_host(r0.data(), Shape{{R, H}}, opt),
               g = Tensor::from_host(g0.data(), Shape{{R, H}}, opt);
        stack.forward(x, r);
        stack.backward(g);
        cudaDeviceSynchronize();
        CHECK(all_close(stack.y_last().to_vector(), wy, 1e-5, 1e-6, "eager y_last"));
        CHECK(all_close(stack.dh0().to_vector(), wdh, 1e-5, 1e-6, "eager dh0"));
        CHECK(all_close(stack.dgammas().to_vector(), wdg, 1e-5, 1e-6, "eager dgammas"));
        CHECK(frac_equal(stack.dh0().to_vector(), wdh) >= 0.999);
        const auto eager_y = stack.y_last().to_vector(), eager_dh = stack.dh0().to_vector(), eager_dg = stack.dgammas().to_vector();

        const auto allocs_before = OwnTensor::cuda::DeviceAllocator::instance().stats().device_allocs;
        CudaGraphRunner runner;
        stack.capture(runner, x, r, g);
        CHECK(OwnTensor::cuda::DeviceAllocator::instance().stats().device_allocs == allocs_before);  // capture allocated nothing
        CHECK(runner.num_nodes() == static_cast<size_t>(3 * L));  // L forward + L backward + L dgamma reductions
        CHECK(current_stream() == nullptr);                       // end_capture reset the stream slot

        // wipe the outputs, replay, compare bit for bit with the eager run
        const_cast<Tensor&>(stack.y_last()).zero_();
        const_cast<Tensor&>(stack.dgammas()).zero_();
        cudaDeviceSynchronize();
        CHECK(runner.replay());
        runner.synchronize();
        CHECK(stack.y_last().to_vector() == eager_y);
        CHECK(stack.dh0().to_vector() == eager_dh);
        CHECK(stack.dgammas().to_vector() == eager_dg);

        // new contents at the same addresses: the graph recomputes from them
        auto x1 = randv(R * H, 21), r1 = randv(R * H, 22), g1 = randv(R * H, 23);
        x.copy_(Tensor::from_host(x1.data(), Shape{{R, H}}, opt));
        r.copy_(Tensor::from_host(r1.data(), Shape{{R, H}}, opt));
        g.copy_(Tensor::from_host(g1.data(), Shape{{R, H}}, opt));
        agb_oracle_residual_stack(x1.data(), r1.data(), gam.data(), g1.data(), wy.data(), wdh.data(), wdg.data(), R, H, L, eps, AGB_RED_F64);
        cudaDeviceSynchronize();
        for (int i = 0; i < 3; ++i) CHECK(runner.replay());
        runner.synchronize();
        CHECK(all_close(stack.y_last().to_vector(), wy, 1e-5, 1e-6, "replayed y_last"));
        CHECK(all_close(stack.dh0().to_vector(), wdh, 1e-5, 1e-6, "replayed dh0"));
        CHECK(all_close(stack.dgammas().to_vector(), wdg, 1e-5, 1e-6, "replayed dgammas"));
    });

    run_test("stack at the benchmark's full size (32 layers x 16384 rows x 4096): graph replay == eager, row slice == oracle", [&] {
        // The launch plans depend on the row count, so the plans the benchmark times are checked here.  Rows are
        // independent in y_last and dh0: the oracle runs the whole 32-layer stack on a strided slice of rows.
        const int LF = 32;
        const int64_t RF = 16384, HF = 4096;
        auto x0 = randv(RF * HF, 31), r0 = randv(RF * HF, 32), g0 = randv(RF * HF, 33), gam = randv(LF * HF, 34, 0.02f, 1.f);
        nn::ResidualRMSNormStack stack(LF, RF, HF, Dtype::Float32, eps, kDev);
        stack.gammas().copy_(Tensor::from_host(gam.data(), Shape{{LF, HF}}, opt));
        Tensor x = Tensor::from_host(x0.data(), Shape{{RF, HF}}, opt), r = Tensor::from_host(r0.data(), Shape{{RF, HF}}, opt),
               g = Tensor::from_host(g0.data(), Shape{{RF, HF}}, opt);
        stack.forward(x, r);
        stack.backward(g);
        cudaDeviceSynchronize();
        const auto eager_y = stack.y_last().to_vector(), eager_dh = stack.dh0().to_vector(), eager_dg = stack.dgammas().to_vector();

        const int64_t NS = 48, stride = 337;
        std::vector<float> sx(NS * HF), sr(NS * HF), sg(NS * HF), wy(NS * HF), wdh(NS * HF), wdg(LF * HF), gy_(NS * HF), gdh(NS * HF);
        for (int64_t i = 0; i < NS; ++i) {
            const int64_t row = i * stride;
            std::copy(x0.begin() + row * HF, x0.begin() + (row + 1) * HF, sx.begin() + i * HF);
            std::copy(r0.begin() + row * HF, r0.begin() + (row + 1) * HF, sr.begin() + i * HF);
            std::copy(g0.begin() + row * HF, g0.begin() + (row + 1) * HF, sg.begin() + i * HF);
            std::copy(eager_y.begin() + row * HF, eager_y.begin() + (row + 1) * HF, gy_.begin() + i * HF);
            std::copy(eager_dh.begin() + row * HF, eager_dh.begin() + (row + 1) * HF, gdh.begin() + i * HF);
        }
        agb_oracle_residual_stack(sx.data(), sr.data(), gam.data(), sg.data(), wy.data(), wdh.data(), wdg.data(), NS, HF, LF, eps, AGB_RED_F64);
        CHECK(all_close(gy_, wy, 1e-5, 1e-6, "full-size y_last, row slice"));
        CHECK(all_close(gdh, wdh, 1e-5, 1e-6, "full-size dh0, row slice"));
        CHECK(frac_equal(gy_, wy) >= 0.999);
        CHECK(frac_equal(gdh, wdh) >= 0.999);

        CudaGraphRunner runner;
        stack.capture(runner, x, r, g);
        CHECK(runner.num_nodes() == static_cast<size_t>(3 * LF));
        const_cast<Tensor&>(stack.y_last()).zero_();
        const_cast<Tensor&>(stack.dgammas()).zero_();
        cudaDeviceSynchronize();
        for (int i = 0; i < 2; ++i) CHECK(runner.replay());
        runner.synchronize();
        CHECK(stack.y_last().to_vector() == eager_y);
        CHECK(stack.dh0().to_vector() == eager_dh);
        CHECK(stack.dgammas().to_vector() == eager_dg);
        CHECK(agb_device_status() == 0);
    });

    run_test("graph API under capture after warm-up (the reference's pattern)", [&] {
        auto xv = randv(64 * 512, 7);
        Tensor xt = Tensor::from_host(xv.data(), Shape{{64, 512}}, opt);
        Value x = make_tensor(xt);
        std::vector<float> eager;
        for (int i = 0; i < 3; ++i) {           // warm-up fills the allocator's cache for stream 0 ...
            Value y = rms(x);
            cudaDeviceSynchronize();
            eager = y.val().to_vector();
        }
        CudaGraphRunner runner;
        {                                       // ... but the runner captures on its own stream: warm that pool too
            set_current_stream(reinterpret_cast<ag_cuda_stream_t>(runner.get_stream()));
            OwnTensor::cuda::setCurrentStream(runner.get_stream());
            { Value y = rms(x); }
            runner.synchronize();
            set_current_stream(nullptr);
            OwnTensor::cuda::setCurrentStream(nullptr);
        }
        runner.begin_capture();
        Value y_captured = rms(x);
        runner.end_capture();
        CHECK(runner.replay());
        runner.synchronize();
        CHECK(y_captured.val().to_vector() == eager);
        // a capture that would need a fresh allocation is refused with a clear error
        CudaGraphRunner cold;
        bool threw = false;
        cold.begin_capture();
        try {
            Tensor big(Shape{{1 << 22}}, opt);  // 16 MB, never cached on this stream
        } catch (const std::runtime_error& e) {
            threw = std::string(e.what()).find("captured") != std::string::npos;
        }
        cold.end_capture();
        CHECK(threw);
    });

    cudaDeviceSynchronize();
    return finish("test_graph_capture_gpu");
}
