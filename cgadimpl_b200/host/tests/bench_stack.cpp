// bench_stack.cpp -- times the fused residual-add + RMSNorm layer stack (forward + VJP through all
// layers) as ONE CUDA graph replayed on ag::CudaGraphRunner's stream.
//   bench_stack [layers=32] [rows=16384] [hidden=4096] [iters=10] [warmup=3] [bf16=0] [option=value ...]
// (trailing option=value pairs go to agb_set_option before anything runs)
// Prints one JSON object: ms per replay (CUDA events around `iters` replays), graph node count,
// row-layers per second and algorithmic GB/s at (7*H*s + 8) bytes per row and layer.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "ad/ag_all.hpp"
#include "agb/agb.h"
#include "nn/rmsnorm_stack.hpp"

using namespace ag;

int main(int argc, char** argv) {
    const int L = argc > 1 ? std::atoi(argv[1]) : 32;
    const int64_t R = argc > 2 ? std::atoll(argv[2]) : 16384;
    const int64_t H = argc > 3 ? std::atoll(argv[3]) : 4096;
    const int iters = argc > 4 ? std::atoi(argv[4]) : 10;
    const int warmup = argc > 5 ? std::atoi(argv[5]) : 3;
    const bool bf16 = argc > 6 && std::atoi(argv[6]) != 0;
    for (int i = 7; i < argc; ++i) {
        std::string kv(argv[i]);
        const size_t eq = kv.find('=');
        if (eq == std::string::npos || agb_set_option(kv.substr(0, eq).c_str(), std::atoll(kv.c_str() + eq + 1)) != 0) {
            std::fprintf(stderr, "bench_stack: bad option '%s'\n", argv[i]);
            return 1;
        }
    }
    try {
        const auto dev = DeviceIndex(Device::CUDA);
        const Dtype dt = bf16 ? Dtype::Bfloat16 : Dtype::Float32;
        const auto opt = TensorOptions().with_device(dev).with_dtype(dt);
        OwnTensor::manual_seed(0);
        nn::ResidualRMSNormStack stack(L, R, H, dt, 1e-6f, dev);
        {   // gamma_l = 1 + 0.02 N(0,1)
            Tensor g = Tensor::randn(Shape{{L, H}}, TensorOptions());
            std::vector<float> v = g.to_vector();
            for (auto& f : v) f = 1.0f + 0.02f * f;
            stack.gammas().copy_(Tensor::from_host(v.data(), Shape{{L, H}}, opt));
        }
        // one [256, H] block of normals tiled over the rows keeps host-side generation short
        auto tiled = [&](unsigned seed) {
            OwnTensor::manual_seed(seed);
            const int64_t blk = R < 256 ? R : 256;
            std::vector<float> b = Tensor::randn(Shape{{blk, H}}, TensorOptions()).to_vector();
            Tensor t(Shape{{R, H}}, opt);
            Tensor blk_dev = Tensor::from_host(b.data(), Shape{{blk, H}}, opt);
            for (int64_t r0 = 0; r0 < R; r0 += blk) {
                const int64_t n = (R - r0 < blk ? R - r0 : blk);
                cudaMemcpy(static_cast<char*>(t.raw()) + r0 * H * dtype_size(dt), blk_dev.raw(), n * H * dtype_size(dt), cudaMemcpyDeviceToDevice);
            }
            return t;
        };
        Tensor x = tiled(1), r = tiled(2), g = tiled(3);
        CudaGraphRunner runner;
        stack.capture(runner, x, r, g);
        for (int i = 0; i < warmup; ++i) runner.replay();
        runner.synchronize();
        // `iters` replays back to back; the first few are also timed on their own: a GPU that starts cool runs
        // them at full clock, a long region settles at whatever the power cap leaves
        cudaEvent_t e0, em, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&em);
        cudaEventCreate(&e1);
        const int head = iters < 5 ? iters : 5;
        cudaEventRecord(e0, runner.get_stream());
        for (int i = 0; i < iters; ++i) {
            runner.replay();
            if (i + 1 == head) cudaEventRecord(em, runner.get_stream());
        }
        cudaEventRecord(e1, runner.get_stream());
        runner.synchronize();
        float ms = 0, ms_head = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        cudaEventElapsedTime(&ms_head, e0, em);
        const double per = ms / iters;
        const double bytes = double(L) * double(R) * (7.0 * H * dtype_size(dt) + 8.0);
        int status = agb_device_status();
        std::printf("{\"layers\": %d, \"rows\": %lld, \"hidden\": %lld, \"io_dtype\": \"%s\", \"iters\": %d, \"warmup\": %d, "
                    "\"ms_per_replay\": %.6f, \"first_replays_ms\": %.6f, \"graph_nodes\": %zu, \"row_layers_per_s\": %.1f, \"gbs\": %.2f, "
                    "\"saved_activation_bytes\": %zu, \"launches_per_replay\": %d, \"device_status\": %d}\n",
                    L, (long long)R, (long long)H, bf16 ? "bfloat16" : "float32", iters, warmup, per, ms_head / head, runner.num_nodes(),
                    double(L) * R / (per * 1e-3), bytes / (per * 1e-3) / 1e9, stack.saved_bytes(), 3 * L, status);
        return status == 0 ? 0 : 1;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "bench_stack: %s\n", e.what());
        return 1;
    }
}
