// bench_api.cpp -- times the path a cgadimpl user calls: ag::rmsnorm (forward node) + ag::backward (reverse
// sweep, vjp_RMSNormAffine) over one [rows, hidden] activation, eagerly and as a CUDA graph replayed on
// ag::CudaGraphRunner's stream.  The reference's counterpart, Benchmark/RMSNormLayer.cpp, is an empty stub.
//   bench_api [rows=32768] [hidden=4096] [iters=50] [warmup=5] [bf16=0]
// Prints one JSON object: ms per step eager and captured, and algorithmic GB/s at (5*H*s + 8) bytes per row.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "ad/ag_all.hpp"
#include "agb/agb.h"

using namespace ag;

int main(int argc, char** argv) {
    const int64_t R = argc > 1 ? std::atoll(argv[1]) : 32768;
    const int64_t H = argc > 2 ? std::atoll(argv[2]) : 4096;
    const int iters = argc > 3 ? std::atoi(argv[3]) : 50;
    const int warmup = argc > 4 ? std::atoi(argv[4]) : 5;
    const bool bf16 = argc > 5 && std::atoi(argv[5]) != 0;
    try {
        const auto dev = DeviceIndex(Device::CUDA);
        const Dtype dt = bf16 ? Dtype::Bfloat16 : Dtype::Float32;
        const float eps = 1e-5f;
        OwnTensor::manual_seed(0);
        auto tiled = [&](unsigned seed, bool req) {   // one [256, H] block of normals tiled over the rows
            OwnTensor::manual_seed(seed);
            const int64_t blk = R < 256 ? R : 256;
            std::vector<float> b = Tensor::randn(Shape{{blk, H}}, TensorOptions()).to_vector();
            Tensor t(Shape{{R, H}}, TensorOptions().with_device(dev).with_dtype(dt).with_req_grad(req));
            Tensor blk_dev = Tensor::from_host(b.data(), Shape{{blk, H}}, TensorOptions().with_device(dev).with_dtype(dt));
            for (int64_t r0 = 0; r0 < R; r0 += blk) {
                const int64_t n = (R - r0 < blk ? R - r0 : blk);
                cudaMemcpy(static_cast<char*>(t.raw()) + r0 * H * dtype_size(dt), blk_dev.raw(), n * H * dtype_size(dt), cudaMemcpyDeviceToDevice);
            }
            return t;
        };
        Tensor gy = tiled(3, false);
        std::vector<float> gv = Tensor::randn(Shape{{H}}, TensorOptions()).to_vector();
        for (auto& f : gv) f = 1.0f + 0.02f * f;
        cudaEvent_t e0, em, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&em);
        cudaEventCreate(&e1);
        const int head = iters < 20 ? iters : 20;   // also timed on their own: the pace before the power cap bites

        // The step a user writes.  Gradients of the leaves are cleared (lazily) every step, so each backward
        // writes them instead of adding to them, like the C-ABI calls the headline numbers time.
        Value x = make_tensor(tiled(1, true), "x");
        // (dgamma is produced in fp32: a 16-bit gamma node takes no gradient through the graph API)
        Value gamma = make_tensor(Tensor::from_host(gv.data(), Shape{{H}}, TensorOptions().with_device(dev).with_dtype(dt).with_req_grad(!bf16)), "gamma");
        auto step = [&] {
            Value y = rmsnorm(x, gamma, eps);
            zero_grad(y);
            backward(y, &gy);
        };

        // eager, on the default stream
        for (int i = 0; i < warmup; ++i) step();
        cudaDeviceSynchronize();
        const uint64_t l0 = agb_launch_count();
        cudaEventRecord(e0, nullptr);
        for (int i = 0; i < iters; ++i) {
            step();
            if (i + 1 == head) cudaEventRecord(em, nullptr);
        }
        cudaEventRecord(e1, nullptr);
        cudaDeviceSynchronize();
        const uint64_t launches_eager = agb_launch_count() - l0;
        float ms_eager = 0, ms_eager_head = 0;
        cudaEventElapsedTime(&ms_eager, e0, e1);
        cudaEventElapsedTime(&ms_eager_head, e0, em);

        // The reference's own composition of the same layer -- ag::rms (no gamma, its hard-coded eps) followed by
        // ag::mul with the [H] gamma, differentiated by vjp_Mul (incl. the reduction over the broadcast rows) and
        // vjp_RMSNorm -- on this library's kernels, for comparison with the fused node (fp32 only: like the
        // fused node, a 16-bit gamma takes no gradient through the graph API).
        float ms_composed = 0;
        uint64_t launches_composed = 0;
        const int citers = iters < 200 ? iters : 200;
        if (!bf16) {
            auto cstep = [&] {
                Value y = mul(rms(x), gamma);
                zero_grad(y);
                backward(y, &gy);
            };
            for (int i = 0; i < warmup; ++i) cstep();
            cudaDeviceSynchronize();
            const uint64_t c0 = agb_launch_count();
            cudaEventRecord(e0, nullptr);
            for (int i = 0; i < citers; ++i) cstep();
            cudaEventRecord(e1, nullptr);
            cudaDeviceSynchronize();
            launches_composed = agb_launch_count() - c0;
            cudaEventElapsedTime(&ms_composed, e0, e1);
        }

        // captured: warm the allocator pool of the runner's stream, then record one step and replay it
        CudaGraphRunner runner;
        set_current_stream(reinterpret_cast<ag_cuda_stream_t>(runner.get_stream()));
        OwnTensor::cuda::setCurrentStream(runner.get_stream());
        Value xg = make_tensor(x.val(), "x");       // same storage, nodes created on the runner's stream
        Value gg = make_tensor(gamma.val(), "gamma");
        Value kept;                                  // the captured step's output node keeps its tensors alive
        auto gstep = [&] {
            kept = rmsnorm(xg, gg, eps);
            zero_grad(kept);
            backward(kept, &gy);
        };
        for (int i = 0; i < 3; ++i) gstep();
        runner.synchronize();
        set_current_stream(nullptr);
        OwnTensor::cuda::setCurrentStream(nullptr);
        runner.begin_capture();
        gstep();
        runner.end_capture();
        for (int i = 0; i < warmup; ++i) runner.replay();
        runner.synchronize();
        cudaEventRecord(e0, runner.get_stream());
        for (int i = 0; i < iters; ++i) runner.replay();
        cudaEventRecord(e1, runner.get_stream());
        runner.synchronize();
        float ms_graph = 0;
        cudaEventElapsedTime(&ms_graph, e0, e1);

        const double bytes = double(R) * (5.0 * H * dtype_size(dt) + 8.0);
        const double pe = ms_eager / iters, pg = ms_graph / iters;
        const int status = agb_device_status();
        std::printf("{\"rows\": %lld, \"hidden\": %lld, \"io_dtype\": \"%s\", \"iters\": %d, \"warmup\": %d, "
                    "\"eager_ms_per_step\": %.6f, \"eager_first_steps_ms\": %.6f, \"eager_gbs\": %.2f, \"graph_ms_per_step\": %.6f, \"graph_gbs\": %.2f, "
                    "\"graph_nodes\": %zu, \"launches_per_step\": %.2f, \"composed_ms_per_step\": %.6f, "
                    "\"composed_launches_per_step\": %.2f, \"device_status\": %d}\n",
                    (long long)R, (long long)H, bf16 ? "bfloat16" : "float32", iters, warmup, pe, ms_eager_head / head,
                    bytes / (pe * 1e-3) / 1e9, pg,
                    bytes / (pg * 1e-3) / 1e9, runner.num_nodes(), double(launches_eager) / iters, ms_composed / citers,
                    double(launches_composed) / citers, status);
        return status == 0 ? 0 : 1;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "bench_api: %s\n", e.what());
        return 1;
    }
}
