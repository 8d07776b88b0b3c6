// test_core_ops_gpu.cpp -- the reference's own gradient checks for the ops on this path
// (cgadimpl/Tests/test_core_ops_gpu.cpp): central finite differences against backward(), max-abs
// error <= 1e-3, on the same shapes: RMSNorm randn [4,10] (:262-267), broadcast Add and Mul
// [4,5] (.) [1,5] including the reduced gradient of the broadcast operand (:182-205), Sum, Mean,
// RowSum (:216-233).  Two deviations keep the check's own noise under its tolerance: the step is
// 1e-2 instead of 1e-4 (fp32 forward values carry ~1e-7 of rounding; 1e-7 / 2e-4 ~ 1e-3), and the
// perturbed losses are summed on the host in double.
#include "ad/ag_all.hpp"
#include "check.hpp"

using namespace ag;

static bool check_grad(const Tensor& analytical, const std::vector<float>& numerical, double tol = 1e-3) {
    auto a = analytical.to_vector();
    if (a.size() != numerical.size()) { std::fprintf(stderr, "  shape mismatch\n"); return false; }
    double err = 0;
    for (size_t i = 0; i < a.size(); ++i) err = std::max(err, std::fabs(double(a[i]) - double(numerical[i])));
    if (err > tol) std::fprintf(stderr, "  max error %.3e > %.1e\n", err, tol);
    return err <= tol;
}

static double host_sum(const Value& v) {
    double s = 0;
    for (float f : v.val().to_vector()) s += f;
    return s;
}

// d sum(func()) / d param by central differences, one element at a time
static std::vector<float> numerical_gradient(Value& param, const std::function<Value()>& func, double h = 1e-2) {
    const Tensor original = param.val().clone();
    const std::vector<float> base = original.to_vector();
    std::vector<float> grad(base.size());
    const DeviceIndex dev = param.val().device();
    for (size_t i = 0; i < base.size(); ++i) {
        std::vector<float> p = base;
        p[i] = static_cast<float>(base[i] + h);
        param.val() = Tensor::from_host(p.data(), original.shape(), ag::options(original)).to(dev);
        const double l1 = host_sum(func());
        p[i] = static_cast<float>(base[i] - h);
        param.val() = Tensor::from_host(p.data(), original.shape(), ag::options(original)).to(dev);
        const double l2 = host_sum(func());
        grad[i] = static_cast<float>((l1 - l2) / (2.0 * h));
    }
    param.val() = original;
    return grad;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 2; }
    OwnTensor::manual_seed(1234);
    const auto opts = TensorOptions().with_device(DeviceIndex(Device::CUDA)).with_req_grad(true);

    run_test("Add (Broadcast)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        Value b = make_tensor(Tensor::randn(Shape{{1, 5}}, opts));
        auto f = [&] { return a + b; };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        CHECK(check_grad(b.grad(), numerical_gradient(b, f)));
    });
    run_test("Mul (Broadcast)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        Value b = make_tensor(Tensor::randn(Shape{{1, 5}}, opts));
        auto f = [&] { return a * b; };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        CHECK(check_grad(b.grad(), numerical_gradient(b, f)));
    });
    run_test("Mul (row statistic and scalar literal)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        Value s = make_tensor(Tensor::randn(Shape{{4, 1}}, opts));
        auto f = [&] { return (a * s) * 0.5f; };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        CHECK(check_grad(s.grad(), numerical_gradient(s, f)));
    });
    run_test("Sum (all)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        auto f = [&] { return sum(a); };
        backward(f());
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
    });
    run_test("Mean (all)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        auto f = [&] { return mean_all(a); };
        backward(f());
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
    });
    run_test("RowSum", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        auto f = [&] { return rowsum(a); };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
    });
    run_test("RowMax forward; its VJP throws like the reference", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 5}}, opts));
        auto v = a.val().to_vector(), m = rowmax(a).val().to_vector();
        for (int r = 0; r < 4; ++r) {
            float want = v[r * 5];
            for (int j = 1; j < 5; ++j) want = std::max(want, v[r * 5 + j]);
            CHECK(m[r] == want);
        }
        bool threw = false;
        try { backward(sum(rowmax(a))); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
    });
    run_test("LayerNorm", [&] {                                   // test_core_ops_gpu.cpp:256-261
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, opts));
        auto f = [&] { return laynor(a); };
        // sum(laynor(a)) is identically zero, so weight the outputs to get a non-trivial gradient
        Value w = make_tensor(Tensor::randn(Shape{{4, 10}}, opts.with_req_grad(false)));
        auto fw = [&] { return laynor(a) * w; };
        backward(sum(fw()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, fw)));
        // forward mode (the reference's jvp_LayerNorm throws; implemented here): central differences along t
        Value y = f();
        Tensor t = Tensor::randn(Shape{{4, 10}}, opts.with_req_grad(false));
        Tensor jt = jvp(y, {{a.node.get(), t}});
        const auto tv = t.to_vector(), base = a.val().to_vector();
        std::vector<float> plus(base), minus(base);
        for (size_t i = 0; i < base.size(); ++i) { plus[i] = float(base[i] + 1e-2 * tv[i]); minus[i] = float(base[i] - 1e-2 * tv[i]); }
        const Tensor keep = a.val().clone();
        a.val() = Tensor::from_host(plus.data(), keep.shape(), ag::options(keep)).to(keep.device());
        const auto yp = f().val().to_vector();
        a.val() = Tensor::from_host(minus.data(), keep.shape(), ag::options(keep)).to(keep.device());
        const auto ym = f().val().to_vector();
        a.val() = keep;
        std::vector<float> fd(yp.size());
        for (size_t i = 0; i < fd.size(); ++i) fd[i] = float((double(yp[i]) - double(ym[i])) / 2e-2);
        CHECK(check_grad(jt, fd));
    });
    run_test("RMSNorm", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, opts));
        auto f = [&] { return rms(a); };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
    });
    run_test("RMSNorm with per-channel gamma (fused node)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, opts));
        Value g = make_tensor(Tensor::randn(Shape{{10}}, opts));
        auto f = [&] { return rmsnorm(a, g, 1e-6f); };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        CHECK(check_grad(g.grad(), numerical_gradient(g, f)));
    });
    run_test("RealRMSNorm (scalar gain; the reference's rules throw)", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, opts));
        auto f = [&] { return realrms(a, 1.5f); };
        Value y = f();
        Node* G = y.node->inputs[1].get();
        zero_grad(y);
        backward(sum(y));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        // dG = sum(yhat): compare with the sum of rms(a)
        const double want = host_sum(rms(a));
        CHECK(std::fabs(G->grad.to_vector()[0] - want) <= 1e-3);
    });
    run_test("SoftmaxRow", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, opts));
        // sum(softmax(a)) is identically 4, so weight the outputs to get a non-trivial gradient
        Value w = make_tensor(Tensor::randn(Shape{{4, 10}}, opts.with_req_grad(false)));
        auto f = [&] { return softmax_row(a) * w; };
        backward(sum(f()));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        // forward-mode against the same finite differences: J t for a tangent t on `a`
        Value y = softmax_row(a);
        Tensor t = Tensor::randn(Shape{{4, 10}}, opts.with_req_grad(false));
        Tensor jt = jvp(y, {{a.node.get(), t}});
        const auto tv = t.to_vector(), base = a.val().to_vector();
        std::vector<float> plus(base), minus(base);
        for (size_t i = 0; i < base.size(); ++i) { plus[i] = float(base[i] + 1e-2 * tv[i]); minus[i] = float(base[i] - 1e-2 * tv[i]); }
        const Tensor keep = a.val().clone();
        a.val() = Tensor::from_host(plus.data(), keep.shape(), ag::options(keep)).to(keep.device());
        const auto yp = softmax_row(a).val().to_vector();
        a.val() = Tensor::from_host(minus.data(), keep.shape(), ag::options(keep)).to(keep.device());
        const auto ym = softmax_row(a).val().to_vector();
        a.val() = keep;
        std::vector<float> fd(yp.size());
        for (size_t i = 0; i < fd.size(); ++i) fd[i] = float((double(yp[i]) - double(ym[i])) / 2e-2);
        CHECK(check_grad(jt, fd));
    });
    run_test("LogSumExpRow", [&] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, opts));
        auto f = [&] { return logsumexp_row(a); };
        Value y = f();
        CHECK(y.shape() == std::vector<int64_t>({4, 1}));
        backward(sum(y));
        CHECK(check_grad(a.grad(), numerical_gradient(a, f)));
        // d logsumexp / dz = softmax(z): with the all-ones seed the gradient IS the softmax, bit for bit
        CHECK(a.grad().to_vector() == softmax_row(a).val().to_vector());
        Tensor t = Tensor::randn(Shape{{4, 10}}, opts.with_req_grad(false));
        Tensor jt = jvp(y, {{a.node.get(), t}});
        CHECK(jt.shape().dims == std::vector<int64_t>({4, 1}));
        const auto sm = softmax_row(a).val().to_vector(), tv = t.to_vector(), got = jt.to_vector();
        for (int r = 0; r < 4; ++r) {
            double want = 0;
            for (int j = 0; j < 10; ++j) want += double(sm[r * 10 + j]) * tv[r * 10 + j];
            CHECK(std::fabs(got[r] - want) <= 1e-5);
        }
    });
    cudaDeviceSynchronize();
    return finish("test_core_ops_gpu");
}
