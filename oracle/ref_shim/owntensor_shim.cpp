// owntensor_shim.cpp -- TEST INFRASTRUCTURE: implementation of the CPU stand-in declared in
// TensorLib.h.  One rounding to fp32 per elementwise call, like a materialised tensor.
#include <algorithm>
#include <cstdlib>
#include <iomanip>
#include <unordered_map>
#include <mutex>
#include <numeric>
#include <ostream>

#include "TensorLib.h"

namespace OwnTensor {

namespace shim {
bool reduce_in_fp64 = false;
}

namespace {
std::mt19937_64 g_rng(0);
std::mutex g_rng_mu;
int64_t prod(const std::vector<int64_t>& d) {
    int64_t n = 1;
    for (auto v : d) n *= v;
    return n;
}
}  // namespace

void manual_seed(uint64_t s) {
    std::lock_guard<std::mutex> lk(g_rng_mu);
    g_rng.seed(s);
}

// Storage pool: freed buffers are kept by size and handed out again, so the dozens of [R,H]
// temporaries the reference creates per step do not each pay for fresh pages (a real tensor
// library pools its allocations too).  Buffers are NOT zero-filled.
namespace {
struct Pool {
    std::mutex mu;
    std::unordered_multimap<size_t, float*> free_list;
    size_t cached_bytes = 0;
    float* get(size_t n) {
        {
            std::lock_guard<std::mutex> lk(mu);
            auto it = free_list.find(n);
            if (it != free_list.end()) {
                float* p = it->second;
                free_list.erase(it);
                cached_bytes -= n * sizeof(float);
                return p;
            }
        }
        void* p = nullptr;
        if (posix_memalign(&p, 64, std::max<size_t>(n, 1) * sizeof(float)) != 0) throw std::bad_alloc();
        return static_cast<float*>(p);
    }
    void put(size_t n, float* p) {
        std::lock_guard<std::mutex> lk(mu);
        if (cached_bytes + n * sizeof(float) > (size_t(24) << 30)) { std::free(p); return; }
        free_list.emplace(n, p);
        cached_bytes += n * sizeof(float);
    }
};
Pool& pool() {
    static Pool* p = new Pool();
    return *p;
}
}  // namespace

Tensor::Tensor(const Shape& s, const TensorOptions& o) : shape_(s), numel_(prod(s.dims)), req_(o.requires_grad) {
    const size_t n = static_cast<size_t>(numel_);
    buf_ = std::shared_ptr<float>(pool().get(n), [n](float* p) { pool().put(n, p); });
    if (n <= 16) std::memset(buf_.get(), 0, n * sizeof(float));  // scalars and empty-shape tensors start defined
}
Tensor Tensor::zeros(const Shape& s, const TensorOptions& o) { return full(s, o, 0.0f); }
Tensor Tensor::ones(const Shape& s, const TensorOptions& o) { return full(s, o, 1.0f); }
Tensor Tensor::full(const Shape& s, const TensorOptions& o, float v) {
    Tensor t(s, o);
    t.fill(v);
    return t;
}
Tensor Tensor::randn(const Shape& s, const TensorOptions& o) {
    Tensor t(s, o);
    std::lock_guard<std::mutex> lk(g_rng_mu);
    std::normal_distribution<float> d(0.f, 1.f);
    for (int64_t i = 0; i < t.numel_; ++i) t.buf_.get()[i] = d(g_rng);
    return t;
}
Tensor Tensor::rand(const Shape& s, const TensorOptions& o) {
    Tensor t(s, o);
    std::lock_guard<std::mutex> lk(g_rng_mu);
    std::uniform_real_distribution<float> d(0.f, 1.f);
    for (int64_t i = 0; i < t.numel_; ++i) t.buf_.get()[i] = d(g_rng);
    return t;
}
Tensor Tensor::clone() const {
    Tensor t(shape_, TensorOptions().with_req_grad(req_));
    if (numel_) std::memcpy(t.data<float>(), data<float>(), sizeof(float) * numel_);
    return t;
}
Tensor Tensor::reshape(const Shape& s) const {
    if (prod(s.dims) != numel_) throw std::runtime_error("reshape: element count differs");
    Tensor t = *this;
    t.shape_ = s;
    return t;
}
Tensor Tensor::t() const {
    const auto& d = shape_.dims;
    if (d.size() < 2) return clone();
    const int64_t R = d[d.size() - 2], C = d.back(), B = numel_ / (R * C);
    Shape s = shape_;
    std::swap(s.dims[d.size() - 2], s.dims[d.size() - 1]);
    Tensor out(s, TensorOptions());
    const float* a = data<float>();
    float* o = out.data<float>();
    for (int64_t b = 0; b < B; ++b)
        for (int64_t r = 0; r < R; ++r)
            for (int64_t c = 0; c < C; ++c) o[b * R * C + c * R + r] = a[b * R * C + r * C + c];
    return out;
}
void Tensor::fill(float v) {
    float* p = buf_.get();
    const int64_t n = numel_;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) p[i] = v;
}
void Tensor::copy_(const Tensor& src) {
    if (src.numel() != numel_) throw std::runtime_error("copy_: size mismatch");
    if (numel_) std::memcpy(data<float>(), src.data<float>(), sizeof(float) * numel_);
}
void Tensor::display(std::ostream& os, int precision) const {
    os << "Tensor[";
    for (size_t i = 0; i < shape_.dims.size(); ++i) os << (i ? "," : "") << shape_.dims[i];
    os << "]";
    for (int64_t i = 0; i < numel_ && i < 32; ++i) os << " " << std::setprecision(precision) << buf_.get()[i];
    os << "\n";
}

// ------------------------------------------------------------------ broadcasting binary ops
namespace {

std::vector<int64_t> broadcast_shape(const std::vector<int64_t>& a, const std::vector<int64_t>& b) {
    const size_t n = std::max(a.size(), b.size());
    std::vector<int64_t> out(n);
    for (size_t i = 0; i < n; ++i) {
        const int64_t da = i + a.size() >= n ? a[i + a.size() - n] : 1;
        const int64_t db = i + b.size() >= n ? b[i + b.size() - n] : 1;
        if (da != db && da != 1 && db != 1) throw std::runtime_error("shapes do not broadcast");
        out[i] = std::max(da, db);
    }
    return out;
}

// strides of `d` viewed against the broadcast shape `out` (0 where broadcast)
std::vector<int64_t> bstrides(const std::vector<int64_t>& d, const std::vector<int64_t>& out) {
    std::vector<int64_t> s(out.size(), 0);
    int64_t st = 1;
    for (int i = static_cast<int>(d.size()) - 1, o = static_cast<int>(out.size()) - 1; i >= 0; --i, --o) {
        s[o] = d[i] == 1 ? 0 : st;
        st *= d[i];
    }
    return s;
}

template <typename F>
Tensor binary(const Tensor& a, const Tensor& b, F f) {
    const auto od = broadcast_shape(a.shape().dims, b.shape().dims);
    Tensor out(Shape{od}, TensorOptions());
    const int64_t n = out.numel();
    const float* pa = a.data<float>();
    const float* pb = b.data<float>();
    float* po = out.data<float>();
    if (n == 0) return out;
    const int64_t H = od.empty() ? 1 : od.back();
    const int64_t R = n / H;
    const auto sa = bstrides(a.shape().dims, od), sb = bstrides(b.shape().dims, od);
    // row base offsets: everything but the last dimension
    auto row_offset = [&](const std::vector<int64_t>& st, int64_t r) {
        int64_t off = 0;
        for (int i = static_cast<int>(od.size()) - 2; i >= 0; --i) {
            off += (r % od[i]) * st[i];
            r /= od[i];
        }
        return off;
    };
    const int64_t la = sa.empty() ? 0 : sa.back(), lb = sb.empty() ? 0 : sb.back();
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < R; ++r) {
        const float* ra = pa + row_offset(sa, r);
        const float* rb = pb + row_offset(sb, r);
        float* ro = po + r * H;
        if (la == 1 && lb == 1) for (int64_t j = 0; j < H; ++j) ro[j] = f(ra[j], rb[j]);
        else if (la == 1) { const float s = rb[0]; for (int64_t j = 0; j < H; ++j) ro[j] = f(ra[j], s); }
        else if (lb == 1) { const float s = ra[0]; for (int64_t j = 0; j < H; ++j) ro[j] = f(s, rb[j]); }
        else ro[0] = f(ra[0], rb[0]);
    }
    return out;
}

template <typename F>
Tensor with_scalar(const Tensor& a, F f) {
    Tensor out(a.shape(), TensorOptions());
    const float* pa = a.data<float>();
    float* po = out.data<float>();
    const int64_t n = a.numel();
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) po[i] = f(pa[i]);
    return out;
}

}  // namespace

Tensor operator+(const Tensor& a, const Tensor& b) { return binary(a, b, [](float x, float y) { return x + y; }); }
Tensor operator-(const Tensor& a, const Tensor& b) { return binary(a, b, [](float x, float y) { return x - y; }); }
Tensor operator*(const Tensor& a, const Tensor& b) { return binary(a, b, [](float x, float y) { return x * y; }); }
Tensor operator/(const Tensor& a, const Tensor& b) { return binary(a, b, [](float x, float y) { return x / y; }); }
Tensor operator+(const Tensor& a, double s) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return x + v; }); }
Tensor operator-(const Tensor& a, double s) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return x - v; }); }
Tensor operator*(const Tensor& a, double s) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return x * v; }); }
Tensor operator/(const Tensor& a, double s) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return x / v; }); }
Tensor operator+(double s, const Tensor& a) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return v + x; }); }
Tensor operator-(double s, const Tensor& a) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return v - x; }); }
Tensor operator*(double s, const Tensor& a) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return v * x; }); }
Tensor operator/(double s, const Tensor& a) { const float v = static_cast<float>(s); return with_scalar(a, [v](float x) { return v / x; }); }

Tensor& Tensor::operator+=(const Tensor& o) {
    // in place, the right operand may broadcast (the reference relies on that in vjp_RowSum / vjp_Sum)
    if (o.shape().dims == shape_.dims) {
        float* a = data<float>();
        const float* b = o.data<float>();
        const int64_t n = numel_;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) a[i] = a[i] + b[i];
        return *this;
    }
    Tensor sum = *this + o;
    if (sum.numel() != numel_) throw std::runtime_error("operator+=: result does not fit the left operand");
    std::memcpy(data<float>(), sum.data<float>(), sizeof(float) * numel_);
    return *this;
}

Tensor& Tensor::operator-=(const Tensor& o) {
    Tensor d = *this - o;
    if (d.numel() != numel_) throw std::runtime_error("operator-=: result does not fit the left operand");
    std::memcpy(data<float>(), d.data<float>(), sizeof(float) * numel_);
    return *this;
}
Tensor& Tensor::operator*=(double s) {
    const float v = static_cast<float>(s);
    float* a = data<float>();
    for (int64_t i = 0; i < numel_; ++i) a[i] = a[i] * v;
    return *this;
}

#define OWNTENSOR_SHIM_UNARY(name, expr) \
    Tensor name(const Tensor& a, cudaStream_t) { return with_scalar(a, [](float x) { return expr; }); }
OWNTENSOR_SHIM_UNARY(exp, std::exp(x)) OWNTENSOR_SHIM_UNARY(log, std::log(x)) OWNTENSOR_SHIM_UNARY(sqrt, std::sqrt(x))
OWNTENSOR_SHIM_UNARY(tanh, std::tanh(x)) OWNTENSOR_SHIM_UNARY(abs, std::fabs(x))
OWNTENSOR_SHIM_UNARY(sign, static_cast<float>((x > 0.f) - (x < 0.f))) OWNTENSOR_SHIM_UNARY(sin, std::sin(x))
OWNTENSOR_SHIM_UNARY(cos, std::cos(x)) OWNTENSOR_SHIM_UNARY(tan, std::tan(x)) OWNTENSOR_SHIM_UNARY(sinh, std::sinh(x))
OWNTENSOR_SHIM_UNARY(cosh, std::cosh(x)) OWNTENSOR_SHIM_UNARY(asin, std::asin(x)) OWNTENSOR_SHIM_UNARY(acos, std::acos(x))
OWNTENSOR_SHIM_UNARY(atan, std::atan(x)) OWNTENSOR_SHIM_UNARY(asinh, std::asinh(x)) OWNTENSOR_SHIM_UNARY(acosh, std::acosh(x))
OWNTENSOR_SHIM_UNARY(atanh, std::atanh(x))
#undef OWNTENSOR_SHIM_UNARY
Tensor square(const Tensor& a, cudaStream_t) { return with_scalar(a, [](float x) { return x * x; }); }
Tensor pow(const Tensor& a, float e, cudaStream_t) { return with_scalar(a, [e](float x) { return std::pow(x, e); }); }

// ------------------------------------------------------------------ reductions
namespace {
enum RedOp { kSum, kMean, kMax };

Tensor reduce(const Tensor& a, const std::vector<int64_t>& axes_in, bool keepdim, RedOp op) {
    const auto& d = a.shape().dims;
    const int nd = static_cast<int>(d.size());
    std::vector<bool> red(nd, axes_in.empty());
    for (auto ax : axes_in) {
        if (ax < 0) ax += nd;
        if (ax < 0 || ax >= nd) throw std::runtime_error("reduce: axis out of range");
        red[ax] = true;
    }
    std::vector<int64_t> od;
    for (int i = 0; i < nd; ++i) {
        if (!red[i]) od.push_back(d[i]);
        else if (keepdim) od.push_back(1);
    }
    if (od.empty()) od.push_back(1);
    Tensor out(Shape{od}, TensorOptions());
    const float* pa = a.data<float>();
    float* po = out.data<float>();
    const bool f64 = shim::reduce_in_fp64;
    auto finish = [&](double sd, float sf, float mx, int64_t count) -> float {
        if (op == kMax) return mx;
        if (op == kSum) return f64 ? static_cast<float>(sd) : sf;
        return f64 ? static_cast<float>(sd / static_cast<double>(count)) : sf / static_cast<float>(count);
    };
    // split dims into leading-reduced / kept / trailing patterns the path uses
    const bool all = std::all_of(red.begin(), red.end(), [](bool b) { return b; });
    const bool last_only = nd >= 1 && red[nd - 1] && std::none_of(red.begin(), red.end() - 1, [](bool b) { return b; });
    const bool lead_only = nd >= 2 && !red[nd - 1] && std::all_of(red.begin(), red.end() - 1, [](bool b) { return b; });
    if (all) {
        double sd = 0;
        float sf = 0, mx = a.numel() ? pa[0] : 0.f;
        for (int64_t i = 0; i < a.numel(); ++i) { sd += pa[i]; sf += pa[i]; mx = std::max(mx, pa[i]); }
        po[0] = finish(sd, sf, mx, a.numel());
    } else if (last_only) {
        const int64_t H = d[nd - 1], R = a.numel() / H;
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < R; ++r) {
            const float* row = pa + r * H;
            double sd = 0;
            float sf = 0, mx = row[0];
            for (int64_t j = 0; j < H; ++j) { sd += row[j]; sf += row[j]; mx = std::max(mx, row[j]); }
            po[r] = finish(sd, sf, mx, H);
        }
    } else if (lead_only) {
        const int64_t H = d[nd - 1], R = a.numel() / H;
        const int64_t CB = 256;
#pragma omp parallel for schedule(static)
        for (int64_t j0 = 0; j0 < H; j0 += CB) {
            const int64_t w = std::min<int64_t>(CB, H - j0);
            double sd[256];
            float sf[256], mx[256];
            for (int64_t j = 0; j < w; ++j) { sd[j] = 0; sf[j] = 0; mx[j] = pa[j0 + j]; }
            for (int64_t r = 0; r < R; ++r) {
                const float* row = pa + r * H + j0;
                for (int64_t j = 0; j < w; ++j) { sd[j] += row[j]; sf[j] += row[j]; mx[j] = std::max(mx[j], row[j]); }
            }
            for (int64_t j = 0; j < w; ++j) po[j0 + j] = finish(sd[j], sf[j], mx[j], R);
        }
    } else {
        // general case: walk every input element, accumulate into its output cell (fp64 scratch)
        std::vector<int64_t> ostride(nd, 0);
        int64_t st = 1;
        for (int i = nd - 1; i >= 0; --i)
            if (!red[i]) { ostride[i] = st; st *= d[i]; }
        const int64_t on = out.numel();
        std::vector<double> sd(on, 0.0);
        std::vector<float> sf(on, 0.f), mx(on, -INFINITY);
        std::vector<int64_t> idx(nd, 0);
        for (int64_t i = 0; i < a.numel(); ++i) {
            int64_t o = 0;
            for (int k = 0; k < nd; ++k) o += idx[k] * ostride[k];
            sd[o] += pa[i]; sf[o] += pa[i]; mx[o] = std::max(mx[o], pa[i]);
            for (int k = nd - 1; k >= 0; --k) { if (++idx[k] < d[k]) break; idx[k] = 0; }
        }
        const int64_t count = on ? a.numel() / on : 0;
        for (int64_t o = 0; o < on; ++o) po[o] = finish(sd[o], sf[o], mx[o], count);
    }
    return out;
}
}  // namespace

Tensor reduce_sum(const Tensor& a, const std::vector<int64_t>& axes, bool keepdim) { return reduce(a, axes, keepdim, kSum); }
Tensor reduce_mean(const Tensor& a, const std::vector<int64_t>& axes, bool keepdim) { return reduce(a, axes, keepdim, kMean); }
Tensor reduce_max(const Tensor& a, const std::vector<int64_t>& axes, bool keepdim) { return reduce(a, axes, keepdim, kMax); }

Tensor matmul(const Tensor& a, const Tensor& b) {
    const auto& da = a.shape().dims;
    const auto& db = b.shape().dims;
    if (da.size() != 2 || db.size() != 2 || da[1] != db[0]) throw std::runtime_error("matmul: 2-D operands with matching inner size only");
    const int64_t M = da[0], K = da[1], N = db[1];
    Tensor out(Shape{{M, N}}, TensorOptions());
    const float* pa = a.data<float>();
    const float* pb = b.data<float>();
    float* po = out.data<float>();
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
            float s = 0.f;
            for (int64_t k = 0; k < K; ++k) s += pa[i * K + k] * pb[k * N + j];
            po[i * N + j] = s;
        }
    return out;
}

}  // namespace OwnTensor
