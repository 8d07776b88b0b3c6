// TensorLib.h -- TEST INFRASTRUCTURE.  A small CPU-only stand-in for the OwnTensor library
// (git submodule `tensor` of cgadimpl, absent from the reference checkout), written from the call
// sites in cgadimpl's sources, so that the reference's OWN op builders and autodiff rules
// (cgadimpl/src/ops/*.cpp, src/autodiff/*.cpp, src/core/*.cpp) can be compiled where they lie
// and run: this pins the reference's composition -- which tensor calls are made, in which order,
// with which temporaries.  What it cannot pin is OwnTensor's own arithmetic: every elementwise
// call here rounds once to fp32, and reductions run left to right in fp32 or, when
// OwnTensor::shim::reduce_in_fp64 is set, in fp64 rounded once.
// fp32 only; numpy-style broadcasting; OpenMP over the outer dimension.
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <iosfwd>
#include <memory>
#include <random>
#include <stdexcept>
#include <type_traits>
#include <vector>

namespace OwnTensor {

namespace shim {
extern bool reduce_in_fp64;
}

enum class Dtype : int { Float32 = 0, Float16, Bfloat16, Float64, Int32, Int64 };
enum class Device : int { CPU = 0, CUDA = 1 };

struct complex32_t { float re{}, im{}; complex32_t() = default; complex32_t(float r) : re(r) {} float real() const { return re; } };
struct complex64_t { float re{}, im{}; complex64_t() = default; complex64_t(float r) : re(r) {} float real() const { return re; } };
struct complex128_t { double re{}, im{}; complex128_t() = default; complex128_t(float r) : re(r) {} double real() const { return re; } };

struct DeviceIndex {
    Device device{Device::CPU};
    int index{0};
    DeviceIndex() = default;
    DeviceIndex(Device d, int i = 0) : device(d), index(i) {}
    bool is_cpu() const { return device == Device::CPU; }
    bool is_cuda() const { return device == Device::CUDA; }
    bool operator==(const DeviceIndex& o) const { return device == o.device && index == o.index; }
    bool operator!=(const DeviceIndex& o) const { return !(*this == o); }
    bool operator==(Device d) const { return device == d; }
    bool operator!=(Device d) const { return device != d; }
};

struct Shape {
    std::vector<int64_t> dims;
};

struct TensorOptions {
    Dtype dtype{Dtype::Float32};
    DeviceIndex device{};
    bool requires_grad{false};
    TensorOptions with_dtype(Dtype d) const { auto o = *this; o.dtype = d; return o; }
    TensorOptions with_device(DeviceIndex d) const { auto o = *this; o.device = d; return o; }
    TensorOptions with_device(Device d) const { return with_device(DeviceIndex(d)); }
    TensorOptions with_req_grad(bool r) const { auto o = *this; o.requires_grad = r; return o; }
};

class Tensor {
public:
    Tensor() = default;
    Tensor(const Shape& s, const TensorOptions& o = {});
    Tensor(const Shape& s, Dtype) : Tensor(s, TensorOptions()) {}

    static Tensor zeros(const Shape& s, const TensorOptions& o = {});
    static Tensor ones(const Shape& s, const TensorOptions& o = {});
    static Tensor full(const Shape& s, const TensorOptions& o, float v);
    static Tensor randn(const Shape& s, const TensorOptions& o = {});
    static Tensor rand(const Shape& s, const TensorOptions& o = {});

    const Shape& shape() const { return shape_; }
    int64_t numel() const { return numel_; }
    Dtype dtype() const { return Dtype::Float32; }
    DeviceIndex device() const { return DeviceIndex(Device::CPU); }
    bool requires_grad() const { return req_; }
    bool is_cpu() const { return true; }
    bool is_cuda() const { return false; }

    template <typename T> T* data() { return reinterpret_cast<T*>(buf_.get()); }
    template <typename T> const T* data() const { return reinterpret_cast<const T*>(buf_.get()); }

    Tensor to_cpu() const { return *this; }
    Tensor to(DeviceIndex) const { return *this; }
    Tensor clone() const;
    Tensor reshape(const Shape& s) const;
    Tensor t() const;  // swaps the last two dimensions
    void fill(float v);
    void copy_(const Tensor& src);
    void display(std::ostream& os, int precision = 4) const;

    Tensor& operator+=(const Tensor& o);
    Tensor& operator-=(const Tensor& o);
    Tensor& operator*=(double s);

private:
    std::shared_ptr<float> buf_;  // uninitialised storage from a size-keyed pool (see owntensor_shim.cpp)
    Shape shape_;
    int64_t numel_{0};
    bool req_{false};
};

Tensor operator+(const Tensor& a, const Tensor& b);
Tensor operator-(const Tensor& a, const Tensor& b);
Tensor operator*(const Tensor& a, const Tensor& b);
Tensor operator/(const Tensor& a, const Tensor& b);
Tensor operator+(const Tensor& a, double s);
Tensor operator-(const Tensor& a, double s);
Tensor operator*(const Tensor& a, double s);
Tensor operator/(const Tensor& a, double s);
Tensor operator+(double s, const Tensor& a);
Tensor operator-(double s, const Tensor& a);
Tensor operator*(double s, const Tensor& a);
Tensor operator/(double s, const Tensor& a);

#define OWNTENSOR_SHIM_UNARY(name) Tensor name(const Tensor& a, cudaStream_t stream = nullptr);
OWNTENSOR_SHIM_UNARY(exp) OWNTENSOR_SHIM_UNARY(log) OWNTENSOR_SHIM_UNARY(sqrt) OWNTENSOR_SHIM_UNARY(tanh)
OWNTENSOR_SHIM_UNARY(abs) OWNTENSOR_SHIM_UNARY(sign) OWNTENSOR_SHIM_UNARY(sin) OWNTENSOR_SHIM_UNARY(cos)
OWNTENSOR_SHIM_UNARY(tan) OWNTENSOR_SHIM_UNARY(sinh) OWNTENSOR_SHIM_UNARY(cosh) OWNTENSOR_SHIM_UNARY(asin)
OWNTENSOR_SHIM_UNARY(acos) OWNTENSOR_SHIM_UNARY(atan) OWNTENSOR_SHIM_UNARY(asinh) OWNTENSOR_SHIM_UNARY(acosh)
OWNTENSOR_SHIM_UNARY(atanh)
#undef OWNTENSOR_SHIM_UNARY
Tensor pow(const Tensor& a, float e, cudaStream_t stream = nullptr);
Tensor square(const Tensor& a, cudaStream_t stream = nullptr);

Tensor reduce_sum(const Tensor& a, const std::vector<int64_t>& axes = {}, bool keepdim = false);
Tensor reduce_mean(const Tensor& a, const std::vector<int64_t>& axes = {}, bool keepdim = false);
Tensor reduce_max(const Tensor& a, const std::vector<int64_t>& axes = {}, bool keepdim = false);
Tensor matmul(const Tensor& a, const Tensor& b);

namespace cuda {
inline void setCurrentStream(cudaStream_t) {}
}

template <typename F>
void dispatch_by_dtype(Dtype, F&& f) {
    f(float{});  // the stand-in holds fp32 only
}

void manual_seed(uint64_t seed);

}  // namespace OwnTensor
