// TensorLib.h -- the minimal device tensor the RMSNorm path needs, under the names cgadimpl's code
// uses for its third-party tensor library (namespace OwnTensor: Tensor, Shape, TensorOptions, Dtype,
// Device, DeviceIndex; cgadimpl/include/tensor.hpp:6-15 re-exports them).  It is a from-scratch
// stand-in for the parts of that API seen at the call sites of the path: storage, factories, host
// <-> device copies and a stream-ordered caching device allocator.  Arithmetic is NOT here: the ops
// and autodiff rules call the CUDA library (agb.h) on raw pointers.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <iosfwd>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace OwnTensor {

enum class Dtype : uint8_t { Float32 = 0, Bfloat16 = 1, Float64 = 2 };
enum class Device : uint8_t { CPU = 0, CUDA = 1 };

inline size_t dtype_size(Dtype d) { return d == Dtype::Float32 ? 4 : (d == Dtype::Bfloat16 ? 2 : 8); }

struct DeviceIndex {
    Device device{Device::CPU};
    int index{0};
    DeviceIndex() = default;
    DeviceIndex(Device d, int i = 0) : device(d), index(i) {}
    bool is_cuda() const { return device == Device::CUDA; }
    bool operator==(const DeviceIndex& o) const { return device == o.device && index == o.index; }
    bool operator!=(const DeviceIndex& o) const { return !(*this == o); }
};

struct Shape {
    std::vector<int64_t> dims;
    Shape() = default;
    Shape(std::vector<int64_t> d) : dims(std::move(d)) {}
    Shape(std::initializer_list<int64_t> d) : dims(d) {}
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : dims) n *= d;
        return n;
    }
    bool operator==(const Shape& o) const { return dims == o.dims; }
};

struct TensorOptions {
    Dtype dtype{Dtype::Float32};
    DeviceIndex device{};
    bool requires_grad{false};
    TensorOptions with_dtype(Dtype d) const { TensorOptions o = *this; o.dtype = d; return o; }
    TensorOptions with_device(DeviceIndex d) const { TensorOptions o = *this; o.device = d; return o; }
    TensorOptions with_device(Device d) const { return with_device(DeviceIndex(d)); }
    TensorOptions with_req_grad(bool r) const { TensorOptions o = *this; o.requires_grad = r; return o; }
};

// ------------------------------------------------------------------ CUDA plumbing
namespace cuda {

// Thread-local "current stream" of the tensor library (the reference sets it next to its own,
// cgadimpl/src/runtime/cuda_graphs.cpp:37-38).
void setCurrentStream(cudaStream_t s);
cudaStream_t getCurrentStream();

struct AllocatorStats {
    size_t bytes_in_use{0}, bytes_cached{0}, device_allocs{0}, cache_hits{0}, peak_in_use{0};
};

// Stream-ordered caching device allocator.  A block freed on stream S is handed out again only to
// requests made on S (stream order then makes the reuse safe without events).  A request that
// misses the cache calls cudaMalloc -- except while the requesting stream is being captured into a
// CUDA graph, where it throws: warm the cache (run once, or reserve()) before capturing.
class DeviceAllocator {
public:
    static DeviceAllocator& instance();
    void* allocate(size_t bytes, int device, cudaStream_t stream);
    void release(void* ptr);                       // returns the block to its stream's cache
    bool owns(void* ptr) const;                    // true for a live block handed out by allocate()
    void reserve(size_t bytes, int device, cudaStream_t stream);  // pre-populates the cache with one block
    void empty_cache();                            // cudaFree of every cached (not in-use) block
    void set_memory_limit(size_t bytes);           // 0 = unlimited; exceeding it throws (never calls cudaMalloc)
    AllocatorStats stats() const;
    ~DeviceAllocator();
private:
    DeviceAllocator();
    struct Impl;
    Impl* impl_;
};

}  // namespace cuda

void manual_seed(uint64_t seed);  // seeds randn / rand (host generator, then copied to the device)

// ------------------------------------------------------------------ Tensor
class Tensor {
public:
    Tensor();                                             // empty (numel 0, no storage)
    Tensor(const Shape& shape, const TensorOptions& opts);  // uninitialised storage

    static Tensor zeros(const Shape& s, const TensorOptions& o = {});
    static Tensor ones(const Shape& s, const TensorOptions& o = {});
    static Tensor full(const Shape& s, const TensorOptions& o, float value);
    static Tensor randn(const Shape& s, const TensorOptions& o = {});
    static Tensor rand(const Shape& s, const TensorOptions& o = {});
    static Tensor from_host(const float* data, const Shape& s, const TensorOptions& o = {});

    const Shape& shape() const { return shape_; }
    int64_t numel() const { return numel_; }
    Dtype dtype() const { return opts_.dtype; }
    DeviceIndex device() const { return opts_.device; }
    bool requires_grad() const { return opts_.requires_grad; }
    void set_requires_grad(bool r) { opts_.requires_grad = r; }
    bool is_cuda() const { return opts_.device.is_cuda(); }
    size_t nbytes() const { return static_cast<size_t>(numel_) * dtype_size(opts_.dtype); }
    bool defined() const { return static_cast<bool>(storage_); }

    template <typename T> T* data() { return static_cast<T*>(raw()); }
    template <typename T> const T* data() const { return static_cast<const T*>(raw()); }
    void* raw() const;

    Tensor to_cpu() const;                    // synchronises the producing stream
    Tensor to(DeviceIndex dev) const;
    Tensor clone() const;
    Tensor reshape(const Shape& s) const;     // shares storage
    void copy_(const Tensor& src);            // same numel and dtype; any device pair
    void fill(float v);
    void zero_();
    std::vector<float> to_vector() const;     // host copy widened to float
    void display(std::ostream& os, int precision = 4) const;

private:
    struct Storage;
    std::shared_ptr<Storage> storage_;
    Shape shape_;
    int64_t numel_{0};
    TensorOptions opts_;
};

}  // namespace OwnTensor
