// tensor.cpp -- storage, factories, copies and the caching device allocator behind TensorLib.h.
#include "TensorLib.h"

#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <iomanip>
#include <map>
#include <mutex>
#include <ostream>
#include <random>
#include <unordered_map>

namespace OwnTensor {

namespace {
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess)
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}
std::mt19937_64& rng() {
    static std::mt19937_64 g(0);
    return g;
}
std::mutex& rng_mu() {
    static std::mutex m;
    return m;
}
uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
float bf16_to_f32(uint16_t b) {
    uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
}  // namespace

void manual_seed(uint64_t seed) {
    std::lock_guard<std::mutex> lk(rng_mu());
    rng().seed(seed);
}

// ------------------------------------------------------------------ streams
namespace cuda {
namespace {
thread_local cudaStream_t t_stream = nullptr;
}
void setCurrentStream(cudaStream_t s) { t_stream = s; }
cudaStream_t getCurrentStream() { return t_stream; }

// ------------------------------------------------------------------ allocator
struct DeviceAllocator::Impl {
    struct Block {
        void* ptr;
        size_t size;
        int device;
        cudaStream_t stream;
    };
    struct Key {
        int device;
        cudaStream_t stream;
        bool operator<(const Key& o) const { return device != o.device ? device < o.device : stream < o.stream; }
    };
    std::mutex mu;
    std::map<Key, std::multimap<size_t, Block>> cache;  // free blocks by (device, stream), then size
    std::unordered_map<void*, Block> live;
    AllocatorStats st;
    size_t limit = 0;
    size_t device_bytes = 0;  // everything obtained from cudaMalloc and not yet cudaFree'd

    static size_t round_size(size_t n) {
        if (n == 0) n = 1;
        const size_t g = n < (1u << 20) ? 512 : (n < (64u << 20) ? (1u << 20) : (16u << 20));
        return (n + g - 1) / g * g;
    }
};

DeviceAllocator::DeviceAllocator() : impl_(new Impl) {}
DeviceAllocator::~DeviceAllocator() {
    // Process exit: the driver reclaims device memory; calling cudaFree here could run after the
    // runtime has shut down.
    delete impl_;
}
DeviceAllocator& DeviceAllocator::instance() {
    static DeviceAllocator* a = new DeviceAllocator();  // intentionally leaked, see the destructor
    return *a;
}

void* DeviceAllocator::allocate(size_t bytes, int device, cudaStream_t stream) {
    const size_t need = Impl::round_size(bytes);
    std::lock_guard<std::mutex> lk(impl_->mu);
    auto& pool = impl_->cache[{device, stream}];
    auto it = pool.lower_bound(need);
    // accept a cached block up to 25 % (or 1 MB) larger than needed
    if (it != pool.end() && it->first <= need + std::max<size_t>(need / 4, 1u << 20)) {
        Impl::Block b = it->second;
        pool.erase(it);
        impl_->live[b.ptr] = b;
        impl_->st.cache_hits++;
        impl_->st.bytes_cached -= b.size;
        impl_->st.bytes_in_use += b.size;
        impl_->st.peak_in_use = std::max(impl_->st.peak_in_use, impl_->st.bytes_in_use);
        return b.ptr;
    }
    if (impl_->limit && impl_->device_bytes + need > impl_->limit)
        throw std::runtime_error("DeviceAllocator: out of memory (limit " + std::to_string(impl_->limit) +
                                 " bytes, in use or cached " + std::to_string(impl_->device_bytes) + ", requested " +
                                 std::to_string(need) + ")");
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (stream != nullptr && cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        throw std::runtime_error(
            "DeviceAllocator: cache miss while the stream is being captured into a CUDA graph; run the "
            "same code once before capturing (or reserve()) so every buffer comes from the cache");
    int prev = 0;
    cuda_check(cudaGetDevice(&prev), "cudaGetDevice");
    if (prev != device) cuda_check(cudaSetDevice(device), "cudaSetDevice");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, need);
    if (prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("DeviceAllocator: cudaMalloc of ") + std::to_string(need) +
                                 " bytes failed: " + cudaGetErrorString(e));
    }
    Impl::Block b{p, need, device, stream};
    impl_->live[p] = b;
    impl_->device_bytes += need;
    impl_->st.device_allocs++;
    impl_->st.bytes_in_use += need;
    impl_->st.peak_in_use = std::max(impl_->st.peak_in_use, impl_->st.bytes_in_use);
    return p;
}

void DeviceAllocator::release(void* ptr) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lk(impl_->mu);
    auto it = impl_->live.find(ptr);
    if (it == impl_->live.end()) return;
    Impl::Block b = it->second;
    impl_->live.erase(it);
    impl_->cache[{b.device, b.stream}].emplace(b.size, b);
    impl_->st.bytes_in_use -= b.size;
    impl_->st.bytes_cached += b.size;
}

bool DeviceAllocator::owns(void* ptr) const {
    std::lock_guard<std::mutex> lk(impl_->mu);
    return impl_->live.count(ptr) != 0;
}

void DeviceAllocator::reserve(size_t bytes, int device, cudaStream_t stream) { release(allocate(bytes, device, stream)); }

void DeviceAllocator::empty_cache() {
    std::lock_guard<std::mutex> lk(impl_->mu);
    for (auto& kv : impl_->cache)
        for (auto& bk : kv.second) {
            cudaFree(bk.second.ptr);
            impl_->device_bytes -= bk.second.size;
            impl_->st.bytes_cached -= bk.second.size;
        }
    impl_->cache.clear();
}
void DeviceAllocator::set_memory_limit(size_t bytes) {
    std::lock_guard<std::mutex> lk(impl_->mu);
    impl_->limit = bytes;
}
AllocatorStats DeviceAllocator::stats() const {
    std::lock_guard<std::mutex> lk(impl_->mu);
    return impl_->st;
}
}  // namespace cuda

// ------------------------------------------------------------------ storage
struct Tensor::Storage {
    void* ptr{nullptr};
    size_t bytes{0};
    DeviceIndex dev;
    Storage(size_t n, DeviceIndex d) : bytes(n), dev(d) {
        if (d.is_cuda()) {
            ptr = cuda::DeviceAllocator::instance().allocate(n, d.index, cuda::getCurrentStream());
        } else {
            ptr = std::aligned_alloc(64, (std::max<size_t>(n, 1) + 63) / 64 * 64);
            if (!ptr) throw std::bad_alloc();
        }
    }
    ~Storage() {
        if (dev.is_cuda()) cuda::DeviceAllocator::instance().release(ptr);
        else std::free(ptr);
    }
    Storage(const Storage&) = delete;
    Storage& operator=(const Storage&) = delete;
};

Tensor::Tensor() = default;
Tensor::Tensor(const Shape& shape, const TensorOptions& opts) : shape_(shape), numel_(shape.numel()), opts_(opts) {
    for (auto d : shape.dims)
        if (d < 0) throw std::invalid_argument("Tensor: negative dimension");
    storage_ = std::make_shared<Storage>(nbytes(), opts.device);
}
void* Tensor::raw() const { return storage_ ? storage_->ptr : nullptr; }

namespace {
// Host float -> tensor of any dtype / device.
void upload(Tensor& t, const std::vector<float>& host) {
    const int64_t n = t.numel();
    std::vector<unsigned char> staged;
    const void* src = host.data();
    if (t.dtype() == Dtype::Bfloat16) {
        staged.resize(static_cast<size_t>(n) * 2);
        auto* o = reinterpret_cast<uint16_t*>(staged.data());
        for (int64_t i = 0; i < n; ++i) o[i] = f32_to_bf16(host[i]);
        src = staged.data();
    } else if (t.dtype() == Dtype::Float64) {
        staged.resize(static_cast<size_t>(n) * 8);
        auto* o = reinterpret_cast<double*>(staged.data());
        for (int64_t i = 0; i < n; ++i) o[i] = host[i];
        src = staged.data();
    }
    if (n == 0) return;
    if (t.is_cuda()) {
        cudaStream_t s = cuda::getCurrentStream();
        cuda_check(cudaMemcpyAsync(t.raw(), src, t.nbytes(), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync H2D");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");  // the staging buffer dies here
    } else {
        std::memcpy(t.raw(), src, t.nbytes());
    }
}
}  // namespace

Tensor Tensor::full(const Shape& s, const TensorOptions& o, float value) {
    Tensor t(s, o);
    t.fill(value);
    return t;
}
Tensor Tensor::zeros(const Shape& s, const TensorOptions& o) {
    Tensor t(s, o);
    t.zero_();
    return t;
}
Tensor Tensor::ones(const Shape& s, const TensorOptions& o) { return full(s, o, 1.0f); }
Tensor Tensor::randn(const Shape& s, const TensorOptions& o) {
    Tensor t(s, o);
    std::vector<float> h(static_cast<size_t>(t.numel()));
    {
        std::lock_guard<std::mutex> lk(rng_mu());
        std::normal_distribution<float> d(0.0f, 1.0f);
        for (auto& v : h) v = d(rng());
    }
    upload(t, h);
    return t;
}
Tensor Tensor::rand(const Shape& s, const TensorOptions& o) {
    Tensor t(s, o);
    std::vector<float> h(static_cast<size_t>(t.numel()));
    {
        std::lock_guard<std::mutex> lk(rng_mu());
        std::uniform_real_distribution<float> d(0.0f, 1.0f);
        for (auto& v : h) v = d(rng());
    }
    upload(t, h);
    return t;
}
Tensor Tensor::from_host(const float* data, const Shape& s, const TensorOptions& o) {
    Tensor t(s, o);
    upload(t, std::vector<float>(data, data + t.numel()));
    return t;
}

void Tensor::zero_() {
    if (numel_ == 0) return;
    if (is_cuda())
        cuda_check(cudaMemsetAsync(raw(), 0, nbytes(), cuda::getCurrentStream()), "cudaMemsetAsync");
    else
        std::memset(raw(), 0, nbytes());
}
void Tensor::fill(float v) {
    if (v == 0.0f) { zero_(); return; }
    upload(*this, std::vector<float>(static_cast<size_t>(numel_), v));
}

void Tensor::copy_(const Tensor& src) {
    if (src.numel() != numel_ || src.dtype() != dtype()) throw std::invalid_argument("copy_: size or dtype mismatch");
    if (numel_ == 0) return;
    cudaStream_t s = cuda::getCurrentStream();
    if (is_cuda() && src.is_cuda()) {
        cuda_check(cudaMemcpyAsync(raw(), src.raw(), nbytes(), cudaMemcpyDeviceToDevice, s), "cudaMemcpyAsync D2D");
    } else if (is_cuda()) {
        cuda_check(cudaMemcpyAsync(raw(), src.raw(), nbytes(), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync H2D");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    } else if (src.is_cuda()) {
        cuda_check(cudaMemcpyAsync(raw(), src.raw(), nbytes(), cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync D2H");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    } else {
        std::memcpy(raw(), src.raw(), nbytes());
    }
}
Tensor Tensor::to(DeviceIndex dev) const {
    if (dev == device()) return *this;
    Tensor t(shape_, opts_.with_device(dev));
    t.copy_(*this);
    return t;
}
Tensor Tensor::to_cpu() const { return to(DeviceIndex(Device::CPU)); }
Tensor Tensor::clone() const {
    Tensor t(shape_, opts_);
    t.copy_(*this);
    return t;
}
Tensor Tensor::reshape(const Shape& s) const {
    if (s.numel() != numel_) throw std::invalid_argument("reshape: element count differs");
    Tensor t = *this;
    t.shape_ = s;
    return t;
}
std::vector<float> Tensor::to_vector() const {
    Tensor h = to_cpu();
    std::vector<float> out(static_cast<size_t>(numel_));
    for (int64_t i = 0; i < numel_; ++i) {
        if (dtype() == Dtype::Float32) out[i] = h.data<float>()[i];
        else if (dtype() == Dtype::Bfloat16) out[i] = bf16_to_f32(h.data<uint16_t>()[i]);
        else out[i] = static_cast<float>(h.data<double>()[i]);
    }
    return out;
}
void Tensor::display(std::ostream& os, int precision) const {
    auto v = to_vector();
    os << "Tensor[";
    for (size_t i = 0; i < shape_.dims.size(); ++i) os << (i ? "," : "") << shape_.dims[i];
    os << "] {";
    const int64_t cols = shape_.dims.empty() ? 1 : shape_.dims.back();
    for (int64_t i = 0; i < numel_ && i < 64; ++i) {
        if (i % cols == 0) os << "\n  ";
        os << std::setprecision(precision) << v[i] << " ";
    }
    if (numel_ > 64) os << "\n  ...";
    os << "\n}\n";
}

}  // namespace OwnTensor
