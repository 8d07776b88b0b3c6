// alloc_cabi.cpp -- the C ABI of include/agb/agb_alloc.h over OwnTensor::cuda::DeviceAllocator.
#include <cstring>
#include <exception>
#include <string>

#include "TensorLib.h"
#include "agb/agb_alloc.h"

namespace {
thread_local std::string t_error;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        t_error = e.what();
    } catch (...) {
        t_error = "unknown error";
    }
    return 1;
}
OwnTensor::cuda::DeviceAllocator& alloc() { return OwnTensor::cuda::DeviceAllocator::instance(); }
}  // namespace

extern "C" {

int agb_malloc_async(void** ptr, size_t bytes, int device, agb_alloc_stream_t stream) {
    if (!ptr) {
        t_error = "ptr is NULL";
        return 1;
    }
    *ptr = nullptr;
    return guarded([&] { *ptr = alloc().allocate(bytes, device, reinterpret_cast<cudaStream_t>(stream)); });
}
int agb_free_async(void* ptr) {
    if (!ptr) return 0;
    if (!alloc().owns(ptr)) {
        t_error = "pointer was not handed out by agb_malloc_async (or was freed already)";
        return 1;
    }
    return guarded([&] { alloc().release(ptr); });
}
int agb_arena_reserve(size_t bytes, int device, agb_alloc_stream_t stream) {
    return guarded([&] { alloc().reserve(bytes, device, reinterpret_cast<cudaStream_t>(stream)); });
}
int agb_alloc_empty_cache(void) {
    return guarded([&] { alloc().empty_cache(); });
}
int agb_alloc_set_limit(size_t bytes) {
    return guarded([&] { alloc().set_memory_limit(bytes); });
}
int agb_alloc_stats(size_t out[5]) {
    if (!out) {
        t_error = "out is NULL";
        return 1;
    }
    return guarded([&] {
        const auto s = alloc().stats();
        out[0] = s.bytes_in_use; out[1] = s.bytes_cached; out[2] = s.device_allocs; out[3] = s.cache_hits; out[4] = s.peak_in_use;
    });
}
const char* agb_alloc_last_error(void) { return t_error.c_str(); }

}  // extern "C"
