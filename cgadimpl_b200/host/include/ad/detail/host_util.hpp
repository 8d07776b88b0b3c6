// host_util.hpp -- internal helpers shared by the op builders and the autodiff rules: shape
// classification, status -> exception, per-stream workspaces and stream guards.
#pragma once
#include <stdexcept>
#include <string>

#include "ad/core/graph.hpp"
#include "agb/agb.h"

namespace ag::detail {

inline void check_status(int st, const char* where) {
    if (st != AGB_OK) throw std::runtime_error(std::string(where) + ": " + agb_last_error());
}

inline int agb_dtype(const Tensor& t) {
    switch (t.dtype()) {
        case Dtype::Float32: return AGB_F32;
        case Dtype::Bfloat16: return AGB_BF16;
        default: throw std::runtime_error("agb: only Float32 and Bfloat16 tensors are supported on this path");
    }
}

inline void require_cuda(const Tensor& t, const char* what) {
    if (!t.is_cuda())
        throw std::runtime_error(std::string(what) + ": tensor is on the CPU; this path has no CPU implementation");
}

struct RowsHidden {
    int64_t rows, hidden;
};
inline RowsHidden rows_hidden(const Tensor& t) {
    const auto& d = t.shape().dims;
    const int64_t h = d.empty() ? 1 : d.back();
    return {h ? t.numel() / h : 0, h};
}

// How `b` broadcasts against `full` ([..., hidden]); throws for shapes outside the path.
int classify_broadcast(const Tensor& full, const Tensor& b);

// Sets the tensor library's current stream (allocation pool) for the lifetime of the guard.
struct StreamGuard {
    cudaStream_t prev;
    explicit StreamGuard(ag_cuda_stream_t s) : prev(OwnTensor::cuda::getCurrentStream()) {
        OwnTensor::cuda::setCurrentStream(reinterpret_cast<cudaStream_t>(s));
    }
    ~StreamGuard() { OwnTensor::cuda::setCurrentStream(prev); }
};

// A device workspace of at least `bytes`, private to (this thread, this stream), kept alive for
// the life of the thread so that captured graphs can keep pointing at it.
void* workspace(size_t bytes, const Tensor& like, ag_cuda_stream_t stream);

// out = a (+|*) b with the broadcasts classify_broadcast knows; op 0 = add, 1 = mul.
Tensor binary_op(int op, const Tensor& a, const Tensor& b, ag_cuda_stream_t stream);

// A [1] scalar operand that lives on the CPU (Value(float) literals) is moved next to `like`.
Tensor on_device_of(const Tensor& t, const Tensor& like);

}  // namespace ag::detail
