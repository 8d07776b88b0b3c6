// cuda_graphs.hpp -- thread-local current stream and the CUDA-graph runner, with the interface of
// cgadimpl/include/ad/runtime/cuda_graphs.hpp:7-61.  Differences: errors throw std::runtime_error
// instead of calling exit() (cgadimpl/src/runtime/cuda_graphs.cpp:12-19), begin_capture() reports
// failure by throwing instead of printing, and replay(n) can launch the graph n times.
#pragma once
#include <cuda_runtime.h>

extern "C" {
typedef struct CUstream_st* ag_cuda_stream_t;
}

namespace ag {

inline ag_cuda_stream_t& _get_stream() {
    static thread_local ag_cuda_stream_t s = nullptr;
    return s;
}
inline ag_cuda_stream_t current_stream() { return _get_stream(); }
inline void set_current_stream(ag_cuda_stream_t s) { _get_stream() = s; }

class CudaGraphRunner {
public:
    CudaGraphRunner();
    ~CudaGraphRunner();
    CudaGraphRunner(const CudaGraphRunner&) = delete;
    CudaGraphRunner& operator=(const CudaGraphRunner&) = delete;

    // Makes the runner's private non-blocking stream the current stream of this thread (for the
    // graph API and for the tensor library) and starts capturing it in thread-local mode.
    void begin_capture();
    // Ends the capture, instantiates the graph and resets both current-stream slots to null.
    void end_capture();
    // Launches the instantiated graph on the private stream; does not synchronise.
    bool replay();
    void synchronize();
    size_t num_nodes() const;  // kernel / memset nodes captured (0 before end_capture)
    bool is_capturing() const { return is_capturing_; }
    cudaStream_t get_stream() const { return stream_; }

private:
    cudaStream_t stream_ = nullptr;
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t instance_ = nullptr;
    bool is_capturing_ = false;
};

}  // namespace ag
