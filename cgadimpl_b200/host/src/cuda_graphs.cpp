// cuda_graphs.cpp -- CudaGraphRunner (cgadimpl/src/runtime/cuda_graphs.cpp:23-76), throwing
// instead of exiting.
#include "ad/runtime/cuda_graphs.hpp"

#include <stdexcept>
#include <string>

#include "TensorLib.h"

namespace ag {
namespace {
void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess)
        throw std::runtime_error(std::string("CudaGraphRunner: ") + what + ": " + cudaGetErrorString(e));
}
}  // namespace

CudaGraphRunner::CudaGraphRunner() { check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "stream create"); }

CudaGraphRunner::~CudaGraphRunner() {
    if (is_capturing_) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(stream_, &g);
        if (g) cudaGraphDestroy(g);
        set_current_stream(nullptr);
        OwnTensor::cuda::setCurrentStream(nullptr);
    }
    if (instance_) cudaGraphExecDestroy(instance_);
    if (graph_) cudaGraphDestroy(graph_);
    if (stream_) cudaStreamDestroy(stream_);
}

void CudaGraphRunner::begin_capture() {
    if (is_capturing_) return;
    if (instance_) { cudaGraphExecDestroy(instance_); instance_ = nullptr; }
    if (graph_) { cudaGraphDestroy(graph_); graph_ = nullptr; }
    set_current_stream(reinterpret_cast<ag_cuda_stream_t>(stream_));
    OwnTensor::cuda::setCurrentStream(stream_);
    cudaError_t e = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        set_current_stream(nullptr);
        OwnTensor::cuda::setCurrentStream(nullptr);
        check(e, "begin capture");
    }
    is_capturing_ = true;
}

void CudaGraphRunner::end_capture() {
    if (!is_capturing_) return;
    cudaError_t e = cudaStreamEndCapture(stream_, &graph_);
    is_capturing_ = false;
    set_current_stream(nullptr);
    OwnTensor::cuda::setCurrentStream(nullptr);
    check(e, "end capture");
    check(cudaGraphInstantiate(&instance_, graph_, 0), "instantiate");
}

bool CudaGraphRunner::replay() {
    if (!instance_) return false;
    check(cudaGraphLaunch(instance_, stream_), "launch");
    return true;
}

void CudaGraphRunner::synchronize() { check(cudaStreamSynchronize(stream_), "synchronize"); }

size_t CudaGraphRunner::num_nodes() const {
    if (!graph_) return 0;
    size_t n = 0;
    if (cudaGraphGetNodes(graph_, nullptr, &n) != cudaSuccess) return 0;
    return n;
}

}  // namespace ag
