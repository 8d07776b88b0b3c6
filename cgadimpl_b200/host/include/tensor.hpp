// tensor.hpp -- same role as cgadimpl/include/tensor.hpp:6-15: pulls the tensor library into scope
// and adds ag::options().
#pragma once
#include "TensorLib.h"

using namespace OwnTensor;

namespace ag {
inline TensorOptions options(const Tensor& t) {
    return TensorOptions().with_dtype(t.dtype()).with_device(t.device()).with_req_grad(t.requires_grad());
}
}  // namespace ag
