// ag_all.hpp -- umbrella header (cgadimpl/include/ad/ag_all.hpp:4-10).
#pragma once
#include <cuda_runtime.h>

#include "ad/autodiff/autodiff.hpp"
#include "ad/autodiff/careful_deletion.hpp"
#include "ad/autodiff/checkpoint.hpp"
#include "ad/detail/autodiff_ops.hpp"
#include "ad/runtime/cuda_graphs.hpp"
#include "ad/utils/debug.hpp"
#include "nn/nn.hpp"
#include "optim.hpp"
