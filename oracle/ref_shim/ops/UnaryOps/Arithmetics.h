// Stand-in for a header of the absent OwnTensor library: everything lives in TensorLib.h.
#pragma once
#include "TensorLib.h"
