// autodiff_ops.hpp -- rule tables (cgadimpl/include/ad/detail/autodiff_ops.hpp:18-40).
#pragma once
#include <functional>

#include "ad/core/graph.hpp"
#include "ad/core/schema.hpp"

namespace ag {
using VjpFn = void (*)(Node* n, const Tensor& gy);
using JvpFn = Tensor (*)(Node* n, const std::function<const Tensor&(Node*)>& tangent_of);
VjpFn vjp_lookup(Op op);
JvpFn jvp_lookup(Op op);
}  // namespace ag

#ifdef AG_EXPOSE_AUTODIFF_RULES
namespace ag::detail {
#define OP(name, arity, str)                    \
    void vjp_##name(Node* n, const Tensor& gy); \
    Tensor jvp_##name(Node* n, const std::function<const Tensor&(Node*)>& tangent_of);
#include "ad/detail/ops.def"
#undef OP
}  // namespace ag::detail
#endif
