// debug.hpp -- the tracing hooks the op builders call (cgadimpl/include/ad/utils/debug.hpp:12-52,
// cgadimpl/src/tools/debug.cpp:17-24, 96-109).  Only the node-creation / backprop / jvp trace lines
// exist here; graph dumps and DOT export are not part of this path.
#pragma once
#include <memory>
#include <string>

#include "ad/core/graph.hpp"

namespace ag::debug {
void enable_tracing(bool on = true);
void enable_grad_tracing(bool on = true);
void enable_jvp_tracing(bool on = true);
void on_node_created(const std::shared_ptr<Node>& n);
void on_backprop_step(Node* n, const Tensor& gy);
void on_jvp_step(Node* n);
void print_tensor(const std::string& label, const Tensor& t);
}  // namespace ag::debug
