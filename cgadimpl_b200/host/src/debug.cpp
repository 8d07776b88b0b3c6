// debug.cpp -- trace lines for node creation, backprop and jvp steps.
#include "ad/utils/debug.hpp"

#include <iostream>
#include <sstream>

namespace ag::debug {
namespace {
bool g_trace = false, g_grad_trace = false, g_jvp_trace = false;
std::string shape_str(const Tensor& t) {
    std::ostringstream os;
    os << "[";
    const auto& d = t.shape().dims;
    for (size_t i = 0; i < d.size(); ++i) os << (i ? "," : "") << d[i];
    os << "]";
    return os.str();
}
}  // namespace

void enable_tracing(bool on) { g_trace = on; }
void enable_grad_tracing(bool on) { g_grad_trace = on; }
void enable_jvp_tracing(bool on) { g_jvp_trace = on; }

void on_node_created(const std::shared_ptr<Node>& n) {
    if (!g_trace) return;
    std::cout << "[" << op_name(n->op) << "]" << (n->requires_grad() ? " (grad)" : "       ") << " value "
              << shape_str(n->value) << " @" << n.get();
    if (n->debug_name && n->debug_name[0]) std::cout << " name=\"" << n->debug_name << "\"";
    std::cout << std::endl;
}
void on_backprop_step(Node* n, const Tensor& gy) {
    if (!g_grad_trace) return;
    std::cout << "[vjp " << op_name(n->op) << "] gy " << shape_str(gy) << " @" << n << std::endl;
}
void on_jvp_step(Node* n) {
    if (!g_jvp_trace) return;
    std::cout << "[jvp " << op_name(n->op) << "] @" << n << std::endl;
}
void print_tensor(const std::string& label, const Tensor& t) {
    std::cout << label << " ";
    t.display(std::cout, 4);
}
}  // namespace ag::debug
