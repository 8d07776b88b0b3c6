// ops.hpp -- Value-level API of the path (cgadimpl/include/ad/ops/ops.hpp:18-125).
#pragma once
#include "ad/core/graph.hpp"
#include "ad/ops/nodeops.hpp"

namespace ag {

Value add(const Value& a, const Value& b);
Value mul(const Value& a, const Value& b);

Value laynor(const Value& x);              // (x - mean) / sqrt(var + 1e-5), no affine parameters
Value rms(const Value& x);                 // x / sqrt(mean(x^2) + 1e-5), no gamma
Value realrms(const Value& x, float g);    // scalar gain

Value sum(const Value& x);
Value mean_all(const Value& x);
Value rowsum(const Value& x);              // [B,C] -> [B,1]
Value rowmax(const Value& x);              // [B,C] -> [B,1]
Value softmax_row(const Value& z);         // softmax over the last axis
Value logsumexp_row(const Value& z);       // [.., C] -> [.., 1]

// additions
Value rmsnorm(const Value& x, const Value& gamma, float eps = 1e-5f);                    // == mul(rms(x), gamma), fused
// == rmsnorm(add(x, r), gamma) with ONE forward kernel.  Builds the same two nodes the unfused
// expression would (an Add node h and an RMSNormAffine node y on top of it) and returns y;
// residual_of(y) is the Add node h = x + r, to feed the next layer's residual stream.
Value add_rmsnorm(const Value& x, const Value& r, const Value& gamma, float eps = 1e-5f);
Value residual_of(const Value& add_rmsnorm_out);

// Recompute of one node from its inputs (value returned, tape restored in place); used by
// checkpointing.  cgadimpl/include/ad/ops/ops.hpp:121-125.
Tensor forward_eval_node(const std::shared_ptr<Node>& node);
Tensor forward_eval_node(Node* node);

inline Value operator+(const Value& a, const Value& b) { return ag::add(a, b); }
inline Value operator*(const Value& a, const Value& b) { return ag::mul(a, b); }

}  // namespace ag
