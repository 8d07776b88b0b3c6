// nodeops.hpp -- forward node builders on the RMSNorm path, signatures as in
// cgadimpl/include/ad/ops/nodeops.hpp:27-133 (shared_ptr<Node> in, shared_ptr<Node> out).
#pragma once
#include <memory>

#include "ad/core/graph.hpp"
#include "ad/utils/debug.hpp"

namespace ag {
namespace detail {

std::shared_ptr<Node> add_nodeops(const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b);
std::shared_ptr<Node> mul_nodeops(const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b);
inline std::shared_ptr<Node> operator+(const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b) { return add_nodeops(a, b); }
inline std::shared_ptr<Node> operator*(const std::shared_ptr<Node>& a, const std::shared_ptr<Node>& b) { return mul_nodeops(a, b); }

std::shared_ptr<Node> laynor_nodeops(const std::shared_ptr<Node>& x);
std::shared_ptr<Node> rms_nodeops(const std::shared_ptr<Node>& x);
std::shared_ptr<Node> realrms_nodeops(const std::shared_ptr<Node>& x, float& g);

std::shared_ptr<Node> sum_nodeops(const std::shared_ptr<Node>& x);
std::shared_ptr<Node> mean_all_nodeops(const std::shared_ptr<Node>& x);
std::shared_ptr<Node> rowsum_nodeops(const std::shared_ptr<Node>& x);
std::shared_ptr<Node> rowmax_nodeops(const std::shared_ptr<Node>& x);
std::shared_ptr<Node> softmax_row_nodeops(const std::shared_ptr<Node>& z);
std::shared_ptr<Node> logsumexp_row_nodeops(const std::shared_ptr<Node>& z);

// additions: the per-channel layer as one node, with and without the residual add
std::shared_ptr<Node> rmsnorm_nodeops(const std::shared_ptr<Node>& x, const std::shared_ptr<Node>& gamma, float eps);
std::shared_ptr<Node> add_rmsnorm_nodeops(const std::shared_ptr<Node>& x, const std::shared_ptr<Node>& r,
                                          const std::shared_ptr<Node>& gamma, float eps);

}  // namespace detail
}  // namespace ag
