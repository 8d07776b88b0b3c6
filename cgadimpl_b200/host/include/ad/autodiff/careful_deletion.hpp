// careful_deletion.hpp -- dropping activations that are no longer (or not yet) needed, with the
// interface of cgadimpl/include/ad/autodiff/careful_deletion.hpp:100-166 minus the in-place
// snapshot machinery, which is not on this path.  Dropping a node's value also drops its tape
// (rstd / yhat of the norm ops): forward_eval_node restores both.
#pragma once
#include <cstddef>
#include <unordered_set>

#include "ad/core/graph.hpp"

namespace ag::memory {

enum class DeletePolicy {
    AlwaysSafe,   // only nodes none of whose inputs still awaits a gradient; checkpoints are kept
    ForwardPass,  // after the forward pass: value and tape go, grad stays; checkpoints may go (they can be recomputed)
    Aggressive,   // like AlwaysSafe but checkpoints may go as well
};

struct DeletionStats {
    size_t nodes_deleted = 0, nodes_skipped = 0, memory_freed = 0;
};

bool try_delete_node(Node* node, DeletePolicy policy = DeletePolicy::AlwaysSafe,
                     const std::unordered_set<Node*>* protected_nodes = nullptr);
// Every node below the root except the root itself and the protected ones; returns how many went.
int sweep_safe_nodes(const Value& root, DeletePolicy policy = DeletePolicy::AlwaysSafe,
                     const std::unordered_set<Node*>& protected_nodes = {});
DeletionStats deletion_stats();
void reset_deletion_stats();

}  // namespace ag::memory
