// checkpoint.hpp -- activation checkpointing over the graph API, with the interface of
// cgadimpl/include/ad/autodiff/checkpoint.hpp:33-214: a node marked as a checkpoint remembers its
// inputs, so its value (and tape) can be dropped after the forward pass and recomputed when the
// backward pass needs it.  Unlike the reference, recompute covers the normalisation ops, the
// backward pass also restores the INPUT values a rule reads (not only the node's own value), and
// a value that was recomputed is dropped again as soon as its last reader has run.
#pragma once
#include <cstddef>
#include <memory>

#include "ad/core/graph.hpp"
#include "ad/ops/ops.hpp"

namespace ag {

struct CheckpointOptions {
    bool save_rng = true;            // no op of this path draws random numbers; kept for source compatibility
    int max_recompute_depth = 1000;  // bound on the recursion through recomputable parents
    bool save_inputs = true;
    bool detach_inputs = false;
    bool force = false;
    bool verbose = false;
};

// Marks v's node and returns v.
Value checkpoint(const Value& v, const CheckpointOptions& opts = CheckpointOptions());
// Breadth-first from the root: every n-th non-leaf node / every non-leaf node at least
// depth_threshold edges away from the root is marked.
void auto_checkpoint_every_n(const Value& root, int n);
void auto_checkpoint_by_depth(const Value& root, int depth_threshold);

struct CheckpointStats {
    size_t total_checkpoints = 0, recompute_calls = 0, successful_recomputes = 0, failed_recomputes = 0;
    size_t total_memory_saved = 0;  // bytes of value + tape of the marked nodes, counted when marked
};
CheckpointStats checkpoint_stats();
void print_checkpoint_stats();
void reset_checkpoint_stats();

namespace checkpoint_impl {
void mark_node_checkpoint(const std::shared_ptr<Node>& node, const CheckpointOptions& opts = CheckpointOptions());
// True when the node has a value afterwards.  Parents without a value are recomputed first when
// they are checkpoints themselves; a missing parent that is not fails the call.
bool recompute_subgraph(const std::shared_ptr<Node>& node);
bool ensure_value_present(const std::shared_ptr<Node>& node);
inline bool is_checkpointed(const std::shared_ptr<Node>& node) { return node && node->is_checkpoint; }
}  // namespace checkpoint_impl

}  // namespace ag
