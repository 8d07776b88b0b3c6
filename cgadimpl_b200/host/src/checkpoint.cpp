// checkpoint.cpp -- marking, recompute and deletion of activations
// (cgadimpl/src/autodiff/checkpoint.cpp:112-226, :321-376; cgadimpl/src/autodiff/careful_deletion.cpp:66-160).
#include "ad/autodiff/checkpoint.hpp"

#include <deque>
#include <iostream>
#include <mutex>
#include <unordered_set>

#include "ad/autodiff/careful_deletion.hpp"

namespace ag {
namespace {

std::mutex g_mu;  // the parallel backward may ask for recomputes from several threads
CheckpointStats g_stats;
memory::DeletionStats g_del;

size_t node_bytes(const Node* n) {
    size_t b = n->value.nbytes();
    for (auto& t : n->tape)
        if (t && t->raw() != n->value.raw()) b += t->nbytes();
    return b;
}

bool has_value(const Node* n) { return n->value.numel() != 0 && n->value.defined(); }

bool recompute_locked(const std::shared_ptr<Node>& node, int depth) {
    if (!node || !node->is_checkpoint) {
        g_stats.failed_recomputes++;
        return false;
    }
    if (has_value(node.get())) return true;
    g_stats.recompute_calls++;
    if (depth <= 0) {
        g_stats.failed_recomputes++;
        return false;
    }
    for (const auto& saved : node->saved_inputs) {
        const auto& parent = saved.node;
        if (!parent || has_value(parent.get())) continue;
        if (!parent->is_checkpoint || !recompute_locked(parent, depth - 1)) {
            g_stats.failed_recomputes++;
            return false;
        }
    }
    try {
        node->inputs.resize(node->saved_inputs.size());
        for (size_t i = 0; i < node->saved_inputs.size(); ++i) {
            node->inputs[i] = node->saved_inputs[i].node;
            if (!node->inputs[i]) throw std::runtime_error("restored input is null");
        }
        node->value = forward_eval_node(node.get());
        g_stats.successful_recomputes++;
        return true;
    } catch (const std::exception& e) {
        std::cerr << "[checkpoint] recompute of '" << node->debug_name << "' failed: " << e.what() << "\n";
        g_stats.failed_recomputes++;
        return false;
    }
}

}  // namespace

namespace checkpoint_impl {

void mark_node_checkpoint(const std::shared_ptr<Node>& node, const CheckpointOptions& opts) {
    if (!node || node->is_checkpoint) return;
    if (node->op == Op::Leaf && !opts.force) return;  // a leaf has nothing to be recomputed from
    std::lock_guard<std::mutex> lk(g_mu);
    node->is_checkpoint = true;
    node->saved_inputs.clear();
    for (auto& p : node->inputs) node->saved_inputs.emplace_back(p ? Value(p) : Value());
    g_stats.total_checkpoints++;
    g_stats.total_memory_saved += node_bytes(node.get());
    if (opts.verbose)
        std::cout << "[checkpoint] marked '" << node->debug_name << "' (" << node_bytes(node.get()) / 1024.0 << " KB)\n";
}

bool recompute_subgraph(const std::shared_ptr<Node>& node) {
    std::lock_guard<std::mutex> lk(g_mu);
    return recompute_locked(node, CheckpointOptions().max_recompute_depth);
}

bool ensure_value_present(const std::shared_ptr<Node>& node) {
    if (!node) return true;
    // only checkpoints ever lose and regain their value, so only they need the lock to be looked at
    if (!node->is_checkpoint) return has_value(node.get());
    return recompute_subgraph(node);
}

}  // namespace checkpoint_impl

Value checkpoint(const Value& v, const CheckpointOptions& opts) {
    checkpoint_impl::mark_node_checkpoint(v.node, opts);
    return v;
}

void auto_checkpoint_every_n(const Value& root, int n) {
    if (n <= 0 || !root.node) return;
    std::unordered_set<Node*> seen;
    std::deque<std::shared_ptr<Node>> q{root.node};
    int counter = 0;
    while (!q.empty()) {
        auto cur = q.front();
        q.pop_front();
        if (!cur || !seen.insert(cur.get()).second) continue;
        if (++counter % n == 0 && !cur->inputs.empty()) checkpoint_impl::mark_node_checkpoint(cur);
        for (auto& p : cur->inputs) q.push_back(p);
    }
}

void auto_checkpoint_by_depth(const Value& root, int depth_threshold) {
    if (!root.node) return;
    std::unordered_set<Node*> seen;
    std::deque<std::pair<std::shared_ptr<Node>, int>> q{{root.node, 0}};
    while (!q.empty()) {
        auto [cur, depth] = q.front();
        q.pop_front();
        if (!cur || !seen.insert(cur.get()).second) continue;
        if (depth >= depth_threshold && !cur->inputs.empty()) checkpoint_impl::mark_node_checkpoint(cur);
        for (auto& p : cur->inputs) q.emplace_back(p, depth + 1);
    }
}

CheckpointStats checkpoint_stats() {
    std::lock_guard<std::mutex> lk(g_mu);
    return g_stats;
}
void reset_checkpoint_stats() {
    std::lock_guard<std::mutex> lk(g_mu);
    g_stats = CheckpointStats();
}
void print_checkpoint_stats() {
    const CheckpointStats s = checkpoint_stats();
    std::cout << "=== Checkpoint Statistics ===\n"
              << "Total checkpoints: " << s.total_checkpoints << "\n"
              << "Successful recomputes: " << s.successful_recomputes << "\n"
              << "Failed recomputes: " << s.failed_recomputes << "\n"
              << "Estimated memory saved: " << s.total_memory_saved / 1024.0 / 1024.0 << " MB\n"
              << "Recompute calls: " << s.recompute_calls << "\n"
              << "=============================\n";
}

namespace memory {

namespace {
bool gradients_done(const Node* n) {
    for (auto& p : n->inputs)
        if (p && p->requires_grad()) return false;
    return true;
}
}  // namespace

bool try_delete_node(Node* node, DeletePolicy policy, const std::unordered_set<Node*>* protected_nodes) {
    if (!node) return false;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!has_value(node)) return false;  // nothing to drop (already gone)
    const bool keep = (protected_nodes && protected_nodes->count(node)) || node->op == Op::Leaf ||
                      (node->is_checkpoint && policy == DeletePolicy::AlwaysSafe) ||
                      // after the forward pass only what can be recomputed may go
                      (policy == DeletePolicy::ForwardPass && !node->is_checkpoint) ||
                      (policy != DeletePolicy::ForwardPass && !gradients_done(node));
    if (keep) {
        g_del.nodes_skipped++;
        return false;
    }
    g_del.memory_freed += node_bytes(node) + (policy != DeletePolicy::ForwardPass ? node->grad.nbytes() : 0);
    if (node->is_checkpoint && node->saved_inputs.empty())
        for (auto& p : node->inputs) node->saved_inputs.emplace_back(p ? Value(p) : Value());
    node->value_released = true;
    node->released_shape = node->value.shape();
    node->released_options = ag::options(node->value);
    node->value = Tensor();
    node->tape.clear();
    if (policy != DeletePolicy::ForwardPass) {
        node->grad = Tensor();
        node->grad_live = false;
    }
    g_del.nodes_deleted++;
    return true;
}

int sweep_safe_nodes(const Value& root, DeletePolicy policy, const std::unordered_set<Node*>& protected_nodes) {
    if (!root.node) return 0;
    int freed = 0;
    for (Node* n : topo_from(root.node.get()))
        if (n != root.node.get() && try_delete_node(n, policy, &protected_nodes)) ++freed;
    return freed;
}

DeletionStats deletion_stats() {
    std::lock_guard<std::mutex> lk(g_mu);
    return g_del;
}
void reset_deletion_stats() {
    std::lock_guard<std::mutex> lk(g_mu);
    g_del = DeletionStats();
}

}  // namespace memory
}  // namespace ag
