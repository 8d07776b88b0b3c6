// autodiff.cpp -- zero_grad / backward / jvp with the semantics of cgadimpl/src/core/autodiff.cpp:
// reverse-topological VJP dispatch with post-accumulate hooks (:75-96), an opt-in multi-threaded
// mode driven by per-node dependency counters (:98-170), and a forward tangent sweep (:221-252).
#include "ad/autodiff/autodiff.hpp"

#include <atomic>
#include <condition_variable>
#include <deque>
#include <exception>
#include <thread>

#include "ad/autodiff/careful_deletion.hpp"
#include "ad/autodiff/checkpoint.hpp"
#include "ad/detail/autodiff_ops.hpp"
#include "ad/detail/host_util.hpp"

namespace ag {

void zero_grad(const Value& root) {
    for (Node* n : topo_from(root.node.get()))
        if (n->requires_grad()) {
            // Lazy: the buffer (if any) is kept, marked empty, and overwritten by the next pass's first
            // contribution; a reader sees zeros through Value::grad().  No memset here.
            std::lock_guard<std::mutex> lock(n->grad_mutex);
            n->grad_live = false;
        }
}

namespace {

// Blocking queue of ready nodes (same job as cgadimpl/include/ad/core/ReadyQueue.hpp:12-51).
class ReadyQueue {
public:
    void push(Node* n) {
        { std::lock_guard<std::mutex> lk(mu_); q_.push_back(n); }
        cv_.notify_one();
    }
    Node* pop() {  // nullptr after shutdown
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || !q_.empty(); });
        if (q_.empty()) return nullptr;
        Node* n = q_.front();
        q_.pop_front();
        return n;
    }
    void shutdown() {
        { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
        cv_.notify_all();
    }
private:
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<Node*> q_;
    bool stop_ = false;
};

void run_hooks(Node* n) {
    for (auto& h : n->post_acc_grad_hooks) h(n);
}

// Which activations a rule reads.  Add / Sum / MeanAll / RowSum only move gy along; Mul, the norm
// rules and logsumexp read their inputs' values; the norm rules also read their own tape (rstd,
// mean, var) and softmax its own value.
bool rule_reads_inputs(Op op) {
    return op == Op::Mul || op == Op::RMSNorm || op == Op::RMSNormAffine || op == Op::RealRMSNorm || op == Op::LayerNorm ||
           op == Op::LogSumExpRow;
}
bool rule_reads_own_tape(Op op) {
    return op == Op::RMSNorm || op == Op::RMSNormAffine || op == Op::RealRMSNorm || op == Op::LayerNorm ||
           op == Op::SoftmaxRow;
}

// Runs n's rule with every activation it reads present: dropped ones are recomputed first
// (cgadimpl/src/core/autodiff.cpp:82-86 restores only the node's own value), and a node that had to
// be recomputed is dropped again afterwards -- all its children have run by then, so nothing reads
// it any more.
void run_rule(Node* n) {
    VjpFn fn = vjp_lookup(n->op);
    if (!fn) return;
    if (n->is_checkpoint && rule_reads_own_tape(n->op) && !checkpoint_impl::ensure_value_present(n->shared_from_this()))
        throw std::runtime_error("autodiff: failed to recompute checkpointed node during backward");
    if (rule_reads_inputs(n->op))
        for (auto& p : n->inputs)
            if (!checkpoint_impl::ensure_value_present(p))
                throw std::runtime_error("autodiff: an input activation is gone and cannot be recomputed");
    fn(n, n->materialized_grad());
    // `value_released` means careful deletion dropped this activation once: whoever brought it back
    // (this rule or a child's) no longer needs it
    if (n->is_checkpoint && n->value_released) memory::try_delete_node(n, memory::DeletePolicy::ForwardPass);
}

}  // namespace

// One stream per graph.  Every rule launches on its node's creation stream, writes its parents' gradients
// there, and the parents' own rules read them on THEIR creation streams; the per-node mutex orders only the
// host-side enqueue, and the caching allocator hands a freed block back to the pool of the stream it was
// allocated on.  So an interior node whose stream differs from its consumer's would race on the GPU.  The
// reference runs everything on one thread-local stream; here that is a checked rule: interior nodes of a
// graph must share one creation stream (the current stream while the graph was built).  Leaves are exempt --
// they are long-lived tensors that the caller orders (e.g. parameters made before a capture stream exists).
void check_single_stream(const std::vector<Node*>& order) {
    for (Node* n : order)
        for (auto& p : n->inputs)
            if (p && !p->is_leaf && p->creation_context.stream != n->creation_context.stream)
                throw std::runtime_error(std::string("autodiff: node '") + op_name(n->op) + "' was built on another stream than its input '" +
                                         op_name(p->op) + "'; build a graph under ONE current stream (ag::set_current_stream) -- "
                                         "gradients and activations are not ordered across streams");
}

void backward(const Value& root, const Tensor* grad_seed, bool enable_parallel) {
    if (!root.node) return;
    auto order = topo_from(root.node.get());
    check_single_stream(order);

    for (Node* n : order) n->child_grad_count = 0;
    for (Node* n : order)
        for (auto& p : n->inputs)
            if (p && p->requires_grad()) p->child_grad_count++;

    if (root.node->requires_grad()) {
        std::lock_guard<std::mutex> lock(root.node->grad_mutex);
        if (grad_seed) {
            root.node->grad = *grad_seed;
        } else {
            detail::StreamGuard g(root.node->creation_context.stream);
            auto opts = ag::options(root.node->value);
            root.node->grad = root.node->value.numel() == 1 ? Tensor::ones(Shape{{1}}, opts)
                                                            : Tensor::ones(root.node->value.shape(), opts);
        }
        root.node->grad_live = true;
    }

    if (!enable_parallel) {
        for (auto it = order.rbegin(); it != order.rend(); ++it) {
            Node* n = *it;
            if (!n->requires_grad()) continue;
            debug::on_backprop_step(n, n->materialized_grad());
            run_rule(n);
            run_hooks(n);
        }
        return;
    }

    // Parallel mode.  A node becomes ready when every child that owes it a gradient has run.
    // Differences from the reference: the main thread blocks on a condition variable instead of
    // polling with 1 ms sleeps, and an exception in a rule is carried to the caller instead of
    // being dropped.
    int pending = 0;
    for (Node* n : order)
        if (n->requires_grad()) ++pending;
    if (pending == 0) return;

    ReadyQueue rq;
    std::mutex done_mu;
    std::condition_variable done_cv;
    std::atomic<int> remaining{pending};
    std::exception_ptr error;

    auto finish_one = [&] {
        if (remaining.fetch_sub(1) == 1) {
            std::lock_guard<std::mutex> lk(done_mu);
            done_cv.notify_all();
        }
    };
    auto fail = [&](std::exception_ptr e) {
        std::lock_guard<std::mutex> lk(done_mu);
        if (!error) error = e;
        remaining = 0;
        done_cv.notify_all();
    };

    for (Node* n : order)
        if (n->requires_grad() && n->child_grad_count == 0) {
            run_hooks(n);
            if (!n->is_leaf) rq.push(n);
            else finish_one();
        }

    auto worker = [&] {
        while (Node* n = rq.pop()) {
            try {
                run_rule(n);
                for (auto& pp : n->inputs) {
                    Node* p = pp.get();
                    if (!p || !p->requires_grad()) continue;
                    if (p->child_grad_count.fetch_sub(1) == 1) {
                        run_hooks(p);
                        if (!p->is_leaf) rq.push(p);
                        else finish_one();
                    }
                }
                finish_one();
            } catch (...) {
                fail(std::current_exception());
            }
        }
    };

    unsigned nthreads = std::thread::hardware_concurrency();
    if (nthreads == 0) nthreads = 1;
    if (nthreads > 16) nthreads = 16;
    std::vector<std::thread> workers;
    for (unsigned i = 0; i < nthreads; ++i) workers.emplace_back(worker);
    {
        std::unique_lock<std::mutex> lk(done_mu);
        done_cv.wait(lk, [&] { return remaining.load() <= 0; });
    }
    rq.shutdown();
    for (auto& w : workers) w.join();
    if (error) std::rethrow_exception(error);
}

Tensor jvp(const Value& root, const std::unordered_map<Node*, Tensor>& seed) {
    if (!root.node) return Tensor();
    auto order = topo_from(root.node.get());
    std::unordered_map<Node*, Tensor> T;
    T.reserve(order.size());
    static const Tensor kEmpty;
    auto tangent_of = [&](Node* p) -> const Tensor& {
        auto it = T.find(p);
        return it != T.end() ? it->second : kEmpty;
    };
    for (Node* n : order) {
        Tensor t;
        if (auto it = seed.find(n); it != seed.end()) {
            t = it->second;
        } else if (n->is_leaf) {
            detail::StreamGuard g(current_stream());
            t = Tensor::zeros(n->value.shape(), ag::options(n->value).with_req_grad(false));
        }
        debug::on_jvp_step(n);
        if (!n->is_leaf) {
            T[n] = t;  // visible to the rule as "no tangent yet"
            if (JvpFn fn = jvp_lookup(n->op)) t = fn(n, tangent_of);
        }
        T[n] = t;
    }
    return T[root.node.get()];
}

}  // namespace ag
