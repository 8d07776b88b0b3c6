// graph.hpp -- Value / Node / topo_from with the members and signatures of
// cgadimpl/include/ad/core/graph.hpp:18-86.  The checkpointing members are used by
// ad/autodiff/checkpoint.hpp; the RNG and version-tracking members are kept as plain fields so code
// that touches them still compiles.
#pragma once
#include <atomic>
#include <functional>
#include <memory>
#include <mutex>
#include <utility>
#include <vector>

#include "ad/core/schema.hpp"
#include "ad/runtime/cuda_graphs.hpp"
#include "tensor.hpp"

namespace ag {
struct Node;
using HookFn = std::function<void(Node*)>;

struct Value {
    std::shared_ptr<Node> node;
    Value();
    explicit Value(std::shared_ptr<Node> n);
    Value(float v);  // scalar literal: a [1] fp32 CPU leaf that does not require grad
    const std::vector<int64_t>& shape() const;
    std::pair<int, int> shape_2d() const;
    Tensor& val();
    const Tensor& val() const;
    Tensor& grad();
    const Tensor& grad() const;
    void register_hook(HookFn hook);
};

struct Node : std::enable_shared_from_this<Node> {
    Tensor value;
    Tensor grad;

    std::vector<std::shared_ptr<Node>> inputs;
    std::vector<Value> saved_inputs;
    std::vector<std::shared_ptr<Tensor>> tape;

    std::vector<uint8_t> saved_rng_blob;
    bool is_checkpoint{false};
    bool has_saved_rng{false};

    const char* debug_name{""};
    Op op{Op::Leaf};
    bool is_leaf{false};
    std::vector<int> input_versions;

    std::atomic<int> child_grad_count{0};
    std::mutex grad_mutex;

    std::vector<HookFn> post_acc_grad_hooks;
    void register_hook(HookFn hook) { post_acc_grad_hooks.push_back(std::move(hook)); }

    struct ExecutionContext {
        ag_cuda_stream_t stream{nullptr};
        DeviceIndex device;
    };
    ExecutionContext creation_context;

    float eps{1e-5f};  // normalisation nodes only (the reference hard-codes 1e-5)

    bool requires_grad_flag_{false};
    bool requires_grad() const { return requires_grad_flag_; }
    // What the value looked like before careful deletion dropped it (zero_grad and the rules that
    // only need a shape keep working on a node whose activation is gone).
    bool value_released{false};
    Shape released_shape;
    TensorOptions released_options;
    const std::vector<int64_t>& shape() const { return value_released && value.numel() == 0 ? released_shape.dims : value.shape().dims; }

    // grad += contribution under grad_mutex; the contribution may be broadcast ([rows,1], [hidden]
    // or [1] against [rows, hidden]), as `grad += gy` is in the reference's row-reduction rules.
    void accumulate_grad(const Tensor& grad_contribution);

    // Lazy gradients.  The reference allocates and zero-fills a full-size gradient for every node that
    // needs one when the node is built (graph.cpp:36) and every rule then reads it back to add to it:
    // one write and one read of [rows, hidden] per node that the arithmetic does not need.  Here `grad`
    // stays unallocated until the first contribution of a backward pass, which WRITES it (no zero fill,
    // no read-back); later contributions add.  zero_grad() only clears `grad_live`.  A reader that goes
    // through Value::grad() / materialized_grad() sees what the reference shows: zeros until something
    // has been accumulated.  Code that touches the `grad` member directly sees an empty tensor (or the
    // previous pass's values after zero_grad) until then.
    bool grad_live{false};          // guarded by grad_mutex: `grad` holds the sum of this pass's contributions
    // With grad_mutex held: makes sure `grad` has the value's shape and returns it; *first says whether the
    // caller must overwrite it (no contribution yet) or add to it.  Marks the gradient live.
    Tensor& open_grad(bool* first);
    // What a reader sees: the accumulated gradient, zeros (allocated on demand) when there is none yet.
    Tensor& materialized_grad();

    Node(const Tensor& v, Op op_, bool req_grad, const char* nm = "");
    Node() = default;
};

inline Value make_tensor(const Tensor& v, const char* name = "") {
    return Value(std::make_shared<Node>(v, Op::Leaf, v.requires_grad(), name));
}

std::vector<Node*> topo_from(Node* root);  // parents before children

inline void Value::register_hook(HookFn hook) {
    if (node) node->register_hook(std::move(hook));
}

}  // namespace ag
