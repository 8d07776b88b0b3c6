// test_host_cpu.cpp -- the parts of the host layer that need no GPU: op registry (names, arities
// and enum values as in the reference's registry), topological order, CPU tensors, broadcast
// classification, the allocator's budget knob (host-side out-of-memory injection) and the error
// behaviour of ops given CPU tensors (there is no CPU implementation of the path).
#include "ad/ag_all.hpp"
#include "ad/detail/host_util.hpp"
#include <unordered_set>

#include "check.hpp"

using namespace ag;

int main() {
    run_test("registry: names, arities, numbering", [] {
        CHECK(static_cast<int>(Op::Leaf) == 0);
        CHECK(static_cast<int>(Op::Add) == 1 && static_cast<int>(Op::Mul) == 3);
        CHECK(static_cast<int>(Op::Sum) == 34 && static_cast<int>(Op::RowMax) == 37);
        CHECK(static_cast<int>(Op::LayerNorm) == 44 && static_cast<int>(Op::RMSNorm) == 45);
        CHECK(static_cast<int>(Op::RealRMSNorm) == 46 && static_cast<int>(Op::MAELoss) == 53);
        CHECK(static_cast<int>(Op::RMSNormAffine) == 54 && OpCount == 55);
        CHECK(std::string(op_name(Op::RMSNorm)) == "rmsnorm" && op_arity(Op::RMSNorm) == 1);
        CHECK(std::string(op_name(Op::RealRMSNorm)) == "realrmsnorm");
        CHECK(std::string(op_name(Op::Add)) == "add" && op_arity(Op::Add) == 2);
        CHECK(std::string(op_name(Op::RowSum)) == "rowsum" && op_arity(Op::Linear) == 3);
        CHECK(op_arity(Op::Leaf) == 0 && op_arity(Op::Dyntanh) == 4);
        CHECK(std::string(op_name(Op::RMSNormAffine)) == "rmsnorm_affine" && op_arity(Op::RMSNormAffine) == 2);
        for (std::size_t i = 0; i < OpCount; ++i) {
            CHECK(vjp_lookup(static_cast<Op>(i)) != nullptr);
            CHECK(jvp_lookup(static_cast<Op>(i)) != nullptr);
        }
    });

    run_test("rules outside the path throw, RowMax like the reference", [] {
        Node n;
        Tensor t;
        bool threw = false;
        try { vjp_lookup(Op::MatMul)(&n, t); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
        threw = false;
        try { vjp_lookup(Op::RowMax)(&n, t); } catch (const std::runtime_error& e) {
            threw = std::string(e.what()).find("RowMax") != std::string::npos;
        }
        CHECK(threw);
    });

    run_test("CPU tensors: factories, copies, reshape", [] {
        OwnTensor::manual_seed(7);
        Tensor a = Tensor::randn(Shape{{3, 5}}, TensorOptions());
        OwnTensor::manual_seed(7);
        Tensor b = Tensor::randn(Shape{{3, 5}}, TensorOptions());
        CHECK(a.to_vector() == b.to_vector());
        CHECK(a.numel() == 15 && a.shape().dims.size() == 2 && !a.is_cuda());
        Tensor z = Tensor::zeros(Shape{{4}}), o = Tensor::ones(Shape{{4}}), f = Tensor::full(Shape{{2, 2}}, TensorOptions(), 2.5f);
        CHECK(z.to_vector() == std::vector<float>(4, 0.f) && o.to_vector() == std::vector<float>(4, 1.f));
        CHECK(f.to_vector() == std::vector<float>(4, 2.5f));
        Tensor c = a.clone();
        c.data<float>()[0] = 42.f;
        CHECK(a.data<float>()[0] != 42.f);
        Tensor r = a.reshape(Shape{{5, 3}});
        CHECK(r.data<float>() == a.data<float>() && r.shape().dims[0] == 5);
        Tensor h = Tensor::full(Shape{{8}}, TensorOptions().with_dtype(Dtype::Bfloat16), 1.0f + 1.0f / 256);
        CHECK(h.nbytes() == 16 && h.to_vector()[3] == 1.0f);  // 1 + 2^-8 rounds to even in bf16
        Tensor e;
        CHECK(!e.defined() && e.numel() == 0);
    });

    run_test("graph: Value, make_tensor, topo_from", [] {
        Value s(2.0f);
        CHECK(s.node->is_leaf && !s.node->requires_grad() && s.val().numel() == 1 && s.val().to_vector()[0] == 2.0f);
        CHECK(s.shape_2d().first == 1 && s.shape_2d().second == 1);
        Value a = make_tensor(Tensor::zeros(Shape{{2, 3}}, TensorOptions().with_req_grad(true)), "a");
        CHECK(a.node->requires_grad() && a.grad().numel() == 6 && std::string(a.node->debug_name) == "a");
        CHECK(a.shape_2d().first == 2 && a.shape_2d().second == 3);
        // a diamond, built by hand: d depends on b and c, both depend on a
        auto mk = [](std::initializer_list<std::shared_ptr<Node>> in) {
            auto n = std::make_shared<Node>(Tensor::zeros(Shape{{1}}), Op::Add, false, "n");
            n->inputs.assign(in.begin(), in.end());
            return n;
        };
        auto b = mk({a.node}), c = mk({a.node}), d = mk({b, c});
        auto order = topo_from(d.get());
        CHECK(order.size() == 4 && order.front() == a.node.get() && order.back() == d.get());
        // a 100000-deep chain must not overflow the stack
        std::shared_ptr<Node> cur = a.node;
        for (int i = 0; i < 100000; ++i) cur = mk({cur});
        CHECK(topo_from(cur.get()).size() == 100001);
        int fired = 0;
        a.register_hook([&](Node*) { ++fired; });
        for (auto& h : a.node->post_acc_grad_hooks) h(a.node.get());
        CHECK(fired == 1);
    });

    run_test("one stream per graph is a checked rule; lazy gradients read as zeros", [] {
        // interior nodes built under different current streams: backward refuses before it launches anything
        Value a = make_tensor(Tensor::zeros(Shape{{2, 3}}, TensorOptions().with_req_grad(true)), "a");
        auto mk = [](std::initializer_list<std::shared_ptr<Node>> in) {
            auto n = std::make_shared<Node>(Tensor::zeros(Shape{{2, 3}}), Op::Add, true, "n");
            n->inputs.assign(in.begin(), in.end());
            return n;
        };
        set_current_stream(reinterpret_cast<ag_cuda_stream_t>(0x10));
        auto b = mk({a.node, a.node});
        set_current_stream(reinterpret_cast<ag_cuda_stream_t>(0x20));
        auto c = mk({b, b});
        set_current_stream(nullptr);
        bool threw = false;
        try {
            backward(Value(c));
        } catch (const std::runtime_error& e) {
            threw = std::string(e.what()).find("ONE current stream") != std::string::npos;
        }
        CHECK(threw);
        // a leaf made under another stream (a parameter that exists before a capture stream does) is allowed:
        // the check passes and the walk reaches the rule (which, on CPU tensors, is where it stops)
        CHECK(b->creation_context.stream != a.node->creation_context.stream);
        // a gradient nobody has contributed to is not allocated, and reads as zeros through Value::grad()
        CHECK(!a.node->grad.defined() && !a.node->grad_live);
        CHECK(a.grad().numel() == 6 && a.grad().to_vector() == std::vector<float>(6, 0.0f));
        a.node->accumulate_grad(Tensor::full(Shape{{2, 3}}, TensorOptions(), 2.0f));   // first contribution: written
        a.node->accumulate_grad(Tensor::full(Shape{{1}}, TensorOptions(), 0.5f));      // second: added (broadcast)
        CHECK(a.grad().to_vector() == std::vector<float>(6, 2.5f));
        zero_grad(a);                                                                  // lazily: marks the buffer empty
        CHECK(!a.node->grad_live && a.grad().to_vector() == std::vector<float>(6, 0.0f));
        a.node->accumulate_grad(Tensor::full(Shape{{1}}, TensorOptions(), 1.5f));      // a broadcast FIRST contribution
        CHECK(a.grad().to_vector() == std::vector<float>(6, 1.5f));
    });

    run_test("broadcast classification", [] {
        Tensor full = Tensor::zeros(Shape{{4, 5}});
        CHECK(detail::classify_broadcast(full, Tensor::zeros(Shape{{4, 5}})) == AGB_BCAST_FULL);
        CHECK(detail::classify_broadcast(full, Tensor::zeros(Shape{{5}})) == AGB_BCAST_LASTVEC);
        CHECK(detail::classify_broadcast(full, Tensor::zeros(Shape{{1, 5}})) == AGB_BCAST_LASTVEC);
        CHECK(detail::classify_broadcast(full, Tensor::zeros(Shape{{4, 1}})) == AGB_BCAST_ROWSTAT);
        CHECK(detail::classify_broadcast(full, Tensor::zeros(Shape{{1}})) == AGB_BCAST_SCALAR);
        CHECK(detail::classify_broadcast(Tensor::zeros(Shape{{2, 3, 8}}), Tensor::zeros(Shape{{2, 3, 1}})) == AGB_BCAST_ROWSTAT);
        bool threw = false;
        try { detail::classify_broadcast(full, Tensor::zeros(Shape{{4}})); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
    });

    run_test("no CPU implementation: ops on CPU tensors throw", [] {
        Value a = make_tensor(Tensor::randn(Shape{{4, 10}}, TensorOptions().with_req_grad(true)));
        bool threw = false;
        try { rms(a); } catch (const std::runtime_error& e) { threw = std::string(e.what()).find("CPU") != std::string::npos; }
        CHECK(threw);
        threw = false;
        try { a + a; } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
    });

    run_test("allocator budget: out-of-memory is raised on the host", [] {
        auto& al = OwnTensor::cuda::DeviceAllocator::instance();
        al.set_memory_limit(1 << 20);
        bool threw = false;
        try { al.allocate(8 << 20, 0, nullptr); } catch (const std::runtime_error& e) {
            threw = std::string(e.what()).find("out of memory") != std::string::npos;
        }
        al.set_memory_limit(0);
        CHECK(threw);
        CHECK(al.stats().device_allocs == 0);
    });

    run_test("thread-local stream slot", [] {
        CHECK(current_stream() == nullptr);
        set_current_stream(reinterpret_cast<ag_cuda_stream_t>(0x10));
        CHECK(current_stream() == reinterpret_cast<ag_cuda_stream_t>(0x10));
        set_current_stream(nullptr);
        Node n(Tensor::zeros(Shape{{1}}), Op::Leaf, false, "ctx");
        CHECK(n.creation_context.stream == nullptr && !n.creation_context.device.is_cuda());
    });

    run_test("checkpoint marking and deletion policies (no kernels)", [] {
        // a hand-built chain leaf -> n1 -> n2 -> n3 -> root of Add nodes over CPU tensors
        Value a = make_tensor(Tensor::zeros(Shape{{2, 3}}, TensorOptions().with_req_grad(true)), "a");
        auto mk = [](std::shared_ptr<Node> in) {
            auto n = std::make_shared<Node>(Tensor::zeros(Shape{{2, 3}}), Op::Add, true, "n");
            n->inputs = {in, in};
            return n;
        };
        auto n1 = mk(a.node), n2 = mk(n1), n3 = mk(n2), root = mk(n3);
        reset_checkpoint_stats();
        memory::reset_deletion_stats();
        auto_checkpoint_every_n(Value(root), 2);           // breadth-first: root(1) n3(2) n2(3) n1(4) a(5)
        CHECK(n3->is_checkpoint && n1->is_checkpoint && !n2->is_checkpoint && !root->is_checkpoint && !a.node->is_checkpoint);
        CHECK(n3->saved_inputs.size() == 2 && n3->saved_inputs[0].node == n2);
        CHECK(checkpoint_stats().total_checkpoints == 2 && checkpoint_stats().total_memory_saved == 2 * 24);
        auto_checkpoint_by_depth(Value(root), 2);          // n2 (depth 2) and n1 (depth 3, already marked); never the leaf
        CHECK(n2->is_checkpoint && !a.node->is_checkpoint && checkpoint_stats().total_checkpoints == 3);
        checkpoint_impl::mark_node_checkpoint(a.node);     // a leaf cannot be recomputed from anything
        CHECK(!a.node->is_checkpoint);
        CHECK(checkpoint_impl::is_checkpointed(n1) && !checkpoint_impl::is_checkpointed(root) && !checkpoint_impl::is_checkpointed(nullptr));

        std::unordered_set<Node*> keep{n2.get()};
        CHECK(memory::sweep_safe_nodes(Value(root), memory::DeletePolicy::AlwaysSafe, keep) == 0);   // checkpoints, pending grads
        CHECK(memory::sweep_safe_nodes(Value(root), memory::DeletePolicy::ForwardPass, keep) == 2);  // n1 and n3
        CHECK(n1->value.numel() == 0 && n3->value.numel() == 0 && n2->value.numel() == 6 && root->value.numel() == 6);
        CHECK(n1->shape() == std::vector<int64_t>({2, 3}) && n1->value_released);
        CHECK(n1->materialized_grad().numel() == 6);       // ForwardPass keeps gradients
        CHECK(memory::deletion_stats().nodes_deleted == 2 && memory::deletion_stats().memory_freed == 2 * 24);
        zero_grad(Value(root));                            // works on dropped nodes: the shape is remembered
        CHECK(n3->materialized_grad().numel() == 6);
        // recompute needs kernels, so on CPU it fails cleanly and is counted
        CHECK(!checkpoint_impl::recompute_subgraph(n3));
        CHECK(checkpoint_stats().failed_recomputes >= 1 && checkpoint_stats().successful_recomputes == 0);
        CHECK(checkpoint_impl::ensure_value_present(n2) && !checkpoint_impl::ensure_value_present(n3));
    });

    return finish("test_host_cpu");
}
