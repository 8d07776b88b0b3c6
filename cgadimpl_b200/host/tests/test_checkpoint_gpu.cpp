// test_checkpoint_gpu.cpp -- activation checkpointing across a residual RMSNorm stack: mark,
// drop the activations after the forward pass, let the backward pass recompute them, and compare
// every gradient bit for bit with the run that kept everything.  Mirrors the scenario of
// cgadimpl/Tests/test_checkpoint.cpp:76-170 (deep model, anchors, sweep, backward) on the ops of
// this path; there the recompute of a normalisation node throws.
#include <unordered_set>

#include "ad/ag_all.hpp"
#include "check.hpp"

using namespace ag;

static const auto kDev = DeviceIndex(Device::CUDA);

static std::vector<float> randv(size_t n, unsigned seed, float scale = 1.f, float shift = 0.f) {
    std::vector<float> v(n);
    uint64_t s = seed * 0x9E3779B97F4A7C15ull + 1;
    for (auto& x : v) {
        double acc = 0;
        for (int k = 0; k < 4; ++k) { s = s * 6364136223846793005ull + 1442695040888963407ull; acc += double(s >> 11) / 9007199254740992.0; }
        x = shift + scale * float((acc - 2.0) * 1.7320508);
    }
    return v;
}
static Value leaf(const std::vector<float>& v, std::vector<int64_t> dims, bool req = true) {
    return make_tensor(Tensor::from_host(v.data(), Shape{dims}, TensorOptions().with_device(kDev).with_req_grad(req)));
}

struct Stack {
    Value x, r, out;
    std::vector<Value> gammas;
    std::vector<Value> hs, ys;  // per layer: the residual sum and the layer output
};

// fused == false builds the reference's composition add -> rms -> mul (three nodes per layer).
static Stack build(int L, int64_t R, int64_t H, bool fused) {
    Stack s;
    s.x = leaf(randv(R * H, 11), {R, H});
    s.r = leaf(randv(R * H, 12), {R, H});
    Value x = s.x, r = s.r;
    for (int l = 0; l < L; ++l) {
        Value g = leaf(randv(H, 100 + l, 0.05f, 1.0f), fused ? std::vector<int64_t>{H} : std::vector<int64_t>{1, H});
        s.gammas.push_back(g);
        Value h, y;
        if (fused) {
            y = add_rmsnorm(x, r, g);
            h = residual_of(y);
        } else {
            h = add(x, r);
            y = mul(rms(h), g);
        }
        s.hs.push_back(h);
        s.ys.push_back(y);
        x = h;
        r = y;
    }
    s.out = r;
    return s;
}

struct Grads {
    std::vector<float> dx, dr;
    std::vector<std::vector<float>> dg;
};
static Grads grads_of(const Stack& s) {
    Grads g{s.x.grad().to_vector(), s.r.grad().to_vector(), {}};
    for (auto& gm : s.gammas) g.dg.push_back(gm.grad().to_vector());
    return g;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 2; }
    const int L = 6;
    const int64_t R = 256, H = 1024;
    const auto seedv = randv(R * H, 7);
    auto& alloc = OwnTensor::cuda::DeviceAllocator::instance();

    for (int fused = 0; fused <= 1; ++fused) {
        const std::string tag = fused ? " (fused nodes)" : " (add / rms / mul nodes)";
        Tensor seed = Tensor::from_host(seedv.data(), Shape{{R, H}}, TensorOptions().with_device(kDev));

        Stack plain = build(L, R, H, fused);
        zero_grad(plain.out);
        backward(plain.out, &seed);
        const Grads want = grads_of(plain);
        const auto out_want = plain.out.val().to_vector();

        run_test("drop + recompute gives the same bits" + tag, [&] {
            reset_checkpoint_stats();
            memory::reset_deletion_stats();
            Stack cp = build(L, R, H, fused);
            // anchors: every second residual sum stays; everything else may be recomputed
            std::unordered_set<Node*> anchors;
            for (int l = 0; l < L; l += 2) anchors.insert(cp.hs[l].node.get());
            for (Node* n : topo_from(cp.out.node.get()))
                if (n->op != Op::Leaf && !anchors.count(n)) checkpoint_impl::mark_node_checkpoint(n->shared_from_this());
            const size_t before = alloc.stats().bytes_in_use;
            const int dropped = memory::sweep_safe_nodes(cp.out, memory::DeletePolicy::ForwardPass, anchors);
            const size_t after = alloc.stats().bytes_in_use;
            const int nodes_per_layer = fused ? 2 : 3;
            CHECK(dropped == L * nodes_per_layer - int(anchors.size()) - 1);          // the root is never dropped
            CHECK(before - after >= size_t(dropped) * size_t(R * H) * sizeof(float));   // the memory really came back
            CHECK(memory::deletion_stats().nodes_deleted == size_t(dropped));
            CHECK(cp.ys[0].val().numel() == 0 && cp.ys[0].node->tape.empty());
            CHECK(cp.ys[0].shape() == std::vector<int64_t>({R, H}));                    // the shape survives the drop
            CHECK(cp.out.val().to_vector() == out_want);

            zero_grad(cp.out);
            backward(cp.out, &seed);
            const Grads got = grads_of(cp);
            CHECK(got.dx == want.dx && got.dr == want.dr);
            for (int l = 0; l < L; ++l) CHECK(got.dg[l] == want.dg[l]);
            const CheckpointStats st = checkpoint_stats();
            CHECK(st.successful_recomputes > 0 && st.failed_recomputes == 0);
            CHECK(st.total_checkpoints == size_t(L * nodes_per_layer) - anchors.size());
            // recomputed activations were dropped again once their last reader had run
            CHECK(cp.ys[1].val().numel() == 0);
            // (gradient buffers are allocated by the backward pass itself, at the first contribution to each node)
            size_t grad_bytes = 0;
            for (Node* n : topo_from(cp.out.node.get())) grad_bytes += n->grad.nbytes();
            CHECK(alloc.stats().bytes_in_use <= before + grad_bytes);
        });

        run_test("parallel backward over dropped activations" + tag, [&] {
            Stack cp = build(L, R, H, fused);
            std::unordered_set<Node*> anchors{cp.hs[0].node.get(), cp.hs[3].node.get()};
            for (Node* n : topo_from(cp.out.node.get()))
                if (n->op != Op::Leaf && !anchors.count(n)) checkpoint(Value(n->shared_from_this()));
            memory::sweep_safe_nodes(cp.out, memory::DeletePolicy::ForwardPass, anchors);
            zero_grad(cp.out);
            backward(cp.out, &seed, /*enable_parallel=*/true);
            const Grads got = grads_of(cp);
            CHECK(got.dx == want.dx && got.dr == want.dr);
            for (int l = 0; l < L; ++l) CHECK(got.dg[l] == want.dg[l]);
        });
    }

    run_test("forward_eval_node restores value and tape of every op", [&] {
        Value x = leaf(randv(R * H, 21), {R, H}), g = leaf(randv(H, 22, 0.05f, 1.0f), {H});
        Value g2 = leaf(randv(H, 22, 0.05f, 1.0f), {1, H});
        std::vector<Value> nodes = {add(x, x), mul(x, g2), rms(x), realrms(x, 1.5f), rmsnorm(x, g), laynor(x),
                                    sum(x), mean_all(x), rowsum(x), rowmax(x), softmax_row(x), logsumexp_row(x)};
        for (auto& v : nodes) {
            const auto val = v.val().to_vector();
            std::vector<std::vector<float>> tape;
            for (auto& t : v.node->tape) tape.push_back(t->to_vector());
            v.node->value = Tensor();
            v.node->tape.clear();
            v.node->value = forward_eval_node(v.node);
            CHECK(v.val().to_vector() == val);
            CHECK(v.node->tape.size() == tape.size());
            for (size_t i = 0; i < tape.size() && i < v.node->tape.size(); ++i) CHECK(v.node->tape[i]->to_vector() == tape[i]);
        }
    });

    run_test("what cannot be recomputed is reported, not guessed", [&] {
        Value x = leaf(randv(R * H, 31), {R, H});
        Value a = add(x, x);          // not a checkpoint
        Value y = checkpoint(rms(a));
        a.node->value = Tensor();     // dropped by hand although nothing can bring it back
        y.node->value = Tensor();
        y.node->tape.clear();
        reset_checkpoint_stats();
        CHECK(!checkpoint_impl::recompute_subgraph(y.node));
        CHECK(checkpoint_stats().failed_recomputes >= 1);
        CHECK(!checkpoint_impl::recompute_subgraph(a.node));   // not marked
        bool threw = false;
        try { forward_eval_node(y.node); } catch (const std::exception&) { threw = true; }
        CHECK(threw);
        // policies: a plain sweep keeps checkpoints and anything whose inputs still await gradients
        Value b = checkpoint(add(x, x));
        CHECK(!memory::try_delete_node(b.node.get(), memory::DeletePolicy::AlwaysSafe));
        CHECK(!memory::try_delete_node(x.node.get(), memory::DeletePolicy::ForwardPass));   // leaf
        Value c = add(x, x);
        CHECK(!memory::try_delete_node(c.node.get(), memory::DeletePolicy::ForwardPass));   // could not be recomputed
        CHECK(memory::try_delete_node(b.node.get(), memory::DeletePolicy::ForwardPass));
    });

    return finish("test_checkpoint_gpu");
}
