// Feed-forwards beside SwiGLU: the plain two-matrix one, and the mixture of experts.
//
// "mlp":  down(act(up x)); activation "relu2": act(z) = max(z, 0)^2.
//
// "moe":  n_experts small gated feed-forwards, of which a row uses top_k.  Router logits z = W_router x are float32
//         (the contraction takes the activations as they are and accumulates in float32).  router "sigmoid_input":
//         scores s = sigmoid(z); the top_k largest are chosen; an expert's weight is its own score, not renormalised,
//         and multiplies the expert's INPUT: out = sum_e expert_e(s_e x).  Expert: g = min(W_gate x, limit),
//         u = clamp(W_up x, -limit, limit), y = g sigmoid(alpha g) (u + 1), output W_down y.  Because both first
//         contractions are linear, s_e is applied to their float32 results.
//         Rows are grouped by expert on the device (experts.cu).  A decode step and short portions never tell the host
//         the routing, so a recorded decode step replays with whatever the router chooses.  A long portion in bfloat16
//         reads the experts' row counts back once (one small copy; such a step is never recorded) and runs the experts'
//         contractions over their runs of rows as ONE grouped launch each of the tensor-core kernel every other
//         projection uses (a table of tiles tells it which rows meet which expert's matrix).
//         router "softmax_grouped": scores s = softmax(z) over n_experts + n_identity router outputs; the choice is made on
//         s + b (b: the tensor router.bias, a number per output) among the outputs of the keep_groups best of n_groups equal
//         groups of neighbours (a group's score: its largest s + b); the top_k chosen outputs weigh in with
//         s / (sum of the chosen s + 1e-20) * route_scale, and the weight multiplies the expert's OUTPUT.  The last
//         n_identity outputs have no expert: their "output" is the feed-forward's input itself.  Expert:
//         W_down (silu(W_gate x) * (W_up x)).  shared_d_ff > 0: one more gated feed-forward of that size ("shared.*" tensors)
//         runs on every row and is added.
#include <algorithm>
#include <cmath>

#include "parts.hpp"

namespace fg {

class PlainMLP : public FeedForward {
public:
    PlainMLP(const Json &p) : E_((int)param_int(p, "hidden_size", "mlp")), F_((int)param_int(p, "d_ff", "mlp")) {
        if (E_ <= 0 || F_ <= 0) fail(FG_E_CONFIG, "mlp: sizes must be positive");
        const Json &a = p.get("activation");
        std::string act = a.is_string() ? a.as_string() : "relu2";
        if (act != "relu2") fail(FG_E_CONFIG, "mlp: activation '" + act + "' is not known (known: relu2)");
    }
    std::vector<TensorDecl> tensor_decls() const override { return {{"up_proj.weight", {F_, E_}}, {"down_proj.weight", {E_, F_}}}; }
    bool can_overwrite() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &) override {
        up_ = Linear(tensor_of(tensors, "up_proj.weight"));
        down_ = Linear(tensor_of(tensors, "down_proj.weight"));
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &, Tensor &residual, Norm *emit_norm) override {
        Tensor t = up_.forward_relu2(rt, xn);
        DeferredNorm started;
        down_.forward(rt, t, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_, F_;
    Linear up_, down_;
};

class MoEFeedForward : public FeedForward {
public:
    MoEFeedForward(const Json &p) {
        const char *me = "moe";
        E_ = (int)param_int(p, "hidden_size", me);
        F_ = (int)param_int(p, "d_ff", me);
        X_ = (int)param_int(p, "n_experts", me);
        top_ = (int)param_int(p, "top_k", me);
        const Json &r = p.get("router");
        std::string kind = r.is_string() ? r.as_string() : "sigmoid_input";
        if (kind != "sigmoid_input" && kind != "softmax_grouped") fail(FG_E_CONFIG, "moe: router '" + kind + "' is not known (known: sigmoid_input, softmax_grouped)");
        grouped_ = kind == "softmax_grouped";
        if (E_ <= 0 || F_ <= 0 || X_ <= 0 || top_ <= 0) fail(FG_E_CONFIG, "moe: sizes must be positive");
        if (grouped_) {
            identity_ = (int)param_int(p, "n_identity", 0, me);
            groups_ = (int)param_int(p, "n_groups", 1, me);
            keep_ = (int)param_int(p, "keep_groups", groups_, me);
            route_scale_ = (float)param_float(p, "route_scale", 1.0, me);
            shared_ff_ = (int)param_int(p, "shared_d_ff", 0, me);
            if (identity_ < 0 || shared_ff_ < 0) fail(FG_E_CONFIG, "moe: n_identity and shared_d_ff cannot be negative");
            const int outputs = X_ + identity_;
            if (groups_ <= 0 || groups_ > 64 || outputs % groups_) fail(FG_E_CONFIG, format("moe: %d router outputs do not form %d equal groups (at most 64)", outputs, groups_));
            if (keep_ <= 0 || keep_ > groups_) fail(FG_E_CONFIG, format("moe: keep_groups %d must lie in 1 .. n_groups (%d)", keep_, groups_));
            if (top_ > keep_ * (outputs / groups_)) fail(FG_E_CONFIG, format("moe: top_k %d exceeds the %d outputs of the groups that stay", top_, keep_ * (outputs / groups_)));
            limit_ = 0.f;                    // the kernels' code for the plain gated form silu(g) * u
            if (shared_ff_ > 0) {
                Json sp = Json::object();
                sp.set("hidden_size", (long long)E_);
                sp.set("d_ff", (long long)shared_ff_);
                shared_ = make_swiglu(sp);
            }
        } else {
            limit_ = (float)param_float(p, "limit", me);
            alpha_ = (float)param_float(p, "alpha", 1.702, me);
            if (!(limit_ > 0.f)) fail(FG_E_CONFIG, "moe: limit must be positive");
        }
        if (top_ > X_ + identity_) fail(FG_E_CONFIG, format("moe: top_k %d exceeds the %d experts", top_, X_ + identity_));
        if (X_ + identity_ > 256 || top_ > 8) fail(FG_E_CONFIG, "moe: the routing kernel takes up to 256 experts and top_k up to 8");
    }
    std::vector<TensorDecl> tensor_decls() const override {
        std::vector<TensorDecl> d = {{"router.weight", {X_ + identity_, E_}}};
        if (grouped_) d.push_back({"router.bias", {X_ + identity_}, false, 0, 0.05f});
        if (shared_)
            for (auto &t : shared_->tensor_decls()) { TensorDecl c = t; c.name = "shared." + t.name; d.push_back(c); }
        for (int e = 0; e < X_; e++) {
            std::string pre = "experts." + std::to_string(e) + ".";
            d.push_back({pre + "gate_proj.weight", {F_, E_}});
            d.push_back({pre + "up_proj.weight", {F_, E_}});
            d.push_back({pre + "down_proj.weight", {E_, F_}});
        }
        return d;
    }
    bool can_overwrite() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        router_ = Linear(tensor_of(tensors, "router.weight"));
        // experts one after another: [X, 2F, E] (gate rows, then up rows) and [X, E, F], in the engine's dtype
        std::vector<Weight> in, out;
        for (int e = 0; e < X_; e++) {
            std::string pre = "experts." + std::to_string(e) + ".";
            in.push_back(tensor_of(tensors, (pre + "gate_proj.weight").c_str()));
            in.push_back(tensor_of(tensors, (pre + "up_proj.weight").c_str()));
            out.push_back(tensor_of(tensors, (pre + "down_proj.weight").c_str()));
        }
        w_in_ = concat_rows(in, rt.dtype, rt.stream);
        w_out_ = concat_rows(out, rt.dtype, rt.stream);
        if (!counts_host_) FG_CUDA(cudaMallocHost((void **)&counts_host_, ((size_t)X_ + identity_ + 1) * sizeof(int)));
        if (grouped_) {
            const Weight &b = tensor_of(tensors, "router.bias");
            route_bias_ = b.t.dtype == FG_F32 ? b : concat_rows({b}, FG_F32, rt.stream);
        }
        if (shared_) {
            std::map<std::string, Weight> mine;
            for (auto &t : shared_->tensor_decls()) mine[t.name] = tensor_of(tensors, ("shared." + t.name).c_str());
            shared_->load(mine, rt);
        }
    }
    ~MoEFeedForward() override {
        if (counts_host_) cudaFreeHost(counts_host_);
        if (tiles_host_) cudaFreeHost(tiles_host_);
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &batch, Tensor &residual, Norm *emit_norm) override {
        if (!shared_) return routed(rt, xn, residual);
        // the routed experts first (they may write instead of add), then the shared expert adds; its output projection is the
        // block's last, so it may start the next norm
        routed(rt, xn, residual);
        const bool was = rt.overwrite;
        rt.overwrite = false;
        DeferredNorm started = shared_->forward(rt, xn, nullptr, batch, residual, emit_norm);
        rt.overwrite = was;
        return started;
    }
    bool supports_deferred_norm() const override { return false; }

private:
    DeferredNorm routed(Runtime &rt, const Tensor &xn, Tensor &residual) {
        const int M = (int)xn.rows, P = M * top_, XR = X_ + identity_;
        if (M == 0) return DeferredNorm();
        if (xn.dtype != rt.dtype) fail(FG_E_INTERNAL, "moe: the input must be in the engine's dtype");
        // plain contraction: float32 accumulation of the activations as they are, float32 logits
        Tensor z = rt.arena->matrix(M, XR, FG_F32);
        const Tensor &R = router_.weight().t;
        if (R.dtype == xn.dtype)
            FG_LAUNCH("mix", fg_moe_logits, xn.data, (int)xn.ld, R.data, (int)R.ld, xn.dtype, z.ptr<float>(), M, XR, E_, rt.stream);
        else
            FG_LAUNCH("core", fg_gemm_generic, xn.data, xn.dtype, (int)xn.ld, R.data, R.dtype, (int)R.ld, z.data, FG_F32, (int)z.ld, 0, M, XR,
                      E_, rt.stream);
        int *ints = (int *)rt.arena->alloc(((size_t)3 * P + XR + 1) * sizeof(int));
        int *pair_expert = ints, *order = ints + P, *slot_of = ints + 2 * P, *offsets = ints + 3 * P;
        float *pair_weight = (float *)rt.arena->alloc((size_t)P * sizeof(float));
        if (grouped_)
            FG_LAUNCH("mix", fg_moe_route_grouped, z.ptr<float>(), route_bias_.t.ptr<float>(), M, XR, top_, groups_, keep_, route_scale_, pair_expert,
                      pair_weight, offsets, order, slot_of, rt.stream);
        else
            FG_LAUNCH("mix", fg_moe_route, z.ptr<float>(), M, X_, top_, pair_expert, pair_weight, offsets, order, slot_of, rt.stream);
        Tensor y = rt.arena->matrix(P, F_, rt.dtype);
        Tensor o = rt.arena->matrix(P, E_, FG_F32);
        // where the routing weight enters: the experts' inputs (through the float32 gate/up results), or their outputs (the sum)
        const float *in_weight = grouped_ ? nullptr : pair_weight;
        auto combine = [&]() {
            if (grouped_)
                FG_LAUNCH("mix", fg_moe_combine_weighted, o.ptr<float>(), (int)o.ld, slot_of, pair_expert, pair_weight, xn.data, (int)xn.ld, xn.dtype, X_,
                          residual.ptr<float>(), M, top_, E_, rt.overwrite ? 0 : 1, rt.stream);
            else
                FG_LAUNCH("mix", fg_moe_combine, o.ptr<float>(), (int)o.ld, slot_of, residual.ptr<float>(), M, top_, E_, rt.overwrite ? 0 : 1, rt.stream);
        };
        if (!rt.recording && !rt.plain_kernels && rt.dtype == FG_BF16 && P >= grouped_from_ && E_ % 8 == 0 && F_ % 8 == 0) {
            // a long portion: the experts' row counts come to the host, and the experts' runs of rows go through the
            // tensor-core contraction; gate and up leave it as float32, so the routing weight and the clamps see what
            // the accumulators held
            FG_CUDA(cudaMemcpyAsync(counts_host_, offsets, ((size_t)XR + 1) * sizeof(int), cudaMemcpyDeviceToHost, rt.stream));
            FG_CUDA(cudaStreamSynchronize(rt.stream));
            Tensor xs = rt.arena->matrix(P, E_, rt.dtype);
            FG_LAUNCH("mix", fg_moe_gather, xn.data, (int)xn.ld, xn.dtype, order, top_, xs.data, P, E_, rt.stream);
            Tensor gu = rt.arena->matrix(P, (int64_t)2 * F_, FG_F32);
            // both contractions as ONE launch each over all experts: a table of tiles {first row, end of the expert's run,
            // the expert's first row in the stack, tile along the outputs}, an expert's tiles side by side so that its
            // weights stay in L2 while its row tiles pass
            const int bn1 = FG_KERNEL("tc", fg_gemm_tc_grouped_bn)(2 * F_), bn2 = FG_KERNEL("tc", fg_gemm_tc_grouped_bn)(E_);
            auto count_tiles = [&](int N, int bn) {
                size_t n = 0;
                for (int e = 0; e < X_; e++) n += (size_t)((counts_host_[e + 1] - counts_host_[e] + 127) / 128) * (size_t)((N + bn - 1) / bn);
                return n;
            };
            const size_t n1 = count_tiles(2 * F_, bn1), n2 = count_tiles(E_, bn2);
            if (tiles_cap_ < n1 + n2) {
                if (tiles_host_) FG_CUDA(cudaFreeHost(tiles_host_));
                tiles_host_ = nullptr;
                tiles_cap_ = std::max<size_t>(2 * (n1 + n2), 1024);
                FG_CUDA(cudaMallocHost((void **)&tiles_host_, tiles_cap_ * 4 * sizeof(int)));
            }
            auto fill = [&](int *t, int N, int bn) {
                for (int e = 0; e < X_; e++) {
                    const int a = counts_host_[e], b = counts_host_[e + 1];
                    for (int qt = 0; qt < (N + bn - 1) / bn; qt++)
                        for (int r = a; r < b; r += 128) { *t++ = r; *t++ = b; *t++ = e * N; *t++ = qt; }
                }
            };
            fill(tiles_host_, 2 * F_, bn1);
            fill(tiles_host_ + 4 * n1, E_, bn2);
            int *tiles_dev = (int *)rt.arena->alloc((n1 + n2) * 4 * sizeof(int));
            // (the stream was waited for above, after this buffer's last copy was queued: it is free to be rewritten)
            FG_CUDA(cudaMemcpyAsync(tiles_dev, tiles_host_, (n1 + n2) * 4 * sizeof(int), cudaMemcpyHostToDevice, rt.stream));
            FG_LAUNCH("tc", fg_gemm_tc_grouped, xs.data, (int)xs.ld, P, w_in_.t.data, (int)w_in_.t.ld, (int)w_in_.t.rows, gu.ptr<float>(),
                      (int)gu.ld, 2 * F_, E_, tiles_dev, (int)n1, rt.stream);
            FG_LAUNCH("mix", fg_moe_act, gu.ptr<float>(), order, in_weight, y.data, y.dtype, P, F_, limit_, alpha_, rt.stream);
            FG_LAUNCH("tc", fg_gemm_tc_grouped, y.data, (int)y.ld, P, w_out_.t.data, (int)w_out_.t.ld, (int)w_out_.t.rows, o.ptr<float>(),
                      (int)o.ld, E_, F_, tiles_dev + 4 * n1, (int)n2, rt.stream);
            combine();
            return DeferredNorm();
        }
        FG_LAUNCH("mix", fg_moe_first, xn.data, (int)xn.ld, w_in_.t.data, y.data, (int)y.ld, rt.dtype, pair_expert, offsets, order, in_weight,
                  M, X_, top_, F_, E_, limit_, alpha_, rt.stream);
        FG_LAUNCH("mix", fg_moe_second, y.data, (int)y.ld, w_out_.t.data, o.ptr<float>(), (int)o.ld, rt.dtype, pair_expert, offsets, order, M,
                  X_, top_, F_, E_, rt.stream);
        combine();
        return DeferredNorm();
    }

    int E_ = 0, F_ = 0, X_ = 0, top_ = 0;
    int identity_ = 0, groups_ = 1, keep_ = 1, shared_ff_ = 0;      // router "softmax_grouped"
    bool grouped_ = false;
    float route_scale_ = 1.f;
    Weight route_bias_;
    std::unique_ptr<FeedForward> shared_;
    float limit_ = 0.f, alpha_ = 1.702f;
    int grouped_from_ = 256;                 // pairs (rows x choices) from which a portion takes the contraction per expert
    Linear router_;
    Weight w_in_, w_out_;
    int *counts_host_ = nullptr;             // pinned: where the experts' runs of slots start
    int *tiles_host_ = nullptr;              // pinned: the tile tables of a long portion's two contractions
    size_t tiles_cap_ = 0;
};

void add_expert_kinds(std::map<std::string, PartFactory> &ffs) {
    ffs["mlp"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<PlainMLP>(p); };
    ffs["moe"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<MoEFeedForward>(p); };
}

}  // namespace fg
