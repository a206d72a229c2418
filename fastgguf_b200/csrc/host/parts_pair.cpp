// "mixer_pair": two mixers side by side.  Both read the same normalised rows h, and their outputs are joined:
//     y = left_scale * f_l(left(h)) + right_scale * f_r(right(h)),
//     f(t) = t / sqrt(mean(t^2) + eps) * w over the model width where "normalize" is true (a plain weight for each side),
//     f(t) = t where it is not.
// The two are any mixer kinds of the registry, {"kind", "params"} under "left" and "right"; their tensors are declared under
// "left.<name>" and "right.<name>", the two norm weights as "left_norm.weight" and "right_norm.weight".  At most one of the
// two may keep keys and values (the schedule entry has one cache); their fixed-size states lie one behind the other in the
// entry's state row, which needs kinds that read the row stride (`strided_state`) as soon as both, or a narrower one, have some.
// Each side writes its output into a float32 buffer of its own; one kernel normalises, weighs and adds both into the stream.
#include "parts.hpp"

namespace fg {

class PairMixer : public Mixer {
public:
    PairMixer(Runtime &rt, const Json &p, BuildContext &ctx) {
        const char *me = "mixer_pair";
        E_ = (int)param_int(p, "hidden_size", me);
        scale_[0] = (float)param_float(p, "left_scale", 1.0, me);
        scale_[1] = (float)param_float(p, "right_scale", 1.0, me);
        normalize_ = p.get("normalize").is_bool() && p.get("normalize").as_bool();
        eps_ = (float)param_float(p, "eps", 1e-6, me);
        if (E_ <= 0) fail(FG_E_CONFIG, "mixer_pair: hidden_size must be positive");
        if (normalize_ && !(eps_ > 0.f)) fail(FG_E_CONFIG, "mixer_pair: eps must be positive");
        const char *side[2] = {"left", "right"};
        for (int i = 0; i < 2; i++) {
            const Json &c = p.get(side[i]);
            if (!c.is_object() || !c.get("kind").is_string() || !c.get("params").is_object())
                fail(FG_E_CONFIG, format("mixer_pair: '%s' must be {\"kind\": ..., \"params\": ...}", side[i]));
            std::unique_ptr<Part> part = build_part(FG_ROLE_MIXER, c.get("kind").as_string(), rt, c.get("params"), ctx);
            child_[i].reset(dynamic_cast<Mixer *>(part.get()));
            if (!child_[i]) fail(FG_E_CONFIG, format("mixer_pair: '%s' is not a mixer", side[i]));
            part.release();
            prefix_[i] = std::string(side[i]) + ".";
        }
        CacheRequest a, b;
        if (child_[0]->cache_request(&a) && child_[1]->cache_request(&b))
            fail(FG_E_CONFIG, "mixer_pair: only one of the two mixers may keep keys and values");
        const int64_t total = state_bytes();
        for (int i = 0; i < 2; i++)
            if (child_[i]->state_bytes() > 0 && child_[i]->state_bytes() != total && !child_[i]->strided_state())
                fail(FG_E_CONFIG, format("mixer_pair: the %s mixer cannot share a state row with another", i ? "right" : "left"));
    }
    std::vector<TensorDecl> tensor_decls() const override {
        std::vector<TensorDecl> d;
        for (int i = 0; i < 2; i++)
            for (TensorDecl t : child_[i]->tensor_decls()) {
                t.name = prefix_[i] + t.name;
                d.push_back(std::move(t));
            }
        if (normalize_) {
            d.push_back({"left_norm.weight", {(int64_t)E_}, false, 1, 0.01f});
            d.push_back({"right_norm.weight", {(int64_t)E_}, false, 1, 0.01f});
        }
        return d;
    }
    bool cache_request(CacheRequest *out) const override { return child_[0]->cache_request(out) || child_[1]->cache_request(out); }
    int64_t state_bytes() const override { return child_[0]->state_bytes() + child_[1]->state_bytes(); }
    bool can_overwrite() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        for (int i = 0; i < 2; i++) {
            std::map<std::string, Weight> mine;
            for (auto &kv : tensors)
                if (kv.first.compare(0, prefix_[i].size(), prefix_[i]) == 0) mine[kv.first.substr(prefix_[i].size())] = kv.second;
            child_[i]->load(mine, rt);
        }
        if (normalize_) {
            norm_w_[0] = concat_rows({tensor_of(tensors, "left_norm.weight")}, FG_F32, rt.stream);
            norm_w_[1] = concat_rows({tensor_of(tensors, "right_norm.weight")}, FG_F32, rt.stream);
        }
    }
    void prepare(Runtime &rt, int max_positions) override {
        for (auto &c : child_) c->prepare(rt, max_positions);
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *) override {
        const int M = (int)xn.rows;
        const bool add = !rt.overwrite;
        Tensor t[2];
        int64_t at = 0;
        for (int i = 0; i < 2; i++) {
            LayerIO mine = io;
            CacheRequest r;
            if (!child_[i]->cache_request(&r)) { mine.group = -1; mine.k_pool = mine.v_pool = nullptr; }
            const int64_t sb = child_[i]->state_bytes();
            mine.state = sb > 0 ? (char *)io.state + at : nullptr;
            mine.state_bytes = sb;
            at += sb;
            t[i] = rt.arena->matrix(M, E_, FG_F32);
            rt.overwrite = child_[i]->can_overwrite();
            if (!rt.overwrite && M > 0) FG_CUDA(cudaMemsetAsync(t[i].data, 0, (size_t)M * E_ * sizeof(float), rt.stream));
            child_[i]->forward(rt, xn, nullptr, b, mine, t[i], nullptr);
        }
        rt.overwrite = false;
        FG_LAUNCH("core", fg_pair_combine, t[0].ptr<float>(), t[1].ptr<float>(), normalize_ ? norm_w_[0].t.ptr<float>() : nullptr,
                  normalize_ ? norm_w_[1].t.ptr<float>() : nullptr, scale_[0], scale_[1], eps_, residual.ptr<float>(), M, E_, add ? 1 : 0, rt.stream);
        return DeferredNorm();
    }

private:
    int E_ = 0;
    float scale_[2] = {1.f, 1.f}, eps_ = 1e-6f;
    bool normalize_ = false;
    std::unique_ptr<Mixer> child_[2];
    std::string prefix_[2];
    Weight norm_w_[2];
};

void add_pair_kinds(std::map<std::string, PartFactory> &mixers) {
    mixers["mixer_pair"] = [](Runtime &rt, const Json &p, BuildContext &c) { return std::make_unique<PairMixer>(rt, p, c); };
}

}  // namespace fg
