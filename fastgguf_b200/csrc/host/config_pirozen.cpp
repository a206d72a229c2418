// The Pirozen decoder's config.json, and the model it describes as data.
//
// Keys: "architecture": "Pirozen"; "vocab", "width"; "norm": {"eps"}; "layers": a list, each
// {"type": "attention", "mixer": {...}, "mlp": {...} | null}; optional "loop": {"start", "stop", "times"}; optional
// "token_side": {"dim"}.
//   attention mixer  {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims",
//                     "scaling": {"factor", "original", "fast", "slow"}}} - mask, rot and rot.scaling are each left out by a
//                    model that has none
//   mlp              {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "identity",
//                     "groups": {"count", "keep"}}, "shared": {"ff"}} - identity, groups and shared are optional
// Every size and constant above comes from the file.  What the design itself fixes is written here once: every layer is a
// parallel block with two norms of the same stream, x += mixer(norm1(x)) + ff(norm2(x)); norms multiply by their weight as
// stored; attention has biases on q, k, v and o, an RMS norm per head on q and k with one weight vector for all heads, rotary
// pairs (i, i + dims / 2), an ordinary softmax over the window and a sigmoid gate per head; the experts are gated by SiLU, the
// router is a softmax with a selection bias, groups and identity experts, and the chosen scores are renormalised; behind the
// feed-forward every layer adds a token input (a slice of a second embedding table, gated by the stream, projected and
// normalised); the head is a matrix of its own.  With "loop", layers start .. stop - 1 run `times` times in a row, every pass
// with caches of its own, and in front of each pass (the first too) the stream becomes W_in [x; embedding output].
// Tensor names: embed, head, final.norm, loop.in, side.embed, l<i>.norm1, l<i>.norm2, l<i>.mix.{q,k,v,o}(.b), l<i>.mix.{q,k}.norm,
// l<i>.mix.g, l<i>.mlp.router, l<i>.mlp.correction, l<i>.mlp.e<j>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down},
// l<i>.side.{gate,proj,norm}.
#include <cmath>

#include "config.hpp"

namespace fg {

static const std::string kPirozenName = "Pirozen";

static const Json *object_or_absent(const Json &d, const std::string &key, const std::string &where) {
    const Json *v = d.find(key);
    if (!v || v->is_null()) return nullptr;
    if (!v->is_object()) fail(FG_E_CONFIG, where + ": '" + key + "' must be an object");
    return v;
}

class PirozenConfig : public ModelConfig {
public:
    struct Layer {
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0, window = 0;
        double scale = 0.0;
        bool rotates = false, scaled = false;
        double rot_base = 0.0, factor = 1.0, original = 0.0, fast = 0.0, slow = 0.0;
        long long rot_dims = 0;
        bool has_mlp = false;
        long long ff = 0, experts = 0, top = 0, identity = 0, groups = 1, keep = 1, shared_ff = 0;
        double route_scale = 1.0;
    };
    Json source;
    long long vocab = 0, width = 0, side_dim = 0;
    double eps = 0.0;
    bool loops = false;
    long long loop_start = 0, loop_stop = 0, loop_times = 1;
    std::vector<Layer> layers;

    static std::unique_ptr<ModelConfig> from_json(const Json &d) {
        auto cfg = std::make_unique<PirozenConfig>();
        PirozenConfig &c = *cfg;
        c.source = d;
        c.vocab = take_int(d, "vocab");
        c.width = take_int(d, "width");
        const Json *norm = object_or_absent(d, "norm", "config.json");
        if (!norm) fail(FG_E_CONFIG, "config.json: 'norm' must be an object");
        c.eps = take_float(*norm, "eps", "config.json norm");
        if (c.vocab <= 0 || c.width <= 0) fail(FG_E_CONFIG, "config.json: vocab and width must be positive");
        if (!(c.eps > 0.0)) fail(FG_E_CONFIG, format("config.json: norm.eps must be positive, got %g", c.eps));
        if (const Json *side = object_or_absent(d, "token_side", "config.json")) {
            c.side_dim = take_int(*side, "dim", "config.json token_side");
            if (c.side_dim <= 0) fail(FG_E_CONFIG, "config.json token_side: dim must be positive");
        }
        const Json *ls = d.find("layers");
        if (!ls || !ls->is_array() || ls->size() == 0) fail(FG_E_CONFIG, "config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < ls->size(); i++) {
            const Json &l = (*ls)[i];
            std::string w = format("config.json layers[%zu]", i);
            if (!l.is_object()) fail(FG_E_CONFIG, w + " must be an object");
            Layer y;
            std::string type = take_string(l, "type", "", w.c_str());
            if (type != "attention") fail(FG_E_CONFIG, w + ": type '" + type + "' is not known (known: attention)");
            const Json *mp = object_or_absent(l, "mixer", w);
            if (!mp) fail(FG_E_CONFIG, w + ": 'mixer' must be an object");
            const Json &m = *mp;
            std::string wm = w + ".mixer";
            y.heads = take_int(m, "heads", wm.c_str());
            y.kv_heads = take_int(m, "kv_heads", y.heads, wm.c_str());
            y.dim = take_int(m, "dim", wm.c_str());
            y.vdim = take_int(m, "vdim", y.dim, wm.c_str());
            if (y.heads <= 0 || y.kv_heads <= 0 || y.dim <= 0 || y.vdim <= 0) fail(FG_E_CONFIG, wm + ": heads, kv_heads, dim and vdim must be positive");
            if (y.heads % y.kv_heads) fail(FG_E_CONFIG, wm + format(": heads (%lld) must be a multiple of kv_heads (%lld)", y.heads, y.kv_heads));
            y.scale = take_float(m, "scale", 1.0 / std::sqrt((double)y.dim), wm.c_str());
            if (const Json *mask = object_or_absent(m, "mask", wm)) {
                y.window = take_int(*mask, "size", (wm + ".mask").c_str());
                if (y.window <= 0) fail(FG_E_CONFIG, wm + ".mask: size must be positive");
            }
            if (const Json *rot = object_or_absent(m, "rot", wm)) {
                std::string wr = wm + ".rot";
                y.rotates = true;
                y.rot_base = take_float(*rot, "base", wr.c_str());
                if (!(y.rot_base > 1.0)) fail(FG_E_CONFIG, wr + ": base must exceed 1");
                y.rot_dims = take_int(*rot, "dims", y.dim, wr.c_str());
                if (y.rot_dims <= 0 || y.rot_dims % 2 || y.rot_dims > y.dim)
                    fail(FG_E_CONFIG, wr + format(": dims must be even, positive and at most dim, got %lld", y.rot_dims));
                if (y.dim % 2) fail(FG_E_CONFIG, wm + format(": a rotated head needs an even dim, got %lld", y.dim));
                if (const Json *sc = object_or_absent(*rot, "scaling", wr)) {
                    std::string ws = wr + ".scaling";
                    y.scaled = true;
                    y.factor = take_float(*sc, "factor", ws.c_str());
                    y.original = take_float(*sc, "original", ws.c_str());
                    y.fast = take_float(*sc, "fast", ws.c_str());
                    y.slow = take_float(*sc, "slow", ws.c_str());
                    if (!(y.factor > 0.0) || !(y.original > 0.0) || !(y.fast > 0.0) || !(y.slow > 0.0)) fail(FG_E_CONFIG, ws + ": every number must be positive");
                }
            }
            if (const Json *mlp = object_or_absent(l, "mlp", w)) {
                std::string wf = w + ".mlp";
                std::string kind = take_string(*mlp, "kind", "moe", wf.c_str());
                if (kind != "moe") fail(FG_E_CONFIG, wf + ": kind '" + kind + "' is not known (known: moe)");
                y.has_mlp = true;
                const Json *ex = object_or_absent(*mlp, "expert", wf), *ro = object_or_absent(*mlp, "router", wf);
                if (!ex || !ro) fail(FG_E_CONFIG, wf + ": 'expert' and 'router' must be objects");
                y.ff = take_int(*ex, "ff", (wf + ".expert").c_str());
                std::string wr = wf + ".router";
                y.experts = take_int(*ro, "experts", wr.c_str());
                y.top = take_int(*ro, "top", wr.c_str());
                y.identity = take_int(*ro, "identity", 0, wr.c_str());
                y.route_scale = take_float(*ro, "scale", 1.0, wr.c_str());
                if (const Json *gr = object_or_absent(*ro, "groups", wr)) {
                    y.groups = take_int(*gr, "count", (wr + ".groups").c_str());
                    y.keep = take_int(*gr, "keep", y.groups, (wr + ".groups").c_str());
                }
                if (const Json *sh = object_or_absent(*mlp, "shared", wf)) y.shared_ff = take_int(*sh, "ff", (wf + ".shared").c_str());
                if (y.ff <= 0 || y.experts <= 0 || y.top <= 0 || y.identity < 0 || y.shared_ff < 0) fail(FG_E_CONFIG, wf + ": sizes must be positive");
                const long long outputs = y.experts + y.identity;
                if (y.groups <= 0 || outputs % y.groups) fail(FG_E_CONFIG, wr + format(": %lld router outputs do not form %lld equal groups", outputs, y.groups));
                if (y.keep <= 0 || y.keep > y.groups) fail(FG_E_CONFIG, wr + format(".groups: keep (%lld) must lie in 1 .. count (%lld)", y.keep, y.groups));
                if (y.top > y.keep * (outputs / y.groups))
                    fail(FG_E_CONFIG, wr + format(": top (%lld) exceeds the %lld outputs of the groups that stay", y.top, y.keep * (outputs / y.groups)));
            }
            c.layers.push_back(std::move(y));
        }
        if (const Json *loop = object_or_absent(d, "loop", "config.json")) {
            c.loops = true;
            c.loop_start = take_int(*loop, "start", "config.json loop");
            c.loop_stop = take_int(*loop, "stop", "config.json loop");
            c.loop_times = take_int(*loop, "times", "config.json loop");
            if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > (long long)c.layers.size() || c.loop_times < 1)
                fail(FG_E_CONFIG, format("config.json loop: need 0 <= start < stop <= %zu and times >= 1", c.layers.size()));
        }
        return cfg;
    }

    long long layer_parameters(const Layer &y) const {
        long long n = width * (y.heads * y.dim + y.kv_heads * (y.dim + y.vdim) + y.heads * y.vdim + y.heads) + y.heads * y.dim +
                      y.kv_heads * (y.dim + y.vdim) + 2 * width + 2 * y.dim;
        if (y.has_mlp) n += width + (y.experts + y.identity) * (width + 1) + 3 * width * (y.experts * y.ff + y.shared_ff);
        if (side_dim > 0) n += 2 * width * side_dim + width;
        return n;
    }
    // parameters a token's step reads: the chosen experts only
    long long active_parameters() const {
        long long n = 2 * vocab * width + width;
        for (auto &run : order()) {
            const Layer &y = layers[(size_t)run.first];
            n += layer_parameters(y);
            if (y.has_mlp) n -= 3 * width * y.ff * (y.experts - std::min(y.top, y.experts));
        }
        return n;
    }
    long long parameter_count() const {
        long long n = 2 * vocab * width + width + (loops ? 2 * width * width : 0) + vocab * side_dim * (long long)layers.size();
        for (auto &y : layers) n += layer_parameters(y);
        return n;
    }
    // the layers in the order they run; true where the loop's input map stands in front
    std::vector<std::pair<long long, bool>> order() const {
        std::vector<std::pair<long long, bool>> o;
        const long long n = (long long)layers.size();
        if (!loops) {
            for (long long i = 0; i < n; i++) o.emplace_back(i, false);
            return o;
        }
        for (long long i = 0; i < loop_start; i++) o.emplace_back(i, false);
        for (long long t = 0; t < loop_times; t++)
            for (long long i = loop_start; i < loop_stop; i++) o.emplace_back(i, i == loop_start);
        for (long long i = loop_stop; i < n; i++) o.emplace_back(i, false);
        return o;
    }

    const std::string &architecture() const override { return kPirozenName; }
    Json to_json() const override { return source; }

    Json describe() const override {
        Json d = Json::object();
        d.set("vocab_size", vocab);
        d.set("hidden_size", width);
        d.set("num_hidden_layers", (long long)layers.size());
        d.set("layer_runs", (long long)order().size());
        d.set("norm_eps", eps);
        long long kv_numbers = 0;
        Json kinds = Json::array();
        for (auto &y : layers) kinds.push(std::string("attention+") + (y.has_mlp ? "moe" : "none"));
        for (auto &run : order()) {
            const Layer &y = layers[(size_t)run.first];
            kv_numbers += y.kv_heads * (y.dim + y.vdim);
        }
        d.set("layer_kinds", kinds);
        d.set("parameters", parameter_count());
        d.set("active_parameters", active_parameters());
        Json kvb = Json::object(), pb = Json::object();
        kvb.set("bfloat16", kv_numbers * 2);
        kvb.set("float32", kv_numbers * 4);
        pb.set("bfloat16", parameter_count() * 2);
        pb.set("float32", parameter_count() * 4);
        d.set("kv_bytes_per_token", kvb);
        d.set("parameter_bytes", pb);
        d.set("state_bytes_per_sequence", 0LL);
        d.set("eos_token_ids", Json::array());
        d.set("defaulted", Json::array());
        return d;
    }

    Json spec() const override;
};

static Json part(const char *kind, Json params, Json tensors = Json::object()) {
    Json p = Json::object();
    p.set("kind", kind);
    p.set("params", std::move(params));
    p.set("tensors", std::move(tensors));
    return p;
}

Json PirozenConfig::spec() const {
    auto norm = [&](const std::string &name) {
        Json p = Json::object();
        p.set("size", width);
        p.set("eps", eps);
        Json t = Json::object();
        t.set("weight", name);
        return part("rmsnorm", p, t);
    };
    Json ls = Json::array(), schedule = Json::array();
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        const std::string pre = format("l%zu.", i), mx = pre + "mix.";
        Json layer = Json::object();
        layer.set("block", "parallel");
        Json mp = Json::object(), mt = Json::object();
        mp.set("hidden_size", width);
        mp.set("n_heads", y.heads);
        mp.set("n_kv_heads", y.kv_heads);
        mp.set("head_dim", y.dim);
        mp.set("v_head_dim", y.vdim);
        mp.set("eps", eps);
        mp.set("scale", y.scale);
        mp.set("window", y.window);
        mp.set("bias", true);
        mp.set("o_bias", true);
        mp.set("qk_norm", "head");
        mp.set("gate", "head");
        if (y.rotates) {
            Json rp = Json::object();
            rp.set("head_dim", y.dim);
            rp.set("theta", y.rot_base);
            rp.set("rotary_dim", y.rot_dims);
            rp.set("layout", "halves");
            if (y.scaled) {
                Json sc = Json::object();
                sc.set("rope_type", "yarn");
                sc.set("factor", y.factor);
                sc.set("original_max_position_embeddings", y.original);
                sc.set("beta_fast", y.fast);
                sc.set("beta_slow", y.slow);
                rp.set("scaling", sc);
            } else rp.set("scaling", Json());
            mp.set("position", part("rope", rp));
        } else mp.set("position", Json());
        for (const char *n : {"q", "k", "v", "o"}) {
            mt.set(std::string(n) + "_proj.weight", mx + n);
            mt.set(std::string(n) + "_proj.bias", mx + n + ".b");
        }
        mt.set("q_norm.weight", mx + "q.norm");
        mt.set("k_norm.weight", mx + "k.norm");
        mt.set("g_proj.weight", mx + "g");
        layer.set("mixer", part("sink_attention", mp, mt));
        layer.set("mixer_norm", norm(pre + "norm1"));
        if (y.has_mlp) {
            const std::string fx = pre + "mlp.";
            Json fp = Json::object(), ft = Json::object();
            fp.set("hidden_size", width);
            fp.set("d_ff", y.ff);
            fp.set("n_experts", y.experts);
            fp.set("top_k", y.top);
            fp.set("router", "softmax_grouped");
            fp.set("n_identity", y.identity);
            fp.set("n_groups", y.groups);
            fp.set("keep_groups", y.keep);
            fp.set("route_scale", y.route_scale);
            fp.set("shared_d_ff", y.shared_ff);
            ft.set("router.weight", fx + "router");
            ft.set("router.bias", fx + "correction");
            for (long long e = 0; e < y.experts; e++)
                for (const char *n : {"gate", "up", "down"}) ft.set(format("experts.%lld.%s_proj.weight", e, n), fx + format("e%lld.%s", e, n));
            if (y.shared_ff > 0)
                for (const char *n : {"gate", "up", "down"}) ft.set(std::string("shared.") + n + "_proj.weight", fx + "shared." + n);
            layer.set("feed_forward", part("moe", fp, ft));
            layer.set("feed_forward_norm", norm(pre + "norm2"));
        } else layer.set("feed_forward", Json());
        if (side_dim > 0) {
            Json sp = Json::object(), st = Json::object();
            sp.set("hidden_size", width);
            sp.set("vocab_size", vocab);
            sp.set("dim", side_dim);
            sp.set("column", side_dim * (long long)i);
            sp.set("table_dim", side_dim * (long long)layers.size());
            sp.set("eps", eps);
            st.set("table", "side.embed");
            st.set("gate", pre + "side.gate");
            st.set("proj", pre + "side.proj");
            st.set("norm", pre + "side.norm");
            layer.set("token_input", part("gated_token_embedding", sp, st));
        }
        ls.push(layer);
    }
    for (auto &run : order()) {
        Json r = Json::object();
        r.set("layer", run.first);
        r.set("cache_from", Json());
        if (run.second) r.set("reenter", true);
        schedule.push(r);
    }
    Json ep = Json::object(), hp = Json::object(), et = Json::object(), ht = Json::object();
    ep.set("vocab_size", vocab);
    ep.set("hidden_size", width);
    hp.set("vocab_size", vocab);
    hp.set("hidden_size", width);
    et.set("weight", "embed");
    ht.set("weight", "head");
    Json s = Json::object();
    s.set("hidden_size", width);
    s.set("vocab_size", vocab);
    s.set("max_positions", 1LL << 20);          // the design has no longest sequence; tables are built for what the cache holds
    s.set("embedding", part("embedding", ep, et));
    s.set("layers", ls);
    s.set("schedule", schedule);
    if (loops) {
        Json rp = Json::object(), rt = Json::object();
        rp.set("hidden_size", width);
        rt.set("weight", "loop.in");
        s.set("reentry", part("concat_linear", rp, rt));
    }
    s.set("final_norm", norm("final.norm"));
    s.set("head", part("lm_head", hp, ht));
    s.set("stop_token_ids", Json::array());
    s.set("ignored_tensors", Json::array());
    return s;
}

std::unique_ptr<ModelConfig> pirozen_config_from_json(const Json &d) { return PirozenConfig::from_json(d); }

}  // namespace fg
