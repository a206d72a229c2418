// The Saluzen decoder's config.json, and the model it describes as data.
//
// Keys: "architecture": "Saluzen"; "vocab", "width"; "norm": {"eps"}; "layers": a list, each
// {"type": "parallel" | "parallel_2" | "latent_attention", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}.
//   parallel mixer          {"left": attention, "right": {"heads", "vdim", "state", "groups", "conv": taps, "norm_groups"}}
//   parallel_2 mixer        {"left": attention, "right": {"heads", "kv_heads", "dim", "vdim", "conv": taps}, "left_scale", "right_scale"}
//   attention (a left side) {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims", "scaling": {"factor", "low", "high",
//                            "original"}}, "mask": {"size"}} - rot, rot.scaling and mask are each left out by a model that has none
//   latent_attention mixer  {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot": {"base", "dims"}, "kv_from": j}
//                           - with kv_from the layer has no key/value latent of its own and reads layer j's (rot may carry the
//                           same scaling as a left side's; the two layers' rotations must then agree in it too)
// Every size and constant above comes from the file.  What the design itself fixes is written here once: a layer is
// x += norm_b(f(norm_a(x))) around the mixer and around the feed-forward, norms multiply by their weight as stored; the dense
// feed-forward is SwiGLU; both left sides have biases on q, k, v and rotate the first rot.dims numbers of a head in halves
// (entry i with entry i + dims/2); "parallel" pairs causal attention whose softmax has a sink of score 0 and a sigmoid gate
// per number with the state-space mixer, normalises both outputs over the width and takes half their sum; "parallel_2" pairs
// attention over runs of mask.size positions with a learned sink and a sigmoid gate per head with the gated delta rule (unit
// vectors with 1e-6 under the root, q times dim^-0.5) and adds them with the file's two scales; latent attention rotates adjacent
// pairs, has neither sink nor gate; the head is a matrix of its own.
// Tensor names: embed, head, final.norm, l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.*, l<i>.mlp.gate / up / down.
#include <cmath>

#include "config.hpp"

namespace fg {

static const std::string kSaluzenName = "Saluzen";

static const Json *saluzen_object(const Json &d, const std::string &key, const std::string &where, bool required) {
    const Json *v = d.find(key);
    if (!v || v->is_null()) {
        if (required) fail(FG_E_CONFIG, where + ": '" + key + "' must be an object");
        return nullptr;
    }
    if (!v->is_object()) fail(FG_E_CONFIG, where + ": '" + key + "' must be an object");
    return v;
}

class SaluzenConfig : public ModelConfig {
public:
    struct Rot {
        bool on = false, scaled = false;
        double base = 0, factor = 1, low = 1, high = 1, original = 0;
        long long dims = 0;
    };
    struct Attention {                          // the left side of a pair
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0, chunk = 0;
        double scale = 0;
        Rot rot;
    };
    struct Layer {
        std::string type;                       // "parallel" | "parallel_2" | "latent_attention"
        Attention left;
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0, taps = 1;       // the right side
        long long state = 0, groups = 1, norm_groups = 1;                       // state space
        double left_scale = 1, right_scale = 1;                                 // parallel_2
        long long rot_dim = 0, kv_rank = 0, q_rank = 0, kv_from = -1;           // latent attention (heads, dim, vdim above)
        double scale = 0;
        Rot rot;
        long long ff = 0;                       // 0: no feed-forward
    };
    Json source;
    long long vocab = 0, width = 0;
    double eps = 0.0;
    std::vector<Layer> layers;

    static Rot read_rot(const Json &m, const std::string &wm, long long dim, bool required, bool allow_scaling) {
        Rot r;
        const Json *rot = saluzen_object(m, "rot", wm, required);
        if (!rot) return r;
        const std::string wr = wm + ".rot";
        r.on = true;
        r.base = take_float(*rot, "base", wr.c_str());
        r.dims = take_int(*rot, "dims", dim, wr.c_str());
        if (!(r.base > 1.0)) fail(FG_E_CONFIG, wr + ": base must exceed 1");
        if (r.dims <= 0 || r.dims % 2 || r.dims > dim) fail(FG_E_CONFIG, wr + format(": dims must be even, positive and at most %lld, got %lld", dim, r.dims));
        if (const Json *sc = saluzen_object(*rot, "scaling", wr, false)) {
            const std::string ws = wr + ".scaling";
            if (!allow_scaling) fail(FG_E_CONFIG, ws + ": this mixer's rotation has no scaling");
            r.scaled = true;
            r.factor = take_float(*sc, "factor", ws.c_str());
            r.low = take_float(*sc, "low", ws.c_str());
            r.high = take_float(*sc, "high", ws.c_str());
            r.original = take_float(*sc, "original", ws.c_str());
            if (!(r.factor > 0.0) || !(r.low > 0.0) || !(r.high > r.low) || !(r.original > 0.0))
                fail(FG_E_CONFIG, ws + ": factor, low and original must be positive and high must exceed low");
        }
        return r;
    }

    static Attention read_attention(const Json &m, const std::string &wm) {
        Attention a;
        a.heads = take_int(m, "heads", wm.c_str());
        a.kv_heads = take_int(m, "kv_heads", a.heads, wm.c_str());
        a.dim = take_int(m, "dim", wm.c_str());
        a.vdim = take_int(m, "vdim", a.dim, wm.c_str());
        if (a.heads <= 0 || a.kv_heads <= 0 || a.dim <= 0 || a.vdim <= 0) fail(FG_E_CONFIG, wm + ": heads, kv_heads, dim and vdim must be positive");
        if (a.heads % a.kv_heads) fail(FG_E_CONFIG, wm + format(": heads (%lld) must be a multiple of kv_heads (%lld)", a.heads, a.kv_heads));
        a.scale = take_float(m, "scale", 1.0 / std::sqrt((double)a.dim), wm.c_str());
        a.rot = read_rot(m, wm, a.dim, false, true);
        if (a.rot.on && a.dim % 2) fail(FG_E_CONFIG, wm + format(": a rotated head needs an even dim, got %lld", a.dim));
        if (const Json *mask = saluzen_object(m, "mask", wm, false)) {
            a.chunk = take_int(*mask, "size", (wm + ".mask").c_str());
            if (a.chunk <= 0) fail(FG_E_CONFIG, wm + ".mask: size must be positive");
        }
        return a;
    }

    static std::unique_ptr<ModelConfig> from_json(const Json &d) {
        auto cfg = std::make_unique<SaluzenConfig>();
        SaluzenConfig &c = *cfg;
        c.source = d;
        c.vocab = take_int(d, "vocab");
        c.width = take_int(d, "width");
        const Json *norm = saluzen_object(d, "norm", "config.json", true);
        c.eps = take_float(*norm, "eps", "config.json norm");
        if (c.vocab <= 0 || c.width <= 0) fail(FG_E_CONFIG, "config.json: vocab and width must be positive");
        if (!(c.eps > 0.0)) fail(FG_E_CONFIG, format("config.json: norm.eps must be positive, got %g", c.eps));
        const Json *ls = d.find("layers");
        if (!ls || !ls->is_array() || ls->size() == 0) fail(FG_E_CONFIG, "config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < ls->size(); i++) {
            const Json &l = (*ls)[i];
            const std::string w = format("config.json layers[%zu]", i);
            if (!l.is_object()) fail(FG_E_CONFIG, w + " must be an object");
            Layer y;
            y.type = take_string(l, "type", "", w.c_str());
            const Json &m = *saluzen_object(l, "mixer", w, true);
            const std::string wm = w + ".mixer";
            if (y.type == "parallel" || y.type == "parallel_2") {
                y.left = read_attention(*saluzen_object(m, "left", wm, true), wm + ".left");
                const Json &r = *saluzen_object(m, "right", wm, true);
                const std::string wr = wm + ".right";
                y.heads = take_int(r, "heads", wr.c_str());
                y.vdim = take_int(r, "vdim", wr.c_str());
                y.taps = take_int(r, "conv", 1, wr.c_str());
                if (y.heads <= 0 || y.vdim <= 0 || y.taps <= 0) fail(FG_E_CONFIG, wr + ": heads, vdim and conv must be positive");
                if (y.type == "parallel") {
                    y.state = take_int(r, "state", wr.c_str());
                    y.groups = take_int(r, "groups", 1, wr.c_str());
                    y.norm_groups = take_int(r, "norm_groups", 1, wr.c_str());
                    if (y.state <= 0 || y.groups <= 0 || y.norm_groups <= 0) fail(FG_E_CONFIG, wr + ": state, groups and norm_groups must be positive");
                    if (y.heads % y.groups) fail(FG_E_CONFIG, wr + format(": heads (%lld) must be a multiple of groups (%lld)", y.heads, y.groups));
                    if ((y.heads * y.vdim) % y.norm_groups)
                        fail(FG_E_CONFIG, wr + format(": heads * vdim (%lld) must be a multiple of norm_groups (%lld)", y.heads * y.vdim, y.norm_groups));
                } else {
                    y.kv_heads = take_int(r, "kv_heads", y.heads, wr.c_str());
                    y.dim = take_int(r, "dim", wr.c_str());
                    if (y.kv_heads <= 0 || y.dim <= 0) fail(FG_E_CONFIG, wr + ": kv_heads and dim must be positive");
                    if (y.heads % y.kv_heads) fail(FG_E_CONFIG, wr + format(": heads (%lld) must be a multiple of kv_heads (%lld)", y.heads, y.kv_heads));
                    y.left_scale = take_float(m, "left_scale", 1.0, wm.c_str());
                    y.right_scale = take_float(m, "right_scale", 1.0, wm.c_str());
                }
            } else if (y.type == "latent_attention") {
                y.heads = take_int(m, "heads", wm.c_str());
                y.dim = take_int(m, "dim", wm.c_str());
                y.vdim = take_int(m, "vdim", y.dim, wm.c_str());
                y.rot_dim = take_int(m, "rot_dim", wm.c_str());
                y.kv_rank = take_int(m, "kv_rank", wm.c_str());
                y.q_rank = take_int(m, "q_rank", wm.c_str());
                if (y.heads <= 0 || y.dim <= 0 || y.vdim <= 0) fail(FG_E_CONFIG, wm + ": heads, dim and vdim must be positive");
                if (y.rot_dim <= 0 || y.rot_dim % 2 || y.kv_rank <= 0 || y.q_rank <= 0)
                    fail(FG_E_CONFIG, wm + ": rot_dim (even), kv_rank and q_rank must be positive");
                y.scale = take_float(m, "scale", 1.0 / std::sqrt((double)(y.dim + y.rot_dim)), wm.c_str());
                y.rot = read_rot(m, wm, y.rot_dim, true, true);
                if (y.rot.dims != y.rot_dim) fail(FG_E_CONFIG, wm + format(".rot: dims (%lld) must equal rot_dim (%lld)", y.rot.dims, y.rot_dim));
                const Json *from = m.find("kv_from");
                if (from && !from->is_null()) {
                    y.kv_from = take_int(m, "kv_from", wm.c_str());
                    if (y.kv_from < 0 || y.kv_from >= (long long)i) fail(FG_E_CONFIG, wm + format(": kv_from must name an earlier layer, got %lld", y.kv_from));
                    const Layer &o = c.layers[(size_t)y.kv_from];
                    if (o.type != "latent_attention" || o.kv_from >= 0)
                        fail(FG_E_CONFIG, wm + format(": kv_from names layer %lld, which keeps no latent of its own", y.kv_from));
                    if (o.kv_rank != y.kv_rank || o.rot_dim != y.rot_dim || o.rot.base != y.rot.base || o.rot.scaled != y.rot.scaled ||
                        (y.rot.scaled && (o.rot.factor != y.rot.factor || o.rot.low != y.rot.low || o.rot.high != y.rot.high || o.rot.original != y.rot.original)))
                        fail(FG_E_CONFIG, wm + format(": kv_rank, rot_dim and rot of layer %lld must equal this layer's", y.kv_from));
                }
            } else {
                fail(FG_E_CONFIG, w + ": type '" + y.type + "' is not known (known: parallel, parallel_2, latent_attention)");
            }
            if (const Json *mlp = saluzen_object(l, "mlp", w, false)) {
                const std::string wf = w + ".mlp";
                const std::string kind = take_string(*mlp, "kind", "dense", wf.c_str());
                if (kind != "dense") fail(FG_E_CONFIG, wf + ": kind '" + kind + "' is not known (known: dense)");
                y.ff = take_int(*mlp, "ff", wf.c_str());
                if (y.ff <= 0) fail(FG_E_CONFIG, wf + ": ff must be positive");
            }
            c.layers.push_back(std::move(y));
        }
        return cfg;
    }

    static long long attention_parameters(const Attention &a, long long width, bool gate_per_head) {
        const long long q = a.heads * a.dim, k = a.kv_heads * a.dim, v = a.kv_heads * a.vdim, o = a.heads * a.vdim;
        return width * (q + k + v + o + (gate_per_head ? a.heads : o)) + q + k + v + (gate_per_head ? a.heads : 0);
    }
    long long layer_parameters(const Layer &y) const {
        long long n = 2 * width + (y.ff ? 2 * width + 3 * width * y.ff : 0);
        if (y.type == "parallel") {
            const long long inner = y.heads * y.vdim, ch = inner + 2 * y.groups * y.state;
            n += attention_parameters(y.left, width, false) + width * (2 * inner + 2 * y.groups * y.state + y.heads) + ch * (y.taps + 1) + 3 * y.heads + inner +
                 width * inner + 2 * width;
        } else if (y.type == "parallel_2") {
            const long long q = y.kv_heads * y.dim, v = y.heads * y.vdim;
            n += attention_parameters(y.left, width, true) + width * (2 * q + 3 * v + 2 * y.heads) + (2 * q + v) * y.taps + 2 * y.heads + y.vdim;
        } else {
            n += width * y.q_rank + y.q_rank + y.q_rank * y.heads * (y.dim + y.rot_dim) + y.kv_rank * y.heads * (y.dim + y.vdim) + width * y.heads * y.vdim;
            if (y.kv_from < 0) n += width * (y.kv_rank + y.rot_dim) + y.kv_rank;
        }
        return n;
    }
    long long parameter_count() const {
        long long n = 2 * vocab * width + width;
        for (auto &y : layers) n += layer_parameters(y);
        return n;
    }

    const std::string &architecture() const override { return kSaluzenName; }
    Json to_json() const override { return source; }

    Json describe() const override {
        Json d = Json::object();
        d.set("vocab_size", vocab);
        d.set("hidden_size", width);
        d.set("num_hidden_layers", (long long)layers.size());
        d.set("layer_runs", (long long)layers.size());
        d.set("norm_eps", eps);
        long long kv_numbers = 0, state_floats = 0;
        Json kinds = Json::array();
        for (auto &y : layers) {
            kinds.push(y.type + "+" + (y.ff ? "dense" : "none"));
            if (y.type == "latent_attention") kv_numbers += y.kv_from < 0 ? y.kv_rank + y.rot_dim : 0;
            else {
                kv_numbers += y.left.kv_heads * (y.left.dim + y.left.vdim);
                if (y.type == "parallel") state_floats += (y.taps - 1) * (y.heads * y.vdim + 2 * y.groups * y.state) + y.heads * y.state * y.vdim;
                else state_floats += (y.taps - 1) * (2 * y.kv_heads * y.dim + y.heads * y.vdim) + y.heads * y.dim * y.vdim;
            }
        }
        d.set("layer_kinds", kinds);
        d.set("parameters", parameter_count());
        Json kvb = Json::object(), pb = Json::object();
        kvb.set("bfloat16", kv_numbers * 2);
        kvb.set("float32", kv_numbers * 4);
        pb.set("bfloat16", parameter_count() * 2);
        pb.set("float32", parameter_count() * 4);
        d.set("kv_bytes_per_token", kvb);
        d.set("parameter_bytes", pb);
        d.set("state_bytes_per_sequence", state_floats * 4);
        d.set("eos_token_ids", Json::array());
        d.set("defaulted", Json::array());
        return d;
    }

    Json spec() const override;
};

static Json saluzen_part(const char *kind, Json params, Json tensors = Json::object()) {
    Json p = Json::object();
    p.set("kind", kind);
    p.set("params", std::move(params));
    p.set("tensors", std::move(tensors));
    return p;
}

static Json saluzen_rope(long long head_dim, const SaluzenConfig::Rot &r, const char *layout) {
    Json rp = Json::object();
    rp.set("head_dim", head_dim);
    rp.set("theta", r.base);
    rp.set("rotary_dim", r.dims);
    rp.set("layout", layout);
    if (r.scaled) {
        Json sc = Json::object();
        sc.set("rope_type", "llama3");
        sc.set("factor", r.factor);
        sc.set("low_freq_factor", r.low);
        sc.set("high_freq_factor", r.high);
        sc.set("original_max_position_embeddings", r.original);
        rp.set("scaling", sc);
    } else rp.set("scaling", Json());
    return saluzen_part("rope", rp);
}

Json SaluzenConfig::spec() const {
    auto norm = [&](const std::string &name) {
        Json p = Json::object();
        p.set("size", width);
        p.set("eps", eps);
        Json t = Json::object();
        t.set("weight", name);
        return saluzen_part("rmsnorm", p, t);
    };
    // the left side of a pair: {"kind", "params"} and its tensors under `pre` (local names get the pair's "left." in front)
    auto left_side = [&](const Attention &a, const std::string &pre, bool learned_sink, const char *gate, Json &tensors) {
        Json mp = Json::object();
        mp.set("hidden_size", width);
        mp.set("n_heads", a.heads);
        mp.set("n_kv_heads", a.kv_heads);
        mp.set("head_dim", a.dim);
        mp.set("v_head_dim", a.vdim);
        mp.set("scale", a.scale);
        mp.set("eps", eps);
        mp.set("chunk", a.chunk);
        mp.set("bias", true);
        if (learned_sink) mp.set("sink", true);
        else mp.set("unit_sink", true);
        mp.set("gate", gate);
        mp.set("position", a.rot.on ? saluzen_rope(a.dim, a.rot, "halves") : Json());
        for (const char *n : {"q", "k", "v"}) {
            tensors.set(std::string("left.") + n + "_proj.weight", pre + n);
            tensors.set(std::string("left.") + n + "_proj.bias", pre + n + ".b");
        }
        if (learned_sink) tensors.set("left.sinks", pre + "sink");
        tensors.set("left.g_proj.weight", pre + "g");
        tensors.set("left.o_proj.weight", pre + "o");
        Json side = Json::object();
        side.set("kind", "sink_attention");
        side.set("params", mp);
        return side;
    };
    Json ls = Json::array(), schedule = Json::array();
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        const std::string pre = format("l%zu.", i), mx = pre + "mix.";
        Json layer = Json::object();
        layer.set("block", "sandwich");
        if (y.type == "latent_attention") {
            Json mp = Json::object(), mt = Json::object();
            mp.set("hidden_size", width);
            mp.set("n_heads", y.heads);
            mp.set("head_dim", y.dim);
            mp.set("v_head_dim", y.vdim);
            mp.set("eps", eps);
            mp.set("rot_dim", y.rot_dim);
            mp.set("kv_rank", y.kv_rank);
            mp.set("q_rank", y.q_rank);
            mp.set("scale", y.scale);
            mp.set("sink", false);
            mp.set("gate", false);
            mp.set("shared_kv", y.kv_from >= 0);
            mp.set("position", saluzen_rope(y.rot_dim, y.rot, "adjacent"));
            mt.set("q_down.weight", mx + "dq");
            mt.set("q_down_norm.weight", mx + "dq.norm");
            mt.set("q_up.weight", mx + "uq");
            if (y.kv_from < 0) {
                mt.set("kv_down.weight", mx + "dkv");
                mt.set("kv_down_norm.weight", mx + "dkv.norm");
            }
            mt.set("k_up.weight", mx + "uk");
            mt.set("v_up.weight", mx + "uv");
            mt.set("o_proj.weight", mx + "o");
            layer.set("mixer", saluzen_part("latent_attention", mp, mt));
        } else {
            Json pp = Json::object(), pt = Json::object(), right = Json::object(), rp = Json::object();
            pp.set("hidden_size", width);
            pp.set("eps", eps);
            rp.set("hidden_size", width);
            rp.set("n_heads", y.heads);
            rp.set("v_head_dim", y.vdim);
            rp.set("conv_taps", y.taps);
            rp.set("eps", eps);
            const std::string rx = mx + "right.";
            if (y.type == "parallel") {
                pp.set("left", left_side(y.left, mx + "left.", false, "full", pt));
                rp.set("state_size", y.state);
                rp.set("n_groups", y.groups);
                rp.set("norm_groups", y.norm_groups);
                right.set("kind", "state_space");
                pt.set("right.in_proj.weight", rx + "in");
                pt.set("right.conv.weight", rx + "conv");
                pt.set("right.conv.bias", rx + "conv.b");
                for (const char *n : {"dt_bias", "A_log", "D"}) pt.set(std::string("right.") + n, rx + n);
                pt.set("right.norm.weight", rx + "norm");
                pt.set("right.o_proj.weight", rx + "o");
                pp.set("normalize", true);
                pp.set("left_scale", 0.5);
                pp.set("right_scale", 0.5);
                pt.set("left_norm.weight", mx + "left.out");
                pt.set("right_norm.weight", mx + "right.out");
            } else {
                pp.set("left", left_side(y.left, mx + "left.", true, "head", pt));
                rp.set("n_kv_heads", y.kv_heads);
                rp.set("head_dim", y.dim);
                rp.set("unit_eps", 1e-6);
                rp.set("q_scale", 1.0 / std::sqrt((double)y.dim));
                right.set("kind", "gated_delta");
                for (const char *n : {"q", "k", "v"}) {
                    pt.set(std::string("right.") + n + "_proj.weight", rx + n);
                    pt.set(std::string("right.") + n + "_conv.weight", rx + n + ".conv");
                }
                pt.set("right.b_proj.weight", rx + "b");
                pt.set("right.a_proj.weight", rx + "a");
                pt.set("right.g_proj.weight", rx + "g");
                pt.set("right.o_proj.weight", rx + "o");
                pt.set("right.A_log", rx + "A_log");
                pt.set("right.dt_bias", rx + "dt_bias");
                pt.set("right.norm.weight", rx + "norm");
                pp.set("normalize", false);
                pp.set("left_scale", y.left_scale);
                pp.set("right_scale", y.right_scale);
            }
            right.set("params", rp);
            pp.set("right", right);
            layer.set("mixer", saluzen_part("mixer_pair", pp, pt));
        }
        layer.set("mixer_norm", norm(pre + "norm1"));
        layer.set("mixer_post_norm", norm(pre + "norm1b"));
        if (y.ff > 0) {
            Json fp = Json::object(), ft = Json::object();
            fp.set("hidden_size", width);
            fp.set("d_ff", y.ff);
            for (const char *n : {"gate", "up", "down"}) ft.set(std::string(n) + "_proj.weight", pre + "mlp." + n);
            layer.set("feed_forward", saluzen_part("swiglu", fp, ft));
            layer.set("feed_forward_norm", norm(pre + "norm2"));
            layer.set("feed_forward_post_norm", norm(pre + "norm2b"));
        } else layer.set("feed_forward", Json());
        ls.push(layer);
        Json r = Json::object();
        r.set("layer", (long long)i);
        r.set("cache_from", y.kv_from >= 0 ? Json(y.kv_from) : Json());
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
    s.set("embedding", saluzen_part("embedding", ep, et));
    s.set("layers", ls);
    s.set("schedule", schedule);
    s.set("final_norm", norm("final.norm"));
    s.set("head", saluzen_part("lm_head", hp, ht));
    s.set("stop_token_ids", Json::array());
    s.set("ignored_tensors", Json::array());
    return s;
}

std::unique_ptr<ModelConfig> saluzen_config_from_json(const Json &d) { return SaluzenConfig::from_json(d); }

}  // namespace fg
