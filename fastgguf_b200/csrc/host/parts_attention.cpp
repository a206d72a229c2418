// Attention mixers beyond the plain grouped-query one of parts.cpp.  Both keep their keys and values in the engine's paged
// cache, take their sizes and constants as parameters, and run the any-size attention kernel with its extensions (capped
// scores, a sink in the softmax, keys that are a latent plus a rotated part); scores, softmax, norms and angles are 32-bit.
//
// "sink_attention": grouped-query attention with everything optional that sits between the projections and the scores -
//     q = W_q h (+ b_q), k, v alike                                   biases
//     a short causal convolution over time on every channel of q, k and v (weights [channels, taps]); the last taps - 1
//       inputs of a sequence are fixed-size state, carried in the engine's state pool
//     q <- q / sqrt(mean(q^2) + eps) * w over ALL of q's rows at once, k alike          ("qk_norm": "whole")
//     rotation of the first rotary_dim numbers of each head, members (2i, 2i + 1) of a pair (position: a "rope" part)
//     score = scale * (q . k), then softcap * tanh(score / softcap)
//     a row sees itself and the window - 1 keys before it
//     the softmax's denominator also holds exp(sink_h), a learned number per head
//     ("chunk": c instead of a window: a row sees the keys of its own run of c positions, runs counted from the sequence's
//     first position, up to itself; "unit_sink": true instead of learned sinks: a sink of score 0, so that the softmax's
//     denominator is one plus the sum)
//   and, as further options: the q/k norm per head with one weight vector [head_dim] for all heads of q and one for all heads
//   of k ("qk_norm": "head"); rotated pairs (i, i + rotary_dim / 2) when the position part's layout is "halves"; a gate per
//   head on the heads' outputs, o_h <- o_h * sigmoid(W_g h)_h with W_g [heads, hidden] ("gate": "head"), or a gate per number,
//   o <- o * sigmoid(W_g h) with W_g [heads * v_head_dim, hidden] ("gate": "full"); a bias on the output
//   projection ("o_bias": true), stored as one more column of the output matrix that meets a column of ones, so the
//   projection's own pass adds it.
//
// "latent_attention": keys and values are linear maps of ONE small latent per token, c = norm(W_dkv h)[0:kv_rank], plus a
// rotated key part of rot_dim numbers that all heads share; queries pass through a latent of their own,
// q = W_uq norm(W_dq h), each head [head_dim unrotated | rot_dim rotated].  score = scale * (q_plain . (W_uk c) + q_rot . k_rot),
// causal, a sink per head, the heads' outputs times sigmoid(W_g h), then W_o.  The cache holds c (in the value pool) and the
// rotated part (in the key pool) only.  The key map is folded into the query, q_abs[h] = W_uk[h]^T q_plain[h], so that a score
// is q_abs . c + q_rot . k_rot, and the value map is applied to the attention's output over the latents,
// o[h] = W_uv[h] (sum_j p_j c_j): the same sums in another order, for prompts, portions and single tokens alike.
// "shared_kv": true: the layer has no W_dkv; its schedule entry reads the latents and rotated key parts that an earlier latent
// attention layer of the same kv_rank, rot_dim and rotation keeps (the entry's cache_from), with W_uk, W_uv, queries and
// everything else of its own.
#include <algorithm>
#include <cmath>

#include "parts.hpp"

namespace fg {

static bool flag(const Json &p, const char *key) { return p.get(key).is_bool() && p.get(key).as_bool(); }

static Weight as_f32(const Weight &w, cudaStream_t s) { return w.t.dtype == FG_F32 ? w : concat_rows({w}, FG_F32, s); }

class SinkAttention : public Mixer {
public:
    SinkAttention(const Json &p, BuildContext &ctx) {
        const char *me = "sink_attention";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        KV_ = (int)param_int(p, "n_kv_heads", H_, me);
        hd_ = (int)param_int(p, "head_dim", me);
        hdv_ = (int)param_int(p, "v_head_dim", hd_, me);
        if (E_ <= 0 || H_ <= 0 || KV_ <= 0 || hd_ <= 0 || hdv_ <= 0) fail(FG_E_CONFIG, "sink_attention: sizes must be positive");
        if (H_ % KV_) fail(FG_E_CONFIG, format("sink_attention: %d heads are not a multiple of %d KV heads", H_, KV_));
        scale_ = (float)param_float(p, "scale", 1.0 / std::sqrt((double)hd_), me);
        window_ = (int)param_int(p, "window", 0, me);
        chunk_ = (int)param_int(p, "chunk", 0, me);
        softcap_ = (float)param_float(p, "softcap", 0.0, me);
        taps_ = (int)param_int(p, "conv_taps", 0, me);
        eps_ = (float)param_float(p, "eps", 1e-6, me);
        bias_ = flag(p, "bias");
        sink_ = flag(p, "sink");
        unit_sink_ = flag(p, "unit_sink");
        if (sink_ && unit_sink_) fail(FG_E_CONFIG, "sink_attention: learned sinks and a unit sink exclude one another");
        if (chunk_ < 0 || (chunk_ > 0 && window_ > 0)) fail(FG_E_CONFIG, "sink_attention: 'chunk' cannot be negative or stand beside a window");
        const Json &qn = p.get("qk_norm");
        if (!qn.is_null() && !(qn.is_string() && (qn.as_string() == "whole" || qn.as_string() == "head")))
            fail(FG_E_CONFIG, "sink_attention: qk_norm " + qn.dump() + " is not known (known: whole, head)");
        qk_norm_ = !qn.is_null();
        norm_per_head_ = qk_norm_ && qn.as_string() == "head";
        const Json &gt = p.get("gate");
        if (!gt.is_null() && !(gt.is_string() && (gt.as_string() == "head" || gt.as_string() == "full")))
            fail(FG_E_CONFIG, "sink_attention: gate " + gt.dump() + " is not known (known: head, full)");
        gate_ = !gt.is_null();
        gate_full_ = gate_ && gt.as_string() == "full";
        o_bias_ = flag(p, "o_bias");
        // columns behind the heads' outputs that carry the output bias: as many as keep a row a multiple of 8 numbers
        pad_ = o_bias_ ? 8 - (int)(((int64_t)H_ * hdv_) % 8) : 0;
        if (window_ < 0 || softcap_ < 0.f || taps_ < 0) fail(FG_E_CONFIG, "sink_attention: window, softcap and conv_taps cannot be negative");
        if (hdv_ > 512) fail(FG_E_CONFIG, format("sink_attention: v_head_dim %d exceeds 512, the largest the kernel takes", hdv_));
        if (((size_t)H_ * hd_ + (size_t)KV_ * (hd_ + hdv_)) * 4 > 200 * 1024) fail(FG_E_CONFIG, "sink_attention: a token's q, k and v exceed what the kernel holds in shared memory");
        const Json &pos = p.get("position");
        if (!pos.is_null()) {
            position_ = dynamic_cast<PositionEncoding *>(ctx.nested(FG_ROLE_POSITION, pos));
            if (!position_) fail(FG_E_CONFIG, "sink_attention: 'position' is not a position encoding");
            if (position_->head_dim() != hd_)
                fail(FG_E_CONFIG, format("sink_attention: the position encoding is built for head_dim %d, the mixer has %d", position_->head_dim(), hd_));
            rot_dims_ = (int)param_int(pos.get("params"), "rotary_dim", hd_, me);
            const Json &layout = pos.get("params").get("layout");
            rot_halves_ = !(layout.is_string() && layout.as_string() == "adjacent");
        }
    }
    std::vector<TensorDecl> tensor_decls() const override {
        const int64_t Q = (int64_t)H_ * hd_, K = (int64_t)KV_ * hd_, V = (int64_t)KV_ * hdv_;
        std::vector<TensorDecl> d = {{"q_proj.weight", {Q, E_}}, {"k_proj.weight", {K, E_}}, {"v_proj.weight", {V, E_}},
                                     {"o_proj.weight", {E_, (int64_t)H_ * hdv_}}};
        if (bias_) for (auto &n : std::vector<std::pair<const char *, int64_t>>{{"q_proj.bias", Q}, {"k_proj.bias", K}, {"v_proj.bias", V}}) d.push_back({n.first, {n.second}});
        if (taps_ > 0)
            for (auto &n : std::vector<std::pair<const char *, int64_t>>{{"q_conv.weight", Q}, {"k_conv.weight", K}, {"v_conv.weight", V}})
                d.push_back({n.first, {n.second, (int64_t)taps_}, false, 0, 0.5f});
        if (qk_norm_) {
            d.push_back({"q_norm.weight", {norm_per_head_ ? (int64_t)hd_ : Q}, false, 1, 0.01f});
            d.push_back({"k_norm.weight", {norm_per_head_ ? (int64_t)hd_ : K}, false, 1, 0.01f});
        }
        if (sink_) d.push_back({"sinks", {(int64_t)H_}, false, 0, 1.0f});
        if (gate_) d.push_back({"g_proj.weight", {gate_full_ ? (int64_t)H_ * hdv_ : (int64_t)H_, E_}});
        if (o_bias_) d.push_back({"o_proj.bias", {(int64_t)E_}});
        return d;
    }
    bool cache_request(CacheRequest *out) const override {
        // (a chunked mask keeps every page: a sequence's pages are given back when it ends)
        out->n_kv_heads = KV_; out->head_dim = hd_; out->window = window_; out->v_head_dim = hdv_; out->keep_first = 0;
        return true;
    }
    int64_t channels() const { return (int64_t)H_ * hd_ + (int64_t)KV_ * (hd_ + hdv_); }
    int64_t state_bytes() const override { return taps_ > 1 ? (int64_t)(taps_ - 1) * channels() * (int64_t)sizeof(float) : 0; }
    bool supports_deferred_norm() const override { return true; }
    bool can_overwrite() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        const Weight &q = tensor_of(tensors, "q_proj.weight"), &k = tensor_of(tensors, "k_proj.weight"), &v = tensor_of(tensors, "v_proj.weight");
        int dt = (q.t.dtype == k.t.dtype && k.t.dtype == v.t.dtype) ? q.t.dtype : FG_F32;
        std::vector<Weight> rows = {q, k, v};
        if (gate_) {
            rows.push_back(tensor_of(tensors, "g_proj.weight"));        // the gate's rows ride in the same contraction
            if (rows.back().t.dtype != dt) dt = FG_F32;
        }
        qkv_ = Linear(concat_rows(rows, dt, rt.stream));
        if (o_bias_) {
            // [W_o | b | 0 ...]: the bias as a column that meets the ones fg_head_gate writes behind the heads' outputs
            const Weight &w = tensor_of(tensors, "o_proj.weight"), &b = tensor_of(tensors, "o_proj.bias");
            const int odt = w.t.dtype == b.t.dtype ? w.t.dtype : FG_F32;
            const Weight wc = w.t.dtype == odt ? w : concat_rows({w}, odt, rt.stream), bc = b.t.dtype == odt ? b : concat_rows({b}, odt, rt.stream);
            const int64_t K0 = (int64_t)H_ * hdv_, K1 = K0 + pad_;
            const size_t es = (size_t)elem_size(odt);
            Weight wide = make_weight(E_, K1, odt, "output projection with its bias column");
            FG_CUDA(cudaMemsetAsync(wide.t.data, 0, (size_t)E_ * K1 * es, rt.stream));
            FG_CUDA(cudaMemcpy2DAsync(wide.t.data, (size_t)K1 * es, wc.t.data, (size_t)wc.t.ld * es, (size_t)K0 * es, (size_t)E_, cudaMemcpyDeviceToDevice, rt.stream));
            FG_CUDA(cudaMemcpy2DAsync((char *)wide.t.data + (size_t)K0 * es, (size_t)K1 * es, bc.t.data, es, es, (size_t)E_, cudaMemcpyDeviceToDevice, rt.stream));
            FG_CUDA(cudaStreamSynchronize(rt.stream));
            o_ = Linear(wide);
        } else {
            o_ = Linear(tensor_of(tensors, "o_proj.weight"));
        }
        auto three = [&](const char *a, const char *b, const char *c, int64_t cols) {
            Weight x = tensor_of(tensors, a), y = tensor_of(tensors, b), z = tensor_of(tensors, c);
            // row-major [channels, cols]: the three lie one after another
            Weight out = make_weight(x.t.numel() / cols + y.t.numel() / cols + z.t.numel() / cols, cols, FG_F32, "per-channel parameters of attention");
            size_t at = 0;
            for (const Weight *w : {&x, &y, &z}) {
                dev_convert(w->t.data, w->t.dtype, (char *)out.t.data + at * 4, FG_F32, w->t.numel(), rt.stream);
                at += (size_t)w->t.numel();
            }
            return out;
        };
        if (bias_) bias_w_ = three("q_proj.bias", "k_proj.bias", "v_proj.bias", 1);
        if (taps_ > 0) conv_w_ = three("q_conv.weight", "k_conv.weight", "v_conv.weight", taps_);
        if (qk_norm_) { qn_w_ = as_f32(tensor_of(tensors, "q_norm.weight"), rt.stream); kn_w_ = as_f32(tensor_of(tensors, "k_norm.weight"), rt.stream); }
        if (sink_) sinks_w_ = as_f32(tensor_of(tensors, "sinks"), rt.stream);
        if (unit_sink_) {
            sinks_w_ = make_weight(1, H_, FG_F32, "unit sinks");
            FG_CUDA(cudaMemsetAsync(sinks_w_.t.data, 0, (size_t)H_ * sizeof(float), rt.stream));
            FG_CUDA(cudaStreamSynchronize(rt.stream));
        }
    }
    void prepare(Runtime &rt, int max_positions) override { if (position_) position_->prepare(rt, max_positions); }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *emit_norm) override {
        if (io.group < 0 || !io.k_pool || !io.write_cache) fail(FG_E_INTERNAL, "sink_attention: the schedule entry has no cache of its own");
        if (taps_ > 1 && (!io.state || io.state_bytes < state_bytes())) fail(FG_E_INTERNAL, "sink_attention: the schedule entry has no state rows");
        const int *table = b.block_tables.at((size_t)io.group);
        // the projections feed a convolution, a norm and a rotation: they stay float32 until those are done
        Tensor proj = qkv_.forward(rt, xn, deferred, Tensor(), FG_F32, false, nullptr, nullptr);
        const int M = (int)proj.rows;
        Tensor q = rt.arena->matrix(M, (int64_t)H_ * hd_, rt.dtype);
        const float *bias = bias_ ? bias_w_.t.ptr<float>() : nullptr;
        FG_LAUNCH("mix", fg_qkv_prepare_ext, proj.ptr<float>(), (int)proj.ld, bias, taps_ > 0 ? conv_w_.t.ptr<float>() : nullptr, taps_,
                  (const float *)io.state, qk_norm_ ? qn_w_.t.ptr<float>() : nullptr, qk_norm_ ? kn_w_.t.ptr<float>() : nullptr, eps_,
                  position_ ? position_->cos_table() : nullptr, position_ ? position_->sin_table() : nullptr, hd_ / 2, position_ ? rot_dims_ : 0,
                  b.positions, b.row_seq, b.cu_rows, b.slots, table, b.table_width, q.data, (int)q.ld, io.k_pool, io.v_pool, rt.dtype, M, H_, KV_,
                  hd_, hdv_, io.page_size, norm_per_head_ ? 1 : 0, rot_halves_ ? 1 : 0, rt.stream);
        if (taps_ > 1)
            FG_LAUNCH("mix", fg_conv_state_update, proj.ptr<float>(), (int)proj.ld, bias, taps_, (float *)io.state, b.cu_rows, b.slots, b.n_seq,
                      (int)channels(), rt.stream);
        // (with an output bias the rows are wider than the heads' outputs: the columns behind them carry the ones)
        Tensor attn = rt.arena->matrix(M, (int64_t)H_ * hdv_ + pad_, rt.dtype);
        const float *sinks = (sink_ || unit_sink_) ? sinks_w_.t.ptr<float>() : nullptr;
        const int mask = chunk_ > 0 ? -chunk_ : window_;     // what the kernels call a window: negative for a chunked mask
        // bfloat16 with head size 64 / 128 for keys and values alike: the tensor-core kernels (a decode step: mma.sync with the
        // pages split over a cluster; portions: tcgen05 tiles of 128 rows, or mma.sync tiles of 64 for a few rows)
        const bool fast = !rt.plain_kernels && rt.dtype == FG_BF16 && io.cache_dtype == FG_BF16 && (hd_ == 64 || hd_ == 128) && hdv_ == hd_ &&
                          io.page_size == 64 && q.ld % 8 == 0 && ((uintptr_t)q.data % 16) == 0;
        if (fast && b.single_token) {
            int n_splits = decode_splits(rt.n_sm, b.n_seq, H_, KV_, b.table_width, hd_);
            float *part_o = nullptr, *part_ml = nullptr;
            if (n_splits != 1 && n_splits != 2 && n_splits != 4 && n_splits != 8) {
                part_o = (float *)rt.arena->alloc((size_t)b.n_seq * H_ * n_splits * hd_ * sizeof(float));
                part_ml = (float *)rt.arena->alloc((size_t)b.n_seq * H_ * n_splits * 2 * sizeof(float));
            }
            FG_LAUNCH("attn", fg_attention_decode_ext, q.data, (int)q.ld, attn.data, (int)attn.ld, b.positions, table, b.table_width, io.k_pool,
                      io.v_pool, b.n_seq, H_, KV_, hd_, io.page_size, scale_, mask, 0, n_splits, part_o, part_ml, softcap_, sinks, rt.stream);
        } else if (fast && b.max_new * (H_ / KV_) >= 64) {
            FG_LAUNCH("attn", fg_attention_prefill_tc_ext, q.data, (int)q.ld, attn.data, (int)attn.ld, b.cu_rows, b.seq_start, table, b.table_width,
                      io.k_pool, io.v_pool, io.n_pages, b.n_seq, b.max_new, H_, KV_, hd_, io.page_size, scale_, mask, 0, softcap_, sinks, rt.stream);
        } else if (fast) {
            FG_LAUNCH("attn", fg_attention_prefill_ext, q.data, (int)q.ld, attn.data, (int)attn.ld, b.cu_rows, b.seq_start, table, b.table_width,
                      io.k_pool, io.v_pool, b.n_seq, b.max_new, H_, KV_, hd_, io.page_size, scale_, mask, 0, softcap_, sinks, rt.stream);
        } else {
            FG_LAUNCH("core", fg_attention_generic_ext, q.data, (int)q.ld, attn.data, (int)attn.ld, rt.dtype, b.positions, b.row_seq, table,
                      b.table_width, io.k_pool, io.v_pool, M, H_, KV_, hd_, hdv_, io.page_size, scale_, mask, 0, softcap_, sinks, 0, rt.stream);
        }
        if (gate_full_)           // in place: a thread reads and writes its own number
            FG_LAUNCH("mix", fg_gate_slice, attn.data, (int)attn.ld, hdv_, proj.ptr<float>() + channels(), (int)proj.ld, attn.data, (int)attn.ld, attn.dtype, M,
                      H_, hdv_, rt.stream);
        if ((gate_ && !gate_full_) || pad_ > 0)
            FG_LAUNCH("mix", fg_head_gate, attn.data, (int)attn.ld, attn.dtype, (gate_ && !gate_full_) ? proj.ptr<float>() + channels() : nullptr, (int)proj.ld,
                      M, H_, hdv_, pad_, rt.stream);
        DeferredNorm started;
        o_.forward(rt, attn, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_ = 0, H_ = 0, KV_ = 0, hd_ = 0, hdv_ = 0, window_ = 0, chunk_ = 0, taps_ = 0, rot_dims_ = 0, pad_ = 0;
    float scale_ = 1.f, softcap_ = 0.f, eps_ = 1e-6f;
    bool bias_ = false, sink_ = false, unit_sink_ = false, qk_norm_ = false, norm_per_head_ = false, rot_halves_ = false, gate_ = false, gate_full_ = false,
         o_bias_ = false;
    PositionEncoding *position_ = nullptr;
    Linear qkv_, o_;
    Weight bias_w_, conv_w_, qn_w_, kn_w_, sinks_w_;
};

class LatentAttention : public Mixer {
public:
    LatentAttention(const Json &p, BuildContext &ctx) {
        const char *me = "latent_attention";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        d_ = (int)param_int(p, "head_dim", me);
        dr_ = (int)param_int(p, "rot_dim", me);
        dv_ = (int)param_int(p, "v_head_dim", d_, me);
        r_ = (int)param_int(p, "kv_rank", me);
        qr_ = (int)param_int(p, "q_rank", me);
        if (E_ <= 0 || H_ <= 0 || d_ <= 0 || dr_ <= 0 || dv_ <= 0 || r_ <= 0 || qr_ <= 0) fail(FG_E_CONFIG, "latent_attention: sizes must be positive");
        if (dr_ % 2) fail(FG_E_CONFIG, format("latent_attention: rot_dim must be even, got %d", dr_));
        if (r_ > 512) fail(FG_E_CONFIG, format("latent_attention: kv_rank %d exceeds 512, the largest the kernel takes", r_));
        scale_ = (float)param_float(p, "scale", 1.0 / std::sqrt((double)(d_ + dr_)), me);
        eps_ = (float)param_float(p, "eps", 1e-6, me);
        sink_ = flag(p, "sink");
        gate_ = flag(p, "gate");
        shared_kv_ = flag(p, "shared_kv");
        const Json &pos = p.get("position");
        position_ = pos.is_null() ? nullptr : dynamic_cast<PositionEncoding *>(ctx.nested(FG_ROLE_POSITION, pos));
        if (!position_) fail(FG_E_CONFIG, "latent_attention: 'position' must be a position encoding for the rotated part");
        if (position_->head_dim() != dr_)
            fail(FG_E_CONFIG, format("latent_attention: the position encoding is built for head_dim %d, the rotated part has %d", position_->head_dim(), dr_));
    }
    std::vector<TensorDecl> tensor_decls() const override {
        const int64_t HV = (int64_t)H_ * dv_;
        std::vector<TensorDecl> d = {{"q_down.weight", {qr_, E_}}, {"q_down_norm.weight", {qr_}, false, 1, 0.01f}, {"q_up.weight", {(int64_t)H_ * (d_ + dr_), qr_}},
                                     {"k_up.weight", {(int64_t)H_ * d_, r_}}, {"v_up.weight", {HV, r_}}, {"o_proj.weight", {E_, HV}}};
        if (!shared_kv_) {
            d.push_back({"kv_down.weight", {(int64_t)r_ + dr_, E_}});
            d.push_back({"kv_down_norm.weight", {r_}, false, 1, 0.01f});
        }
        if (gate_) d.push_back({"g_proj.weight", {HV, E_}});
        if (sink_) d.push_back({"sinks", {(int64_t)H_}, false, 0, 1.0f});
        return d;
    }
    bool cache_request(CacheRequest *out) const override {
        // one "head" a position: the rotated key part in the key pool, the latent in the value pool
        out->n_kv_heads = 1; out->head_dim = dr_; out->window = 0; out->v_head_dim = r_; out->keep_first = 0;
        return true;
    }
    bool supports_deferred_norm() const override { return true; }
    bool can_overwrite() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        const Weight &dq = tensor_of(tensors, "q_down.weight");
        std::vector<Weight> parts = {dq};
        bool same = true;
        if (!shared_kv_) { parts.push_back(tensor_of(tensors, "kv_down.weight")); same = parts.back().t.dtype == dq.t.dtype; }
        if (gate_) { parts.push_back(tensor_of(tensors, "g_proj.weight")); same = same && parts.back().t.dtype == dq.t.dtype; }
        down_ = Linear(concat_rows(parts, same ? dq.t.dtype : FG_F32, rt.stream));
        q_up_ = Linear(tensor_of(tensors, "q_up.weight"));
        k_up_ = tensor_of(tensors, "k_up.weight");
        v_up_ = tensor_of(tensors, "v_up.weight");
        k_lin_ = Linear(k_up_);
        v_lin_ = Linear(v_up_);
        o_ = Linear(tensor_of(tensors, "o_proj.weight"));
        qn_w_ = as_f32(tensor_of(tensors, "q_down_norm.weight"), rt.stream);
        if (!shared_kv_) kvn_w_ = as_f32(tensor_of(tensors, "kv_down_norm.weight"), rt.stream);
        if (sink_) sinks_w_ = as_f32(tensor_of(tensors, "sinks"), rt.stream);
    }
    void prepare(Runtime &rt, int max_positions) override { position_->prepare(rt, max_positions); }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *emit_norm) override {
        if (io.group < 0 || !io.k_pool || (!shared_kv_ && !io.write_cache)) fail(FG_E_INTERNAL, "latent_attention: the schedule entry has no cache of its own");
        if (shared_kv_ && io.write_cache) fail(FG_E_CONFIG, "latent_attention: a layer without a key/value latent of its own must read an earlier entry's cache");
        const int *table = b.block_tables.at((size_t)io.group);
        const float *cos_t = position_->cos_table(), *sin_t = position_->sin_table();
        // [q latent | kv latent and rotated key part | gate], float32: norms and the rotation read them
        Tensor down = down_.forward(rt, xn, deferred, Tensor(), FG_F32, false, nullptr, nullptr);
        const int M = (int)down.rows;
        Tensor cq = rt.arena->matrix(M, qr_, rt.dtype);
        FG_LAUNCH("mix", fg_rmsnorm_strided, down.ptr<float>(), (int)down.ld, qn_w_.t.ptr<float>(), cq.data, cq.dtype, (int)cq.ld, M, qr_, eps_, rt.stream);
        Tensor q = q_up_.forward(rt, cq, nullptr, Tensor(), FG_F32, false, nullptr, nullptr);
        if (!shared_kv_)
            FG_LAUNCH("mix", fg_latent_append, down.ptr<float>() + qr_, (int)down.ld, kvn_w_.t.ptr<float>(), eps_, cos_t, sin_t, dr_ / 2, b.positions,
                      b.row_seq, table, b.table_width, io.k_pool, io.v_pool, rt.dtype, M, r_, dr_, io.page_size, rt.stream);
        Tensor o = rt.arena->matrix(M, (int64_t)H_ * dv_, rt.dtype);
        const float *gate = gate_ ? down.ptr<float>() + qr_ + (shared_kv_ ? 0 : r_ + dr_) : nullptr;
        const float *sinks = sink_ ? sinks_w_.t.ptr<float>() : nullptr;
        const int HQ = d_ + dr_;
        // A step of whole prompts in bfloat16 whose head sizes the tensor-core kernels take: ordinary multi-head attention over
        // keys and values expanded for the step's tokens (nothing older is in the cache), in pools of the step's own.
        bool whole_prompts = !b.single_token && !b.host_seq_start.empty() && !rt.plain_kernels && rt.dtype == FG_BF16 && (HQ == 64 || HQ == 128) &&
                             dv_ <= HQ && io.page_size == 64 && b.n_seq <= 1024 && k_up_.t.dtype == FG_BF16 && v_up_.t.dtype == FG_BF16;
        for (size_t s = 0; whole_prompts && s < b.host_seq_start.size(); s++) whole_prompts = b.host_seq_start[s] == 0;
        if (whole_prompts) {
            const int P = io.page_size;
            int n_pages = 0, width = 1;
            for (int s = 0; s < b.n_seq; s++) {
                const int n = (b.host_cu_rows[(size_t)s + 1] - b.host_cu_rows[(size_t)s] + P - 1) / P;
                n_pages += n;
                width = std::max(width, n);
            }
            Tensor cn = rt.arena->matrix(M, r_, FG_BF16);
            Tensor kr;                               // shared latents: the owner's rotated key parts of the step's rows, out of its cache
            if (shared_kv_) {
                kr = rt.arena->matrix(M, dr_, FG_F32);
                FG_LAUNCH("mix", fg_latent_fetch, io.k_pool, io.v_pool, io.cache_dtype, b.positions, b.row_seq, table, b.table_width, P, cn.data, (int)cn.ld,
                          kr.ptr<float>(), (int)kr.ld, M, r_, dr_, rt.stream);
            } else
                FG_LAUNCH("mix", fg_rmsnorm_strided, down.ptr<float>() + qr_, (int)down.ld, kvn_w_.t.ptr<float>(), cn.data, cn.dtype, (int)cn.ld, M, r_, eps_,
                          rt.stream);
            Tensor kp = k_lin_.forward(rt, cn, nullptr, Tensor(), FG_BF16, false, nullptr, nullptr);
            Tensor vp = v_lin_.forward(rt, cn, nullptr, Tensor(), FG_BF16, false, nullptr, nullptr);
            int *tmp_table = (int *)rt.arena->alloc((size_t)b.n_seq * width * sizeof(int));
            const size_t pool_elems = (size_t)n_pages * H_ * P * HQ;
            Tensor qx = rt.arena->matrix(M, (int64_t)H_ * HQ, FG_BF16), ox = rt.arena->matrix(M, (int64_t)H_ * HQ, FG_BF16);
            void *Kx = rt.arena->alloc(pool_elems * 2), *Vx = rt.arena->alloc(pool_elems * 2);
            // a sequence's last page is filled only as far as the sequence goes, and the attention kernel reads whole pages: what lies
            // behind must be numbers (a masked key has weight zero, but zero times whatever the arena held before need not be zero)
            FG_CUDA(cudaMemsetAsync(Kx, 0, pool_elems * 2, rt.stream));
            FG_CUDA(cudaMemsetAsync(Vx, 0, pool_elems * 2, rt.stream));
            FG_LAUNCH("mix", fg_seq_page_table, b.cu_rows, b.n_seq, width, P, tmp_table, rt.stream);
            FG_LAUNCH("mix", fg_latent_expand_ext, q.ptr<float>(), (int)q.ld, shared_kv_ ? kr.ptr<float>() : down.ptr<float>(),
                      shared_kv_ ? (int)kr.ld : (int)down.ld, shared_kv_ ? 0 : qr_ + r_, kp.data, (int)kp.ld, vp.data, (int)vp.ld, cos_t, sin_t, dr_ / 2,
                      b.positions, b.row_seq, tmp_table, width, qx.data, Kx, Vx, M, H_, d_, dr_, dv_, P, shared_kv_ ? 1 : 0, rt.stream);
            if (b.max_new >= 64)
                FG_LAUNCH("attn", fg_attention_prefill_tc_ext, qx.data, (int)qx.ld, ox.data, (int)ox.ld, b.cu_rows, b.seq_start, tmp_table, width, Kx, Vx,
                          n_pages, b.n_seq, b.max_new, H_, H_, HQ, P, scale_, 0, 0, 0.f, sinks, rt.stream);
            else
                FG_LAUNCH("attn", fg_attention_prefill_ext, qx.data, (int)qx.ld, ox.data, (int)ox.ld, b.cu_rows, b.seq_start, tmp_table, width, Kx, Vx,
                          b.n_seq, b.max_new, H_, H_, HQ, P, scale_, 0, 0, 0.f, sinks, rt.stream);
            FG_LAUNCH("mix", fg_gate_slice, ox.data, (int)ox.ld, HQ, gate, (int)down.ld, o.data, (int)o.ld, o.dtype, M, H_, dv_, rt.stream);
        } else {
            // per head [q_abs (kv_rank) | q_rot (rot_dim)]
            Tensor qf = rt.arena->matrix(M, (int64_t)H_ * (r_ + dr_), rt.dtype);
            FG_LAUNCH("mix", fg_head_gemm, q.data, q.dtype, (int)q.ld, d_ + dr_, k_up_.t.data, k_up_.t.dtype, (int)k_up_.t.ld, 1, qf.data, qf.dtype,
                      (int)qf.ld, r_ + dr_, nullptr, 0, M, r_, d_, H_, rt.stream);
            FG_LAUNCH("mix", fg_rope_pairs, q.ptr<float>(), (int)q.ld, d_ + dr_, d_, qf.data, qf.dtype, (int)qf.ld, r_ + dr_, r_, b.positions, cos_t, sin_t,
                      dr_ / 2, M, H_, dr_, rt.stream);
            Tensor lat = rt.arena->matrix(M, (int64_t)H_ * r_, rt.dtype);
            if (b.single_token && M <= 65535 && !rt.plain_kernels && rt.dtype == FG_BF16 && io.cache_dtype == FG_BF16 &&
                FG_KERNEL("mix", fg_latent_decode_mma_ok)(r_, dr_, io.page_size)) {
                // tensor cores: a block per (row, 16 heads, split of the pages), enough blocks to fill the GPU
                const int blocks = M * ((H_ + 15) / 16), pages = b.max_len / io.page_size + 1;
                int n_splits = std::max(1, std::min({(rt.n_sm + blocks - 1) / blocks, 32, pages}));
                const long long floats = FG_KERNEL("mix", fg_latent_decode_scratch_floats)(M, H_, r_, n_splits);
                float *part = floats > 0 ? (float *)rt.arena->alloc((size_t)floats * sizeof(float)) : nullptr;
                FG_LAUNCH("mix", fg_latent_decode_mma, qf.data, (int)qf.ld, lat.data, (int)lat.ld, b.positions, b.row_seq, table, b.table_width, io.k_pool,
                          io.v_pool, M, H_, r_, dr_, io.page_size, scale_, sinks, n_splits, part, rt.stream);
            } else if (b.single_token && dr_ <= 128 && dr_ % 4 == 0 && r_ % 4 == 0 && M <= 65535) {
                // a block per (row, 8 heads, split of the keys): enough blocks to fill the GPU, at least 8 keys a warp
                const int blocks = M * ((H_ + 7) / 8);
                int n_splits = std::max(1, std::min({(rt.n_sm + blocks - 1) / blocks, 16, (b.max_len + 63) / 64}));
                const long long floats = FG_KERNEL("mix", fg_latent_decode_scratch_floats)(M, H_, r_, n_splits);
                float *part = floats > 0 ? (float *)rt.arena->alloc((size_t)floats * sizeof(float)) : nullptr;
                FG_LAUNCH("mix", fg_latent_decode, qf.data, (int)qf.ld, lat.data, (int)lat.ld, rt.dtype, b.positions, b.row_seq, table, b.table_width,
                          io.k_pool, io.v_pool, M, H_, r_, dr_, io.page_size, scale_, sinks, n_splits, part, rt.stream);
            } else {
                FG_LAUNCH("core", fg_attention_generic_ext, qf.data, (int)qf.ld, lat.data, (int)lat.ld, rt.dtype, b.positions, b.row_seq, table, b.table_width,
                          io.k_pool, io.v_pool, M, H_, 1, dr_, r_, io.page_size, scale_, 0, 0, 0.f, sinks, 1, rt.stream);
            }
            FG_LAUNCH("mix", fg_head_gemm, lat.data, lat.dtype, (int)lat.ld, r_, v_up_.t.data, v_up_.t.dtype, (int)v_up_.t.ld, 0, o.data, o.dtype, (int)o.ld,
                      dv_, gate, (int)down.ld, M, dv_, r_, H_, rt.stream);
        }
        DeferredNorm started;
        o_.forward(rt, o, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_ = 0, H_ = 0, d_ = 0, dr_ = 0, dv_ = 0, r_ = 0, qr_ = 0;
    float scale_ = 1.f, eps_ = 1e-6f;
    bool sink_ = false, gate_ = false, shared_kv_ = false;
    PositionEncoding *position_ = nullptr;
    Linear down_, q_up_, o_, k_lin_, v_lin_;
    Weight k_up_, v_up_, qn_w_, kvn_w_, sinks_w_;
};

void add_attention_kinds(std::map<std::string, PartFactory> &mixers) {
    mixers["sink_attention"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<SinkAttention>(p, c); };
    mixers["latent_attention"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<LatentAttention>(p, c); };
}

}  // namespace fg
