// Mixers that carry a state of fixed size from token to token instead of keys and values per position: retention, gated
// linear attention, and - behind a short convolution, with one decay per head and token - the state-space form and the gated
// delta rule.
//
// "retention": linear attention with a fixed decay per head and neither softmax nor denominator.  With the layer's
// normalised input h, per head (q, k of size head_dim, v of size v_head_dim):
//     q = W_q h, k = W_k h, v = W_v h, g = W_g h       no biases; the four projections are ONE contraction
//     q, k rotated by the position encoding (if any); k times k_scale afterwards
//     S_t = decay_head S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
//     y = concat_heads(o / sqrt(mean(o^2) + eps)) * silu(g),  output W_o y
// The state S [heads, head_dim, v_head_dim] is float32 whatever the engine's dtype, one row of the engine's state pool
// per sequence slot (zeroed when a sequence takes the slot), and so are the projections' results that enter the
// recurrence: the contraction writes float32 and the kernels of retention.cu keep rotation, decay powers, scores, the
// unit norm and the gate in float32; y takes the engine's dtype for the output projection.
// A decode step and short portions walk their tokens one after another with S in shared memory; portions of
// `chunk_threshold` tokens and more run in chunks over all sequences at once (retention.cu says how).
#include <cmath>

#include "parts.hpp"

namespace fg {

class RetentionMixer : public Mixer {
public:
    RetentionMixer(const Json &p, BuildContext &ctx) {
        const char *me = "retention";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        dk_ = (int)param_int(p, "head_dim", me);
        dv_ = (int)param_int(p, "v_head_dim", dk_, me);
        eps_ = (float)param_float(p, "eps", me);
        k_scale_ = (float)param_float(p, "k_scale", 1.0 / std::sqrt((double)dk_), me);
        if (E_ <= 0 || H_ <= 0 || dk_ <= 0 || dv_ <= 0) fail(FG_E_CONFIG, "retention: sizes must be positive");
        if (dk_ % 2) fail(FG_E_CONFIG, format("retention: head_dim must be even, got %d", dk_));
        if (dv_ > 256) fail(FG_E_CONFIG, format("retention: v_head_dim %d exceeds 256, the largest the kernels take", dv_));
        if ((size_t)dk_ * dv_ > 40 * 1024) fail(FG_E_CONFIG, "retention: a head's state exceeds what the kernels hold in shared memory");
        if (!(eps_ > 0.f)) fail(FG_E_CONFIG, "retention: eps must be positive");
        const Json &d = p.get("decay");
        if (!d.is_array() || (int)d.size() != H_) fail(FG_E_CONFIG, format("retention: 'decay' must list one number for each of the %d heads", H_));
        for (auto &v : d.items()) {
            if (!v.is_number() || v.is_bool() || !(v.as_double() >= 0.0) || !(v.as_double() <= 1.0))
                fail(FG_E_CONFIG, "retention: a decay must be a number in [0, 1], got " + v.dump());
            decay_.push_back((float)v.as_double());
            all_positive_ = all_positive_ && v.as_double() > 0.0;
        }
        const Json &pos = p.get("position");
        if (!pos.is_null()) {
            position_ = dynamic_cast<PositionEncoding *>(ctx.nested(FG_ROLE_POSITION, pos));
            if (!position_) fail(FG_E_CONFIG, "retention: 'position' is not a position encoding");
            if (position_->head_dim() != dk_)
                fail(FG_E_CONFIG, format("retention: the position encoding is built for head_dim %d, the mixer has %d", position_->head_dim(), dk_));
        }
    }
    std::vector<TensorDecl> tensor_decls() const override {
        int64_t Q = (int64_t)H_ * dk_, V = (int64_t)H_ * dv_;
        return {{"q_proj.weight", {Q, E_}}, {"k_proj.weight", {Q, E_}}, {"v_proj.weight", {V, E_}}, {"g_proj.weight", {V, E_}},
                {"o_proj.weight", {E_, V}}};
    }
    bool can_overwrite() const override { return true; }
    int64_t state_bytes() const override { return (int64_t)H_ * dk_ * dv_ * (int64_t)sizeof(float); }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        Weight q = tensor_of(tensors, "q_proj.weight"), k = tensor_of(tensors, "k_proj.weight");
        const Weight &v = tensor_of(tensors, "v_proj.weight"), &g = tensor_of(tensors, "g_proj.weight");
        if (position_ && !position_->permutation().empty()) {
            // the kernels rotate pairs (j, j + head_dim / 2); q . k does not change under a common permutation of both
            const std::vector<int> &perm = position_->permutation();
            std::vector<int64_t> rows;
            for (int h = 0; h < H_; h++)
                for (int i = 0; i < dk_; i++) rows.push_back((int64_t)h * dk_ + perm[(size_t)i]);
            q = gather_rows(q, rows, rt.stream);
            k = gather_rows(k, rows, rt.stream);
        }
        bool same = q.t.dtype == k.t.dtype && k.t.dtype == v.t.dtype && v.t.dtype == g.t.dtype;
        proj_ = Linear(concat_rows({q, k, v, g}, same ? q.t.dtype : FG_F32, rt.stream));
        o_ = Linear(tensor_of(tensors, "o_proj.weight"));
        decay_dev_ = make_weight(1, H_, FG_F32, "retention decays");
        FG_CUDA(cudaMemcpyAsync(decay_dev_.t.data, decay_.data(), decay_.size() * sizeof(float), cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaStreamSynchronize(rt.stream));
    }
    void prepare(Runtime &rt, int max_positions) override {
        if (position_) { position_->prepare(rt, max_positions); return; }
        // no rotation: identity tables, so that one kernel serves both
        if (ident_cos_.buffer && ident_positions_ >= max_positions) return;
        int half = dk_ / 2;
        std::vector<float> c((size_t)max_positions * half, 1.0f);
        ident_cos_ = make_weight(max_positions, half, FG_F32, "identity rotation tables");
        ident_sin_ = make_weight(max_positions, half, FG_F32, "identity rotation tables");
        FG_CUDA(cudaMemcpyAsync(ident_cos_.t.data, c.data(), c.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaMemsetAsync(ident_sin_.t.data, 0, c.size() * 4, rt.stream));
        FG_CUDA(cudaStreamSynchronize(rt.stream));
        ident_positions_ = max_positions;
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *emit_norm) override {
        if (!io.state || io.state_bytes < state_bytes()) fail(FG_E_INTERNAL, "retention: the schedule entry has no state rows");
        const float *cos_t = position_ ? position_->cos_table() : ident_cos_.t.ptr<float>();
        const float *sin_t = position_ ? position_->sin_table() : ident_sin_.t.ptr<float>();
        // what enters the recurrence stays float32: the contraction accumulates in float32 and writes it as it is
        Tensor proj = proj_.forward(rt, xn, nullptr, Tensor(), FG_F32, false, nullptr, nullptr);
        const int M = (int)proj.rows;
        Tensor y = rt.arena->matrix(M, (int64_t)H_ * dv_, rt.dtype);
        const int *host_cu = b.host_cu_rows.empty() ? nullptr : b.host_cu_rows.data();
        const int RC = FG_KERNEL("mix", fg_retention_chunk_tokens)();
        bool chunked = host_cu && !b.single_token && all_positive_ && b.max_new >= chunk_threshold_ &&
                       FG_KERNEL("mix", fg_retention_chunked_ok)(dk_, dv_);
        if (chunked) {
            // the host knows only how many chunks the step has; the kernels plan them from the step's row offsets
            int n_chunks = 0;
            for (int s = 0; s < b.n_seq; s++) n_chunks += (host_cu[s + 1] - host_cu[s] + RC - 1) / RC;
            int *plan = (int *)rt.arena->alloc(((size_t)2 * n_chunks + b.n_seq + 1) * sizeof(int));
            float *U = (float *)rt.arena->alloc((size_t)n_chunks * H_ * dk_ * dv_ * sizeof(float));
            FG_LAUNCH("mix", fg_retention_chunked, proj.ptr<float>(), (int)proj.ld, y.data, y.dtype, (int)y.ld, b.positions, b.cu_rows,
                      b.slots, cos_t, sin_t, decay_dev_.t.ptr<float>(), (float *)io.state, plan, U, b.n_seq, n_chunks, H_, dk_, dv_,
                      k_scale_, eps_, rt.stream);
        } else {
            FG_LAUNCH("mix", fg_retention, proj.ptr<float>(), (int)proj.ld, y.data, y.dtype, (int)y.ld, b.positions, b.cu_rows, b.slots, cos_t,
                      sin_t, decay_dev_.t.ptr<float>(), (float *)io.state, b.n_seq, H_, dk_, dv_, k_scale_, eps_, rt.stream);
        }
        DeferredNorm started;
        o_.forward(rt, y, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_ = 0, H_ = 0, dk_ = 0, dv_ = 0, chunk_threshold_ = 16, ident_positions_ = 0;
    float eps_ = 0.f, k_scale_ = 1.f;
    bool all_positive_ = true;
    std::vector<float> decay_;
    PositionEncoding *position_ = nullptr;
    Linear proj_, o_;
    Weight decay_dev_, ident_cos_, ident_sin_;
};

// "gated_linear_attention": linear attention whose state decays per key channel by a factor the token itself decides.
// With the layer's normalised input h, per head (q, k of size head_dim, v of size v_head_dim):
//     q = W_q h * q_scale, k = W_k h, v = W_v h, g = W_g h       no biases
//     a = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau)                 a decay per key channel, through a low-rank pair
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
//     y = concat_heads(o / sqrt(mean(o^2) + eps) * w_norm) * silu(g),  output W_o y
// decay_rank (the inner size of the low-rank pair) may be left to the checkpoint's tensor shapes.  q, k, v, g and the
// low-rank input are ONE contraction with float32 output; the decay logits, their log-sigmoid, the state, the unit norm and
// the gate stay float32 in every engine dtype (gla.cu), y takes the engine's dtype for the output projection.
class GatedLinearAttention : public Mixer {
public:
    GatedLinearAttention(const Json &p, BuildContext &) {
        const char *me = "gated_linear_attention";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        dk_ = (int)param_int(p, "head_dim", me);
        dv_ = (int)param_int(p, "v_head_dim", dk_, me);
        rank_ = (int)param_int(p, "decay_rank", -1, me);
        eps_ = (float)param_float(p, "eps", me);
        tau_ = (float)param_float(p, "tau", 1.0, me);
        q_scale_ = (float)param_float(p, "q_scale", 1.0 / std::sqrt((double)dk_), me);
        if (E_ <= 0 || H_ <= 0 || dk_ <= 0 || dv_ <= 0 || rank_ == 0 || rank_ < -1) fail(FG_E_CONFIG, "gated_linear_attention: sizes must be positive");
        if (dv_ > 256) fail(FG_E_CONFIG, format("gated_linear_attention: v_head_dim %d exceeds 256, the largest the kernels take", dv_));
        if ((size_t)dk_ * dv_ > 40 * 1024) fail(FG_E_CONFIG, "gated_linear_attention: a head's state exceeds what the kernels hold in shared memory");
        if (!(eps_ > 0.f) || !(tau_ > 0.f)) fail(FG_E_CONFIG, "gated_linear_attention: eps and tau must be positive");
    }
    std::vector<TensorDecl> tensor_decls() const override {
        int64_t Q = (int64_t)H_ * dk_, V = (int64_t)H_ * dv_, R = rank_;
        return {{"q_proj.weight", {Q, E_}}, {"k_proj.weight", {Q, E_}}, {"v_proj.weight", {V, E_}}, {"g_proj.weight", {V, E_}},
                {"o_proj.weight", {E_, V}}, {"decay_down.weight", {R, E_}}, {"decay_up.weight", {Q, R}}, {"decay_up.bias", {Q}, false, 0, 1.0f},
                {"norm.weight", {dv_}, false, 1, 0.01f}};
    }
    bool can_overwrite() const override { return true; }
    bool supports_deferred_norm() const override { return true; }
    int64_t state_bytes() const override { return (int64_t)H_ * dk_ * dv_ * (int64_t)sizeof(float); }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        const Weight &q = tensor_of(tensors, "q_proj.weight"), &k = tensor_of(tensors, "k_proj.weight");
        const Weight &v = tensor_of(tensors, "v_proj.weight"), &g = tensor_of(tensors, "g_proj.weight");
        const Weight &a1 = tensor_of(tensors, "decay_down.weight"), &a2 = tensor_of(tensors, "decay_up.weight");
        if (a1.t.rows != a2.t.cols)
            fail(FG_E_WEIGHTS, format("gated_linear_attention: the decay's low-rank pair disagrees on its inner size (%lld against %lld)",
                                      (long long)a1.t.rows, (long long)a2.t.cols));
        rank_ = (int)a1.t.rows;
        bool same = q.t.dtype == k.t.dtype && k.t.dtype == v.t.dtype && v.t.dtype == g.t.dtype && g.t.dtype == a1.t.dtype;
        proj_ = Linear(concat_rows({q, k, v, g, a1}, same ? q.t.dtype : FG_F32, rt.stream));
        up_ = Linear(a2);
        o_ = Linear(tensor_of(tensors, "o_proj.weight"));
        bias_ = concat_rows({tensor_of(tensors, "decay_up.bias")}, FG_F32, rt.stream);
        norm_ = concat_rows({tensor_of(tensors, "norm.weight")}, FG_F32, rt.stream);
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *emit_norm) override {
        if (!io.state || io.state_bytes < state_bytes()) fail(FG_E_INTERNAL, "gated_linear_attention: the schedule entry has no state rows");
        // what enters the recurrence stays float32: the contraction accumulates in float32 and writes it as it is
        Tensor proj = proj_.forward(rt, xn, deferred, Tensor(), FG_F32, false, nullptr, nullptr);
        const int M = (int)proj.rows;
        const int64_t low_at = (int64_t)2 * H_ * dk_ + (int64_t)2 * H_ * dv_;
        Tensor low = proj;
        low.data = proj.ptr<float>() + low_at;
        low.cols = rank_;
        Tensor z = up_.forward(rt, low, nullptr, Tensor(), FG_F32, false, nullptr, nullptr);
        Tensor y = rt.arena->matrix(M, (int64_t)H_ * dv_, rt.dtype);
        const int *host_cu = b.host_cu_rows.empty() ? nullptr : b.host_cu_rows.data();
        const int GC = FG_KERNEL("mix", fg_gla_chunk_tokens)();
        bool chunked = host_cu && !b.single_token && b.max_new >= chunk_threshold_ && FG_KERNEL("mix", fg_gla_chunked_ok)(dk_, dv_);
        if (chunked) {
            int n_chunks = 0;
            for (int s = 0; s < b.n_seq; s++) n_chunks += (host_cu[s + 1] - host_cu[s] + GC - 1) / GC;
            int *plan = (int *)rt.arena->alloc(((size_t)2 * n_chunks + b.n_seq + 1) * sizeof(int));
            float *U = (float *)rt.arena->alloc((size_t)n_chunks * H_ * dk_ * dv_ * sizeof(float));
            float *D = (float *)rt.arena->alloc((size_t)n_chunks * H_ * dk_ * (1 + GC) * sizeof(float));     // decays and cumulative log decays
            FG_LAUNCH("mix", fg_gla_chunked, proj.ptr<float>(), (int)proj.ld, z.ptr<float>(), (int)z.ld, bias_.t.ptr<float>(), norm_.t.ptr<float>(),
                      y.data, y.dtype, (int)y.ld, b.cu_rows, b.slots, (float *)io.state, plan, U, D, b.n_seq, n_chunks, H_, dk_, dv_, tau_,
                      q_scale_, eps_, rt.stream);
        } else {
            FG_LAUNCH("mix", fg_gla, proj.ptr<float>(), (int)proj.ld, z.ptr<float>(), (int)z.ld, bias_.t.ptr<float>(), norm_.t.ptr<float>(), y.data,
                      y.dtype, (int)y.ld, b.cu_rows, b.slots, (float *)io.state, b.n_seq, H_, dk_, dv_, tau_, q_scale_, eps_, rt.stream);
        }
        DeferredNorm started;
        o_.forward(rt, y, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_ = 0, H_ = 0, dk_ = 0, dv_ = 0, rank_ = -1, chunk_threshold_ = 32;
    float eps_ = 0.f, tau_ = 1.f, q_scale_ = 1.f;
    Linear proj_, up_, o_;
    Weight bias_, norm_;
};

// What the two mixers below share: a short causal convolution with SiLU in front of the recurrence, whose last taps - 1 inputs
// are the first part of the mixer's state row, and the recurrence of recurrence.cu behind it, whose state is the second part.
static Weight f32_rows(const std::vector<Weight> &parts, cudaStream_t s) { return concat_rows(parts, FG_F32, s); }
// Floats of a sequence's recurrence state, as recurrence.cu lays it out: a column of a head's [d, dv] state is shared by R
// lanes, the smallest power of two that leaves a lane at most 16 rows, and rows are padded to a multiple of R.  (Computed
// here so that sizing a cache needs no kernel library; load() checks it against the library's own answer.)
static int64_t recurrence_state_floats(int H, int d, int dv, const char *who) {
    int R = 1;
    while (R < 32 && (d + R - 1) / R > 16) R *= 2;
    if ((d + R - 1) / R > 16) fail(FG_E_CONFIG, std::string(who) + ": the state of a head exceeds what the kernel takes");
    return (int64_t)H * ((d + R - 1) / R) * dv * R;
}
static void check_state_floats(int H, int d, int dv, const char *who) {
    if (FG_KERNEL("mix", fg_decay_recurrence_state_floats)(H, d, dv) != recurrence_state_floats(H, d, dv, who))
        fail(FG_E_INTERNAL, std::string(who) + ": host and kernel library disagree on the size of a state row");
}

// "state_space": the state-space form with a scalar decay per head and token ("duality").  With the normalised input h,
// inner = n_heads * v_head_dim, N = state_size and G = n_groups (head h uses group h / (n_heads / G)):
//     W_in h = [z: inner | x: inner | B: G N | C: G N | dt: n_heads]
//     (x, B, C) <- silu(causal convolution over time per channel + bias)          weights [inner + 2 G N, taps]
//     dt <- softplus(dt + dt_bias);  S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T (S: [N, v_head_dim]);  y_t = S_t^T C_t + D x_t
//     y <- y * silu(z), then an RMS norm in norm_groups equal parts of the inner channels, times a weight [inner]; output W_o y
// Projections leave their contraction as float32; convolution, decays, steps, state, gate and norm are float32 on the FMA units
// in every engine dtype; only the normalised y takes the engine's dtype, as the output projection's input.
class StateSpaceMixer : public Mixer {
public:
    StateSpaceMixer(const Json &p, BuildContext &) {
        const char *me = "state_space";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        dv_ = (int)param_int(p, "v_head_dim", me);
        N_ = (int)param_int(p, "state_size", me);
        G_ = (int)param_int(p, "n_groups", 1, me);
        taps_ = (int)param_int(p, "conv_taps", 1, me);
        norm_groups_ = (int)param_int(p, "norm_groups", 1, me);
        eps_ = (float)param_float(p, "eps", me);
        if (E_ <= 0 || H_ <= 0 || dv_ <= 0 || N_ <= 0 || G_ <= 0 || taps_ <= 0 || norm_groups_ <= 0) fail(FG_E_CONFIG, "state_space: sizes must be positive");
        if (H_ % G_) fail(FG_E_CONFIG, format("state_space: %d heads are not a multiple of %d groups", H_, G_));
        if ((H_ * dv_) % norm_groups_) fail(FG_E_CONFIG, format("state_space: %d inner channels do not split into %d norm groups", H_ * dv_, norm_groups_));
        if (N_ > 512) fail(FG_E_CONFIG, format("state_space: state_size %d exceeds 512, the largest the kernel takes", N_));
        if (!(eps_ > 0.f)) fail(FG_E_CONFIG, "state_space: eps must be positive");
    }
    int64_t inner() const { return (int64_t)H_ * dv_; }
    int64_t conv_channels() const { return inner() + (int64_t)2 * G_ * N_; }
    int64_t conv_floats() const { return (int64_t)(taps_ - 1) * conv_channels(); }
    std::vector<TensorDecl> tensor_decls() const override {
        const int64_t I = inner(), C = conv_channels();
        return {{"in_proj.weight", {2 * I + 2 * G_ * N_ + H_, E_}}, {"conv.weight", {C, (int64_t)taps_}, false, 0, 0.5f}, {"conv.bias", {C}, false, 0, 0.3f},
                {"dt_bias", {(int64_t)H_}, false, 0, 1.0f}, {"A_log", {(int64_t)H_}, false, 0, 1.0f}, {"D", {(int64_t)H_}, false, 1, 0.3f},
                {"norm.weight", {I}, false, 1, 0.01f}, {"o_proj.weight", {E_, I}}};
    }
    bool can_overwrite() const override { return true; }
    bool strided_state() const override { return true; }
    int64_t state_bytes() const override {
        return (conv_floats() + recurrence_state_floats(H_, N_, dv_, "state_space")) * (int64_t)sizeof(float);
    }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        check_state_floats(H_, N_, dv_, "state_space");
        in_ = Linear(tensor_of(tensors, "in_proj.weight"));
        o_ = Linear(tensor_of(tensors, "o_proj.weight"));
        conv_w_ = f32_rows({tensor_of(tensors, "conv.weight")}, rt.stream);
        conv_b_ = f32_rows({tensor_of(tensors, "conv.bias")}, rt.stream);
        dt_bias_ = f32_rows({tensor_of(tensors, "dt_bias")}, rt.stream);
        a_log_ = f32_rows({tensor_of(tensors, "A_log")}, rt.stream);
        skip_ = f32_rows({tensor_of(tensors, "D")}, rt.stream);
        norm_ = f32_rows({tensor_of(tensors, "norm.weight")}, rt.stream);
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *emit_norm) override {
        if (!io.state || io.state_bytes < state_bytes()) fail(FG_E_INTERNAL, "state_space: the schedule entry has no state rows");
        const long long stride = (long long)(io.state_stride / (int64_t)sizeof(float));
        const int I = (int)inner(), C = (int)conv_channels(), GN = G_ * N_;
        Tensor proj = in_.forward(rt, xn, nullptr, Tensor(), FG_F32, false, nullptr, nullptr);
        const int M = (int)proj.rows, ld = (int)proj.ld;
        float *state = (float *)io.state;
        Tensor xbc = rt.arena->matrix(M, C, FG_F32);
        FG_LAUNCH("mix", fg_conv1d_silu, proj.ptr<float>() + I, ld, conv_w_.t.ptr<float>(), conv_b_.t.ptr<float>(), taps_, state, stride, b.row_seq, b.cu_rows,
                  b.slots, xbc.ptr<float>(), (int)xbc.ld, M, C, rt.stream);
        if (taps_ > 1)
            FG_LAUNCH("mix", fg_conv1d_state, proj.ptr<float>() + I, ld, taps_, state, stride, b.cu_rows, b.slots, b.n_seq, C, rt.stream);
        float *decay = (float *)rt.arena->alloc((size_t)2 * M * H_ * sizeof(float)), *step = decay + (size_t)M * H_;
        FG_LAUNCH("mix", fg_decay_gates, proj.ptr<float>() + I + C, ld, nullptr, 0, a_log_.t.ptr<float>(), dt_bias_.t.ptr<float>(), 0, decay, step, M, H_,
                  rt.stream);
        Tensor y = rt.arena->matrix(M, I, FG_F32);
        const int xl = (int)xbc.ld;
        FG_LAUNCH("mix", fg_decay_recurrence, xbc.ptr<float>() + I + GN, xl, xbc.ptr<float>() + I, xl, xbc.ptr<float>(), xl, decay, step, skip_.t.ptr<float>(),
                  y.ptr<float>(), (int)y.ld, b.cu_rows, b.slots, state + conv_floats(), stride, b.n_seq, H_, G_, N_, dv_, 0, rt.stream);
        Tensor yn = rt.arena->matrix(M, I, rt.dtype);
        FG_LAUNCH("mix", fg_gated_group_norm, y.ptr<float>(), (int)y.ld, proj.ptr<float>(), ld, norm_.t.ptr<float>(), I, yn.data, yn.dtype, (int)yn.ld, M, I,
                  I / norm_groups_, eps_, 1, rt.stream);
        DeferredNorm started;
        o_.forward(rt, yn, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_ = 0, H_ = 0, dv_ = 0, N_ = 0, G_ = 1, taps_ = 1, norm_groups_ = 1;
    float eps_ = 0.f;
    Linear in_, o_;
    Weight conv_w_, conv_b_, dt_bias_, a_log_, skip_, norm_;
};

// "gated_delta": the gated delta rule.  With the normalised input h, n_kv_heads heads of q and k (size head_dim) and n_heads
// heads of v (size v_head_dim), head h using q/k head h / (n_heads / n_kv_heads):
//     q, k, v <- silu(causal convolution over time per channel of W_q h, W_k h, W_v h)      weights [channels, taps], no bias
//     q <- q / sqrt(sum(q^2) + unit_eps) * q_scale and k <- k / sqrt(sum(k^2) + unit_eps), per head
//     beta = sigmoid(W_b h), g = exp(-exp(A_log) softplus(W_a h + dt_bias)), one each per head
//     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                          (S: [head_dim, v_head_dim])
//     y = o / sqrt(mean(o^2) + eps) * w (w [v_head_dim], shared by heads) * silu(W_g h); output W_o y
// The six projections are ONE contraction with float32 output; everything up to y is float32 in every engine dtype.
class GatedDeltaMixer : public Mixer {
public:
    GatedDeltaMixer(const Json &p, BuildContext &) {
        const char *me = "gated_delta";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        G_ = (int)param_int(p, "n_kv_heads", H_, me);
        d_ = (int)param_int(p, "head_dim", me);
        dv_ = (int)param_int(p, "v_head_dim", d_, me);
        taps_ = (int)param_int(p, "conv_taps", 1, me);
        eps_ = (float)param_float(p, "eps", me);
        unit_eps_ = (float)param_float(p, "unit_eps", 1e-6, me);
        q_scale_ = (float)param_float(p, "q_scale", 1.0 / std::sqrt((double)d_), me);
        if (E_ <= 0 || H_ <= 0 || G_ <= 0 || d_ <= 0 || dv_ <= 0 || taps_ <= 0) fail(FG_E_CONFIG, "gated_delta: sizes must be positive");
        if (H_ % G_) fail(FG_E_CONFIG, format("gated_delta: %d heads are not a multiple of %d key heads", H_, G_));
        if (d_ > 512) fail(FG_E_CONFIG, format("gated_delta: head_dim %d exceeds 512, the largest the kernel takes", d_));
        if (!(eps_ > 0.f) || !(unit_eps_ >= 0.f)) fail(FG_E_CONFIG, "gated_delta: eps must be positive");
    }
    int64_t conv_channels() const { return (int64_t)2 * G_ * d_ + (int64_t)H_ * dv_; }
    int64_t conv_floats() const { return (int64_t)(taps_ - 1) * conv_channels(); }
    std::vector<TensorDecl> tensor_decls() const override {
        const int64_t Q = (int64_t)G_ * d_, V = (int64_t)H_ * dv_;
        return {{"q_proj.weight", {Q, E_}}, {"k_proj.weight", {Q, E_}}, {"v_proj.weight", {V, E_}}, {"b_proj.weight", {(int64_t)H_, E_}},
                {"a_proj.weight", {(int64_t)H_, E_}}, {"g_proj.weight", {V, E_}}, {"o_proj.weight", {E_, V}},
                {"q_conv.weight", {Q, (int64_t)taps_}, false, 0, 0.5f}, {"k_conv.weight", {Q, (int64_t)taps_}, false, 0, 0.5f},
                {"v_conv.weight", {V, (int64_t)taps_}, false, 0, 0.5f}, {"A_log", {(int64_t)H_}, false, 0, 1.0f}, {"dt_bias", {(int64_t)H_}, false, 0, 1.0f},
                {"norm.weight", {(int64_t)dv_}, false, 1, 0.01f}};
    }
    bool can_overwrite() const override { return true; }
    bool strided_state() const override { return true; }
    int64_t state_bytes() const override {
        return (conv_floats() + recurrence_state_floats(H_, d_, dv_, "gated_delta")) * (int64_t)sizeof(float);
    }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        check_state_floats(H_, d_, dv_, "gated_delta");
        std::vector<Weight> rows;
        bool same = true;
        for (const char *n : {"q_proj.weight", "k_proj.weight", "v_proj.weight", "b_proj.weight", "a_proj.weight", "g_proj.weight"}) {
            rows.push_back(tensor_of(tensors, n));
            same = same && rows.back().t.dtype == rows.front().t.dtype;
        }
        proj_ = Linear(concat_rows(rows, same ? rows.front().t.dtype : FG_F32, rt.stream));
        o_ = Linear(tensor_of(tensors, "o_proj.weight"));
        // [channels, taps] row-major: the three lie one after another
        conv_w_ = make_weight(conv_channels(), taps_, FG_F32, "convolution weights of the delta rule");
        size_t at = 0;
        for (const char *n : {"q_conv.weight", "k_conv.weight", "v_conv.weight"}) {
            const Weight &w = tensor_of(tensors, n);
            dev_convert(w.t.data, w.t.dtype, (char *)conv_w_.t.data + at * 4, FG_F32, w.t.numel(), rt.stream);
            at += (size_t)w.t.numel();
        }
        a_log_ = f32_rows({tensor_of(tensors, "A_log")}, rt.stream);
        dt_bias_ = f32_rows({tensor_of(tensors, "dt_bias")}, rt.stream);
        norm_ = f32_rows({tensor_of(tensors, "norm.weight")}, rt.stream);
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &b, const LayerIO &io, Tensor &residual,
                         Norm *emit_norm) override {
        if (!io.state || io.state_bytes < state_bytes()) fail(FG_E_INTERNAL, "gated_delta: the schedule entry has no state rows");
        const long long stride = (long long)(io.state_stride / (int64_t)sizeof(float));
        const int Q = G_ * d_, V = H_ * dv_, C = (int)conv_channels();
        Tensor proj = proj_.forward(rt, xn, nullptr, Tensor(), FG_F32, false, nullptr, nullptr);
        const int M = (int)proj.rows, ld = (int)proj.ld;
        float *state = (float *)io.state;
        Tensor qkv = rt.arena->matrix(M, C, FG_F32);
        const int xl = (int)qkv.ld;
        FG_LAUNCH("mix", fg_conv1d_silu, proj.ptr<float>(), ld, conv_w_.t.ptr<float>(), nullptr, taps_, state, stride, b.row_seq, b.cu_rows, b.slots,
                  qkv.ptr<float>(), xl, M, C, rt.stream);
        if (taps_ > 1) FG_LAUNCH("mix", fg_conv1d_state, proj.ptr<float>(), ld, taps_, state, stride, b.cu_rows, b.slots, b.n_seq, C, rt.stream);
        FG_LAUNCH("mix", fg_unit_heads, qkv.ptr<float>(), xl, G_, d_, unit_eps_, q_scale_, M, rt.stream);
        FG_LAUNCH("mix", fg_unit_heads, qkv.ptr<float>() + Q, xl, G_, d_, unit_eps_, 1.0f, M, rt.stream);
        float *decay = (float *)rt.arena->alloc((size_t)2 * M * H_ * sizeof(float)), *step = decay + (size_t)M * H_;
        FG_LAUNCH("mix", fg_decay_gates, proj.ptr<float>() + C + H_, ld, proj.ptr<float>() + C, ld, a_log_.t.ptr<float>(), dt_bias_.t.ptr<float>(), 1, decay,
                  step, M, H_, rt.stream);
        Tensor o = rt.arena->matrix(M, V, FG_F32);
        FG_LAUNCH("mix", fg_decay_recurrence, qkv.ptr<float>(), xl, qkv.ptr<float>() + Q, xl, qkv.ptr<float>() + 2 * Q, xl, decay, step, nullptr, o.ptr<float>(),
                  (int)o.ld, b.cu_rows, b.slots, state + conv_floats(), stride, b.n_seq, H_, G_, d_, dv_, 1, rt.stream);
        Tensor y = rt.arena->matrix(M, V, rt.dtype);
        FG_LAUNCH("mix", fg_gated_group_norm, o.ptr<float>(), (int)o.ld, proj.ptr<float>() + C + 2 * H_, ld, norm_.t.ptr<float>(), dv_, y.data, y.dtype,
                  (int)y.ld, M, V, dv_, eps_, 0, rt.stream);
        DeferredNorm started;
        o_.forward(rt, y, nullptr, residual, FG_F32, !rt.overwrite, emit_norm, &started);
        return started;
    }

private:
    int E_ = 0, H_ = 0, G_ = 0, d_ = 0, dv_ = 0, taps_ = 1;
    float eps_ = 0.f, unit_eps_ = 1e-6f, q_scale_ = 1.f;
    Linear proj_, o_;
    Weight conv_w_, a_log_, dt_bias_, norm_;
};

void add_recurrent_kinds(std::map<std::string, PartFactory> &mixers) {
    mixers["gated_linear_attention"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<GatedLinearAttention>(p, c); };
    mixers["retention"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<RetentionMixer>(p, c); };
    mixers["state_space"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<StateSpaceMixer>(p, c); };
    mixers["gated_delta"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<GatedDeltaMixer>(p, c); };
}

}  // namespace fg
