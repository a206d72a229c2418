/* The C interface of the kernel libraries (libfg_core.so, libfg_tc.so, libfg_attn.so).
 *
 * Every function launches on `stream` and returns 0, a cudaError_t, or one of the FG_ERR_* codes
 * below; none allocates device memory.  Pointers are device pointers unless said otherwise.
 * dtype codes: FG_F32 = 0, FG_BF16 = 1.  Page pools are [pages, kv_heads, page, head_dim]; block
 * tables are [sequences, table_width] int32 page ids (a value pool has head size hdv where a function names one).  The Python package calls these through ctypes
 * (fastgguf_b200/ops); the formulas each one follows are cited in its .cu file.
 */
#pragma once
#include <cuda_runtime.h>

#define FG_F32 0
#define FG_BF16 1
#define FG_ERR_BAD_DTYPE 10001
#define FG_ERR_BAD_SIZE 10002
#define FG_ERR_PIPELINE 10003      /* a bounded device-side wait ran out */
#define FG_ERR_TENSORMAP 10004

#ifdef __cplusplus
extern "C" {
#endif

/* ---- libfg_core: row-wise kernels, plain contraction, any-size attention, sampling */
int fg_embed_gather(const void *table, int table_dtype, const int *tokens, float *x, int M, int E, cudaStream_t stream);
int fg_embed_gather_scaled(const void *table, int table_dtype, const int *tokens, float *x, int M, int E, float scale,
                           cudaStream_t stream);
int fg_embed_gather_norm(const void *table, int table_dtype, const int *tokens, float *x, const float *norm_w,
                         void *xw, float *ss, int M, int E, cudaStream_t stream);
int fg_rmsnorm(const float *x, const float *w, const int *rows, void *out, int out_dtype, int R, int E, float eps,
               cudaStream_t stream);
int fg_rope_append(void *qkv, int dtype, int ld, const int *positions, const int *row_seq, const int *block_table,
                   int table_width, void *k_pool, void *v_pool, const float *cos_t, const float *sin_t, int M, int H,
                   int KV, int hd, int page_size, int write_kv, cudaStream_t stream);
/* keys [KV, hd] and values [KV, hdv] of each row to their pages, unrotated; k_off: where the keys start in a row */
int fg_kv_append(const void *qkv, int dtype, int ld, int k_off, const int *positions, const int *row_seq,
                 const int *block_table, int table_width, void *k_pool, void *v_pool, int M, int KV, int hd, int hdv,
                 int page_size, cudaStream_t stream);
/* x += t / rms(t) * w_post; with w_next also out = x / rms(x) * w_next (out_dtype) */
int fg_norm_add_norm(const float *t, const float *w_post, float *x, const float *w_next, void *out, int out_dtype,
                     int M, int E, float eps_post, float eps_next, cudaStream_t stream);
int fg_activation(void *z, int dtype, long long total, int kind /* 0: relu(z)^2 */, cudaStream_t stream);
int fg_softcap(float *logits, int R, int V, int ld, float cap, cudaStream_t stream);
int fg_concat2(const float *a, int lda, const float *b, int ldb, void *out, int out_dtype, int ldo, int M, int E,
               cudaStream_t stream);
int fg_silu_mul(const void *gu, void *out, int dtype, int M, int F, cudaStream_t stream);
/* out (+)= scale_a * f_a(a) + scale_b * f_b(b) over float32 rows [M, E]; f(t) = t / rms(t) * w with a weight, t itself without */
int fg_pair_combine(const float *a, const float *b, const float *w_a, const float *w_b, float scale_a, float scale_b, float eps,
                    float *out, int M, int E, int accumulate, cudaStream_t stream);
/* out_a = x / rms(x) * w_a and out_b = x / rms(x) * w_b of the same float32 rows, one pass */
int fg_rmsnorm_pair(const float *x, const float *w_a, const float *w_b, void *out_a, void *out_b, int out_dtype, int R, int E,
                    float eps_a, float eps_b, cudaStream_t stream);
/* the float32 rows themselves in another dtype */
int fg_cast_rows(const float *x, int ldx, void *out, int out_dtype, int ldo, int M, int E, cudaStream_t stream);
/* out[m, j] = gelu_tanh(z[m, j]) * table[tokens[m], col0 + j], j < D */
int fg_gelu_mul_gather(const float *z, int ldz, const void *table, int table_dtype, int ldt, int col0, const int *tokens, void *out,
                       int out_dtype, int ldo, int M, int D, cudaStream_t stream);
int fg_decode_advance(int *tokens, int *positions, const int *next_tokens, const int *active, int B, cudaStream_t stream);
int fg_gemm_generic(const void *A, int a_dtype, int lda, const void *W, int w_dtype, int ldw, void *C, int out_dtype,
                    int ldc, int accumulate, int M, int N, int K, cudaStream_t stream);
int fg_attention_generic(const void *q, int ldq, void *out, int ldo, int dtype, const int *positions,
                         const int *row_seq, const int *block_table, int table_width, const void *k_pool,
                         const void *v_pool, int M, int H, int KV, int hd, int page_size, float scale, int window,
                         cudaStream_t stream);
/* the same with values of head size hdv and, with a window, the sequence's first keep_first keys visible as well */
/* softcap > 0: scores capped by softcap * tanh(score / softcap); sinks: a float per query head that joins the softmax's denominator;
   latent: the cache holds a latent (v_pool, hdv numbers, also the value) and a rotated key part (k_pool, hd numbers) a position,
   and a query head has hdv + hd numbers */
int fg_attention_generic_ext(const void *q, int ldq, void *out, int ldo, int dtype, const int *positions,
                             const int *row_seq, const int *block_table, int table_width, const void *k_pool,
                             const void *v_pool, int M, int H, int KV, int hd, int hdv, int page_size, float scale,
                             int window, int keep_first, float softcap, const float *sinks, int latent, cudaStream_t stream);
int fg_attention_generic_kept(const void *q, int ldq, void *out, int ldo, int dtype, const int *positions,
                              const int *row_seq, const int *block_table, int table_width, const void *k_pool,
                              const void *v_pool, int M, int H, int KV, int hd, int hdv, int page_size, float scale,
                              int window, int keep_first, cudaStream_t stream);
int fg_sample(float *logits, int B, int V, int ldl, float temp, int top_k, float top_p, float repeat_penalty,
              int repeat_last_n, const int *seq_slot, unsigned long long *rng, int *hist, int hist_cap,
              int *hist_count, const int *stop_ids, int n_stop, int *out_tokens,
              unsigned long long *scratch /* [B, 4096] or null */, cudaStream_t stream);
int fg_argmax(const float *logits, int B, int V, int ldl, int *out, cudaStream_t stream);

/* ---- libfg_mix: retention (linear attention with a fixed decay per head) and the mixture of experts */
/* proj rows: q [H, dk] | k [H, dk] | v [H, dv] | g [H, dv] float32; state [slots, H, dk, dv] float32; out [M, H * dv] */
int fg_retention(const float *proj, int ld, void *out, int out_dtype, int ldo, const int *positions, const int *cu_rows,
                 const int *slots, const float *cos_t, const float *sin_t, const float *decay, float *state, int n_seq,
                 int H, int dk, int dv, float k_scale, float eps, cudaStream_t stream);
int fg_retention_chunk_tokens(void);
int fg_retention_chunked_ok(int dk, int dv);
int fg_retention_chunked(const float *proj, int ld, void *out, int out_dtype, int ldo, const int *positions,
                         const int *cu_rows, const int *slots, const float *cos_t, const float *sin_t,
                         const float *decay, float *state, int *plan, float *U, int n_seq, int n_chunks, int H, int dk,
                         int dv, float k_scale, float eps, cudaStream_t stream);
/* gated linear attention (gla.cu): proj rows q [H, dk] | k [H, dk] | v [H, dv] | g [H, dv] float32, z rows [H, dk] decay logits
   without their bias; state [slots, H, dk, dv] float32; out [M, H * dv] */
int fg_gla(const float *proj, int ld, const float *z, int ldz, const float *z_bias, const float *norm_w, void *out, int out_dtype,
           int ldo, const int *cu_rows, const int *slots, float *state, int n_seq, int H, int dk, int dv, float tau, float q_scale,
           float eps, cudaStream_t stream);
int fg_gla_chunk_tokens(void);
int fg_gla_chunked_ok(int dk, int dv);
int fg_gla_chunked(const float *proj, int ld, const float *z, int ldz, const float *z_bias, const float *norm_w, void *out,
                   int out_dtype, int ldo, const int *cu_rows, const int *slots, float *state, int *plan, float *U, float *D,
                   int n_seq, int n_chunks, int H, int dk, int dv, float tau, float q_scale, float eps, cudaStream_t stream);
/* recurrences with one decay a head and token (recurrence.cu): S <- a S; u = b (v - [delta] S^T k); S <- S + k u^T;
   o = S^T q + skip v.  q, k [M, Hq, d], v [M, H, dv], decay and step [M, H], out [M, H * dv], all float32; a sequence's state
   row (state_stride floats apart) holds fg_decay_recurrence_state_floats(H, d, dv) floats in the kernel's own layout */
int fg_decay_recurrence_lanes(int d);
long long fg_decay_recurrence_state_floats(int H, int d, int dv);
int fg_decay_recurrence(const float *q, int ldq, const float *k, int ldk, const float *v, int ldv, const float *decay,
                        const float *step, const float *skip, float *out, int ldo, const int *cu_rows, const int *slots,
                        float *state, long long state_stride, int n_seq, int H, int Hq, int d, int dv, int delta,
                        cudaStream_t stream);
/* out = silu(bias + causal convolution over time of each channel), weights [C, taps]; a sequence's last taps - 1 inputs live in
   its state row [taps - 1, C]; fg_conv1d_state brings them up to date after the step's rows have been read */
int fg_conv1d_silu(const float *in, int ld, const float *w, const float *bias, int taps, const float *state, long long state_stride,
                   const int *row_seq, const int *cu_rows, const int *slots, float *out, int ldo, int M, int C, cudaStream_t stream);
int fg_conv1d_state(const float *in, int ld, int taps, float *state, long long state_stride, const int *cu_rows, const int *slots,
                    int n_seq, int C, cudaStream_t stream);
/* mode 0: step = softplus(a_raw + dt_bias), decay = exp(-exp(A_log) step); mode 1: decay = exp(-exp(A_log) softplus(a_raw +
   dt_bias)), step = sigmoid(b_raw); decay and step [M, H] */
int fg_decay_gates(const float *a_raw, int lda, const float *b_raw, int ldb, const float *A_log, const float *dt_bias, int mode,
                   float *decay, float *step, int M, int H, cudaStream_t stream);
int fg_unit_heads(float *x, int ld, int n_heads, int d, float eps, float scale, int M, cudaStream_t stream);
/* gate_first: t = y silu(g), out = t / rms(t) * w over groups of `group` channels; else out = y / rms(y) * w[c % w_period] * silu(g) */
int fg_gated_group_norm(const float *y, int ldy, const float *g, int ldg, const float *w, int w_period, void *out, int out_dtype,
                        int ldo, int M, int C, int group, float eps, int gate_first, cudaStream_t stream);
/* between an attention mixer's projections and its attention kernel (attention_prep.cu) */
int fg_qkv_prepare(const float *proj, int ld, const float *bias, const float *conv_w, int taps, const float *conv_state,
                   const float *qn_w, const float *kn_w, float eps, const float *cos_t, const float *sin_t, int tbl_half,
                   int rot_dims, const int *positions, const int *row_seq, const int *cu_rows, const int *slots,
                   const int *block_table, int table_width, void *q_out, int ldq, void *k_pool, void *v_pool, int dtype, int M,
                   int H, int KV, int hd, int hdv, int page_size, cudaStream_t stream);
/* the same with the norm per head (weights [hd]) instead of over the whole of q and of k, and with rotated pairs
   (i, i + rot_dims / 2) instead of (2i, 2i + 1) */
int fg_qkv_prepare_ext(const float *proj, int ld, const float *bias, const float *conv_w, int taps, const float *conv_state,
                       const float *qn_w, const float *kn_w, float eps, const float *cos_t, const float *sin_t, int tbl_half,
                       int rot_dims, const int *positions, const int *row_seq, const int *cu_rows, const int *slots,
                       const int *block_table, int table_width, void *q_out, int ldq, void *k_pool, void *v_pool, int dtype, int M,
                       int H, int KV, int hd, int hdv, int page_size, int norm_per_head, int rot_halves, cudaStream_t stream);
/* x[m, h * DV + j] *= sigmoid(gate[m, h]) in place (gate null: none); `pad` columns behind the heads become (1, 0, 0, ...) */
int fg_head_gate(void *x, int ldx, int dtype, const float *gate, int ldg, int M, int H, int DV, int pad, cudaStream_t stream);
int fg_conv_state_update(const float *proj, int ld, const float *bias, int taps, float *conv_state, const int *cu_rows,
                         const int *slots, int n_seq, int C, cudaStream_t stream);
int fg_latent_append(const float *kv, int ld, const float *norm_w, float eps, const float *cos_t, const float *sin_t, int tbl_half,
                     const int *positions, const int *row_seq, const int *block_table, int table_width, void *k_pool,
                     void *v_pool, int dtype, int M, int rank, int rot_dim, int page_size, cudaStream_t stream);
int fg_rope_pairs(const float *in, int ld_in, int in_stride, int in_off, void *out, int out_dtype, int ld_out, int out_stride,
                  int out_off, const int *positions, const float *cos_t, const float *sin_t, int tbl_half, int M, int H, int dims,
                  cudaStream_t stream);
int fg_rmsnorm_strided(const float *x, int ldx, const float *w, void *out, int out_dtype, int ldo, int R, int E, float eps,
                       cudaStream_t stream);
int fg_head_gemm(const void *A, int a_dtype, int lda, int a_stride, const void *W, int w_dtype, int ldw, int transposed, void *C,
                 int c_dtype, int ldc, int c_stride, const float *gate, int ldg, int M, int N, int K, int H, cudaStream_t stream);
/* latent attention on the cache of latents (attention_latent.cu) */
long long fg_latent_decode_scratch_floats(int M, int H, int R, int n_splits);
int fg_latent_decode(const void *q, int ldq, void *out, int ldo, int dtype, const int *positions, const int *row_seq,
                     const int *block_table, int table_width, const void *k_pool, const void *v_pool, int M, int H, int R,
                     int DR, int page_size, float scale, const float *sinks, int n_splits, float *part, cudaStream_t stream);
int fg_latent_decode_mma_ok(int R, int DR, int page_size);
int fg_latent_decode_mma(const void *q, int ldq, void *out, int ldo, const int *positions, const int *row_seq,
                         const int *block_table, int table_width, const void *k_pool, const void *v_pool, int M, int H, int R,
                         int DR, int page_size, float scale, const float *sinks, int n_splits, float *part, cudaStream_t stream);
int fg_seq_page_table(const int *cu_rows, int n_seq, int width, int page_size, int *table, cudaStream_t stream);
int fg_latent_expand(const float *q, int ldq, const float *kv, int ldkv, int rot_at, const void *kp, int ldkp, const void *vp,
                     int ldvp, const float *cos_t, const float *sin_t, int tbl_half, const int *positions, const int *row_seq,
                     const int *table, int width, void *qx, void *Kx, void *Vx, int M, int H, int D, int DR, int DV,
                     int page_size, cudaStream_t stream);
/* the same for a key part that is rotated already (key_rotated != 0), and a row's latent (c_out, the cache's dtype) and rotated
   key part (kr_out, float32) out of a cache of latents, for a layer that reads another layer's cache */
int fg_latent_expand_ext(const float *q, int ldq, const float *kv, int ldkv, int rot_at, const void *kp, int ldkp, const void *vp,
                         int ldvp, const float *cos_t, const float *sin_t, int tbl_half, const int *positions, const int *row_seq,
                         const int *table, int width, void *qx, void *Kx, void *Vx, int M, int H, int D, int DR, int DV,
                         int page_size, int key_rotated, cudaStream_t stream);
int fg_latent_fetch(const void *k_pool, const void *v_pool, int dtype, const int *positions, const int *row_seq, const int *table,
                    int width, int page_size, void *c_out, int ldc, float *kr_out, int ldk, int M, int R, int DR, cudaStream_t stream);
int fg_gate_slice(const void *x, int ldx, int stride, const float *gate, int ldg, void *out, int ldo, int dtype, int M, int H,
                  int DV, cudaStream_t stream);
int fg_moe_logits(const void *x, int ldx, const void *W, int ldw, int dtype, float *z, int M, int X, int E, cudaStream_t stream);
int fg_moe_gather(const void *x, int ldx, int dtype, const int *order, int top, void *xs, int P, int E, cudaStream_t stream);
int fg_moe_act(const float *gu, const int *order, const float *pair_weight, void *y, int dtype, int P, int F, float limit,
               float alpha, cudaStream_t stream);
int fg_moe_route(const float *logits, int M, int X, int top, int *pair_expert, float *pair_weight, int *offsets, int *order,
                 int *slot_of, cudaStream_t stream);
/* softmax scores, choice on score + bias among the `keep` best of n_groups groups, weights = chosen scores / their sum * scale */
int fg_moe_route_grouped(const float *logits, const float *bias, int M, int X, int top, int n_groups, int keep, float scale,
                         int *pair_expert, float *pair_weight, int *offsets, int *order, int *slot_of, cudaStream_t stream);
/* pair_weight null: the inputs are not weighted; limit <= 0: the activation is silu(gate) * up */
int fg_moe_first(const void *x, int ldx, const void *w_in, void *y, int ldy, int dtype, const int *pair_expert,
                 const int *offsets, const int *order, const float *pair_weight, int M, int X, int top, int F, int E,
                 float limit, float alpha, cudaStream_t stream);
int fg_moe_second(const void *y, int ldy, const void *w_out, float *out, int ldo, int dtype, const int *pair_expert,
                  const int *offsets, const int *order, int M, int X, int top, int F, int E, cudaStream_t stream);
int fg_moe_combine(const float *slot_out, int ld, const int *slot_of, float *t, int M, int top, int E, int accumulate,
                   cudaStream_t stream);
/* t[r] (+)= sum_k w[r, k] * (expert[r, k] < n_real ? slot_out[slot_of[r, k]] : x[r]) */
int fg_moe_combine_weighted(const float *slot_out, int ld, const int *slot_of, const int *pair_expert, const float *pair_weight,
                            const void *x, int ldx, int dtype, int n_real, float *t, int M, int top, int E, int accumulate,
                            cudaStream_t stream);

/* ---- libfg_tc: bf16 contraction on tcgen05 / TMA / tensor memory
 * epi: 0 bf16 out, 1 f32 out, 2 f32 out += (residual add), 3 silu(gate) * up on interleaved rows, 4 bf16 out of max(x, 0)^2 */
int fg_gemm_tc(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi, int M, int N, int K,
               int force_splits, const float *ss_in, int ss_tiles, int ss_size, float ss_eps, const float *norm_w,
               void *xw_out, float *ss_out, int *ss_tiles_out /* host */, cudaStream_t stream);
/* the same with device memory the call may use: with fg_gemm_tc_workspace_bytes(M, N, K, epi) of it (0: none needed) a
   prefill contraction of few output tiles is split along K over all SMs and summed, in order, by a second kernel */
int fg_gemm_tc_ws(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi, int M, int N, int K,
                  int force_splits, const float *ss_in, int ss_tiles, int ss_size, float ss_eps, const float *norm_w,
                  void *xw_out, float *ss_out, int *ss_tiles_out /* host */, void *workspace, long long workspace_bytes,
                  cudaStream_t stream);
long long fg_gemm_tc_workspace_bytes(int M, int N, int K, int epi);
int fg_gemm_tc_max_ss_tiles(int N);
/* grouped contraction over runs of rows, each with its own matrix of a stack (see gemm_tc.cu); tiles: device int4 table */
int fg_gemm_tc_grouped_bn(int N);
int fg_gemm_tc_grouped(const void *X, int ldx, int rows, const void *W, int ldw, int stack_rows, float *out, int ldc, int N, int K,
                       const void *tiles, int n_tiles, cudaStream_t stream);
int fg_gemm_tc_error(void);
/* tests only: shorten the bounded waits and make the decode kernel's pipeline stall, see gemm_tc.cu */
int fg_gemm_tc_test_hook(long long wait_limit_cycles, int skip_copy);

/* ---- libfg_attn: bf16 tensor-core attention over the paged cache (head sizes 64 and 128, pages of 64) */
int fg_attention_decode(const void *q, int ldq, void *out, int ldo, const int *positions, const int *block_table,
                        int table_width, const void *k_pool, const void *v_pool, int B, int H, int KV, int hd,
                        int page_size, float scale, int window, int n_splits, float *part_o, float *part_ml,
                        cudaStream_t stream);
int fg_attention_decode_fused(const void *qkv, int ldq, void *out, int ldo, const int *positions,
                              const int *block_table, int table_width, void *k_pool, void *v_pool, const float *cos_t,
                              const float *sin_t, int B, int H, int KV, int hd, int page_size, float scale, int window,
                              int n_splits, cudaStream_t stream);
int fg_attention_prefill(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                         const int *block_table, int table_width, const void *k_pool, const void *v_pool, int n_seq,
                         int max_new, int H, int KV, int hd, int page_size, float scale, int window, cudaStream_t stream);
/* the three above with the first keep_first keys of a sequence visible in front of a window */
/* the same with capped scores (softcap > 0) and a sink per query head (sinks, or null) */
int fg_attention_decode_ext(const void *q, int ldq, void *out, int ldo, const int *positions, const int *block_table,
                            int table_width, const void *k_pool, const void *v_pool, int B, int H, int KV, int hd,
                            int page_size, float scale, int window, int keep_first, int n_splits, float *part_o,
                            float *part_ml, float softcap, const float *sinks, cudaStream_t stream);
int fg_attention_prefill_ext(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                             const int *block_table, int table_width, const void *k_pool, const void *v_pool, int n_seq,
                             int max_new, int H, int KV, int hd, int page_size, float scale, int window, int keep_first,
                             float softcap, const float *sinks, cudaStream_t stream);
int fg_attention_prefill_tc_ext(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                                const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                                int n_pool_pages, int n_seq, int max_new, int H, int KV, int hd, int page_size, float scale,
                                int window, int keep_first, float softcap, const float *sinks, cudaStream_t stream);
int fg_attention_decode_kept(const void *q, int ldq, void *out, int ldo, const int *positions, const int *block_table,
                             int table_width, const void *k_pool, const void *v_pool, int B, int H, int KV, int hd,
                             int page_size, float scale, int window, int keep_first, int n_splits, float *part_o,
                             float *part_ml, cudaStream_t stream);
int fg_attention_decode_fused_kept(const void *qkv, int ldq, void *out, int ldo, const int *positions,
                                   const int *block_table, int table_width, void *k_pool, void *v_pool,
                                   const float *cos_t, const float *sin_t, int B, int H, int KV, int hd, int page_size,
                                   float scale, int window, int keep_first, int n_splits, cudaStream_t stream);
int fg_attention_prefill_kept(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                              const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                              int n_seq, int max_new, int H, int KV, int hd, int page_size, float scale, int window,
                              int keep_first, cudaStream_t stream);
int fg_attention_prefill_tc(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                            const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                            int n_pages, int n_seq, int max_new, int H, int KV, int hd, int page_size, float scale,
                            int window, cudaStream_t stream);
int fg_attention_prefill_tc_kept(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                                 const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                                 int n_pages, int n_seq, int max_new, int H, int KV, int hd, int page_size, float scale,
                                 int window, int keep_first, cudaStream_t stream);
int fg_attention_prefill_tc_error(void);
int fg_attention_prefill_tc_variant(int bits);   /* bit 0 / 1: two score tiles at head size 64 / 128; negative: by shape */
int fg_attention_prefill_tc_test_hook(long long wait_limit_cycles, int skip_copy);   /* tests only */
/* fg_attention_decode_noalloc: see fastgguf_noalloc.h */

#ifdef __cplusplus
}
#endif
