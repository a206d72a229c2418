// Row-wise kernels of the decoder: embedding gather, RMSNorm, rotary encoding with cache
// append, SiLU-multiply.  Each takes both storage dtypes (f32, bf16) and computes in f32.
//
// Reference formulas (file fastgguf.c of the reference engine):
//   embedding  read_embedding            :4576-4581   x = Emb[token, :]
//   RMSNorm    rmsnorm_w                 :3100-3105   y = x * (1/sqrt(mean(x^2) + eps)) * w
//   RoPE       apply_rope                :3123-3145   (a, b) <- (a cos - b sin, a sin + b cos)
//   cache      forward                   :4720, 4738-4739   K stored after RoPE, V raw
//   SiLU-mul   silu_f, forward           :3118, 4876  t = g / (1 + exp(-g)) * u
#include "common.cuh"

// ------------------------------------------------------------------ embedding gather
template <typename TW>
__global__ void embed_gather_kernel(const TW *__restrict__ table, const int *__restrict__ tokens,
                                    float *__restrict__ x, int E, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    int m = blockIdx.x;
    const TW *row = table + (size_t)tokens[m] * E;
    float *out = x + (size_t)m * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[i] = to_f32<TW>(row[i]) * scale;
}

// x = table[token] * scale (embd_scale of the reference, fastgguf.c:4652; 1 for most models)
extern "C" int fg_embed_gather_scaled(const void *table, int table_dtype, const int *tokens, float *x,
                                      int M, int E, float scale, cudaStream_t stream) {
    if (M <= 0) return 0;
    int threads = E >= 1024 ? 256 : 128;
    if (table_dtype == FG_F32)
        return fg_launch(embed_gather_kernel<float>, dim3(M), dim3(threads), 0, stream, (const float *)table, tokens, x, E, scale);
    else if (table_dtype == FG_BF16)
        return fg_launch(embed_gather_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (const bf16 *)table, tokens, x, E, scale);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}

extern "C" int fg_embed_gather(const void *table, int table_dtype, const int *tokens, float *x,
                               int M, int E, cudaStream_t stream) {
    return fg_embed_gather_scaled(table, table_dtype, tokens, x, M, E, 1.0f, stream);
}

// The same gather that also starts a deferred RMSNorm: xw = bf16(x * norm_w) and the row's sum of squares
// (one "tile"), for a contraction that applies 1/rms in its epilogue.
template <typename TW>
__global__ void embed_gather_norm_kernel(const TW *__restrict__ table, const int *__restrict__ tokens,
                                         float *__restrict__ x, const float *__restrict__ norm_w,
                                         bf16 *__restrict__ xw, float *__restrict__ ss, int E) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    int m = blockIdx.x;
    const TW *row = table + (size_t)tokens[m] * E;
    float acc = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = to_f32<TW>(row[i]);
        x[(size_t)m * E + i] = v;
        xw[(size_t)m * E + i] = __float2bfloat16_rn(v * norm_w[i]);
        acc += v * v;
    }
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) ss[m] = acc;
}

extern "C" int fg_embed_gather_norm(const void *table, int table_dtype, const int *tokens, float *x,
                                    const float *norm_w, void *xw, float *ss, int M, int E, cudaStream_t stream) {
    if (M <= 0) return 0;
    int threads = E >= 1024 ? 256 : 128;
    if (table_dtype == FG_F32)
        return fg_launch(embed_gather_norm_kernel<float>, dim3(M), dim3(threads), 0, stream, (const float *)table, tokens, x,
                         norm_w, (bf16 *)xw, ss, E);
    if (table_dtype == FG_BF16)
        return fg_launch(embed_gather_norm_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (const bf16 *)table, tokens, x,
                         norm_w, (bf16 *)xw, ss, E);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  `rows` (optional) names the input row of each output row, so the
// final norm runs only on the rows whose logits are wanted.  Statistics in f32 with a fixed
// reduction order: a row's result does not depend on what else is in the batch.
template <typename TO> __device__ __forceinline__ void store4(TO *dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float *dst, float a, float b, float c, float d) {
    *(float4 *)dst = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16 *dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2 *)dst = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
}

// VEC: rows are read and written four elements at a time (E % 4 == 0, 16-byte aligned rows)
template <typename TO, bool VEC>
__global__ void rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                               const int *__restrict__ rows, TO *__restrict__ out, int E, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    int r = blockIdx.x;
    const float *xi = x + (size_t)(rows ? rows[r] : r) * E;
    TO *o = out + (size_t)r * E;
    float ss = 0.f;
    if (VEC) {
        const float4 *x4 = (const float4 *)xi;
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
            float4 v = x4[i];
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) { float v = xi[i]; ss += v * v; }
    }
    ss = block_sum(ss, scratch);
    float inv = 1.0f / sqrtf(ss / (float)E + eps);
    if (VEC) {
        const float4 *x4 = (const float4 *)xi, *w4 = (const float4 *)w;
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
            float4 v = x4[i], g = w4[i];
            store4<TO>(o + 4 * i, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = from_f32<TO>(xi[i] * inv * w[i]);
    }
}

extern "C" int fg_rmsnorm(const float *x, const float *w, const int *rows, void *out, int out_dtype,
                          int R, int E, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    bool vec = E % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
    int per = vec ? E / 4 : E;
    int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    if (out_dtype == FG_F32) {
        if (vec) return fg_launch(rmsnorm_kernel<float, true>, dim3(R), dim3(threads), 0, stream, x, w, rows, (float *)out, E, eps);
        return fg_launch(rmsnorm_kernel<float, false>, dim3(R), dim3(threads), 0, stream, x, w, rows, (float *)out, E, eps);
    } else if (out_dtype == FG_BF16) {
        if (vec) return fg_launch(rmsnorm_kernel<bf16, true>, dim3(R), dim3(threads), 0, stream, x, w, rows, (bf16 *)out, E, eps);
        return fg_launch(rmsnorm_kernel<bf16, false>, dim3(R), dim3(threads), 0, stream, x, w, rows, (bf16 *)out, E, eps);
    }
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ RoPE + cache append
// qkv: [M, ld] rows of (q heads | k heads | v heads).  q is rotated in place; k is rotated and
// written, v copied, into the sequence's page at the row's position.  Pairs are (j, j + hd/2).
// cos/sin: [max_pos, hd/2] f32, built on the host in double.  Page pools: [n_pages, KV, P, hd].
template <typename T>
__global__ void rope_append_kernel(T *__restrict__ qkv, int ld, const int *__restrict__ positions,
                                   const int *__restrict__ row_seq, const int *__restrict__ block_table,
                                   int table_width, T *__restrict__ k_pool, T *__restrict__ v_pool,
                                   const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                   int H, int KV, int hd, int page_size, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    int m = blockIdx.x;
    int pos = positions[m];
    int half = hd >> 1;
    T *row = qkv + (size_t)m * ld;
    const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
    // q heads
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        int h = i / half, j = i - h * half;
        T *p = row + h * hd;
        float a = to_f32<T>(p[j]), b = to_f32<T>(p[j + half]);
        float c = cs[j], s = sn[j];
        p[j] = from_f32<T>(a * c - b * s);
        p[j + half] = from_f32<T>(a * s + b * c);
    }
    if (!write_kv) return;
    int page = block_table[(size_t)row_seq[m] * table_width + pos / page_size];
    int off = pos % page_size;
    const T *krow = row + H * hd, *vrow = krow + KV * hd;
    for (int i = threadIdx.x; i < KV * half; i += blockDim.x) {
        int h = i / half, j = i - h * half;
        const T *p = krow + h * hd;
        float a = to_f32<T>(p[j]), b = to_f32<T>(p[j + half]);
        float c = cs[j], s = sn[j];
        T *dst = k_pool + (((size_t)page * KV + h) * page_size + off) * hd;
        dst[j] = from_f32<T>(a * c - b * s);
        dst[j + half] = from_f32<T>(a * s + b * c);
    }
    for (int i = threadIdx.x; i < KV * hd; i += blockDim.x) {
        int h = i / hd, d = i - h * hd;
        v_pool[(((size_t)page * KV + h) * page_size + off) * hd + d] = vrow[i];
    }
}

// bf16 rows with head sizes that are multiples of 16: eight pairs (two 16-byte loads) a thread
__global__ void rope_append_vec_kernel(bf16 *__restrict__ qkv, int ld, const int *__restrict__ positions,
                                       const int *__restrict__ row_seq, const int *__restrict__ block_table,
                                       int table_width, bf16 *__restrict__ k_pool, bf16 *__restrict__ v_pool,
                                       const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                       int H, int KV, int hd, int page_size, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, pos = positions[m], half = hd >> 1, cph = half >> 3;   // chunks of 8 pairs per head
    bf16 *row = qkv + (size_t)m * ld;
    const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
    size_t kv_base = 0;
    if (write_kv) {
        int page = block_table[(size_t)row_seq[m] * table_width + pos / page_size];
        kv_base = ((size_t)page * KV * page_size + pos % page_size) * hd;              // + h * page_size * hd
    }
    const int n_rot = (H + (write_kv ? KV : 0)) * cph;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        int h = i / cph, j0 = (i - h * cph) * 8;
        const bf16 *src = row + (size_t)h * hd;                                         // k heads follow the q heads
        uint4 lo = *(const uint4 *)(src + j0), hi = *(const uint4 *)(src + j0 + half);
        float4 c0 = *(const float4 *)(cs + j0), c1 = *(const float4 *)(cs + j0 + 4);
        float4 s0 = *(const float4 *)(sn + j0), s1 = *(const float4 *)(sn + j0 + 4);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const __nv_bfloat162 *lp = (const __nv_bfloat162 *)&lo, *hp = (const __nv_bfloat162 *)&hi;
        uint4 olo, ohi;
        __nv_bfloat162 *ol = (__nv_bfloat162 *)&olo, *oh = (__nv_bfloat162 *)&ohi;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float2 a = __bfloat1622float2(lp[e]), b = __bfloat1622float2(hp[e]);
            ol[e] = __floats2bfloat162_rn(a.x * c[2 * e] - b.x * sv[2 * e], a.y * c[2 * e + 1] - b.y * sv[2 * e + 1]);
            oh[e] = __floats2bfloat162_rn(a.x * sv[2 * e] + b.x * c[2 * e], a.y * sv[2 * e + 1] + b.y * c[2 * e + 1]);
        }
        bf16 *dst = h < H ? row + (size_t)h * hd : k_pool + kv_base + (size_t)(h - H) * page_size * hd;
        *(uint4 *)(dst + j0) = olo;
        *(uint4 *)(dst + j0 + half) = ohi;
    }
    if (!write_kv) return;
    const bf16 *vrow = row + (size_t)(H + KV) * hd;
    for (int i = threadIdx.x; i < KV * (hd >> 3); i += blockDim.x) {
        int h = i / (hd >> 3), d0 = (i - h * (hd >> 3)) * 8;
        *(uint4 *)(v_pool + kv_base + (size_t)h * page_size * hd + d0) = *(const uint4 *)(vrow + (size_t)h * hd + d0);
    }
}

extern "C" int fg_rope_append(void *qkv, int dtype, int ld, const int *positions, const int *row_seq,
                              const int *block_table, int table_width, void *k_pool, void *v_pool,
                              const float *cos_t, const float *sin_t, int M, int H, int KV, int hd,
                              int page_size, int write_kv, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (hd % 2) return FG_ERR_BAD_SIZE;
    int work = H * hd / 2;
    int threads = work >= 1024 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == FG_BF16 && hd % 16 == 0 && ld % 8 == 0 && ((uintptr_t)qkv & 15) == 0 &&
        (!write_kv || ((((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0))) {
        int items = (H + KV) * (hd / 16);
        return fg_launch(rope_append_vec_kernel, dim3(M), dim3(items >= 256 ? 256 : (items >= 128 ? 128 : 64)), 0, stream,
                         (bf16 *)qkv, ld, positions, row_seq, block_table, table_width, (bf16 *)k_pool, (bf16 *)v_pool,
                         cos_t, sin_t, H, KV, hd, page_size, write_kv);
    }
    if (dtype == FG_F32)
        return fg_launch(rope_append_kernel<float>, dim3(M), dim3(threads), 0, stream, (float *)qkv, ld, positions, row_seq, block_table,
            table_width, (float *)k_pool, (float *)v_pool, cos_t, sin_t, H, KV, hd, page_size, write_kv);
    else if (dtype == FG_BF16)
        return fg_launch(rope_append_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (bf16 *)qkv, ld, positions, row_seq, block_table,
            table_width, (bf16 *)k_pool, (bf16 *)v_pool, cos_t, sin_t, H, KV, hd, page_size, write_kv);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ cache append without rotation
// For mixers whose scores do not depend on positions, and whose values may be of another size than their
// keys: k heads [KV, hd] and v heads [KV, hdv] of each row are copied to the row's place in its page.
// qkv rows: (q heads | k heads | v heads).  Pools: k [n_pages, KV, P, hd], v [n_pages, KV, P, hdv].
template <typename T>
__global__ void kv_append_kernel(const T *__restrict__ qkv, int ld, int k_off, const int *__restrict__ positions,
                                 const int *__restrict__ row_seq, const int *__restrict__ block_table, int table_width,
                                 T *__restrict__ k_pool, T *__restrict__ v_pool, int KV, int hd, int hdv, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, pos = positions[m];
    const int page = block_table[(size_t)row_seq[m] * table_width + pos / page_size], off = pos % page_size;
    const T *krow = qkv + (size_t)m * ld + k_off, *vrow = krow + (size_t)KV * hd;
    for (int i = threadIdx.x; i < KV * hd; i += blockDim.x) {
        int h = i / hd, d = i - h * hd;
        k_pool[(((size_t)page * KV + h) * page_size + off) * hd + d] = krow[i];
    }
    for (int i = threadIdx.x; i < KV * hdv; i += blockDim.x) {
        int h = i / hdv, d = i - h * hdv;
        v_pool[(((size_t)page * KV + h) * page_size + off) * hdv + d] = vrow[i];
    }
}

extern "C" int fg_kv_append(const void *qkv, int dtype, int ld, int k_off, const int *positions, const int *row_seq,
                            const int *block_table, int table_width, void *k_pool, void *v_pool, int M, int KV, int hd,
                            int hdv, int page_size, cudaStream_t stream) {
    if (M <= 0) return 0;
    int work = KV * (hd > hdv ? hd : hdv);
    int threads = work >= 1024 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == FG_F32)
        return fg_launch(kv_append_kernel<float>, dim3(M), dim3(threads), 0, stream, (const float *)qkv, ld, k_off, positions, row_seq,
                         block_table, table_width, (float *)k_pool, (float *)v_pool, KV, hd, hdv, page_size);
    if (dtype == FG_BF16)
        return fg_launch(kv_append_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (const bf16 *)qkv, ld, k_off, positions, row_seq,
                         block_table, table_width, (bf16 *)k_pool, (bf16 *)v_pool, KV, hd, hdv, page_size);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ norm of a sublayer's output, residual add, next norm
// For blocks that normalise a sublayer's output before adding it: x[m] += t[m] / rms(t[m]) * w_post, and,
// when w_next is given, out[m] = x[m] / rms(x[m]) * w_next for the sublayer that reads x next - one pass over
// the row instead of three kernels.  Statistics and the sum are 32-bit; one block a row, fixed reduction order.
// VEC: rows are read and written four elements at a time (E % 4 == 0, 16-byte aligned rows)
template <typename TO, bool VEC>
__global__ void norm_add_norm_kernel(const float *__restrict__ t, const float *__restrict__ w_post, float *__restrict__ x,
                                     const float *__restrict__ w_next, TO *__restrict__ out, int E, float eps_post,
                                     float eps_next) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float row[];        // [E] the updated residual row, when a next norm is wanted
    pdl_launch_dependents_small_step(gridDim.x);
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * E;
    float ss = 0.f;
    if (VEC) {
        const float4 *t4 = (const float4 *)(t + base);
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) { float4 v = t4[i]; ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w; }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) { float v = t[base + i]; ss += v * v; }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)E + eps_post);
    float ss2 = 0.f;
    if (VEC) {
        const float4 *t4 = (const float4 *)(t + base), *w4 = (const float4 *)w_post;
        float4 *x4 = (float4 *)(x + base), *r4 = (float4 *)row;
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
            float4 a = t4[i], g = w4[i], v = x4[i];
            v.x += a.x * inv * g.x; v.y += a.y * inv * g.y; v.z += a.z * inv * g.z; v.w += a.w * inv * g.w;
            x4[i] = v;
            if (w_next) { r4[i] = v; ss2 += v.x * v.x; ss2 += v.y * v.y; ss2 += v.z * v.z; ss2 += v.w * v.w; }
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float v = x[base + i] + t[base + i] * inv * w_post[i];
            x[base + i] = v;
            if (w_next) { row[i] = v; ss2 += v * v; }
        }
    }
    if (!w_next) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)E + eps_next);
    if (VEC) {
        const float4 *r4 = (const float4 *)row, *w4 = (const float4 *)w_next;
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
            float4 v = r4[i], g = w4[i];
            store4<TO>(out + base + 4 * i, v.x * inv2 * g.x, v.y * inv2 * g.y, v.z * inv2 * g.z, v.w * inv2 * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) out[base + i] = from_f32<TO>(row[i] * inv2 * w_next[i]);
    }
}

extern "C" int fg_norm_add_norm(const float *t, const float *w_post, float *x, const float *w_next, void *out, int out_dtype,
                                int M, int E, float eps_post, float eps_next, cudaStream_t stream) {
    if (M <= 0) return 0;
    size_t smem = w_next ? (size_t)E * sizeof(float) : 0;
    if (smem > 48 * 1024) return FG_ERR_BAD_SIZE;
    const bool vec = E % 4 == 0 && ((((uintptr_t)t) | ((uintptr_t)w_post) | ((uintptr_t)x) | ((uintptr_t)w_next) | ((uintptr_t)out)) & 15) == 0;
    int per = vec ? E / 4 : E;
    int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    const bool wide = out_dtype == FG_F32 || !w_next;
    if (!wide && out_dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
#define NAN_LAUNCH(TO, VEC) fg_launch(norm_add_norm_kernel<TO, VEC>, dim3(M), dim3(threads), smem, stream, t, w_post, x, w_next, (TO *)out, E, \
                                      eps_post, eps_next)
    if (wide) return vec ? NAN_LAUNCH(float, true) : NAN_LAUNCH(float, false);
    return vec ? NAN_LAUNCH(bf16, true) : NAN_LAUNCH(bf16, false);
#undef NAN_LAUNCH
}

// ------------------------------------------------------------------ two mixers side by side
// out (+)= scale_a * f_a(a) + scale_b * f_b(b) over float32 rows [M, E], f(t) = t / sqrt(mean(t^2) + eps) * w where a weight is
// given and t itself where it is not.  One block a row; statistics and the sum are 32-bit, fixed reduction order.
__global__ void pair_combine_kernel(const float *__restrict__ a, const float *__restrict__ b, const float *__restrict__ w_a,
                                    const float *__restrict__ w_b, float scale_a, float scale_b, float eps, float *__restrict__ out,
                                    int E, int accumulate) {
    __shared__ float scratch[32];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * E;
    float inv_a = 1.f, inv_b = 1.f;
    if (w_a) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) { const float v = a[base + i]; ss = fmaf(v, v, ss); }
        inv_a = 1.0f / sqrtf(block_sum(ss, scratch) / (float)E + eps);
    }
    if (w_b) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) { const float v = b[base + i]; ss = fmaf(v, v, ss); }
        inv_b = 1.0f / sqrtf(block_sum(ss, scratch) / (float)E + eps);
    }
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float ta = w_a ? a[base + i] * inv_a * w_a[i] : a[base + i], tb = w_b ? b[base + i] * inv_b * w_b[i] : b[base + i];
        const float v = fmaf(scale_a, ta, scale_b * tb);
        out[base + i] = accumulate ? out[base + i] + v : v;
    }
}

extern "C" int fg_pair_combine(const float *a, const float *b, const float *w_a, const float *w_b, float scale_a, float scale_b,
                               float eps, float *out, int M, int E, int accumulate, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (E <= 0) return FG_ERR_BAD_SIZE;
    const int threads = E >= 2048 ? 256 : 128;
    return fg_launch(pair_combine_kernel, dim3(M), dim3(threads), 0, stream, a, b, w_a, w_b, scale_a, scale_b, eps, out, E, accumulate);
}

// ------------------------------------------------------------------ activations in place
// kind 0: relu(z)^2.  In f32; the result is stored in the buffer's dtype.
template <typename T>
__global__ void activation_kernel(T *__restrict__ z, size_t total, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        float v = to_f32<T>(z[i]);
        v = v > 0.f ? v * v : 0.f;
        z[i] = from_f32<T>(v);
    }
}

extern "C" int fg_activation(void *z, int dtype, long long total, int kind, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (kind != 0) return FG_ERR_BAD_SIZE;
    size_t want = ((size_t)total + 255) / 256;
    int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    if (dtype == FG_F32) return fg_launch(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float *)z, (size_t)total, kind);
    if (dtype == FG_BF16) return fg_launch(activation_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16 *)z, (size_t)total, kind);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ soft cap of logits
// z <- cap * tanh(z / cap), in place on float32 logits [R, V] with row stride ld.
__global__ void softcap_kernel(float *__restrict__ z, int V, int ld, size_t total, float cap, float inv_cap) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        size_t r = i / V;
        float *p = z + r * ld + (i - r * V);
        *p = cap * tanhf(*p * inv_cap);
    }
}

extern "C" int fg_softcap(float *logits, int R, int V, int ld, float cap, cudaStream_t stream) {
    size_t total = (size_t)R * V;
    if (total == 0) return 0;
    if (!(cap > 0.f)) return FG_ERR_BAD_SIZE;
    size_t want = (total + 255) / 256;
    int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    return fg_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, logits, V, ld, total, cap, 1.0f / cap);
}

// ------------------------------------------------------------------ SiLU(g) * u
// gu: [M, 2F] rows of (gate | up); out: [M, F].
template <typename T>
__global__ void silu_mul_kernel(const T *__restrict__ gu, T *__restrict__ out, size_t total, int F) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        size_t m = i / F;
        int f = (int)(i - m * F);
        float g = to_f32<T>(gu[m * 2 * F + f]), u = to_f32<T>(gu[m * 2 * F + F + f]);
        out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

extern "C" int fg_silu_mul(const void *gu, void *out, int dtype, int M, int F, cudaStream_t stream) {
    size_t total = (size_t)M * F;
    if (total == 0) return 0;
    int threads = 256;
    size_t want = (total + threads - 1) / threads;
    int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    if (dtype == FG_F32)
        return fg_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *)gu, (float *)out, total, F);
    else if (dtype == FG_BF16)
        return fg_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (const bf16 *)gu, (bf16 *)out, total, F);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ decode feedback
// After a decode step of a fixed-shape (graph-replayed) batch: the sampled token of every row
// becomes its next input, and live rows move on by one position.
__global__ void decode_advance_kernel(int *__restrict__ tokens, int *__restrict__ positions,
                                      const int *__restrict__ next_tokens, const int *__restrict__ active, int B) {
    pdl_launch_dependents();
    pdl_wait();
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    tokens[b] = next_tokens[b];
    if (active[b]) positions[b] += 1;
}

extern "C" int fg_decode_advance(int *tokens, int *positions, const int *next_tokens, const int *active, int B,
                                 cudaStream_t stream) {
    if (B <= 0) return 0;
    return fg_launch(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, positions, next_tokens, active, B);
}

// ------------------------------------------------------------------ two float32 matrices side by side
// out[m, 0 .. E) = a[m, :], out[m, E .. 2 E) = b[m, :], in the contraction's input dtype
template <typename T>
__global__ void concat2_kernel(const float *__restrict__ a, int lda, const float *__restrict__ b, int ldb, T *__restrict__ out, int ldo,
                               size_t total, int E) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        size_t m = i / (2 * (size_t)E);
        int c = (int)(i - m * 2 * (size_t)E);
        out[m * ldo + c] = from_f32<T>(c < E ? a[m * lda + c] : b[m * ldb + c - E]);
    }
}

extern "C" int fg_concat2(const float *a, int lda, const float *b, int ldb, void *out, int out_dtype, int ldo, int M, int E,
                          cudaStream_t stream) {
    size_t total = (size_t)M * 2 * (size_t)E;
    if (total == 0) return 0;
    size_t want = (total + 255) / 256;
    int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    if (out_dtype == FG_F32) return fg_launch(concat2_kernel<float>, dim3(blocks), dim3(256), 0, stream, a, lda, b, ldb, (float *)out, ldo, total, E);
    if (out_dtype == FG_BF16) return fg_launch(concat2_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, a, lda, b, ldb, (bf16 *)out, ldo, total, E);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ two norms of the same rows
// Blocks whose two sublayers each normalise the SAME stream with a weight of their own: out_a = x / rms(x) * w_a and
// out_b = x / rms(x) * w_b (one statistic when the eps agree, which is the case the kernel is for; two otherwise), one pass
// over the row.  Statistics are 32-bit; one block a row, fixed reduction order.
template <typename TO>
__global__ void rmsnorm_pair_kernel(const float *__restrict__ x, const float *__restrict__ w_a, const float *__restrict__ w_b,
                                    TO *__restrict__ out_a, TO *__restrict__ out_b, int E, float eps_a, float eps_b, int vec) {
    __shared__ float scratch[32];
    // (no early release of the successor: this kernel stands between two tensor-memory contractions, and the second must not
    // start beside the first while this one sits resident and waiting; the successor starts when this kernel has finished)
    pdl_wait();
    const float *xi = x + (size_t)blockIdx.x * E;
    TO *oa = out_a + (size_t)blockIdx.x * E, *ob = out_b + (size_t)blockIdx.x * E;
    if (vec) {
        // four neighbours a thread and pass (16-byte loads of the row and of both weights); the order in which the squares are
        // added depends on E alone
        float ss = 0.f;
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4 *>(xi + i);
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        const float inv_a = 1.0f / sqrtf(ss / (float)E + eps_a), inv_b = 1.0f / sqrtf(ss / (float)E + eps_b);
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4 *>(xi + i);
            const float4 a = *reinterpret_cast<const float4 *>(w_a + i), b = *reinterpret_cast<const float4 *>(w_b + i);
            store4<TO>(oa + i, v.x * inv_a * a.x, v.y * inv_a * a.y, v.z * inv_a * a.z, v.w * inv_a * a.w);
            store4<TO>(ob + i, v.x * inv_b * b.x, v.y * inv_b * b.y, v.z * inv_b * b.z, v.w * inv_b * b.w);
        }
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) { float v = xi[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv_a = 1.0f / sqrtf(ss / (float)E + eps_a), inv_b = 1.0f / sqrtf(ss / (float)E + eps_b);
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float v = xi[i];
        oa[i] = from_f32<TO>(v * inv_a * w_a[i]);
        ob[i] = from_f32<TO>(v * inv_b * w_b[i]);
    }
}

extern "C" int fg_rmsnorm_pair(const float *x, const float *w_a, const float *w_b, void *out_a, void *out_b, int out_dtype, int R, int E,
                               float eps_a, float eps_b, cudaStream_t stream) {
    if (R <= 0) return 0;
    const int threads = E >= 4096 ? 512 : (E >= 1024 ? 256 : (E >= 256 ? 128 : 64));
    const int vec = (E % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)w_a) | ((uintptr_t)w_b) | ((uintptr_t)out_a) | ((uintptr_t)out_b)) & 15) == 0) ? 1 : 0;
    if (out_dtype == FG_F32)
        return fg_launch(rmsnorm_pair_kernel<float>, dim3(R), dim3(threads), 0, stream, x, w_a, w_b, (float *)out_a, (float *)out_b, E, eps_a, eps_b,
                         vec);
    if (out_dtype == FG_BF16)
        return fg_launch(rmsnorm_pair_kernel<bf16>, dim3(R), dim3(threads), 0, stream, x, w_a, w_b, (bf16 *)out_a, (bf16 *)out_b, E, eps_a, eps_b,
                         vec);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ the stream as a contraction's input
// out[m, c] = T(x[m, c]): the float32 stream itself (no norm) rounded to the activation dtype.
template <typename T>
__global__ void cast_rows_kernel(const float *__restrict__ x, int ldx, T *__restrict__ out, int ldo, size_t total, int E, int vec) {
    // (no early release of the successor: this kernel stands between two tensor-memory contractions, and the second must not
    // start beside the first while this one sits resident and waiting; the successor starts when this kernel has finished)
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (vec) {
        // four neighbours of a row a thread: one 16-byte load
        const size_t quads = total / 4;
        const int per_row = E / 4;
        for (; i < quads; i += stride) {
            const size_t m = i / (size_t)per_row;
            const int c = (int)(i - m * (size_t)per_row) * 4;
            const float4 v = *reinterpret_cast<const float4 *>(x + m * ldx + c);
            store4<T>(out + m * ldo + c, v.x, v.y, v.z, v.w);
        }
        return;
    }
    for (; i < total; i += stride) {
        const size_t m = i / (size_t)E;
        const int c = (int)(i - m * (size_t)E);
        out[m * ldo + c] = from_f32<T>(x[m * ldx + c]);
    }
}

extern "C" int fg_cast_rows(const float *x, int ldx, void *out, int out_dtype, int ldo, int M, int E, cudaStream_t stream) {
    const size_t total = (size_t)M * (size_t)E;
    if (total == 0) return 0;
    const int vec = (E % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)out)) & 15) == 0) ? 1 : 0;
    const size_t want = ((vec ? total / 4 : total) + 255) / 256;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    if (out_dtype == FG_F32) return fg_launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, ldx, (float *)out, ldo, total, E, vec);
    if (out_dtype == FG_BF16) return fg_launch(cast_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, ldx, (bf16 *)out, ldo, total, E, vec);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ gelu(z) * (a slice of a token's row of a table)
// out[m, j] = gelu_tanh(z[m, j]) * table[tokens[m], col0 + j], j < D, with
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).  z is float32; the product is formed in float32.
__device__ __forceinline__ float gelu_tanh_f32(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TT, typename TO>
__global__ void gelu_mul_gather_kernel(const float *__restrict__ z, int ldz, const TT *__restrict__ table, int ldt, int col0,
                                       const int *__restrict__ tokens, TO *__restrict__ out, int ldo, size_t total, int D) {
    // (no early release of the successor: this kernel stands between two tensor-memory contractions, and the second must not
    // start beside the first while this one sits resident and waiting; the successor starts when this kernel has finished)
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t m = i / (size_t)D;
        const int j = (int)(i - m * (size_t)D);
        const float e = to_f32<TT>(table[(size_t)tokens[m] * ldt + col0 + j]);
        out[m * ldo + j] = from_f32<TO>(gelu_tanh_f32(z[m * ldz + j]) * e);
    }
}

extern "C" int fg_gelu_mul_gather(const float *z, int ldz, const void *table, int table_dtype, int ldt, int col0, const int *tokens,
                                  void *out, int out_dtype, int ldo, int M, int D, cudaStream_t stream) {
    const size_t total = (size_t)M * (size_t)D;
    if (total == 0) return 0;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
#define GMG_LAUNCH(TT, TO) fg_launch(gelu_mul_gather_kernel<TT, TO>, dim3(blocks), dim3(256), 0, stream, z, ldz, (const TT *)table, ldt, col0, tokens, \
                                     (TO *)out, ldo, total, D)
    if (table_dtype == FG_F32 && out_dtype == FG_F32) return GMG_LAUNCH(float, float);
    if (table_dtype == FG_BF16 && out_dtype == FG_BF16) return GMG_LAUNCH(bf16, bf16);
    if (table_dtype == FG_F32 && out_dtype == FG_BF16) return GMG_LAUNCH(float, bf16);
    if (table_dtype == FG_BF16 && out_dtype == FG_F32) return GMG_LAUNCH(bf16, float);
#undef GMG_LAUNCH
    return FG_ERR_BAD_DTYPE;
}
