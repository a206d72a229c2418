// Attention over the paged cache for any head size and any dtype: the true 32-bit path and
// the any-size fallback.  One block per (token row, query head).
//
// Reference formulas (fastgguf.c): scores s_p = scale * (q . K[p]) for p in [lo, pos]
// (:3246, :3317), the mask is the loop range (:4782, :5030-5035), softmax with max
// subtraction (:3147-3156), o = sum_p w_p V[p] (:3320-3323); query head h uses KV head
// h / (H / KV) (:4781).  A window of w keeps only the last w positions (:4754-4758); a negative window -c is a chunked mask:
// a row sees the keys of its own run of c positions (runs counted from the sequence's first position) up to itself.
// keep_first > 0 adds the sequence's first keep_first positions to what a windowed row sees (they keep
// their places; a row sees each key once).  Values may have another size (hdv) than keys (hd).
// softcap c > 0: a score becomes c * tanh(score / c) after the scale.  sinks: one float per query head whose
// exponential joins the softmax's denominator - a key without a value; it is neither scaled nor capped.  The running
// maximum and sum simply start at (sink, 1) instead of (-inf, 0).
// latent != 0: the cache holds one small latent per position in v_pool (hdv numbers, which serve as the value as
// well) and a rotated key part in k_pool (hd numbers); a query row then has hdv + hd numbers a head, and a score is
// q[0:hdv] . latent + q[hdv:] . rotated part.  This is attention over keys and values that are linear maps of the
// latent, with the key map folded into the query and the value map applied to the output by the caller.
//
// Keys are visited in chunks of CHUNK visible keys, the kept first ones and then the window from lo, with a running maximum and
// sum in f32 (online softmax).  Within a chunk a thread scores whole keys; for the weighted sum of
// values the chunk's keys are dealt to the warps in equal runs, every lane owns output dimensions
// (lane, lane + 32, ...), and the warps' partial sums are added in warp order.  All of that depends
// only on the row's own position, so a row's result is the same whatever else is in the batch and
// however the tokens were cut into steps.
#include "common.cuh"

#define ATT_THREADS 256
#define ATT_WARPS (ATT_THREADS / 32)
#define MAX_DPL 16                    // output dimensions a lane owns at most: value sizes up to 512
#define CHUNK 1024

template <typename T, int DPL>          // DPL: output dimensions a lane owns (32 * DPL >= head size)
__global__ void __launch_bounds__(ATT_THREADS)
attention_generic_kernel(const T *__restrict__ q, int ldq, T *__restrict__ out, int ldo,
                         const int *__restrict__ positions, const int *__restrict__ row_seq,
                         const int *__restrict__ block_table, int table_width,
                         const T *__restrict__ k_pool, const T *__restrict__ v_pool,
                         int H, int KV, int hd, int hdv, int page_size, float scale, int window, int keep_first,
                         float softcap, const float *__restrict__ sinks, int latent) {
    extern __shared__ float smem[];
    const int qd = latent ? hdv + hd : hd;      // numbers a query head holds
    float *qs = smem;                 // [qd]
    float *sc = smem + qd;            // [CHUNK]
    __shared__ float scratch[32];
    int m = blockIdx.x, h = blockIdx.y;
    int kvh = h / (H / KV);
    int pos = positions[m];
    int lo = first_visible_key(pos, window);
    const int n_first = min(keep_first, lo);          // kept first keys that lie in front of the window
    const int n_keys = n_first + pos - lo + 1;        // visible key v is position v (v < n_first) or lo + v - n_first
    const int *bt = block_table + (size_t)row_seq[m] * table_width;
    const T *qrow = q + (size_t)m * ldq + (size_t)h * qd;
    for (int d = threadIdx.x; d < qd; d += ATT_THREADS) qs[d] = to_f32<T>(qrow[d]);
    const float *qk = latent ? qs + hdv : qs;   // the part of the query that meets k_pool
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *part = sc + CHUNK;         // [ATT_WARPS][hdv] partial value sums of a chunk
    float m_run = sinks ? sinks[h] : -INFINITY, l_run = sinks ? 1.f : 0.f;
    float acc[DPL];               // warp 0 keeps the running output: dims lane + 32 j
#pragma unroll
    for (int j = 0; j < DPL; j++) acc[j] = 0.f;
    for (int c0 = 0; c0 < n_keys; c0 += CHUNK) {
        int n = min(CHUNK, n_keys - c0);
        float cmax = -INFINITY;
        for (int i = threadIdx.x; i < n; i += ATT_THREADS) {
            int p = c0 + i < n_first ? c0 + i : lo + (c0 + i - n_first);
            const T *kr = k_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + p % page_size) * hd;
            float s = 0.f;
            if (sizeof(T) == 4 && (hd & 3) == 0) {
                // 16-byte loads along the key's row (rows of a pool start 16-byte aligned when hd is a multiple of 4)
                for (int d = 0; d < hd; d += 4) {
                    const float4 kv4 = *(const float4 *)((const float *)kr + d);
                    s = fmaf(qk[d], kv4.x, s);
                    s = fmaf(qk[d + 1], kv4.y, s);
                    s = fmaf(qk[d + 2], kv4.z, s);
                    s = fmaf(qk[d + 3], kv4.w, s);
                }
            } else {
                for (int d = 0; d < hd; d++) s = fmaf(qk[d], to_f32<T>(kr[d]), s);
            }
            if (latent) {
                const T *lr = v_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + p % page_size) * hdv;
                for (int d = 0; d < hdv; d++) s = fmaf(qs[d], to_f32<T>(lr[d]), s);
            }
            s *= scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            sc[i] = s;
            cmax = fmaxf(cmax, s);
        }
        cmax = block_max(cmax, scratch);
        float m_new = fmaxf(m_run, cmax);
        float csum = 0.f;
        for (int i = threadIdx.x; i < n; i += ATT_THREADS) {
            float e = expf(sc[i] - m_new);
            sc[i] = e;
            csum += e;
        }
        csum = block_sum(csum, scratch);   // its barriers also publish sc[] to every thread
        float corr = expf(m_run - m_new);  // 0 on the first chunk without a sink (m_run = -inf)
        l_run = l_run * corr + csum;
        // values: warp w takes keys [w * run, (w + 1) * run) of the chunk, page by page, eight rows in flight
        const int run = (n + ATT_WARPS - 1) / ATT_WARPS;
        const int i_end = min(n, (warp + 1) * run);
        float pv[DPL];
#pragma unroll
        for (int j = 0; j < DPL; j++) pv[j] = 0.f;
        for (int i = warp * run; i < i_end;) {
            const int vi = c0 + i;
            const int p = vi < n_first ? vi : lo + (vi - n_first), off = p % page_size;
            // a run of keys within one page, and within the kept first keys or within the window
            const int cnt = min(min(page_size - off, i_end - i), vi < n_first ? n_first - vi : i_end - i);
            const T *vr = v_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + off) * hdv;
            for (int u0 = 0; u0 < cnt; u0 += 8) {
                float v[8][DPL];
#pragma unroll
                for (int u = 0; u < 8; u++)
#pragma unroll
                    for (int j = 0; j < DPL; j++) {
                        const int d = lane + 32 * j;
                        v[u][j] = (u0 + u < cnt && d < hdv) ? to_f32<T>(vr[(size_t)(u0 + u) * hdv + d]) : 0.f;
                    }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    if (u0 + u >= cnt) break;
                    const float w = sc[i + u0 + u];
#pragma unroll
                    for (int j = 0; j < DPL; j++) pv[j] = fmaf(w, v[u][j], pv[j]);
                }
            }
            i += cnt;
        }
#pragma unroll
        for (int j = 0; j < DPL; j++)
            if (lane + 32 * j < hdv) part[warp * hdv + lane + 32 * j] = pv[j];
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < DPL; j++) {
                const int d = lane + 32 * j;
                if (d >= hdv) break;
                float t = 0.f;
                for (int w = 0; w < ATT_WARPS; w++) t += part[w * hdv + d];     // warp order
                acc[j] = acc[j] * corr + t;
            }
        }
        m_run = m_new;
        __syncthreads();                   // sc[] and part[] are rewritten by the next chunk
    }
    if (warp == 0) {
        T *orow = out + (size_t)m * ldo + (size_t)h * hdv;
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
        for (int j = 0; j < DPL; j++)
            if (lane + 32 * j < hdv) orow[lane + 32 * j] = from_f32<T>(acc[j] * inv);
    }
}

extern "C" int fg_attention_generic_ext(const void *q, int ldq, void *out, int ldo, int dtype,
                                        const int *positions, const int *row_seq, const int *block_table,
                                        int table_width, const void *k_pool, const void *v_pool,
                                        int M, int H, int KV, int hd, int hdv, int page_size, float scale, int window,
                                        int keep_first, float softcap, const float *sinks, int latent, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (hdv > 32 * MAX_DPL || hd <= 0 || hdv <= 0 || H % KV != 0 || H > 65535 || keep_first < 0 || softcap < 0.f) return FG_ERR_BAD_SIZE;
    dim3 grid(M, H);
    size_t smem = (size_t)((latent ? hd + hdv : hd) + CHUNK + ATT_WARPS * hdv) * sizeof(float);
    if (smem > 48 * 1024) return FG_ERR_BAD_SIZE;
#define ATT_LAUNCH(T, DPL) attention_generic_kernel<T, DPL><<<grid, ATT_THREADS, smem, stream>>>((const T *)q, ldq, (T *)out, ldo, \
        positions, row_seq, block_table, table_width, (const T *)k_pool, (const T *)v_pool, H, KV, hd, hdv, page_size, scale, window, \
        window > 0 ? keep_first : 0, softcap, sinks, latent)
#define ATT_BY_SIZE(T) do { if (hdv <= 64) ATT_LAUNCH(T, 2); else if (hdv <= 128) ATT_LAUNCH(T, 4); else if (hdv <= 256) ATT_LAUNCH(T, 8); \
                            else ATT_LAUNCH(T, 16); } while (0)
    if (dtype == FG_F32) ATT_BY_SIZE(float);
    else if (dtype == FG_BF16) ATT_BY_SIZE(bf16);
    else return FG_ERR_BAD_DTYPE;
#undef ATT_BY_SIZE
#undef ATT_LAUNCH
    return FG_LAUNCH_CHECK();
}

extern "C" int fg_attention_generic_kept(const void *q, int ldq, void *out, int ldo, int dtype,
                                         const int *positions, const int *row_seq, const int *block_table,
                                         int table_width, const void *k_pool, const void *v_pool,
                                         int M, int H, int KV, int hd, int hdv, int page_size, float scale, int window,
                                         int keep_first, cudaStream_t stream) {
    if (hd > 256 || hdv > 256) return FG_ERR_BAD_SIZE;
    return fg_attention_generic_ext(q, ldq, out, ldo, dtype, positions, row_seq, block_table, table_width, k_pool, v_pool, M, H, KV,
                                    hd, hdv, page_size, scale, window, keep_first, 0.f, nullptr, 0, stream);
}

extern "C" int fg_attention_generic(const void *q, int ldq, void *out, int ldo, int dtype,
                                    const int *positions, const int *row_seq, const int *block_table,
                                    int table_width, const void *k_pool, const void *v_pool,
                                    int M, int H, int KV, int hd, int page_size, float scale, int window,
                                    cudaStream_t stream) {
    return fg_attention_generic_kept(q, ldq, out, ldo, dtype, positions, row_seq, block_table, table_width, k_pool, v_pool, M, H, KV,
                                     hd, hd, page_size, scale, window, 0, stream);
}
