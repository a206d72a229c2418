// Latent attention: what runs on the cache of latents.
//
// The cache holds, per position, a latent c (R numbers, in the value pool) and a rotated key part (DR numbers, in the key
// pool); pages are [page][position in page][R] and [page][position in page][DR].  Every head's key is [W_uk[h] c | rotated
// part] and its value W_uv[h] c.
//
//   * fg_latent_decode: a step of single tokens (or any few rows), in the absorbed form - the caller has folded W_uk into
//     the query, so a query head is [q_abs (R) | q_rot (DR)], a score is q_abs . c + q_rot . rotated part, and the result is
//     sum_j p_j c_j per head (the caller applies W_uv).  One block per (row, group of up to 8 heads, split of the keys); a
//     warp takes a key at a time with its numbers spread over the lanes (one coalesced read of the latent serves the score
//     of every head of the group AND their weighted sums), running maximum and sum per head and warp; the warps' partial
//     results are merged in warp order, the splits' by a second kernel in split order.  A sink joins one warp's sum once.
//   * fg_latent_expand: a step of whole prompts (every sequence starts at its first token) runs as ordinary multi-head
//     attention on the tensor cores over keys and values expanded for the step's tokens only: this kernel lays q out as
//     [q_plain | rotated q_rot] per head and writes K = [W_uk c | rotated part] and V = [W_uv c | zeros] into pools of the
//     step's own pages [page][head][64][HQ], numbered by fg_seq_page_table.
//   * fg_gate_slice: out[m, h, 0 .. dv) = x[m, h, 0 .. dv) * sigmoid(gate[m, h, 0 .. dv)) out of heads of width HQ.
// Scores, softmax statistics and angles are 32-bit.
#include "common.cuh"

#define LAT_WARPS 8
#define LAT_HG 8                      // heads a block serves

// four consecutive numbers of a cache row
__device__ __forceinline__ void load4(const float *p, float (&v)[4]) { const float4 t = *(const float4 *)p; v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
__device__ __forceinline__ void load4(const bf16 *p, float (&v)[4]) {
    const uint2 t = *(const uint2 *)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162 *)&t.x, b = *(const __nv_bfloat162 *)&t.y;
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ float lat_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// A lane holds the numbers 4 lane + 128 i + (0 .. 3), i < NG, of a latent (R a multiple of 4, up to 128 NG) and 4 lane + (0 .. 3)
// of the rotated part (DR a multiple of 4, up to 128): cache rows are read as 8- or 16-byte pieces that a warp's lanes cover
// without a gap, and the query's numbers come from shared memory as 16-byte reads without a bank conflict.  The query is
// multiplied by scale * log2(e) when it is staged, so scores live in the base-2 domain; a row's running sums are rescaled only
// when its maximum moves.  The next key's row is on its way while this one is worked on.
template <typename T, int NG>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_decode_kernel(const T *__restrict__ q, int ldq, T *__restrict__ out, int ldo, const int *__restrict__ positions,
                     const int *__restrict__ row_seq, const int *__restrict__ block_table, int table_width, const T *__restrict__ k_pool,
                     const T *__restrict__ v_pool, int H, int R, int DR, int page_size, float scale, const float *__restrict__ sinks,
                     int n_splits, float *__restrict__ part) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_row = blockIdx.y, h0 = blockIdx.x * LAT_HG, split = blockIdx.z;
    const int nh = min(LAT_HG, H - h0);
    const int QD = R + DR;
    const float LOG2E_F = 1.4426950408889634f;
    float *qs = sm;                                   // [LAT_HG][QD], times scale * log2(e)
    float *merge = sm + LAT_HG * QD;                  // [LAT_WARPS][LAT_HG][R + 4]: rows stay 16-byte aligned
    const int pos = positions[m_row];
    const int *bt = block_table + (size_t)row_seq[m_row] * table_width;
    for (int e = threadIdx.x; e < LAT_HG * QD; e += LAT_WARPS * 32) {
        const int hh = e / QD, d = e - hh * QD;
        qs[e] = hh < nh ? to_f32<T>(q[(size_t)m_row * ldq + (size_t)(h0 + hh) * QD + d]) * (scale * LOG2E_F) : 0.f;
    }
    __syncthreads();
    float mx[LAT_HG], l[LAT_HG], acc[LAT_HG][NG][4];
#pragma unroll
    for (int hh = 0; hh < LAT_HG; hh++) {
        mx[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
        for (int i = 0; i < NG; i++) acc[hh][i][0] = acc[hh][i][1] = acc[hh][i][2] = acc[hh][i][3] = 0.f;
    }
    if (sinks && split == 0 && warp == 0) {
#pragma unroll
        for (int hh = 0; hh < LAT_HG; hh++)
            if (hh < nh) { mx[hh] = sinks[h0 + hh] * LOG2E_F; l[hh] = 1.f; }
    }
    const int stride = n_splits * LAT_WARPS;
    const bool rot_lane = 4 * lane < DR;
    float c[NG][4], kr[4], cn[NG][4], krn[4];
    auto fetch = [&](int key, float (&cc)[NG][4], float (&kk)[4]) {
        const size_t at = (size_t)bt[key / page_size] * page_size + key % page_size;
#pragma unroll
        for (int i = 0; i < NG; i++) {
            if (4 * lane + 128 * i < R) load4(v_pool + at * R + 4 * lane + 128 * i, cc[i]);
            else cc[i][0] = cc[i][1] = cc[i][2] = cc[i][3] = 0.f;
        }
        if (rot_lane) load4(k_pool + at * DR + 4 * lane, kk);
        else kk[0] = kk[1] = kk[2] = kk[3] = 0.f;
    };
    int key = split * LAT_WARPS + warp;
    if (key <= pos) fetch(key, cn, krn);
    for (; key <= pos; key += stride) {
#pragma unroll
        for (int i = 0; i < NG; i++)
#pragma unroll
            for (int e = 0; e < 4; e++) c[i][e] = cn[i][e];
#pragma unroll
        for (int e = 0; e < 4; e++) kr[e] = krn[e];
        if (key + stride <= pos) fetch(key + stride, cn, krn);
#pragma unroll
        for (int hh = 0; hh < LAT_HG; hh++) {
            if (hh >= nh) break;
            const float *qh = qs + hh * QD;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < NG; i++) {
                if (4 * lane + 128 * i < R) {
                    const float4 q4 = *(const float4 *)(qh + 4 * lane + 128 * i);
                    s = fmaf(q4.x, c[i][0], s); s = fmaf(q4.y, c[i][1], s); s = fmaf(q4.z, c[i][2], s); s = fmaf(q4.w, c[i][3], s);
                }
            }
            if (rot_lane) {
                const float4 q4 = *(const float4 *)(qh + R + 4 * lane);
                s = fmaf(q4.x, kr[0], s); s = fmaf(q4.y, kr[1], s); s = fmaf(q4.z, kr[2], s); s = fmaf(q4.w, kr[3], s);
            }
            s = warp_sum(s);
            if (s > mx[hh]) {                            // the same in every lane: the maximum moves, the sums follow
                const float corr = lat_ex2(mx[hh] - s);  // 0 at a warp's first key
                l[hh] *= corr;
#pragma unroll
                for (int i = 0; i < NG; i++)
#pragma unroll
                    for (int e = 0; e < 4; e++) acc[hh][i][e] *= corr;
                mx[hh] = s;
            }
            const float p = lat_ex2(s - mx[hh]);
            l[hh] += p;
#pragma unroll
            for (int i = 0; i < NG; i++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[hh][i][e] = fmaf(p, c[i][e], acc[hh][i][e]);
        }
    }
    // the warps' partial results, merged in warp order
#pragma unroll
    for (int hh = 0; hh < LAT_HG; hh++) {
        float *dst = merge + ((size_t)warp * LAT_HG + hh) * (R + 4);
#pragma unroll
        for (int i = 0; i < NG; i++)
            if (4 * lane + 128 * i < R) *(float4 *)(dst + 4 * lane + 128 * i) = make_float4(acc[hh][i][0], acc[hh][i][1], acc[hh][i][2], acc[hh][i][3]);
        if (lane == 0) { dst[R] = mx[hh]; dst[R + 1] = l[hh]; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nh * R; e += LAT_WARPS * 32) {
        const int hh = e / R, d = e - hh * R;
        float M = -INFINITY;
        for (int w = 0; w < LAT_WARPS; w++) M = fmaxf(M, merge[((size_t)w * LAT_HG + hh) * (R + 4) + R]);
        float L = 0.f, O = 0.f;
        for (int w = 0; w < LAT_WARPS; w++) {
            const float *src = merge + ((size_t)w * LAT_HG + hh) * (R + 4);
            const float wgt = src[R] == -INFINITY ? 0.f : lat_ex2(src[R] - M);
            L = fmaf(src[R + 1], wgt, L);
            O = fmaf(src[d], wgt, O);
        }
        if (n_splits == 1) {
            out[(size_t)m_row * ldo + (size_t)(h0 + hh) * R + d] = from_f32<T>(L > 0.f ? O / L : 0.f);
        } else {
            float *pr = part + (((size_t)m_row * H + h0 + hh) * n_splits + split) * (R + 2);
            pr[d] = O;
            if (d == 0) { pr[R] = M; pr[R + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------------------------- the same on the tensor cores
// bfloat16, pages of 64 positions, R a multiple of 64, DR a multiple of 16.  One block per (row, 16 heads, split of the
// PAGES); per page: (1) S = Q K^T, warp w the page's keys 8 w .. 8 w + 7 as m16n8k16 MMAs whose B operand - a key's numbers
// along k - is read straight from the cache rows; (2) the scores meet in shared memory, warp w runs the online softmax of
// rows 2 w and 2 w + 1 (running maximum and sum per row in shared memory) and leaves bfloat16 weights there; (3) O += P V,
// warp w the latent's columns w R / 8 .. , the B operand - two keys of one column - packed from 16-bit reads of the cache rows.
#define LM_WARPS 8
#define LM_HEADS 16
__device__ __forceinline__ void lat_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>                     // n-tiles of 8 latent columns a warp owns: R = 64 NT
__global__ void __launch_bounds__(LM_WARPS * 32)
latent_decode_mma_kernel(const bf16 *__restrict__ q, int ldq, bf16 *__restrict__ out, int ldo, const int *__restrict__ positions,
                         const int *__restrict__ row_seq, const int *__restrict__ block_table, int table_width, const bf16 *__restrict__ k_pool,
                         const bf16 *__restrict__ v_pool, int H, int DR, float scale_log2, const float *__restrict__ sinks, int n_splits,
                         float *__restrict__ part) {
    constexpr int R = 64 * NT, PG = 64;
    extern __shared__ __align__(16) uint8_t lm_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, cp = (lane & 3) * 2;
    const int m_row = blockIdx.y, h0 = blockIdx.x * LM_HEADS, split = blockIdx.z;
    const int nh = min(LM_HEADS, H - h0);
    const int QD = R + DR, QS = QD + 8, PS = PG + 8;
    bf16 *Qs = (bf16 *)lm_smem;                                   // [16][QS]
    bf16 *Ps = Qs + LM_HEADS * QS;                                // [16][PS]
    float *Ss = (float *)(Ps + LM_HEADS * PS);                    // [16][PG + 1]
    float *m_s = Ss + LM_HEADS * (PG + 1), *l_s = m_s + LM_HEADS, *corr_s = l_s + LM_HEADS;
    const int pos = positions[m_row];
    const int *bt = block_table + (size_t)row_seq[m_row] * table_width;
    for (int e = threadIdx.x; e < LM_HEADS * QD; e += LM_WARPS * 32) {
        const int hh = e / QD, d = e - hh * QD;
        Qs[hh * QS + d] = hh < nh ? q[(size_t)m_row * ldq + (size_t)(h0 + hh) * QD + d] : __float2bfloat16_rn(0.f);
    }
    if (threadIdx.x < LM_HEADS) {
        const bool sink = sinks && split == 0 && threadIdx.x < nh;
        m_s[threadIdx.x] = sink ? sinks[h0 + threadIdx.x] * 1.4426950408889634f : -INFINITY;
        l_s[threadIdx.x] = sink ? 1.f : 0.f;
    }
    __syncthreads();
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    const int last_page = pos / PG;
    for (int pg = split; pg <= last_page; pg += n_splits) {
        const size_t base = (size_t)bt[pg] * PG;
        // (1) scores of this warp's eight keys
        {
            const size_t at = base + 8 * warp + r;
            const bf16 *lat = v_pool + at * R, *rot = k_pool + at * DR;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int kc = 0; kc < QD; kc += 16) {
                const bf16 *qa = Qs + r * QS + kc + cp;
                const uint32_t a0 = *(const uint32_t *)qa, a1 = *(const uint32_t *)(qa + 8 * QS), a2 = *(const uint32_t *)(qa + 8),
                               a3 = *(const uint32_t *)(qa + 8 * QS + 8);
                const bf16 *kb = (kc < R ? lat + kc : rot + (kc - R)) + cp;
                lat_mma(c, a0, a1, a2, a3, *(const uint32_t *)kb, *(const uint32_t *)(kb + 8));
            }
            const int col = 8 * warp + cp, key = pg * PG + col;
            Ss[r * (PG + 1) + col] = key <= pos ? c[0] * scale_log2 : -INFINITY;
            Ss[r * (PG + 1) + col + 1] = key + 1 <= pos ? c[1] * scale_log2 : -INFINITY;
            Ss[(r + 8) * (PG + 1) + col] = key <= pos ? c[2] * scale_log2 : -INFINITY;
            Ss[(r + 8) * (PG + 1) + col + 1] = key + 1 <= pos ? c[3] * scale_log2 : -INFINITY;
        }
        __syncthreads();
        // (2) online softmax of rows 2 warp, 2 warp + 1
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int row = 2 * warp + k;
            const float v0 = Ss[row * (PG + 1) + lane], v1 = Ss[row * (PG + 1) + lane + 32];
            const float m_old = m_s[row], m_new = fmaxf(m_old, warp_max(fmaxf(v0, v1)));
            const float p0 = m_new == -INFINITY ? 0.f : lat_ex2(v0 - m_new), p1 = m_new == -INFINITY ? 0.f : lat_ex2(v1 - m_new);
            const float sum = warp_sum(p0 + p1);
            Ps[row * PS + lane] = __float2bfloat16_rn(p0);
            Ps[row * PS + lane + 32] = __float2bfloat16_rn(p1);
            __syncwarp();
            if (lane == 0) {
                const float corr = m_old == -INFINITY ? 0.f : lat_ex2(m_old - m_new);
                corr_s[row] = corr;
                l_s[row] = l_s[row] * corr + sum;
                m_s[row] = m_new;
            }
        }
        __syncthreads();
        // (3) O += P V on this warp's columns
        {
            const float c0 = corr_s[r], c1 = corr_s[r + 8];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { o[nt][0] *= c0; o[nt][1] *= c0; o[nt][2] *= c1; o[nt][3] *= c1; }
            const unsigned short *V = (const unsigned short *)(v_pool + base * R);
#pragma unroll
            for (int ks = 0; ks < PG; ks += 16) {
                const bf16 *pa = Ps + r * PS + ks + cp;
                const uint32_t a0 = *(const uint32_t *)pa, a1 = *(const uint32_t *)(pa + 8 * PS), a2 = *(const uint32_t *)(pa + 8),
                               a3 = *(const uint32_t *)(pa + 8 * PS + 8);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const unsigned short *vb = V + (size_t)(ks + cp) * R + warp * (R / 8) + nt * 8 + r;
                    const uint32_t b0 = (uint32_t)vb[0] | ((uint32_t)vb[R] << 16), b1 = (uint32_t)vb[8 * R] | ((uint32_t)vb[9 * R] << 16);
                    lat_mma(o[nt], a0, a1, a2, a3, b0, b1);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int row = r + 8 * k;
        if (row >= nh) continue;
        const float M = m_s[row], L = l_s[row];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int col = warp * (R / 8) + nt * 8 + cp;
            const float x0 = o[nt][2 * k], x1 = o[nt][2 * k + 1];
            if (n_splits == 1) {
                const float inv = L > 0.f ? 1.0f / L : 0.f;
                __nv_bfloat162 t = __floats2bfloat162_rn(x0 * inv, x1 * inv);
                *(uint32_t *)(out + (size_t)m_row * ldo + (size_t)(h0 + row) * R + col) = *(uint32_t *)&t;
            } else {
                float *pr = part + (((size_t)m_row * H + h0 + row) * n_splits + split) * (R + 2);
                pr[col] = x0; pr[col + 1] = x1;
                if (warp == 0 && nt == 0 && cp == 0) { pr[R] = M; pr[R + 1] = L; }
            }
        }
    }
}

template <typename T>
__global__ void latent_merge_kernel(const float *__restrict__ part, T *__restrict__ out, int ldo, int H, int R, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int m_row = blockIdx.y, h = blockIdx.x;
    const float *pr = part + ((size_t)m_row * H + h) * n_splits * (R + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, pr[(size_t)s * (R + 2) + R]);
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
        float L = 0.f, O = 0.f;
        for (int s = 0; s < n_splits; s++) {                 // split order
            const float *src = pr + (size_t)s * (R + 2);
            const float wgt = src[R] == -INFINITY ? 0.f : lat_ex2(src[R] - M);       // maxima are in the base-2 domain
            L = fmaf(src[R + 1], wgt, L);
            O = fmaf(src[d], wgt, O);
        }
        out[(size_t)m_row * ldo + (size_t)h * R + d] = from_f32<T>(L > 0.f ? O / L : 0.f);
    }
}

// table[s][i] = first page of sequence s in the step's own pools + i, for i < pages of s; sequences one after another
__global__ void seq_page_table_kernel(const int *__restrict__ cu_rows, int n_seq, int width, int page_size, int *__restrict__ table) {
    __shared__ int base[1025];
    // (only steps of whole prompts run this kernel, between two tensor-memory kernels: its successor is released when it ends)
    pdl_wait();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int s = 0; s < n_seq; s++) { base[s] = at; at += (cu_rows[s + 1] - cu_rows[s] + page_size - 1) / page_size; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_seq * width; e += blockDim.x) {
        const int s = e / width, i = e - s * width;
        const int n = (cu_rows[s + 1] - cu_rows[s] + page_size - 1) / page_size;
        table[e] = i < n ? base[s] + i : 0;
    }
}

// q: [M, H * (D + DR)] float32; kv: a row's [.. | rotated key part (DR, not yet rotated)] float32 at column rot_at;
// kp: [M, H * D] = W_uk c, vp: [M, H * DV] = W_uv c (bf16).  Writes qx [M, H * HQ] (HQ = D + DR) and the step's K and V pools.
__global__ void __launch_bounds__(256)
latent_expand_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ kv, int ldkv, int rot_at, const bf16 *__restrict__ kp,
                     int ldkp, const bf16 *__restrict__ vp, int ldvp, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                     int tbl_half, const int *__restrict__ positions, const int *__restrict__ row_seq, const int *__restrict__ table,
                     int width, bf16 *__restrict__ qx, bf16 *__restrict__ Kx, bf16 *__restrict__ Vx, int H, int D, int DR, int DV,
                     int page_size, int key_rotated) {
    __shared__ float krot[128];
    pdl_launch_dependents_small_step(gridDim.x);
    pdl_wait();
    const int m = blockIdx.x, HQ = D + DR;
    const int pos = positions[m];
    const float *cs = cos_t + (size_t)pos * tbl_half, *sn = sin_t + (size_t)pos * tbl_half;
    for (int i = threadIdx.x; i < DR / 2; i += blockDim.x) {
        const float a = kv[(size_t)m * ldkv + rot_at + 2 * i], b = kv[(size_t)m * ldkv + rot_at + 2 * i + 1];
        krot[2 * i] = key_rotated ? a : a * cs[i] - b * sn[i];          // (key_rotated: the part comes from a cache, rotated already)
        krot[2 * i + 1] = key_rotated ? b : b * cs[i] + a * sn[i];
    }
    __syncthreads();
    const size_t slot = (size_t)table[(size_t)row_seq[m] * width + pos / page_size];
    for (int e = threadIdx.x; e < H * HQ; e += blockDim.x) {
        const int h = e / HQ, d = e - h * HQ;
        const float *qh = q + (size_t)m * ldq + (size_t)h * HQ;
        float qv;
        if (d < D) qv = qh[d];
        else {
            const int i = (d - D) >> 1;
            const float a = qh[D + 2 * i], b = qh[D + 2 * i + 1];
            qv = ((d - D) & 1) ? b * cs[i] + a * sn[i] : a * cs[i] - b * sn[i];
        }
        qx[(size_t)m * H * HQ + e] = __float2bfloat16_rn(qv);
        const size_t at = ((slot * H + h) * page_size + pos % page_size) * HQ + d;
        Kx[at] = d < D ? kp[(size_t)m * ldkp + (size_t)h * D + d] : __float2bfloat16_rn(krot[d - D]);
        Vx[at] = d < DV ? vp[(size_t)m * ldvp + (size_t)h * DV + d] : __float2bfloat16_rn(0.f);
    }
}

template <typename T>
__global__ void gate_slice_kernel(const T *__restrict__ x, int ldx, int stride, const float *__restrict__ gate, int ldg, T *__restrict__ out,
                                  int ldo, int H, int DV) {
    pdl_wait();             // (stands between two tensor-memory kernels: its successor is released when it ends, not here)
    const int m = blockIdx.x;
    for (int e = threadIdx.x; e < H * DV; e += blockDim.x) {
        const int h = e / DV, d = e - h * DV;
        float v = to_f32<T>(x[(size_t)m * ldx + (size_t)h * stride + d]);
        if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + e]));
        out[(size_t)m * ldo + e] = from_f32<T>(v);
    }
}

static size_t latent_smem(int R, int DR) { return ((size_t)LAT_HG * (R + DR) + (size_t)LAT_WARPS * LAT_HG * (R + 4)) * sizeof(float); }

// floats of scratch `part` needs: rows * H * n_splits * (R + 2) (none with one split)
extern "C" long long fg_latent_decode_scratch_floats(int M, int H, int R, int n_splits) {
    return n_splits > 1 ? (long long)M * H * n_splits * (R + 2) : 0;
}

template <typename T, int NG>
static int launch_latent(const void *q, int ldq, void *out, int ldo, const int *positions, const int *row_seq, const int *block_table,
                         int table_width, const void *k_pool, const void *v_pool, int M, int H, int R, int DR, int page_size, float scale,
                         const float *sinks, int n_splits, float *part, cudaStream_t stream) {
    static FgPerDevice setup;
    const size_t smem = latent_smem(R, DR);
    if (fg_needs_setup(setup)) {
        cudaError_t e = cudaFuncSetAttribute(latent_decode_kernel<T, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    int code = fg_launch(latent_decode_kernel<T, NG>, dim3((H + LAT_HG - 1) / LAT_HG, M, n_splits), dim3(LAT_WARPS * 32), smem, stream, (const T *)q,
                         ldq, (T *)out, ldo, positions, row_seq, block_table, table_width, (const T *)k_pool, (const T *)v_pool, H, R, DR, page_size,
                         scale, sinks, n_splits, part);
    if (code || n_splits == 1) return code;
    return fg_launch(latent_merge_kernel<T>, dim3(H, M), dim3(128), 0, stream, (const float *)part, (T *)out, ldo, H, R, n_splits);
}

// q: [M, H * (R + DR)], out: [M, H * R], both of the cache's dtype.
extern "C" int fg_latent_decode(const void *q, int ldq, void *out, int ldo, int dtype, const int *positions, const int *row_seq,
                                const int *block_table, int table_width, const void *k_pool, const void *v_pool, int M, int H, int R,
                                int DR, int page_size, float scale, const float *sinks, int n_splits, float *part, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (H <= 0 || R <= 0 || R > 512 || R % 4 || DR <= 0 || DR > 128 || DR % 4 || n_splits < 1 || M > 65535 || n_splits > 65535) return FG_ERR_BAD_SIZE;
    if (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return FG_ERR_BAD_SIZE;
    if (n_splits > 1 && !part) return FG_ERR_BAD_SIZE;
    if (latent_smem(R, DR) > 200 * 1024) return FG_ERR_BAD_SIZE;
    const int ng = (R + 127) / 128;
#define LAT_RUN(T, NL) launch_latent<T, NL>(q, ldq, out, ldo, positions, row_seq, block_table, table_width, k_pool, v_pool, M, H, R, DR, page_size, \
                                             scale, sinks, n_splits, part, stream)
#define LAT_BY_SIZE(T) (ng <= 1 ? LAT_RUN(T, 1) : ng <= 2 ? LAT_RUN(T, 2) : ng <= 3 ? LAT_RUN(T, 3) : LAT_RUN(T, 4))
    if (dtype == FG_F32) return LAT_BY_SIZE(float);
    if (dtype == FG_BF16) return LAT_BY_SIZE(bf16);
#undef LAT_BY_SIZE
#undef LAT_RUN
    return FG_ERR_BAD_DTYPE;
}

static size_t latent_mma_smem(int R, int DR) {
    return (size_t)LM_HEADS * (R + DR + 8) * 2 + (size_t)LM_HEADS * (64 + 8) * 2 + (size_t)LM_HEADS * 65 * 4 + 3 * LM_HEADS * 4;
}

// 1 if the tensor-core form takes these sizes (bfloat16 only)
extern "C" int fg_latent_decode_mma_ok(int R, int DR, int page_size) { return page_size == 64 && R % 64 == 0 && R >= 64 && R <= 512 && DR % 16 == 0 && DR > 0; }

// q: [M, H * (R + DR)], out: [M, H * R] bfloat16; n_splits over the PAGES of a sequence; part as for fg_latent_decode
extern "C" int fg_latent_decode_mma(const void *q, int ldq, void *out, int ldo, const int *positions, const int *row_seq,
                                    const int *block_table, int table_width, const void *k_pool, const void *v_pool, int M, int H, int R,
                                    int DR, int page_size, float scale, const float *sinks, int n_splits, float *part, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!fg_latent_decode_mma_ok(R, DR, page_size) || H <= 0 || n_splits < 1 || M > 65535 || n_splits > 65535) return FG_ERR_BAD_SIZE;
    if ((n_splits > 1 && !part) || ldq % 2 || ldo % 2 || ((uintptr_t)q & 3) || ((uintptr_t)out & 3) || ((uintptr_t)k_pool & 3) || ((uintptr_t)v_pool & 3))
        return FG_ERR_BAD_SIZE;
    const size_t smem = latent_mma_smem(R, DR);
    const dim3 grid((H + LM_HEADS - 1) / LM_HEADS, M, n_splits);
    const float scale_log2 = scale * 1.4426950408889634f;
    int code = FG_ERR_BAD_SIZE;
#define LM_RUN(NT) code = fg_launch(latent_decode_mma_kernel<NT>, grid, dim3(LM_WARPS * 32), smem, stream, (const bf16 *)q, ldq, (bf16 *)out, ldo, \
                                    positions, row_seq, block_table, table_width, (const bf16 *)k_pool, (const bf16 *)v_pool, H, DR, scale_log2, sinks, \
                                    n_splits, part)
    switch (R / 64) {
        case 1: LM_RUN(1); break; case 2: LM_RUN(2); break; case 3: LM_RUN(3); break; case 4: LM_RUN(4); break;
        case 5: LM_RUN(5); break; case 6: LM_RUN(6); break; case 7: LM_RUN(7); break; case 8: LM_RUN(8); break;
    }
#undef LM_RUN
    if (code || n_splits == 1) return code;
    return fg_launch(latent_merge_kernel<bf16>, dim3(H, M), dim3(128), 0, stream, (const float *)part, (bf16 *)out, ldo, H, R, n_splits);
}

extern "C" int fg_seq_page_table(const int *cu_rows, int n_seq, int width, int page_size, int *table, cudaStream_t stream) {
    if (n_seq <= 0 || width <= 0) return 0;
    if (n_seq > 1024) return FG_ERR_BAD_SIZE;
    return fg_launch(seq_page_table_kernel, dim3(1), dim3(256), 0, stream, cu_rows, n_seq, width, page_size, table);
}

extern "C" int fg_latent_expand_ext(const float *q, int ldq, const float *kv, int ldkv, int rot_at, const void *kp, int ldkp, const void *vp,
                                int ldvp, const float *cos_t, const float *sin_t, int tbl_half, const int *positions, const int *row_seq,
                                const int *table, int width, void *qx, void *Kx, void *Vx, int M, int H, int D, int DR, int DV,
                                int page_size, int key_rotated, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (H <= 0 || D <= 0 || DR <= 0 || DR % 2 || DR > 128 || DV <= 0 || DV > D + DR || DR / 2 > tbl_half) return FG_ERR_BAD_SIZE;
    return fg_launch(latent_expand_kernel, dim3(M), dim3(256), 0, stream, q, ldq, kv, ldkv, rot_at, (const bf16 *)kp, ldkp, (const bf16 *)vp, ldvp,
                     cos_t, sin_t, tbl_half, positions, row_seq, table, width, (bf16 *)qx, (bf16 *)Kx, (bf16 *)Vx, H, D, DR, DV, page_size, key_rotated);
}

extern "C" int fg_latent_expand(const float *q, int ldq, const float *kv, int ldkv, int rot_at, const void *kp, int ldkp, const void *vp, int ldvp,
                                const float *cos_t, const float *sin_t, int tbl_half, const int *positions, const int *row_seq,
                                const int *table, int width, void *qx, void *Kx, void *Vx, int M, int H, int D, int DR, int DV,
                                int page_size, cudaStream_t stream) {
    return fg_latent_expand_ext(q, ldq, kv, ldkv, rot_at, kp, ldkp, vp, ldvp, cos_t, sin_t, tbl_half, positions, row_seq, table, width, qx, Kx, Vx, M,
                                H, D, DR, DV, page_size, 0, stream);
}

// A row's latent and rotated key part out of a cache of latents (one "head" a position: the rotated part in k_pool, the
// latent in v_pool): c_out [M, R] in the cache's dtype, kr_out [M, DR] float32.  For a layer that reads another layer's cache.
template <typename T>
__global__ void latent_fetch_kernel(const T *__restrict__ k_pool, const T *__restrict__ v_pool, const int *__restrict__ positions,
                                    const int *__restrict__ row_seq, const int *__restrict__ table, int width, int page_size,
                                    T *__restrict__ c_out, int ldc, float *__restrict__ kr_out, int ldk, int R, int DR) {
    pdl_wait();
    const int m = blockIdx.x, pos = positions[m];
    const size_t at = (size_t)table[(size_t)row_seq[m] * width + pos / page_size] * page_size + pos % page_size;
    for (int i = threadIdx.x; i < R; i += blockDim.x) c_out[(size_t)m * ldc + i] = v_pool[at * R + i];
    for (int i = threadIdx.x; i < DR; i += blockDim.x) kr_out[(size_t)m * ldk + i] = to_f32<T>(k_pool[at * DR + i]);
}

extern "C" int fg_latent_fetch(const void *k_pool, const void *v_pool, int dtype, const int *positions, const int *row_seq, const int *table,
                               int width, int page_size, void *c_out, int ldc, float *kr_out, int ldk, int M, int R, int DR, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (R <= 0 || DR <= 0) return FG_ERR_BAD_SIZE;
    if (dtype == FG_F32)
        return fg_launch(latent_fetch_kernel<float>, dim3(M), dim3(128), 0, stream, (const float *)k_pool, (const float *)v_pool, positions,
                                  row_seq, table, width, page_size, (float *)c_out, ldc, kr_out, ldk, R, DR);
    if (dtype == FG_BF16)
        return fg_launch(latent_fetch_kernel<bf16>, dim3(M), dim3(128), 0, stream, (const bf16 *)k_pool, (const bf16 *)v_pool, positions,
                                  row_seq, table, width, page_size, (bf16 *)c_out, ldc, kr_out, ldk, R, DR);
    return FG_ERR_BAD_DTYPE;
}

extern "C" int fg_gate_slice(const void *x, int ldx, int stride, const float *gate, int ldg, void *out, int ldo, int dtype, int M, int H,
                             int DV, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (H <= 0 || DV <= 0 || DV > stride) return FG_ERR_BAD_SIZE;
    if (dtype == FG_F32) return fg_launch(gate_slice_kernel<float>, dim3(M), dim3(256), 0, stream, (const float *)x, ldx, stride, gate, ldg, (float *)out, ldo, H, DV);
    if (dtype == FG_BF16) return fg_launch(gate_slice_kernel<bf16>, dim3(M), dim3(256), 0, stream, (const bf16 *)x, ldx, stride, gate, ldg, (bf16 *)out, ldo, H, DV);
    return FG_ERR_BAD_DTYPE;
}
