// What stands between an attention mixer's projections and its attention kernel when the mixer does more than rotate:
//
//   * fg_qkv_prepare: per token row, on the float32 projections q | k | v of a step - add the biases; run a short causal
//     convolution over time on every channel (y_t = sum_j w[c, j] u_(t - taps + 1 + j), zeros in front of the sequence; the
//     sequence's last taps - 1 inputs live in its state row between steps); normalise the WHOLE q and the whole k of the
//     token (x / sqrt(mean(x^2) + eps) * w over all heads at once); rotate the first rot_dims numbers of every head, members
//     (2i, 2i + 1) of a pair, by the token's position; write q for the attention kernel and append k and v to the paged
//     cache.  Every stage is optional (a null pointer or a zero size turns it off).  Sums, statistics and angles are 32-bit.
//   * fg_conv_state_update: after it, the sequences' new last taps - 1 inputs go to their state rows.
//   * fg_latent_append: a token's latent (normalised) goes to the value pool, its shared rotated key part to the key pool.
//   * fg_rope_pairs: rotation of adjacent pairs on a slice of every head, from one buffer into another.
//   * fg_rmsnorm_strided: RMS norm of float32 rows that are a slice of a wider matrix.
//   * fg_head_gemm: one small contraction per head, C[m, h, :] = A[m, h, :] W_h^T (or W_h), optionally times sigmoid(gate).
#include "common.cuh"

#define PREP_THREADS 256

// cos/sin: [positions, tbl_half] float32, column i = pair i.
template <typename T>
__global__ void __launch_bounds__(1024)
qkv_prepare_kernel(const float *__restrict__ proj, int ld, const float *__restrict__ bias, const float *__restrict__ conv_w, int taps,
                   const float *__restrict__ conv_state, const float *__restrict__ qn_w, const float *__restrict__ kn_w, float eps,
                   const float *__restrict__ cos_t, const float *__restrict__ sin_t, int tbl_half, int rot_dims,
                   const int *__restrict__ positions, const int *__restrict__ row_seq, const int *__restrict__ cu_rows,
                   const int *__restrict__ slots, const int *__restrict__ block_table, int table_width, T *__restrict__ q_out, int ldq,
                   T *__restrict__ k_pool, T *__restrict__ v_pool, int H, int KV, int hd, int hdv, int page_size, int norm_per_head,
                   int rot_halves) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents_small_step(gridDim.x);
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
    const int Cq = H * hd, Ck = KV * hd, C = Cq + Ck + KV * hdv;
    const int seq = row_seq[m], pos = positions[m];
    const int i_step = m - cu_rows[seq];                 // the token's index among the step's tokens of its sequence
    const float *mine = proj + (size_t)m * ld;
    if (conv_w) {
        const float *st = conv_state + (size_t)slots[seq] * (taps - 1) * C;
        for (int c = tid; c < C; c += nthr) {
            const float b = bias ? bias[c] : 0.f;
            float acc = 0.f;
            for (int j = 0; j < taps; j++) {
                const int back = taps - 1 - j;           // the input `back` tokens ago
                float u;
                if (back <= i_step) u = proj[(size_t)(m - back) * ld + c] + b;
                else u = st[(size_t)(taps - 1 - (back - i_step)) * C + c];      // from before this step (zeros before the sequence)
                acc = fmaf(conv_w[(size_t)c * taps + j], u, acc);
            }
            row[c] = acc;
        }
    } else {
        for (int c = tid; c < C; c += nthr) row[c] = mine[c] + (bias ? bias[c] : 0.f);
    }
    __syncthreads();
    if (qn_w && norm_per_head) {
        // every head of q and of k by itself: x / sqrt(mean(x^2) + eps) * w with ONE weight vector [hd] for all heads of q and
        // one for all heads of k; a warp takes a head, its lanes the head's numbers, the sum by a shuffle tree
        const int warp = tid >> 5, lane = tid & 31, n_warps = nthr >> 5;
        for (int head = warp; head < H + KV; head += n_warps) {
            float *p = row + (size_t)head * hd;
            const float *w = head < H ? qn_w : kn_w;
            float ss = 0.f;
            for (int d = lane; d < hd; d += 32) ss = fmaf(p[d], p[d], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
            for (int d = lane; d < hd; d += 32) p[d] = p[d] * inv * w[d];
        }
        __syncthreads();
    } else if (qn_w) {
        float sq = 0.f, sk = 0.f;
        for (int c = tid; c < Cq; c += nthr) sq = fmaf(row[c], row[c], sq);
        for (int c = tid; c < Ck; c += nthr) sk = fmaf(row[Cq + c], row[Cq + c], sk);
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        const float iq = 1.0f / sqrtf(sq / (float)Cq + eps), ik = 1.0f / sqrtf(sk / (float)Ck + eps);
        for (int c = tid; c < Cq; c += nthr) row[c] = row[c] * iq * qn_w[c];
        for (int c = tid; c < Ck; c += nthr) row[Cq + c] = row[Cq + c] * ik * kn_w[c];
        __syncthreads();
    }
    const int rh = rot_dims / 2;
    if (rh > 0) {
        const float *cs = cos_t + (size_t)pos * tbl_half, *sn = sin_t + (size_t)pos * tbl_half;
        for (int e = tid; e < (H + KV) * rh; e += nthr) {
            const int head = e / rh, i = e - head * rh;
            // q heads and k heads lie one after another, all of size hd; a pair is (2i, 2i + 1), or (i, i + rot_dims / 2)
            float *p = row + (size_t)head * hd + (rot_halves ? i : 2 * i);
            const int other = rot_halves ? rh : 1;
            const float a = p[0], b = p[other], c = cs[i], s = sn[i];
            p[0] = a * c - b * s;
            p[other] = b * c + a * s;
        }
        __syncthreads();
    }
    for (int c = tid; c < Cq; c += nthr) q_out[(size_t)m * ldq + c] = from_f32<T>(row[c]);
    if (k_pool) {
        const int page = block_table[(size_t)seq * table_width + pos / page_size], off = pos % page_size;
        for (int c = tid; c < Ck; c += nthr) {
            const int kvh = c / hd, d = c - kvh * hd;
            k_pool[(((size_t)page * KV + kvh) * page_size + off) * hd + d] = from_f32<T>(row[Cq + c]);
        }
        for (int c = tid; c < KV * hdv; c += nthr) {
            const int kvh = c / hdv, d = c - kvh * hdv;
            v_pool[(((size_t)page * KV + kvh) * page_size + off) * hdv + d] = from_f32<T>(row[Cq + Ck + c]);
        }
    }
}

// state[slot][j][c], j < taps - 1: the sequence's input (projection + bias) of taps - 1 - j tokens before its end
__global__ void conv_state_update_kernel(const float *__restrict__ proj, int ld, const float *__restrict__ bias, int taps,
                                         float *__restrict__ conv_state, const int *__restrict__ cu_rows, const int *__restrict__ slots,
                                         int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r0 = cu_rows[seq], n = cu_rows[seq + 1] - r0;
    if (n <= 0) return;
    float *st = conv_state + (size_t)slots[seq] * (taps - 1) * C;
    const float b = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps - 1; j++) {
        const int idx = n - (taps - 1) + j;              // index among the step's tokens
        // an older input moves up: it is read at j + n > j, before anything at or above it is written
        st[(size_t)j * C + c] = idx >= 0 ? proj[(size_t)(r0 + idx) * ld + c] + b : st[(size_t)(j + n) * C + c];
    }
}

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
latent_append_kernel(const float *__restrict__ kv, int ld, const float *__restrict__ norm_w, float eps, const float *__restrict__ cos_t,
                     const float *__restrict__ sin_t, int tbl_half, const int *__restrict__ positions, const int *__restrict__ row_seq,
                     const int *__restrict__ block_table, int table_width, T *__restrict__ k_pool, T *__restrict__ v_pool, int rank,
                     int rot_dim, int page_size) {
    __shared__ float scratch[32];
    pdl_launch_dependents_small_step(gridDim.x);
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[m];
    const int page = block_table[(size_t)row_seq[m] * table_width + pos / page_size], off = pos % page_size;
    const float *src = kv + (size_t)m * ld;
    float ss = 0.f;
    for (int c = tid; c < rank; c += PREP_THREADS) ss = fmaf(src[c], src[c], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    T *lat = v_pool + ((size_t)page * page_size + off) * rank;
    for (int c = tid; c < rank; c += PREP_THREADS) lat[c] = from_f32<T>(src[c] * inv * norm_w[c]);
    T *kr = k_pool + ((size_t)page * page_size + off) * rot_dim;
    const float *cs = cos_t + (size_t)pos * tbl_half, *sn = sin_t + (size_t)pos * tbl_half;
    for (int i = tid; i < rot_dim / 2; i += PREP_THREADS) {
        const float a = src[rank + 2 * i], b = src[rank + 2 * i + 1], c = cs[i], s = sn[i];
        kr[2 * i] = from_f32<T>(a * c - b * s);
        kr[2 * i + 1] = from_f32<T>(b * c + a * s);
    }
}

// out[m, h * out_stride + out_off + (0 .. dims)) = rotation of in[m, h * in_stride + in_off + (0 .. dims))
template <typename T>
__global__ void rope_pairs_kernel(const float *__restrict__ in, int ld_in, int in_stride, int in_off, T *__restrict__ out, int ld_out,
                                  int out_stride, int out_off, const int *__restrict__ positions, const float *__restrict__ cos_t,
                                  const float *__restrict__ sin_t, int tbl_half, int H, int dims) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, rh = dims / 2;
    const int pos = positions[m];
    const float *cs = cos_t + (size_t)pos * tbl_half, *sn = sin_t + (size_t)pos * tbl_half;
    for (int e = threadIdx.x; e < H * rh; e += blockDim.x) {
        const int h = e / rh, i = e - h * rh;
        const float *p = in + (size_t)m * ld_in + (size_t)h * in_stride + in_off + 2 * i;
        T *o = out + (size_t)m * ld_out + (size_t)h * out_stride + out_off + 2 * i;
        const float a = p[0], b = p[1], c = cs[i], s = sn[i];
        o[0] = from_f32<T>(a * c - b * s);
        o[1] = from_f32<T>(b * c + a * s);
    }
}

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
rmsnorm_strided_kernel(const float *__restrict__ x, int ldx, const float *__restrict__ w, T *__restrict__ out, int ldo, int E, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents_small_step(gridDim.x);
    pdl_wait();
    const float *src = x + (size_t)blockIdx.x * ldx;
    float ss = 0.f;
    for (int c = threadIdx.x; c < E; c += PREP_THREADS) ss = fmaf(src[c], src[c], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)E + eps);
    for (int c = threadIdx.x; c < E; c += PREP_THREADS) out[(size_t)blockIdx.x * ldo + c] = from_f32<T>(src[c] * inv * w[c]);
}

// C[m, h * c_stride + n] = sum_k A[m, h * a_stride + k] * W_h[n, k]; W_h[n, k] is w[(h * N + n) * ldw + k], or, transposed,
// w[(h * K + k) * ldw + n].  gate (float32, [M, ldg], column h * N + n): the result is multiplied by sigmoid(gate).
// 64 x 64 output tiles, 16 x 16 threads of 4 x 4 outputs, K in steps of 16; sums run along k in order.
#define HG_T 64
#define HG_K 16
__global__ void __launch_bounds__(256)
head_gemm_kernel(const void *__restrict__ A, int a_dtype, int lda, int a_stride, const void *__restrict__ W, int w_dtype, int ldw,
                 int transposed, void *__restrict__ Cm, int c_dtype, int ldc, int c_stride, const float *__restrict__ gate, int ldg, int M,
                 int N, int K) {
    __shared__ float As[HG_K][HG_T + 1], Ws[HG_K][HG_T + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z, m0 = blockIdx.y * HG_T, n0 = blockIdx.x * HG_T;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += HG_K) {
        for (int e = threadIdx.x; e < HG_T * HG_K; e += 256) {
            const int r = e / HG_K, k = e - r * HG_K;      // k fastest: rows of A and of W are read along k
            const int m = m0 + r, n = n0 + r;
            As[k][r] = (m < M && k0 + k < K) ? load_as(A, a_dtype, (size_t)m * lda + (size_t)h * a_stride + k0 + k) : 0.f;
            if (!transposed) Ws[k][r] = (n < N && k0 + k < K) ? load_as(W, w_dtype, ((size_t)h * N + n) * ldw + k0 + k) : 0.f;
        }
        if (transposed)
            for (int e = threadIdx.x; e < HG_T * HG_K; e += 256) {
                const int k = e / HG_T, r = e - k * HG_T;  // n fastest: a row of the stored matrix runs along n
                const int n = n0 + r;
                Ws[k][r] = (n < N && k0 + k < K) ? load_as(W, w_dtype, ((size_t)h * K + k0 + k) * ldw + n) : 0.f;
            }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HG_K; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m >= M || n >= N) continue;
            float v = acc[i][j];
            if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + (size_t)h * N + n]));
            store_as(Cm, c_dtype, (size_t)m * ldc + (size_t)h * c_stride + n, v);
        }
}

// The same contraction for a few rows (a decode step): every weight is read once, 16-byte or coalesced, for all rows.
// TRANSPOSED: a thread per output n (a stored row runs along n, so neighbouring threads read neighbouring numbers), sums along
// k in order; else a warp per output n with its lanes along k (a stored row runs along k) and a shuffle tree at the end.
#define HV_ROWS 16
template <bool TRANSPOSED>
__global__ void __launch_bounds__(256)
head_gemv_kernel(const void *__restrict__ A, int a_dtype, int lda, int a_stride, const void *__restrict__ W, int w_dtype, int ldw,
                 void *__restrict__ Cm, int c_dtype, int ldc, int c_stride, const float *__restrict__ gate, int ldg, int M, int N, int K) {
    extern __shared__ float as[];                       // [M][K]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    for (int e = threadIdx.x; e < M * K; e += 256) {
        const int m = e / K, k = e - m * K;
        as[e] = load_as(A, a_dtype, (size_t)m * lda + (size_t)h * a_stride + k);
    }
    __syncthreads();
    float acc[HV_ROWS];
#pragma unroll
    for (int m = 0; m < HV_ROWS; m++) acc[m] = 0.f;
    int n;
    if (TRANSPOSED) {
        n = blockIdx.x * 256 + threadIdx.x;
        if (n >= N) return;
        // sixteen weights are on their way before the first of them is used
        for (int k0 = 0; k0 < K; k0 += 16) {
            float w[16];
#pragma unroll
            for (int u = 0; u < 16; u++) w[u] = k0 + u < K ? load_as(W, w_dtype, ((size_t)h * K + k0 + u) * ldw + n) : 0.f;
#pragma unroll
            for (int u = 0; u < 16; u++) {
                if (k0 + u >= K) break;
#pragma unroll
                for (int m = 0; m < HV_ROWS; m++)
                    if (m < M) acc[m] = fmaf(as[m * K + k0 + u], w[u], acc[m]);
            }
        }
    } else {
        const int lane = threadIdx.x & 31;
        n = blockIdx.x * 8 + (threadIdx.x >> 5);
        if (n >= N) return;
        for (int k0 = lane; k0 < K; k0 += 256) {
            float w[8];
#pragma unroll
            for (int u = 0; u < 8; u++) w[u] = k0 + 32 * u < K ? load_as(W, w_dtype, ((size_t)h * N + n) * ldw + k0 + 32 * u) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (k0 + 32 * u >= K) break;
#pragma unroll
                for (int m = 0; m < HV_ROWS; m++)
                    if (m < M) acc[m] = fmaf(as[m * K + k0 + 32 * u], w[u], acc[m]);
            }
        }
#pragma unroll
        for (int m = 0; m < HV_ROWS; m++)
            if (m < M) acc[m] = warp_sum(acc[m]);
        if (lane != 0) return;
    }
#pragma unroll
    for (int m = 0; m < HV_ROWS; m++) {
        if (m >= M) break;
        float v = acc[m];
        if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + (size_t)h * N + n]));
        store_as(Cm, c_dtype, (size_t)m * ldc + (size_t)h * c_stride + n, v);
    }
}

// norm_per_head: the norm weights are [hd] and every head of q and of k is normalised by itself (else: [H * hd] / [KV * hd], the
// whole of q and of k at once); rot_halves: a rotated pair is (i, i + rot_dims / 2) of a head (else (2i, 2i + 1))
extern "C" int fg_qkv_prepare_ext(const float *proj, int ld, const float *bias, const float *conv_w, int taps, const float *conv_state,
                                  const float *qn_w, const float *kn_w, float eps, const float *cos_t, const float *sin_t, int tbl_half,
                                  int rot_dims, const int *positions, const int *row_seq, const int *cu_rows, const int *slots,
                                  const int *block_table, int table_width, void *q_out, int ldq, void *k_pool, void *v_pool, int dtype, int M,
                                  int H, int KV, int hd, int hdv, int page_size, int norm_per_head, int rot_halves, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (H <= 0 || KV <= 0 || hd <= 0 || hdv <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > hd || rot_dims / 2 > tbl_half) return FG_ERR_BAD_SIZE;
    if (conv_w && (taps < 1 || (taps > 1 && !conv_state))) return FG_ERR_BAD_SIZE;
    if ((qn_w == nullptr) != (kn_w == nullptr)) return FG_ERR_BAD_SIZE;
    const size_t smem = ((size_t)H * hd + (size_t)KV * (hd + hdv)) * sizeof(float);
    if (smem > 200 * 1024) return FG_ERR_BAD_SIZE;
    static FgPerDevice setup[2];
    if (smem > 48 * 1024 && fg_needs_setup(setup[dtype == FG_F32 ? 0 : 1])) {
        cudaError_t e = dtype == FG_F32 ? cudaFuncSetAttribute(qkv_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                        : cudaFuncSetAttribute(qkv_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    // few rows (a decode step) leave most of the GPU idle: a row's channels are then spread over more threads
    const int C_all = H * hd + KV * (hd + hdv);
    const int threads = (M < 64 && C_all >= 2048) ? 1024 : PREP_THREADS;
    if (dtype == FG_F32)
        return fg_launch(qkv_prepare_kernel<float>, dim3(M), dim3(threads), smem, stream, proj, ld, bias, conv_w, taps, conv_state, qn_w, kn_w,
                         eps, cos_t, sin_t, tbl_half, rot_dims, positions, row_seq, cu_rows, slots, block_table, table_width, (float *)q_out,
                         ldq, (float *)k_pool, (float *)v_pool, H, KV, hd, hdv, page_size, norm_per_head, rot_halves);
    if (dtype == FG_BF16)
        return fg_launch(qkv_prepare_kernel<bf16>, dim3(M), dim3(threads), smem, stream, proj, ld, bias, conv_w, taps, conv_state, qn_w, kn_w,
                         eps, cos_t, sin_t, tbl_half, rot_dims, positions, row_seq, cu_rows, slots, block_table, table_width, (bf16 *)q_out, ldq,
                         (bf16 *)k_pool, (bf16 *)v_pool, H, KV, hd, hdv, page_size, norm_per_head, rot_halves);
    return FG_ERR_BAD_DTYPE;
}

extern "C" int fg_qkv_prepare(const float *proj, int ld, const float *bias, const float *conv_w, int taps, const float *conv_state,
                              const float *qn_w, const float *kn_w, float eps, const float *cos_t, const float *sin_t, int tbl_half,
                              int rot_dims, const int *positions, const int *row_seq, const int *cu_rows, const int *slots,
                              const int *block_table, int table_width, void *q_out, int ldq, void *k_pool, void *v_pool, int dtype, int M,
                              int H, int KV, int hd, int hdv, int page_size, cudaStream_t stream) {
    return fg_qkv_prepare_ext(proj, ld, bias, conv_w, taps, conv_state, qn_w, kn_w, eps, cos_t, sin_t, tbl_half, rot_dims, positions, row_seq,
                              cu_rows, slots, block_table, table_width, q_out, ldq, k_pool, v_pool, dtype, M, H, KV, hd, hdv, page_size, 0, 0, stream);
}

// ------------------------------------------------------------------ a gate per head on the heads' outputs
// x[m, h * DV + j] *= sigmoid(gate[m, h]) in place (gate float32, one number a head and row; null: no gate), and `pad` columns
// behind the heads are set to (1, 0, 0, ...): with the output projection's bias stored as column H * DV of its matrix, the
// projection adds the bias in the same pass.
template <typename T>
__global__ void head_gate_kernel(T *__restrict__ x, int ldx, const float *__restrict__ gate, int ldg, int H, int DV, int pad, int vec) {
    extern __shared__ float head_gate_sig[];        // the row's H gates
    // (no early release of the successor: this kernel stands between two tensor-memory contractions, and the second must not
    // start beside the first while this one sits resident and waiting; the successor starts when this kernel has finished)
    pdl_wait();
    const int m = blockIdx.x;
    T *row = x + (size_t)m * ldx;
    if (gate) {
        for (int h = threadIdx.x; h < H; h += blockDim.x) head_gate_sig[h] = 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + h]));
        __syncthreads();
        if (vec) {
            // 16 bytes a thread; DV is a multiple of the run, so a run lies in one head
            constexpr int PER = 16 / sizeof(T);
            for (int e = threadIdx.x * PER; e < H * DV; e += blockDim.x * PER) {
                const float g = head_gate_sig[e / DV];
                uint4 raw = *reinterpret_cast<const uint4 *>(row + e);
                T *v = reinterpret_cast<T *>(&raw);
#pragma unroll
                for (int i = 0; i < PER; i++) v[i] = from_f32<T>(to_f32<T>(v[i]) * g);
                *reinterpret_cast<uint4 *>(row + e) = raw;
            }
        } else {
            for (int e = threadIdx.x; e < H * DV; e += blockDim.x) row[e] = from_f32<T>(to_f32<T>(row[e]) * head_gate_sig[e / DV]);
        }
    }
    for (int e = threadIdx.x; e < pad; e += blockDim.x) row[H * DV + e] = from_f32<T>(e == 0 ? 1.0f : 0.0f);
}

extern "C" int fg_head_gate(void *x, int ldx, int dtype, const float *gate, int ldg, int M, int H, int DV, int pad, cudaStream_t stream) {
    if (M <= 0 || (!gate && pad <= 0)) return 0;
    if (H * DV + pad > ldx || H > 8192) return FG_ERR_BAD_SIZE;
    const int threads = H * DV >= 4096 ? 256 : 128;
    const size_t smem = (size_t)H * sizeof(float);
    const int per = dtype == FG_F32 ? 4 : 8;
    const int vec = (DV % per == 0 && ldx % per == 0 && ((uintptr_t)x & 15) == 0) ? 1 : 0;
    if (dtype == FG_F32) return fg_launch(head_gate_kernel<float>, dim3(M), dim3(threads), smem, stream, (float *)x, ldx, gate, ldg, H, DV, pad, vec);
    if (dtype == FG_BF16) return fg_launch(head_gate_kernel<bf16>, dim3(M), dim3(threads), smem, stream, (bf16 *)x, ldx, gate, ldg, H, DV, pad, vec);
    return FG_ERR_BAD_DTYPE;
}

extern "C" int fg_conv_state_update(const float *proj, int ld, const float *bias, int taps, float *conv_state, const int *cu_rows,
                                    const int *slots, int n_seq, int C, cudaStream_t stream) {
    if (n_seq <= 0 || taps <= 1) return 0;
    if (C <= 0) return FG_ERR_BAD_SIZE;
    return fg_launch(conv_state_update_kernel, dim3(n_seq, (C + 255) / 256), dim3(256), 0, stream, proj, ld, bias, taps, conv_state, cu_rows, slots, C);
}

extern "C" int fg_latent_append(const float *kv, int ld, const float *norm_w, float eps, const float *cos_t, const float *sin_t, int tbl_half,
                                const int *positions, const int *row_seq, const int *block_table, int table_width, void *k_pool,
                                void *v_pool, int dtype, int M, int rank, int rot_dim, int page_size, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (rank <= 0 || rot_dim <= 0 || rot_dim % 2 || rot_dim / 2 > tbl_half) return FG_ERR_BAD_SIZE;
    if (dtype == FG_F32)
        return fg_launch(latent_append_kernel<float>, dim3(M), dim3(PREP_THREADS), 0, stream, kv, ld, norm_w, eps, cos_t, sin_t, tbl_half, positions,
                         row_seq, block_table, table_width, (float *)k_pool, (float *)v_pool, rank, rot_dim, page_size);
    if (dtype == FG_BF16)
        return fg_launch(latent_append_kernel<bf16>, dim3(M), dim3(PREP_THREADS), 0, stream, kv, ld, norm_w, eps, cos_t, sin_t, tbl_half, positions,
                         row_seq, block_table, table_width, (bf16 *)k_pool, (bf16 *)v_pool, rank, rot_dim, page_size);
    return FG_ERR_BAD_DTYPE;
}

extern "C" int fg_rope_pairs(const float *in, int ld_in, int in_stride, int in_off, void *out, int out_dtype, int ld_out, int out_stride,
                             int out_off, const int *positions, const float *cos_t, const float *sin_t, int tbl_half, int M, int H, int dims,
                             cudaStream_t stream) {
    if (M <= 0 || dims <= 0) return 0;
    if (dims % 2 || dims / 2 > tbl_half || H <= 0) return FG_ERR_BAD_SIZE;
    const int threads = H * dims / 2 >= 256 ? 256 : 64;
    if (out_dtype == FG_F32)
        return fg_launch(rope_pairs_kernel<float>, dim3(M), dim3(threads), 0, stream, in, ld_in, in_stride, in_off, (float *)out, ld_out, out_stride,
                         out_off, positions, cos_t, sin_t, tbl_half, H, dims);
    if (out_dtype == FG_BF16)
        return fg_launch(rope_pairs_kernel<bf16>, dim3(M), dim3(threads), 0, stream, in, ld_in, in_stride, in_off, (bf16 *)out, ld_out, out_stride,
                         out_off, positions, cos_t, sin_t, tbl_half, H, dims);
    return FG_ERR_BAD_DTYPE;
}

extern "C" int fg_rmsnorm_strided(const float *x, int ldx, const float *w, void *out, int out_dtype, int ldo, int R, int E, float eps,
                                  cudaStream_t stream) {
    if (R <= 0) return 0;
    if (E <= 0) return FG_ERR_BAD_SIZE;
    if (out_dtype == FG_F32) return fg_launch(rmsnorm_strided_kernel<float>, dim3(R), dim3(PREP_THREADS), 0, stream, x, ldx, w, (float *)out, ldo, E, eps);
    if (out_dtype == FG_BF16) return fg_launch(rmsnorm_strided_kernel<bf16>, dim3(R), dim3(PREP_THREADS), 0, stream, x, ldx, w, (bf16 *)out, ldo, E, eps);
    return FG_ERR_BAD_DTYPE;
}

extern "C" int fg_head_gemm(const void *A, int a_dtype, int lda, int a_stride, const void *W, int w_dtype, int ldw, int transposed, void *C,
                            int c_dtype, int ldc, int c_stride, const float *gate, int ldg, int M, int N, int K, int H, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || H <= 0) return 0;
    if (K <= 0 || H > 65535) return FG_ERR_BAD_SIZE;
    for (int d : {a_dtype, w_dtype, c_dtype})
        if (d != FG_F32 && d != FG_BF16) return FG_ERR_BAD_DTYPE;
    if (M <= HV_ROWS && (size_t)M * K * sizeof(float) <= 48 * 1024) {
        const size_t smem = (size_t)M * K * sizeof(float);
        if (transposed)
            return fg_launch(head_gemv_kernel<true>, dim3((N + 255) / 256, H), dim3(256), smem, stream, A, a_dtype, lda, a_stride, W, w_dtype, ldw, C,
                             c_dtype, ldc, c_stride, gate, ldg, M, N, K);
        return fg_launch(head_gemv_kernel<false>, dim3((N + 7) / 8, H), dim3(256), smem, stream, A, a_dtype, lda, a_stride, W, w_dtype, ldw, C, c_dtype,
                         ldc, c_stride, gate, ldg, M, N, K);
    }
    dim3 grid((N + HG_T - 1) / HG_T, (M + HG_T - 1) / HG_T, H);
    if (grid.y > 65535) return FG_ERR_BAD_SIZE;
    return fg_launch(head_gemm_kernel, grid, dim3(256), 0, stream, A, a_dtype, lda, a_stride, W, w_dtype, ldw, transposed, C, c_dtype, ldc, c_stride,
                     gate, ldg, M, N, K);
}
