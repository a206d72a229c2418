// Recurrent mixers whose state decays by ONE factor per head and token: the state-space form ("duality") and the gated
// delta rule, and what stands between their projections and the recurrence.
//
// Both are one recurrence over a state S [d, dv] per head, with a token's key k and query q (size d), value v (size dv),
// decay a in (0, 1], step b and a skip weight D:
//     S <- a S;   u = b (v - [delta] S^T k);   S <- S + k u^T;   o = S^T q + D v
//   state space:  k = B_t, q = C_t, v = x_t, b = dt_t = softplus(dt + bias), a = exp(-exp(A_log) dt_t), no delta term, D per head
//   delta rule:   k, q unit vectors (q also times d^-1/2), b = sigmoid(.), a = exp(-exp(A_log) softplus(. + bias)), D = 0
// Every column of S (one value channel) runs by itself: S[:, j] only meets v[j].  So a column belongs to R neighbouring
// lanes of a warp, lane r holding rows r, r + R, ... in registers; the two sums over rows are shuffles inside those R
// lanes and nothing else crosses threads.  A block stages TC tokens' k, q, v, a and b in shared memory, walks them without
// a barrier, and goes on to the next TC.  State, decays, steps and sums are 32-bit in every engine dtype.
// A sequence's state row holds S as [head][row / R][column][row % R], so that a warp reads and writes whole lines.
//
// Around it:
//   fg_conv1d_silu / fg_conv1d_state: the short causal convolution over time per channel (weights [channels, taps], the
//     last column meets the current token), then SiLU; the last taps - 1 inputs of a sequence are part of its state row.
//   fg_decay_gates: a and b of every (token, head) from the projections' raw numbers.
//   fg_unit_heads: x / sqrt(sum(x^2) + eps) * scale per head.
//   fg_gated_group_norm: the gate and the norm behind the recurrence, in either order.
#include "common.cuh"

#define REC_THREADS 256
#define REC_RPL 16                  // rows of a column a lane holds at most
#define REC_TC 16                   // tokens staged at a time

__device__ __forceinline__ float rec_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float rec_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rec_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ------------------------------------------------------------------ convolution
// out[m, c] = silu(bias[c] + sum_j w[c, j] * u(t - taps + 1 + j)), u = the channel's inputs of the row's sequence: rows of
// this step where there are some, else the sequence's state (its last taps - 1 inputs, oldest first; zeros at its start).
__global__ void __launch_bounds__(256)
conv1d_silu_kernel(const float *__restrict__ in, int ld, const float *__restrict__ w, const float *__restrict__ bias, int taps,
                   const float *__restrict__ state, long long state_stride, const int *__restrict__ row_seq,
                   const int *__restrict__ cu_rows, const int *__restrict__ slots, float *__restrict__ out, int ldo, int C) {
    pdl_wait();
    const int m = blockIdx.x;
    const int s = row_seq[m], first = cu_rows[s], i = m - first;
    const float *st = state + (size_t)slots[s] * state_stride;
    for (int c = blockIdx.y * 256 + threadIdx.x; c < C; c += gridDim.y * 256) {
        float acc = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps; j++) {
            const int t = i - (taps - 1) + j;
            const float u = t >= 0 ? in[(size_t)(first + t) * ld + c] : st[(size_t)(taps - 1 + t) * C + c];
            acc = fmaf(w[(size_t)c * taps + j], u, acc);
        }
        out[(size_t)m * ldo + c] = rec_silu(acc);
    }
}

// the sequences' last taps - 1 inputs to their state rows (a kernel of its own: no row may read a state another has replaced)
__global__ void __launch_bounds__(256)
conv1d_state_kernel(const float *__restrict__ in, int ld, int taps, float *__restrict__ state, long long state_stride,
                    const int *__restrict__ cu_rows, const int *__restrict__ slots, int C) {
    pdl_wait();
    const int s = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= C) return;
    const int first = cu_rows[s], n = cu_rows[s + 1] - first;
    if (n <= 0) return;
    float *st = state + (size_t)slots[s] * state_stride;
    for (int u = 0; u < taps - 1; u++) {
        const int t = n - (taps - 1) + u;               // ascending u: an old entry is read before its place is rewritten
        st[(size_t)u * C + c] = t >= 0 ? in[(size_t)(first + t) * ld + c] : st[(size_t)(u + n) * C + c];
    }
}

// ------------------------------------------------------------------ decays and steps
// mode 0: b = softplus(a_raw + dt_bias), a = exp(-exp(A_log) b)                    (one raw number a head)
// mode 1: a = exp(-exp(A_log) softplus(a_raw + dt_bias)), b = sigmoid(b_raw)
__global__ void decay_gates_kernel(const float *__restrict__ a_raw, int lda, const float *__restrict__ b_raw, int ldb,
                                   const float *__restrict__ A_log, const float *__restrict__ dt_bias, int mode,
                                   float *__restrict__ decay, float *__restrict__ step, int M, int H) {
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= M * H) return;
    const int m = e / H, h = e % H;
    const float sp = rec_softplus(a_raw[(size_t)m * lda + h] + dt_bias[h]);
    decay[e] = expf(-expf(A_log[h]) * sp);
    step[e] = mode == 0 ? sp : rec_sigmoid(b_raw[(size_t)m * ldb + h]);
}

// x[m, h, :] <- x / sqrt(sum(x^2) + eps) * scale, a warp a (row, head)
__global__ void __launch_bounds__(256)
unit_heads_kernel(float *__restrict__ x, int ld, int n_heads, int d, float eps, float scale, int M) {
    pdl_wait();
    const int id = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (id >= M * n_heads) return;
    float *p = x + (size_t)(id / n_heads) * ld + (size_t)(id % n_heads) * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    const float f = scale / sqrtf(ss + eps);
    for (int i = lane; i < d; i += 32) p[i] *= f;
}

// ------------------------------------------------------------------ the recurrence, token by token
template <bool DELTA>
__global__ void __launch_bounds__(REC_THREADS)
decay_recurrence_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ k, int ldk, const float *__restrict__ v, int ldv,
                        const float *__restrict__ decay, const float *__restrict__ step, const float *__restrict__ skip,
                        float *__restrict__ out, int ldo, const int *__restrict__ cu_rows, const int *__restrict__ slots,
                        float *__restrict__ state, long long state_stride, int H, int Hq, int d, int dv, int R, int cols) {
    extern __shared__ __align__(16) float sm[];
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = cu_rows[seq], row1 = cu_rows[seq + 1];
    if (row1 <= row0) return;
    const int epl = (d + R - 1) / R, dp = epl * R;          // rows a lane holds; rows with padding
    const int c0 = blockIdx.z * cols;                       // this block's first column
    const int cl = tid / R, r = tid % R, c = c0 + cl;
    const bool live = cl < cols && c < dv;
    const int hq = h / (H / Hq);
    float *qs = sm, *ks = qs + REC_TC * dp, *vs = ks + REC_TC * dp, *as = vs + REC_TC * cols, *bs = as + REC_TC;
    float *Sg = state + (size_t)slots[seq] * state_stride + (size_t)h * epl * dv * R;
    float S[REC_RPL];
#pragma unroll
    for (int e = 0; e < REC_RPL; e++) S[e] = (live && e < epl) ? Sg[((size_t)e * dv + c) * R + r] : 0.f;
    const float Dh = skip ? skip[h] : 0.f;
    for (int t0 = row0; t0 < row1; t0 += REC_TC) {
        const int n = min(REC_TC, row1 - t0);
        __syncthreads();                                    // the tokens before have been walked by every warp
        for (int e = tid; e < n * dp; e += REC_THREADS) {
            const int t = e / dp, i = e % dp;
            qs[e] = i < d ? q[(size_t)(t0 + t) * ldq + (size_t)hq * d + i] : 0.f;
            ks[e] = i < d ? k[(size_t)(t0 + t) * ldk + (size_t)hq * d + i] : 0.f;
        }
        for (int e = tid; e < n * cols; e += REC_THREADS) {
            const int t = e / cols, j = e % cols;
            vs[e] = c0 + j < dv ? v[(size_t)(t0 + t) * ldv + (size_t)h * dv + c0 + j] : 0.f;
        }
        if (tid < n) { as[tid] = decay[(size_t)(t0 + tid) * H + h]; bs[tid] = step[(size_t)(t0 + tid) * H + h]; }
        __syncthreads();
        if ((tid & ~31) / R >= cols) continue;              // a warp without a column (whole warps only: the shuffles below name every lane)
        for (int t = 0; t < n; t++) {
            const float a = as[t], vj = cl < cols ? vs[t * cols + cl] : 0.f;
            const float *kt = ks + t * dp + r, *qt = qs + t * dp + r;
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < REC_RPL; e++)
                if (e < epl) {
                    S[e] *= a;
                    if (DELTA) dot = fmaf(S[e], kt[e * R], dot);
                }
            if (DELTA)
                for (int o = R >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float u = bs[t] * (vj - dot);
            float o_sum = 0.f;
#pragma unroll
            for (int e = 0; e < REC_RPL; e++)
                if (e < epl) {
                    S[e] = fmaf(kt[e * R], u, S[e]);
                    o_sum = fmaf(S[e], qt[e * R], o_sum);
                }
            for (int o = R >> 1; o > 0; o >>= 1) o_sum += __shfl_xor_sync(0xffffffffu, o_sum, o);
            if (r == 0 && live) out[(size_t)(t0 + t) * ldo + (size_t)h * dv + c] = fmaf(Dh, vj, o_sum);
        }
    }
    if (live)
#pragma unroll
        for (int e = 0; e < REC_RPL; e++)
            if (e < epl) Sg[((size_t)e * dv + c) * R + r] = S[e];
}

// ------------------------------------------------------------------ gate and norm behind the recurrence
// gate_first: t = y * silu(g), out = t / rms_group(t) * w[c]                         (groups of `group` neighbouring channels)
// else:       out = y / rms_group(y) * w[c % w_period] * silu(g)
template <typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float *__restrict__ y, int ldy, const float *__restrict__ g, int ldg, const float *__restrict__ w,
                        int w_period, TO *__restrict__ out, int ldo, int C, int group, float eps, int gate_first) {
    pdl_wait();
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *yr = y + (size_t)m * ldy, *gr = g + (size_t)m * ldg;
    TO *orow = out + (size_t)m * ldo;
    for (int grp = blockIdx.y * 8 + warp; grp * group < C; grp += gridDim.y * 8) {
        const int b0 = grp * group;
        float ss = 0.f;
        for (int i = lane; i < group; i += 32) {
            const float t = gate_first ? yr[b0 + i] * rec_silu(gr[b0 + i]) : yr[b0 + i];
            ss = fmaf(t, t, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)group + eps);
        for (int i = lane; i < group; i += 32) {
            const int c = b0 + i;
            const float sg = rec_silu(gr[c]);
            orow[c] = from_f32<TO>(gate_first ? yr[c] * sg * inv * w[c % w_period] : yr[c] * inv * w[c % w_period] * sg);
        }
    }
}

// ------------------------------------------------------------------ launchers
extern "C" int fg_conv1d_silu(const float *in, int ld, const float *w, const float *bias, int taps, const float *state,
                              long long state_stride, const int *row_seq, const int *cu_rows, const int *slots, float *out, int ldo,
                              int M, int C, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (C <= 0 || taps <= 0 || (taps > 1 && !state)) return FG_ERR_BAD_SIZE;
    return fg_launch_in_order(conv1d_silu_kernel, dim3(M, (C + 1023) / 1024), dim3(256), 0, stream, in, ld, w, bias, taps, state, state_stride,
                              row_seq, cu_rows, slots, out, ldo, C);
}

extern "C" int fg_conv1d_state(const float *in, int ld, int taps, float *state, long long state_stride, const int *cu_rows,
                               const int *slots, int n_seq, int C, cudaStream_t stream) {
    if (n_seq <= 0 || taps <= 1) return 0;
    if (C <= 0) return FG_ERR_BAD_SIZE;
    return fg_launch_in_order(conv1d_state_kernel, dim3(n_seq, (C + 255) / 256), dim3(256), 0, stream, in, ld, taps, state, state_stride, cu_rows,
                              slots, C);
}

extern "C" int fg_decay_gates(const float *a_raw, int lda, const float *b_raw, int ldb, const float *A_log, const float *dt_bias,
                              int mode, float *decay, float *step, int M, int H, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (H <= 0 || (mode != 0 && mode != 1) || (mode == 1 && !b_raw)) return FG_ERR_BAD_SIZE;
    return fg_launch_in_order(decay_gates_kernel, dim3((M * H + 255) / 256), dim3(256), 0, stream, a_raw, lda, b_raw, ldb, A_log, dt_bias, mode,
                              decay, step, M, H);
}

extern "C" int fg_unit_heads(float *x, int ld, int n_heads, int d, float eps, float scale, int M, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (n_heads <= 0 || d <= 0) return FG_ERR_BAD_SIZE;
    return fg_launch_in_order(unit_heads_kernel, dim3((M * n_heads + 7) / 8), dim3(256), 0, stream, x, ld, n_heads, d, eps, scale, M);
}

// lanes that share a column of the state: the smallest power of two that leaves a lane at most REC_RPL rows
extern "C" int fg_decay_recurrence_lanes(int d) {
    int R = 1;
    while (R < 32 && (d + R - 1) / R > REC_RPL) R *= 2;
    return (d + R - 1) / R > REC_RPL ? 0 : R;
}
// floats of a sequence's state: [H][rows a lane][dv][R]
extern "C" long long fg_decay_recurrence_state_floats(int H, int d, int dv) {
    const int R = fg_decay_recurrence_lanes(d);
    return R ? (long long)H * ((d + R - 1) / R) * dv * R : -1;
}

extern "C" int fg_decay_recurrence(const float *q, int ldq, const float *k, int ldk, const float *v, int ldv, const float *decay,
                                   const float *step, const float *skip, float *out, int ldo, const int *cu_rows, const int *slots,
                                   float *state, long long state_stride, int n_seq, int H, int Hq, int d, int dv, int delta,
                                   cudaStream_t stream) {
    if (n_seq <= 0) return 0;
    const int R = fg_decay_recurrence_lanes(d);
    if (!R || H <= 0 || Hq <= 0 || H % Hq || dv <= 0 || H > 65535) return FG_ERR_BAD_SIZE;
    const int per_block = REC_THREADS / R, cols = per_block < dv ? per_block : dv, tiles = (dv + cols - 1) / cols;
    const int dp = (d + R - 1) / R * R;
    const size_t smem = (size_t)(REC_TC * (2 * dp + cols) + 2 * REC_TC) * sizeof(float);
    static FgPerDevice setup_a, setup_b;
    if (delta) {
        if (fg_needs_setup(setup_a)) cudaFuncSetAttribute(decay_recurrence_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    } else {
        if (fg_needs_setup(setup_b)) cudaFuncSetAttribute(decay_recurrence_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    }
    if (smem > 96 * 1024) return FG_ERR_BAD_SIZE;
    dim3 grid(n_seq, H, tiles);
    if (delta)
        return fg_launch_in_order(decay_recurrence_kernel<true>, grid, dim3(REC_THREADS), smem, stream, q, ldq, k, ldk, v, ldv, decay, step, skip, out,
                                  ldo, cu_rows, slots, state, state_stride, H, Hq, d, dv, R, cols);
    return fg_launch_in_order(decay_recurrence_kernel<false>, grid, dim3(REC_THREADS), smem, stream, q, ldq, k, ldk, v, ldv, decay, step, skip, out,
                              ldo, cu_rows, slots, state, state_stride, H, Hq, d, dv, R, cols);
}

extern "C" int fg_gated_group_norm(const float *y, int ldy, const float *g, int ldg, const float *w, int w_period, void *out,
                                   int out_dtype, int ldo, int M, int C, int group, float eps, int gate_first, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (C <= 0 || group <= 0 || C % group || w_period <= 0) return FG_ERR_BAD_SIZE;
    const int groups = C / group;
    dim3 grid(M, groups >= 64 ? 4 : 1);
    if (out_dtype == FG_F32)
        return fg_launch_in_order(gated_group_norm_kernel<float>, grid, dim3(256), 0, stream, y, ldy, g, ldg, w, w_period, (float *)out, ldo, C, group,
                                  eps, gate_first);
    if (out_dtype == FG_BF16)
        return fg_launch_in_order(gated_group_norm_kernel<bf16>, grid, dim3(256), 0, stream, y, ldy, g, ldg, w, w_period, (bf16 *)out, ldo, C, group,
                                  eps, gate_first);
    return FG_ERR_BAD_DTYPE;
}
