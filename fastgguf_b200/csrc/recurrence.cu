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
// a barrier while the next TC are being copied, and goes on.  State, decays, steps and sums are 32-bit in every engine dtype.
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
#define REC_TC 16                   // tokens staged at a time (fewer where a head's rows are many)

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
__device__ __forceinline__ void rec_copy4(float *dst, const float *src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void rec_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void rec_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// Shared memory holds TWO sets of TC tokens: while the warps walk one, the copies of the next are in flight (cp.async, four
// bytes each, since a lane's rows r, r + R, ... of k and q are laid side by side: [token][r][row / R], rows padded with zeros
// to `stride` floats, so that a lane reads its rows as 16-byte pieces and the R lanes of a column hit different banks).
// the sum of x over the R neighbouring lanes that share a column (R a power of two)
__device__ __forceinline__ float rec_lanes_sum(float x, int R) {
    if (R > 16) x += __shfl_xor_sync(0xffffffffu, x, 16);
    if (R > 8) x += __shfl_xor_sync(0xffffffffu, x, 8);
    if (R > 4) x += __shfl_xor_sync(0xffffffffu, x, 4);
    if (R > 2) x += __shfl_xor_sync(0xffffffffu, x, 2);
    if (R > 1) x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x;
}

// NJ: 16-byte pieces of rows a lane holds (its rows padded to 4 * NJ; the padding's k and q are zero, so its state stays zero)
template <bool DELTA, int NJ>
__global__ void __launch_bounds__(REC_THREADS, 1)
decay_recurrence_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ k, int ldk, const float *__restrict__ v, int ldv,
                        const float *__restrict__ decay, const float *__restrict__ step, const float *__restrict__ skip,
                        float *__restrict__ out, int ldo, const int *__restrict__ cu_rows, const int *__restrict__ slots,
                        float *__restrict__ state, long long state_stride, int H, int Hq, int d, int dv, int R, int logR, int cols,
                        int TC, int stride) {
    extern __shared__ __align__(16) float sm[];
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, NT = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31, n_warps = NT >> 5;
    const int row0 = cu_rows[seq], row1 = cu_rows[seq + 1];
    if (row1 <= row0) return;
    const int epl = (d + R - 1) / R;                        // rows a lane holds
    const int c0 = blockIdx.z * cols;                       // this block's first column
    const int cl = tid >> logR, r = tid & (R - 1), c = c0 + cl;
    const bool live = cl < cols && c < dv;
    const int hq = h / (H / Hq);
    const int qk_floats = TC * R * stride, set_floats = (2 * qk_floats + TC * cols + 2 * TC + 3) & ~3;      // one set: q, k, v, decays, steps
    for (int e = tid; e < 2 * set_floats; e += NT) sm[e] = 0.f;       // the padding stays zero for good
    float *Sg = state + (size_t)slots[seq] * state_stride + (size_t)h * epl * dv * R;
    float S[4 * NJ];
#pragma unroll
    for (int e = 0; e < 4 * NJ; e++) S[e] = (live && e < epl) ? Sg[((size_t)e * dv + c) * R + r] : 0.f;
    const float Dh = skip ? skip[h] : 0.f;
    __syncthreads();
    // the copies of the tokens from t0 on into set `b`: a warp a token, its lanes along the rows
    auto fetch = [&](int t0, int b) {
        const int n = min(TC, row1 - t0);
        float *qs = sm + b * set_floats, *ks = qs + qk_floats, *vs = ks + qk_floats, *as = vs + TC * cols, *bs = as + TC;
        for (int t = warp; t < n; t += n_warps) {
            const float *qg = q + (size_t)(t0 + t) * ldq + (size_t)hq * d, *kg = k + (size_t)(t0 + t) * ldk + (size_t)hq * d;
            for (int i = lane; i < d; i += 32) {
                const int at = (t * R + (i & (R - 1))) * stride + (i >> logR);
                rec_copy4(qs + at, qg + i);
                rec_copy4(ks + at, kg + i);
            }
            const float *vg = v + (size_t)(t0 + t) * ldv + (size_t)h * dv + c0;
            for (int j = lane; j < cols; j += 32)
                if (c0 + j < dv) rec_copy4(vs + t * cols + j, vg + j);
        }
        if (tid < n) {
            rec_copy4(as + tid, decay + (size_t)(t0 + tid) * H + h);
            rec_copy4(bs + tid, step + (size_t)(t0 + tid) * H + h);
        }
        rec_commit();
    };
    const bool warp_on = ((tid & ~31) >> logR) < cols;      // a warp without a column sits the walk out (whole warps only: the shuffles name every lane)
    const int tok4 = R * stride / 4;                        // 16-byte pieces between two tokens' rows
    fetch(row0, 0);
    int b = 0;
    for (int t0 = row0; t0 < row1; t0 += TC, b ^= 1) {
        const int n = min(TC, row1 - t0);
        fetch(t0 + TC, b ^ 1);                               // (an empty group behind the last tokens)
        rec_wait_all_but_one();
        __syncthreads();                                    // everybody's copies of this set have landed
        const float *qs = sm + b * set_floats, *ks = qs + qk_floats, *vs = ks + qk_floats, *as = vs + TC * cols, *bs = as + TC;
        if (warp_on) {
            const float4 *kt = (const float4 *)(ks + r * stride), *qt = (const float4 *)(qs + r * stride);
            const float *vt = vs + (cl < cols ? cl : 0);
            float *og = out + (size_t)t0 * ldo + (size_t)h * dv + c;
            // four tokens at a time: the sums over a column's R lanes that give the outputs are not part of the chain from
            // token to token, so the four of them are formed together behind the four updates (their shuffles overlap)
            for (int tb = 0; tb < n; tb += 4) {
                float o_part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (tb + u < n) {
                        const float a = as[tb + u], vj = vt[(tb + u) * cols];
                        float4 k4[NJ];
                        float d0 = 0.f, d1 = 0.f;
#pragma unroll
                        for (int j = 0; j < NJ; j++) {
                            k4[j] = kt[j];
                            S[4 * j] *= a; S[4 * j + 1] *= a; S[4 * j + 2] *= a; S[4 * j + 3] *= a;
                            if (DELTA) {
                                d0 = fmaf(S[4 * j], k4[j].x, d0); d1 = fmaf(S[4 * j + 1], k4[j].y, d1);
                                d0 = fmaf(S[4 * j + 2], k4[j].z, d0); d1 = fmaf(S[4 * j + 3], k4[j].w, d1);
                            }
                        }
                        const float dot = DELTA ? rec_lanes_sum(d0 + d1, R) : 0.f;
                        const float w = bs[tb + u] * (vj - dot);
                        float o0 = 0.f, o1 = 0.f;
#pragma unroll
                        for (int j = 0; j < NJ; j++) {
                            const float4 q4 = qt[j];
                            S[4 * j] = fmaf(k4[j].x, w, S[4 * j]); S[4 * j + 1] = fmaf(k4[j].y, w, S[4 * j + 1]);
                            S[4 * j + 2] = fmaf(k4[j].z, w, S[4 * j + 2]); S[4 * j + 3] = fmaf(k4[j].w, w, S[4 * j + 3]);
                            o0 = fmaf(S[4 * j], q4.x, o0); o1 = fmaf(S[4 * j + 1], q4.y, o1);
                            o0 = fmaf(S[4 * j + 2], q4.z, o0); o1 = fmaf(S[4 * j + 3], q4.w, o1);
                        }
                        o_part[u] = o0 + o1;
                    }
                    kt += tok4; qt += tok4;
                }
#pragma unroll
                for (int u = 0; u < 4; u++) o_part[u] = rec_lanes_sum(o_part[u], R);
                if (r == 0 && live) {
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (tb + u < n) og[(size_t)(tb + u) * ldo] = fmaf(Dh, vt[(tb + u) * cols], o_part[u]);
                }
            }
        }
        __syncthreads();                                    // this set is free for the copies of the tokens after the next
    }
    if (live)
#pragma unroll
        for (int e = 0; e < 4 * NJ; e++)
            if (e < epl) Sg[((size_t)e * dv + c) * R + r] = S[e];
}

// ------------------------------------------------------------------ gate and norm behind the recurrence
// gate_first: t = y * silu(g), out = t / rms_group(t) * w[c]                         (groups of `group` neighbouring channels)
// else:       out = y / rms_group(y) * w[c % w_period] * silu(g)
template <typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float *__restrict__ y, int ldy, const float *__restrict__ g, int ldg, const float *__restrict__ w,
                        int w_period, TO *__restrict__ out, int ldo, int C, int group, float eps, int gate_first) {
    __shared__ float scratch[32];
    pdl_wait();
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *yr = y + (size_t)m * ldy, *gr = g + (size_t)m * ldg;
    TO *orow = out + (size_t)m * ldo;
    const bool whole = w_period >= C, by_group = w_period == group;
    if (group >= 1024) {
        // few wide groups: the whole block takes a group (fixed reduction order: lanes, then warps in order)
        for (int b0 = blockIdx.y * group; b0 < C; b0 += gridDim.y * group) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < group; i += 256) {
                const float t = gate_first ? yr[b0 + i] * rec_silu(gr[b0 + i]) : yr[b0 + i];
                ss = fmaf(t, t, ss);
            }
            const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)group + eps);
            for (int i = threadIdx.x; i < group; i += 256) {
                const int c = b0 + i;
                const float sg = rec_silu(gr[c]);
                const float wc = w[whole ? c : (by_group ? i : c % w_period)];        // (no division where the weight spans the row or a group)
                orow[c] = from_f32<TO>(gate_first ? yr[c] * sg * inv * wc : yr[c] * inv * wc * sg);
            }
        }
        return;
    }
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
            const float wc = w[whole ? c : (by_group ? i : c % w_period)];        // (no division where the weight spans the row or a group)
                orow[c] = from_f32<TO>(gate_first ? yr[c] * sg * inv * wc : yr[c] * inv * wc * sg);
        }
    }
}

// ------------------------------------------------------------------ launchers
extern "C" int fg_conv1d_silu(const float *in, int ld, const float *w, const float *bias, int taps, const float *state,
                              long long state_stride, const int *row_seq, const int *cu_rows, const int *slots, float *out, int ldo,
                              int M, int C, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (C <= 0 || taps <= 0 || (taps > 1 && !state)) return FG_ERR_BAD_SIZE;
    return fg_launch(conv1d_silu_kernel, dim3(M, (C + 1023) / 1024), dim3(256), 0, stream, in, ld, w, bias, taps, state, state_stride,
                              row_seq, cu_rows, slots, out, ldo, C);
}

extern "C" int fg_conv1d_state(const float *in, int ld, int taps, float *state, long long state_stride, const int *cu_rows,
                               const int *slots, int n_seq, int C, cudaStream_t stream) {
    if (n_seq <= 0 || taps <= 1) return 0;
    if (C <= 0) return FG_ERR_BAD_SIZE;
    return fg_launch(conv1d_state_kernel, dim3(n_seq, (C + 255) / 256), dim3(256), 0, stream, in, ld, taps, state, state_stride, cu_rows,
                              slots, C);
}

extern "C" int fg_decay_gates(const float *a_raw, int lda, const float *b_raw, int ldb, const float *A_log, const float *dt_bias,
                              int mode, float *decay, float *step, int M, int H, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (H <= 0 || (mode != 0 && mode != 1) || (mode == 1 && !b_raw)) return FG_ERR_BAD_SIZE;
    return fg_launch(decay_gates_kernel, dim3((M * H + 255) / 256), dim3(256), 0, stream, a_raw, lda, b_raw, ldb, A_log, dt_bias, mode,
                              decay, step, M, H);
}

extern "C" int fg_unit_heads(float *x, int ld, int n_heads, int d, float eps, float scale, int M, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (n_heads <= 0 || d <= 0) return FG_ERR_BAD_SIZE;
    return fg_launch(unit_heads_kernel, dim3((M * n_heads + 7) / 8), dim3(256), 0, stream, x, ld, n_heads, d, eps, scale, M);
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
    // Blocks of 256 threads where there are many (sequence, head) pairs; fewer threads a block - down to two warps - where the
    // blocks would not fill the GPU otherwise: a token's work in a warp is a chain of dependent instructions, and warps that
    // share a scheduler lengthen every token's turn.
    int n_sm = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    int threads = REC_THREADS;
    while (threads > 64 && (long long)n_seq * H * ((dv + threads / R - 1) / (threads / R)) < 2LL * n_sm && threads / 2 >= R) threads /= 2;
    const int per_block = threads / R, cols = per_block < dv ? per_block : dv, tiles = (dv + cols - 1) / cols;
    int logR = 0;
    while ((1 << logR) < R) logR++;
    const int epl = (d + R - 1) / R, stride = (epl + 3) / 4 * 4 + 4;
    // two sets of TC tokens in shared memory; fewer tokens a set where a head is large
    int TC = REC_TC;
    auto bytes = [&](int tc) { return (size_t)2 * ((2 * tc * R * stride + tc * cols + 2 * tc + 3) & ~3) * sizeof(float); };
    while (TC > 2 && bytes(TC) > 96 * 1024) TC /= 2;
    const size_t smem = bytes(TC);
    if (smem > 96 * 1024) return FG_ERR_BAD_SIZE;
    dim3 grid(n_seq, H, tiles);
    const int NJ = (epl + 3) / 4;
#define REC_LAUNCH(DELTA, NJ_)                                                                                                            \
    do {                                                                                                                                  \
        static FgPerDevice setup;                                                                                                         \
        if (fg_needs_setup(setup)) cudaFuncSetAttribute(decay_recurrence_kernel<DELTA, NJ_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
        return fg_launch(decay_recurrence_kernel<DELTA, NJ_>, grid, dim3(threads), smem, stream, q, ldq, k, ldk, v, ldv, decay, step, skip, out, \
                                  ldo, cu_rows, slots, state, state_stride, H, Hq, d, dv, R, logR, cols, TC, stride);                      \
    } while (0)
    if (delta) {
        if (NJ == 1) REC_LAUNCH(true, 1);
        if (NJ == 2) REC_LAUNCH(true, 2);
        if (NJ == 3) REC_LAUNCH(true, 3);
        REC_LAUNCH(true, 4);
    }
    if (NJ == 1) REC_LAUNCH(false, 1);
    if (NJ == 2) REC_LAUNCH(false, 2);
    if (NJ == 3) REC_LAUNCH(false, 3);
    REC_LAUNCH(false, 4);
#undef REC_LAUNCH
}

extern "C" int fg_gated_group_norm(const float *y, int ldy, const float *g, int ldg, const float *w, int w_period, void *out,
                                   int out_dtype, int ldo, int M, int C, int group, float eps, int gate_first, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (C <= 0 || group <= 0 || C % group || w_period <= 0) return FG_ERR_BAD_SIZE;
    const int groups = C / group;
    dim3 grid(M, group >= 1024 ? (groups < 4 ? groups : 4) : groups >= 64 ? 4 : 1);
    if (out_dtype == FG_F32)
        return fg_launch(gated_group_norm_kernel<float>, grid, dim3(256), 0, stream, y, ldy, g, ldg, w, w_period, (float *)out, ldo, C, group,
                                  eps, gate_first);
    if (out_dtype == FG_BF16)
        return fg_launch(gated_group_norm_kernel<bf16>, grid, dim3(256), 0, stream, y, ldy, g, ldg, w, w_period, (bf16 *)out, ldo, C, group,
                                  eps, gate_first);
    return FG_ERR_BAD_DTYPE;
}
