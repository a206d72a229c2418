// Mixture of experts: routing, the experts' contractions over rows grouped by expert, and the sum.
//
//   scores s = sigmoid(z) of the router logits z (float32); a row uses the `top` experts with the largest scores, each
//   weighted by its own score (kind 0: as it is, not renormalised).  The weight multiplies the expert's INPUT:
//       out = sum_e expert_e(s_e h),   expert(x) = W_down act(W_gate x, W_up x)
//   and since both first contractions are linear in x, s_e is applied to their float32 results instead of to h.
//   act, kind 0:  g = min(g, limit), u = clamp(u, -limit, limit), y = g * sigmoid(alpha g) * (u + 1).
//
// Layout.  A "pair" p = row * top + k is a row's k-th choice.  route() writes the pair's expert and weight and groups
// pairs by expert: `order[slot] = pair`, `slot_of[pair] = slot`, expert e owning slots [offsets[e], offsets[e + 1]).
// The contractions run over slots, so that a tile of rows shares one expert's weights; all sizes that depend on the
// routing stay on the device (only the per-expert path of long portions, at the end of this file, has the host read the
// experts' row counts).  An output element is summed along k in the same order whichever
// tile or slot its row lands in, and a row's experts are added in the order of its choices, so a row's result does not
// depend on what else is in the step.
//
// Weights: w_in [X, 2F, E] (gate rows, then up rows, of each expert), w_out [X, E, F]; activations and weights share
// the engine's dtype T, accumulation is float32.
#include "common.cuh"

#define MOE_MAX_EXPERTS 256
#define MOE_MAX_TOP 8

// ------------------------------------------------------------------ router logits
// z[m, e] = x[m] . W[e], float32 accumulation of the inputs as they are.  A block per row: every thread takes runs of
// 16 bytes of the row and of each expert's weights (the router's few rows stay in cache), eight experts at a time; the
// threads' sums are added in a fixed order.  (The general contraction kernel spends a 64-wide tile on these few outputs.)
template <typename T>
__global__ void __launch_bounds__(256)
moe_logits_kernel(const T *__restrict__ x, int ldx, const T *__restrict__ W, int ldw, float *__restrict__ z, int X, int E, int vec) {
    __shared__ float part[8][8];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int VEC = 16 / (int)sizeof(T);
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T *xr = x + (size_t)m * ldx;
    for (int e0 = 0; e0 < X; e0 += 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (vec) {
            for (int k = threadIdx.x * VEC; k < E; k += 256 * VEC) {
                const uint4 xv = *(const uint4 *)(xr + k);
                const T *xe = (const T *)&xv;
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    if (e0 + u >= X) break;
                    const uint4 wv = *(const uint4 *)(W + (size_t)(e0 + u) * ldw + k);
                    const T *we = (const T *)&wv;
#pragma unroll
                    for (int i = 0; i < VEC; i++) acc[u] = fmaf(to_f32<T>(xe[i]), to_f32<T>(we[i]), acc[u]);
                }
            }
        } else {
            for (int k = threadIdx.x; k < E; k += 256) {
                const float xv = to_f32<T>(xr[k]);
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (e0 + u < X) acc[u] = fmaf(xv, to_f32<T>(W[(size_t)(e0 + u) * ldw + k]), acc[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            float v = warp_sum(acc[u]);
            if (lane == 0) part[warp][u] = v;
        }
        __syncthreads();
        if (threadIdx.x < 8 && e0 + threadIdx.x < X) {
            float v = 0.f;
            for (int w = 0; w < 8; w++) v += part[w][threadIdx.x];
            z[(size_t)m * X + e0 + threadIdx.x] = v;
        }
        __syncthreads();
    }
}

extern "C" int fg_moe_logits(const void *x, int ldx, const void *W, int ldw, int dtype, float *z, int M, int X, int E, cudaStream_t stream) {
    if (M <= 0) return 0;
    const int per = dtype == FG_F32 ? 4 : 8;
    const int vec = E % per == 0 && ldx % per == 0 && ldw % per == 0 && ((((uintptr_t)x) | ((uintptr_t)W)) & 15) == 0;
    if (dtype == FG_F32)
        return fg_launch(moe_logits_kernel<float>, dim3(M), dim3(256), 0, stream, (const float *)x, ldx, (const float *)W, ldw, z, X, E, vec);
    if (dtype == FG_BF16)
        return fg_launch(moe_logits_kernel<bf16>, dim3(M), dim3(256), 0, stream, (const bf16 *)x, ldx, (const bf16 *)W, ldw, z, X, E, vec);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ routing
// One block.  logits: [M, X] float32.
__global__ void __launch_bounds__(1024)
moe_route_kernel(const float *__restrict__ logits, int M, int X, int top, int *__restrict__ pair_expert, float *__restrict__ pair_weight,
                 int *__restrict__ offsets, int *__restrict__ order, int *__restrict__ slot_of) {
    __shared__ int counts[MOE_MAX_EXPERTS], cursor[MOE_MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < X; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < M; r += blockDim.x) {
        const float *z = logits + (size_t)r * X;
        int chosen[MOE_MAX_TOP];
        for (int k = 0; k < top; k++) {
            int best = -1;
            float bz = 0.f;
            for (int e = 0; e < X; e++) {
                bool taken = false;
                for (int q = 0; q < k; q++) taken = taken || chosen[q] == e;
                if (taken) continue;
                float v = z[e];
                if (best < 0 || v > bz) { best = e; bz = v; }       // sigmoid is monotonic: the largest logit; ties to the lower index
            }
            chosen[k] = best;
            pair_expert[(size_t)r * top + k] = best;
            pair_weight[(size_t)r * top + k] = 1.0f / (1.0f + expf(-bz));
            atomicAdd(&counts[best], 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < X; e++) { offsets[e] = at; cursor[e] = at; at += counts[e]; }
        offsets[X] = at;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < M * top; p += blockDim.x) {
        int slot = atomicAdd(&cursor[pair_expert[p]], 1);
        order[slot] = p;
        slot_of[p] = slot;
    }
}

extern "C" int fg_moe_route(const float *logits, int M, int X, int top, int *pair_expert, float *pair_weight, int *offsets, int *order,
                            int *slot_of, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (X <= 0 || X > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP || top > X) return FG_ERR_BAD_SIZE;
    int threads = M >= 1024 ? 1024 : ((M + 31) / 32) * 32;
    return fg_launch(moe_route_kernel, dim3(1), dim3(threads), 0, stream, logits, M, X, top, pair_expert, pair_weight, offsets, order,
                     slot_of);
}

// ------------------------------------------------------------------ routing, kind 1: softmax scores, a selection bias, groups
// scores s = softmax(z) over all X router outputs; the choice is made on c = s + bias (bias: a float per output), the
// weights from s.  The outputs form n_groups equal runs of neighbours; a group's score is its largest c, and only outputs of
// the `keep` best groups can be chosen (the others count as minus infinity, whatever sign c has).  The `top` outputs with the
// largest c are taken (ties to the lower index); their weights are s / (sum of the chosen s + 1e-20) * scale.  Outputs at and
// beyond n_real have no expert behind them (the caller gives them a meaning, e.g. "the input itself"); they are routed,
// grouped and counted like the others.  One block; a thread a row.  logits: [M, X] float32.  CACHED: the row's X scores are
// formed once and kept in shared memory ([X][threads], so that a warp's accesses fall into different banks); otherwise every
// use forms them again (the same operations, the same values).
template <bool CACHED>
__global__ void __launch_bounds__(1024)
moe_route_grouped_kernel(const float *__restrict__ logits, const float *__restrict__ bias, int M, int X, int top, int n_groups, int keep,
                         float scale, int *__restrict__ pair_expert, float *__restrict__ pair_weight, int *__restrict__ offsets,
                         int *__restrict__ order, int *__restrict__ slot_of) {
    __shared__ int counts[MOE_MAX_EXPERTS], cursor[MOE_MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < X; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    const int per = X / n_groups;
    extern __shared__ float route_scores[];
    float *sc = route_scores + threadIdx.x;
    const int B = blockDim.x;
    for (int r = threadIdx.x; r < M; r += blockDim.x) {
        const float *z = logits + (size_t)r * X;
        float zmax = z[0];
        for (int e = 1; e < X; e++) zmax = fmaxf(zmax, z[e]);
        float sum = 0.f;
        for (int e = 0; e < X; e++) {
            const float x = expf(z[e] - zmax);
            if (CACHED) sc[e * B] = x;
            sum += x;
        }
        const float inv = 1.0f / sum;
        if (CACHED)
            for (int e = 0; e < X; e++) sc[e * B] *= inv;
        auto score = [&](int e) { return CACHED ? sc[e * B] : expf(z[e] - zmax) * inv; };
        // the groups that stay: `keep` times the best group not yet taken
        unsigned long long allowed = 0ull;
        for (int k = 0; k < keep; k++) {
            int best = -1;
            float bs = 0.f;
            for (int g = 0; g < n_groups; g++) {
                if (allowed >> g & 1ull) continue;
                float gs = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; e++) gs = fmaxf(gs, score(e) + (bias ? bias[e] : 0.f));
                if (best < 0 || gs > bs) { best = g; bs = gs; }
            }
            allowed |= 1ull << best;
        }
        int chosen[MOE_MAX_TOP];
        float s_of[MOE_MAX_TOP], total = 0.f;
        for (int k = 0; k < top; k++) {
            int best = -1;
            float bc = 0.f, bsc = 0.f;
            for (int e = 0; e < X; e++) {
                if (!(allowed >> (e / per) & 1ull)) continue;
                bool taken = false;
                for (int q = 0; q < k; q++) taken = taken || chosen[q] == e;
                if (taken) continue;
                const float se = score(e), c = se + (bias ? bias[e] : 0.f);
                if (best < 0 || c > bc) { best = e; bc = c; bsc = se; }
            }
            chosen[k] = best;
            s_of[k] = bsc;
            total += bsc;
        }
        const float norm = scale / (total + 1e-20f);
        for (int k = 0; k < top; k++) {
            pair_expert[(size_t)r * top + k] = chosen[k];
            pair_weight[(size_t)r * top + k] = s_of[k] * norm;
            atomicAdd(&counts[chosen[k]], 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < X; e++) { offsets[e] = at; cursor[e] = at; at += counts[e]; }
        offsets[X] = at;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < M * top; p += blockDim.x) {
        int slot = atomicAdd(&cursor[pair_expert[p]], 1);
        order[slot] = p;
        slot_of[p] = slot;
    }
}

extern "C" int fg_moe_route_grouped(const float *logits, const float *bias, int M, int X, int top, int n_groups, int keep, float scale,
                                    int *pair_expert, float *pair_weight, int *offsets, int *order, int *slot_of, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (X <= 0 || X > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP || n_groups <= 0 || n_groups > 64 || X % n_groups || keep <= 0 ||
        keep > n_groups || top > keep * (X / n_groups))
        return FG_ERR_BAD_SIZE;
    int threads = M >= 1024 ? 1024 : ((M + 31) / 32) * 32;
    const size_t smem = (size_t)X * threads * sizeof(float);
    if (smem <= 160 * 1024) {
        static bool raised = false;
        if (!raised) {
            cudaError_t e = cudaFuncSetAttribute(moe_route_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e != cudaSuccess) return (int)e;
            raised = true;
        }
        return fg_launch(moe_route_grouped_kernel<true>, dim3(1), dim3(threads), smem, stream, logits, bias, M, X, top, n_groups, keep, scale,
                         pair_expert, pair_weight, offsets, order, slot_of);
    }
    return fg_launch(moe_route_grouped_kernel<false>, dim3(1), dim3(threads), 0, stream, logits, bias, M, X, top, n_groups, keep, scale, pair_expert,
                     pair_weight, offsets, order, slot_of);
}

// limit > 0: the clamped form above; limit <= 0: the plain gated form silu(g) * u, silu(z) = z * sigmoid(z)
__device__ __forceinline__ float expert_act(float g, float u, float limit, float alpha) {
    if (!(limit > 0.f)) return g / (1.0f + expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

// ------------------------------------------------------------------ tiles of 64 slots x 64 outputs on the FMA units
// The tile of a block: walk the experts, each padded to whole tiles; blocks beyond the last tile leave.
#define MT 64
#define MK 16

__device__ __forceinline__ bool moe_find_tile(const int *__restrict__ offsets, int X, int tile, int *expert, int *slot0, int *slot1) {
    for (int e = 0; e < X; e++) {
        const int a = offsets[e], b = offsets[e + 1], nt = (b - a + MT - 1) / MT;
        if (tile < nt) { *expert = e; *slot0 = a + tile * MT; *slot1 = min(b, a + (tile + 1) * MT); return true; }
        tile -= nt;
    }
    return false;
}

// FIRST: y[slot, n] = act(w (x . gate_n), w (x . up_n)) with x = xn[pair / top]; else out[slot, n] = y[slot] . down_n
template <typename T, bool FIRST>
__global__ void __launch_bounds__(256)
moe_tile_kernel(const T *__restrict__ A, int lda, const T *__restrict__ W, void *__restrict__ out, int ldo,
                const int *__restrict__ offsets, const int *__restrict__ order, const float *__restrict__ pair_weight, int X, int top,
                int N, int K, float limit, float alpha) {
    __shared__ float As[MK][MT + 1], Bs[FIRST ? 2 : 1][MK][MT + 1];
    __shared__ int arow[MT];
    pdl_launch_dependents();
    pdl_wait();
    int e, s0, s1;
    if (!moe_find_tile(offsets, X, blockIdx.y, &e, &s0, &s1)) return;
    const int n0 = blockIdx.x * MT, tid = threadIdx.x;
    if (tid < MT) arow[tid] = s0 + tid < s1 ? (FIRST ? order[s0 + tid] / top : s0 + tid) : -1;
    __syncthreads();
    const T *We = W + (size_t)e * (FIRST ? 2 : 1) * N * K;
    const int tx = tid & 15, ty = tid >> 4;          // outputs n0 + tx + 16 j, slots s0 + ty + 16 i
    float acc[FIRST ? 2 : 1][4][4] = {};
    for (int k0 = 0; k0 < K; k0 += MK) {
        for (int i = tid; i < MT * MK; i += 256) {
            const int r = i / MK, k = i % MK;
            const int ar = arow[r];
            As[k][r] = (ar >= 0 && k0 + k < K) ? to_f32<T>(A[(size_t)ar * lda + k0 + k]) : 0.f;
            const bool ok = n0 + r < N && k0 + k < K;
            Bs[0][k][r] = ok ? to_f32<T>(We[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
            if (FIRST) Bs[FIRST ? 1 : 0][k][r] = ok ? to_f32<T>(We[(size_t)(N + n0 + r) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MK; k++) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; j++) { b[j] = Bs[0][k][tx + 16 * j]; b2[j] = FIRST ? Bs[FIRST ? 1 : 0][k][tx + 16 * j] : 0.f; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[0][i][j] = fmaf(a[i], b[j], acc[0][i][j]);
                    if (FIRST) acc[FIRST ? 1 : 0][i][j] = fmaf(a[i], b2[j], acc[FIRST ? 1 : 0][i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int slot = s0 + ty + 16 * i;
        if (slot >= s1) continue;
        const float w = (FIRST && pair_weight) ? pair_weight[order[slot]] : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            if (FIRST) ((T *)out)[(size_t)slot * ldo + n] = from_f32<T>(expert_act(w * acc[0][i][j], w * acc[FIRST ? 1 : 0][i][j], limit, alpha));
            else ((float *)out)[(size_t)slot * ldo + n] = acc[0][i][j];
        }
    }
}

// ------------------------------------------------------------------ a few rows (decode): a warp per output, weights streamed once per pair
// (Pairs of one expert read the same rows at about the same time, so the second reader finds them in L2.  The kernel
// further down reads an expert's rows once for all its slots; this one takes what that one refuses.)
// output rows a warp takes together: gate and up double the loads of a row, so two there and four for down
#define MR_ROWS_OF(FIRST) ((FIRST) ? 2 : 4)
template <typename T, bool FIRST>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const T *__restrict__ A, int lda, const T *__restrict__ W, void *__restrict__ out, int ldo,
                const int *__restrict__ pair_expert, const int *__restrict__ order, const float *__restrict__ pair_weight, int top,
                int X, int N, int K, float limit, float alpha) {
    extern __shared__ __align__(16) float xs[];      // [K] the slot's input row
    pdl_launch_dependents();
    pdl_wait();
    const int slot = blockIdx.y, pair = order[slot], e = pair_expert[pair];
    if (e >= X) return;                              // a choice without an expert behind it (the caller handles it)
    const T *a = A + (size_t)(FIRST ? pair / top : slot) * lda;
    for (int k = threadIdx.x; k < K; k += 256) xs[k] = to_f32<T>(a[k]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T *We = W + (size_t)e * (FIRST ? 2 : 1) * N * K;
    const float w = (FIRST && pair_weight) ? pair_weight[pair] : 1.0f;
    constexpr int VEC = 16 / (int)sizeof(T);         // elements a 16-byte load brings
    const bool vec = (K % VEC) == 0 && (((uintptr_t)W) & 15) == 0;
    constexpr int MR_ROWS = MR_ROWS_OF(FIRST);
    // a warp takes MR_ROWS neighbouring output rows at a time: their weight rows are fetched together, so that many
    // 16-byte loads are in flight in every lane
    for (int n0 = (blockIdx.x * 8 + warp) * MR_ROWS; n0 < N; n0 += gridDim.x * 8 * MR_ROWS) {
        float sg[MR_ROWS], su[MR_ROWS];
#pragma unroll
        for (int r = 0; r < MR_ROWS; r++) sg[r] = su[r] = 0.f;
        if (vec) {
#pragma unroll 2
            for (int k = lane * VEC; k < K; k += 32 * VEC) {
                uint4 gv[MR_ROWS], uv[MR_ROWS];
#pragma unroll
                for (int r = 0; r < MR_ROWS; r++) {
                    const int n = min(n0 + r, N - 1);                  // rows past the end repeat the last one; never stored
                    gv[r] = *(const uint4 *)(We + (size_t)n * K + k);
                    if (FIRST) uv[r] = *(const uint4 *)(We + (size_t)(N + n) * K + k);
                }
                float x[VEC];
#pragma unroll
                for (int i = 0; i < VEC; i += 4) *(float4 *)(x + i) = *(const float4 *)(xs + k + i);
#pragma unroll
                for (int r = 0; r < MR_ROWS; r++) {
                    const T *ge = (const T *)&gv[r], *ue = (const T *)&uv[r];
#pragma unroll
                    for (int i = 0; i < VEC; i++) {
                        sg[r] = fmaf(x[i], to_f32<T>(ge[i]), sg[r]);
                        if (FIRST) su[r] = fmaf(x[i], to_f32<T>(ue[i]), su[r]);
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
#pragma unroll
                for (int r = 0; r < MR_ROWS; r++) {
                    const int n = min(n0 + r, N - 1);
                    sg[r] = fmaf(xs[k], to_f32<T>(We[(size_t)n * K + k]), sg[r]);
                    if (FIRST) su[r] = fmaf(xs[k], to_f32<T>(We[(size_t)(N + n) * K + k]), su[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MR_ROWS; r++) {
            sg[r] = warp_sum(sg[r]);
            if (FIRST) su[r] = warp_sum(su[r]);
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < MR_ROWS; r++) {
                const int n = n0 + r;
                if (n >= N) break;
                if (FIRST) ((T *)out)[(size_t)slot * ldo + n] = from_f32<T>(expert_act(w * sg[r], w * su[r], limit, alpha));
                else ((float *)out)[(size_t)slot * ldo + n] = sg[r];
            }
        }
    }
}

// ------------------------------------------------------------------ a few rows (decode), an expert's weights read once
// grid (blocks of output rows, experts).  A block of expert e takes the expert's slots up to four at a time: their input
// rows wait in shared memory as float32, and every warp reads its MR_ROWS weight rows once, in runs of 16 bytes, for
// all of them - where the kernel above reads them once per slot and leaves it to L2 to see the repeats.  Experts no row
// chose leave at once.  Sums run along k in the same order as above, so a slot's result does not depend on its company.
#define MG_SLOTS 4
// FASTGGUF_MOE_GROUPED=0: the kernel above instead (for measurements)
static bool moe_grouped_enabled() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("FASTGGUF_MOE_GROUPED"); v = !(e && e[0] == '0'); }
    return v != 0;
}
template <typename T, bool FIRST, int CNT>
__device__ __forceinline__ void moe_group_rows(const T *__restrict__ We, const float *xs, void *__restrict__ out, int ldo, int s0,
                                               const float (&w)[MG_SLOTS], int N, int K, float limit, float alpha, int n0, int lane) {
    constexpr int R = MR_ROWS_OF(FIRST), VEC = 16 / (int)sizeof(T);
    float sg[CNT][R], su[CNT][R];
#pragma unroll
    for (int i = 0; i < CNT; i++)
#pragma unroll
        for (int r = 0; r < R; r++) sg[i][r] = su[i][r] = 0.f;
#pragma unroll 2
    for (int k = lane * VEC; k < K; k += 32 * VEC) {
        uint4 gv[R], uv[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int n = min(n0 + r, N - 1);
            gv[r] = *(const uint4 *)(We + (size_t)n * K + k);
            if (FIRST) uv[r] = *(const uint4 *)(We + (size_t)(N + n) * K + k);
        }
#pragma unroll
        for (int i = 0; i < CNT; i++) {
            float x[VEC];
#pragma unroll
            for (int j = 0; j < VEC; j += 4) *(float4 *)(x + j) = *(const float4 *)(xs + i * K + k + j);
#pragma unroll
            for (int r = 0; r < R; r++) {
                const T *ge = (const T *)&gv[r], *ue = (const T *)&uv[r];
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    sg[i][r] = fmaf(x[j], to_f32<T>(ge[j]), sg[i][r]);
                    if (FIRST) su[i][r] = fmaf(x[j], to_f32<T>(ue[j]), su[i][r]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < CNT; i++)
#pragma unroll
        for (int r = 0; r < R; r++) {
            sg[i][r] = warp_sum(sg[i][r]);
            if (FIRST) su[i][r] = warp_sum(su[i][r]);
        }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < CNT; i++)
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int n = n0 + r;
                if (n >= N) break;
                if (FIRST) ((T *)out)[(size_t)(s0 + i) * ldo + n] = from_f32<T>(expert_act(w[i] * sg[i][r], w[i] * su[i][r], limit, alpha));
                else ((float *)out)[(size_t)(s0 + i) * ldo + n] = sg[i][r];
            }
    }
}

template <typename T, bool FIRST>
__global__ void __launch_bounds__(256)
moe_rows_grouped_kernel(const T *__restrict__ A, int lda, const T *__restrict__ W, void *__restrict__ out, int ldo,
                        const int *__restrict__ offsets, const int *__restrict__ order, const float *__restrict__ pair_weight, int top,
                        int N, int K, float limit, float alpha) {
    extern __shared__ __align__(16) float xs[];      // [MG_SLOTS][K]
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.y, s_begin = offsets[e], s_end = offsets[e + 1];
    if (s_end <= s_begin) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T *We = W + (size_t)e * (FIRST ? 2 : 1) * N * K;
    const int n0 = (blockIdx.x * 8 + warp) * MR_ROWS_OF(FIRST);
    for (int s0 = s_begin; s0 < s_end; s0 += MG_SLOTS) {
        const int cnt = min(MG_SLOTS, s_end - s0);
        __syncthreads();                             // the rows of the group before are no longer read
        for (int i = 0; i < cnt; i++) {
            const T *a = A + (size_t)(FIRST ? order[s0 + i] / top : s0 + i) * lda;
            for (int k = threadIdx.x; k < K; k += 256) xs[i * K + k] = to_f32<T>(a[k]);
        }
        __syncthreads();
        float w[MG_SLOTS];
#pragma unroll
        for (int i = 0; i < MG_SLOTS; i++) w[i] = (FIRST && pair_weight && i < cnt) ? pair_weight[order[s0 + i]] : 1.0f;
        if (n0 >= N) continue;
        switch (cnt) {
        case 1: moe_group_rows<T, FIRST, 1>(We, xs, out, ldo, s0, w, N, K, limit, alpha, n0, lane); break;
        case 2: moe_group_rows<T, FIRST, 2>(We, xs, out, ldo, s0, w, N, K, limit, alpha, n0, lane); break;
        case 3: moe_group_rows<T, FIRST, 3>(We, xs, out, ldo, s0, w, N, K, limit, alpha, n0, lane); break;
        default: moe_group_rows<T, FIRST, 4>(We, xs, out, ldo, s0, w, N, K, limit, alpha, n0, lane); break;
        }
    }
}

// takes sizes whose rows allow 16-byte loads and whose four input rows fit shared memory
static bool moe_grouped_ok(int dtype, int K, const void *W) {
    const int per = dtype == FG_F32 ? 4 : 8;
    return K % per == 0 && (((uintptr_t)W) & 15) == 0 && (size_t)MG_SLOTS * K * sizeof(float) <= 96 * 1024;
}
template <typename T, bool FIRST>
static int moe_grouped_launch(const void *A, int lda, const void *W, void *out, int ldo, const int *offsets, const int *order,
                              const float *pair_weight, int X, int top, int N, int K, float limit, float alpha, cudaStream_t stream) {
    static FgPerDevice setup;
    if (fg_needs_setup(setup)) {
        cudaError_t e = cudaFuncSetAttribute(moe_rows_grouped_kernel<T, FIRST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    const int per_block = 8 * MR_ROWS_OF(FIRST);
    return fg_launch(moe_rows_grouped_kernel<T, FIRST>, dim3((N + per_block - 1) / per_block, X), dim3(256), (size_t)MG_SLOTS * K * sizeof(float),
                     stream, (const T *)A, lda, (const T *)W, out, ldo, offsets, order, pair_weight, top, N, K, limit, alpha);
}

// y: [M * top, F] in T.  x: [M, E].  w_in: [X, 2F, E].
extern "C" int fg_moe_first(const void *x, int ldx, const void *w_in, void *y, int ldy, int dtype, const int *pair_expert,
                            const int *offsets, const int *order, const float *pair_weight, int M, int X, int top, int F, int E,
                            float limit, float alpha, cudaStream_t stream) {
    if (M <= 0) return 0;
    const int P = M * top;
    if (dtype != FG_F32 && dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
    if (P <= 64 && moe_grouped_ok(dtype, E, w_in) && moe_grouped_enabled()) {
        if (dtype == FG_F32) return moe_grouped_launch<float, true>(x, ldx, w_in, y, ldy, offsets, order, pair_weight, X, top, F, E, limit, alpha, stream);
        return moe_grouped_launch<bf16, true>(x, ldx, w_in, y, ldy, offsets, order, pair_weight, X, top, F, E, limit, alpha, stream);
    }
    if (P <= 64 && (size_t)E * 4 <= 48 * 1024) {
        dim3 grid((F + 8 * MR_ROWS_OF(true) - 1) / (8 * MR_ROWS_OF(true)), P);
        if (dtype == FG_F32)
            return fg_launch(moe_rows_kernel<float, true>, grid, dim3(256), (size_t)E * 4, stream, (const float *)x, ldx, (const float *)w_in,
                             y, ldy, pair_expert, order, pair_weight, top, X, F, E, limit, alpha);
        return fg_launch(moe_rows_kernel<bf16, true>, grid, dim3(256), (size_t)E * 4, stream, (const bf16 *)x, ldx, (const bf16 *)w_in, y, ldy,
                         pair_expert, order, pair_weight, top, X, F, E, limit, alpha);
    }
    dim3 grid((F + MT - 1) / MT, (P + MT - 1) / MT + X);
    if (grid.y > 65535) return FG_ERR_BAD_SIZE;
    if (dtype == FG_F32)
        return fg_launch(moe_tile_kernel<float, true>, grid, dim3(256), 0, stream, (const float *)x, ldx, (const float *)w_in, y, ldy, offsets,
                         order, pair_weight, X, top, F, E, limit, alpha);
    return fg_launch(moe_tile_kernel<bf16, true>, grid, dim3(256), 0, stream, (const bf16 *)x, ldx, (const bf16 *)w_in, y, ldy, offsets, order,
                     pair_weight, X, top, F, E, limit, alpha);
}

// out: [M * top, E] float32.  y: [M * top, F].  w_out: [X, E, F].
extern "C" int fg_moe_second(const void *y, int ldy, const void *w_out, float *out, int ldo, int dtype, const int *pair_expert,
                             const int *offsets, const int *order, int M, int X, int top, int F, int E, cudaStream_t stream) {
    if (M <= 0) return 0;
    const int P = M * top;
    if (dtype != FG_F32 && dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
    if (P <= 64 && moe_grouped_ok(dtype, F, w_out) && moe_grouped_enabled()) {
        if (dtype == FG_F32) return moe_grouped_launch<float, false>(y, ldy, w_out, out, ldo, offsets, order, nullptr, X, top, E, F, 0.f, 0.f, stream);
        return moe_grouped_launch<bf16, false>(y, ldy, w_out, out, ldo, offsets, order, nullptr, X, top, E, F, 0.f, 0.f, stream);
    }
    if (P <= 64 && (size_t)F * 4 <= 48 * 1024) {
        dim3 grid((E + 8 * MR_ROWS_OF(false) - 1) / (8 * MR_ROWS_OF(false)), P);
        if (dtype == FG_F32)
            return fg_launch(moe_rows_kernel<float, false>, grid, dim3(256), (size_t)F * 4, stream, (const float *)y, ldy, (const float *)w_out,
                             (void *)out, ldo, pair_expert, order, (const float *)nullptr, top, X, E, F, 0.f, 0.f);
        return fg_launch(moe_rows_kernel<bf16, false>, grid, dim3(256), (size_t)F * 4, stream, (const bf16 *)y, ldy, (const bf16 *)w_out,
                         (void *)out, ldo, pair_expert, order, (const float *)nullptr, top, X, E, F, 0.f, 0.f);
    }
    dim3 grid((E + MT - 1) / MT, (P + MT - 1) / MT + X);
    if (grid.y > 65535) return FG_ERR_BAD_SIZE;
    if (dtype == FG_F32)
        return fg_launch(moe_tile_kernel<float, false>, grid, dim3(256), 0, stream, (const float *)y, ldy, (const float *)w_out, (void *)out,
                         ldo, offsets, order, (const float *)nullptr, X, top, E, F, 0.f, 0.f);
    return fg_launch(moe_tile_kernel<bf16, false>, grid, dim3(256), 0, stream, (const bf16 *)y, ldy, (const bf16 *)w_out, (void *)out, ldo,
                     offsets, order, (const float *)nullptr, X, top, E, F, 0.f, 0.f);
}

// ------------------------------------------------------------------ long portions: the experts' contractions as plain ones
// With the rows of each expert side by side (xs[slot] = x[order[slot] / top]) an expert's contraction is an ordinary one
// over its run of slots, which the engine's tensor-core kernels take; these two kernels are what is left around them.
template <typename T>
__global__ void moe_gather_kernel(const T *__restrict__ x, int ldx, const int *__restrict__ order, int top, T *__restrict__ xs, int E) {
    pdl_launch_dependents();
    pdl_wait();
    const int slot = blockIdx.x;
    const T *src = x + (size_t)(order[slot] / top) * ldx;
    T *dst = xs + (size_t)slot * E;
    if (sizeof(T) == 2 && (E & 7) == 0 && (ldx & 7) == 0 && (((uintptr_t)x | (uintptr_t)xs) & 15) == 0) {
        for (int i = threadIdx.x; i < E / 8; i += blockDim.x) ((uint4 *)dst)[i] = ((const uint4 *)src)[i];
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) dst[i] = src[i];
    }
}

extern "C" int fg_moe_gather(const void *x, int ldx, int dtype, const int *order, int top, void *xs, int P, int E, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (dtype == FG_F32) return fg_launch(moe_gather_kernel<float>, dim3(P), dim3(128), 0, stream, (const float *)x, ldx, order, top, (float *)xs, E);
    if (dtype == FG_BF16) return fg_launch(moe_gather_kernel<bf16>, dim3(P), dim3(128), 0, stream, (const bf16 *)x, ldx, order, top, (bf16 *)xs, E);
    return FG_ERR_BAD_DTYPE;
}

// gu: [P, 2F] float32 (gate | up) of each slot -> y[P, F] = act(w gate, w up), w the slot's routing weight
template <typename T>
__global__ void moe_act_kernel(const float *__restrict__ gu, const int *__restrict__ order, const float *__restrict__ pair_weight,
                               T *__restrict__ y, int F, float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const int slot = blockIdx.x;
    const float w = pair_weight ? pair_weight[order[slot]] : 1.0f;
    const float *g = gu + (size_t)slot * 2 * F, *u = g + F;
    for (int i = threadIdx.x; i < F; i += blockDim.x) y[(size_t)slot * F + i] = from_f32<T>(expert_act(w * g[i], w * u[i], limit, alpha));
}

extern "C" int fg_moe_act(const float *gu, const int *order, const float *pair_weight, void *y, int dtype, int P, int F, float limit,
                          float alpha, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (dtype == FG_F32) return fg_launch(moe_act_kernel<float>, dim3(P), dim3(256), 0, stream, gu, order, pair_weight, (float *)y, F, limit, alpha);
    if (dtype == FG_BF16) return fg_launch(moe_act_kernel<bf16>, dim3(P), dim3(256), 0, stream, gu, order, pair_weight, (bf16 *)y, F, limit, alpha);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ sum of a row's experts, in the order of its choices
__global__ void moe_combine_kernel(const float *__restrict__ slot_out, int ld, const int *__restrict__ slot_of, float *__restrict__ t,
                                   int top, int E, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; k++) s += slot_out[(size_t)slot_of[r * top + k] * ld + i];
        if (accumulate) t[(size_t)r * E + i] += s;
        else t[(size_t)r * E + i] = s;
    }
}

extern "C" int fg_moe_combine(const float *slot_out, int ld, const int *slot_of, float *t, int M, int top, int E, int accumulate,
                              cudaStream_t stream) {
    if (M <= 0) return 0;
    return fg_launch(moe_combine_kernel, dim3(M), dim3(E >= 1024 ? 256 : 128), 0, stream, slot_out, ld, slot_of, t, top, E, accumulate);
}

// ------------------------------------------------------------------ weighted sum of a row's experts, in the order of its choices
// t[r] (+)= sum_k w[r, k] * (expert[r, k] < n_real ? slot_out[slot_of[r, k]] : x[r]): the routing weight multiplies the expert's
// OUTPUT, and a choice at or beyond n_real stands for the row's own input x (an "identity expert").
template <typename T>
__global__ void moe_combine_weighted_kernel(const float *__restrict__ slot_out, int ld, const int *__restrict__ slot_of,
                                            const int *__restrict__ pair_expert, const float *__restrict__ pair_weight,
                                            const T *__restrict__ x, int ldx, int n_real, float *__restrict__ t, int top, int E, int accumulate,
                                            int vec) {
    // the row's choices once: where each one's output lies (null: the row's own input) and its weight
    __shared__ const float *src[MOE_MAX_TOP];
    __shared__ float wt[MOE_MAX_TOP];
    // (no early release of the successor: this kernel stands between two tensor-memory contractions, and the second must not
    // start beside the first while this one sits resident and waiting; the successor starts when this kernel has finished)
    pdl_wait();
    const int r = blockIdx.x;
    if (threadIdx.x < top) {
        const int p = r * top + threadIdx.x;
        src[threadIdx.x] = pair_expert[p] < n_real ? slot_out + (size_t)slot_of[p] * ld : nullptr;
        wt[threadIdx.x] = pair_weight[p];
    }
    __syncthreads();
    const T *xr = x + (size_t)r * ldx;
    float *tr = t + (size_t)r * E;
    if (vec) {
        // four neighbours a thread: 16-byte loads of the experts' outputs and of the sum
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; k++) {
                float4 v;
                if (src[k]) v = *reinterpret_cast<const float4 *>(src[k] + i);
                else v = make_float4(to_f32<T>(xr[i]), to_f32<T>(xr[i + 1]), to_f32<T>(xr[i + 2]), to_f32<T>(xr[i + 3]));
                const float w = wt[k];
                s.x = fmaf(w, v.x, s.x); s.y = fmaf(w, v.y, s.y); s.z = fmaf(w, v.z, s.z); s.w = fmaf(w, v.w, s.w);
            }
            float4 *o = reinterpret_cast<float4 *>(tr + i);
            if (accumulate) { const float4 a = *o; s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
            *o = s;
        }
        return;
    }
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; k++) s = fmaf(wt[k], src[k] ? src[k][i] : to_f32<T>(xr[i]), s);
        if (accumulate) tr[i] += s;
        else tr[i] = s;
    }
}

extern "C" int fg_moe_combine_weighted(const float *slot_out, int ld, const int *slot_of, const int *pair_expert, const float *pair_weight,
                                       const void *x, int ldx, int dtype, int n_real, float *t, int M, int top, int E, int accumulate,
                                       cudaStream_t stream) {
    if (M <= 0) return 0;
    if (top <= 0 || top > MOE_MAX_TOP) return FG_ERR_BAD_SIZE;
    const int threads = E >= 1024 ? 256 : 128;
    const int vec = (E % 4 == 0 && ld % 4 == 0 && ((uintptr_t)slot_out & 15) == 0 && ((uintptr_t)t & 15) == 0) ? 1 : 0;
    if (dtype == FG_F32)
        return fg_launch(moe_combine_weighted_kernel<float>, dim3(M), dim3(threads), 0, stream, slot_out, ld, slot_of, pair_expert, pair_weight,
                         (const float *)x, ldx, n_real, t, top, E, accumulate, vec);
    if (dtype == FG_BF16)
        return fg_launch(moe_combine_weighted_kernel<bf16>, dim3(M), dim3(threads), 0, stream, slot_out, ld, slot_of, pair_expert, pair_weight,
                         (const bf16 *)x, ldx, n_real, t, top, E, accumulate, vec);
    return FG_ERR_BAD_DTYPE;
}
