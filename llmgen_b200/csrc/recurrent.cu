// Kernels of mixers that carry a fixed-size state from token to token instead of reading a cache of keys:
//
//   short_conv          a causal convolution over time on each channel by itself, whose first tokens of a step read the
//                       last inputs of the step before out of the request's state
//   conv_state_update   leaves the last K - 1 inputs of every sequence in its state
//   rglru_gates         per block of channels two small square products (recurrence gate and input gate) and from them
//                       the coefficients of the recurrence  S_t = a_t S_(t-1) + b_t
//   rglru_scan          that recurrence over each sequence's new tokens, times the other branch's gelu
//   delta_scan          the gated delta rule with a decay per key channel:
//                       S <- diag(g) S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q
//   token_shift_mix     several blends of every token's row with the row of the token before it, the last row of a
//                       sequence kept in its state:  m_i[t] = x[t] + (x[t-1] - x[t]) mu_i
//   decay_scan          linear attention with a decay per key channel, in two orders of a token's steps:
//                       S <- diag(a) S + k v^T;  o = S^T q                       (read after the update)
//                       o = (S + diag(u) k v^T)^T q;  S <- diag(a) S + k v^T     (read before it, a bonus on the own key)
//
// A step's sequences are given as everywhere else: sequence s owns token rows [cu_q[s], cu_q[s+1]), its state lies in
// slot state_slots[s] (-1: none; the sequence then starts from zeros and leaves nothing).  Rows beyond cu_q[n_seqs]
// belong to no sequence and are skipped, sequences without tokens too, so every launch here follows from a step's shape.
// Every state is float32; gates, decays, their logarithms and exponentials, unit norms and the recurrences are float32
// arithmetic in both storage dtypes.  The arithmetic of a token does not depend on where a step was cut.
#define LLMK_MODULE_NAME "recurrent"
#include "common.cuh"
#include <algorithm>

LLMK_DEFINE_LAST_ERROR()

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ int seq_of_row(const int* __restrict__ cu_q, int n_seqs, int t) {
    if (t >= cu_q[n_seqs]) return -1;
    int lo = 0, hi = n_seqs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cu_q[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------------------------------------ short convolution
// out[t, c] = act( sum_i taps[c, i] in(j - (K-1) + i, c) + conv_bias[c] ), j the token's index in its portion;
// in(r, c) = x[row of r, c] + in_bias[c] for r >= 0, else the state's row K - 1 + r (zeros for a fresh request).
template <typename T>
__global__ void short_conv_kernel(float* __restrict__ out, long long out_ld, const T* __restrict__ x, long long x_ld,
                                  const float* __restrict__ in_bias, const float* __restrict__ taps,
                                  const float* __restrict__ conv_bias, const float* __restrict__ state, long long state_ld,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int n_seqs, int C, int K,
                                  int act) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int s = seq_of_row(cu_q, n_seqs, t);
    if (s < 0) return;
    const int q_beg = cu_q[s];
    const int j = t - q_beg;
    const int slot = state_slots[s];
    const float b = in_bias ? in_bias[c] : 0.f;
    float acc = conv_bias ? conv_bias[c] : 0.f;
    for (int i = 0; i < K; ++i) {
        const int r = j - (K - 1) + i;
        float v;
        if (r >= 0) v = to_float(x[(size_t)(q_beg + r) * x_ld + c]) + b;
        else v = slot >= 0 ? state[(size_t)slot * state_ld + (size_t)(K - 1 + r) * C + c] : 0.f;
        acc = fmaf(taps[(size_t)c * K + i], v, acc);
    }
    out[(size_t)t * out_ld + c] = act == 1 ? acc / (1.0f + expf(-acc)) : acc;
}

template <typename T>
__global__ void conv_state_update_kernel(float* __restrict__ state, long long state_ld, const T* __restrict__ x, long long x_ld,
                                         const float* __restrict__ in_bias, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slots, int C, int K) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int q_beg = cu_q[s], n = cu_q[s + 1] - q_beg;
    const int slot = state_slots[s];
    if (n <= 0 || slot < 0) return;
    float* st = state + (size_t)slot * state_ld + c;
    const float b = in_bias ? in_bias[c] : 0.f;
    float old[MAX_TAPS];
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i) old[i] = i < K - 1 ? st[(size_t)i * C] : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i) {
        if (i >= K - 1) break;
        const int idx = n + i - (K - 1);      // among the step's own inputs
        float v;
        if (idx >= 0) v = to_float(x[(size_t)(q_beg + idx) * x_ld + c]) + b;
        else v = old[n + i];
        st[(size_t)i * C] = v;
    }
}

// Both in one launch for steps of a few tokens (single decoded tokens above all): a thread per (sequence, channel) walks
// the sequence's tokens with the last K - 1 inputs in registers and leaves them in the state.  The sum of a token is the
// one `short_conv_kernel` makes, term by term.
constexpr int SHORT_CONV_FEW_TOKENS = 64;

template <typename T>
__global__ void short_conv_few_kernel(float* __restrict__ out, long long out_ld, const T* __restrict__ x, long long x_ld,
                                      const float* __restrict__ in_bias, const float* __restrict__ taps,
                                      const float* __restrict__ conv_bias, float* __restrict__ state, long long state_ld,
                                      const int* __restrict__ cu_q, const int* __restrict__ state_slots, int C, int K, int act,
                                      int update_state) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int q_beg = cu_q[s], n = cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = state_slots[s];
    float* st = slot >= 0 && K > 1 ? state + (size_t)slot * state_ld + c : nullptr;
    const float b = in_bias ? in_bias[c] : 0.f, cb = conv_bias ? conv_bias[c] : 0.f;
    float w[MAX_TAPS], tp[MAX_TAPS];
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i) {
        tp[i] = i < K ? taps[(size_t)c * K + i] : 0.f;
        w[i] = (i < K - 1 && st) ? st[(size_t)i * C] : 0.f;       // w[0 .. K-2]: the inputs before the token, oldest first
    }
    for (int j = 0; j < n; ++j) {
        const float v = to_float(x[(size_t)(q_beg + j) * x_ld + c]) + b;
        float acc = cb;
#pragma unroll
        for (int i = 0; i < MAX_TAPS; ++i) {
            if (i < K - 1) acc = fmaf(tp[i], w[i], acc);
            else if (i == K - 1) acc = fmaf(tp[i], v, acc);
        }
        out[(size_t)(q_beg + j) * out_ld + c] = act == 1 ? acc / (1.0f + expf(-acc)) : acc;
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < K - 1) w[i] = i + 1 < K - 1 ? w[i + 1] : v;
    }
    if (st && update_state) {
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < K - 1) st[(size_t)i * C] = w[i];
    }
}

LLMK_EXPORT int llmk_short_conv(float* out, long long out_ld, const void* x, long long x_ld, const float* in_bias,
                                const float* taps, const float* conv_bias, float* state, long long state_ld, const int* cu_q,
                                const int* state_slots, int n_seqs, int n_tokens, int C, int K, int act, int update_state,
                                int dtype, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0 || C <= 0) return LLMK_OK;
    if (K < 1 || K > MAX_TAPS) LLMK_FAIL("short_conv: %d taps (1 to %d are built)", K, MAX_TAPS);
    if (!out || !x || !taps || (!state && K > 1) || !cu_q || !state_slots) LLMK_FAIL("short_conv: bad arguments");
    if (act != 0 && act != 1) LLMK_FAIL("short_conv: unknown activation %d (0: none, 1: silu)", act);
    if (n_tokens > 65535 || n_seqs > 65535) LLMK_FAIL("short_conv: a step of %d tokens in %d sequences is too large", n_tokens, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    dim3 grid(ceil_div(C, threads), n_tokens), ugrid(ceil_div(C, threads), n_seqs);
    cudaError_t e;
    if (n_tokens <= SHORT_CONV_FEW_TOKENS) {
        if (dtype == LLMK_F32)
            e = llmk_launch(short_conv_few_kernel<float>, ugrid, dim3(threads), 0, s, true, out, out_ld, (const float*)x, x_ld, in_bias,
                            taps, conv_bias, state, state_ld, cu_q, state_slots, C, K, act, update_state);
        else if (dtype == LLMK_BF16)
            e = llmk_launch(short_conv_few_kernel<bf16>, ugrid, dim3(threads), 0, s, true, out, out_ld, (const bf16*)x, x_ld, in_bias,
                            taps, conv_bias, state, state_ld, cu_q, state_slots, C, K, act, update_state);
        else
            LLMK_FAIL("short_conv: unknown dtype %d", dtype);
        LLMK_CHECK_LAUNCH_RC("short_conv", e);
        return LLMK_OK;
    }
    if (dtype == LLMK_F32) {
        e = llmk_launch(short_conv_kernel<float>, grid, dim3(threads), 0, s, true, out, out_ld, (const float*)x, x_ld, in_bias, taps,
                        conv_bias, (const float*)state, state_ld, cu_q, state_slots, n_seqs, C, K, act);
        if (e == cudaSuccess && update_state && K > 1)
            e = llmk_launch(conv_state_update_kernel<float>, ugrid, dim3(threads), 0, s, true, state, state_ld, (const float*)x, x_ld,
                            in_bias, cu_q, state_slots, C, K);
    } else if (dtype == LLMK_BF16) {
        e = llmk_launch(short_conv_kernel<bf16>, grid, dim3(threads), 0, s, true, out, out_ld, (const bf16*)x, x_ld, in_bias, taps,
                        conv_bias, (const float*)state, state_ld, cu_q, state_slots, n_seqs, C, K, act);
        if (e == cudaSuccess && update_state && K > 1)
            e = llmk_launch(conv_state_update_kernel<bf16>, ugrid, dim3(threads), 0, s, true, state, state_ld, (const bf16*)x, x_ld,
                            in_bias, cu_q, state_slots, C, K);
    } else
        LLMK_FAIL("short_conv: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("short_conv", e);
    return LLMK_OK;
}

// ------------------------------------------------------------------------------------------------ RG-LRU
// Block (tile of `GATE_OUT` outputs, block of channels b, tile of TT tokens): r = sigmoid(Ra_b u_b + ba), i = sigmoid(Ri_b u_b + bi),
// log a = -scale r softplus(lam), a = exp(log a), b = sqrt(1 - a^2) i u.  What leaves is c = 1 - a = -expm1(log a), not a: many
// a lie just below 1, where a float holds 1 - a to a few digits only and an exponential's last-bit error, always on the
// same side, would add up over the thousands of tokens such a channel remembers; 1 - a^2 = c (2 - c) without cancellation.
constexpr int GATE_OUT = 128;

template <typename T, int TT>
__global__ void __launch_bounds__(GATE_OUT) rglru_gates_kernel(float* __restrict__ a_out, float* __restrict__ b_out,
                                                               const float* __restrict__ u, const T* __restrict__ Wa,
                                                               const T* __restrict__ Wi, const float* __restrict__ ba,
                                                               const float* __restrict__ bi, const float* __restrict__ lam,
                                                               int n_tokens, int C, int n, float decay_scale, int vec_ok) {
    extern __shared__ __align__(16) float Us[];   // [TT][n]
    const int b = blockIdx.y, t0 = blockIdx.z * TT;
    const int o = blockIdx.x * GATE_OUT + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    for (int idx = threadIdx.x; idx < TT * n; idx += GATE_OUT) {
        const int tt = idx / n, k = idx % n;
        Us[idx] = t0 + tt < n_tokens ? u[(size_t)(t0 + tt) * C + (size_t)b * n + k] : 0.f;
    }
    __syncthreads();
    if (o >= n) return;
    float accA[TT], accI[TT];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) accA[tt] = accI[tt] = 0.f;
    const T* wa = Wa + ((size_t)b * n + o) * n;
    const T* wi = Wi + ((size_t)b * n + o) * n;
    constexpr int VN = Vec16<T>::N;
    int k = 0;
    if (vec_ok) {
        for (; k + VN <= n; k += VN) {
            Vec16<T> va, vi;
            va.raw = *reinterpret_cast<const decltype(va.raw)*>(wa + k);
            vi.raw = *reinterpret_cast<const decltype(vi.raw)*>(wi + k);
            float fa[VN], fi[VN];
            va.unpack(fa);
            vi.unpack(fi);
            // u comes four values a read (the rows of Us begin on 16-byte boundaries: n is a multiple of four here)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
                for (int j4 = 0; j4 < VN / 4; ++j4) {
                    const float4 u4 = *reinterpret_cast<const float4*>(Us + tt * n + k + 4 * j4);
                    accA[tt] = fmaf(fa[4 * j4], u4.x, accA[tt]);
                    accA[tt] = fmaf(fa[4 * j4 + 1], u4.y, accA[tt]);
                    accA[tt] = fmaf(fa[4 * j4 + 2], u4.z, accA[tt]);
                    accA[tt] = fmaf(fa[4 * j4 + 3], u4.w, accA[tt]);
                    accI[tt] = fmaf(fi[4 * j4], u4.x, accI[tt]);
                    accI[tt] = fmaf(fi[4 * j4 + 1], u4.y, accI[tt]);
                    accI[tt] = fmaf(fi[4 * j4 + 2], u4.z, accI[tt]);
                    accI[tt] = fmaf(fi[4 * j4 + 3], u4.w, accI[tt]);
                }
            }
        }
    }
    for (; k < n; ++k) {
        const float fa = to_float(wa[k]), fi = to_float(wi[k]);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            const float uv = Us[tt * n + k];
            accA[tt] = fmaf(fa, uv, accA[tt]);
            accI[tt] = fmaf(fi, uv, accI[tt]);
        }
    }
    const int c = b * n + o;
    const float sp = softplusf_(lam[c]);
    const float bias_a = ba ? ba[c] : 0.f, bias_i = bi ? bi[c] : 0.f;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        const int t = t0 + tt;
        if (t >= n_tokens) break;
        const float r = sigmoidf_(accA[tt] + bias_a);
        const float ig = sigmoidf_(accI[tt] + bias_i);
        const float loga = -decay_scale * r * sp;
        const float om = -expm1f(loga);
        a_out[(size_t)t * C + c] = om;
        b_out[(size_t)t * C + c] = sqrtf(om * (2.0f - om)) * ig * Us[tt * n + o];
    }
}

// Thread (sequence, channel): S = a S + b = (S - c S) + b over the sequence's new tokens (c = 1 - a, see above),
// out = S * gelu_tanh(y + y_bias).
template <typename T>
__global__ void rglru_scan_kernel(T* __restrict__ out, long long out_ld, const float* __restrict__ a, const float* __restrict__ bx,
                                  const T* __restrict__ y, long long y_ld, const float* __restrict__ y_bias,
                                  float* __restrict__ state, long long state_ld, const int* __restrict__ cu_q,
                                  const int* __restrict__ state_slots, int C) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int q_beg = cu_q[s], q_end = cu_q[s + 1];
    if (q_end <= q_beg) return;
    const int slot = state_slots[s];
    float S = slot >= 0 ? state[(size_t)slot * state_ld + c] : 0.f;
    const float yb = y_bias ? y_bias[c] : 0.f;
    int t = q_beg;
    for (; t + 4 <= q_end; t += 4) {
        float av[4], bv[4], yv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            av[i] = a[(size_t)(t + i) * C + c];
            bv[i] = bx[(size_t)(t + i) * C + c];
            yv[i] = to_float(y[(size_t)(t + i) * y_ld + c]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            S = fmaf(-av[i], S, S) + bv[i];
            out[(size_t)(t + i) * out_ld + c] = from_float<T>(S * gelu_tanhf_(yv[i] + yb));
        }
    }
    for (; t < q_end; ++t) {
        S = fmaf(-a[(size_t)t * C + c], S, S) + bx[(size_t)t * C + c];
        out[(size_t)t * out_ld + c] = from_float<T>(S * gelu_tanhf_(to_float(y[(size_t)t * y_ld + c]) + yb));
    }
    if (slot >= 0) state[(size_t)slot * state_ld + c] = S;
}

// The same scan for long portions, in three launches that run side by side over segments of SCAN_SEG tokens: every
// segment from an empty state (its local states stay in `bx`, the product of its decays and its last local state in
// `seg`), then a thread per (sequence, channel) takes the carried state through the segments' ends, then every segment
// adds its share of the state it was entered with.  Segments are counted sequence by sequence: segment j of the launch
// is the k-th of the first sequence s with j < sum of ceil(n_s' / SCAN_SEG) over s' <= s.
constexpr int SCAN_SEG = 64;

__device__ __forceinline__ bool find_segment(const int* __restrict__ cu_q, int n_seqs, int j, int* t0, int* t1) {
    for (int s = 0; s < n_seqs; ++s) {
        const int beg = cu_q[s], n = cu_q[s + 1] - beg;
        const int segs = (n + SCAN_SEG - 1) / SCAN_SEG;
        if (j < segs) {
            *t0 = beg + j * SCAN_SEG;
            *t1 = min(*t0 + SCAN_SEG, beg + n);
            return true;
        }
        j -= segs;
    }
    return false;
}

__global__ void rglru_segment_local_kernel(const float* __restrict__ a, float* __restrict__ bx, float* __restrict__ seg_p,
                                           float* __restrict__ seg_f, const int* __restrict__ cu_q, int n_seqs, int C) {
    const int j = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    int t0, t1;
    if (c >= C || !find_segment(cu_q, n_seqs, j, &t0, &t1)) return;
    // the product of the segment's decays as the exponential of their logarithms' sum: a running product would be
    // rounded at every token, always the same way where the decays hardly change, and the carried state takes a
    // segment's error 1 / (1 - product) times
    float S = 0.f, L = 0.f;
    int t = t0;
    for (; t + 8 <= t1; t += 8) {          // eight tokens' loads in flight at a time
        float cv[8], bv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            cv[i] = a[(size_t)(t + i) * C + c];
            bv[i] = bx[(size_t)(t + i) * C + c];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            S = fmaf(-cv[i], S, S) + bv[i];
            L += log1pf(-cv[i]);
            bx[(size_t)(t + i) * C + c] = S;
        }
    }
    for (; t < t1; ++t) {
        const float cv = a[(size_t)t * C + c];
        S = fmaf(-cv, S, S) + bx[(size_t)t * C + c];
        L += log1pf(-cv);
        bx[(size_t)t * C + c] = S;
    }
    seg_p[(size_t)j * C + c] = expf(L);
    seg_f[(size_t)j * C + c] = S;
}

// seg_f[j] becomes the state segment j is entered with
__global__ void rglru_segment_carry_kernel(const float* __restrict__ seg_p, float* __restrict__ seg_f, float* __restrict__ state,
                                           long long state_ld, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                           int C) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int n = cu_q[s + 1] - cu_q[s];
    if (n <= 0) return;
    int j = 0;
    for (int k = 0; k < s; ++k) j += (cu_q[k + 1] - cu_q[k] + SCAN_SEG - 1) / SCAN_SEG;
    const int slot = state_slots[s];
    float carry = slot >= 0 ? state[(size_t)slot * state_ld + c] : 0.f;
    const int segs = (n + SCAN_SEG - 1) / SCAN_SEG;
    for (int k = 0; k < segs; ++k, ++j) {
        const float in = carry;
        carry = fmaf(seg_p[(size_t)j * C + c], carry, seg_f[(size_t)j * C + c]);
        seg_f[(size_t)j * C + c] = in;
    }
    if (slot >= 0) state[(size_t)slot * state_ld + c] = carry;
}

template <typename T>
__global__ void rglru_segment_finish_kernel(T* __restrict__ out, long long out_ld, const float* __restrict__ a,
                                            const float* __restrict__ local, const float* __restrict__ seg_in,
                                            const T* __restrict__ y, long long y_ld, const float* __restrict__ y_bias,
                                            const int* __restrict__ cu_q, int n_seqs, int C) {
    const int j = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    int t0, t1;
    if (c >= C || !find_segment(cu_q, n_seqs, j, &t0, &t1)) return;
    const float in = seg_in[(size_t)j * C + c];
    const float yb = y_bias ? y_bias[c] : 0.f;
    float L = 0.f;
    int t = t0;
    for (; t + 8 <= t1; t += 8) {
        float cv[8], lv[8], yv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            cv[i] = a[(size_t)(t + i) * C + c];
            lv[i] = local[(size_t)(t + i) * C + c];
            yv[i] = to_float(y[(size_t)(t + i) * y_ld + c]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            L += log1pf(-cv[i]);
            const float S = fmaf(expf(L), in, lv[i]);
            out[(size_t)(t + i) * out_ld + c] = from_float<T>(S * gelu_tanhf_(yv[i] + yb));
        }
    }
    for (; t < t1; ++t) {
        L += log1pf(-a[(size_t)t * C + c]);
        const float S = fmaf(expf(L), in, local[(size_t)t * C + c]);
        out[(size_t)t * out_ld + c] = from_float<T>(S * gelu_tanhf_(to_float(y[(size_t)t * y_ld + c]) + yb));
    }
}

// Rows of float32 scratch [rows, C] that `llmk_rglru` needs for a step of this shape: the two coefficient arrays and, for
// the steps whose scan runs in segments, two values a segment.
static bool rglru_in_segments(int n_tokens, int dtype) { return dtype == LLMK_BF16 && n_tokens >= 8 * SCAN_SEG; }
LLMK_EXPORT long long llmk_rglru_scratch_rows(int n_tokens, int n_seqs, int dtype) {
    long long rows = 2LL * n_tokens;
    if (rglru_in_segments(n_tokens, dtype)) rows += 2LL * (n_tokens / SCAN_SEG + n_seqs);
    return rows;
}

template <typename T>
static int launch_rglru(void* out, long long out_ld, float* a_buf, float* b_buf, const float* u, const void* Wa, const void* Wi,
                        const float* ba, const float* bi, const float* lam, const void* y, long long y_ld, const float* y_bias,
                        float* state, long long state_ld, const int* cu_q, const int* state_slots, int n_seqs, int n_tokens, int C,
                        int blocks, float decay_scale, cudaStream_t s) {
    const int n = C / blocks;
    constexpr int VN = Vec16<T>::N;
    const int vec_ok = (n % VN == 0 && host_aligned16(Wa) && host_aligned16(Wi)) ? 1 : 0;
    // tokens a block of the gates' kernel takes: as many as keep its rows of u within 64 KB of shared memory
    int tt = 16;
    while (tt > 1 && (size_t)tt * n * sizeof(float) > 64 * 1024) tt >>= 1;
    if (n_tokens <= 4 && tt > 4) tt = 4;
    const size_t smem = (size_t)tt * n * sizeof(float);
    if (smem > 200 * 1024) LLMK_FAIL("rglru: blocks of %d channels do not fit shared memory", n);
    dim3 ggrid(ceil_div(n, GATE_OUT), blocks, ceil_div(n_tokens, tt));
    if (ggrid.z > 65535) LLMK_FAIL("rglru: a step of %d tokens is too large", n_tokens);
    cudaError_t e;
#define LAUNCH_GATES(TTV)                                                                                                       \
    do {                                                                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(rglru_gates_kernel<T, TTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        e = llmk_launch(rglru_gates_kernel<T, TTV>, ggrid, dim3(GATE_OUT), smem, s, true, a_buf, b_buf, u, (const T*)Wa, (const T*)Wi, \
                        ba, bi, lam, n_tokens, C, n, decay_scale, vec_ok);                                                        \
    } while (0)
    if (tt == 16) LAUNCH_GATES(16);
    else if (tt == 8) LAUNCH_GATES(8);
    else if (tt == 4) LAUNCH_GATES(4);
    else if (tt == 2) LAUNCH_GATES(2);
    else LAUNCH_GATES(1);
#undef LAUNCH_GATES
    LLMK_CHECK_LAUNCH_RC("rglru_gates", e);
    const int threads = 128;
    if (rglru_in_segments(n_tokens, sizeof(T) == 2 ? LLMK_BF16 : LLMK_F32)) {
        const int max_segs = n_tokens / SCAN_SEG + n_seqs;
        float* seg_p = b_buf + (size_t)n_tokens * C;
        float* seg_f = seg_p + (size_t)max_segs * C;
        if (max_segs > 65535) LLMK_FAIL("rglru: a step of %d tokens is too large", n_tokens);
        e = llmk_launch(rglru_segment_local_kernel, dim3(ceil_div(C, threads), max_segs), dim3(threads), 0, s, true,
                        (const float*)a_buf, b_buf, seg_p, seg_f, cu_q, n_seqs, C);
        LLMK_CHECK_LAUNCH_RC("rglru_segment_local", e);
        e = llmk_launch(rglru_segment_carry_kernel, dim3(ceil_div(C, threads), n_seqs), dim3(threads), 0, s, true,
                        (const float*)seg_p, seg_f, state, state_ld, cu_q, state_slots, C);
        LLMK_CHECK_LAUNCH_RC("rglru_segment_carry", e);
        e = llmk_launch(rglru_segment_finish_kernel<T>, dim3(ceil_div(C, threads), max_segs), dim3(threads), 0, s, true, (T*)out,
                        out_ld, (const float*)a_buf, (const float*)b_buf, (const float*)seg_f, (const T*)y, y_ld, y_bias, cu_q,
                        n_seqs, C);
        LLMK_CHECK_LAUNCH_RC("rglru_segment_finish", e);
        return LLMK_OK;
    }
    e = llmk_launch(rglru_scan_kernel<T>, dim3(ceil_div(C, threads), n_seqs), dim3(threads), 0, s, true, (T*)out, out_ld,
                    (const float*)a_buf, (const float*)b_buf, (const T*)y, y_ld, y_bias, state, state_ld, cu_q, state_slots, C);
    LLMK_CHECK_LAUNCH_RC("rglru_scan", e);
    return LLMK_OK;
}

// out[t, c] (storage dtype) = S_t[c] * gelu_tanh(y[t, c] + y_bias[c]);  u float32 [n_tokens, C] is the convolution's output;
// a_buf: float32 scratch [n_tokens, C]; b_buf: the same, followed by what `llmk_rglru_scratch_rows` adds for the segments.
// The float32 engine always scans a sequence's tokens in turn (a thread per channel); the bfloat16 engine cuts steps of
// 512 tokens and more into segments.
LLMK_EXPORT int llmk_rglru(void* out, long long out_ld, float* a_buf, float* b_buf, const float* u, const void* Wa, const void* Wi,
                           const float* ba, const float* bi, const float* lam, const void* y, long long y_ld, const float* y_bias,
                           float* state, long long state_ld, const int* cu_q, const int* state_slots, int n_seqs, int n_tokens, int C,
                           int blocks, float decay_scale, int dtype, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return LLMK_OK;
    if (C <= 0 || blocks <= 0 || C % blocks != 0) LLMK_FAIL("rglru: %d channels are not cut evenly into %d blocks", C, blocks);
    if (!out || !a_buf || !b_buf || !u || !Wa || !Wi || !lam || !y || !state || !cu_q || !state_slots) LLMK_FAIL("rglru: bad arguments");
    if (n_seqs > 65535 || blocks > 65535) LLMK_FAIL("rglru: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == LLMK_F32)
        return launch_rglru<float>(out, out_ld, a_buf, b_buf, u, Wa, Wi, ba, bi, lam, y, y_ld, y_bias, state, state_ld, cu_q,
                                   state_slots, n_seqs, n_tokens, C, blocks, decay_scale, s);
    if (dtype == LLMK_BF16)
        return launch_rglru<bf16>(out, out_ld, a_buf, b_buf, u, Wa, Wi, ba, bi, lam, y, y_ld, y_bias, state, state_ld, cu_q,
                                  state_slots, n_seqs, n_tokens, C, blocks, decay_scale, s);
    LLMK_FAIL("rglru: unknown dtype %d", dtype);
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// Two launches.  `delta_prep`, a block per token, works in place: q and k (float32, after convolution and silu) become
// unit vectors per head (q also times key_dim^-1/2), the decays' pre-activations become 1 - g = -expm1(-exp(A_log_h)
// softplus(x + dt_bias)) (a decay just below 1 keeps its digits only as its distance from 1), beta goes through its sigmoid,
// and q . k of every key head is left beside it.  With S' = diag(g) S the token's read-out is
// o = S^T q = S'^T q + (q . k) d, so both dot products over the key channels run over S' in one pass and the update
// S = S' + k d^T ends the token: one chain of dependent steps a token instead of two.
// `delta_scan`, a block of four warps per (sequence, head, tile of value columns): SL lanes share one column of S, each
// holding a contiguous run of DSL key channels, so the dot products of a token over the key channels end in log2(SL)
// shuffles.  A token's time is its chain of dependent steps (there is one warp a scheduler), which is shortest with many
// lanes a column: 16 for key widths from 33 (8 value columns a block, 128 blocks for 8 heads of 128 columns).  The tokens come in chunks of DELTA_CHUNK through shared memory, the next chunk copied
// (cp.async) while the columns walk the present one token by token.
constexpr int DELTA_CHUNK = 16;
constexpr int DELTA_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(256) delta_prep_kernel(float* __restrict__ qkv, long long qkv_ld, float* __restrict__ decay,
                                                         float* __restrict__ beta_out, const T* __restrict__ beta, long long beta_ld,
                                                         const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                         int H, int G, int D, float unit_eps, float q_scale) {
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    for (int head = warp; head < G; head += warps) {              // q and k of one key head, and their dot product
        float* xq = qkv + t * qkv_ld + (size_t)head * D;
        float* xk = xq + (size_t)G * D;
        float sq = 0.f, sk = 0.f;
        for (int d = lane; d < D; d += 32) {
            sq += xq[d] * xq[d];
            sk += xk[d] * xk[d];
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float qv = xq[d] * fq, kv = xk[d] * fk;
            xq[d] = qv;
            xk[d] = kv;
            dot = fmaf(qv, kv, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) beta_out[t * (H + G) + H + head] = dot;
    }
    const int HD = H * D;
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
        const float neg_exp_a = -expf(a_log[i / D]);
        decay[t * HD + i] = -expm1f(neg_exp_a * softplusf_(decay[t * HD + i] + dt_bias[i]));
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) beta_out[t * (H + G) + h] = sigmoidf_(to_float(beta[t * beta_ld + h]));
}

struct DeltaParams {
    float* out;              // [n_tokens, H * E]
    const float* qkv;        // [n_tokens, ld]: q at column 0, k at G * D, v at 2 * G * D, prepared
    long long qkv_ld;
    const float* beta;       // [n_tokens, H + G]: beta of every head, then q . k of every key head
    const float* decay;      // [n_tokens, H * D]: 1 - g
    float* state;            // [slots, state_ld]: S [H][D][E]
    long long state_ld;
    const int* cu_q;
    const int* state_slots;
    int H, G, D, E, vec_ok;
};

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// One chunk's rows into shared memory: q, k, 1 - g as [CHUNK][SL slices][STRIDE] (the padding keeps the slices' 16-byte
// reads on different banks), v as [CHUNK][COLS], then beta [CHUNK] and q . k [CHUNK].
template <int DSL, int SL, int WARPS = 4>
struct DeltaShape {
    static constexpr int STRIDE = DSL == 4 ? 12 : DSL + 4;
    static constexpr int ROW = SL * STRIDE;
    static constexpr int COLS = WARPS * (32 / SL);
    static constexpr int BUF = DELTA_CHUNK * (3 * ROW + COLS) + 2 * DELTA_CHUNK;
};

template <int DSL, int SL, int WARPS = 4>
__device__ __forceinline__ void delta_load_chunk(const DeltaParams& p, float* buf, int t_first, int nc, int h, int kvh, int e0) {
    using Sh = DeltaShape<DSL, SL, WARPS>;
    constexpr int ROW = Sh::ROW, COLS = Sh::COLS, STRIDE = Sh::STRIDE;
    float* qs = buf;
    float* ks = qs + DELTA_CHUNK * ROW;
    float* gs = ks + DELTA_CHUNK * ROW;
    float* vs = gs + DELTA_CHUNK * ROW;
    float* bs = vs + DELTA_CHUNK * COLS;
    const int D = p.D, E = p.E, GD = p.G * p.D;
    if (p.vec_ok) {
        const int vecs = D / 4;
        for (int idx = threadIdx.x; idx < nc * vecs; idx += WARPS * 32) {
            const int tt = idx / vecs, d = (idx % vecs) * 4;
            const size_t t = (size_t)(t_first + tt);
            const int at = tt * ROW + (d / DSL) * STRIDE + d % DSL;
            cp_async16(qs + at, p.qkv + t * p.qkv_ld + (size_t)kvh * D + d);
            cp_async16(ks + at, p.qkv + t * p.qkv_ld + GD + (size_t)kvh * D + d);
            cp_async16(gs + at, p.decay + t * ((size_t)p.H * D) + (size_t)h * D + d);
        }
        for (int idx = threadIdx.x; idx < nc * (COLS / 4); idx += WARPS * 32) {
            const int tt = idx / (COLS / 4), cc = (idx % (COLS / 4)) * 4;
            if (e0 + cc < E) cp_async16(vs + tt * COLS + cc, p.qkv + (size_t)(t_first + tt) * p.qkv_ld + 2 * GD + (size_t)h * E + e0 + cc);
        }
    } else {
        for (int idx = threadIdx.x; idx < nc * D; idx += WARPS * 32) {
            const int tt = idx / D, d = idx % D;
            const size_t t = (size_t)(t_first + tt);
            const int at = tt * ROW + (d / DSL) * STRIDE + d % DSL;
            qs[at] = p.qkv[t * p.qkv_ld + (size_t)kvh * D + d];
            ks[at] = p.qkv[t * p.qkv_ld + GD + (size_t)kvh * D + d];
            gs[at] = p.decay[t * ((size_t)p.H * D) + (size_t)h * D + d];
        }
        for (int idx = threadIdx.x; idx < nc * COLS; idx += WARPS * 32) {
            const int tt = idx / COLS, cc = idx % COLS;
            if (e0 + cc < E) vs[idx] = p.qkv[(size_t)(t_first + tt) * p.qkv_ld + 2 * GD + (size_t)h * E + e0 + cc];
        }
    }
    if (threadIdx.x < nc) {
        const float* row = p.beta + (size_t)(t_first + threadIdx.x) * (p.H + p.G);
        bs[threadIdx.x] = row[h];
        bs[DELTA_CHUNK + threadIdx.x] = row[p.H + kvh];
    }
}

template <int DSL, int SL>
__global__ void __launch_bounds__(DELTA_THREADS) delta_scan_kernel(DeltaParams p) {
    using Sh = DeltaShape<DSL, SL>;
    constexpr int ROW = Sh::ROW, COLS = Sh::COLS, STRIDE = Sh::STRIDE, BUF = Sh::BUF;
    extern __shared__ __align__(16) float sm[];
    const int s = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slice = lane % SL, col = warp * (32 / SL) + lane / SL;
    const int e = e0 + col;
    const int D = p.D, E = p.E;
    const int kvh = h / (p.H / p.G);
    // channels beyond key_dim, and value columns beyond value_dim, hold zeros throughout (no decay: 1 - g = 0)
    for (int i = threadIdx.x; i < 2 * BUF; i += DELTA_THREADS) sm[i] = 0.f;
    pdl_launch_dependents();
    pdl_wait();
    const int q_beg = p.cu_q[s], n = p.cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = p.state_slots[s];
    float S[DSL];
    float* st = slot >= 0 ? p.state + (size_t)slot * p.state_ld + (size_t)h * D * E : nullptr;
#pragma unroll
    for (int i = 0; i < DSL; ++i) {
        const int d = slice * DSL + i;
        S[i] = (st && d < D && e < E) ? st[(size_t)d * E + e] : 0.f;
    }
    __syncthreads();
    delta_load_chunk<DSL, SL>(p, sm, q_beg, min(DELTA_CHUNK, n), h, kvh, e0);
    int turn = 0;
    for (int c0 = 0; c0 < n; c0 += DELTA_CHUNK, turn ^= 1) {
        const int nc = min(DELTA_CHUNK, n - c0);
        cp_async_wait_all();
        __syncthreads();      // this chunk has arrived, and the chunk before is consumed by every warp
        if (c0 + DELTA_CHUNK < n)
            delta_load_chunk<DSL, SL>(p, sm + (turn ^ 1) * BUF, q_beg + c0 + DELTA_CHUNK, min(DELTA_CHUNK, n - c0 - DELTA_CHUNK), h, kvh, e0);
        const float* buf = sm + turn * BUF;
        const float* vs = buf + 3 * DELTA_CHUNK * ROW;
        const float* bs = vs + DELTA_CHUNK * COLS;
        auto token = [&](int tt) {
            const float4* qr = reinterpret_cast<const float4*>(buf + tt * ROW + slice * STRIDE);
            const float4* kr = reinterpret_cast<const float4*>(buf + DELTA_CHUNK * ROW + tt * ROW + slice * STRIDE);
            const float4* gr = reinterpret_cast<const float4*>(buf + 2 * DELTA_CHUNK * ROW + tt * ROW + slice * STRIDE);
            float4 kk[DSL / 4];
            float ks4[4] = {0.f, 0.f, 0.f, 0.f}, qs4[4] = {0.f, 0.f, 0.f, 0.f};   // four sums in turn: short chains of dependent adds
#pragma unroll
            for (int i = 0; i < DSL / 4; ++i) {
                const float4 g4 = gr[i], k4 = kr[i], q4 = qr[i];
                kk[i] = k4;
                S[4 * i] = fmaf(-g4.x, S[4 * i], S[4 * i]);
                S[4 * i + 1] = fmaf(-g4.y, S[4 * i + 1], S[4 * i + 1]);
                S[4 * i + 2] = fmaf(-g4.z, S[4 * i + 2], S[4 * i + 2]);
                S[4 * i + 3] = fmaf(-g4.w, S[4 * i + 3], S[4 * i + 3]);
                ks4[0] = fmaf(k4.x, S[4 * i], ks4[0]);
                ks4[1] = fmaf(k4.y, S[4 * i + 1], ks4[1]);
                ks4[2] = fmaf(k4.z, S[4 * i + 2], ks4[2]);
                ks4[3] = fmaf(k4.w, S[4 * i + 3], ks4[3]);
                qs4[0] = fmaf(q4.x, S[4 * i], qs4[0]);
                qs4[1] = fmaf(q4.y, S[4 * i + 1], qs4[1]);
                qs4[2] = fmaf(q4.z, S[4 * i + 2], qs4[2]);
                qs4[3] = fmaf(q4.w, S[4 * i + 3], qs4[3]);
            }
            float kS = (ks4[0] + ks4[1]) + (ks4[2] + ks4[3]);
            float qS = (qs4[0] + qs4[1]) + (qs4[2] + qs4[3]);
#pragma unroll
            for (int o = 1; o < SL; o <<= 1) {
                kS += __shfl_xor_sync(0xffffffffu, kS, o);
                qS += __shfl_xor_sync(0xffffffffu, qS, o);
            }
            const float dlt = bs[tt] * (vs[tt * COLS + col] - kS);
            const float o = fmaf(bs[DELTA_CHUNK + tt], dlt, qS);
#pragma unroll
            for (int i = 0; i < DSL / 4; ++i) {
                S[4 * i] = fmaf(kk[i].x, dlt, S[4 * i]);
                S[4 * i + 1] = fmaf(kk[i].y, dlt, S[4 * i + 1]);
                S[4 * i + 2] = fmaf(kk[i].z, dlt, S[4 * i + 2]);
                S[4 * i + 3] = fmaf(kk[i].w, dlt, S[4 * i + 3]);
            }
            if (slice == 0 && e < E) p.out[(size_t)(q_beg + c0 + tt) * ((size_t)p.H * E) + (size_t)h * E + e] = o;
        };
        if (nc == DELTA_CHUNK) {      // a whole chunk: the addresses are constants, and a token's tail runs under the next one's head
#pragma unroll
            for (int tt = 0; tt < DELTA_CHUNK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nc; ++tt) token(tt);
        }
    }
    if (st) {
#pragma unroll
        for (int i = 0; i < DSL; ++i) {
            const int d = slice * DSL + i;
            if (d < D && e < E) st[(size_t)d * E + e] = S[i];
        }
    }
}

template <int DSL, int SL>
static cudaError_t launch_delta(const DeltaParams& p, int n_seqs, cudaStream_t s) {
    using Sh = DeltaShape<DSL, SL>;
    const size_t smem = 2 * (size_t)Sh::BUF * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<DSL, SL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    dim3 grid(n_seqs, p.H, ceil_div(p.E, Sh::COLS));
    return llmk_launch(delta_scan_kernel<DSL, SL>, grid, dim3(DELTA_THREADS), smem, s, true, p);
}

// qkv float32 [n_tokens, >= 2 G D + H E] and decay float32 [n_tokens, H D] are rewritten in place by the preparation;
// beta_buf: float32 scratch [n_tokens, H + G].  dtype: of `beta` (the storage dtype of the projection it is a column of).
LLMK_EXPORT int llmk_delta_scan(float* out, float* qkv, long long qkv_ld, const void* beta, long long beta_ld, float* decay,
                                float* beta_buf, const float* dt_bias, const float* a_log, float* state, long long state_ld,
                                const int* cu_q, const int* state_slots, int n_seqs, int n_tokens, int H, int G, int D, int E,
                                float unit_eps, float q_scale, int dtype, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return LLMK_OK;
    if (H <= 0 || G <= 0 || H % G != 0) LLMK_FAIL("delta_scan: %d heads are not a multiple of %d key heads", H, G);
    if (D <= 0 || D > 256 || E <= 0) LLMK_FAIL("delta_scan: key width %d (at most 256) or value width %d", D, E);
    if (!out || !qkv || !beta || !decay || !beta_buf || !dt_bias || !a_log || !state || !cu_q || !state_slots) LLMK_FAIL("delta_scan: bad arguments");
    if (H > 65535 || ceil_div(E, 8) > 65535) LLMK_FAIL("delta_scan: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(delta_prep_kernel<float>, dim3(n_tokens), dim3(256), 0, s, true, qkv, qkv_ld, decay, beta_buf, (const float*)beta,
                        beta_ld, dt_bias, a_log, H, G, D, unit_eps, q_scale);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(delta_prep_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, true, qkv, qkv_ld, decay, beta_buf, (const bf16*)beta,
                        beta_ld, dt_bias, a_log, H, G, D, unit_eps, q_scale);
    else
        LLMK_FAIL("delta_scan: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("delta_prep", e);
    DeltaParams p;
    p.out = out; p.qkv = qkv; p.qkv_ld = qkv_ld; p.beta = beta_buf; p.decay = decay;
    p.state = state; p.state_ld = state_ld; p.cu_q = cu_q; p.state_slots = state_slots;
    p.H = H; p.G = G; p.D = D; p.E = E;
    // 16-byte copies: every row of q, k, v and of the decays begins on a 16-byte boundary
    p.vec_ok = (D % 4 == 0 && E % 4 == 0 && qkv_ld % 4 == 0 && host_aligned16(qkv) && host_aligned16(decay)) ? 1 : 0;
    if (D <= 32) e = launch_delta<4, 8>(p, n_seqs, s);
    else if (D <= 64) e = launch_delta<4, 16>(p, n_seqs, s);
    else if (D <= 128) e = launch_delta<8, 16>(p, n_seqs, s);
    else e = launch_delta<16, 16>(p, n_seqs, s);
    LLMK_CHECK_LAUNCH_RC("delta_scan", e);
    return LLMK_OK;
}


// ------------------------------------------------------------------------------------------------ token shift
// out[i][t, c] = x[t, c] + (prev(t)[c] - x[t, c]) * mu[i][c] for i < n_mix, prev(t) the row of the token before t in its
// sequence: the row above inside a step, the state's row for a step's first token (zeros for a fresh request).  The thread
// that reads a sequence's state row also leaves the sequence's last row there, after reading, so that no other thread's
// read meets the write.
template <typename T>
__global__ void token_shift_mix_kernel(T* __restrict__ out, long long out_plane, const T* __restrict__ x, long long x_ld,
                                       const float* __restrict__ mu, float* __restrict__ state, long long state_ld,
                                       const int* __restrict__ cu_q, const int* __restrict__ state_slots, int n_seqs, int W,
                                       int n_mix) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= W) return;
    const int s = seq_of_row(cu_q, n_seqs, t);
    if (s < 0) return;
    const int q_beg = cu_q[s], q_end = cu_q[s + 1];
    const float cur = to_float(x[(size_t)t * x_ld + c]);
    float prev;
    if (t > q_beg) {
        prev = to_float(x[(size_t)(t - 1) * x_ld + c]);
    } else {
        const int slot = state_slots[s];
        float* st = slot >= 0 ? state + (size_t)slot * state_ld + c : nullptr;
        prev = st ? *st : 0.f;
        if (st) *st = to_float(x[(size_t)(q_end - 1) * x_ld + c]);
    }
    const float d = prev - cur;
    for (int i = 0; i < n_mix; ++i)
        out[(size_t)i * out_plane + (size_t)t * W + c] = from_float<T>(fmaf(d, mu[(size_t)i * W + c], cur));
}

// out: [n_mix] planes of [n_tokens, W] of the storage dtype, `out_plane` elements apart; mu float32 [n_mix, W];
// state float32, the row of slot s at state + s * state_ld.
LLMK_EXPORT int llmk_token_shift_mix(void* out, long long out_plane, const void* x, long long x_ld, const float* mu, float* state,
                                     long long state_ld, const int* cu_q, const int* state_slots, int n_seqs, int n_tokens, int W,
                                     int n_mix, int dtype, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return LLMK_OK;
    if (W <= 0 || n_mix <= 0 || !out || !x || !mu || !state || !cu_q || !state_slots) LLMK_FAIL("token_shift_mix: bad arguments");
    if (n_tokens > 65535) {
        // the grid's second dimension counts tokens
        LLMK_FAIL("token_shift_mix: %d token rows exceed 65535", n_tokens);
    }
    dim3 grid(ceil_div(W, 256), n_tokens);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(token_shift_mix_kernel<float>, grid, dim3(256), 0, s, true, (float*)out, out_plane, (const float*)x, x_ld, mu, state,
                        state_ld, cu_q, state_slots, n_seqs, W, n_mix);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(token_shift_mix_kernel<bf16>, grid, dim3(256), 0, s, true, (bf16*)out, out_plane, (const bf16*)x, x_ld, mu, state,
                        state_ld, cu_q, state_slots, n_seqs, W, n_mix);
    else
        LLMK_FAIL("token_shift_mix: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("token_shift_mix", e);
    return LLMK_OK;
}

// ------------------------------------------------------------------------------------------------ decay per key channel
// Two launches, as for the delta rule.  `decay_prep`, a block per token: q, k, v of the storage dtype go into one float32
// row [q * q_scale | k | v]; the decays' pre-activations z (float32, [H * D]) become 1 - a, with
//     mode 0   a = sigmoid(z + b)^(1 / tau)   log a = -softplus(-(z + b)) / tau
//     mode 1   a = exp(-exp(z + b))           log a = -exp(z + b)
// and 1 - a = -expm1(log a): a decay just below one keeps its digits only as its distance from one.  Beside them the
// token's own term, dot[h] = sum_d q_d k_d u_d (u the bonus [H, D], or ones).
// `decay_scan` has the delta rule's shape (a block per (sequence, head, tile of value columns), SL lanes a column of S,
// chunks of tokens through shared memory): the token's read-out is q^T S' + dot * v with S' the state after its decay
// (read after the update: (S' + k v^T)^T q = S'^T q + (q.k) v), or q^T S + dot * v with the state before it.
enum { DECAY_SIGMOID_POW = 0, DECAY_EXP_EXP = 1 };

template <typename T>
__global__ void __launch_bounds__(256) decay_prep_kernel(float* __restrict__ qkv, long long qkv_ld, float* __restrict__ decay,
                                                         float* __restrict__ dots, const T* __restrict__ q, long long q_ld,
                                                         const T* __restrict__ k, long long k_ld, const T* __restrict__ v,
                                                         long long v_ld, const float* __restrict__ bias, const float* __restrict__ bonus,
                                                         int H, int D, int E, int mode, float inv_tau, float q_scale) {
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    float* row = qkv + t * qkv_ld;
    const int HD = H * D, HE = H * E;
    for (int head = warp; head < H; head += warps) {
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) {
            const int i = head * D + d;
            const float qv = to_float(q[t * q_ld + i]) * q_scale, kv = to_float(k[t * k_ld + i]);
            row[i] = qv;
            row[HD + i] = kv;
            dot = fmaf(qv * (bonus ? bonus[i] : 1.f), kv, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) {
            dots[t * 2 * H + head] = 1.f;
            dots[t * 2 * H + H + head] = dot;
        }
    }
    for (int i = threadIdx.x; i < HE; i += blockDim.x) row[2 * HD + i] = to_float(v[t * v_ld + i]);
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
        const float z = decay[t * HD + i] + (bias ? bias[i] : 0.f);
        const float log_a = mode == DECAY_SIGMOID_POW ? -softplusf_(-z) * inv_tau : -expf(z);
        decay[t * HD + i] = -expm1f(log_a);
    }
}

// Long sequences are walked in segments side by side (PART 1, then PART 2); PART 0 walks whole sequences.  With
// S_end = diag(P) S_start + L for a segment (P the product of its decays, L its state from nothing):
//   PART 1   segment 0 of a sequence runs as in PART 0, from the request's state and with its read-outs, and leaves its
//            end state; every later segment but the last starts from nothing, reads nothing out and leaves L and P
//            (P = exp(sum log1p(-(1 - a))): a running product would round at every token, the same way where decays
//            hardly change)
//   PART 2   every segment but the first folds the states before it into its start (S <- P_i S + L_i, a few reads of the
//            state a block), walks its tokens with their read-outs, and the last leaves the request's state
// A token's arithmetic is PART 0's; what differs is the grouping of the sums that make a segment's start.
struct DecaySegments {
    float* state;            // [n_seqs * max_segs][H][D][E]: segment j of sequence s at s * max_segs + j
    float* decay;            // [n_seqs * max_segs][H][D]: P
    int seg_len, max_segs;
};

// Whole sequences are walked by the delta rule's blocks of four warps (a token's chain is shortest with one warp a
// scheduler).  Segments are walked by blocks of eight: twice the columns share a chunk's rows of q, k and 1 - a, the same
// shared memory holds twice the warps an SM, and with every SM full that is worth more than the longer chain (one
// sequence of 2,048 tokens, 8 heads of 128 x 128: 324 us against 346; 32 heads of 64 x 64: 370 against 466 whole).
constexpr int decay_warps(int part) { return part == 0 ? 4 : 8; }

template <int DSL, int SL, bool READ_FIRST, int PART>
__global__ void __launch_bounds__(decay_warps(PART) * 32, 3) decay_scan_kernel(DeltaParams p, DecaySegments g) {
    constexpr int DECAY_WARPS = decay_warps(PART), DECAY_THREADS = DECAY_WARPS * 32;
    using Sh = DeltaShape<DSL, SL, DECAY_WARPS>;
    constexpr int ROW = Sh::ROW, COLS = Sh::COLS, STRIDE = Sh::STRIDE, BUF = Sh::BUF;
    extern __shared__ __align__(16) float sm[];
    const int s = PART == 0 ? blockIdx.x : blockIdx.x / g.max_segs;
    const int j = PART == 0 ? 0 : blockIdx.x % g.max_segs;
    const int h = blockIdx.y, e0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slice = lane % SL, col = warp * (32 / SL) + lane / SL;
    const int e = e0 + col;
    const int D = p.D, E = p.E;
    // channels beyond key_dim, and value columns beyond value_dim, hold zeros throughout (no decay: 1 - a = 0)
    for (int i = threadIdx.x; i < 2 * BUF; i += DECAY_THREADS) sm[i] = 0.f;
    pdl_launch_dependents();
    pdl_wait();
    int q_beg = p.cu_q[s], n = p.cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    int n_segs = 1;
    if (PART != 0) {
        n_segs = ceil_div(n, g.seg_len);
        if (j >= n_segs || (PART == 1 && j > 0 && j == n_segs - 1) || (PART == 2 && j == 0)) return;
        q_beg += j * g.seg_len;
        n = min(g.seg_len, n - j * g.seg_len);
    }
    const bool read_out = PART != 1 || j == 0;
    const int slot = p.state_slots[s];
    float S[DSL];
    float* st = slot >= 0 ? p.state + (size_t)slot * p.state_ld + (size_t)h * D * E : nullptr;
    const size_t seg_first = (size_t)s * (PART == 0 ? 0 : g.max_segs);
    if (PART == 2) {
        const float* L = g.state + (seg_first * p.H + h) * (size_t)D * E;
#pragma unroll
        for (int i = 0; i < DSL; ++i) {
            const int d = slice * DSL + i;
            S[i] = (d < D && e < E) ? L[(size_t)d * E + e] : 0.f;
        }
        for (int seg = 1; seg < j; ++seg) {
            const float* Ls = g.state + ((seg_first + seg) * p.H + h) * (size_t)D * E;
            const float* Ps = g.decay + ((seg_first + seg) * p.H + h) * (size_t)D;
#pragma unroll
            for (int i = 0; i < DSL; ++i) {
                const int d = slice * DSL + i;
                if (d < D && e < E) S[i] = fmaf(Ps[d], S[i], Ls[(size_t)d * E + e]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < DSL; ++i) {
            const int d = slice * DSL + i;
            S[i] = (j == 0 && st && d < D && e < E) ? st[(size_t)d * E + e] : 0.f;
        }
    }
    if (PART == 1 && j > 0 && blockIdx.z == 0) {
        for (int d = threadIdx.x; d < D; d += DECAY_THREADS) {
            const float* c = p.decay + (size_t)q_beg * ((size_t)p.H * D) + (size_t)h * D + d;
            float sum = 0.f;
            for (int t = 0; t < n; ++t) sum += log1pf(-c[(size_t)t * ((size_t)p.H * D)]);
            g.decay[((seg_first + j) * p.H + h) * (size_t)D + d] = expf(sum);
        }
    }
    __syncthreads();
    delta_load_chunk<DSL, SL, DECAY_WARPS>(p, sm, q_beg, min(DELTA_CHUNK, n), h, h, e0);
    int turn = 0;
    for (int c0 = 0; c0 < n; c0 += DELTA_CHUNK, turn ^= 1) {
        const int nc = min(DELTA_CHUNK, n - c0);
        cp_async_wait_all();
        __syncthreads();      // this chunk has arrived, and the chunk before is consumed by every warp
        if (c0 + DELTA_CHUNK < n)
            delta_load_chunk<DSL, SL, DECAY_WARPS>(p, sm + (turn ^ 1) * BUF, q_beg + c0 + DELTA_CHUNK, min(DELTA_CHUNK, n - c0 - DELTA_CHUNK), h, h, e0);
        const float* buf = sm + turn * BUF;
        const float* vs = buf + 3 * DELTA_CHUNK * ROW;
        const float* bs = vs + DELTA_CHUNK * COLS;
        auto token = [&](int tt) {
            const float4* qr = reinterpret_cast<const float4*>(buf + tt * ROW + slice * STRIDE);
            const float4* kr = reinterpret_cast<const float4*>(buf + DELTA_CHUNK * ROW + tt * ROW + slice * STRIDE);
            const float4* gr = reinterpret_cast<const float4*>(buf + 2 * DELTA_CHUNK * ROW + tt * ROW + slice * STRIDE);
            const float val = vs[tt * COLS + col];
            float qs4[4] = {0.f, 0.f, 0.f, 0.f};      // four sums in turn: short chains of dependent adds
#pragma unroll
            for (int i = 0; i < DSL / 4; ++i) {
                const float4 g4 = gr[i], k4 = kr[i];
                const float4 q4 = read_out ? qr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                if (READ_FIRST && read_out) {
                    qs4[0] = fmaf(q4.x, S[4 * i], qs4[0]);
                    qs4[1] = fmaf(q4.y, S[4 * i + 1], qs4[1]);
                    qs4[2] = fmaf(q4.z, S[4 * i + 2], qs4[2]);
                    qs4[3] = fmaf(q4.w, S[4 * i + 3], qs4[3]);
                }
                S[4 * i] = fmaf(-g4.x, S[4 * i], S[4 * i]);
                S[4 * i + 1] = fmaf(-g4.y, S[4 * i + 1], S[4 * i + 1]);
                S[4 * i + 2] = fmaf(-g4.z, S[4 * i + 2], S[4 * i + 2]);
                S[4 * i + 3] = fmaf(-g4.w, S[4 * i + 3], S[4 * i + 3]);
                if (!READ_FIRST && read_out) {
                    qs4[0] = fmaf(q4.x, S[4 * i], qs4[0]);
                    qs4[1] = fmaf(q4.y, S[4 * i + 1], qs4[1]);
                    qs4[2] = fmaf(q4.z, S[4 * i + 2], qs4[2]);
                    qs4[3] = fmaf(q4.w, S[4 * i + 3], qs4[3]);
                }
                S[4 * i] = fmaf(k4.x, val, S[4 * i]);
                S[4 * i + 1] = fmaf(k4.y, val, S[4 * i + 1]);
                S[4 * i + 2] = fmaf(k4.z, val, S[4 * i + 2]);
                S[4 * i + 3] = fmaf(k4.w, val, S[4 * i + 3]);
            }
            if (read_out) {
                float qS = (qs4[0] + qs4[1]) + (qs4[2] + qs4[3]);
#pragma unroll
                for (int o = 1; o < SL; o <<= 1) qS += __shfl_xor_sync(0xffffffffu, qS, o);
                if (slice == 0 && e < E)
                    p.out[(size_t)(q_beg + c0 + tt) * ((size_t)p.H * E) + (size_t)h * E + e] = fmaf(bs[DELTA_CHUNK + tt], val, qS);
            }
        };
        if (nc == DELTA_CHUNK) {
#pragma unroll
            for (int tt = 0; tt < DELTA_CHUNK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nc; ++tt) token(tt);
        }
    }
    // the request's state is left by the block that walked the sequence's last tokens; a segment before it leaves its own
    float* leave = (j == n_segs - 1) ? st : (PART == 1 ? g.state + ((seg_first + j) * p.H + h) * (size_t)D * E : nullptr);
    if (leave) {
#pragma unroll
        for (int i = 0; i < DSL; ++i) {
            const int d = slice * DSL + i;
            if (d < D && e < E) leave[(size_t)d * E + e] = S[i];
        }
    }
}

template <int DSL, int SL, bool READ_FIRST, int PART>
static cudaError_t launch_decay_part(const DeltaParams& p, const DecaySegments& g, int n_seqs, cudaStream_t s) {
    constexpr int DECAY_WARPS = decay_warps(PART), DECAY_THREADS = DECAY_WARPS * 32;
    using Sh = DeltaShape<DSL, SL, DECAY_WARPS>;
    const size_t smem = 2 * (size_t)Sh::BUF * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decay_scan_kernel<DSL, SL, READ_FIRST, PART>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    dim3 grid(PART == 0 ? n_seqs : n_seqs * g.max_segs, p.H, ceil_div(p.E, Sh::COLS));
    return llmk_launch(decay_scan_kernel<DSL, SL, READ_FIRST, PART>, grid, dim3(DECAY_THREADS), smem, s, true, p, g);
}

template <int DSL, int SL>
static cudaError_t launch_decay(const DeltaParams& p, const DecaySegments& g, int n_seqs, bool read_first, cudaStream_t s) {
    if (!g.state) {
        return read_first ? launch_decay_part<DSL, SL, true, 0>(p, g, n_seqs, s) : launch_decay_part<DSL, SL, false, 0>(p, g, n_seqs, s);
    }
    cudaError_t e = read_first ? launch_decay_part<DSL, SL, true, 1>(p, g, n_seqs, s) : launch_decay_part<DSL, SL, false, 1>(p, g, n_seqs, s);
    if (e != cudaSuccess) return e;
    return read_first ? launch_decay_part<DSL, SL, true, 2>(p, g, n_seqs, s) : launch_decay_part<DSL, SL, false, 2>(p, g, n_seqs, s);
}

// Steps of a few token rows (single decoded tokens, short portions): one launch.  A block per (sequence, head, 64 value
// columns) prepares a token's q, k and 1 - a itself (the arithmetic of `decay_prep`), keeps its part of S in registers
// over the sequence's tokens (a thread holds every fourth key channel of one column, so a row of S is read by
// consecutive threads), and adds up the four partial read-outs of a column through shared memory.
constexpr int DECAY_STEP_MAX_TOKENS = 32;

template <typename T, bool READ_FIRST, int NR>
__global__ void __launch_bounds__(256) decay_step_kernel(float* __restrict__ out, const T* __restrict__ q, long long q_ld,
                                                         const T* __restrict__ k, long long k_ld, const T* __restrict__ v, long long v_ld,
                                                         const float* __restrict__ z, const float* __restrict__ bias,
                                                         const float* __restrict__ bonus, float* __restrict__ state, long long state_ld,
                                                         const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int D,
                                                         int E, int mode, float inv_tau, float q_scale) {
    __shared__ float sq[4 * NR], sk[4 * NR], sc[4 * NR];
    __shared__ float partial[4][64];
    __shared__ float warp_dots[8];
    const int s = blockIdx.x, h = blockIdx.y;
    const int ce = threadIdx.x & 63, part = threadIdx.x >> 6, e = blockIdx.z * 64 + ce;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    const int q_beg = cu_q[s], n = cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = state_slots[s];
    float* st = slot >= 0 ? state + (size_t)slot * state_ld + (size_t)h * D * E : nullptr;
    float S[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int d = part + 4 * i;
        S[i] = (st && d < D && e < E) ? st[(size_t)d * E + e] : 0.f;
    }
    for (int t = 0; t < n; ++t) {
        const size_t row = (size_t)(q_beg + t);
        float dot = 0.f;
        for (int d = threadIdx.x; d < 4 * NR; d += 256) {
            float qv = 0.f, kv = 0.f, c = 0.f;
            if (d < D) {
                const int i = h * D + d;
                qv = to_float(q[row * q_ld + i]) * q_scale;
                kv = to_float(k[row * k_ld + i]);
                const float x = z[row * ((size_t)H * D) + i] + (bias ? bias[i] : 0.f);
                const float log_a = mode == DECAY_SIGMOID_POW ? -softplusf_(-x) * inv_tau : -expf(x);
                c = -expm1f(log_a);
                dot = fmaf(qv * (bonus ? bonus[i] : 1.f), kv, dot);
            }
            sq[d] = qv;
            sk[d] = kv;
            sc[d] = c;
        }
        dot = warp_sum(dot);
        if (lane == 0) warp_dots[warp] = dot;
        __syncthreads();
        dot = ((warp_dots[0] + warp_dots[1]) + (warp_dots[2] + warp_dots[3])) + ((warp_dots[4] + warp_dots[5]) + (warp_dots[6] + warp_dots[7]));
        const float val = e < E ? to_float(v[row * v_ld + (size_t)h * E + e]) : 0.f;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int d = part + 4 * i;
            if (READ_FIRST) acc[i & 3] = fmaf(sq[d], S[i], acc[i & 3]);
            S[i] = fmaf(-sc[d], S[i], S[i]);
            if (!READ_FIRST) acc[i & 3] = fmaf(sq[d], S[i], acc[i & 3]);
            S[i] = fmaf(sk[d], val, S[i]);
        }
        partial[part][ce] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        __syncthreads();
        if (part == 0 && e < E) {
            const float qS = (partial[0][ce] + partial[1][ce]) + (partial[2][ce] + partial[3][ce]);
            out[row * ((size_t)H * E) + (size_t)h * E + e] = fmaf(dot, val, qS);
        }
        __syncthreads();      // the next token's q, k, 1 - a and partial sums go where this one's were read
    }
    if (st) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int d = part + 4 * i;
            if (d < D && e < E) st[(size_t)d * E + e] = S[i];
        }
    }
}

template <typename T>
static cudaError_t launch_decay_step(float* out, const void* q, long long q_ld, const void* k, long long k_ld, const void* v, long long v_ld,
                                     const float* z, const float* bias, const float* bonus, float* state, long long state_ld,
                                     const int* cu_q, const int* state_slots, int n_seqs, int H, int D, int E, int mode, float inv_tau,
                                     float q_scale, bool read_first, cudaStream_t s) {
    dim3 grid(n_seqs, H, ceil_div(E, 64));
#define LLMK_DECAY_STEP(RF, NR)                                                                                                    \
    return llmk_launch(decay_step_kernel<T, RF, NR>, grid, dim3(256), 0, s, true, out, (const T*)q, q_ld, (const T*)k, k_ld,      \
                       (const T*)v, v_ld, z, bias, bonus, state, state_ld, cu_q, state_slots, H, D, E, mode, inv_tau, q_scale)
    if (D <= 64) {
        if (read_first) LLMK_DECAY_STEP(true, 16);
        LLMK_DECAY_STEP(false, 16);
    }
    if (D <= 128) {
        if (read_first) LLMK_DECAY_STEP(true, 32);
        LLMK_DECAY_STEP(false, 32);
    }
    if (read_first) LLMK_DECAY_STEP(true, 64);
    LLMK_DECAY_STEP(false, 64);
#undef LLMK_DECAY_STEP
}

// Steps of DECAY_SEGMENTS_MIN_TOKENS token rows and more, of at most DECAY_SEGMENTS_MAX_SEQS sequences, are walked in
// segments when the caller gives scratch for them: as many as fill the SMs once and the scratch holds, of 64 tokens at
// least.
constexpr int DECAY_SEGMENTS_MIN_TOKENS = 256, DECAY_SEGMENTS_MAX_SEQS = 8;

// q, k [n_tokens, H * D] and v [n_tokens, H * E] of the storage dtype (rows q_ld, k_ld, v_ld apart); decay float32
// [n_tokens, H * D]: the pre-activations, rewritten in place (left alone by steps of a few rows); bias float32 [H * D] or null; bonus float32 [H * D] or null;
// qkv_buf float32 scratch [n_tokens, 2 H D + H E]; dots float32 scratch [n_tokens, 2 H]; state float32, S [H][D][E] of slot
// s at state + s * state_ld; out float32 [n_tokens, H * E].  read_first != 0: a token reads the state before its own
// decay and key enter it (its own key counts `bonus` times); else after both.  seg_scratch (float32, seg_floats values, or
// null): room for the segments' states and decay products; without it every sequence is walked whole.  *launches (or
// null) receives the number of kernels launched.
LLMK_EXPORT int llmk_decay_scan(float* out, const void* q, long long q_ld, const void* k, long long k_ld, const void* v, long long v_ld,
                                float* decay, const float* bias, const float* bonus, float* qkv_buf, float* dots, float* state,
                                long long state_ld, const int* cu_q, const int* state_slots, int n_seqs, int n_tokens, int H, int D,
                                int E, int mode, float tau, float q_scale, int read_first, float* seg_scratch, long long seg_floats,
                                int* launches, int dtype, void* stream) {
    if (launches) *launches = 0;
    if (n_seqs <= 0 || n_tokens <= 0) return LLMK_OK;
    if (H <= 0 || D <= 0 || D > 256 || E <= 0) LLMK_FAIL("decay_scan: heads %d, key width %d (at most 256), value width %d", H, D, E);
    if (mode != DECAY_SIGMOID_POW && mode != DECAY_EXP_EXP) LLMK_FAIL("decay_scan: unknown decay form %d", mode);
    if (mode == DECAY_SIGMOID_POW && !(tau > 0.f)) LLMK_FAIL("decay_scan: tau %g must be positive", (double)tau);
    if (!out || !q || !k || !v || !decay || !qkv_buf || !dots || !state || !cu_q || !state_slots) LLMK_FAIL("decay_scan: bad arguments");
    if (H > 65535 || ceil_div(E, 8) > 65535) LLMK_FAIL("decay_scan: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    const long long qkv_ld = 2LL * H * D + (long long)H * E;
    const float inv_tau = mode == DECAY_SIGMOID_POW ? 1.0f / tau : 1.0f;
    cudaError_t e;
    if (dtype != LLMK_F32 && dtype != LLMK_BF16) LLMK_FAIL("decay_scan: unknown dtype %d", dtype);
    if (n_tokens <= DECAY_STEP_MAX_TOKENS) {
        if (dtype == LLMK_F32)
            e = launch_decay_step<float>(out, q, q_ld, k, k_ld, v, v_ld, decay, bias, bonus, state, state_ld, cu_q, state_slots, n_seqs, H, D, E,
                                         mode, inv_tau, q_scale, read_first != 0, s);
        else
            e = launch_decay_step<bf16>(out, q, q_ld, k, k_ld, v, v_ld, decay, bias, bonus, state, state_ld, cu_q, state_slots, n_seqs, H, D, E,
                                        mode, inv_tau, q_scale, read_first != 0, s);
        LLMK_CHECK_LAUNCH_RC("decay_step", e);
        if (launches) *launches = 1;
        return LLMK_OK;
    }
    if (dtype == LLMK_F32)
        e = llmk_launch(decay_prep_kernel<float>, dim3(n_tokens), dim3(256), 0, s, true, qkv_buf, qkv_ld, decay, dots, (const float*)q, q_ld,
                        (const float*)k, k_ld, (const float*)v, v_ld, bias, bonus, H, D, E, mode, inv_tau, q_scale);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(decay_prep_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, true, qkv_buf, qkv_ld, decay, dots, (const bf16*)q, q_ld,
                        (const bf16*)k, k_ld, (const bf16*)v, v_ld, bias, bonus, H, D, E, mode, inv_tau, q_scale);
    else
        LLMK_FAIL("decay_scan: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("decay_prep", e);
    DeltaParams p;
    p.out = out; p.qkv = qkv_buf; p.qkv_ld = qkv_ld; p.beta = dots; p.decay = decay;
    p.state = state; p.state_ld = state_ld; p.cu_q = cu_q; p.state_slots = state_slots;
    p.H = H; p.G = H; p.D = D; p.E = E;
    p.vec_ok = (D % 4 == 0 && E % 4 == 0 && host_aligned16(qkv_buf) && host_aligned16(decay)) ? 1 : 0;
    DecaySegments g;
    g.state = nullptr; g.decay = nullptr; g.seg_len = 0; g.max_segs = 1;
    if (seg_scratch && n_tokens >= DECAY_SEGMENTS_MIN_TOKENS && n_seqs <= DECAY_SEGMENTS_MAX_SEQS) {
        // As many segments as fill the SMs once: however the step's rows are shared out among its sequences, a pass runs
        // about (segments - 1) x heads x column tiles blocks, and a block that waits for a place costs a whole segment's
        // time.  Two segments gain nothing (each pass walks one of them).  On a B200, one sequence of 2,048 tokens:
        // 4 heads of 128 x 128 in 7 segments 216 us against 588 whole (8: 235, 4: 337), 16 heads of 64 x 64 in 4 segments
        // 257 against 433 (7: 273); 32 heads of 64 x 64 fill the SMs as they are (466; 4 segments: 480).
        static int sms = 0, smem_sm = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        }
        const int dsl = D <= 64 ? 4 : (D <= 128 ? 8 : 16), sl = D <= 32 ? 8 : 16;
        const int stride = dsl == 4 ? 12 : dsl + 4, cols = decay_warps(1) * (32 / sl);
        const long long smem_block = 2LL * (DELTA_CHUNK * (3 * sl * stride + cols) + 2 * DELTA_CHUNK) * 4 + 1024;
        const long long places = (long long)sms * std::max<long long>(1, std::min<long long>(smem_sm / smem_block, 2048 / (decay_warps(1) * 32)));
        const long long base = (long long)H * ceil_div(E, cols);
        const long long per_seg = (long long)H * ((long long)D * E + D);
        long long segs = std::min<long long>(places / base + 1, seg_floats / (per_seg * n_seqs));
        segs = std::min<long long>(segs, n_tokens / 64);
        if (segs >= 3) {
            g.seg_len = ceil_div(ceil_div(n_tokens, (int)segs), 16) * 16;
            g.max_segs = ceil_div(n_tokens, g.seg_len);
            g.state = seg_scratch;
            g.decay = seg_scratch + (long long)n_seqs * g.max_segs * H * D * E;
        }
    }
    const bool rf = read_first != 0;
    if (D <= 32) e = launch_decay<4, 8>(p, g, n_seqs, rf, s);
    else if (D <= 64) e = launch_decay<4, 16>(p, g, n_seqs, rf, s);
    else if (D <= 128) e = launch_decay<8, 16>(p, g, n_seqs, rf, s);
    else e = launch_decay<16, 16>(p, g, n_seqs, rf, s);
    LLMK_CHECK_LAUNCH_RC("decay_scan", e);
    if (launches) *launches = g.state ? 3 : 2;
    return LLMK_OK;
}
