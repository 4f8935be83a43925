// Recurrent mixers whose gates read the current token only, and matrix memories that are read and written by rank-one
// steps:
//
//   min_gru         S_t = (1 - z_t) S_(t-1) + z_t c_t per channel, z = sigmoid(.), c = u + 1/2 where u >= 0 and sigmoid(u)
//                   below; out = S_t * silu(g_t); token by token for steps of a few rows, tiles of 32 tokens scanned by a warp else
//   mlstm_gates     the log gates of a matrix memory with a running maximum, i = cap tanh(. / cap) and
//                   f = logsigmoid(cap tanh(. / cap)) per token and head, with the token's own q . k
//   mlstm_maxima    m_t = max(f_t + m_(t-1), i_t) along each sequence (m carried in the state, 0 for a fresh request); what
//                   the memory's step needs follows from it where it is used: exp(f + m_(t-1) - m_t), exp(i - m_t), exp(-m_t)
//   delta_rule_prep the generalized delta rule's vectors per token and head: the decay w = exp(-c0 sigmoid(z + w0)), the unit
//                   key u = k / sqrt(sum k^2 + unit_eps), the removal b = sigmoid(a + a0) u, and the dots b . r and k . r
//   memory_scan     the memory S [key_dim, value_dim] per head over each sequence's new tokens, in two forms:
//                     delta   S_t = diag(w) S - b (u^T S) + k v^T (both terms read the old S);  o = S_t^T r
//                     mlstm   S_t = keep S + take k v^T, n_t = keep n + take k;
//                             o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + den_eps)
//                   With the old S the read-out is  o = (w r)^T S - (b . r)(u^T S) + (k . r) v  (delta) and
//                   keep q^T S + take (k . q) v  (mlstm), so a token is one pass over its part of S: the dot products
//                   first, then the update.
//
// A step's sequences are given as everywhere else: sequence s owns token rows [cu_q[s], cu_q[s+1]), its state lies in
// slot state_slots[s] (-1: none; the sequence then starts from zeros and leaves nothing).  Rows beyond cu_q[n_seqs]
// belong to no sequence and are skipped, sequences without tokens too, so every launch here follows from a step's shape.
// States, gates, decays, their logarithms and exponentials, unit norms and the recurrences are float32 arithmetic in both
// storage dtypes.  The arithmetic of a token does not depend on where a step was cut.
#define LLMK_MODULE_NAME "memory_scan"
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
// log(sigmoid(x)) = -softplus(-x)
__device__ __forceinline__ float logsigmoidf_(float x) { return x < -20.f ? x : -log1pf(expf(-x)); }

// ------------------------------------------------------------------------------------------------------- min_gru
// A thread per (sequence, channel) walks the sequence's tokens.  zxg [n, 3C] float32: z, u and g side by side.
template <typename T>
__global__ void min_gru_kernel(T* __restrict__ out, const float* __restrict__ zxg, long long ld, const float* __restrict__ bz,
                               const float* __restrict__ bx, float* __restrict__ state, long long state_ld,
                               const int* __restrict__ cu_q, const int* __restrict__ state_slots, int C) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (c >= C) return;
    const int q_beg = cu_q[s], n = cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = state_slots[s];
    float S = slot >= 0 ? state[(size_t)slot * state_ld + c] : 0.f;
    const float b_z = bz ? bz[c] : 0.f, b_x = bx ? bx[c] : 0.f;
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        const float* row = zxg + (size_t)(q_beg + j) * ld;
        const float z = sigmoidf_(row[c] + b_z);
        const float u = row[C + c] + b_x;
        const float g = row[2 * C + c];
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
        S = fmaf(z, cand - S, S);                       // (1 - z) S + z cand
        out[(size_t)(q_beg + j) * C + c] = from_float<T>(S * (g * sigmoidf_(g)));
    }
    if (slot >= 0) state[(size_t)slot * state_ld + c] = S;
}

// The same recurrence for steps of many tokens: a block takes 32 channels of one sequence and walks its tokens 32 at a time.
// Warp w first makes (1 - z, z cand, silu(g)) of the tile's token w for the 32 channels (rows read whole), then scans channel
// w over the tile's tokens: steps S -> a S + b compose as (a1, b1) then (a2, b2) = (a1 a2, b1 a2 + b2), five rounds over the
// lanes; then token w's row goes out.  The sums of a token are regrouped, not changed, against the walk above.
constexpr int GT = 32;
template <typename T>
__global__ void __launch_bounds__(GT* GT) min_gru_tile_kernel(T* __restrict__ out, const float* __restrict__ zxg, long long ld,
                                                              const float* __restrict__ bz, const float* __restrict__ bx,
                                                              float* __restrict__ state, long long state_ld,
                                                              const int* __restrict__ cu_q, const int* __restrict__ state_slots, int C) {
    __shared__ float sa[GT][GT + 1], sb[GT][GT + 1];
    const int s = blockIdx.y, cb = blockIdx.x * GT;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    const int q_beg = cu_q[s], n = cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = state_slots[s];
    const int c_row = cb + lane, c_scan = cb + w;                 // this thread's channel as a reader of rows, and as a scanner
    const float b_z = (bz && c_row < C) ? bz[c_row] : 0.f, b_x = (bx && c_row < C) ? bx[c_row] : 0.f;
    float carry = (slot >= 0 && c_scan < C) ? state[(size_t)slot * state_ld + c_scan] : 0.f;
    for (int t0 = 0; t0 < n; t0 += GT) {
        const int nt = min(GT, n - t0);
        float gs = 0.f, a = 1.f, b = 0.f;
        if (w < nt && c_row < C) {
            const float* row = zxg + (size_t)(q_beg + t0 + w) * ld;
            const float z = sigmoidf_(row[c_row] + b_z);
            const float u = row[C + c_row] + b_x;
            const float g = row[2 * C + c_row];
            a = 1.f - z;
            b = z * (u >= 0.f ? u + 0.5f : sigmoidf_(u));
            gs = g * sigmoidf_(g);
        }
        sa[w][lane] = a;
        sb[w][lane] = b;
        __syncthreads();
        a = sa[lane][w];          // token `lane` of channel `w`
        b = sb[lane][w];
#pragma unroll
        for (int o = 1; o < GT; o <<= 1) {
            const float pa = __shfl_up_sync(0xffffffffu, a, o), pb = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) {
                b = fmaf(pb, a, b);
                a *= pa;
            }
        }
        const float S = fmaf(a, carry, b);
        carry = __shfl_sync(0xffffffffu, S, nt - 1);
        __syncthreads();
        sa[lane][w] = S;
        __syncthreads();
        if (w < nt && c_row < C) out[(size_t)(q_beg + t0 + w) * C + c_row] = from_float<T>(sa[w][lane] * gs);
        __syncthreads();
    }
    if (slot >= 0 && c_scan < C && lane == 0) state[(size_t)slot * state_ld + c_scan] = carry;
}

// ------------------------------------------------------------------------------------------------------- mlstm gates
// A warp per (token, head): gates[t, h] = (i, f, (q . k) q_scale, -).
template <typename T>
__global__ void mlstm_gates_kernel(float* __restrict__ gates, const T* __restrict__ q, long long ldq, const T* __restrict__ k,
                                   long long ldk, const T* __restrict__ gi, long long ldi, const T* __restrict__ gf, long long ldf,
                                   const float* __restrict__ bi, const float* __restrict__ bf, const int* __restrict__ cu_q,
                                   int n_seqs, int n_rows, int H, int D, float cap, float q_scale) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();
    if (w >= (long long)n_rows * H) return;
    const int t = (int)(w / H), h = (int)(w % H);
    if (t >= cu_q[n_seqs]) return;
    const T* qr = q + (size_t)t * ldq + (size_t)h * D;
    const T* kr = k + (size_t)t * ldk + (size_t)h * D;
    float dot = 0.f;
    for (int d = lane; d < D; d += 32) dot = fmaf(to_float(qr[d]), to_float(kr[d]), dot);
    dot = warp_sum(dot);
    if (lane == 0) {
        const float xi = to_float(gi[(size_t)t * ldi + h]) + (bi ? bi[h] : 0.f);
        const float xf = to_float(gf[(size_t)t * ldf + h]) + (bf ? bf[h] : 0.f);
        float4 o;
        o.x = cap * tanhf(xi / cap);
        o.y = logsigmoidf_(cap * tanhf(xf / cap));
        o.z = dot * q_scale;
        o.w = 0.f;
        reinterpret_cast<float4*>(gates)[(size_t)t * H + h] = o;
    }
}

// A warp per (sequence, head) takes the tokens 32 at a time: gates[t, h].w <- m_(t-1), the maximum before the token.  A token's
// step m -> max(f + m, i) composes with the next, (f1, i1) then (f2, i2) = (f1 + f2, max(i1 + f2, i2)), so five rounds over the
// lanes give every token's maximum.  What the memory's step needs follows from (i, f, m_(t-1)) alone, m_t = max(f + m_(t-1), i),
// keep = exp(f + m_(t-1) - m_t), take = exp(i - m_t), exp(-m_t), and is made where it is used.
__global__ void mlstm_maxima_kernel(float* __restrict__ gates, float* __restrict__ m_state, long long state_ld,
                                    const int* __restrict__ cu_q, const int* __restrict__ state_slots, int n_seqs, int H) {
    const int lane = threadIdx.x & 31;
    const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();
    if (idx >= n_seqs * H) return;
    const int s = idx / H, h = idx % H;
    const int q_beg = cu_q[s], n = cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = state_slots[s];
    float m = slot >= 0 ? m_state[(size_t)slot * state_ld + h] : 0.f;
    float4* g = reinterpret_cast<float4*>(gates);
    for (int t0 = 0; t0 < n; t0 += 32) {
        const int nt = min(32, n - t0);
        float4* at = g + (size_t)(q_beg + t0 + lane) * H + h;
        float f = 0.f, i = -INFINITY;                     // beyond the sequence: the step that changes nothing
        if (lane < nt) {
            const float2 gate = *reinterpret_cast<const float2*>(at);
            i = gate.x;
            f = gate.y;
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float pf = __shfl_up_sync(0xffffffffu, f, o), pi = __shfl_up_sync(0xffffffffu, i, o);
            if (lane >= o) {
                i = fmaxf(pi + f, i);
                f += pf;
            }
        }
        const float after = fmaxf(f + m, i);
        float before = __shfl_up_sync(0xffffffffu, after, 1);
        if (lane == 0) before = m;
        if (lane < nt) at->w = before;
        m = __shfl_sync(0xffffffffu, after, nt - 1);
    }
    if (slot >= 0 && lane == 0) m_state[(size_t)slot * state_ld + h] = m;
}

// ------------------------------------------------------------------------------------------------------- delta rule prep
// A block per token, a warp per head in turn.  aux[t] = [w | b | u] (H D each), dots[t, h] = (b . r, k . r).
template <typename T>
__global__ void delta_rule_prep_kernel(float* __restrict__ aux, float* __restrict__ dots, const T* __restrict__ r, long long ldr,
                                       const T* __restrict__ k, long long ldk, const T* __restrict__ a, long long lda,
                                       const float* __restrict__ decay, long long ldd, const float* __restrict__ a_bias,
                                       const float* __restrict__ w_bias, const int* __restrict__ cu_q, int n_seqs, int H, int D,
                                       float decay_scale, float unit_eps) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    if (t >= cu_q[n_seqs]) return;
    const int HD = H * D;
    float* wt = aux + (size_t)t * 3 * HD;
    for (int h = warp; h < H; h += nwarps) {
        const T* kr = k + (size_t)t * ldk + (size_t)h * D;
        const T* rr = r + (size_t)t * ldr + (size_t)h * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float kv = to_float(kr[d]);
            ss = fmaf(kv, kv, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + unit_eps);
        float br = 0.f, kdr = 0.f;
        for (int d = lane; d < D; d += 32) {
            const int c = h * D + d;
            const float kv = to_float(kr[d]), rv = to_float(rr[d]);
            const float u = kv * inv;
            const float b = sigmoidf_(to_float(a[(size_t)t * lda + c]) + (a_bias ? a_bias[c] : 0.f)) * u;
            const float w = expf(-decay_scale * sigmoidf_(decay[(size_t)t * ldd + c] + (w_bias ? w_bias[c] : 0.f)));
            wt[c] = w;
            wt[HD + c] = b;
            wt[2 * HD + c] = u;
            br = fmaf(b, rv, br);
            kdr = fmaf(kv, rv, kdr);
        }
        br = warp_sum(br);
        kdr = warp_sum(kdr);
        if (lane == 0) {
            dots[((size_t)t * H + h) * 2] = br;
            dots[((size_t)t * H + h) * 2 + 1] = kdr;
        }
    }
}

// ------------------------------------------------------------------------------------------------------- memory scan
// A block per (tile of CT value columns, head, sequence); sixteen lanes share a column of S, lane j of them holding key
// rows j DPL .. j DPL + DPL - 1.  A chunk of TC tokens' vectors is staged in shared memory, then walked token by token.
constexpr int LANES = 16;     // lanes that share a column
constexpr int CT = 8;         // value columns a block
constexpr int TC = 8;         // tokens a chunk: LANES * CT threads fetch one token's vectors by sixteen of them each
enum { FORM_DELTA = 0, FORM_MLSTM = 1 };

struct ScanParams {
    float* out;               // [n, H E]
    const void *r, *k, *v;    // storage type, rows ldr / ldk / ldv apart
    long long ldr, ldk, ldv;
    const float* aux;         // delta: [n, 3 H D] = w | b | u
    const float* dots;        // delta: [n, H, 2] = (b . r, k . r); mlstm: [n, H, 4] = (i, f, (q . k) q_scale, m before the token)
    float* state;             // [slots, state_ld]: S [H, D, E], then (mlstm) n [H, D]
    long long state_ld;
    const int *cu_q, *state_slots;
    int H, D, E;
    float r_scale, den_eps;
};

// A value's bits in a 32-bit register (a 16-bit load extends into one by itself), and back.
// The loads are volatile asm so that they are issued where they stand, a chunk ahead of their use, and not moved down to it.
__device__ __forceinline__ uint32_t load_bits(const float* p) {
    uint32_t v;
    asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t load_bits(const bf16* p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
template <typename T> __device__ __forceinline__ float bits_value(uint32_t b);
template <> __device__ __forceinline__ float bits_value<float>(uint32_t b) { return __uint_as_float(b); }
template <> __device__ __forceinline__ float bits_value<bf16>(uint32_t b) { return __uint_as_float(b << 16); }

// A lane's DPL rows of one of a token's vectors (rows l DPL ..), zeros beyond D; sixteen bytes at a time where the sizes allow.
template <int DPL>
__device__ __forceinline__ void lane_rows(float (&dst)[DPL], const float* __restrict__ src, int l, int D, bool vec4) {
    if (DPL % 4 == 0 && vec4) {
#pragma unroll
        for (int i4 = 0; i4 < DPL / 4; ++i4) {
            const int d = l * DPL + 4 * i4;
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (d < D) t = *reinterpret_cast<const float4*>(src + d);
            dst[4 * i4] = t.x; dst[4 * i4 + 1] = t.y; dst[4 * i4 + 2] = t.z; dst[4 * i4 + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = l * DPL + i;
            dst[i] = d < D ? src[d] : 0.f;
        }
    }
}

// FULL: the key width is exactly 16 DPL (a compile-time number then: no row of a lane lies beyond it).
template <typename T, int FORM, int DPL, bool FULL>
__global__ void __launch_bounds__(LANES* CT) memory_scan_kernel(ScanParams p) {
    extern __shared__ __align__(16) float sm[];
    const int tile = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
    const int tid = threadIdx.x, l = tid % LANES, col = tid / LANES;
    const int D = FULL ? LANES * DPL : p.D, E = p.E, H = p.H;
    const int e = tile * CT + col;
    const bool live = e < E;
    // per token in the chunk: r [D], k [D], (delta) w [D], b [D], u [D]; v [CT]; scalars [4]
    static_assert(TC * LANES == LANES * CT && CT + 4 <= LANES, "the staging's thread layout");
    const int vecs = FORM == FORM_DELTA ? 5 : 2;
    const int per_tok = vecs * D + CT + 4;
    pdl_launch_dependents();
    pdl_wait();
    const int q_beg = p.cu_q[s], n = p.cu_q[s + 1] - q_beg;
    if (n <= 0) return;
    const int slot = p.state_slots[s];
    float* Sg = slot >= 0 ? p.state + (size_t)slot * p.state_ld + (size_t)h * D * E : nullptr;
    float* ng = (slot >= 0 && FORM == FORM_MLSTM) ? p.state + (size_t)slot * p.state_ld + (size_t)H * D * E + (size_t)h * D : nullptr;
    // lane l of a column holds key rows l DPL .. l DPL + DPL - 1 (rows beyond D stay zero: their vectors are read as zeros)
    const bool vec4 = DPL % 4 == 0 && (FULL || D % 4 == 0);
    float S[DPL], nv[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = l * DPL + i;
        S[i] = (Sg && live && d < D) ? Sg[(size_t)d * E + e] : 0.f;
        nv[i] = (ng && d < D) ? ng[d] : 0.f;
    }
    const T* rp = static_cast<const T*>(p.r);
    const T* kp = static_cast<const T*>(p.k);
    const T* vp = static_cast<const T*>(p.v);
    const int HD = H * D, HE = H * E;
    float* out_col = p.out + (size_t)q_beg * HE + (size_t)h * E + e;
    // Staging: thread (sj, sl) = (tid / 16, tid % 16) fetches, for token sj of a chunk, the values d = sl + 16 i of every vector
    // (and one value column, one scalar); a chunk's values wait in registers while the chunk before is walked.
    const int sj = tid / LANES, sl = tid % LANES;
    uint32_t raw_rk[2 * DPL], raw_v = 0;                // a value's bits as loaded, one register each: nothing here waits for a load; `put` converts
    float raw_aux[(FORM == FORM_DELTA ? 3 : 1) * DPL], raw_s = 0.f;
    float4 raw_g = make_float4(0.f, 0.f, 0.f, 0.f);
    auto fetch = [&](int c0) {
        const int nt = min(TC, n - c0);
        if (sj >= nt) return;
        const size_t t = (size_t)(q_beg + c0 + sj);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = sl + LANES * i;
            if (d < D) {
                raw_rk[i] = load_bits(rp + t * p.ldr + (size_t)h * D + d);
                raw_rk[DPL + i] = load_bits(kp + t * p.ldk + (size_t)h * D + d);
                if (FORM == FORM_DELTA) {
#pragma unroll
                    for (int w = 0; w < 3; ++w) raw_aux[w * DPL + i] = __uint_as_float(load_bits(p.aux + t * 3 * HD + (size_t)w * HD + (size_t)h * D + d));
                }
            }
        }
        if (sl < CT) {
            const int ee = tile * CT + sl;
            if (ee < E) raw_v = load_bits(vp + t * p.ldv + (size_t)h * E + ee);
        } else if (sl < CT + 4) {
            if (FORM == FORM_DELTA) raw_s = sl - CT < 2 ? p.dots[(t * H + h) * 2 + (sl - CT)] : 0.f;
            else raw_g = reinterpret_cast<const float4*>(p.dots)[t * H + h];
        }
    };
    auto put = [&](int c0) {
        const int nt = min(TC, n - c0);
        if (sj >= nt) return;
        float* tk = sm + sj * per_tok;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = sl + LANES * i;
            if (d < D) {
                tk[d] = bits_value<T>(raw_rk[i]) * p.r_scale;
                tk[D + d] = bits_value<T>(raw_rk[DPL + i]);
                if (FORM == FORM_DELTA) {
#pragma unroll
                    for (int w = 0; w < 3; ++w) tk[(2 + w) * D + d] = raw_aux[w * DPL + i];
                }
            }
        }
        if (sl < CT) {
            tk[vecs * D + sl] = tile * CT + sl < E ? bits_value<T>(raw_v) : 0.f;
        } else if (sl < CT + 4) {
            const int q = sl - CT;
            float val = raw_s;
            if (FORM == FORM_MLSTM) {
                // (i, f, (q . k) q_scale, m before the token) -> keep, take, exp(-m_t), take (q . k) q_scale
                const float4 g = raw_g;
                const float mn = fmaxf(g.y + g.w, g.x);
                const float take = expf(g.x - mn);
                val = q == 0 ? expf(g.y + g.w - mn) : q == 1 ? take : q == 2 ? expf(-mn) : take * g.z;
            }
            tk[vecs * D + sl] = val;
        }
    };
    fetch(0);
    for (int c0 = 0; c0 < n; c0 += TC) {
        const int nt = min(TC, n - c0);
        __syncthreads();
        put(c0);
        __syncthreads();
        if (c0 + TC < n) fetch(c0 + TC);
        auto walk = [&](int j) {
            const float* tk = sm + j * per_tok;
            const float v_e = tk[vecs * D + col];
            const float* sc = tk + vecs * D + CT;
            float rr[DPL], kk[DPL];
            lane_rows<DPL>(rr, tk, l, D, vec4);
            lane_rows<DPL>(kk, tk + D, l, D, vec4);
            if (FORM == FORM_DELTA) {
                float ww[DPL], bb[DPL], uu[DPL];
                lane_rows<DPL>(ww, tk + 2 * D, l, D, vec4);
                lane_rows<DPL>(bb, tk + 3 * D, l, D, vec4);
                lane_rows<DPL>(uu, tk + 4 * D, l, D, vec4);
                float seen = 0.f, read = 0.f;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    seen = fmaf(uu[i], S[i], seen);
                    read = fmaf(ww[i] * rr[i], S[i], read);
                }
#pragma unroll
                for (int o = LANES / 2; o > 0; o >>= 1) {
                    seen += __shfl_xor_sync(0xffffffffu, seen, o);
                    read += __shfl_xor_sync(0xffffffffu, read, o);
                }
#pragma unroll
                for (int i = 0; i < DPL; ++i) S[i] = fmaf(kk[i], v_e, fmaf(ww[i], S[i], -bb[i] * seen));
                if (l == 0 && live) out_col[(size_t)(c0 + j) * HE] = read - sc[0] * seen + sc[1] * v_e;
            } else {
                const float keep = sc[0], take = sc[1], em = sc[2], kq = sc[3];
                float read = 0.f, nq = 0.f;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    read = fmaf(rr[i], S[i], read);
                    nq = fmaf(rr[i], nv[i], nq);
                }
#pragma unroll
                for (int o = LANES / 2; o > 0; o >>= 1) {
                    read += __shfl_xor_sync(0xffffffffu, read, o);
                    nq += __shfl_xor_sync(0xffffffffu, nq, o);
                }
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const float tk_d = take * kk[i];
                    S[i] = fmaf(tk_d, v_e, keep * S[i]);
                    nv[i] = fmaf(keep, nv[i], tk_d);
                }
                if (l == 0 && live) {
                    const float num = fmaf(keep, read, kq * v_e);
                    const float den = fmaxf(fabsf(fmaf(keep, nq, kq)), em) + p.den_eps;
                    out_col[(size_t)(c0 + j) * HE] = num / den;
                }
            }
        };
        if (nt == TC) {
            // a whole chunk, unrolled: a token's reads of shared memory stand beside the shuffles of the token before
#pragma unroll
            for (int j = 0; j < TC; ++j) walk(j);
        } else {
            for (int j = 0; j < nt; ++j) walk(j);
        }
    }
    if (Sg && live) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = l * DPL + i;
            if (d < D) Sg[(size_t)d * E + e] = S[i];
        }
    }
    if (ng && tile == 0 && col == 0) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = l * DPL + i;
            if (d < D) ng[d] = nv[i];
        }
    }
}

template <typename T, int FORM>
int launch_scan(const ScanParams& p, int n_seqs, cudaStream_t st) {
    const int vecs = FORM == FORM_DELTA ? 5 : 2;
    const size_t smem = (size_t)TC * (vecs * p.D + CT + 4) * sizeof(float);
    const dim3 grid(ceil_div(p.E, CT), p.H, n_seqs), block(LANES * CT);
    const int dpl = ceil_div(p.D, LANES);
#define SCAN_CASE(N)                                                                                                           \
    if (dpl <= N) {                                                                                                            \
        if (p.D == LANES * N)                                                                                                  \
            LLMK_CHECK_LAUNCH_RC("memory_scan", llmk_launch(memory_scan_kernel<T, FORM, N, true>, grid, block, smem, st, true, p)); \
        else                                                                                                                   \
            LLMK_CHECK_LAUNCH_RC("memory_scan", llmk_launch(memory_scan_kernel<T, FORM, N, false>, grid, block, smem, st, true, p)); \
        return LLMK_OK;                                                                                                        \
    }
    SCAN_CASE(1) SCAN_CASE(2) SCAN_CASE(4) SCAN_CASE(8) SCAN_CASE(16)
#undef SCAN_CASE
    LLMK_FAIL("memory_scan: key width %d exceeds 256", p.D);
}

}  // namespace

// out[t, c] = S_t * silu(g_t) with S_t = (1 - z) S_(t-1) + z cand over each sequence; zxg float32 [n, 3C] rows `ld` apart;
// state [slots, >= C] float32 rows `state_ld` apart.
// Steps of up to this many token rows walk token by token, a thread a channel; longer ones scan tiles of 32 tokens.
constexpr int MIN_GRU_FEW_TOKENS = 64;
LLMK_EXPORT int llmk_min_gru(void* out, const float* zxg, long long ld, const float* bz, const float* bx, float* state,
                             long long state_ld, const int* cu_q, const int* state_slots, int n_seqs, int n_rows, int C, int dtype,
                             void* stream) {
    if (n_seqs <= 0 || C <= 0) return LLMK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_rows > MIN_GRU_FEW_TOKENS) {
        const dim3 tgrid(ceil_div(C, GT), n_seqs), tblock(GT * GT);
        if (dtype == LLMK_F32)
            LLMK_CHECK_LAUNCH_RC("min_gru", llmk_launch(min_gru_tile_kernel<float>, tgrid, tblock, 0, st, true, (float*)out, zxg, ld, bz, bx,
                                                        state, state_ld, cu_q, state_slots, C));
        else
            LLMK_CHECK_LAUNCH_RC("min_gru", llmk_launch(min_gru_tile_kernel<bf16>, tgrid, tblock, 0, st, true, (bf16*)out, zxg, ld, bz, bx,
                                                        state, state_ld, cu_q, state_slots, C));
        return LLMK_OK;
    }
    const dim3 grid(ceil_div(C, 128), n_seqs), block(128);
    if (dtype == LLMK_F32)
        LLMK_CHECK_LAUNCH_RC("min_gru", llmk_launch(min_gru_kernel<float>, grid, block, 0, st, true, (float*)out, zxg, ld, bz, bx, state,
                                                    state_ld, cu_q, state_slots, C));
    else
        LLMK_CHECK_LAUNCH_RC("min_gru", llmk_launch(min_gru_kernel<bf16>, grid, block, 0, st, true, (bf16*)out, zxg, ld, bz, bx, state,
                                                    state_ld, cu_q, state_slots, C));
    return LLMK_OK;
}

// gates [n, H, 4] float32 <- (i, f, (q . k) q_scale, m before the token) per token and head; m [slots, >= H] carried in the state.
LLMK_EXPORT int llmk_mlstm_gates(float* gates, const void* q, long long ldq, const void* k, long long ldk, const void* gi, long long ldi,
                                 const void* gf, long long ldf, const float* bi, const float* bf, float* m_state, long long state_ld,
                                 const int* cu_q, const int* state_slots, int n_seqs, int n_rows, int H, int D, float cap, float q_scale,
                                 int dtype, void* stream) {
    if (n_seqs <= 0 || n_rows <= 0) return LLMK_OK;
    if (!(cap > 0.f)) LLMK_FAIL("mlstm_gates: the gates' bound must be positive");
    if (!host_aligned16(gates)) LLMK_FAIL("mlstm_gates: the gates' array must lie on a 16-byte boundary");
    cudaStream_t st = (cudaStream_t)stream;
    const int warps = 8;
    const dim3 grid(ceil_div(n_rows * H, warps)), block(warps * 32);
    if (dtype == LLMK_F32)
        LLMK_CHECK_LAUNCH_RC("mlstm_gates", llmk_launch(mlstm_gates_kernel<float>, grid, block, 0, st, true, gates, (const float*)q, ldq,
                                                        (const float*)k, ldk, (const float*)gi, ldi, (const float*)gf, ldf, bi, bf, cu_q,
                                                        n_seqs, n_rows, H, D, cap, q_scale));
    else
        LLMK_CHECK_LAUNCH_RC("mlstm_gates", llmk_launch(mlstm_gates_kernel<bf16>, grid, block, 0, st, true, gates, (const bf16*)q, ldq,
                                                        (const bf16*)k, ldk, (const bf16*)gi, ldi, (const bf16*)gf, ldf, bi, bf, cu_q,
                                                        n_seqs, n_rows, H, D, cap, q_scale));
    LLMK_CHECK_LAUNCH_RC("mlstm_maxima", llmk_launch(mlstm_maxima_kernel, dim3(ceil_div(n_seqs * H, 4)), dim3(128), 0, st, true, gates,
                                                     m_state, state_ld, cu_q, state_slots, n_seqs, H));
    return LLMK_OK;
}

// aux [n, 3 H D] float32 = w | b | u and dots [n, H, 2] = (b . r, k . r) of the generalized delta rule.
LLMK_EXPORT int llmk_delta_rule_prep(float* aux, float* dots, const void* r, long long ldr, const void* k, long long ldk, const void* a,
                                     long long lda, const float* decay, long long ldd, const float* a_bias, const float* w_bias,
                                     const int* cu_q, int n_seqs, int n_rows, int H, int D, float decay_scale, float unit_eps, int dtype,
                                     void* stream) {
    if (n_seqs <= 0 || n_rows <= 0) return LLMK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int warps = H < 8 ? (H < 1 ? 1 : H) : 8;
    const dim3 grid(n_rows), block(warps * 32);
    if (dtype == LLMK_F32)
        LLMK_CHECK_LAUNCH_RC("delta_rule_prep", llmk_launch(delta_rule_prep_kernel<float>, grid, block, 0, st, true, aux, dots,
                                                            (const float*)r, ldr, (const float*)k, ldk, (const float*)a, lda, decay, ldd,
                                                            a_bias, w_bias, cu_q, n_seqs, H, D, decay_scale, unit_eps));
    else
        LLMK_CHECK_LAUNCH_RC("delta_rule_prep", llmk_launch(delta_rule_prep_kernel<bf16>, grid, block, 0, st, true, aux, dots,
                                                            (const bf16*)r, ldr, (const bf16*)k, ldk, (const bf16*)a, lda, decay, ldd,
                                                            a_bias, w_bias, cu_q, n_seqs, H, D, decay_scale, unit_eps));
    return LLMK_OK;
}

// The memory's walk over each sequence's new tokens (see the top of the file).  form 0: delta, 1: mlstm.
LLMK_EXPORT int llmk_memory_scan(float* out, const void* r, long long ldr, const void* k, long long ldk, const void* v, long long ldv,
                                 const float* aux, const float* dots, float* state, long long state_ld, const int* cu_q,
                                 const int* state_slots, int n_seqs, int H, int D, int E, int form, float r_scale, float den_eps,
                                 int dtype, void* stream) {
    if (n_seqs <= 0) return LLMK_OK;
    if (H <= 0 || D <= 0 || E <= 0 || D > 256) LLMK_FAIL("memory_scan: heads %d, key width %d (at most 256), value width %d", H, D, E);
    if (form != FORM_DELTA && form != FORM_MLSTM) LLMK_FAIL("memory_scan: unknown form %d", form);
    if (form == FORM_DELTA && !aux) LLMK_FAIL("memory_scan: the delta form needs its vectors");
    ScanParams p;
    p.out = out; p.r = r; p.k = k; p.v = v; p.ldr = ldr; p.ldk = ldk; p.ldv = ldv; p.aux = aux; p.dots = dots; p.state = state;
    p.state_ld = state_ld; p.cu_q = cu_q; p.state_slots = state_slots; p.H = H; p.D = D; p.E = E; p.r_scale = r_scale; p.den_eps = den_eps;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == LLMK_F32)
        return form == FORM_DELTA ? launch_scan<float, FORM_DELTA>(p, n_seqs, st) : launch_scan<float, FORM_MLSTM>(p, n_seqs, st);
    return form == FORM_DELTA ? launch_scan<bf16, FORM_DELTA>(p, n_seqs, st) : launch_scan<bf16, FORM_MLSTM>(p, n_seqs, st);
}
