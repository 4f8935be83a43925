// Linear attention with a per-head decay and a state carried from token to token (the "lightning" mixer):
//
//   q_t = act(q~_t), k_t = act(k~_t) [dim], v_t = act(v~_t) [vdim]      act = silu (or none), float32
//   S_t = lambda_h S_(t-1) + k_t (x) v_t          S [dim, vdim] float32, per (request, head), zero at the start
//   o_t = S_t^T q_t                               float32 [vdim]
//
// A prompt portion of n tokens is taken in chunks of C = 32 tokens.  With S the state before a chunk and i, j
// counting inside it:
//   A_ij = (q_i . k_j) lambda^(i-j)  for j <= i             scores, float32, no softmax
//   o_i  = lambda^(i+1) S^T q_i + sum_(j<=i) A_ij v_j
//   S'   = lambda^n S + sum_j lambda^(n-1-j) k_j (x) v_j     n = tokens of this chunk
// which is the recurrence above written out, so a single decoded token (n = 1) and a portion cut anywhere give the
// same values up to float32 rounding.  Everything is float32 on the CUDA cores: the state, the decay powers, the
// scores and their products with v.
//
// Work split: one block per (sequence, head, slice of 32 value columns): a column of S never meets another
// column, so slices of vdim are independent.  Thread (e, g) = (lane, warp) keeps S[d, e] for d = g, g + 8, ... in
// registers and a copy of the block's S in shared memory for the S^T q products.
//
// A step of more than 256 tokens cuts every sequence's tokens into segments of 256 that run side by side, each from an
// empty state; a scan over the segments' end states gives the state before each segment (and the request's new
// state), and a third launch adds that state's share, lambda^(i+1) S_before^T q_i, to the segment's outputs.  A
// prompt's chunks then no longer form one chain of dependent steps on a handful of SMs.
//
// A sequence whose state slot is negative or that brings no tokens (the padding of a step laid out for replay) is
// skipped.
#define LLMK_MODULE_NAME "linear_attention"
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int LA_C = 32;        // tokens per chunk
constexpr int LA_WARPS = 8;
constexpr int LA_EV = 32;       // value columns per block

struct LinAttnParams {
    const void* q;              // rows of the packed projection; q, k, v start at these pointers
    const void* k;
    const void* v;
    long long ld;               // row stride of the packed projection, in elements
    float* out;                 // [tokens, heads * vdim] float32
    float* state;               // [slots, heads, dim, vdim] float32
    const float* decay;         // [heads]
    const int* cu_q;            // [seqs + 1]
    const int* state_slots;     // [seqs]
    int heads, dim, vdim, silu;
    // segments > 1: a sequence's tokens are cut into segments of LA_SEG, each run by a block of its own from an
    // empty state; `seg_state` [segments of all sequences][heads][dim][vdim] receives each segment's end state
    int segments, n_seqs;
    float* seg_state;
};

constexpr int LA_SEG = 256;     // tokens per segment (a multiple of the chunk)

// Index of sequence s's first segment among all segments of the step, and how many it has.
__device__ __forceinline__ int la_segment_base(const int* cu_q, int s, int& count) {
    int base = 0;
    for (int i = 0; i < s; ++i) base += max(1, ceil_div(cu_q[i + 1] - cu_q[i], LA_SEG));
    count = max(1, ceil_div(cu_q[s + 1] - cu_q[s], LA_SEG));
    return base;
}

__device__ __forceinline__ float la_act(float x, int silu) { return silu ? __fdividef(x, 1.0f + __expf(-x)) : x; }

template <typename T, int DPT>
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_kernel(LinAttnParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.dim, E = p.vdim;
    const int DP = D + 1;                  // rows of k: a lane per row reads without bank conflicts
    const int DQ = (D + 3) & ~3;           // rows of q: read as float4 broadcasts
    float* Qs = smem;                      // [C][DQ]
    float* Ks = Qs + LA_C * DQ;            // [C][D + 1]
    float* Kt = Ks + LA_C * DP;            // [D][C]: the keys once more, a key dimension's 32 tokens side by side
    float* Vs = Kt + D * LA_C;             // [C][EV]
    float* As = Vs + LA_C * LA_EV;         // [C][C + 1]
    float* Ss = As + LA_C * (LA_C + 1);    // [D][EV]
    float* pw = Ss + D * LA_EV;            // [C + 1] powers of the decay
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int vsplits = ceil_div(p.vdim, LA_EV);
    const int s = blockIdx.x, h = blockIdx.y, e0 = ((int)blockIdx.z % vsplits) * LA_EV;
    const int seg = (int)blockIdx.z / vsplits;
    const int e = e0 + lane;
    const bool e_ok = e < E;
    const float lam = p.decay[h];
    if (threadIdx.x <= LA_C) pw[threadIdx.x] = powf(lam, (float)threadIdx.x);
    pdl_launch_dependents();
    pdl_wait();
    const int slot = p.state_slots[s];
    int t_beg = p.cu_q[s], n_tok = p.cu_q[s + 1] - t_beg;
    if (slot < 0 || n_tok <= 0) return;
    float* Sg = p.state + (((size_t)slot * p.heads + h) * D) * E;
    const bool local = p.segments > 1;      // this block runs one segment from an empty state
    if (local) {
        if (seg * LA_SEG >= n_tok) return;
        int count;
        const int base = la_segment_base(p.cu_q, s, count);
        Sg = p.seg_state + (((size_t)(base + seg) * p.heads + h) * D) * E;
        t_beg += seg * LA_SEG;
        n_tok = min(LA_SEG, n_tok - seg * LA_SEG);
    }
    float S[DPT];
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int d = g + LA_WARPS * r;
        S[r] = (d < D && e_ok && !local) ? Sg[(size_t)d * E + e] : 0.f;
        if (d < D) Ss[d * LA_EV + lane] = S[r];
    }
    const T* qb = static_cast<const T*>(p.q) + (size_t)h * D;
    const T* kb = static_cast<const T*>(p.k) + (size_t)h * D;
    const T* vb = static_cast<const T*>(p.v) + (size_t)h * E;
    constexpr int VN = Vec16<T>::N;
    const bool vec_ok = D % VN == 0 && p.ld % VN == 0 && aligned16(qb) && aligned16(kb);
    for (int c0 = 0; c0 < n_tok; c0 += LA_C) {
        const int n = min(LA_C, n_tok - c0);
        __syncthreads();                    // the chunk before is consumed, Ss and pw are written
        if (vec_ok) {
            // 16 bytes of q and of k per thread and turn
            const int vecs = D / VN;
            for (int idx = threadIdx.x; idx < LA_C * vecs; idx += blockDim.x) {
                const int i = idx / vecs, d = (idx % vecs) * VN;
                float qf[VN], kf[VN];
                if (i < n) {
                    const size_t row = (size_t)(t_beg + c0 + i) * p.ld;
                    Vec16<T> qv, kv;
                    qv.raw = *reinterpret_cast<const decltype(qv.raw)*>(qb + row + d);
                    kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(kb + row + d);
                    qv.unpack(qf);
                    kv.unpack(kf);
#pragma unroll
                    for (int u = 0; u < VN; ++u) {
                        qf[u] = la_act(qf[u], p.silu);
                        kf[u] = la_act(kf[u], p.silu);
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < VN; ++u) qf[u] = kf[u] = 0.f;
                }
#pragma unroll
                for (int u = 0; u < VN; ++u) {
                    Qs[i * DQ + d + u] = qf[u];
                    Ks[i * DP + d + u] = kf[u];
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < LA_C * D; idx += blockDim.x) {
                const int i = idx / D, d = idx % D;
                float qv = 0.f, kv = 0.f;
                if (i < n) {
                    const size_t row = (size_t)(t_beg + c0 + i) * p.ld;
                    qv = la_act(to_float(qb[row + d]), p.silu);
                    kv = la_act(to_float(kb[row + d]), p.silu);
                }
                Qs[i * DQ + d] = qv;
                Ks[i * DP + d] = kv;
            }
        }
        for (int idx = threadIdx.x; idx < LA_C * LA_EV; idx += blockDim.x) {
            const int i = idx / LA_EV, ee = idx % LA_EV;
            float vv = 0.f;
            if (i < n && e0 + ee < E) vv = la_act(to_float(vb[(size_t)(t_beg + c0 + i) * p.ld + e0 + ee]), p.silu);
            Vs[idx] = vv;
        }
        __syncthreads();
        // the keys once more, transposed (read by the state's update, two barriers from here)
        for (int d = g; d < D; d += LA_WARPS) Kt[d * LA_C + lane] = Ks[lane * DP + d];
        // scores: warp g takes rows i = g, g + 8, g + 16, g + 24 together, lane j the key; a key value is read once
        // for the four rows, the queries come as float4 broadcasts
        {
            constexpr int R = LA_C / LA_WARPS;
            float a[R];
#pragma unroll
            for (int r = 0; r < R; ++r) a[r] = 0.f;
            const float* kj = Ks + lane * DP;
            for (int d4 = 0; d4 < D / 4; ++d4) {
                const float k0 = kj[4 * d4], k1 = kj[4 * d4 + 1], k2 = kj[4 * d4 + 2], k3 = kj[4 * d4 + 3];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float4 q = *reinterpret_cast<const float4*>(Qs + (g + LA_WARPS * r) * DQ + 4 * d4);
                    a[r] = fmaf(q.x, k0, a[r]); a[r] = fmaf(q.y, k1, a[r]); a[r] = fmaf(q.z, k2, a[r]); a[r] = fmaf(q.w, k3, a[r]);
                }
            }
            for (int d = D & ~3; d < D; ++d) {
                const float kv = kj[d];
#pragma unroll
                for (int r = 0; r < R; ++r) a[r] = fmaf(Qs[(g + LA_WARPS * r) * DQ + d], kv, a[r]);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = g + LA_WARPS * r;
                As[i * (LA_C + 1) + lane] = (lane <= i && i < n) ? a[r] * pw[i - lane] : 0.f;
            }
        }
        __syncthreads();
        // outputs: thread (e, g) takes rows i = g, g + 8, g + 16, g + 24
        {
            float acc[LA_C / LA_WARPS];
#pragma unroll
            for (int r = 0; r < LA_C / LA_WARPS; ++r) acc[r] = 0.f;
            for (int d4 = 0; d4 < D / 4; ++d4) {
                const float s0 = Ss[(4 * d4) * LA_EV + lane], s1 = Ss[(4 * d4 + 1) * LA_EV + lane];
                const float s2 = Ss[(4 * d4 + 2) * LA_EV + lane], s3 = Ss[(4 * d4 + 3) * LA_EV + lane];
#pragma unroll
                for (int r = 0; r < LA_C / LA_WARPS; ++r) {
                    const float4 q = *reinterpret_cast<const float4*>(Qs + (g + LA_WARPS * r) * DQ + 4 * d4);
                    acc[r] = fmaf(q.x, s0, acc[r]); acc[r] = fmaf(q.y, s1, acc[r]); acc[r] = fmaf(q.z, s2, acc[r]); acc[r] = fmaf(q.w, s3, acc[r]);
                }
            }
            for (int d = D & ~3; d < D; ++d) {
                const float sv = Ss[d * LA_EV + lane];
#pragma unroll
                for (int r = 0; r < LA_C / LA_WARPS; ++r) acc[r] = fmaf(Qs[(g + LA_WARPS * r) * DQ + d], sv, acc[r]);
            }
#pragma unroll
            for (int r = 0; r < LA_C / LA_WARPS; ++r) {
                const int i = g + LA_WARPS * r;
                if (i >= n) continue;
                float o = acc[r] * pw[i + 1];
                for (int j = 0; j <= i; ++j) o = fmaf(As[i * (LA_C + 1) + j], Vs[j * LA_EV + lane], o);
                if (e_ok) p.out[(size_t)(t_beg + c0 + i) * ((size_t)p.heads * E) + (size_t)h * E + e] = o;
            }
        }
        __syncthreads();                    // every reader of Ss is done
        // state: S[d, e] = lambda^n S[d, e] + sum_j lambda^(n-1-j) k_j[d] v_j[e]
        {
            const float keep = pw[n];
            float add[DPT];
#pragma unroll
            for (int r = 0; r < DPT; ++r) add[r] = 0.f;
            // sixteen tokens at a time: their decayed values in registers, a key dimension's sixteen tokens as four float4
            // broadcasts (rows beyond the chunk hold zeros)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float vw[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const int j = 16 * half + u;
                    vw[u] = j < n ? Vs[j * LA_EV + lane] * pw[n - 1 - j] : 0.f;
                }
#pragma unroll
                for (int r = 0; r < DPT; ++r) {
                    const int d = g + LA_WARPS * r;
                    if (d < D) {
                        const float4* kt = reinterpret_cast<const float4*>(Kt + d * LA_C + 16 * half);
#pragma unroll
                        for (int u4 = 0; u4 < 4; ++u4) {
                            const float4 k = kt[u4];
                            add[r] = fmaf(k.x, vw[4 * u4], add[r]); add[r] = fmaf(k.y, vw[4 * u4 + 1], add[r]);
                            add[r] = fmaf(k.z, vw[4 * u4 + 2], add[r]); add[r] = fmaf(k.w, vw[4 * u4 + 3], add[r]);
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < DPT; ++r) {
                const int d = g + LA_WARPS * r;
                S[r] = fmaf(keep, S[r], add[r]);
                if (d < D) Ss[d * LA_EV + lane] = S[r];
            }
        }
    }
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int d = g + LA_WARPS * r;
        if (d < D && e_ok) Sg[(size_t)d * E + e] = S[r];
    }
}

// Scan over a sequence's segments, a thread per entry (d, e) of the state: `seg_state[g]` holds segment g's end state
// from an empty start and receives the state BEFORE segment g; the request's state receives the state after the last
// one.  S_before(g + 1) = lambda^len(g) S_before(g) + S_local(g).  The segments' values are asked for eight at a time
// before the chain of multiply-adds that needs them.
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_scan_kernel(LinAttnParams p) {
    const int D = p.dim, E = p.vdim;
    const int s = blockIdx.x, h = blockIdx.y;
    const int entry = blockIdx.z * blockDim.x + threadIdx.x;        // d * E + e
    pdl_launch_dependents();
    pdl_wait();
    const int slot = p.state_slots[s];
    const int n_tok = p.cu_q[s + 1] - p.cu_q[s];
    if (slot < 0 || n_tok <= 0 || entry >= D * E) return;
    int count;
    const int base = la_segment_base(p.cu_q, s, count);
    const float lam = p.decay[h];
    const float full = powf(lam, (float)LA_SEG);
    float* Sg = p.state + ((size_t)slot * p.heads + h) * D * E + entry;
    const size_t stride = (size_t)p.heads * D * E;
    float* loc = p.seg_state + ((size_t)base * p.heads + h) * D * E + entry;
    float S = *Sg;
    for (int k0 = 0; k0 < count; k0 += 8) {
        float end_local[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) end_local[u] = k0 + u < count ? loc[(size_t)(k0 + u) * stride] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (k0 + u >= count) break;
            loc[(size_t)(k0 + u) * stride] = S;
            const int len = min(LA_SEG, n_tok - (k0 + u) * LA_SEG);
            S = fmaf(len == LA_SEG ? full : powf(lam, (float)len), S, end_local[u]);
        }
    }
    *Sg = S;
}

// The share of the state before a segment in the segment's outputs: out[i, e] += lambda^(i + 1) sum_d q_i[d] S_before[d, e],
// i counting inside the segment.  One block per (sequence, head, 32 value columns x segment), chunks of 32 tokens.
template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_carry_kernel(LinAttnParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.dim, E = p.vdim;
    const int DP = (D + 3) & ~3;           // rows of q, read as float4 broadcasts
    float* Qs = smem;                      // [C][DP]
    float* Ss = Qs + LA_C * DP;            // [D][EV]
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int vsplits = ceil_div(E, LA_EV);
    const int s = blockIdx.x, h = blockIdx.y, e0 = ((int)blockIdx.z % vsplits) * LA_EV, seg = (int)blockIdx.z / vsplits;
    const int e = e0 + lane;
    pdl_launch_dependents();
    pdl_wait();
    const int slot = p.state_slots[s];
    const int n_all = p.cu_q[s + 1] - p.cu_q[s];
    if (slot < 0 || n_all <= 0 || seg * LA_SEG >= n_all) return;
    int count;
    const int base = la_segment_base(p.cu_q, s, count);
    const float* Sb = p.seg_state + (((size_t)(base + seg) * p.heads + h) * D) * E;
    const int t_beg = p.cu_q[s] + seg * LA_SEG, n_tok = min(LA_SEG, n_all - seg * LA_SEG);
    const float lam = p.decay[h];
    for (int idx = threadIdx.x; idx < D * LA_EV; idx += blockDim.x) {
        const int d = idx / LA_EV, ee = idx % LA_EV;
        Ss[idx] = e0 + ee < E ? Sb[(size_t)d * E + e0 + ee] : 0.f;
    }
    const T* qb = static_cast<const T*>(p.q) + (size_t)h * D;
    constexpr int VN = Vec16<T>::N;
    const bool vec_ok = D % VN == 0 && p.ld % VN == 0 && aligned16(qb);
    for (int c0 = 0; c0 < n_tok; c0 += LA_C) {
        const int n = min(LA_C, n_tok - c0);
        __syncthreads();
        if (vec_ok) {
            const int vecs = D / VN;
            for (int idx = threadIdx.x; idx < LA_C * vecs; idx += blockDim.x) {
                const int i = idx / vecs, d = (idx % vecs) * VN;
                float qf[VN];
                if (i < n) {
                    Vec16<T> qv;
                    qv.raw = *reinterpret_cast<const decltype(qv.raw)*>(qb + (size_t)(t_beg + c0 + i) * p.ld + d);
                    qv.unpack(qf);
#pragma unroll
                    for (int u = 0; u < VN; ++u) qf[u] = la_act(qf[u], p.silu);
                } else {
#pragma unroll
                    for (int u = 0; u < VN; ++u) qf[u] = 0.f;
                }
#pragma unroll
                for (int u = 0; u < VN; ++u) Qs[i * DP + d + u] = qf[u];
            }
        } else {
            for (int idx = threadIdx.x; idx < LA_C * D; idx += blockDim.x) {
                const int i = idx / D, d = idx % D;
                Qs[i * DP + d] = i < n ? la_act(to_float(qb[(size_t)(t_beg + c0 + i) * p.ld + d]), p.silu) : 0.f;
            }
        }
        __syncthreads();
        float acc[LA_C / LA_WARPS];
#pragma unroll
        for (int r = 0; r < LA_C / LA_WARPS; ++r) acc[r] = 0.f;
        for (int d4 = 0; d4 < D / 4; ++d4) {
            const float s0 = Ss[(4 * d4) * LA_EV + lane], s1 = Ss[(4 * d4 + 1) * LA_EV + lane];
            const float s2 = Ss[(4 * d4 + 2) * LA_EV + lane], s3 = Ss[(4 * d4 + 3) * LA_EV + lane];
#pragma unroll
            for (int r = 0; r < LA_C / LA_WARPS; ++r) {
                const float4 q = *reinterpret_cast<const float4*>(Qs + (g + LA_WARPS * r) * DP + 4 * d4);
                acc[r] = fmaf(q.x, s0, acc[r]); acc[r] = fmaf(q.y, s1, acc[r]); acc[r] = fmaf(q.z, s2, acc[r]); acc[r] = fmaf(q.w, s3, acc[r]);
            }
        }
        for (int d = D & ~3; d < D; ++d) {
            const float sv = Ss[d * LA_EV + lane];
#pragma unroll
            for (int r = 0; r < LA_C / LA_WARPS; ++r) acc[r] = fmaf(Qs[(g + LA_WARPS * r) * DP + d], sv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < LA_C / LA_WARPS; ++r) {
            const int i = g + LA_WARPS * r;
            if (i < n && e < E) {
                float* o = p.out + (size_t)(t_beg + c0 + i) * ((size_t)p.heads * E) + (size_t)h * E + e;
                *o = fmaf(powf(lam, (float)(c0 + i + 1)), acc[r], *o);
            }
        }
    }
}

template <typename T, int DPT>
static int launch_linear_attention(const LinAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(linear_attention_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("linear_attention: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
    }
    LLMK_CHECK_LAUNCH_RC("linear_attention", llmk_launch(linear_attention_kernel<T, DPT>, grid, dim3(LA_WARPS * 32), smem, s, true, p));
    return LLMK_OK;
}

template <typename T>
static int dispatch_linear_attention(const LinAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    const int dpt = ceil_div(p.dim, LA_WARPS);
    if (dpt <= 4) return launch_linear_attention<T, 4>(p, grid, smem, s);
    if (dpt <= 8) return launch_linear_attention<T, 8>(p, grid, smem, s);
    if (dpt <= 16) return launch_linear_attention<T, 16>(p, grid, smem, s);
    return launch_linear_attention<T, 32>(p, grid, smem, s);
}

// q, k, v: pointers to the first row's q, k and v inside the packed projection (rows `ld` elements apart, heads
// side by side); out float32 [tokens, heads * vdim]; state float32 [slots, heads, dim, vdim]; decay float32 [heads].
// Floats of scratch that a step of `n_tokens` tokens in `n_seqs` sequences needs for its segments' states (0: the step
// runs without segments).
LLMK_EXPORT long long llmk_linear_attention_scratch_floats(int n_tokens, int n_seqs, int heads, int dim, int vdim) {
    if (n_tokens <= LA_SEG) return 0;
    return (long long)(n_tokens / LA_SEG + n_seqs) * heads * dim * vdim;
}

// n_tokens: rows of `out` (all tokens of the step).  With more than LA_SEG of them a sequence's tokens are cut into
// segments that run side by side (three launches: segments from an empty state, the scan over their end states, the
// carried state's share of the outputs) and `seg_state` must hold llmk_linear_attention_scratch_floats(...) floats.
LLMK_EXPORT int llmk_linear_attention(float* out, const void* q, const void* k, const void* v, long long ld, float* state,
                                      const float* decay, const int* cu_q, const int* state_slots, int n_seqs, int heads,
                                      int dim, int vdim, int silu, int n_tokens, float* seg_state, int dtype, void* stream) {
    if (n_seqs <= 0) return LLMK_OK;
    if (heads <= 0 || dim <= 0 || vdim <= 0) LLMK_FAIL("linear_attention: bad sizes (heads %d, dim %d, vdim %d)", heads, dim, vdim);
    if (dim > 32 * LA_WARPS) LLMK_FAIL("linear_attention: dim %d is more than %d", dim, 32 * LA_WARPS);
    if (heads > 65535) LLMK_FAIL("linear_attention: too many heads");
    LinAttnParams p;
    p.q = q; p.k = k; p.v = v; p.ld = ld; p.out = out; p.state = state; p.decay = decay; p.cu_q = cu_q;
    p.state_slots = state_slots; p.heads = heads; p.dim = dim; p.vdim = vdim; p.silu = silu;
    p.n_seqs = n_seqs;
    p.segments = n_tokens > LA_SEG ? ceil_div(n_tokens, LA_SEG) : 1;
    p.seg_state = seg_state;
    if (p.segments > 1 && !seg_state) LLMK_FAIL("linear_attention: %d tokens need scratch for the segments' states", n_tokens);
    if (dtype != LLMK_F32 && dtype != LLMK_BF16) LLMK_FAIL("linear_attention: unknown dtype %d", dtype);
    const int vsplits = ceil_div(vdim, LA_EV);
    if ((long long)vsplits * p.segments > 65535) LLMK_FAIL("linear_attention: too many segments");
    const size_t smem = ((size_t)LA_C * (((dim + 3) & ~3) + dim + 1) + (size_t)dim * LA_C + LA_C * LA_EV + LA_C * (LA_C + 1) +
                         (size_t)dim * LA_EV + LA_C + 1) * sizeof(float);
    dim3 grid(n_seqs, heads, vsplits * p.segments);
    cudaStream_t s = (cudaStream_t)stream;
    const int rc = dtype == LLMK_F32 ? dispatch_linear_attention<float>(p, grid, smem, s) : dispatch_linear_attention<bf16>(p, grid, smem, s);
    if (rc != LLMK_OK || p.segments == 1) return rc;
    LLMK_CHECK_LAUNCH_RC("linear_attention_scan", llmk_launch(linear_attention_scan_kernel, dim3(n_seqs, heads, ceil_div(dim * vdim, LA_WARPS * 32)),
                                                              dim3(LA_WARPS * 32), 0, s, true, p));
    const size_t smem_c = ((size_t)LA_C * ((dim + 3) & ~3) + (size_t)dim * LA_EV) * sizeof(float);
    if (dtype == LLMK_F32) {
        if (smem_c > 48 * 1024) cudaFuncSetAttribute(linear_attention_carry_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);
        LLMK_CHECK_LAUNCH_RC("linear_attention_carry", llmk_launch(linear_attention_carry_kernel<float>, grid, dim3(LA_WARPS * 32), smem_c, s, true, p));
    } else {
        if (smem_c > 48 * 1024) cudaFuncSetAttribute(linear_attention_carry_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);
        LLMK_CHECK_LAUNCH_RC("linear_attention_carry", llmk_launch(linear_attention_carry_kernel<bf16>, grid, dim3(LA_WARPS * 32), smem_c, s, true, p));
    }
    return LLMK_OK;
}
