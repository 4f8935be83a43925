// Attention whose keys and values are expanded from one cached latent vector per token (multi-head latent
// attention).  Per token the cache holds  z = [c | kr]:  c = rmsnorm(c~) * gain  [rank]  and one rotated key part
// kr [rot] shared by all heads; head h's key is [Wuk_h c | kr] and its value Wuv_h c.  Instead of expanding the
// keys of the whole context, the query is taken into the latent space and the output out of it:
//
//   score_ij = (qn_i . Wuk_h c_j + qr_i . kr_j) * scale = ([Wuk_h^T qn_i | qr_i] . z_j) * scale
//   o_i      = Wuv_h (sum_j p_ij c_j)
//
// so the attention itself is one shared "kv head" of width rank + rot whose values are the first `rank` entries of
// the same cached vector.  Four kernels:
//
//   latent_prep      per token: cq = rmsnorm(dq~) * gain (the query's latent, for the product that follows);
//                    c and the rotated kr written to the token's place in the paged cache
//   latent_absorb    qa[t, h] = [Wuk_h^T qn | rotate(qr)]                      float32 [tokens, heads, rank + rot]
//                    (or, with Wuk folded into the query's up-projection at load, one product and `latent_rotate`)
//   latent_attention causal softmax attention of qa over the cached z; float32 scores, weights and sums
//                    (+ latent_reduce for key parts, flash-decoding)            float32 [tokens, heads, rank]
//   latent_expand    out[t, h] = (Wuv_h oa[t, h]) * sigmoid(g[t, h])           storage dtype [tokens, heads * vdim]
//
// Rotation: pairs (2i, 2i + 1) ("interleaved") or (i, i + rot/2) ("half"), by the angle whose cos / sin the tables
// hold per position.  Positions, angles, norms, scores, softmax and all sums are float32; the cache and the
// matrices have the storage dtype.
#define LLMK_MODULE_NAME "latent_attention"
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

__device__ __forceinline__ void rotate_into(float* dst, const float* src, int rot, int pairing, const float* cs, const float* sn,
                                            int i) {
    // pair i of rot / 2
    const int a = pairing == LLMK_PAIR_INTERLEAVED ? 2 * i : i;
    const int b = pairing == LLMK_PAIR_INTERLEAVED ? 2 * i + 1 : i + rot / 2;
    const float u = src[a], v = src[b], c = cs[i], s = sn[i];
    dst[a] = u * c - v * s;
    dst[b] = v * c + u * s;
}

// ---------------------------------------------------------------------------------------------- prep
// One block per token.  `dq` [q_rank] and `dkv` [rank + rot] are read from the packed projection row.
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ packed, long long ld, int dq_off, int dkv_off, int q_rank, int rank, int rot,
                                   const float* __restrict__ q_gain, const float* __restrict__ kv_gain, float eps,
                                   T* __restrict__ cq_out, T* __restrict__ cache, const int* __restrict__ positions,
                                   const int* __restrict__ slots, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   int pairing) {
    extern __shared__ float sm[];   // rot floats in, rot floats out, 33 scratch
    float* kr_in = sm;
    float* kr_out = sm + rot;
    float* scratch = sm + 2 * rot;
    const size_t t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const T* row = packed + t * ld;
    if (cq_out && q_rank > 0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_float(row[dq_off + i]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float rinv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq_out[t * q_rank + i] = from_float<T>(to_float(row[dq_off + i]) * rinv * q_gain[i]);
    }
    const int slot = slots ? slots[t] : -1;
    if (slot < 0 || !cache) return;      // a row that belongs to no sequence, or a pass that stores nothing
    T* z = cache + (size_t)slot * (rank + rot);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(row[dkv_off + i]);
        ss += v * v;
    }
    for (int i = threadIdx.x; i < rot; i += blockDim.x) kr_in[i] = to_float(row[dkv_off + rank + i]);
    ss = block_sum(ss, scratch);         // also orders kr_in
    const float rinv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) z[i] = from_float<T>(to_float(row[dkv_off + i]) * rinv * kv_gain[i]);
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x)
        rotate_into(kr_out, kr_in, rot, pairing, cos_t + (size_t)pos * (rot / 2), sin_t + (size_t)pos * (rot / 2), i);
    __syncthreads();
    for (int i = threadIdx.x; i < rot; i += blockDim.x) z[rank + i] = from_float<T>(kr_out[i]);
}

LLMK_EXPORT int llmk_latent_prep(const void* packed, long long ld, int dq_off, int dkv_off, int q_rank, int rank, int rot,
                                 const float* q_gain, const float* kv_gain, float eps, void* cq_out, void* cache,
                                 const int* positions, const int* slots, const float* cos_t, const float* sin_t, int pairing,
                                 int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    if (rank <= 0 || rot < 0 || rot % 2 != 0) LLMK_FAIL("latent_prep: bad sizes (rank %d, rot %d)", rank, rot);
    if (pairing != LLMK_PAIR_INTERLEAVED && pairing != LLMK_PAIR_HALF_SPLIT) LLMK_FAIL("latent_prep: unknown rotary pairing %d", pairing);
    const size_t smem = ((size_t)2 * rot + 33) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(latent_prep_kernel<float>, dim3(n_tokens), dim3(128), smem, s, true, (const float*)packed, ld, dq_off, dkv_off,
                        q_rank, rank, rot, q_gain, kv_gain, eps, (float*)cq_out, (float*)cache, positions, slots, cos_t, sin_t, pairing);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(latent_prep_kernel<bf16>, dim3(n_tokens), dim3(128), smem, s, true, (const bf16*)packed, ld, dq_off, dkv_off,
                        q_rank, rank, rot, q_gain, kv_gain, eps, (bf16*)cq_out, (bf16*)cache, positions, slots, cos_t, sin_t, pairing);
    else
        LLMK_FAIL("latent_prep: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("latent_prep", e);
    return LLMK_OK;
}

// -------------------------------------------------------------------------------------------- absorb
// Block (tile of TT tokens, head).  q [tokens, heads * (dim + rot)] of T; wuk [heads * dim, rank] of T (as stored:
// row h * dim + d is key dimension d of head h); qa float32 [tokens, heads, rank + rot].
constexpr int LT_TT = 16;

template <typename T>
__global__ void __launch_bounds__(128) latent_absorb_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ wuk,
                                                            float* __restrict__ qa, const int* __restrict__ positions,
                                                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                            int n_tokens, int heads, int dim, int rot, int rank, int pairing) {
    extern __shared__ float sm[];   // [TT][dim] unrotated parts, [TT][rot] rotated parts in, [TT][rot] out
    float* qn = sm;
    float* qr = qn + LT_TT * dim;
    float* qo = qr + LT_TT * rot;
    const int t0 = blockIdx.x * LT_TT, h = blockIdx.y;
    const int n = min(LT_TT, n_tokens - t0);
    pdl_launch_dependents();
    pdl_wait();
    const int hd = dim + rot;
    for (int idx = threadIdx.x; idx < LT_TT * hd; idx += blockDim.x) {
        const int i = idx / hd, d = idx % hd;
        const float v = i < n ? to_float(q[(size_t)(t0 + i) * ldq + (size_t)h * hd + d]) : 0.f;
        if (d < dim) qn[i * dim + d] = v; else qr[i * rot + d - dim] = v;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < LT_TT * (rot / 2); idx += blockDim.x) {
        const int i = idx / (rot / 2), pr = idx % (rot / 2);
        if (i < n) {
            const int pos = positions[t0 + i];
            rotate_into(qo + i * rot, qr + i * rot, rot, pairing, cos_t + (size_t)pos * (rot / 2), sin_t + (size_t)pos * (rot / 2), pr);
        }
    }
    const int za = rank + rot;
    const T* w = wuk + (size_t)h * dim * rank;
    // this block's slice of the latent's columns: a thread per column, the loads of W eight rows ahead of their use
    const int r = blockIdx.z * blockDim.x + threadIdx.x;
    if (r < rank) {
        float acc[LT_TT];
#pragma unroll
        for (int i = 0; i < LT_TT; ++i) acc[i] = 0.f;
        int d = 0;
        for (; d + 8 <= dim; d += 8) {
            float wv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) wv[u] = to_float(w[(size_t)(d + u) * rank + r]);
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int i = 0; i < LT_TT; ++i) acc[i] = fmaf(qn[i * dim + d + u], wv[u], acc[i]);
        }
        for (; d < dim; ++d) {
            const float wv = to_float(w[(size_t)d * rank + r]);
#pragma unroll
            for (int i = 0; i < LT_TT; ++i) acc[i] = fmaf(qn[i * dim + d], wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < LT_TT; ++i)
            if (i < n) qa[((size_t)(t0 + i) * heads + h) * za + r] = acc[i];
    }
    __syncthreads();
    if (blockIdx.z == 0)
        for (int idx = threadIdx.x; idx < LT_TT * rot; idx += blockDim.x) {
            const int i = idx / rot, dd = idx % rot;
            if (i < n) qa[((size_t)(t0 + i) * heads + h) * za + rank + dd] = qo[idx];
        }
}

LLMK_EXPORT int llmk_latent_absorb(float* qa, const void* q, long long ldq, const void* wuk, const int* positions,
                                   const float* cos_t, const float* sin_t, int n_tokens, int heads, int dim, int rot, int rank,
                                   int pairing, int dtype, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    if (heads <= 0 || heads > 65535 || dim < 0 || rot < 0 || rot % 2 != 0 || rank <= 0) LLMK_FAIL("latent_absorb: bad sizes");
    if (pairing != LLMK_PAIR_INTERLEAVED && pairing != LLMK_PAIR_HALF_SPLIT) LLMK_FAIL("latent_absorb: unknown rotary pairing %d", pairing);
    const size_t smem = (size_t)LT_TT * (dim + 2 * rot) * sizeof(float);
    dim3 grid(ceil_div(n_tokens, LT_TT), heads, ceil_div(rank, 128));
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_absorb_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(latent_absorb_kernel<float>, grid, dim3(128), smem, s, true, (const float*)q, ldq, (const float*)wuk, qa, positions,
                        cos_t, sin_t, n_tokens, heads, dim, rot, rank, pairing);
    } else if (dtype == LLMK_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_absorb_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(latent_absorb_kernel<bf16>, grid, dim3(128), smem, s, true, (const bf16*)q, ldq, (const bf16*)wuk, qa, positions,
                        cos_t, sin_t, n_tokens, heads, dim, rot, rank, pairing);
    } else
        LLMK_FAIL("latent_absorb: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("latent_absorb", e);
    return LLMK_OK;
}

// -------------------------------------------------------------------------------------------- rotate
// For queries that were projected straight into the latent space (Wuk folded into Wuq when the model was loaded):
// the rotated part of every head of qa [tokens, heads, rank + rot] is turned in place.  One block per token.
__global__ void latent_rotate_kernel(float* __restrict__ qa, const int* __restrict__ positions, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int heads, int rank, int rot, int pairing) {
    const size_t t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int half = rot / 2;
    const int pos = positions[t];
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        float* q = qa + (t * heads + h) * (size_t)(rank + rot) + rank;
        const int a = pairing == LLMK_PAIR_INTERLEAVED ? 2 * i : i;
        const int b = pairing == LLMK_PAIR_INTERLEAVED ? 2 * i + 1 : i + half;
        const float u = q[a], v = q[b], c = cs[i], sv = sn[i];
        q[a] = u * c - v * sv;
        q[b] = v * c + u * sv;
    }
}

LLMK_EXPORT int llmk_latent_rotate(float* qa, const int* positions, const float* cos_t, const float* sin_t, int n_tokens, int heads,
                                   int rank, int rot, int pairing, void* stream) {
    if (n_tokens <= 0 || rot <= 0) return LLMK_OK;
    if (rot % 2 != 0 || heads <= 0 || rank < 0) LLMK_FAIL("latent_rotate: bad sizes");
    if (pairing != LLMK_PAIR_INTERLEAVED && pairing != LLMK_PAIR_HALF_SPLIT) LLMK_FAIL("latent_rotate: unknown rotary pairing %d", pairing);
    LLMK_CHECK_LAUNCH_RC("latent_rotate", llmk_launch(latent_rotate_kernel, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, true, qa, positions,
                                                      cos_t, sin_t, heads, rank, rot, pairing));
    return LLMK_OK;
}

// ----------------------------------------------------------------------------------------- attention
// One block per (tile of queries of one sequence, chunk of heads, key part): up to 32 rows = bq queries x gc
// heads, four rows a warp; every tile of 32 cached vectors is read once (16-byte loads) for all rows of the block.
// Sequence s owns query rows [cu_q[s], cu_q[s+1]) and has ctx[s] keys after this step; query j of the portion sits at
// position ctx - q_len + j and sees keys 0..position.  The step's own vectors were written to the cache before.
// A lane owns one key of the tile for the scores (the queries come as float4 broadcasts) and 1/32 of the latent's
// values for the weighted sums.
constexpr int LT_WARPS = 8;
constexpr int LT_R = 4;                     // rows a warp
constexpr int LT_ROWS = LT_WARPS * LT_R;
constexpr int LT_KT = 32;

struct LatentAttnParams {
    const float* qa;           // [tokens, heads, za]
    const void* cache;         // [pages, page_size, za]
    float* out;                // [tokens, heads, rank]
    bf16* out_hm;              // or, if set: bfloat16 [heads, t_pad, rank] (head-major, for the grouped product that follows)
    int t_pad;
    const int* block_tables;
    const int* ctx_len;
    const int* cu_q;
    const int* tile_seq;
    const int* tile_q0;
    float* part_o;
    float* part_ml;
    int max_blocks, heads, rank, za, page_size, num_parts, bq, gc, chunks;
    float scale;
};

template <typename T, int RL>
__global__ void __launch_bounds__(LT_WARPS * 32) latent_attention_kernel(LatentAttnParams p) {
    extern __shared__ __align__(16) float smem[];
    const int za = p.za, rank = p.rank;
    const int zq = (za + 3) & ~3;           // a row of queries starts on 16 bytes
    float* Qs = smem;                       // [ROWS][zq], pre-multiplied by scale
    float* Zs = Qs + LT_ROWS * zq;          // [KT][za + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    const int s = p.tile_seq[blockIdx.x];
    if (s < 0) return;                      // padding of a tile list of fixed length
    const int q0 = p.tile_q0[blockIdx.x];
    const int chunk = blockIdx.y, part = blockIdx.z;
    const int q_beg = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q_beg;
    const int ctx = p.ctx_len[s];
    const int nq_tile = min(p.bq, q_len - q0);
    const bool padding = ctx < q_len || nq_tile <= 0;
    const int first_pos = ctx - q_len + q0;
    int k_beg = 0, k_end = 0;
    if (!padding) k_end = first_pos + nq_tile;
    if (p.num_parts > 1) {
        const int part_size = ceil_div(ceil_div(max(ctx, 1), p.num_parts), LT_KT) * LT_KT;
        k_beg = max(k_beg, part * part_size);
        k_end = min(k_end, (part + 1) * part_size);
    }
    const T* zc = static_cast<const T*>(p.cache);
    const int* bt = p.block_tables + (size_t)s * p.max_blocks;
    const int rows = p.bq * p.gc;
    if (p.num_parts > 1 && k_beg >= k_end) {
        // a key part beyond this sequence's keys: its rows say "nothing seen" and the block leaves at once
        for (int r = threadIdx.x; r < rows; r += blockDim.x) {
            const int qi = r / p.gc, hh = chunk * p.gc + r % p.gc;
            if (qi < max(nq_tile, 0) && hh < p.heads) {
                const size_t row = ((size_t)(q_beg + q0 + qi) * p.heads + hh) * p.num_parts + part;
                p.part_ml[row * 2] = -INFINITY;
                p.part_ml[row * 2 + 1] = 0.f;
            }
        }
        return;
    }
    // the block's queries: a warp per row and turn, the lanes across the row (16 bytes each where rows allow it)
    const bool q_vec = (za & 3) == 0;
    for (int r = warp; r < LT_ROWS; r += LT_WARPS) {
        const int qi = r / p.gc, hh = chunk * p.gc + r % p.gc;
        const bool live = r < rows && qi < nq_tile && hh < p.heads;
        const float* src = p.qa + ((size_t)(q_beg + q0 + (live ? qi : 0)) * p.heads + (live ? hh : 0)) * za;
        float* dst = Qs + r * zq;
        if (q_vec) {
            for (int d4 = lane; d4 < zq / 4; d4 += 32) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) {
                    v = *reinterpret_cast<const float4*>(src + 4 * d4);
                    v.x *= p.scale; v.y *= p.scale; v.z *= p.scale; v.w *= p.scale;
                }
                *reinterpret_cast<float4*>(dst + 4 * d4) = v;
            }
        } else {
            for (int d = lane; d < zq; d += 32) dst[d] = (live && d < za) ? src[d] * p.scale : 0.f;
        }
    }
    int r_of[LT_R], qi_of[LT_R], head_of[LT_R];
    bool valid[LT_R];
    bool any_valid = false;
#pragma unroll
    for (int i = 0; i < LT_R; ++i) {
        r_of[i] = warp + i * LT_WARPS;
        qi_of[i] = r_of[i] / p.gc;
        head_of[i] = chunk * p.gc + r_of[i] % p.gc;
        valid[i] = r_of[i] < rows && qi_of[i] < nq_tile && head_of[i] < p.heads && !padding;
        any_valid = any_valid || valid[i];
    }
    float m[LT_R], l[LT_R];
    float acc[LT_R][RL];
#pragma unroll
    for (int i = 0; i < LT_R; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < RL; ++j) acc[i][j] = 0.f;
    }
    constexpr int VN = Vec16<T>::N;
    const bool vec_fill = za % VN == 0 && aligned16(zc);
    const int vecs = za / VN;

    for (int t0 = k_beg; t0 < k_end; t0 += LT_KT) {
        __syncthreads();                    // the tile before is consumed (and Qs written, the first time)
        // the tile's cached vectors: a warp takes keys warp, warp + 8, ...; the page of each is looked up once and the
        // lanes go across the vector, so the loads of a warp's four keys are in flight together
#pragma unroll
        for (int kk = 0; kk < LT_KT / LT_WARPS; ++kk) {
            const int key = warp + kk * LT_WARPS;
            const int kpos = t0 + key;
            const bool live = kpos < k_end;
            const T* src = zc;
            if (live) src = zc + ((size_t)bt[kpos / p.page_size] * p.page_size + kpos % p.page_size) * za;
            float* dst = Zs + key * (za + 1);
            if (vec_fill) {
                for (int vec = lane; vec < vecs; vec += 32) {
                    float f[VN];
                    if (live) {
                        Vec16<T> v;
                        v.raw = *reinterpret_cast<const decltype(v.raw)*>(src + (size_t)vec * VN);
                        v.unpack(f);
                    } else {
#pragma unroll
                        for (int i = 0; i < VN; ++i) f[i] = 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < VN; ++i) dst[vec * VN + i] = f[i];
                }
            } else {
                for (int d = lane; d < za; d += 32) dst[d] = live ? to_float(src[d]) : 0.f;
            }
        }
        __syncthreads();
        if (!any_valid) continue;
        float sc[LT_R];
#pragma unroll
        for (int i = 0; i < LT_R; ++i) sc[i] = 0.f;
        {
            const float* kr = Zs + lane * (za + 1);
            const float4* q4[LT_R];
#pragma unroll
            for (int i = 0; i < LT_R; ++i) q4[i] = reinterpret_cast<const float4*>(Qs + r_of[i] * zq);
            const int d4_end = za / 4;
            for (int d4 = 0; d4 < d4_end; ++d4) {
                const float k0 = kr[4 * d4], k1 = kr[4 * d4 + 1], k2 = kr[4 * d4 + 2], k3 = kr[4 * d4 + 3];
#pragma unroll
                for (int i = 0; i < LT_R; ++i) {
                    const float4 q = q4[i][d4];
                    sc[i] = fmaf(q.x, k0, sc[i]); sc[i] = fmaf(q.y, k1, sc[i]);
                    sc[i] = fmaf(q.z, k2, sc[i]); sc[i] = fmaf(q.w, k3, sc[i]);
                }
            }
            for (int d = 4 * d4_end; d < za; ++d) {
                const float kv = kr[d];
#pragma unroll
                for (int i = 0; i < LT_R; ++i) sc[i] = fmaf(Qs[r_of[i] * zq + d], kv, sc[i]);
            }
        }
        const int kpos = t0 + lane;
        float pr[LT_R];
#pragma unroll
        for (int i = 0; i < LT_R; ++i) {
            const int qpos = first_pos + qi_of[i];
            const bool ok = valid[i] && kpos < k_end && kpos <= qpos;
            const float sv = ok ? sc[i] : -INFINITY;
            const float tmax = warp_max(sv);
            const float m_new = fmaxf(m[i], tmax);
            float corr = 1.f;
            pr[i] = 0.f;
            if (m_new > -INFINITY) {
                corr = m[i] > -INFINITY ? expf(m[i] - m_new) : 0.f;
                pr[i] = ok ? expf(sv - m_new) : 0.f;
                m[i] = m_new;
            }
            l[i] = l[i] * corr + warp_sum(pr[i]);
#pragma unroll
            for (int j = 0; j < RL; ++j) acc[i][j] *= corr;
        }
        const int kmax = min(LT_KT, k_end - t0);
        for (int k = 0; k < kmax; ++k) {
            float pk[LT_R];
#pragma unroll
            for (int i = 0; i < LT_R; ++i) pk[i] = __shfl_sync(0xffffffffu, pr[i], k);
            const float* vr = Zs + k * (za + 1);
#pragma unroll
            for (int j = 0; j < RL; ++j) {
                const int d = lane + 32 * j;
                if (d < rank) {
                    const float v = vr[d];
#pragma unroll
                    for (int i = 0; i < LT_R; ++i) acc[i][j] = fmaf(pk[i], v, acc[i][j]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < LT_R; ++i) {
        const bool owned = r_of[i] < rows && qi_of[i] < max(nq_tile, 0) && head_of[i] < p.heads;
        if (!owned) continue;
        const size_t tok = (size_t)(q_beg + q0 + qi_of[i]);
        if (p.num_parts > 1) {
            const size_t row = (tok * p.heads + head_of[i]) * p.num_parts + part;
#pragma unroll
            for (int j = 0; j < RL; ++j) {
                const int d = lane + 32 * j;
                if (d < rank) p.part_o[row * rank + d] = acc[i][j];
            }
            if (lane == 0) {
                p.part_ml[row * 2] = m[i];
                p.part_ml[row * 2 + 1] = l[i];
            }
        } else {
            float* o = p.out + (tok * p.heads + head_of[i]) * rank;
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
            for (int j = 0; j < RL; ++j) {
                const int d = lane + 32 * j;
                if (d < rank) o[d] = acc[i][j] * inv;
            }
        }
    }
}

// ------------------------------------------------------------------------------ attention, tensor cores
// The same attention for bfloat16 caches whose sizes fit (za a multiple of 16, rank a multiple of 64), on the tensor
// cores by `mma.sync.m16n8k16` with float32 accumulators:
//   S = Q Z^T          Q rounded to bfloat16 as it enters shared memory, Z as cached; scores float32
//   O += P Z[:, :rank] the float32 weights P enter as three bfloat16 terms (p = p1 + p2 + p3, 24 bits of mantissa: every
//                      product p_i z is exact in float32 and the sum is a float32 sum), so the weights are not rounded
// A block has 8 warps = 2 groups of 16 rows x 4: for the scores a warp takes its group's rows and 8 of the tile's 32
// keys; the scores pass through shared memory, every warp of a group then does the group's softmax and takes a
// quarter of the latent's values for the weighted sums.  Rows, tiles, key parts and the merge are those of the
// kernel above.
constexpr int MT_KT = 32;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// p = t1 + t2 + t3 with bfloat16 terms; returns the packed pairs of two neighbouring weights
__device__ __forceinline__ void split3(float p0, float p1, uint32_t& w1, uint32_t& w2, uint32_t& w3) {
    const float a0 = __bfloat162float(__float2bfloat16_rn(p0)), a1 = __bfloat162float(__float2bfloat16_rn(p1));
    const float r0 = p0 - a0, r1 = p1 - a1;
    const float b0 = __bfloat162float(__float2bfloat16_rn(r0)), b1 = __bfloat162float(__float2bfloat16_rn(r1));
    w1 = pack_bf16(a0, a1);
    w2 = pack_bf16(b0, b1);
    w3 = pack_bf16(r0 - b0, r1 - b1);
}

template <int NT>       // most tiles of 8 latent values a warp accumulates (rank / 32 of them are used)
__global__ void __launch_bounds__(256) latent_attention_mma_kernel(LatentAttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_mma[];
    const int za = p.za, rank = p.rank;
    const int zp = za + 8;                                  // row stride: consecutive rows 16 bytes apart in the banks
    bf16* Qs = reinterpret_cast<bf16*>(smem_mma);            // [32][zp]
    bf16* Zs = Qs + LT_ROWS * zp;                            // [32][zp]
    float* Ss = reinterpret_cast<float*>(Zs + MT_KT * zp);   // [32][33]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = warp >> 2, wq = warp & 3;                 // group of 16 rows, quarter
    pdl_launch_dependents();
    pdl_wait();
    const int s = p.tile_seq[blockIdx.x];
    if (s < 0) return;
    const int q0 = p.tile_q0[blockIdx.x];
    const int chunk = blockIdx.y, part = blockIdx.z;
    const int q_beg = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q_beg;
    const int ctx = p.ctx_len[s];
    const int nq_tile = min(p.bq, q_len - q0);
    const bool padding = ctx < q_len || nq_tile <= 0;
    const int first_pos = ctx - q_len + q0;
    int k_beg = 0, k_end = 0;
    if (!padding) k_end = first_pos + nq_tile;
    if (p.num_parts > 1) {
        const int part_size = ceil_div(ceil_div(max(ctx, 1), p.num_parts), MT_KT) * MT_KT;
        k_beg = max(k_beg, part * part_size);
        k_end = min(k_end, (part + 1) * part_size);
    }
    const int rows = p.bq * p.gc;
    if (p.num_parts > 1 && k_beg >= k_end) {
        for (int r = threadIdx.x; r < rows; r += blockDim.x) {
            const int qi = r / p.gc, hh = chunk * p.gc + r % p.gc;
            if (qi < max(nq_tile, 0) && hh < p.heads) {
                const size_t row = ((size_t)(q_beg + q0 + qi) * p.heads + hh) * p.num_parts + part;
                p.part_ml[row * 2] = -INFINITY;
                p.part_ml[row * 2 + 1] = 0.f;
            }
        }
        return;
    }
    const bf16* zc = static_cast<const bf16*>(p.cache);
    const int* bt = p.block_tables + (size_t)s * p.max_blocks;
    // the block's queries, rounded to bfloat16
    for (int r = warp; r < LT_ROWS; r += LT_WARPS) {
        const int qi = r / p.gc, hh = chunk * p.gc + r % p.gc;
        const bool live = r < rows && qi < nq_tile && hh < p.heads;
        const float* src = p.qa + ((size_t)(q_beg + q0 + (live ? qi : 0)) * p.heads + (live ? hh : 0)) * za;
        for (int d = lane * 2; d < za; d += 64) {
            float2 v = make_float2(0.f, 0.f);
            if (live) v = *reinterpret_cast<const float2*>(src + d);
            *reinterpret_cast<__nv_bfloat162*>(Qs + r * zp + d) = __floats2bfloat162_rn(v.x, v.y);
        }
    }
    // this lane's two rows of its group: g and g + 8
    int qpos[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rg * 16 + (lane >> 2) + 8 * i;
        const int qi = r / p.gc, hh = chunk * p.gc + r % p.gc;
        valid[i] = r < rows && qi < nq_tile && hh < p.heads && !padding;
        qpos[i] = first_pos + qi;
    }
    const bool group_live = rg * 16 < rows && (rg * 16) / p.gc < nq_tile;      // uniform over the warp
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    const int nt = rank / 32;                    // tiles of 8 values this warp accumulates
    const int d0 = wq * nt * 8;
    const int vecs = za / 8;
    const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(Qs);
    const uint32_t zs_addr = (uint32_t)__cvta_generic_to_shared(Zs);

    for (int t0 = k_beg; t0 < k_end; t0 += MT_KT) {
        __syncthreads();                         // the tile before is consumed (and Qs written, the first time)
        // the tile's cached vectors: a warp takes keys warp, warp + 8, ...; the pages of its four keys are looked up
        // first, then the lanes go across the vectors, the loads of two keys in flight before their stores
        {
            const bf16* src[MT_KT / LT_WARPS];
#pragma unroll
            for (int kk = 0; kk < MT_KT / LT_WARPS; ++kk) {
                const int kpos = t0 + warp + kk * LT_WARPS;
                src[kk] = kpos < k_end ? zc + ((size_t)bt[kpos / p.page_size] * p.page_size + kpos % p.page_size) * za : nullptr;
            }
#pragma unroll
            for (int kk = 0; kk < MT_KT / LT_WARPS; kk += 2) {
                for (int vec = lane; vec < vecs; vec += 32) {
                    uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
                    if (src[kk]) v0 = *reinterpret_cast<const uint4*>(src[kk] + (size_t)vec * 8);
                    if (src[kk + 1]) v1 = *reinterpret_cast<const uint4*>(src[kk + 1] + (size_t)vec * 8);
                    *reinterpret_cast<uint4*>(Zs + (warp + kk * LT_WARPS) * zp + vec * 8) = v0;
                    *reinterpret_cast<uint4*>(Zs + (warp + (kk + 1) * LT_WARPS) * zp + vec * 8) = v1;
                }
            }
        }
        __syncthreads();
        // scores of the group's 16 rows with keys 8 wq .. 8 wq + 7
        if (group_live) {
            // four accumulators in turn, so that consecutive products do not wait for one another
            float c4[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e) c4[u][e] = 0.f;
            const uint32_t a_base = qs_addr + (uint32_t)(((rg * 16 + (lane & 15)) * zp + (lane >> 4) * 8) * 2);
            const uint32_t b_base = zs_addr + (uint32_t)(((wq * 8 + (lane & 7)) * zp + ((lane >> 3) & 1) * 8) * 2);
            const int steps = za / 16;
            int ks = 0;
            for (; ks + 4 <= steps; ks += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint32_t a[4], b[2];
                    ldmatrix_x4(a, a_base + (uint32_t)((ks + u) * 32));
                    ldmatrix_x2(b, b_base + (uint32_t)((ks + u) * 32));
                    mma_bf16(c4[u], a, b[0], b[1]);
                }
            }
            for (; ks < steps; ++ks) {
                uint32_t a[4], b[2];
                ldmatrix_x4(a, a_base + (uint32_t)(ks * 32));
                ldmatrix_x2(b, b_base + (uint32_t)(ks * 32));
                mma_bf16(c4[0], a, b[0], b[1]);
            }
            float c[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) c[e] = (c4[0][e] + c4[1][e]) + (c4[2][e] + c4[3][e]);
            float* srow = Ss + (rg * 16 + (lane >> 2)) * 33 + wq * 8 + (lane & 3) * 2;
            srow[0] = c[0] * p.scale;
            srow[1] = c[1] * p.scale;
            srow[8 * 33] = c[2] * p.scale;
            srow[8 * 33 + 1] = c[3] * p.scale;
        }
        __syncthreads();
        if (!group_live) continue;
        // the group's softmax (every warp of the group does it) in the layout of the next product's first operand
        float pv[2][2][2][2];                    // [row i][step of 16 keys t][half h][e]
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = 16 * t + 8 * h + (lane & 3) * 2 + e;
                        const int kpos = t0 + col;
                        const bool ok = valid[i] && kpos < k_end && kpos <= qpos[i];
                        const float sv = ok ? Ss[(rg * 16 + (lane >> 2) + 8 * i) * 33 + col] : -INFINITY;
                        pv[i][t][h][e] = sv;
                        tmax[i] = fmaxf(tmax[i], sv);
                    }
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            const float m_new = fmaxf(m[i], tmax[i]);
            corr[i] = 1.f;
            float sum = 0.f;
            if (m_new > -INFINITY) {
                corr[i] = m[i] > -INFINITY ? expf(m[i] - m_new) : 0.f;
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float sv = pv[i][t][h][e];
                            const float pe = sv > -INFINITY ? expf(sv - m_new) : 0.f;
                            pv[i][t][h][e] = pe;
                            sum += pe;
                        }
                m[i] = m_new;
            } else {
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int e = 0; e < 2; ++e) pv[i][t][h][e] = 0.f;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l[i] = l[i] * corr[i] + sum;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            acc[j][0] *= corr[0]; acc[j][1] *= corr[0];
            acc[j][2] *= corr[1]; acc[j][3] *= corr[1];
        }
        // weights as three bfloat16 terms, per step of 16 keys: a0 (row g, keys 0-7), a1 (row g + 8), a2 (row g, keys 8-15), a3
        uint32_t pa[2][3][4];
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    split3(pv[i][t][h][0], pv[i][t][h][1], pa[t][0][2 * h + i], pa[t][1][2 * h + i], pa[t][2][2 * h + i]);
        // weighted sums over this warp's quarter of the latent's values
        const uint32_t v_base = zs_addr + (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * zp + d0 + (lane >> 4) * 8) * 2);
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
            if (2 * jp >= nt) break;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, v_base + (uint32_t)((t * 16 * zp + jp * 16) * 2));
#pragma unroll
                for (int term = 0; term < 3; ++term) {
                    mma_bf16(acc[2 * jp], pa[t][term], b[0], b[1]);
                    mma_bf16(acc[2 * jp + 1], pa[t][term], b[2], b[3]);
                }
            }
        }
    }
    if (!group_live) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rg * 16 + (lane >> 2) + 8 * i;
        if (!(r < rows && r / p.gc < max(nq_tile, 0) && chunk * p.gc + r % p.gc < p.heads)) continue;     // nobody's row
        const size_t tokhead = (size_t)(q_beg + q0 + r / p.gc) * p.heads + chunk * p.gc + r % p.gc;
        if (p.num_parts > 1) {
            const size_t row = tokhead * p.num_parts + part;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (j >= nt) break;
                const int d = d0 + j * 8 + (lane & 3) * 2;
                p.part_o[row * rank + d] = acc[j][2 * i];
                p.part_o[row * rank + d + 1] = acc[j][2 * i + 1];
            }
            if (wq == 0 && (lane & 3) == 0) {
                p.part_ml[row * 2] = m[i];
                p.part_ml[row * 2 + 1] = l[i];
            }
        } else {
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
            if (p.out_hm) {
                bf16* o = p.out_hm + ((size_t)(chunk * p.gc + r % p.gc) * p.t_pad + (size_t)(q_beg + q0 + r / p.gc)) * rank;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if (j >= nt) break;
                    const int d = d0 + j * 8 + (lane & 3) * 2;
                    *reinterpret_cast<__nv_bfloat162*>(o + d) = __floats2bfloat162_rn(acc[j][2 * i] * inv, acc[j][2 * i + 1] * inv);
                }
                continue;
            }
            float* o = p.out + tokhead * rank;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (j >= nt) break;
                const int d = d0 + j * 8 + (lane & 3) * 2;
                o[d] = acc[j][2 * i] * inv;
                o[d + 1] = acc[j][2 * i + 1] * inv;
            }
        }
    }
}

// One block per (token, head): merge the key parts in part order.  The parts' weights e^(m_p - M) are computed once,
// then every thread adds up its values of the latent over the parts.
__global__ void __launch_bounds__(128) latent_reduce_kernel(float* __restrict__ out, const float* __restrict__ part_o,
                                                            const float* __restrict__ part_ml, int rank, int num_parts,
                                                            bf16* __restrict__ out_hm, int heads, int t_pad) {
    extern __shared__ float wgt[];     // [num_parts] weights, then 1 / denominator
    const size_t row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* ml = part_ml + row * num_parts * 2;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float M = -INFINITY;
        for (int pt = lane; pt < num_parts; pt += 32)
            if (ml[2 * pt + 1] > 0.f) M = fmaxf(M, ml[2 * pt]);
        M = warp_max(M);
        float denom = 0.f;
        for (int pt = lane; pt < num_parts; pt += 32) {
            const float w = ml[2 * pt + 1] > 0.f ? expf(ml[2 * pt] - M) : 0.f;
            wgt[pt] = w;
            denom += w * ml[2 * pt + 1];
        }
        // the denominator in part order, so that it does not depend on how the lanes were summed
        __syncwarp();
        if (lane == 0) {
            float d = 0.f;
            for (int pt = 0; pt < num_parts; ++pt) d += wgt[pt] * ml[2 * pt + 1];
            wgt[num_parts] = d > 0.f ? 1.0f / d : 0.f;
        }
        (void)denom;
    }
    __syncthreads();
    const float inv = wgt[num_parts];
    const float* po = part_o + row * num_parts * rank;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float v = 0.f;
#pragma unroll 4
        for (int pt = 0; pt < num_parts; ++pt)
            if (wgt[pt] != 0.f) v = fmaf(wgt[pt], po[(size_t)pt * rank + d], v);     // a part that saw nothing wrote nothing
        if (out_hm) out_hm[((row % heads) * t_pad + row / heads) * rank + d] = __float2bfloat16_rn(v * inv);
        else out[row * rank + d] = v * inv;
    }
}

template <typename T, int RL>
static int launch_latent_attention(const LatentAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<T, RL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("latent_attention: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
    }
    LLMK_CHECK_LAUNCH_RC("latent_attention", llmk_launch(latent_attention_kernel<T, RL>, grid, dim3(LT_WARPS * 32), smem, s, true, p));
    return LLMK_OK;
}

template <typename T>
static int dispatch_latent_attention(const LatentAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    const int rl = ceil_div(p.rank, 32);
    if (rl <= 1) return launch_latent_attention<T, 1>(p, grid, smem, s);
    if (rl <= 2) return launch_latent_attention<T, 2>(p, grid, smem, s);
    if (rl <= 4) return launch_latent_attention<T, 4>(p, grid, smem, s);
    if (rl <= 8) return launch_latent_attention<T, 8>(p, grid, smem, s);
    return launch_latent_attention<T, 16>(p, grid, smem, s);
}

template <int NT>
static int launch_latent_attention_mma(const LatentAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("latent_attention: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
    }
    LLMK_CHECK_LAUNCH_RC("latent_attention", llmk_launch(latent_attention_mma_kernel<NT>, grid, dim3(LT_WARPS * 32), smem, s, true, p));
    return LLMK_OK;
}

static int g_latent_mma = 1;     // 0: the float32 kernel for bfloat16 caches too (for measurements and tests)
LLMK_EXPORT void llmk_latent_attention_set_mma(int on) { g_latent_mma = on; }

// Queries per tile for `heads` heads: rows = bq * gc <= 32.
LLMK_EXPORT int llmk_latent_attention_tile_queries(int heads) {
    if (heads <= 0) return 0;
    const int gc = heads < LT_ROWS ? heads : LT_ROWS;
    return LT_ROWS / gc;
}

// 1 if a bfloat16 cache of these sizes goes through the tensor cores (and may then leave its result head-major).
LLMK_EXPORT int llmk_latent_attention_on_tensor_cores(int rank, int rot, int dtype) {
    return dtype == LLMK_BF16 && g_latent_mma && (rank + rot) % 16 == 0 && rank % 64 == 0 && rank <= 512;
}

// out_hm (optional, tensor-core form only): the result as bfloat16 [heads, t_pad, rank] instead of float32 in `out`.
LLMK_EXPORT int llmk_latent_attention(float* out, const float* qa, const void* cache, const int* block_tables, int max_blocks,
                                      const int* ctx_len, const int* cu_q, const int* tile_seq, const int* tile_q0, int n_tiles,
                                      int n_tokens, int heads, int rank, int rot, int page_size, float scale, int num_parts,
                                      float* scratch, void* out_hm, int t_pad, int dtype, void* stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return LLMK_OK;
    if (heads <= 0 || rank <= 0 || rank > 512 || rot < 0) LLMK_FAIL("latent_attention: bad sizes (heads %d, rank %d, rot %d)", heads, rank, rot);
    if (page_size <= 0) LLMK_FAIL("latent_attention: page_size %d", page_size);
    if (num_parts < 1 || num_parts > 65535 || (num_parts > 1 && !scratch)) LLMK_FAIL("latent_attention: bad split (%d parts)", num_parts);
    LatentAttnParams p;
    p.gc = heads < LT_ROWS ? heads : LT_ROWS;
    p.bq = LT_ROWS / p.gc;
    p.chunks = ceil_div(heads, p.gc);
    p.qa = qa; p.cache = cache; p.out = out; p.block_tables = block_tables; p.ctx_len = ctx_len; p.cu_q = cu_q;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.max_blocks = max_blocks; p.heads = heads; p.rank = rank; p.za = rank + rot;
    p.page_size = page_size; p.num_parts = num_parts; p.scale = scale;
    p.part_o = scratch;
    p.part_ml = num_parts > 1 ? scratch + (size_t)n_tokens * heads * num_parts * rank : nullptr;
    p.out_hm = static_cast<bf16*>(out_hm);
    p.t_pad = t_pad;
    const size_t smem = ((size_t)LT_ROWS * ((p.za + 3) & ~3) + (size_t)LT_KT * (p.za + 1)) * sizeof(float);
    if (smem > 220 * 1024) LLMK_FAIL("latent_attention: cached vectors of %d values do not fit shared memory", p.za);
    dim3 grid(n_tiles, p.chunks, num_parts);
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    const bool mma = llmk_latent_attention_on_tensor_cores(rank, rot, dtype) && host_aligned16(cache) && ((uintptr_t)qa & 7) == 0;
    if (out_hm && (!mma || t_pad < n_tokens)) LLMK_FAIL("latent_attention: a head-major result needs the tensor-core form and room for %d tokens", n_tokens);
    if (mma) {
        const size_t smem_mma = ((size_t)(LT_ROWS + MT_KT) * (p.za + 8)) * sizeof(bf16) + (size_t)LT_ROWS * 33 * sizeof(float);
        const int nt = rank / 32;
        rc = nt <= 2 ? launch_latent_attention_mma<2>(p, grid, smem_mma, s)
             : nt <= 4 ? launch_latent_attention_mma<4>(p, grid, smem_mma, s)
             : nt <= 8 ? launch_latent_attention_mma<8>(p, grid, smem_mma, s)
                       : launch_latent_attention_mma<16>(p, grid, smem_mma, s);
    } else if (dtype == LLMK_F32)
        rc = dispatch_latent_attention<float>(p, grid, smem, s);
    else if (dtype == LLMK_BF16)
        rc = dispatch_latent_attention<bf16>(p, grid, smem, s);
    else
        LLMK_FAIL("latent_attention: unknown dtype %d", dtype);
    if (rc != LLMK_OK) return rc;
    if (num_parts > 1) {
        const int n_rows = n_tokens * heads;
        LLMK_CHECK_LAUNCH_RC("latent_reduce", llmk_launch(latent_reduce_kernel, dim3(n_rows), dim3(128), (size_t)(num_parts + 1) * sizeof(float), s,
                                                          true, out, (const float*)p.part_o, (const float*)p.part_ml, rank, num_parts,
                                                          mma ? p.out_hm : nullptr, heads, p.t_pad));
    }
    return LLMK_OK;
}

// ---------------------------------------------------------------------------------------------- gate
// After the grouped product Wuv_h oa_h: out[t, h * vdim + j] = (T)(o[(h * t_pad + t) * vdim + j] * sigmoid(g[t, h * vdim + j])),
// o float32 head-major.
template <typename T>
__global__ void latent_gate_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ g, long long ldg, int n_tokens,
                                   int heads, int vdim, int t_pad) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)n_tokens * heads * vdim;
    const int wide = heads * vdim;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t t = (size_t)(i / wide);
        const int c = (int)(i % wide), h = c / vdim, j = c % vdim;
        float v = o[((size_t)h * t_pad + t) * vdim + j];
        if (g) v *= 1.0f / (1.0f + expf(-to_float(g[t * ldg + c])));
        out[i] = from_float<T>(v);
    }
}

LLMK_EXPORT int llmk_latent_gate(void* out, const float* o, const void* g, long long ldg, int n_tokens, int heads, int vdim, int t_pad,
                                 int dtype, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    long long blocks = ((long long)n_tokens * heads * vdim + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(latent_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, (float*)out, o, (const float*)g, ldg, n_tokens,
                        heads, vdim, t_pad);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(latent_gate_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, (bf16*)out, o, (const bf16*)g, ldg, n_tokens,
                        heads, vdim, t_pad);
    else
        LLMK_FAIL("latent_gate: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("latent_gate", e);
    return LLMK_OK;
}

// -------------------------------------------------------------------------------------------- expand
// Block (tile of TT tokens, head, slice of `cols` output values of the head); a warp per output value j:
// out[t, h * vdim + j] = (wuv[h * vdim + j, :] . oa[t, h, :]) * sigmoid(g[t, h * vdim + j]).  With few tokens a head's
// outputs are cut into slices of 32 so that there are blocks for the SMs; with many, one block takes the whole head and
// reads its rows of oa once.
template <typename T>
__global__ void __launch_bounds__(256) latent_expand_kernel(T* __restrict__ out, const float* __restrict__ oa, const T* __restrict__ wuv,
                                                            const T* __restrict__ g, long long ldg, int n_tokens, int heads, int rank,
                                                            int vdim, int cols) {
    extern __shared__ float os[];   // [TT][rank]
    const int t0 = blockIdx.x * LT_TT, h = blockIdx.y;
    const int n = min(LT_TT, n_tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    for (int idx = threadIdx.x; idx < LT_TT * rank; idx += blockDim.x) {
        const int i = idx / rank, r = idx % rank;
        os[idx] = i < n ? oa[((size_t)(t0 + i) * heads + h) * rank + r] : 0.f;
    }
    __syncthreads();
    const int j_end = min(vdim, (int)(blockIdx.z + 1) * cols);
    for (int j = blockIdx.z * cols + warp; j < j_end; j += nwarps) {
        const T* w = wuv + ((size_t)h * vdim + j) * rank;
        float acc[LT_TT];
#pragma unroll
        for (int i = 0; i < LT_TT; ++i) acc[i] = 0.f;
        for (int r = lane; r < rank; r += 32) {
            const float wv = to_float(w[r]);
#pragma unroll
            for (int i = 0; i < LT_TT; ++i) acc[i] = fmaf(os[i * rank + r], wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < LT_TT; ++i) acc[i] = warp_sum(acc[i]);
        if (lane < n) {
            float v = 0.f;
#pragma unroll
            for (int i = 0; i < LT_TT; ++i)
                if (i == lane) v = acc[i];
            const size_t col = (size_t)h * vdim + j;
            float gate = 1.f;
            if (g) gate = 1.0f / (1.0f + expf(-to_float(g[(size_t)(t0 + lane) * ldg + col])));
            out[(size_t)(t0 + lane) * ((size_t)heads * vdim) + col] = from_float<T>(v * gate);
        }
    }
}

LLMK_EXPORT int llmk_latent_expand(void* out, const float* oa, const void* wuv, const void* g, long long ldg, int n_tokens, int heads,
                                   int rank, int vdim, int dtype, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    if (heads <= 0 || heads > 65535 || rank <= 0 || vdim <= 0) LLMK_FAIL("latent_expand: bad sizes");
    const size_t smem = (size_t)LT_TT * rank * sizeof(float);
    const int cols = n_tokens <= 4 * LT_TT ? 32 : vdim;
    dim3 grid(ceil_div(n_tokens, LT_TT), heads, ceil_div(vdim, cols));
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_expand_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(latent_expand_kernel<float>, grid, dim3(256), smem, s, true, (float*)out, oa, (const float*)wuv, (const float*)g, ldg,
                        n_tokens, heads, rank, vdim, cols);
    } else if (dtype == LLMK_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_expand_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(latent_expand_kernel<bf16>, grid, dim3(256), smem, s, true, (bf16*)out, oa, (const bf16*)wuv, (const bf16*)g, ldg,
                        n_tokens, heads, rank, vdim, cols);
    } else
        LLMK_FAIL("latent_expand: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("latent_expand", e);
    return LLMK_OK;
}
