// Causal grouped-query attention over the paged cache for prompts and prompt portions in bfloat16 whose softmax
// weights must stay 32-bit: the products run on the tensor cores (`mma.sync.m16n8k16`, bfloat16 operands, float32
// accumulators), everything between them on the CUDA cores in float32.
//
//   S = Q K^T      Q and K are the cache's bfloat16 values, every product exact, sums float32
//   scores         s * scale, then (softcap > 0) softcap * tanh(s / softcap), the causal (and window, or block) mask, the row's
//                  running maximum and sum, the weights exp(s - m): float32, `tanhf` and `exp2f` at full precision
//   O += P V       a float32 weight enters as THREE bfloat16 terms p = p1 + p2 + p3 (24 bits of mantissa), so every
//                  product with a bfloat16 value is what float32 arithmetic would give; three MMAs a step
//   finish         the sink (one more term exp(0) in the denominator), the division, the output gate sigmoid(g)
//
// Block = 64 queries of one sequence x one query head, four warps of 16 rows; keys in tiles of 64 through shared
// memory: 16-byte `cp.async` copies out of the pages into two buffers, the next tile on its way while this one is used.  Semantics as in csrc/attention.cu (which takes float32, single tokens in
// parts, and every size this kernel refuses): query j of a portion sits at position ctx - q_len + j.
// Taken: key width and value width 64 or 128 each.
#define LLMK_MODULE_NAME "attention_mma"
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

namespace {

constexpr int BM = 64, BN = 64, WARPS = 4;

struct Params {
    const bf16* q;
    const bf16* kcache;
    const bf16* vcache;
    bf16* out;
    const bf16* gate;
    const float* sink_values;     // with `sink`: the sink's score per query head [nq]; null: 0
    const float* turn_cos;        // [positions, VD / 2] (with turn_sin): every head's row is turned back in pairs (m, m + VD / 2) by minus
    const float* turn_sin;        // its query's position before the gate; null: rows leave as they are
    int gate_heads;               // 1: the gate is one number per head, [tokens, nq]
    const int* block_tables;
    const int* ctx_len;
    const int* cu_q;
    const int* tile_seq;
    const int* tile_q0;
    long long q_stride, o_stride, gate_stride;
    int max_blocks, nq, nkv, page_size, window, sink, chunk;     // chunk > 0: a query sees the keys of its own block of that many positions
    float scale, softcap;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// tanh(x) = 1 - 2 / (1 + e^(2x)): an absolute error of a few 1e-7, which is what a score needs (it is an exponent)
__device__ __forceinline__ float tanh_abs(float x) { return 1.0f - __fdividef(2.0f, 1.0f + exp2f(x * 2.8853900817779268f)); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// x = a + b + c with a, b, c bfloat16: the three most significant pieces of a float32
__device__ __forceinline__ void split3(float x, float& a, float& b, float& c) {
    a = __bfloat162float(__float2bfloat16_rn(x));
    const float r = x - a;
    b = __bfloat162float(__float2bfloat16_rn(r));
    c = __bfloat162float(__float2bfloat16_rn(r - b));
}

template <int HD, int VD>
__global__ void __launch_bounds__(WARPS * 32) attention_mma_kernel(Params p) {
    constexpr int QLD = HD + 8, VLD = VD + 8;      // rows 16 bytes longer: the eight rows of an ldmatrix fall on different banks
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);      // [BM][QLD]
    bf16* Kbuf = Qs + BM * QLD;                         // 2 x [BN][QLD]
    bf16* Vbuf = Kbuf + 2 * BN * QLD;                   // 2 x [BN][VLD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int s = p.tile_seq[blockIdx.x];
    pdl_launch_dependents();
    pdl_wait();
    if (s < 0) return;
    const int q0 = p.tile_q0[blockIdx.x];
    const int head = blockIdx.y;
    const int kvh = head / (p.nq / p.nkv);
    const int q_beg = p.cu_q[s], q_len = p.cu_q[s + 1] - q_beg, ctx = p.ctx_len[s];
    const int nq_tile = min(BM, q_len - q0);
    if (nq_tile <= 0 || ctx < q_len) {
        // rows of padding: zeros
        for (int idx = threadIdx.x; idx < max(nq_tile, 0) * VD; idx += blockDim.x)
            p.out[(size_t)(q_beg + q0 + idx / VD) * p.o_stride + (size_t)head * VD + idx % VD] = __float2bfloat16_rn(0.f);
        return;
    }
    const int first_pos = ctx - q_len + q0;
    const int k_end = first_pos + nq_tile;
    int k_beg = p.window > 0 ? max(0, first_pos - p.window + 1) / BN * BN : 0;
    if (p.chunk > 0) k_beg = max(k_beg, first_pos / p.chunk * p.chunk / BN * BN);
    const int* bt = p.block_tables + (size_t)s * p.max_blocks;

    for (int idx = threadIdx.x; idx < BM * (HD / 8); idx += blockDim.x) {
        const int r = idx / (HD / 8), v = idx % (HD / 8);
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r < nq_tile) val = *reinterpret_cast<const uint4*>(p.q + (size_t)(q_beg + q0 + r) * p.q_stride + (size_t)head * HD + v * 8);
        *reinterpret_cast<uint4*>(Qs + r * QLD + v * 8) = val;
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int j = 0; j < HD / 16; ++j)
        ldmatrix_x4(qf[j], Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QLD + j * 16 + (lane >> 4) * 8);

    float o[VD / 8][4];
#pragma unroll
    for (int n = 0; n < VD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int qpos[2] = {first_pos + warp * 16 + g, first_pos + warp * 16 + g + 8};
    const int kmin[2] = {p.chunk > 0 ? qpos[0] / p.chunk * p.chunk : 0, p.chunk > 0 ? qpos[1] / p.chunk * p.chunk : 0};
    const float inv_cap = p.softcap > 0.f ? 1.0f / p.softcap : 0.f;
    constexpr float LOG2E = 1.4426950408889634f;

    constexpr int VECS = HD / 8 + VD / 8;
    auto load_tile = [&](int t0, int buf) {
        bf16* Kd = Kbuf + buf * BN * QLD;
        bf16* Vd = Vbuf + buf * BN * VLD;
#pragma unroll 4
        for (int idx = threadIdx.x; idx < BN * VECS; idx += WARPS * 32) {
            const int key = idx / VECS, v = idx % VECS;
            const int kpos = t0 + key;
            bf16* dst = v < HD / 8 ? Kd + key * QLD + v * 8 : Vd + key * VLD + (v - HD / 8) * 8;
            const int page = kpos < k_end ? bt[kpos / p.page_size] : -1;      // -1 too: a page the window has passed
            if (page >= 0) {
                const size_t row = ((size_t)page * p.nkv + kvh) * p.page_size + kpos % p.page_size;
                cp_async16(dst, v < HD / 8 ? p.kcache + row * HD + v * 8 : p.vcache + row * VD + (v - HD / 8) * 8);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_tile(k_beg, 0);
    int turn = 0;
    for (int t0 = k_beg; t0 < k_end; t0 += BN, turn ^= 1) {
        cp_async_wait_all();
        __syncthreads();          // this tile has arrived, and the tile before is consumed by every warp
        if (t0 + BN < k_end) load_tile(t0 + BN, turn ^ 1);
        const bf16* Ks = Kbuf + turn * BN * QLD;
        const bf16* Vs = Vbuf + turn * BN * VLD;
        // a warp whose rows all lie before this tile's first key has nothing to do in it (causal)
        if (first_pos + warp * 16 + 15 < t0) continue;

        float sc[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
#pragma unroll
            for (int n2 = 0; n2 < BN / 16; ++n2) {
                uint32_t kb[4];
                ldmatrix_x4(kb, Ks + (n2 * 16 + (lane >> 4) * 8 + (lane & 7)) * QLD + j * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(sc[2 * n2], qf[j], kb[0], kb[1]);
                mma_bf16(sc[2 * n2 + 1], qf[j], kb[2], kb[3]);
            }
        }
        // scores, mask, the rows' maxima
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const int kpos = t0 + n * 8 + 2 * tq + (e & 1);
                float v = sc[n][e] * p.scale;
                if (p.softcap > 0.f) v = p.softcap * tanh_abs(v * inv_cap);
                const bool vis = kpos <= qpos[r] && kpos < k_end && (p.window <= 0 || kpos > qpos[r] - p.window) && kpos >= kmin[r];
                v = vis ? v : -INFINITY;
                sc[n][e] = v;
                mx[r] = fmaxf(mx[r], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            alpha[r] = (m[r] == -INFINITY) ? 0.f : exp2f((m[r] - m_new) * LOG2E);
            m[r] = m_new;
            l[r] *= alpha[r];
        }
#pragma unroll
        for (int n = 0; n < VD / 8; ++n) {
            o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
            o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
        }
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const float pv = (sc[n][e] == -INFINITY) ? 0.f : exp2f((sc[n][e] - m[r]) * LOG2E);
                sc[n][e] = pv;
                l[r] += pv;
            }
        }
        // O += P V, sixteen keys a step, the weights in three bfloat16 terms
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
            uint32_t pa[3][4];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int n = 2 * j + (q4 >> 1), e = (q4 & 1) * 2;
                float a0, b0, c0, a1, b1, c1;
                split3(sc[n][e], a0, b0, c0);
                split3(sc[n][e + 1], a1, b1, c1);
                pa[0][q4] = pack2(a0, a1);
                pa[1][q4] = pack2(b0, b1);
                pa[2][q4] = pack2(c0, c1);
            }
#pragma unroll
            for (int n2 = 0; n2 < VD / 16; ++n2) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, Vs + (j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VLD + n2 * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int term = 2; term >= 0; --term) {          // smallest terms first
                    mma_bf16(o[2 * n2], pa[term], vb[0], vb[1]);
                    mma_bf16(o[2 * n2 + 1], pa[term], vb[2], vb[3]);
                }
            }
        }
    }
    // the rows' sums over the four threads that share a row, the sink, the gate, the division
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        if (row >= nq_tile) continue;
        float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
        if (p.sink && l[r] > 0.f) {
            const float z = p.sink_values ? p.sink_values[head] : 0.f;
            const float M = fmaxf(m[r], z);
            const float w = expf(m[r] - M);
            inv = w / (l[r] * w + expf(z - M));
        }
        const size_t tok = (size_t)(q_beg + q0 + row);
        bf16* dst = p.out + tok * p.o_stride + (size_t)head * VD;
        const bf16* gt = p.gate ? p.gate + tok * p.gate_stride + (size_t)head * (p.gate_heads ? 1 : VD) : nullptr;
        const float head_gate = (gt && p.gate_heads) ? 1.0f / (1.0f + expf(-__bfloat162float(gt[0]))) : 1.f;
        if (p.turn_cos) {
            // the thread holds columns n * 8 + 2 tq (+ 1) for every n: a column and the one half a head on are both its own
            const float* cs = p.turn_cos + (size_t)qpos[r] * (VD / 2);
            const float* sn = p.turn_sin + (size_t)qpos[r] * (VD / 2);
#pragma unroll
            for (int n = 0; n < VD / 16; ++n) {
                const int col = n * 8 + 2 * tq;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float lo = o[n][2 * r + e], hi = o[n + VD / 16][2 * r + e];
                    const float c = cs[col + e], sv = sn[col + e];
                    o[n][2 * r + e] = lo * c + hi * sv;
                    o[n + VD / 16][2 * r + e] = hi * c - lo * sv;
                }
            }
        }
#pragma unroll
        for (int n = 0; n < VD / 8; ++n) {
            const int col = n * 8 + 2 * tq;
            float v0 = o[n][2 * r] * inv * head_gate, v1 = o[n][2 * r + 1] * inv * head_gate;
            if (gt && !p.gate_heads) {
                v0 *= 1.0f / (1.0f + expf(-__bfloat162float(gt[col])));
                v1 *= 1.0f / (1.0f + expf(-__bfloat162float(gt[col + 1])));
            }
            *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(v0, v1);
        }
    }
}

template <int HD, int VD>
int launch(const Params& p, dim3 grid, cudaStream_t s) {
    const size_t smem = ((size_t)(BM + 2 * BN) * (HD + 8) + (size_t)2 * BN * (VD + 8)) * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("attention_mma: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    LLMK_CHECK_LAUNCH_RC("attention_mma", llmk_launch(attention_mma_kernel<HD, VD>, grid, dim3(WARPS * 32), smem, s, true, p));
    return LLMK_OK;
}

}  // namespace

// Queries per tile (0: the kernel does not take these sizes).
LLMK_EXPORT int llmk_attention_mma_tile_queries(int nq, int nkv, int hd, int vd) {
    if (nkv <= 0 || nq <= 0 || nq % nkv != 0) return 0;
    if ((hd != 64 && hd != 128) || (vd != 64 && vd != 128)) return 0;
    return BM;
}

// out[t, nq*vd] (bfloat16) = attention of q[t] (bfloat16) over the paged cache [pages, nkv, page_size, hd | vd].
// tile_seq / tile_q0 list tiles of 64 queries; an entry with sequence -1 is skipped.
LLMK_EXPORT int llmk_attention_mma(void* out, long long o_stride, const void* q, long long q_stride, const void* kcache,
                                   const void* vcache, const int* block_tables, int max_blocks, const int* ctx_len, const int* cu_q,
                                   const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv, int hd, int vd,
                                   int page_size, int window, float scale, float softcap, int sink, const float* sink_values, const void* gate,
                                   long long gate_stride, int chunk, int gate_heads, const float* turn_cos, const float* turn_sin,
                                   void* stream) {
    if (n_tiles <= 0) return LLMK_OK;
    if (llmk_attention_mma_tile_queries(nq, nkv, hd, vd) == 0)
        LLMK_FAIL("attention_mma: not taken (heads %d/%d, key width %d and value width %d must be 64 or 128)", nq, nkv, hd, vd);
    if (q_stride % 8 != 0 || o_stride % 2 != 0 || !host_aligned16(q) || !host_aligned16(kcache) || !host_aligned16(vcache) ||
        (reinterpret_cast<uintptr_t>(out) & 3) != 0 || page_size <= 0)
        LLMK_FAIL("attention_mma: q and the cache must start on 16-byte boundaries, q's row stride a multiple of 8");
    if (nq > 65535) LLMK_FAIL("attention_mma: grid too large");
    Params p;
    p.q = (const bf16*)q; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache; p.out = (bf16*)out;
    p.gate = (const bf16*)gate; p.sink_values = sink_values; p.gate_heads = gate_heads ? 1 : 0;
    p.turn_cos = (turn_cos && turn_sin) ? turn_cos : nullptr; p.turn_sin = turn_sin; p.block_tables = block_tables; p.ctx_len = ctx_len; p.cu_q = cu_q;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.q_stride = q_stride; p.o_stride = o_stride; p.gate_stride = gate_stride;
    p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window; p.sink = sink ? 1 : 0; p.chunk = chunk > 0 ? chunk : 0;
    p.scale = scale; p.softcap = softcap;
    dim3 grid(n_tiles, nq);
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64 && vd == 64) return launch<64, 64>(p, grid, s);
    if (hd == 64) return launch<64, 128>(p, grid, s);
    if (vd == 64) return launch<128, 64>(p, grid, s);
    return launch<128, 128>(p, grid, s);
}
