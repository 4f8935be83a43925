// A routed feed-forward (mixture of experts) without a trip to the host, so that a step holding one can be
// recorded into a CUDA graph: every launch has a shape that follows from (tokens, experts, top) alone.
//
//   moe_route     per token: z = Wr h (+ b) (float32), s = sigmoid(z) or softmax(z), the `top` largest s choose experts;
//                 slot t * top + c holds (expert, weight); or the `top` largest z choose and the weights are the softmax
//                 over the chosen z alone
//   moe_plan      one block: slots grouped by expert, cut into tiles of TT rows of one expert each; the list of tiles
//                 has a fixed length (slots / TT + experts), padded with expert -1
//   moe_experts   grid (tiles, column blocks): first product of a tile's rows with its expert's matrices and the
//                 gated activation, or the second product (down); float32 sums on the CUDA cores (the float32 path, and
//                 operands the tensor-core product refuses)
//   moe_gather    for the tensor-core path: the rows (times their weights) sorted by expert into tiles of 128, every
//                 expert's rows starting on a tile; the grouped product of csrc/gemm_tc.cu then takes the list of the
//                 tiles' experts from the device
//   moe_combine   per token: shared expert's output (if any) + its slots' outputs in slot order
//
// The weight multiplies the expert's input (mode "input") or its output (mode "output").
// Gated activation: g' = min(g, L), u' = clamp(u, -L, L), y = g' sigmoid(alpha g') (u' + 1)   (L <= 0: no clamp),
// or the plain gated unit y = g sigmoid(g) u.
#define LLMK_MODULE_NAME "moe"
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int MOE_TT = 16;      // rows per tile
constexpr int MOE_KC = 256;     // input values per pass through shared memory

// ---------------------------------------------------------------------------------------------- route
// One block per token: the warps share the experts (a warp per dot product, float32 sums in a fixed order), warp 0 then
// scores and picks.  scoring 0: sigmoid, 1: softmax over all experts, 2: the logits themselves choose, and the weights
// are the softmax over the chosen logits.
template <typename T>
__global__ void __launch_bounds__(256) moe_route_kernel(const T* __restrict__ h, long long ldh, const float* __restrict__ wr,
                                                        const float* __restrict__ bias, int* __restrict__ slot_expert,
                                                        float* __restrict__ slot_weight, int K, int E, int top, int scoring,
                                                        int renorm) {
    extern __shared__ float sm[];   // [K] the row in float32, [E] scores
    float* xs = sm;
    float* s = sm + K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const size_t t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const T* x = h + t * ldh;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float(x[k]);
    __syncthreads();
    const bool vec = (K & 3) == 0;
    for (int e = warp; e < E; e += nwarps) {
        const float* w = wr + (size_t)e * K;
        float acc = 0.f;
        if (vec) {
            for (int k = lane * 4; k < K; k += 128) {
                const float4 a = *reinterpret_cast<const float4*>(xs + k);
                const float4 b = __ldg(reinterpret_cast<const float4*>(w + k));
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], w[k], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) s[e] = acc + (bias ? bias[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    if (scoring == 2) {
        // the logits choose
    } else if (scoring == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(s[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) s[e] = expf(s[e] - mx) / sum;
    } else {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
    }
    __syncwarp();
    float total = 0.f;
    for (int c = 0; c < top; ++c) {
        // the largest remaining score; ties and values that compare with nothing (NaN) go to the smallest index
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = s[e];
            if (v > best) { best = v; arg = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= E) { arg = c < E ? c : 0; best = 0.f; }     // nothing comparable was left: a padded row's garbage
        total += best;
        if (lane == 0) {
            slot_expert[t * top + c] = arg;
            slot_weight[t * top + c] = best;
            s[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (scoring == 2) {
        // softmax over the chosen logits; the first chosen is the largest
        if (lane == 0) {
            const float mx = slot_weight[t * top];
            float sum = 0.f;
            for (int c = 0; c < top; ++c) sum += expf(slot_weight[t * top + c] - mx);
            for (int c = 0; c < top; ++c) slot_weight[t * top + c] = expf(slot_weight[t * top + c] - mx) / sum;
        }
        return;
    }
    if (renorm && lane == 0)
        for (int c = 0; c < top; ++c) slot_weight[t * top + c] /= total;
}

LLMK_EXPORT int llmk_moe_route(const void* h, long long ldh, const float* wr, const float* bias, int* slot_expert, float* slot_weight,
                               int n_tokens, int K, int E, int top, int scoring, int renorm, int dtype, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    if (E <= 0 || top <= 0 || top > E || K <= 0) LLMK_FAIL("moe_route: bad sizes (experts %d, top %d, width %d)", E, top, K);
    if (scoring < 0 || scoring > 2) LLMK_FAIL("moe_route: unknown scoring %d", scoring);
    const size_t smem = ((size_t)K + E) * sizeof(float);
    if (smem > 200 * 1024) LLMK_FAIL("moe_route: a row of %d values and %d experts do not fit shared memory", K, E);
    const int threads = E >= 8 ? 256 : 32 * E;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(moe_route_kernel<float>, dim3(n_tokens), dim3(threads), smem, s, true, (const float*)h, ldh, wr, bias, slot_expert,
                        slot_weight, K, E, top, scoring, renorm);
    } else if (dtype == LLMK_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(moe_route_kernel<bf16>, dim3(n_tokens), dim3(threads), smem, s, true, (const bf16*)h, ldh, wr, bias, slot_expert,
                        slot_weight, K, E, top, scoring, renorm);
    } else
        LLMK_FAIL("moe_route: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("moe_route", e);
    return LLMK_OK;
}

// ----------------------------------------------------------------------------------------------- plan
// order[pos] = slot, pos_of_slot[slot] = pos, slots of one expert side by side (in no particular order: every row
// is computed by itself).  tile_expert[i], tile_start[i], tile_rows[i] for i < max_tiles; expert -1 pads.
// `padded`: every expert's rows begin on a multiple of `tt` (whole tiles per expert, for the grouped tensor-core product);
// order[pos] is then -1 where a tile has no row.
__global__ void moe_plan_kernel(const int* __restrict__ slot_expert, int n_slots, int E, int max_tiles, int tt, int padded,
                                int* __restrict__ order, int* __restrict__ pos_of_slot, int* __restrict__ tile_expert,
                                int* __restrict__ tile_start, int* __restrict__ tile_rows) {
    extern __shared__ int sh[];     // counts [E], offsets [E], cursors [E]
    int* count = sh;
    int* offset = sh + E;
    int* cursor = sh + 2 * E;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int e = slot_expert[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            offset[e] = at;
            cursor[e] = at;
            for (int r = 0; r < count[e] && tile < max_tiles; r += tt, ++tile) {
                tile_expert[tile] = e;
                tile_start[tile] = at + r;
                tile_rows[tile] = min(tt, count[e] - r);
            }
            at += padded ? ceil_div(count[e], tt) * tt : count[e];
        }
        for (; tile < max_tiles; ++tile) {
            tile_expert[tile] = -1;
            tile_start[tile] = 0;
            tile_rows[tile] = 0;
        }
    }
    if (padded)
        for (int i = threadIdx.x; i < max_tiles * tt; i += blockDim.x) order[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int e = slot_expert[i];
        if (e >= 0 && e < E) {
            const int pos = atomicAdd(&cursor[e], 1);
            order[pos] = i;
            pos_of_slot[i] = pos;
        } else {
            pos_of_slot[i] = -1;
        }
    }
}

// The most tiles of `tile` rows (0: this module's own 16) that `n_slots` rows in `E` groups can need.
LLMK_EXPORT int llmk_moe_max_tiles(int n_slots, int E, int tile) {
    const int tt = tile > 0 ? tile : MOE_TT;
    // a group's last tile is partial: at most min(E, n_slots) of them
    return n_slots / tt + (E < n_slots ? E : n_slots);
}

// tile: rows per tile (0: 16, what `moe_experts` takes); padded != 0: experts' rows start on tile boundaries and `order`
// has max_tiles * tile entries.
LLMK_EXPORT int llmk_moe_plan(const int* slot_expert, int n_slots, int E, int tile, int padded, int* order, int* pos_of_slot,
                              int* tile_expert, int* tile_start, int* tile_rows, void* stream) {
    if (n_slots <= 0) return LLMK_OK;
    const int tt = tile > 0 ? tile : MOE_TT;
    const size_t smem = (size_t)3 * E * sizeof(int);
    if (smem > 48 * 1024) LLMK_FAIL("moe_plan: %d experts are too many", E);
    LLMK_CHECK_LAUNCH_RC("moe_plan", llmk_launch(moe_plan_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, true, slot_expert, n_slots, E,
                                                 llmk_moe_max_tiles(n_slots, E, tile), tt, padded, order, pos_of_slot, tile_expert, tile_start,
                                                 tile_rows));
    return LLMK_OK;
}

// --------------------------------------------------------------------------------------------- gather
// xs[pos, :] = (T)(weight * h[token of order[pos], :]) for the rows a padded plan filled; rows of padding are zeroed.
template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ xs, const T* __restrict__ h, long long ldh, const int* __restrict__ order,
                                  const float* __restrict__ slot_weight, int top, int K, int scale_rows) {
    const size_t pos = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int slot = order[pos];
    T* dst = xs + pos * K;
    if (slot < 0) {
        for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_float<T>(0.f);
        return;
    }
    const float w = scale_rows ? slot_weight[slot] : 1.f;
    const T* src = h + (size_t)(slot / top) * ldh;
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_float<T>(to_float(src[k]) * w);
}

LLMK_EXPORT int llmk_moe_gather(void* xs, const void* h, long long ldh, const int* order, const float* slot_weight, int n_rows, int top,
                                int K, int scale_rows, int dtype, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(moe_gather_kernel<float>, dim3(n_rows), dim3(128), 0, s, true, (float*)xs, (const float*)h, ldh, order, slot_weight, top, K, scale_rows);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(moe_gather_kernel<bf16>, dim3(n_rows), dim3(128), 0, s, true, (bf16*)xs, (const bf16*)h, ldh, order, slot_weight, top, K, scale_rows);
    else
        LLMK_FAIL("moe_gather: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("moe_gather", e);
    return LLMK_OK;
}

// -------------------------------------------------------------------------------------------- experts
// Block (tile, block of 128 output columns); a thread per output column keeps the sums of the tile's rows.
// FIRST: x = weight * h[token] (or h[token]), K = width, N = ff; y[pos, f] = act(x . Wgate[e, f], x . Wup[e, f])   float32
// else:  x = y[pos], K = ff, N = width; out[pos, c] = (x . Wdown[e, c]) (* weight)                                  float32
template <typename T, bool FIRST>
__global__ void __launch_bounds__(128) moe_experts_kernel(float* __restrict__ out, const void* __restrict__ in, long long ld_in,
                                                          const T* __restrict__ w0, const T* __restrict__ w1,
                                                          const int* __restrict__ order, const float* __restrict__ slot_weight,
                                                          const int* __restrict__ tile_expert, const int* __restrict__ tile_start,
                                                          const int* __restrict__ tile_rows, int top, int K, int N, int scale_rows,
                                                          float alpha, float limit, int plain) {
    __shared__ float xs[MOE_TT][MOE_KC];
    __shared__ int src_row[MOE_TT];
    __shared__ float row_w[MOE_TT];
    pdl_launch_dependents();
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int start = tile_start[blockIdx.x], n = tile_rows[blockIdx.x];
    const int col = blockIdx.y * blockDim.x + threadIdx.x;
    if (threadIdx.x < MOE_TT) {
        const int i = threadIdx.x;
        const int slot = i < n ? order[start + i] : -1;
        src_row[i] = slot < 0 ? -1 : (FIRST ? slot / top : start + i);
        row_w[i] = (slot >= 0 && scale_rows) ? slot_weight[slot] : 1.f;
    }
    __syncthreads();
    const T* wa = w0 + ((size_t)e * N + (col < N ? col : 0)) * K;
    const T* wb = FIRST ? w1 + ((size_t)e * N + (col < N ? col : 0)) * K : nullptr;
    float acc0[MOE_TT], acc1[FIRST ? MOE_TT : 1];
#pragma unroll
    for (int i = 0; i < MOE_TT; ++i) acc0[i] = 0.f;
    if (FIRST) {
#pragma unroll
        for (int i = 0; i < MOE_TT; ++i) acc1[i] = 0.f;
    }
    for (int k0 = 0; k0 < K; k0 += MOE_KC) {
        const int kc = min(MOE_KC, K - k0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < MOE_TT * MOE_KC; idx += blockDim.x) {
            const int i = idx / MOE_KC, k = idx % MOE_KC;
            float v = 0.f;
            if (src_row[i] >= 0 && k < kc) {
                if (FIRST)
                    v = to_float(static_cast<const T*>(in)[(size_t)src_row[i] * ld_in + k0 + k]) * row_w[i];
                else
                    v = static_cast<const float*>(in)[(size_t)src_row[i] * ld_in + k0 + k];
            }
            xs[i][k] = v;
        }
        __syncthreads();
        if (col < N) {
            for (int k = 0; k < kc; ++k) {
                const float a = to_float(wa[k0 + k]);
#pragma unroll
                for (int i = 0; i < MOE_TT; ++i) acc0[i] = fmaf(xs[i][k], a, acc0[i]);
                if (FIRST) {
                    const float b = to_float(wb[k0 + k]);
#pragma unroll
                    for (int i = 0; i < MOE_TT; ++i) acc1[i] = fmaf(xs[i][k], b, acc1[i]);
                }
            }
        }
    }
    if (col >= N) return;
#pragma unroll
    for (int i = 0; i < MOE_TT; ++i) {
        if (i >= n) continue;
        float v;
        if (FIRST) {
            float g = acc0[i], u = acc1[i];
            if (plain) {
                v = g / (1.0f + expf(-g)) * u;
            } else {
                if (limit > 0.f) {
                    g = fminf(g, limit);
                    u = fminf(fmaxf(u, -limit), limit);
                }
                v = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
            }
        } else {
            v = acc0[i] * row_w[i];
        }
        out[(size_t)(start + i) * N + col] = v;
    }
}

// plain != 0: the gated unit is silu(g) u (alpha and limit unused).
// first != 0: in = h [tokens, width] of the storage dtype, w0 / w1 = gate / up [E, ff, width], out = y [slots, ff]; the rows
//             are multiplied by their weights when weight_on_input.
// first == 0: in = y [slots, ff] float32, w0 = down [E, width, ff], out [slots, width]; multiplied by the weights
//             when !weight_on_input.
LLMK_EXPORT int llmk_moe_experts(float* out, const void* in, long long ld_in, const void* w0, const void* w1, const int* order,
                                 const float* slot_weight, const int* tile_expert, const int* tile_start, const int* tile_rows,
                                 int n_slots, int E, int top, int K, int N, int first, int weight_on_input, float alpha, float limit,
                                 int plain, int dtype, void* stream) {
    if (n_slots <= 0) return LLMK_OK;
    dim3 grid(llmk_moe_max_tiles(n_slots, E, 0), ceil_div(N, 128));
    cudaStream_t s = (cudaStream_t)stream;
    const int scale_rows = first ? (weight_on_input ? 1 : 0) : (weight_on_input ? 0 : 1);
    cudaError_t e;
    if (dtype == LLMK_F32) {
        if (first)
            e = llmk_launch(moe_experts_kernel<float, true>, grid, dim3(128), 0, s, true, out, in, ld_in, (const float*)w0, (const float*)w1, order,
                            slot_weight, tile_expert, tile_start, tile_rows, top, K, N, scale_rows, alpha, limit, plain);
        else
            e = llmk_launch(moe_experts_kernel<float, false>, grid, dim3(128), 0, s, true, out, in, ld_in, (const float*)w0, (const float*)w1, order,
                            slot_weight, tile_expert, tile_start, tile_rows, top, K, N, scale_rows, alpha, limit, plain);
    } else if (dtype == LLMK_BF16) {
        if (first)
            e = llmk_launch(moe_experts_kernel<bf16, true>, grid, dim3(128), 0, s, true, out, in, ld_in, (const bf16*)w0, (const bf16*)w1, order,
                            slot_weight, tile_expert, tile_start, tile_rows, top, K, N, scale_rows, alpha, limit, plain);
        else
            e = llmk_launch(moe_experts_kernel<bf16, false>, grid, dim3(128), 0, s, true, out, in, ld_in, (const bf16*)w0, (const bf16*)w1, order,
                            slot_weight, tile_expert, tile_start, tile_rows, top, K, N, scale_rows, alpha, limit, plain);
    } else
        LLMK_FAIL("moe_experts: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("moe_experts", e);
    return LLMK_OK;
}

// -------------------------------------------------------------------------------------------- combine
// out[t, c] (float32) = (shared ? shared[t, c] : 0) + sum over the token's slots, in slot order, of rows[pos_of_slot, c]
// (times the slot's weight where `slot_weight` is given: the weight on an expert's output).
template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ out, const float* __restrict__ rows, const int* __restrict__ pos_of_slot,
                                   const T* __restrict__ shared_out, const float* __restrict__ slot_weight, int n_tokens, int top,
                                   int H) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)n_tokens * H;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t t = (size_t)(i / H);
        const int c = (int)(i % H);
        float v = shared_out ? to_float(shared_out[i]) : 0.f;
        for (int k = 0; k < top; ++k) {
            const int pos = pos_of_slot[t * top + k];
            if (pos >= 0) v += slot_weight ? slot_weight[t * top + k] * rows[(size_t)pos * H + c] : rows[(size_t)pos * H + c];
        }
        out[i] = v;
    }
}

LLMK_EXPORT int llmk_moe_combine(float* out, const float* rows, const int* pos_of_slot, const void* shared_out, const float* slot_weight,
                                 int n_tokens, int top, int H, int dtype, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    long long blocks = ((long long)n_tokens * H + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(moe_combine_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, out, rows, pos_of_slot, (const float*)shared_out,
                        slot_weight, n_tokens, top, H);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(moe_combine_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, out, rows, pos_of_slot, (const bf16*)shared_out,
                        slot_weight, n_tokens, top, H);
    else
        LLMK_FAIL("moe_combine: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("moe_combine", e);
    return LLMK_OK;
}
