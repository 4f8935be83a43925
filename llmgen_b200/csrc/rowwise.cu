// Row-wise kernels of layers that normalise a sublayer's OUTPUT before it joins the residual stream
// (x <- x + norm(sublayer(x))), and of the sublayers such layers are made of:
//
//   norm_add        resid[r, :] += rmsnorm(y[r, :]) * w, and a copy of the new residual row in the storage dtype
//                   for the products that read the residual itself; y may be a weighted sum of two products
//                   (a y + b y2), and the copy may be the next sublayer's normed input, rmsnorm(resid) * w_next,
//                   for layers that norm a sublayer's input as well as its output
//   scaled_sum      out (float32) = a y + b y2, for consumers that take one array
//   cast_rows       out = (T) in, float32 in
//   act_rows        relu(x)^2, tanh(x), gelu_tanh(x), the clamped gated unit  g' s(alpha g') (u' + 1)  with g' = min(g, L), u' = clamp(u, -L, L),
//                   or the gated units gelu_tanh(g) u and silu(g) u
//   gated_rmsnorm   out[r, :] = rmsnorm(o[r, :]) * w * sigmoid(g[r, :])   (or, without gains, o * sigmoid(g)); the gate may
//                   pass silu instead, or enter as it is; the gains may differ between `w_rows` consecutive rows (heads)
//   add_bias        y[r, :] += b, y an array of T or of float32, or the float32 slices of a product (the first slice takes it)
//   concat_stream   out[r, :] = [ (T)(resid[r, :] + delta[r, :]) | (T) x0[r, :] ]: the operand of a product that mixes the
//                   residual stream with the embedding's output
//   stream_step     layers that keep several residual streams x_1 .. x_S per token (hyper-connections): one kernel ends a
//                   sublayer, x_t <- sum_s mix[s, t] x_s + out[t] y, and begins the next, rmsnorm(sum_t in[t] x_t) * w
//   stream_spread / stream_collapse   every stream = one row; one row = the sum of the streams
//
// Sums of squares, gains, the residual and the activations' arithmetic are float32 in both storage dtypes.
#define LLMK_MODULE_NAME "rowwise"
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

// y is a [n, H] array of T (splits == 0), or `splits` float32 slices `split_stride` floats apart, added in slice order.
template <typename T>
__device__ __forceinline__ float load_sum(const void* y, size_t at, int splits, long long split_stride) {
    if (splits == 0) return to_float(static_cast<const T*>(y)[at]);
    const float* p = static_cast<const float*>(y) + at;
    float acc = p[0];
    for (int s = 1; s < splits; ++s) acc += p[(size_t)s * split_stride];
    return acc;
}

template <typename T>
__global__ void norm_add_kernel(float* __restrict__ resid, const void* __restrict__ y, const float* __restrict__ w,
                                T* __restrict__ copy, int H, float eps, int splits, long long split_stride,
                                const void* __restrict__ y2, int splits2, long long split_stride2, float a, float b,
                                const float* __restrict__ w_next, float eps_next) {
    extern __shared__ float srow[];  // H floats + 33 scratch
    float* scratch = srow + H;
    const size_t r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = load_sum<T>(y, r * H + i, splits, split_stride);
        if (y2) v = a * v + b * load_sum<T>(y2, r * H + i, splits2, split_stride2);
        srow[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    if (!w_next) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = resid[r * H + i] + srow[i] * rinv * w[i];
            resid[r * H + i] = v;
            if (copy) copy[r * H + i] = from_float<T>(v);
        }
        return;
    }
    // the copy is the next sublayer's input: the new row normed once more, with the next norm's gains
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = resid[r * H + i] + srow[i] * rinv * w[i];
        resid[r * H + i] = v;
        srow[i] = v;
        ss2 += v * v;
    }
    ss2 = block_sum(ss2, scratch);
    const float rinv2 = 1.0f / sqrtf(ss2 / (float)H + eps_next);
    for (int i = threadIdx.x; i < H; i += blockDim.x) copy[r * H + i] = from_float<T>(srow[i] * rinv2 * w_next[i]);
}

// y2 (with its own slices) null: resid += rmsnorm(y) w.  Else resid += rmsnorm(a y + b y2) w.  w_next non-null: `copy`
// receives rmsnorm(new row) * w_next (eps_next inside the root) instead of the new row.
LLMK_EXPORT int llmk_norm_add2(float* resid, const void* y, const float* w, void* copy, int n_rows, int H, float eps,
                               int splits, long long split_stride, const void* y2, int splits2, long long split_stride2,
                               float a, float b, const float* w_next, float eps_next, int dtype, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (H <= 0 || !y || !w || !resid) LLMK_FAIL("norm_add: bad arguments (H %d)", H);
    if (w_next && !copy) LLMK_FAIL("norm_add: the next norm's output needs a place");
    const size_t smem = ((size_t)H + 33) * sizeof(float);
    if (smem > 200 * 1024) LLMK_FAIL("norm_add: a row of %d values does not fit shared memory", H);
    const int threads = H >= 2048 ? 512 : H >= 512 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(norm_add_kernel<float>, dim3(n_rows), dim3(threads), smem, s, true, resid, y, w, (float*)copy, H, eps, splits, split_stride,
                        y2, splits2, split_stride2, a, b, w_next, eps_next);
    } else if (dtype == LLMK_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = llmk_launch(norm_add_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, true, resid, y, w, (bf16*)copy, H, eps, splits, split_stride,
                        y2, splits2, split_stride2, a, b, w_next, eps_next);
    } else
        LLMK_FAIL("norm_add: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("norm_add", e);
    return LLMK_OK;
}

LLMK_EXPORT int llmk_norm_add(float* resid, const void* y, const float* w, void* copy, int n_rows, int H, float eps,
                              int splits, long long split_stride, int dtype, void* stream) {
    return llmk_norm_add2(resid, y, w, copy, n_rows, H, eps, splits, split_stride, nullptr, 0, 0, 1.f, 0.f, nullptr, 0.f, dtype, stream);
}

// out[i] (float32) = a * y[i] + b * y2[i]; y and y2 arrays of T or float32 slices.
template <typename T>
__global__ void scaled_sum_kernel(float* __restrict__ out, const void* __restrict__ y, int splits, long long split_stride,
                                  const void* __restrict__ y2, int splits2, long long split_stride2, float a, float b, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = a * load_sum<T>(y, (size_t)i, splits, split_stride) + b * load_sum<T>(y2, (size_t)i, splits2, split_stride2);
}

LLMK_EXPORT int llmk_scaled_sum(float* out, const void* y, int splits, long long split_stride, const void* y2, int splits2,
                                long long split_stride2, float a, float b, long long n, int dtype, void* stream) {
    if (n <= 0) return LLMK_OK;
    if (!out || !y || !y2) LLMK_FAIL("scaled_sum: bad arguments");
    long long blocks = (n + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(scaled_sum_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, out, y, splits, split_stride, y2, splits2, split_stride2, a, b, n);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(scaled_sum_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, out, y, splits, split_stride, y2, splits2, split_stride2, a, b, n);
    else
        LLMK_FAIL("scaled_sum: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("scaled_sum", e);
    return LLMK_OK;
}

template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ in, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_float<T>(in[i]);
}

LLMK_EXPORT int llmk_cast_rows(void* out, const float* in, long long n, int dtype, void* stream) {
    if (n <= 0) return LLMK_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(cast_rows_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, (float*)out, in, n);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(cast_rows_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, (bf16*)out, in, n);
    else
        LLMK_FAIL("cast_rows: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("cast_rows", e);
    return LLMK_OK;
}

// mode 0: out[r, f] = relu(x[r, f])^2, x [n, F]
// mode 1: x [n, 2F], gate in columns [0, F), up in [F, 2F):
//         g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1)
// mode 2: x [n, 2F] as in mode 1: out = gelu_tanh(gate) * up, gelu_tanh(z) = z / 2 (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
// mode 3: out[r, f] = tanh(x[r, f]), x [n, F]
// mode 4: x [n, 2F] as in mode 2 (groups too): out = silu(gate) * up
// mode 5: out[r, f] = gelu_tanh(x[r, f]), x [n, F]
enum { ACT_RELU2 = 0, ACT_CLAMPED_GLU = 1, ACT_GELU_TANH_GLU = 2, ACT_TANH = 3, ACT_SILU_GLU = 4, ACT_GELU_TANH = 5 };

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void act_rows_kernel(T* __restrict__ out, const void* __restrict__ x, int n, int F, long long ld, int mode,
                                float alpha, float limit, int splits, long long split_stride, int group) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)n * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t r = (size_t)(i / F);
        const int f = (int)(i % F);
        float v;
        if (mode == ACT_RELU2) {
            const float a = fmaxf(load_sum<T>(x, r * ld + f, splits, split_stride), 0.f);
            v = a * a;
        } else if (mode == ACT_TANH) {
            v = tanhf(load_sum<T>(x, r * ld + f, splits, split_stride));
        } else if (mode == ACT_GELU_TANH) {
            v = gelu_tanh(load_sum<T>(x, r * ld + f, splits, split_stride));
        } else if (mode == ACT_GELU_TANH_GLU || mode == ACT_SILU_GLU) {
            // gate and up alternate in groups of `group` columns (group = F: all gates, then all ups)
            const size_t gc = r * ld + (size_t)(f / group) * 2 * group + f % group;
            const float g = load_sum<T>(x, gc, splits, split_stride);
            v = (mode == ACT_SILU_GLU ? g / (1.0f + expf(-g)) : gelu_tanh(g)) * load_sum<T>(x, gc + group, splits, split_stride);
        } else {
            const float g = fminf(load_sum<T>(x, r * ld + f, splits, split_stride), limit);
            const float u = fminf(fmaxf(load_sum<T>(x, r * ld + F + f, splits, split_stride), -limit), limit);
            v = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
        }
        out[i] = from_float<T>(v);
    }
}

// The gated forms over whole 16-byte vectors: a thread takes one vector of gates, the vector of ups beside it, and writes
// one vector (rows that are no partial sums, column counts and strides in whole vectors).  The arithmetic is the scalar
// kernel's.
template <typename T>
__global__ void __launch_bounds__(256) act_rows_vec_kernel(T* __restrict__ out, const T* __restrict__ x, int n, int F, long long ld,
                                                           int mode, float alpha, float limit, int group) {
    constexpr int N = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int vecs = F / N;
    const long long total = (long long)n * vecs;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t r = (size_t)(i / vecs);
        const int f = (int)(i % vecs) * N;
        size_t gc, uc;
        if (mode == ACT_CLAMPED_GLU) {
            gc = r * ld + f;
            uc = gc + F;
        } else {
            gc = r * ld + (size_t)(f / group) * 2 * group + f % group;
            uc = gc + group;
        }
        Vec16<T> gv, uv, y;
        gv.raw = *reinterpret_cast<const decltype(gv.raw)*>(x + gc);
        uv.raw = *reinterpret_cast<const decltype(uv.raw)*>(x + uc);
        float g[N], u[N], v[N];
        gv.unpack(g);
        uv.unpack(u);
#pragma unroll
        for (int k = 0; k < N; ++k) {
            if (mode == ACT_CLAMPED_GLU) {
                const float gg = fminf(g[k], limit), uu = fminf(fmaxf(u[k], -limit), limit);
                v[k] = gg / (1.0f + expf(-alpha * gg)) * (uu + 1.0f);
            } else {
                v[k] = (mode == ACT_SILU_GLU ? g[k] / (1.0f + expf(-g[k])) : gelu_tanh(g[k])) * u[k];
            }
        }
        y.pack(v);
        *reinterpret_cast<decltype(y.raw)*>(out + (size_t)r * F + f) = y.raw;
    }
}

template <typename T>
static bool act_rows_vec_ok(const void* out, const void* x, int F, long long ld, int mode, int splits, int group) {
    constexpr int N = 16 / (int)sizeof(T);
    const bool gated = mode == ACT_CLAMPED_GLU || mode == ACT_SILU_GLU || mode == ACT_GELU_TANH_GLU;
    return gated && splits == 0 && F % N == 0 && group % N == 0 && ld % N == 0 && host_aligned16(out) && host_aligned16(x);
}

LLMK_EXPORT int llmk_act_rows(void* out, const void* x, int n, int F, long long ld, int mode, float alpha, float limit,
                              int splits, long long split_stride, int group, int dtype, void* stream) {
    if (n <= 0 || F <= 0) return LLMK_OK;
    if (group <= 0) group = F;
    if (F % group != 0) LLMK_FAIL("act_rows: groups of %d columns do not divide %d", group, F);
    if (mode < ACT_RELU2 || mode > ACT_GELU_TANH) LLMK_FAIL("act_rows: unknown activation %d", mode);
    long long blocks = ((long long)n * F + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if ((dtype == LLMK_BF16 && act_rows_vec_ok<bf16>(out, x, F, ld, mode, splits, group)) ||
        (dtype == LLMK_F32 && act_rows_vec_ok<float>(out, x, F, ld, mode, splits, group))) {
        const int N = dtype == LLMK_BF16 ? 8 : 4;
        long long vblocks = ((long long)n * (F / N) + 255) / 256;
        if (vblocks > device_sm_count() * 16) vblocks = device_sm_count() * 16;
        if (dtype == LLMK_BF16)
            e = llmk_launch(act_rows_vec_kernel<bf16>, dim3((unsigned)vblocks), dim3(256), 0, s, true, (bf16*)out, (const bf16*)x, n, F, ld, mode, alpha, limit, group);
        else
            e = llmk_launch(act_rows_vec_kernel<float>, dim3((unsigned)vblocks), dim3(256), 0, s, true, (float*)out, (const float*)x, n, F, ld, mode, alpha, limit, group);
        LLMK_CHECK_LAUNCH_RC("act_rows", e);
        return LLMK_OK;
    }
    if (dtype == LLMK_F32)
        e = llmk_launch(act_rows_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, (float*)out, x, n, F, ld, mode, alpha, limit, splits, split_stride, group);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(act_rows_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, (bf16*)out, x, n, F, ld, mode, alpha, limit, splits, split_stride, group);
    else
        LLMK_FAIL("act_rows: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("act_rows", e);
    return LLMK_OK;
}

// out[r, i] = o[r, i] * (w ? rsqrt(mean(o[r, :]^2) + eps) * w[i] : 1) * gate(g[r, i]); o float32 [n, H], g of T with rows `ldg`
// apart.  gate_act 0: sigmoid(g); 1: silu(g); 2: g as it is.  heads > 1: a row is one head of a token, r = token * heads +
// head; the gate's rows are tokens ([n / heads, heads * H], `ldg` apart), and with w_rows = heads every head has gains of
// its own, w [heads, H] (w_rows = 1: one vector for all).
enum { GATE_SIGMOID = 0, GATE_SILU = 1, GATE_PLAIN = 2 };
template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ g,
                                     const float* __restrict__ w, int H, long long ldg, float eps, int gate_act, int w_rows,
                                     int heads) {
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    float rinv = 1.f;
    if (w) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = o[r * H + i];
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        rinv = 1.0f / sqrtf(ss / (float)H + eps);
    }
    const size_t head = r % (size_t)heads;
    const float* wr = w ? w + (head % (size_t)w_rows) * H : nullptr;
    const T* gr = g + (r / (size_t)heads) * ldg + head * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float gv = to_float(gr[i]);
        const float sg = 1.0f / (1.0f + expf(-gv));
        const float gate = gate_act == GATE_SIGMOID ? sg : gate_act == GATE_SILU ? gv * sg : gv;
        out[r * H + i] = from_float<T>(o[r * H + i] * rinv * (wr ? wr[i] : 1.f) * gate);
    }
}

// The same for short rows (a head's values): a warp a row, eight rows a block, no block-wide sum.
template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_warp_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ g,
                                                                 const float* __restrict__ w, int n_rows, int H, long long ldg, float eps,
                                                                 int gate_act, int w_rows, int heads) {
    const size_t r = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (r >= (size_t)n_rows) return;
    float rinv = 1.f;
    if (w) {
        float ss = 0.f;
        for (int i = lane; i < H; i += 32) {
            const float v = o[r * H + i];
            ss += v * v;
        }
        ss = warp_sum(ss);
        rinv = 1.0f / sqrtf(ss / (float)H + eps);
    }
    const size_t head = r % (size_t)heads;
    const float* wr = w ? w + (head % (size_t)w_rows) * H : nullptr;
    const T* gr = g + (r / (size_t)heads) * ldg + head * H;
    for (int i = lane; i < H; i += 32) {
        const float gv = to_float(gr[i]);
        const float sg = 1.0f / (1.0f + expf(-gv));
        const float gate = gate_act == GATE_SIGMOID ? sg : gate_act == GATE_SILU ? gv * sg : gv;
        out[r * H + i] = from_float<T>(o[r * H + i] * rinv * (wr ? wr[i] : 1.f) * gate);
    }
}

LLMK_EXPORT int llmk_gated_rmsnorm(void* out, const float* o, const void* g, const float* w, int n_rows, int H, long long ldg,
                                   float eps, int gate_act, int w_rows, int heads, int dtype, void* stream) {
    if (n_rows <= 0 || H <= 0) return LLMK_OK;
    if (gate_act < GATE_SIGMOID || gate_act > GATE_PLAIN || heads < 1 || (w_rows != 1 && w_rows != heads))
        LLMK_FAIL("gated_rmsnorm: gate form %d, %d heads a token, %d rows of gains", gate_act, heads, w_rows);
    const int threads = H >= 2048 ? 512 : H >= 512 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (H <= 256 && n_rows >= 64 && (dtype == LLMK_F32 || dtype == LLMK_BF16)) {
        const dim3 grid((unsigned)ceil_div(n_rows, 8));
        if (dtype == LLMK_F32)
            e = llmk_launch(gated_rmsnorm_warp_kernel<float>, grid, dim3(256), 0, s, true, (float*)out, o, (const float*)g, w, n_rows, H, ldg, eps, gate_act, w_rows, heads);
        else
            e = llmk_launch(gated_rmsnorm_warp_kernel<bf16>, grid, dim3(256), 0, s, true, (bf16*)out, o, (const bf16*)g, w, n_rows, H, ldg, eps, gate_act, w_rows, heads);
        LLMK_CHECK_LAUNCH_RC("gated_rmsnorm", e);
        return LLMK_OK;
    }
    if (dtype == LLMK_F32)
        e = llmk_launch(gated_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, true, (float*)out, o, (const float*)g, w, H, ldg, eps, gate_act, w_rows, heads);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(gated_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, true, (bf16*)out, o, (const bf16*)g, w, H, ldg, eps, gate_act, w_rows, heads);
    else
        LLMK_FAIL("gated_rmsnorm: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("gated_rmsnorm", e);
    return LLMK_OK;
}

// y[r, i] += b[i].  y is [n, H] of T (rows `ld` apart), or float32 (dtype of the ARRAY, which may differ from the engine's).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ b, int n, int H, long long ld) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)n * H;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t at = (size_t)(i / H) * ld + (size_t)(i % H);
        y[at] = from_float<T>(to_float(y[at]) + b[i % H]);
    }
}

LLMK_EXPORT int llmk_add_bias(void* y, const float* b, int n, int H, long long ld, int dtype, void* stream) {
    if (n <= 0 || H <= 0) return LLMK_OK;
    if (!y || !b || ld < H) LLMK_FAIL("add_bias: bad arguments (H %d, ld %lld)", H, ld);
    long long blocks = ((long long)n * H + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(add_bias_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, (float*)y, b, n, H, ld);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(add_bias_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, (bf16*)y, b, n, H, ld);
    else
        LLMK_FAIL("add_bias: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("add_bias", e);
    return LLMK_OK;
}

template <typename T>
__global__ void concat_stream_kernel(T* __restrict__ out, const float* __restrict__ resid, const void* __restrict__ delta,
                                     const float* __restrict__ x0, int n, int H, int splits, long long split_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)n * H;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t r = (size_t)(i / H), c = (size_t)(i % H);
        float v = resid[i];
        if (delta) v += load_sum<T>(delta, (size_t)i, splits, split_stride);
        out[r * 2 * H + c] = from_float<T>(v);
        out[r * 2 * H + H + c] = from_float<T>(x0[i]);
    }
}

LLMK_EXPORT int llmk_concat_stream(void* out, const float* resid, const void* delta, const float* x0, int n, int H, int splits,
                                   long long split_stride, int dtype, void* stream) {
    if (n <= 0 || H <= 0) return LLMK_OK;
    if (!out || !resid || !x0) LLMK_FAIL("concat_stream: bad arguments");
    long long blocks = ((long long)n * H + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(concat_stream_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, (float*)out, resid, delta, x0, n, H, splits, split_stride);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(concat_stream_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, (bf16*)out, resid, delta, x0, n, H, splits, split_stride);
    else
        LLMK_FAIL("concat_stream: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("concat_stream", e);
    return LLMK_OK;
}

// ------------------------------------------------------------------------------------------------ several residual streams
// streams [n, S, H] float32.  With y (an array of T, float32 slices, or a y + b y2): every stream is rewritten from all the old
// ones, x_t <- sum_s mix[s * S + t] x_s + out_coef[t] y.  With next_in: normed[r, :] = rmsnorm(sum_t next_in[t] x_t) * next_gain
// (the new streams), the input of the sublayer that follows.  Either half may be absent.  A block per token row.
constexpr int MAX_STREAMS = 16;

// MS: the most streams this instance takes (4, 8 or 16); the loops over streams are unrolled to it, except the outer one of 16.
template <typename T, int MS>
__global__ void __launch_bounds__(512) stream_step_kernel(float* __restrict__ streams, const void* __restrict__ y, int splits, long long split_stride,
                                   const void* __restrict__ y2, int splits2, long long split_stride2, float a, float b,
                                   const float* __restrict__ mix, const float* __restrict__ out_coef,
                                   const float* __restrict__ next_in, const float* __restrict__ next_gain, float eps,
                                   T* __restrict__ normed, int S, int H) {
    extern __shared__ float srow[];  // H floats + 33 scratch + S * S + 2 * S coefficients
    float* scratch = srow + H;
    float* coef = scratch + 33;      // mix [S, S], out [S], in [S]
    const size_t r = blockIdx.x;
    for (int i = threadIdx.x; i < S * S + 2 * S; i += blockDim.x) {
        float c = 0.f;
        if (i < S * S) c = mix ? mix[i] : 0.f;
        else if (i < S * S + S) c = out_coef ? out_coef[i - S * S] : 0.f;
        else c = next_in ? next_in[i - S * S - S] : 0.f;
        coef[i] = c;
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    float* xs = streams + r * S * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x[MS];
#pragma unroll
        for (int s = 0; s < MS; ++s)
            if (s < S) x[s] = xs[(size_t)s * H + i];
        float u = 0.f;
        if (y) {
            float v = load_sum<T>(y, r * H + i, splits, split_stride);
            if (y2) v = a * v + b * load_sum<T>(y2, r * H + i, splits2, split_stride2);
            // every new stream from the old ones (x stays as it was read); the next sublayer's sum is taken on the way
#pragma unroll(MS <= 8 ? MS : 1)
            for (int t = 0; t < MS; ++t) {
                if (t < S) {
                    float acc = coef[S * S + t] * v;
#pragma unroll
                    for (int s = 0; s < MS; ++s)
                        if (s < S) acc = fmaf(coef[s * S + t], x[s], acc);
                    xs[(size_t)t * H + i] = acc;
                    u = fmaf(coef[S * S + S + t], acc, u);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < MS; ++t)
                if (t < S) u = fmaf(coef[S * S + S + t], x[t], u);
        }
        if (next_in) {
            srow[i] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!next_in) return;
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) normed[r * H + i] = from_float<T>(srow[i] * rinv * next_gain[i]);
}

LLMK_EXPORT int llmk_stream_step(float* streams, const void* y, int splits, long long split_stride, const void* y2, int splits2,
                                 long long split_stride2, float a, float b, const float* mix, const float* out_coef,
                                 const float* next_in, const float* next_gain, float eps, void* normed, int n_rows, int S, int H,
                                 int dtype, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (S <= 0 || S > MAX_STREAMS || H <= 0 || !streams) LLMK_FAIL("stream_step: %d streams (at most %d) of %d values", S, MAX_STREAMS, H);
    if (y && (!mix || !out_coef)) LLMK_FAIL("stream_step: a sublayer's output needs the streams' coefficients");
    if (next_in && (!next_gain || !normed)) LLMK_FAIL("stream_step: the next sublayer's input needs gains and a place");
    const size_t smem = ((size_t)H + 33 + S * S + 2 * S) * sizeof(float);
    if (smem > 200 * 1024) LLMK_FAIL("stream_step: a row of %d values does not fit shared memory", H);
    const int threads = H >= 2048 ? 512 : H >= 512 ? 256 : 128;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
#define STREAM_STEP_LAUNCH(TYPE, MS)                                                                                                   \
    do {                                                                                                                               \
        if (smem > 48 * 1024) cudaFuncSetAttribute(stream_step_kernel<TYPE, MS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        e = llmk_launch(stream_step_kernel<TYPE, MS>, dim3(n_rows), dim3(threads), smem, st, true, streams, y, splits, split_stride, y2, \
                        splits2, split_stride2, a, b, mix, out_coef, next_in, next_gain, eps, (TYPE*)normed, S, H);                    \
    } while (0)
    if (dtype == LLMK_F32) {
        if (S <= 4) STREAM_STEP_LAUNCH(float, 4); else if (S <= 8) STREAM_STEP_LAUNCH(float, 8); else STREAM_STEP_LAUNCH(float, 16);
    } else if (dtype == LLMK_BF16) {
        if (S <= 4) STREAM_STEP_LAUNCH(bf16, 4); else if (S <= 8) STREAM_STEP_LAUNCH(bf16, 8); else STREAM_STEP_LAUNCH(bf16, 16);
    } else
        LLMK_FAIL("stream_step: unknown dtype %d", dtype);
#undef STREAM_STEP_LAUNCH
    LLMK_CHECK_LAUNCH_RC("stream_step", e);
    return LLMK_OK;
}

// collapse == 0: streams[r, s, :] = row[r, :] for every s.  collapse != 0: row[r, :] = sum_s streams[r, s, :].
__global__ void stream_spread_kernel(float* __restrict__ streams, float* __restrict__ row, long long n, int S, int H, int collapse) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n * H; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / H;
        const int c = (int)(i % H);
        float* xs = streams + (size_t)r * S * H + c;
        if (collapse) {
            float acc = xs[0];
            for (int s = 1; s < S; ++s) acc += xs[(size_t)s * H];
            row[i] = acc;
        } else {
            const float v = row[i];
            for (int s = 0; s < S; ++s) xs[(size_t)s * H] = v;
        }
    }
}

LLMK_EXPORT int llmk_stream_spread(float* streams, float* row, int n_rows, int S, int H, int collapse, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (S <= 0 || H <= 0) LLMK_FAIL("stream_spread: %d streams of %d values", S, H);
    long long blocks = ((long long)n_rows * H + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    LLMK_CHECK_LAUNCH_RC("stream_spread", llmk_launch(stream_spread_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, true,
                                                      streams, row, (long long)n_rows, S, H, collapse));
    return LLMK_OK;
}
