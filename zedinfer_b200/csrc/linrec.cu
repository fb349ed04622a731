// Linear recurrences with a matrix state per head, over the tokens of one step:
//
//   zi_linear_state         per head a state S (dim x vdim, float32) walked token by token in one of two rules:
//                             delta  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                                    with q, k made unit vectors per head (q also times q_scale), beta = sigmoid(b) and a
//                                    decay per head and key entry g = exp(-exp(A_log) softplus(a + dt_bias))
//                             decay  S <- lambda S + k v^T;  o = S^T q          (lambda a constant of the head)
//                           the state read from and written back to the request's slot
//   zi_group_rmsnorm_gate   out = unit_rms_per_group(y) * w * sigmoid(z)
//
// Everything that enters the recurrence is float32: unit vectors, sigmoid, softplus, exponentials, decays, the state,
// the sums.  A token's sums have one order that depends on the sizes alone, and tokens are walked one by one, so a token's
// result does not depend on how its request was cut into steps or on what else is in the batch.
//
// A request's state slot (float32) holds S laid out [heads, vdim, dim]: a column's key entries are consecutive.  Slot -1
// (a row of padding): the state is zero and nothing is written.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(linrec)

#define LR_THREADS 128
#define LR_COLS 16               // columns of S per block: 8 lanes share a column
#define LR_CHUNK 16              // tokens staged in shared memory at a time

struct LinearStateArgs {
    const void* q; const void* k; const void* v; const void* a; const void* b;
    long long ldq, ldk, ldv, lda, ldb;
    const float* dt_bias;        // [heads * dim]   (delta)
    const float* a_log;          // [heads]         (delta)
    const float* decay;          // [heads]         (decay)
    float* state; long long slot_stride;
    const int* slots; const int* bounds;
    float* y;                    // [tokens, heads * vdim]
    int n_segments, heads, kv_heads, dim, vdim, act_silu;
    float q_scale, unit_eps;
};

__device__ __forceinline__ float lr_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float lr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float lr_silu(float x) { return x / (1.0f + expf(-x)); }

// A thread holds R entries of one column: entries i * 32 + sub * 4 + e (i < R / 4, e < 4), sub = lane & 7, so that the
// eight lanes of a column read 128 consecutive bytes of a staged vector at a time.  DP = 8 * R >= dim; what lies past
// dim is zero.
template <typename T, int R, bool DELTA>
__global__ void __launch_bounds__(LR_THREADS)
linear_state_kernel(const LinearStateArgs p, int tiles) {
    constexpr int DP = 8 * R;
    extern __shared__ float smem[];
    float* sq = smem;                              // [LR_CHUNK][DP]
    float* sk = sq + LR_CHUNK * DP;                // [LR_CHUNK][DP]
    float* sg = sk + LR_CHUNK * DP;                // [LR_CHUNK][DP]   (delta only)
    float* sv = sg + (DELTA ? LR_CHUNK * DP : 0);  // [LR_CHUNK][LR_COLS]
    float* sbeta = sv + LR_CHUNK * LR_COLS;        // [LR_CHUNK]
    float* sqk = sbeta + LR_CHUNK;                 // [LR_CHUNK]
    const int seg = blockIdx.x / tiles, tile = blockIdx.x - seg * tiles, h = blockIdx.y;
    const int kvh = h / (p.heads / p.kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 7;
    const int col = tile * LR_COLS + (threadIdx.x >> 3);
    const bool live = col < p.vdim;
    const int t0 = p.bounds ? p.bounds[2 * seg] : seg, t1 = p.bounds ? p.bounds[2 * seg + 1] : seg + 1;
    const int slot = p.slots[seg];
    const int dim = p.dim, vdim = p.vdim;
    const T* q = (const T*)p.q; const T* k = (const T*)p.k; const T* v = (const T*)p.v;
    const T* a = (const T*)p.a; const T* b = (const T*)p.b;

    float S[R];
    float* srow = (slot >= 0 && live) ? p.state + (size_t)slot * p.slot_stride + ((size_t)h * vdim + col) * dim : nullptr;
#pragma unroll
    for (int i = 0; i < R / 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int d = i * 32 + sub * 4 + e;
            S[i * 4 + e] = (srow && d < dim) ? srow[d] : 0.0f;
        }
    const float lam = DELTA ? 0.0f : p.decay[h];
    const float rate = DELTA ? expf(p.a_log[h]) : 0.0f;

    for (int c0 = t0; c0 < t1; c0 += LR_CHUNK) {
        const int cnt = min(LR_CHUNK, t1 - c0);
        __syncthreads();                                                   // the last chunk has been walked
        // ---- stage: q, k (unit vectors in the delta rule), the decays, q . k; a warp per token
        for (int tt = warp; tt < cnt; tt += LR_THREADS / 32) {
            const size_t n = (size_t)(c0 + tt);
            const T* qr = q + n * p.ldq + (size_t)kvh * dim;
            const T* kr = k + n * p.ldk + (size_t)kvh * dim;
            float qv[DP / 32], kv[DP / 32];
            float qq = 0.0f, kk = 0.0f;
#pragma unroll
            for (int j = 0; j < DP / 32; ++j) {
                const int d = lane + 32 * j;
                float x = d < dim ? to_f32<T>(qr[d]) : 0.0f, z = d < dim ? to_f32<T>(kr[d]) : 0.0f;
                if (p.act_silu) { x = lr_silu(x); z = lr_silu(z); }
                qv[j] = x; kv[j] = z;
                qq = fmaf(x, x, qq); kk = fmaf(z, z, kk);
            }
            float qs = p.q_scale, ks = 1.0f;
            if (DELTA) {
                qq = warp_sum(qq); kk = warp_sum(kk);
                qs = p.q_scale / sqrtf(qq + p.unit_eps);
                ks = 1.0f / sqrtf(kk + p.unit_eps);
            }
            float dot = 0.0f;
#pragma unroll
            for (int j = 0; j < DP / 32; ++j) {
                const int d = lane + 32 * j;
                const float x = qv[j] * qs, z = kv[j] * ks;
                sq[tt * DP + d] = x; sk[tt * DP + d] = z;
                dot = fmaf(x, z, dot);
                if (DELTA) {
                    float g = 1.0f;
                    if (d < dim) {
                        const float pre = to_f32<T>(a[n * p.lda + (size_t)h * dim + d]) + p.dt_bias[(size_t)h * dim + d];
                        g = expf(-rate * lr_softplus(pre));
                    }
                    sg[tt * DP + d] = g;
                }
            }
            dot = warp_sum(dot);
            if (lane == 0) {
                sqk[tt] = dot;
                sbeta[tt] = DELTA ? lr_sigmoid(to_f32<T>(b[n * p.ldb + h])) : 1.0f;
            }
        }
        for (int idx = threadIdx.x; idx < cnt * LR_COLS; idx += LR_THREADS) {
            const int tt = idx / LR_COLS, c = tile * LR_COLS + (idx - tt * LR_COLS);
            float x = c < vdim ? to_f32<T>(v[(size_t)(c0 + tt) * p.ldv + (size_t)h * vdim + c]) : 0.0f;
            if (p.act_silu) x = lr_silu(x);
            sv[idx] = x;
        }
        __syncthreads();
        // ---- walk
        for (int tt = 0; tt < cnt; ++tt) {
            float kr[R];
            float kS = 0.0f, qS = 0.0f;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const int at = tt * DP + i * 32 + sub * 4;
                const float4 k4 = *reinterpret_cast<const float4*>(sk + at);
                const float4 q4 = *reinterpret_cast<const float4*>(sq + at);
                float4 g4 = make_float4(lam, lam, lam, lam);
                if (DELTA) g4 = *reinterpret_cast<const float4*>(sg + at);
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s = S[i * 4 + e] * gg[e];
                    S[i * 4 + e] = s;
                    kr[i * 4 + e] = kk[e];
                    if (DELTA) kS = fmaf(kk[e], s, kS);
                    qS = fmaf(qq[e], s, qS);
                }
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                if (DELTA) kS += __shfl_xor_sync(0xffffffffu, kS, o);
                qS += __shfl_xor_sync(0xffffffffu, qS, o);
            }
            const float vv = sv[tt * LR_COLS + (threadIdx.x >> 3)];
            const float u = DELTA ? sbeta[tt] * (vv - kS) : vv;
#pragma unroll
            for (int i = 0; i < R; ++i) S[i] = fmaf(kr[i], u, S[i]);
            if (sub == 0 && live) p.y[(size_t)(c0 + tt) * ((size_t)p.heads * vdim) + (size_t)h * vdim + col] = fmaf(sqk[tt], u, qS);
        }
    }
    if (srow) {
#pragma unroll
        for (int i = 0; i < R / 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = i * 32 + sub * 4 + e;
                if (d < dim) srow[d] = S[i * 4 + e];
            }
    }
}

template <typename T, int R, bool DELTA>
static int launch_linear_state(const LinearStateArgs& p, cudaStream_t stream) {
    const int tiles = (p.vdim + LR_COLS - 1) / LR_COLS;
    const size_t smem = ((size_t)LR_CHUNK * 8 * R * (DELTA ? 3 : 2) + LR_CHUNK * LR_COLS + 2 * LR_CHUNK) * sizeof(float);
    if (smem > 48 * 1024) {
        static bool raised = false;       // per instantiation
        if (!raised) {
            cudaFuncSetAttribute(linear_state_kernel<T, R, DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            raised = true;
        }
    }
    linear_state_kernel<T, R, DELTA><<<dim3((unsigned)(p.n_segments * tiles), (unsigned)p.heads), LR_THREADS, smem, stream>>>(p, tiles);
    return zi_check_launch("linear_state");
}

template <typename T, bool DELTA>
static int pick_linear_state(const LinearStateArgs& p, cudaStream_t stream) {
    if (p.dim <= 32) return launch_linear_state<T, 4, DELTA>(p, stream);
    if (p.dim <= 64) return launch_linear_state<T, 8, DELTA>(p, stream);
    if (p.dim <= 128) return launch_linear_state<T, 16, DELTA>(p, stream);
    return launch_linear_state<T, 32, DELTA>(p, stream);
}

ZI_EXPORT int zi_linear_state(int rule, const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                              const void* a, long long lda, const void* b, long long ldb, int dtype, const float* dt_bias,
                              const float* a_log, const float* decay, float* state, long long slot_stride, const int* slots,
                              const int* bounds, float* y, int n_tokens, int n_segments, int heads, int kv_heads, int dim, int vdim,
                              int act_silu, float q_scale, float unit_eps, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segments <= 0) return 0;
    if (rule != 0 && rule != 1) return zi_fail("linear_state: rule %d is neither 0 (delta) nor 1 (decay)", rule);
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return zi_fail("linear_state: %d heads cannot share %d query/key heads", heads, kv_heads);
    if (dim <= 0 || dim > 256 || vdim <= 0) return zi_fail("linear_state: dim=%d must lie in 1 .. 256 and vdim=%d be positive", dim, vdim);
    if (heads > 65535) return zi_fail("linear_state: too many heads: %d", heads);
    if (rule == 0 && (!a || !b || !dt_bias || !a_log)) return zi_fail("linear_state: the delta rule needs a, b, dt_bias and A_log");
    if (rule == 1 && !decay) return zi_fail("linear_state: the decay rule needs the heads' decays");
    if (!bounds && n_segments != n_tokens) return zi_fail("linear_state: without bounds every segment is one token");
    LinearStateArgs p;
    p.q = q; p.k = k; p.v = v; p.a = a; p.b = b;
    p.ldq = ldq; p.ldk = ldk; p.ldv = ldv; p.lda = lda; p.ldb = ldb;
    p.dt_bias = dt_bias; p.a_log = a_log; p.decay = decay;
    p.state = state; p.slot_stride = slot_stride; p.slots = slots; p.bounds = bounds; p.y = y;
    p.n_segments = n_segments; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim; p.act_silu = act_silu;
    p.q_scale = q_scale; p.unit_eps = unit_eps;
    ZI_DISPATCH(dtype, T, {
        if (rule == 0) return pick_linear_state<T, true>(p, stream);
        return pick_linear_state<T, false>(p, stream);
    });
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[n, c] = y[n, c] / sqrt(mean_group(y^2) + eps) * w[c mod w_len] * sigmoid(z[n, c]); the mean over each of n_groups
// equal parts of a row.  y float32; z (rows may be strided) and out of the step's type.  One block per row; a group's sum
// is taken by one warp when there are at least as many groups as warps, else by the whole block, group after group.
// ---------------------------------------------------------------------------------------
#define GN_THREADS 256
template <typename T, typename TW>
__global__ void __launch_bounds__(GN_THREADS)
group_rmsnorm_gate_kernel(const float* __restrict__ y, const T* __restrict__ z, long long ldz, const TW* __restrict__ w, int w_len,
                          T* __restrict__ out, int inner, int n_groups, float eps) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, gw = inner / n_groups;
    const float* yr = y + (size_t)n * inner;
    const T* zr = z + (size_t)n * ldz;
    T* orow = out + (size_t)n * inner;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (n_groups >= GN_THREADS / 32) {
        for (int g = warp; g < n_groups; g += GN_THREADS / 32) {
            float ss = 0.0f;
            for (int j = lane; j < gw; j += 32) { const float x = yr[g * gw + j]; ss = fmaf(x, x, ss); }
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)gw + eps);
            for (int j = lane; j < gw; j += 32) {
                const int c = g * gw + j;
                orow[c] = from_f32<T>(yr[c] * r * to_f32<TW>(w[c % w_len]) * lr_sigmoid(to_f32<T>(zr[c])));
            }
        }
        return;
    }
    for (int g = 0; g < n_groups; ++g) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < gw; j += GN_THREADS) { const float x = yr[g * gw + j]; ss = fmaf(x, x, ss); }
        ss = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(ss / (float)gw + eps);
        for (int j = threadIdx.x; j < gw; j += GN_THREADS) {
            const int c = g * gw + j;
            orow[c] = from_f32<T>(yr[c] * r * to_f32<TW>(w[c % w_len]) * lr_sigmoid(to_f32<T>(zr[c])));
        }
    }
}

ZI_EXPORT int zi_group_rmsnorm_gate(const float* y, const void* z, int dtype, long long ldz, const void* w, int w_dtype, int w_len,
                                    void* out, int n_tokens, int inner, int n_groups, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (inner <= 0 || n_groups <= 0 || inner % n_groups) return zi_fail("group_rmsnorm_gate: %d groups do not divide %d", n_groups, inner);
    if (w_len <= 0 || inner % w_len) return zi_fail("group_rmsnorm_gate: a weight of %d entries does not tile a row of %d", w_len, inner);
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        group_rmsnorm_gate_kernel<T, TW><<<n_tokens, GN_THREADS, 0, stream>>>(y, (const T*)z, ldz, (const TW*)w, w_len, (T*)out, inner,
                                                                            n_groups, eps);
    }););
    return zi_check_launch("group_rmsnorm_gate");
}
