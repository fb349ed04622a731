// Linear recurrences with a matrix state per head, over the tokens of one step:
//
//   zi_linear_state         per head a state S (dim x vdim, float32) walked token by token in one of two rules:
//                             delta  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                                    with q, k made unit vectors per head (q also times q_scale), beta = sigmoid(b) and a
//                                    decay per head and key entry g = exp(-exp(A_log) softplus(a + dt_bias))
//                                    (or, with decay_per_head, one decay per head: a and dt_bias then hold one number per head)
//                             decay  S <- lambda S + k v^T;  o = S^T q          (lambda a constant of the head)
//                             forget S <- diag(f) S + (1 - f) v^T;  o = S^T q   with the gate per head and key entry
//                                    f = l + (1 - l) sigmoid(a), l a lower bound per head and key entry; 1 - f stands
//                                    where the other rules have a key
//                           the state read from and written back to the request's slot
//   zi_group_rmsnorm_gate   out = unit_rms_per_group(y) * w * gate(z), the gate sigmoid, SiLU or none
//
// Everything that enters the recurrence is float32: unit vectors, sigmoid, softplus, exponentials, decays, the state,
// the sums.  A token's sums have one order that depends on the sizes alone, and tokens are walked one by one, so a token's
// result does not depend on how its request was cut into steps or on what else is in the batch.
//
// A request's state slot (float32) holds S laid out [heads, vdim, dim]: a column's key entries are consecutive.  Slot -1
// (a row of padding): the state is zero and nothing is written.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(linrec)

#define LR_THREADS 128            // of the kernel that makes inputs ready
#define LR_LANES 8               // lanes that share a column of S
#define LR_COLS 16               // columns of S per block.  Measured on 2,048 tokens of 12 heads of 128 x 128: 8, 16 or 32 lanes
                                 // with 4 to 64 columns per block all take 0.5 to 1.3 ms; this one is the quickest
#define LR_CHUNK 16              // tokens staged in shared memory at a time by the walk that makes its own inputs ready
#define LR_WALK_CHUNK 32         // and by the walk over records (two such chunks are in shared memory)

struct LinearStateArgs {
    const void* q; const void* k; const void* v; const void* a; const void* b;
    long long ldq, ldk, ldv, lda, ldb;
    const float* dt_bias;        // [heads * dim]   (delta; forget: the gates' lower bounds)
    const float* a_log;          // [heads]         (delta)
    const float* decay;          // [heads]         (decay)
    float* state; long long slot_stride;
    const int* slots; const int* bounds;
    float* y;                    // [tokens, heads * vdim]
    int n_segments, heads, kv_heads, dim, vdim;
    int act_silu;                // bit 0: SiLU on q, bit 1: on k, bit 2: on v
    int decay_per_head;          // delta: a is [tokens, heads] and dt_bias [heads]: one decay per head instead of one per key entry
    float q_scale, unit_eps;
};

// The rules: which of them keeps a decay per key entry in a token's record, and which corrects the write by what the state
// already answers to the key.
#define LR_DELTA 0
#define LR_DECAY 1
#define LR_FORGET 2
#define LR_PER_ENTRY(RULE) ((RULE) != LR_DECAY)

__device__ __forceinline__ float lr_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float lr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float lr_silu(float x) { return x / (1.0f + expf(-x)); }

// ---- what both forms of the walk share, so that a token has the same bits whichever form walked it ------------------
// One warp makes a token's query and key of one query/key head ready: SiLU where asked, unit vectors (times q_scale for the
// query) in the delta rule, zero past dim; DP floats each to dq and dk (shared or global memory).  Returns q . k.
template <typename T, int DP, bool DELTA>
__device__ __forceinline__ float lr_ready_qk(const T* __restrict__ qr, const T* __restrict__ kr, int dim, int act_silu, float q_scale,
                                             float unit_eps, int lane, float* dq, float* dk) {
    float qv[DP / 32], kv[DP / 32];
    float qq = 0.0f, kk = 0.0f;
#pragma unroll
    for (int j = 0; j < DP / 32; ++j) {
        const int d = lane + 32 * j;
        float x = d < dim ? to_f32<T>(qr[d]) : 0.0f, z = d < dim ? to_f32<T>(kr[d]) : 0.0f;
        if (act_silu & 1) x = lr_silu(x);
        if (act_silu & 2) z = lr_silu(z);
        qv[j] = x; kv[j] = z;
        qq = fmaf(x, x, qq); kk = fmaf(z, z, kk);
    }
    float qs = q_scale, ks = 1.0f;
    if (DELTA) {
        qq = warp_sum(qq); kk = warp_sum(kk);
        qs = q_scale / sqrtf(qq + unit_eps);
        ks = 1.0f / sqrtf(kk + unit_eps);
    }
    float dot = 0.0f;
#pragma unroll
    for (int j = 0; j < DP / 32; ++j) {
        const int d = lane + 32 * j;
        const float x = qv[j] * qs, z = kv[j] * ks;
        dq[d] = x; dk[d] = z;
        dot = fmaf(x, z, dot);
    }
    return warp_sum(dot);
}

// The decay of one head and key entry: exp(-rate softplus(a + dt_bias)).
__device__ __forceinline__ float lr_decay(float a, float dt_bias, float rate) { return expf(-rate * lr_softplus(a + dt_bias)); }

// One warp makes everything ready that token n brings to head h's walk besides its values: query dq, key dk and, where the
// rule keeps one per key entry, decays dg (DP floats each, zero past dim).  Returns q . k.  rate: exp(A_log) of the head.
template <typename T, int DP, int RULE>
__device__ __forceinline__ float lr_ready_token(const LinearStateArgs& p, size_t n, int h, int kvh, float rate, int lane, float* dq,
                                                float* dk, float* dg) {
    const int dim = p.dim;
    if (RULE == LR_FORGET) {
        const T* qr = (const T*)p.q + n * p.ldq + (size_t)h * dim;
        const T* ar = (const T*)p.a + n * p.lda + (size_t)h * dim;
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < DP / 32; ++j) {
            const int d = lane + 32 * j;
            float x = 0.0f, f = 0.0f, w = 0.0f;
            if (d < dim) {
                x = to_f32<T>(qr[d]);
                if (p.act_silu & 1) x = lr_silu(x);
                x *= p.q_scale;
                const float low = p.dt_bias[(size_t)h * dim + d];
                f = low + (1.0f - low) * lr_sigmoid(to_f32<T>(ar[d]));
                w = 1.0f - f;
            }
            dq[d] = x; dk[d] = w; dg[d] = f;
            dot = fmaf(x, w, dot);
        }
        return warp_sum(dot);
    }
    const float dot = lr_ready_qk<T, DP, RULE == LR_DELTA>((const T*)p.q + n * p.ldq + (size_t)kvh * dim, (const T*)p.k + n * p.ldk + (size_t)kvh * dim,
                                                           dim, p.act_silu, p.q_scale, p.unit_eps, lane, dq, dk);
    if (RULE == LR_DELTA) {
        const T* a = (const T*)p.a;
        if (p.decay_per_head) {
            const float g = lr_decay(to_f32<T>(a[n * p.lda + h]), p.dt_bias[h], rate);
#pragma unroll
            for (int j = 0; j < DP / 32; ++j) {
                const int d = lane + 32 * j;
                dg[d] = d < dim ? g : 0.0f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < DP / 32; ++j) {
                const int d = lane + 32 * j;
                dg[d] = d < dim ? lr_decay(to_f32<T>(a[n * p.lda + (size_t)h * dim + d]), p.dt_bias[(size_t)h * dim + d], rate) : 0.0f;
            }
        }
    }
    return dot;
}

// One token through the R entries a thread holds of its column.  A column is shared by LANES lanes; a thread holds entries
// i * 4 LANES + sub * 4 + e (i < R / 4, e < 4), sub = lane % LANES, so that the lanes of a column read consecutive bytes of
// a staged vector and the columns of a warp read it as one broadcast; sk, sq, sg: the token's staged key, query and decays
// (R LANES floats each; what lies past dim is zero).  The column's output is o = q . S after the write
// = q . (g S) + (q . k) u.
//
// A token's walk comes in two halves, for callers that take several tokens in one stretch of straight-line code: the read-outs'
// sums over the lanes wait for one another side by side at the end, and a token's loads and products stand before the
// sums of the token before it.  Only the sum over k of the delta rule lies between one token's state and the next one's.
// lr_walk_token is the two halves and the sums for one token, so a token has the same bits whoever walks it.  The sums
// within a thread run in four chains (entry e of every group of four), which keeps consecutive instructions independent.
template <int R, int LANES, int RULE>
__device__ __forceinline__ void lr_token_local(float (&S)[R], float (&kr)[R], const float* sk, const float* sq, const float* sg, float lam,
                                               int sub, float& ks, float& qs) {
    float kS[4] = {0.0f, 0.0f, 0.0f, 0.0f}, qS[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < R / 4; ++i) {
        const int at = i * 4 * LANES + sub * 4;
        const float4 k4 = *reinterpret_cast<const float4*>(sk + at);
        const float4 q4 = *reinterpret_cast<const float4*>(sq + at);
        float4 g4 = make_float4(lam, lam, lam, lam);
        if (LR_PER_ENTRY(RULE)) g4 = *reinterpret_cast<const float4*>(sg + at);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float s = S[i * 4 + e] * gg[e];
            S[i * 4 + e] = s;
            kr[i * 4 + e] = kk[e];
            if (RULE == LR_DELTA) kS[e] = fmaf(kk[e], s, kS[e]);
            qS[e] = fmaf(qq[e], s, qS[e]);
        }
    }
    ks = (kS[0] + kS[1]) + (kS[2] + kS[3]);
    qs = (qS[0] + qS[1]) + (qS[2] + qS[3]);
}

template <int R>
__device__ __forceinline__ void lr_token_write(float (&S)[R], const float (&kr)[R], float u) {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = fmaf(kr[i], u, S[i]);
}

// Returns the column's output on all its lanes.
template <int R, int LANES, int RULE>
__device__ __forceinline__ float lr_walk_token(float (&S)[R], const float* sk, const float* sq, const float* sg, float lam, float vv,
                                               float beta, float qk, int sub) {
    float kr[R], ks, qs;
    lr_token_local<R, LANES, RULE>(S, kr, sk, sq, sg, lam, sub, ks, qs);
    float u = vv;
    if (RULE == LR_DELTA) {
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) ks += __shfl_xor_sync(0xffffffffu, ks, o);
        u = beta * (vv - ks);
    }
    lr_token_write<R>(S, kr, u);
#pragma unroll
    for (int o = 1; o < LANES; o <<= 1) qs += __shfl_xor_sync(0xffffffffu, qs, o);
    return fmaf(qk, u, qs);
}

// ---- the walk that makes its own inputs ready (steps of single tokens) -----------------------------------------------------
// DP = LANES * R >= dim; what lies past dim is zero.
template <typename T, int R, int LANES, int COLS, int RULE>
__global__ void __launch_bounds__(COLS * LANES)
linear_state_kernel(const LinearStateArgs p, int tiles) {
    constexpr int DP = LANES * R, NT = COLS * LANES;
    extern __shared__ float smem[];
    float* sq = smem;                              // [LR_CHUNK][DP]
    float* sk = sq + LR_CHUNK * DP;                // [LR_CHUNK][DP]
    float* sg = sk + LR_CHUNK * DP;                // [LR_CHUNK][DP]   (rules with a decay per key entry)
    float* sv = sg + (LR_PER_ENTRY(RULE) ? LR_CHUNK * DP : 0);  // [LR_CHUNK][COLS]
    float* sbeta = sv + LR_CHUNK * COLS;        // [LR_CHUNK]
    float* sqk = sbeta + LR_CHUNK;                 // [LR_CHUNK]
    const int seg = blockIdx.x / tiles, tile = blockIdx.x - seg * tiles, h = blockIdx.y;
    const int kvh = h / (p.heads / p.kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = threadIdx.x % LANES;
    const int col = tile * COLS + threadIdx.x / LANES;
    const bool live = col < p.vdim;
    const int t0 = p.bounds ? p.bounds[2 * seg] : seg, t1 = p.bounds ? p.bounds[2 * seg + 1] : seg + 1;
    const int slot = p.slots[seg];
    const int dim = p.dim, vdim = p.vdim;
    const T* v = (const T*)p.v;
    const T* b = (const T*)p.b;

    float S[R];
    float* srow = (slot >= 0 && live) ? p.state + (size_t)slot * p.slot_stride + ((size_t)h * vdim + col) * dim : nullptr;
#pragma unroll
    for (int i = 0; i < R / 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int d = i * 4 * LANES + sub * 4 + e;
            S[i * 4 + e] = (srow && d < dim) ? srow[d] : 0.0f;
        }
    const float lam = RULE == LR_DECAY ? p.decay[h] : 0.0f;
    const float rate = RULE == LR_DELTA ? expf(p.a_log[h]) : 0.0f;

    for (int c0 = t0; c0 < t1; c0 += LR_CHUNK) {
        const int cnt = min(LR_CHUNK, t1 - c0);
        __syncthreads();                                                   // the last chunk has been walked
        // ---- stage: q, k (unit vectors in the delta rule), the decays, q . k; a warp per token
        for (int tt = warp; tt < cnt; tt += NT / 32) {
            const size_t n = (size_t)(c0 + tt);
            const float dot = lr_ready_token<T, DP, RULE>(p, n, h, kvh, rate, lane, sq + tt * DP, sk + tt * DP, sg + tt * DP);
            if (lane == 0) {
                sqk[tt] = dot;
                sbeta[tt] = RULE == LR_DELTA ? lr_sigmoid(to_f32<T>(b[n * p.ldb + h])) : 1.0f;
            }
        }
        for (int idx = threadIdx.x; idx < cnt * COLS; idx += NT) {
            const int tt = idx / COLS, c = tile * COLS + (idx - tt * COLS);
            float x = c < vdim ? to_f32<T>(v[(size_t)(c0 + tt) * p.ldv + (size_t)h * vdim + c]) : 0.0f;
            if (p.act_silu & 4) x = lr_silu(x);
            sv[idx] = x;
        }
        __syncthreads();
        // ---- walk
        for (int tt = 0; tt < cnt; ++tt) {
            const float o = lr_walk_token<R, LANES, RULE>(S, sk + tt * DP, sq + tt * DP, sg + tt * DP, lam, sv[tt * COLS + threadIdx.x / LANES],
                                                           sbeta[tt], sqk[tt], sub);
            if (sub == 0 && live) p.y[(size_t)(c0 + tt) * ((size_t)p.heads * vdim) + (size_t)h * vdim + col] = o;
        }
    }
    if (srow) {
#pragma unroll
        for (int i = 0; i < R / 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = i * 4 * LANES + sub * 4 + e;
                if (d < dim) srow[d] = S[i * 4 + e];
            }
    }
}

template <typename T, int R, int LANES, int COLS, int RULE>
static int launch_linear_state(const LinearStateArgs& p, cudaStream_t stream) {
    const int tiles = (p.vdim + COLS - 1) / COLS;
    const size_t smem = ((size_t)LR_CHUNK * LANES * R * (LR_PER_ENTRY(RULE) ? 3 : 2) + LR_CHUNK * COLS + 2 * LR_CHUNK) * sizeof(float);
    if (smem > 48 * 1024) {
        static bool raised = false;       // per instantiation
        if (!raised) {
            cudaFuncSetAttribute(linear_state_kernel<T, R, LANES, COLS, RULE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            raised = true;
        }
    }
    linear_state_kernel<T, R, LANES, COLS, RULE><<<dim3((unsigned)(p.n_segments * tiles), (unsigned)p.heads), COLS * LANES, smem, stream>>>(p, tiles);
    return zi_check_launch("linear_state");
}

// ---- the walk over inputs made ready beforehand (steps that bring portions of prompts) ---------------------------------
// Making a token ready (loads from global memory, unit vectors, softplus and exponentials) does not depend on the state, so
// for long segments it runs first, over all tokens and heads at once, and leaves per token and head one record of float32
//   [ q DP | k DP | g DP (rules with a decay per key entry) | beta, q . k, 0, 0 ]
// and the values [tiles * COLS] (SiLU applied where asked, zero past vdim).  The walk then only copies records into
// shared memory, two chunks in flight, and walks.  Both forms call the same functions on a token, so its result has the
// same bits in either.
template <int RULE, int DP> struct LrRecord { static constexpr int SIZE = (LR_PER_ENTRY(RULE) ? 3 : 2) * DP + 4; };

template <typename T, int DP, int RULE>
__global__ void __launch_bounds__(LR_THREADS)
linear_state_ready_kernel(const LinearStateArgs p, float* __restrict__ rec, float* __restrict__ pv, int n_tokens, int vp) {
    constexpr int REC = LrRecord<RULE, DP>::SIZE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (LR_THREADS / 32) + warp;
    if (pair >= (long long)n_tokens * p.heads) return;
    const size_t n = (size_t)(pair / p.heads);
    const int h = (int)(pair - (long long)n * p.heads), kvh = h / (p.heads / p.kv_heads);
    const int dim = p.dim, vdim = p.vdim;
    const T* v = (const T*)p.v;
    float* r = rec + (size_t)pair * REC;
    const float rate = RULE == LR_DELTA ? expf(p.a_log[h]) : 0.0f;
    const float dot = lr_ready_token<T, DP, RULE>(p, n, h, kvh, rate, lane, r, r + DP, r + 2 * DP);
    float beta = 1.0f;
    if (RULE == LR_DELTA) beta = lr_sigmoid(to_f32<T>(((const T*)p.b)[n * p.ldb + h]));
    if (lane < 4) r[REC - 4 + lane] = lane == 0 ? beta : (lane == 1 ? dot : 0.0f);
    float* vr = pv + (size_t)pair * vp;
    for (int c = lane; c < vp; c += 32) {
        float x = c < vdim ? to_f32<T>(v[n * p.ldv + (size_t)h * vdim + c]) : 0.0f;
        if (p.act_silu & 4) x = lr_silu(x);
        vr[c] = x;
    }
}

__device__ __forceinline__ void lr_copy16(float* dst, const float* src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(src) : "memory");
}

template <int R, int LANES, int COLS, int RULE>
__global__ void __launch_bounds__(COLS * LANES)
linear_state_walk_kernel(const LinearStateArgs p, const float* __restrict__ rec, const float* __restrict__ pv, int tiles) {
    constexpr int DP = LANES * R, NT = COLS * LANES, REC = LrRecord<RULE, DP>::SIZE;
    constexpr int STAGE = LR_WALK_CHUNK * (REC + COLS);                      // a chunk's records, then its values
    extern __shared__ __align__(16) float smem[];
    const int seg = blockIdx.x / tiles, tile = blockIdx.x - seg * tiles, h = blockIdx.y;
    const int sub = threadIdx.x % LANES;
    const int col = tile * COLS + threadIdx.x / LANES;
    const bool live = col < p.vdim;
    const int t0 = p.bounds ? p.bounds[2 * seg] : seg, t1 = p.bounds ? p.bounds[2 * seg + 1] : seg + 1;
    const int slot = p.slots[seg];
    const int dim = p.dim, vdim = p.vdim, vp = tiles * COLS;

    float S[R];
    float* srow = (slot >= 0 && live) ? p.state + (size_t)slot * p.slot_stride + ((size_t)h * vdim + col) * dim : nullptr;
#pragma unroll
    for (int i = 0; i < R / 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int d = i * 4 * LANES + sub * 4 + e;
            S[i * 4 + e] = (srow && d < dim) ? srow[d] : 0.0f;
        }
    const float lam = RULE == LR_DECAY ? p.decay[h] : 0.0f;

    auto fetch = [&](int c0, float* dst) {
        const int cnt = min(LR_WALK_CHUNK, t1 - c0);
        for (int idx = threadIdx.x; idx < cnt * (REC / 4); idx += NT) {
            const int tt = idx / (REC / 4), g = idx - tt * (REC / 4);
            lr_copy16(dst + tt * REC + g * 4, rec + ((size_t)(c0 + tt) * p.heads + h) * REC + g * 4);
        }
        for (int idx = threadIdx.x; idx < cnt * (COLS / 4); idx += NT) {
            const int tt = idx / (COLS / 4), g = idx - tt * (COLS / 4);
            lr_copy16(dst + LR_WALK_CHUNK * REC + tt * COLS + g * 4, pv + ((size_t)(c0 + tt) * p.heads + h) * vp + tile * COLS + g * 4);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    if (t0 < t1) fetch(t0, smem);
    int s = 0;
    for (int c0 = t0; c0 < t1; c0 += LR_WALK_CHUNK, s ^= 1) {
        const int cnt = min(LR_WALK_CHUNK, t1 - c0);
        if (c0 + LR_WALK_CHUNK < t1) {
            fetch(c0 + LR_WALK_CHUNK, smem + (s ^ 1) * STAGE);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();                                                   // everyone's copies of this chunk have landed
        const float* st = smem + s * STAGE;
        const float* sv = st + LR_WALK_CHUNK * REC + threadIdx.x / LANES;
        float* yc = p.y + (size_t)c0 * ((size_t)p.heads * vdim) + (size_t)h * vdim + col;
        int tt = 0;
        // four tokens at a time, in straight-line code
        for (; tt + 4 <= cnt; tt += 4) {
            float qs[4], u[4], qk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* r = st + (tt + j) * REC;
                float kr[R], ks;
                lr_token_local<R, LANES, RULE>(S, kr, r + DP, r, r + 2 * DP, lam, sub, ks, qs[j]);
                u[j] = sv[(tt + j) * COLS];
                qk[j] = r[REC - 3];
                if (RULE == LR_DELTA) {
#pragma unroll
                    for (int o = 1; o < LANES; o <<= 1) ks += __shfl_xor_sync(0xffffffffu, ks, o);
                    u[j] = r[REC - 4] * (u[j] - ks);
                }
                lr_token_write<R>(S, kr, u[j]);
            }
#pragma unroll
            for (int o = 1; o < LANES; o <<= 1)
#pragma unroll
                for (int j = 0; j < 4; ++j) qs[j] += __shfl_xor_sync(0xffffffffu, qs[j], o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (sub == 0 && live) yc[(size_t)(tt + j) * ((size_t)p.heads * vdim)] = fmaf(qk[j], u[j], qs[j]);
        }
        for (; tt < cnt; ++tt) {
            const float* r = st + tt * REC;
            const float o = lr_walk_token<R, LANES, RULE>(S, r + DP, r, r + 2 * DP, lam, sv[tt * COLS], r[REC - 4], r[REC - 3], sub);
            if (sub == 0 && live) yc[(size_t)tt * ((size_t)p.heads * vdim)] = o;
        }
        __syncthreads();                                                   // this chunk's buffer may be filled again
    }
    if (srow) {
#pragma unroll
        for (int i = 0; i < R / 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = i * 4 * LANES + sub * 4 + e;
                if (d < dim) srow[d] = S[i * 4 + e];
            }
    }
}

template <typename T, int R, int LANES, int COLS, int RULE>
static int launch_linear_state_ready(const LinearStateArgs& p, float* work, int n_tokens, cudaStream_t stream) {
    constexpr int REC = LrRecord<RULE, LANES * R>::SIZE;
    const int tiles = (p.vdim + COLS - 1) / COLS, vp = tiles * COLS;
    const long long pairs = (long long)n_tokens * p.heads;
    float* rec = work;
    float* pv = work + (size_t)pairs * REC;
    const long long blocks = (pairs + LR_THREADS / 32 - 1) / (LR_THREADS / 32);
    if (blocks > 2147483647LL) return zi_fail("linear_state: %lld tokens x heads are too many for one step", pairs);
    linear_state_ready_kernel<T, LANES * R, RULE><<<(unsigned)blocks, LR_THREADS, 0, stream>>>(p, rec, pv, n_tokens, vp);
    if (int rc = zi_check_launch("linear_state_ready")) return rc;
    const size_t smem = (size_t)2 * LR_WALK_CHUNK * (REC + COLS) * sizeof(float);
    if (smem > 48 * 1024) {
        static bool raised = false;       // per instantiation
        if (!raised) {
            cudaFuncSetAttribute(linear_state_walk_kernel<R, LANES, COLS, RULE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            raised = true;
        }
    }
    linear_state_walk_kernel<R, LANES, COLS, RULE><<<dim3((unsigned)(p.n_segments * tiles), (unsigned)p.heads), COLS * LANES, smem, stream>>>(p, rec, pv, tiles);
    return zi_check_launch("linear_state_walk");
}

// floats of workspace the form with inputs made ready needs for a step
static long long linear_state_work_floats(int rule, int n_tokens, int heads, int dim, int vdim) {
    const int dp = dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256;
    const int cols = LR_COLS;
    const int rec = (LR_PER_ENTRY(rule) ? 3 : 2) * dp + 4, vp = (vdim + cols - 1) / cols * cols;
    return (long long)n_tokens * heads * (rec + vp);
}

ZI_EXPORT long long zi_linear_state_work_floats(int rule, int n_tokens, int heads, int dim, int vdim) {
    return linear_state_work_floats(rule, n_tokens, heads, dim, vdim);
}

template <typename T, int RULE>
static int pick_linear_state_ready(const LinearStateArgs& p, float* work, int n_tokens, cudaStream_t stream) {
    if (p.dim <= 32) return launch_linear_state_ready<T, 4, LR_LANES, LR_COLS, RULE>(p, work, n_tokens, stream);
    if (p.dim <= 64) return launch_linear_state_ready<T, 8, LR_LANES, LR_COLS, RULE>(p, work, n_tokens, stream);
    if (p.dim <= 128) return launch_linear_state_ready<T, 16, LR_LANES, LR_COLS, RULE>(p, work, n_tokens, stream);
    return launch_linear_state_ready<T, 32, LR_LANES, LR_COLS, RULE>(p, work, n_tokens, stream);
}

template <typename T, int RULE>
static int pick_linear_state(const LinearStateArgs& p, cudaStream_t stream) {
    if (p.dim <= 32) return launch_linear_state<T, 4, LR_LANES, LR_COLS, RULE>(p, stream);
    if (p.dim <= 64) return launch_linear_state<T, 8, LR_LANES, LR_COLS, RULE>(p, stream);
    if (p.dim <= 128) return launch_linear_state<T, 16, LR_LANES, LR_COLS, RULE>(p, stream);
    return launch_linear_state<T, 32, LR_LANES, LR_COLS, RULE>(p, stream);
}

ZI_EXPORT int zi_linear_state(int rule, const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                              const void* a, long long lda, const void* b, long long ldb, int dtype, const float* dt_bias,
                              const float* a_log, const float* decay, float* state, long long slot_stride, const int* slots,
                              const int* bounds, float* y, int n_tokens, int n_segments, int heads, int kv_heads, int dim, int vdim,
                              int act_silu, int decay_per_head, float q_scale, float unit_eps, float* work, long long work_floats, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segments <= 0) return 0;
    if (rule < 0 || rule > 2) return zi_fail("linear_state: rule %d is none of 0 (delta), 1 (decay), 2 (forget)", rule);
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return zi_fail("linear_state: %d heads cannot share %d query/key heads", heads, kv_heads);
    if (dim <= 0 || dim > 256 || vdim <= 0) return zi_fail("linear_state: dim=%d must lie in 1 .. 256 and vdim=%d be positive", dim, vdim);
    if (heads > 65535) return zi_fail("linear_state: too many heads: %d", heads);
    if (rule == 0 && (!a || !b || !dt_bias || !a_log)) return zi_fail("linear_state: the delta rule needs a, b, dt_bias and A_log");
    if (rule == 1 && !decay) return zi_fail("linear_state: the decay rule needs the heads' decays");
    if (rule == 2 && (!a || !dt_bias || heads != kv_heads)) return zi_fail("linear_state: the forget rule needs the gates, their lower bounds and a query head per head");
    if (!bounds && n_segments != n_tokens) return zi_fail("linear_state: without bounds every segment is one token");
    LinearStateArgs p;
    p.q = q; p.k = k; p.v = v; p.a = a; p.b = b;
    p.ldq = ldq; p.ldk = ldk; p.ldv = ldv; p.lda = lda; p.ldb = ldb;
    p.dt_bias = dt_bias; p.a_log = a_log; p.decay = decay;
    p.state = state; p.slot_stride = slot_stride; p.slots = slots; p.bounds = bounds; p.y = y;
    p.n_segments = n_segments; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim; p.act_silu = act_silu; p.decay_per_head = decay_per_head;
    p.q_scale = q_scale; p.unit_eps = unit_eps;
    if (work) {
        // inputs made ready first, then the walk
        if (((size_t)work & 15) != 0) return zi_fail("linear_state: the workspace must start on a 16-byte boundary");
        if (work_floats < linear_state_work_floats(rule, n_tokens, heads, dim, vdim))
            return zi_fail("linear_state: a workspace of %lld floats is too small for %d tokens", work_floats, n_tokens);
        ZI_DISPATCH(dtype, T, {
            if (rule == LR_DELTA) return pick_linear_state_ready<T, LR_DELTA>(p, work, n_tokens, stream);
            if (rule == LR_FORGET) return pick_linear_state_ready<T, LR_FORGET>(p, work, n_tokens, stream);
            return pick_linear_state_ready<T, LR_DECAY>(p, work, n_tokens, stream);
        });
        return 0;
    }
    ZI_DISPATCH(dtype, T, {
        if (rule == LR_DELTA) return pick_linear_state<T, LR_DELTA>(p, stream);
        if (rule == LR_FORGET) return pick_linear_state<T, LR_FORGET>(p, stream);
        return pick_linear_state<T, LR_DECAY>(p, stream);
    });
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[n, c] = y[n, c] / sqrt(mean_group(y^2) + eps) * w[c mod w_len] * gate(z[n, c]), gate 0: sigmoid, 1: SiLU, 2: none (z unused); the mean over each of n_groups
// equal parts of a row.  y float32; z (rows may be strided) and out of the step's type.  One block per row; a group's sum
// is taken by one warp when there are at least as many groups as warps, else by the whole block, group after group.
// ---------------------------------------------------------------------------------------
#define GN_THREADS 256
template <typename T>
__device__ __forceinline__ float gn_gate(const T* zr, int c, int gate) {
    if (gate == 2) return 1.0f;
    const float z = to_f32<T>(zr[c]);
    return gate == 1 ? lr_silu(z) : lr_sigmoid(z);
}

template <typename T, typename TW>
__global__ void __launch_bounds__(GN_THREADS)
group_rmsnorm_gate_kernel(const float* __restrict__ y, const T* __restrict__ z, long long ldz, const TW* __restrict__ w, int w_len,
                          T* __restrict__ out, int inner, int n_groups, float eps, int gate) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, gw = inner / n_groups;
    const float* yr = y + (size_t)n * inner;
    const T* zr = gate == 2 ? nullptr : z + (size_t)n * ldz;
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
                orow[c] = from_f32<T>(yr[c] * r * to_f32<TW>(w[c % w_len]) * gn_gate<T>(zr, c, gate));
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
            orow[c] = from_f32<T>(yr[c] * r * to_f32<TW>(w[c % w_len]) * gn_gate<T>(zr, c, gate));
        }
    }
}

ZI_EXPORT int zi_group_rmsnorm_gate(const float* y, const void* z, int dtype, long long ldz, const void* w, int w_dtype, int w_len,
                                    void* out, int n_tokens, int inner, int n_groups, float eps, int gate, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (inner <= 0 || n_groups <= 0 || inner % n_groups) return zi_fail("group_rmsnorm_gate: %d groups do not divide %d", n_groups, inner);
    if (gate < 0 || gate > 2 || (gate != 2 && !z)) return zi_fail("group_rmsnorm_gate: gate %d is none of 0 (sigmoid), 1 (SiLU), 2 (none), or its input is missing", gate);
    if (w_len <= 0 || inner % w_len) return zi_fail("group_rmsnorm_gate: a weight of %d entries does not tile a row of %d", w_len, inner);
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        group_rmsnorm_gate_kernel<T, TW><<<n_tokens, GN_THREADS, 0, stream>>>(y, (const T*)z, ldz, (const TW*)w, w_len, (T*)out, inner,
                                                                            n_groups, eps, gate);
    }););
    return zi_check_launch("group_rmsnorm_gate");
}
