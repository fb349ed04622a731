// Routed feed-forward (mixture of experts) on the device, without a trip to the host:
//
//   zi_route_topk     float32 router logits [n, E] -> the `top` largest per token (lowest index wins a tie) and the
//                     softmax over those alone, in float32
//   zi_moe_group      the (token, choice) pairs grouped by expert: offsets[E + 1], sorted row -> pair, pair -> sorted row
//   zi_moe_gemm       grouped product: C[r, :] = A[src(r), :] . W[e(r)]^T for the sorted rows r of every expert, tiles
//                     found on the device from the offsets; optional clamped, gated activation in the epilogue
//   zi_moe_combine    out[t, :] = sum_j weight[t, j] * Y[row(t, j), :] (+ a shared expert's output), j in order
//
// A row's result depends on its own operands alone (one k-ascending chain per output element), so the order of rows
// inside an expert's group, which comes from atomics, changes no value.
#include "zi_common.cuh"
#include <mma.h>

ZI_DEFINE_LAST_ERROR(moe)

// ---------------------------------------------------------------------------------------
// Router: top-k and softmax over the chosen, one warp per token.
// ---------------------------------------------------------------------------------------
#define RT_WARPS 4
#define RT_MAX_PER_LANE 32            // experts <= 1024
__global__ void __launch_bounds__(RT_WARPS * 32)
route_topk_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int top, int* __restrict__ idx,
                  float* __restrict__ wts, int score, const float* __restrict__ choice_bias) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RT_WARPS + warp;
    if (t >= n_tokens) return;
    const float* z = logits + (size_t)t * n_experts;
    float v[RT_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < RT_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < n_experts ? z[e] : -INFINITY;
    }
    float first = 0.0f, denom = 0.0f;
    float zmax = 0.0f, zsum = 1.0f;
    if (score == 2) {
        // every expert's share of the softmax over all of them; the choice goes by share + choice_bias, the weight is the share
        zmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < RT_MAX_PER_LANE; ++i) zmax = fmaxf(zmax, v[i]);
        zmax = warp_max(zmax);
        zsum = 0.0f;
#pragma unroll
        for (int i = 0; i < RT_MAX_PER_LANE; ++i)
            if (lane + 32 * i < n_experts) zsum += expf(v[i] - zmax);
        zsum = warp_sum(zsum);
#pragma unroll
        for (int i = 0; i < RT_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < n_experts) v[i] = expf(v[i] - zmax) / zsum + (choice_bias ? choice_bias[e] : 0.0f);
        }
    }
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < RT_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < n_experts && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (j == 0) first = best;                       // the largest of all: the softmax's reference point
        const float p = score == 2 ? expf(z[best_e] - zmax) / zsum : score == 1 ? 1.0f / (1.0f + expf(-best)) : expf(best - first);
        denom += p;
        if (lane == 0) { idx[(size_t)t * top + j] = best_e; wts[(size_t)t * top + j] = p; }
#pragma unroll
        for (int i = 0; i < RT_MAX_PER_LANE; ++i)
            if (lane + 32 * i == best_e) v[i] = -INFINITY;
    }
    __syncwarp();
    if (lane == 0 && score == 0)
        for (int j = 0; j < top; ++j) wts[(size_t)t * top + j] = wts[(size_t)t * top + j] / denom;
}

// score 0: the weights are the softmax over the chosen logits; 1: each chosen expert's own sigmoid(logit), not renormalised;
// 2: each chosen expert's share of the softmax over all experts, not renormalised, the choice going by share + choice_bias
// (float32 per expert, or null)
ZI_EXPORT int zi_route_topk(const float* logits, int n_tokens, int n_experts, int top, int* idx, float* wts, int score,
                            const float* choice_bias, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts <= 0 || n_experts > 32 * RT_MAX_PER_LANE) return zi_fail("route_topk: %d experts (1..%d)", n_experts, 32 * RT_MAX_PER_LANE);
    if (top <= 0 || top > n_experts) return zi_fail("route_topk: top=%d of %d experts", top, n_experts);
    if (score < 0 || score > 2) return zi_fail("route_topk: unknown score rule %d", score);
    if (choice_bias && score != 2) return zi_fail("route_topk: a bias on the choice goes with score rule 2 only");
    route_topk_kernel<<<(n_tokens + RT_WARPS - 1) / RT_WARPS, RT_WARPS * 32, 0, stream>>>(logits, n_tokens, n_experts, top, idx, wts, score,
                                                                                         choice_bias);
    return zi_check_launch("route_topk");
}

// ---------------------------------------------------------------------------------------
// The router in one kernel: logits z[e] = x . Wr[e] + b[e] in float32 (x and Wr of any storage type), the `top`
// largest and the softmax over them.  A block takes one or four tokens: their rows of x wait in shared memory as float32,
// every warp takes experts w, w + 8, ... for all of them; a lane's partial sum runs over k in rising order and the warp adds the lanes in a
// fixed order, so a token's logits depend on nothing else in the step.  Then warp r chooses for the block's token r as
// route_topk_kernel does.
// ---------------------------------------------------------------------------------------
#define RF_WARPS 8
// RF_TOK tokens per block (one per warp when it comes to choosing), so that a weight row is read once for all of them:
// four for steps of many tokens, one for decode steps, whose few tokens want as many blocks as they can get.
template <typename TX, typename TW, int RF_TOK>
__global__ void __launch_bounds__(RF_WARPS * 32)
route_fused_kernel(const TX* __restrict__ x, long long ldx, const TW* __restrict__ w, const float* __restrict__ bias,
                   int n_tokens, int K, int n_experts, int top, int* __restrict__ idx, float* __restrict__ wts,
                   float* __restrict__ logits_out, int score, const float* __restrict__ choice_bias) {
    extern __shared__ __align__(16) float rf_smem[];              // x rows [RF_TOK][K], then logits [RF_TOK][n_experts], twice
    float* xs = rf_smem;
    float* z = rf_smem + RF_TOK * K;
    float* share = z + RF_TOK * n_experts;                        // score rule 2: every expert's share of the softmax over all
    const int t0 = blockIdx.x * RF_TOK, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int toks = n_tokens - t0 < RF_TOK ? n_tokens - t0 : RF_TOK;
    // Rows that are read eight values per lane (vec) lie in two halves: values 8c .. 8c+3 of chunk c at 4c, values
    // 8c+4 .. 8c+7 at K/2 + 4c, so that the lanes of a warp read consecutive 16 bytes and meet no bank twice.
    const bool vec = K % 8 == 0 && (((uintptr_t)w) & 15) == 0;
    if (vec && ldx % 8 == 0 && (((uintptr_t)x) & 31) == 0) {
        for (int i = threadIdx.x * 8; i < RF_TOK * K; i += RF_WARPS * 32 * 8) {
            const int r = i / K, k = i - r * K;
            float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if (r < toks) load8(x + (size_t)(t0 + r) * ldx + k, v);
            *reinterpret_cast<float4*>(xs + r * K + (k >> 1)) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(xs + r * K + (K >> 1) + (k >> 1)) = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
        for (int i = threadIdx.x; i < RF_TOK * K; i += RF_WARPS * 32) {
            const int r = i / K, k = i - r * K;
            const int at = vec ? ((k & 7) < 4 ? ((k >> 3) << 2) + (k & 3) : (K >> 1) + ((k >> 3) << 2) + (k & 3)) : k;
            xs[r * K + at] = r < toks ? to_f32<TX>(x[(size_t)(t0 + r) * ldx + k]) : 0.0f;
        }
    }
    __syncthreads();
    for (int e = warp; e < n_experts; e += RF_WARPS) {
        const TW* wr = w + (size_t)e * K;
        float acc[RF_TOK];
#pragma unroll
        for (int r = 0; r < RF_TOK; ++r) acc[r] = 0.0f;
        if (vec) {
            for (int k = lane * 8; k < K; k += 256) {
                float wv[8];
                load8(wr + k, wv);
#pragma unroll
                for (int r = 0; r < RF_TOK; ++r) {
                    const float4 x0 = *reinterpret_cast<const float4*>(xs + r * K + (k >> 1));
                    const float4 x1 = *reinterpret_cast<const float4*>(xs + r * K + (K >> 1) + (k >> 1));
                    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r] = fmaf(xv[i], wv[i], acc[r]);
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                const float wv = to_f32<TW>(wr[k]);
#pragma unroll
                for (int r = 0; r < RF_TOK; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < RF_TOK; ++r) {
            const float sum = warp_sum(acc[r]);
            if (lane == 0 && r < toks) {
                const float v = sum + (bias ? bias[e] : 0.0f);
                z[r * n_experts + e] = v;
                if (logits_out) logits_out[(size_t)(t0 + r) * n_experts + e] = v;
            }
        }
    }
    __syncthreads();
    if (warp >= toks) return;                       // warp r chooses for token t0 + r
    const int t = t0 + warp;
    float* zt = z + warp * n_experts;
    float* st = share + warp * n_experts;
    float first = 0.0f, denom = 0.0f;
    if (score == 2) {
        float zmax = -INFINITY, zsum = 0.0f;
        for (int e = lane; e < n_experts; e += 32) zmax = fmaxf(zmax, zt[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < n_experts; e += 32) zsum += expf(zt[e] - zmax);
        zsum = warp_sum(zsum);
        for (int e = lane; e < n_experts; e += 32) {
            const float p = expf(zt[e] - zmax) / zsum;
            st[e] = p;
            zt[e] = p + (choice_bias ? choice_bias[e] : 0.0f);      // what the choice goes by
        }
        __syncwarp();
    }
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = zt[e];
            if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (j == 0) first = best;
        const float p = score == 2 ? st[best_e] : score == 1 ? 1.0f / (1.0f + expf(-best)) : expf(best - first);
        denom += p;
        if (lane == 0) {
            idx[(size_t)t * top + j] = best_e;
            wts[(size_t)t * top + j] = p;
            zt[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0 && score == 0)
        for (int j = 0; j < top; ++j) wts[(size_t)t * top + j] = wts[(size_t)t * top + j] / denom;
}

// logits_out: optional float32 [n_tokens, n_experts] (tests).  bias: float32 or null.  score: as zi_route_topk.
ZI_EXPORT int zi_route(const void* x, int x_dtype, long long ldx, const void* w, int w_dtype, const float* bias, int n_tokens,
                       int K, int n_experts, int top, int* idx, float* wts, float* logits_out, int score, const float* choice_bias,
                       cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (score < 0 || score > 2) return zi_fail("route: unknown score rule %d", score);
    if (choice_bias && score != 2) return zi_fail("route: a bias on the choice goes with score rule 2 only");
    if (K <= 0 || n_experts <= 0 || n_experts > 4096) return zi_fail("route: K=%d experts=%d", K, n_experts);
    if (top <= 0 || top > n_experts) return zi_fail("route: top=%d of %d experts", top, n_experts);
    const int tok = n_tokens > 64 ? 4 : 1;
    const size_t smem = (size_t)tok * ((size_t)K + 2 * (size_t)n_experts) * sizeof(float);
    if (smem > 200 * 1024) return zi_fail("route: a row of %d values and %d logits do not fit shared memory", K, n_experts);
    ZI_DISPATCH(x_dtype, TX, ZI_DISPATCH(w_dtype, TW, {
        auto fn = tok == 4 ? route_fused_kernel<TX, TW, 4> : route_fused_kernel<TX, TW, 1>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return zi_fail("route: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        }
        fn<<<(n_tokens + tok - 1) / tok, RF_WARPS * 32, smem, stream>>>((const TX*)x, ldx, (const TW*)w, bias, n_tokens, K, n_experts, top,
                                                                        idx, wts, logits_out, score, choice_bias);
    }););
    return zi_check_launch("route");
}

// ---------------------------------------------------------------------------------------
// Grouping: one block.  offsets[e] .. offsets[e + 1] are the sorted rows of expert e.  A pair whose expert is n_experts or
// more (an expert without weights, which returns its input) gets no sorted row: pair_row is -1 there.
// ---------------------------------------------------------------------------------------
#define GROUP_THREADS 1024
__global__ void __launch_bounds__(GROUP_THREADS)
moe_group_kernel(const int* __restrict__ idx, int n_pairs, int n_experts, int* __restrict__ offsets,
                 int* __restrict__ row_pair, int* __restrict__ pair_row) {
    extern __shared__ int sh[];                 // counts[E], then cursors[E]
    int* counts = sh;
    int* cursor = sh + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += GROUP_THREADS) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += GROUP_THREADS)
        if (idx[p] < n_experts) atomicAdd(&counts[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += counts[e];
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += GROUP_THREADS) {
        if (idx[p] >= n_experts) { pair_row[p] = -1; continue; }
        const int r = atomicAdd(&cursor[idx[p]], 1);
        row_pair[r] = p;
        pair_row[p] = r;
    }
}

ZI_EXPORT int zi_moe_group(const int* idx, int n_pairs, int n_experts, int* offsets, int* row_pair, int* pair_row,
                           cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts <= 0 || n_experts > 4096) return zi_fail("moe_group: %d experts", n_experts);
    moe_group_kernel<<<1, GROUP_THREADS, 2 * n_experts * sizeof(int), stream>>>(idx, n_pairs, n_experts, offsets, row_pair, pair_row);
    return zi_check_launch("moe_group");
}

// Grouping with every expert's rows padded to a multiple of `pad` (the row tile of the tcgen05 grouped product):
// starts[e] is the first sorted row of expert e (a multiple of pad), row_pair[r] the pair at sorted row r or -1 for a
// row of padding, pair_row its inverse, tile_expert[t] the expert of row tile t or -1 behind the last one.
// row_pair has n_rows_max = tiles_max * pad entries, tile_expert tiles_max.
__global__ void __launch_bounds__(GROUP_THREADS)
moe_group_padded_kernel(const int* __restrict__ idx, int n_pairs, int n_experts, int pad, int tiles_max,
                        int* __restrict__ starts, int* __restrict__ row_pair, int* __restrict__ pair_row,
                        int* __restrict__ tile_expert) {
    extern __shared__ int sh[];                 // counts[E], then cursors[E]
    int* counts = sh;
    int* cursor = sh + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += GROUP_THREADS) counts[e] = 0;
    for (int r = threadIdx.x; r < tiles_max * pad; r += GROUP_THREADS) row_pair[r] = -1;
    for (int t = threadIdx.x; t < tiles_max; t += GROUP_THREADS) tile_expert[t] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += GROUP_THREADS)
        if (idx[p] < n_experts) atomicAdd(&counts[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            starts[e] = run;
            cursor[e] = run;
            const int tiles = (counts[e] + pad - 1) / pad;
            for (int t = 0; t < tiles; ++t) tile_expert[run / pad + t] = e;
            run += tiles * pad;
        }
        starts[n_experts] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += GROUP_THREADS) {
        if (idx[p] >= n_experts) { pair_row[p] = -1; continue; }
        const int r = atomicAdd(&cursor[idx[p]], 1);
        row_pair[r] = p;
        pair_row[p] = r;
    }
}

ZI_EXPORT int zi_moe_group_padded(const int* idx, int n_pairs, int n_experts, int pad, int tiles_max, int* starts,
                                  int* row_pair, int* pair_row, int* tile_expert, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts <= 0 || n_experts > 4096 || pad <= 0) return zi_fail("moe_group: %d experts, pad %d", n_experts, pad);
    if ((long long)tiles_max * pad < (long long)n_pairs + (long long)n_experts * (pad - 1))
        return zi_fail("moe_group: %d tiles of %d rows cannot hold %d pairs of %d experts", tiles_max, pad, n_pairs, n_experts);
    moe_group_padded_kernel<<<1, GROUP_THREADS, 2 * n_experts * sizeof(int), stream>>>(idx, n_pairs, n_experts, pad, tiles_max,
                                                                                      starts, row_pair, pair_row, tile_expert);
    return zi_check_launch("moe_group_padded");
}

// Rows of x brought into sorted order: out[r, :] = x[row_pair[r] / pairs_per_src, :] (times scale[row_pair[r]] where a
// scale per pair is given, rounded once), zeros for a row of padding.
// bfloat16, K % 8 == 0, 16-byte aligned rows.
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ row_pair,
                                       int pairs_per_src, bf16* __restrict__ out, int n_rows, int k8,
                                       const float* __restrict__ scale) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n_rows * k8;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / k8), c = (int)(i - (long long)r * k8);
        const int pair = row_pair[r];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (pair >= 0) v = *reinterpret_cast<const uint4*>(x + (size_t)(pair / pairs_per_src) * ldx + c * 8);
        if (scale && pair >= 0) {
            float f[8];
            load8(reinterpret_cast<const bf16*>(&v), f);
            const float sc = scale[pair];
#pragma unroll
            for (int q = 0; q < 8; ++q) f[q] *= sc;
            store8(reinterpret_cast<bf16*>(&v), f);
        }
        *reinterpret_cast<uint4*>(out + (size_t)r * k8 * 8 + c * 8) = v;
    }
}

ZI_EXPORT int zi_moe_gather_rows(const void* x, long long ldx, const int* row_pair, int pairs_per_src, void* out, int n_rows,
                                 int K, const float* scale, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || (((uintptr_t)x | (uintptr_t)out) & 15) || pairs_per_src <= 0)
        return zi_fail("moe_gather_rows: K=%d and the rows must be multiples of 8 elements and 16-byte aligned", K);
    const long long total = (long long)n_rows * (K / 8);
    const long long want = (total + 255) / 256;
    moe_gather_rows_kernel<<<(int)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>((const bf16*)x, ldx, row_pair, pairs_per_src,
                                                                                       (bf16*)out, n_rows, K / 8, scale);
    return zi_check_launch("moe_gather_rows");
}

// ---------------------------------------------------------------------------------------
// Grouped product.  Sorted row r belongs to expert e with offsets[e] <= r < offsets[e + 1]; its A row is
// A[src, :] with src = row_pair[r] / pairs_per_src (row_pair null: src = r).  W is [E, N_w, K].
//   gated == 0: C[r, n] = A[src] . W[e, n]                                  (N_w = N)
//   gated == 1: W holds gate rows then up rows (N_w = 2 N);
//               C[r, n] = act(A[src] . W[e, n], A[src] . W[e, N + n])       (see clamped_gate)
//   gated == 2: C[r, n] = max(A[src] . W[e, n], 0)^2                        (N_w = N)
// a_scale (optional, float32, one per pair): the A row of sorted row r is multiplied by a_scale[row_pair[r]] (row_pair
// null: a_scale[r]) and rounded to A's storage type before the product: a router weight on an expert's input.
// Block b walks the experts' tiles of TM rows: the block's (expert, first row) is found from the offsets.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float clamped_gate(float g, float u, float limit, float slope, float up_offset) {
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return (g / (1.0f + expf(-slope * g))) * (u + up_offset);
}

__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int n_experts, int tile, int tm, int* expert,
                                          int* row0, int* row_end) {
    int t = tile;
    for (int e = 0; e < n_experts; ++e) {
        const int lo = offsets[e], hi = offsets[e + 1];
        const int tiles = (hi - lo + tm - 1) / tm;
        if (t < tiles) {
            *expert = e;
            *row0 = lo + t * tm;
            *row_end = hi;
            return true;
        }
        t -= tiles;
    }
    return false;
}

// SIMT form: float32 FMA chains in rising k, any operand types (the whole 32-bit path, and bfloat16 shapes the
// tensor-core form does not take).
#define GM 32
#define GN 64
#define GK 16
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ row_pair, int pairs_per_src,
                     const TW* __restrict__ W, const int* __restrict__ offsets, int n_experts, TC* __restrict__ C,
                     long long ldc, int N, int K, int gated, float limit, float slope, float up_offset,
                     const float* __restrict__ a_scale) {
    __shared__ float As[GK][GM + 1];
    __shared__ float Ws[2][GK][GN + 1];
    __shared__ int src_rows[GM];
    __shared__ float src_scale[GM];
    __shared__ int tile_info[3];
    const bool relu2 = gated == 2;
    gated = gated == 1;
    if (threadIdx.x == 0) {
        int e = 0, r0 = 0, rend = 0;
        if (!find_tile(offsets, n_experts, blockIdx.y, GM, &e, &r0, &rend)) e = -1;
        tile_info[0] = e; tile_info[1] = r0; tile_info[2] = rend;
    }
    __syncthreads();
    const int e = tile_info[0], r0 = tile_info[1], rend = tile_info[2];
    if (e < 0) return;
    const int tid = threadIdx.x;
    if (tid < GM) {
        const int r = r0 + tid;
        src_rows[tid] = r < rend ? (row_pair ? row_pair[r] / pairs_per_src : r) : -1;
        src_scale[tid] = (a_scale && r < rend) ? a_scale[row_pair ? row_pair[r] : r] : 1.0f;
    }
    __syncthreads();
    const int n0 = blockIdx.x * GN;
    const int n_w = gated ? 2 * N : N;
    const TW* We = W + (size_t)e * n_w * K;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads: 2 rows x 4 columns each
    float acc[2][2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[h][i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += GK) {
        // A tile: 32 rows x 16 k = 512 values, two per thread
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int i = tid * 2 + q, r = i / GK, k = k0 + i % GK;
            const int src = src_rows[r];
            float av = (src >= 0 && k < K) ? to_f32<TA>(A[(size_t)src * lda + k]) : 0.0f;
            if (a_scale) av = to_f32<TA>(from_f32<TA>(src_scale[r] * av));
            As[i % GK][r] = av;
        }
        // W tile(s): 64 rows x 16 k = 1024 values, four per thread
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int i = tid * 4 + q, r = i / GK, k = k0 + i % GK;
            const int n = n0 + r;
            const bool ok = n < N && k < K;
            Ws[0][i % GK][r] = ok ? to_f32<TW>(We[(size_t)n * K + k]) : 0.0f;
            if (gated) Ws[1][i % GK][r] = ok ? to_f32<TW>(We[(size_t)(N + n) * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float a[2], w[4];
            a[0] = As[kk][ty * 2]; a[1] = As[kk][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[0][kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[0][i][j] = fmaf(a[i], w[j], acc[0][i][j]);
            if (gated) {
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = Ws[1][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[1][i][j] = fmaf(a[i], w[j], acc[1][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = r0 + ty * 2 + i;
        if (r >= rend) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[0][i][j];
            if (gated) {
                // the two halves are rounded to the storage type first, as a separate product would have stored them
                const float g = to_f32<TC>(from_f32<TC>(v)), u = to_f32<TC>(from_f32<TC>(acc[1][i][j]));
                v = clamped_gate(g, u, limit, slope, up_offset);
            } else if (relu2) {
                v = fmaxf(to_f32<TC>(from_f32<TC>(v)), 0.0f);
                v = v * v;
            }
            C[(size_t)r * ldc + n] = from_f32<TC>(v);
        }
    }
}

// Few rows (decode steps): the product is bound by reading every used expert's weight once.  A block takes one
// expert and 32 (gated: 16) output columns, a warp four (two) of them: it streams those columns' weight rows (and, gated, the up rows
// that pair with them) with 16-byte loads, four or eight independent ones per lane and step, against up to GV_ROWS of
// the expert's rows of A that wait in shared memory as float32; float32 FMAs, lanes added in a fixed order.  An
// expert with more rows takes them GV_ROWS at a time (its weight rows then come from L2).  Experts without rows cost
// an empty block.
#define GV_ROWS 4
#define GV_WARPS 8
// columns per warp: four, or two with the gate (twice the sums and weights per column); either way at most 128
// registers, so that two blocks share an SM and one's start and end overlap with the other's streaming
#define GV_COLS (GATED ? 2 : 4)
template <typename TA, typename TW, typename TC, bool GATED>
__global__ void __launch_bounds__(GV_WARPS * 32, 2)
moe_gemv_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ row_pair, int pairs_per_src,
                const TW* __restrict__ W, const int* __restrict__ offsets, TC* __restrict__ C, long long ldc, int N, int K,
                float limit, float slope, float up_offset, const float* __restrict__ a_scale, int relu2) {
    extern __shared__ __align__(16) float gv_x[];                 // [GV_ROWS][K]
    const int e = blockIdx.y, lo = offsets[e], hi = offsets[e + 1];
    if (lo >= hi) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * GV_WARPS + warp) * GV_COLS;
    const TW* we = W + (size_t)e * (GATED ? 2 * N : N) * K;
    const TW* wg[GV_COLS];
#pragma unroll
    for (int c = 0; c < GV_COLS; ++c) wg[c] = we + (size_t)(n0 + c < N ? n0 + c : 0) * K;      // columns beyond N: a valid row, never stored
    const size_t up = (size_t)N * K;
    const bool vec = K % 8 == 0 && ((((uintptr_t)W) & 31) == 0);
    const bool vec_a = K % 8 == 0 && lda % 8 == 0 && ((((uintptr_t)A) & 31) == 0);
    for (int r0 = lo; r0 < hi; r0 += GV_ROWS) {
        const int rows = hi - r0 < GV_ROWS ? hi - r0 : GV_ROWS;
        __syncthreads();
        // rows that are read eight values per lane (vec) lie in two halves, as in route_fused_kernel
        if (vec && vec_a) {
            for (int i = threadIdx.x * 8; i < rows * K; i += GV_WARPS * 32 * 8) {
                const int r = i / K, k = i - r * K;
                const int src = row_pair ? row_pair[r0 + r] / pairs_per_src : r0 + r;
                float v[8];
                load8(A + (size_t)src * lda + k, v);
                if (a_scale) {
                    const float sc = a_scale[row_pair ? row_pair[r0 + r] : r0 + r];
#pragma unroll
                    for (int q = 0; q < 8; ++q) v[q] = to_f32<TA>(from_f32<TA>(sc * v[q]));
                }
                *reinterpret_cast<float4*>(gv_x + r * K + (k >> 1)) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(gv_x + r * K + (K >> 1) + (k >> 1)) = make_float4(v[4], v[5], v[6], v[7]);
            }
        } else {
            for (int i = threadIdx.x; i < rows * K; i += GV_WARPS * 32) {
                const int r = i / K, k = i - r * K;
                const int src = row_pair ? row_pair[r0 + r] / pairs_per_src : r0 + r;
                const int at = vec ? ((k & 7) < 4 ? ((k >> 3) << 2) + (k & 3) : (K >> 1) + ((k >> 3) << 2) + (k & 3)) : k;
                float av = to_f32<TA>(A[(size_t)src * lda + k]);
                if (a_scale) av = to_f32<TA>(from_f32<TA>(a_scale[row_pair ? row_pair[r0 + r] : r0 + r] * av));
                gv_x[r * K + at] = av;
            }
        }
        __syncthreads();
        if (n0 >= N) continue;
        float ag[GV_COLS][GV_ROWS], au[GV_COLS][GV_ROWS];
#pragma unroll
        for (int c = 0; c < GV_COLS; ++c)
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) ag[c][r] = au[c][r] = 0.0f;
        if (vec) {
#pragma unroll 2
            for (int k = lane * 8; k < K; k += 256) {
                float wv[GV_COLS][8], uv[GV_COLS][8];
#pragma unroll
                for (int c = 0; c < GV_COLS; ++c) {
                    load8(wg[c] + k, wv[c]);
                    if (GATED) load8(wg[c] + up + k, uv[c]);
                }
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r) {
                    if (r < rows) {
                        const float4 x0 = *reinterpret_cast<const float4*>(gv_x + r * K + (k >> 1));
                        const float4 x1 = *reinterpret_cast<const float4*>(gv_x + r * K + (K >> 1) + (k >> 1));
                        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int c = 0; c < GV_COLS; ++c)
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                ag[c][r] = fmaf(xv[i], wv[c][i], ag[c][r]);
                                if (GATED) au[c][r] = fmaf(xv[i], uv[c][i], au[c][r]);
                            }
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
#pragma unroll
                for (int c = 0; c < GV_COLS; ++c) {
                    const float wv = to_f32<TW>(wg[c][k]), uv = GATED ? to_f32<TW>(wg[c][up + k]) : 0.0f;
#pragma unroll
                    for (int r = 0; r < GV_ROWS; ++r) {
                        if (r < rows) {
                            ag[c][r] = fmaf(gv_x[r * K + k], wv, ag[c][r]);
                            if (GATED) au[c][r] = fmaf(gv_x[r * K + k], uv, au[c][r]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < GV_COLS; ++c)
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) {
                float g = warp_sum(ag[c][r]);
                float u = GATED ? warp_sum(au[c][r]) : 0.0f;
                if (lane == 0 && r < rows && n0 + c < N) {
                    if (GATED) {
                        // the two halves are rounded to the storage type first, as a separate product would have stored them
                        g = clamped_gate(to_f32<TC>(from_f32<TC>(g)), to_f32<TC>(from_f32<TC>(u)), limit, slope, up_offset);
                    } else if (relu2) {
                        g = fmaxf(to_f32<TC>(from_f32<TC>(g)), 0.0f);
                        g = g * g;
                    }
                    C[(size_t)(r0 + r) * ldc + n0 + c] = from_f32<TC>(g);
                }
            }
    }
}

// Tensor-core form (bfloat16 operands, float32 accumulation): 64 sorted rows x 64 columns per block, four warps of
// 16 rows each, `wmma` 16x16x16 fragments; A rows gathered through the row map into shared memory, W rows read in
// place.  K % 16 == 0 and 16-byte aligned rows.
#define TM_ 64
#define TN_ 64
#define TK_ 32
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ A, long long lda, const int* __restrict__ row_pair, int pairs_per_src,
                    const bf16* __restrict__ W, const int* __restrict__ offsets, int n_experts, bf16* C,
                    long long ldc, int N, int K, int gated, float limit, float slope, float up_offset,
                    const float* __restrict__ a_scale) {
    using namespace nvcuda;
    const bool relu2 = gated == 2;
    gated = gated == 1;
    __shared__ float src_scale[TM_];
    __shared__ __align__(32) bf16 As[TM_][TK_ + 8];
    __shared__ __align__(32) bf16 Ws[2][TN_][TK_ + 8];
    __shared__ __align__(32) float Cs[4][16][TN_ + 4];
    __shared__ int src_rows[TM_];
    __shared__ int tile_info[3];
    if (threadIdx.x == 0) {
        int e = 0, r0 = 0, rend = 0;
        if (!find_tile(offsets, n_experts, blockIdx.y, TM_, &e, &r0, &rend)) e = -1;
        tile_info[0] = e; tile_info[1] = r0; tile_info[2] = rend;
    }
    __syncthreads();
    const int e = tile_info[0], r0 = tile_info[1], rend = tile_info[2];
    if (e < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < TM_) {
        const int r = r0 + tid;
        src_rows[tid] = r < rend ? (row_pair ? row_pair[r] / pairs_per_src : r) : -1;
        src_scale[tid] = (a_scale && r < rend) ? a_scale[row_pair ? row_pair[r] : r] : 1.0f;
    }
    __syncthreads();
    const int n0 = blockIdx.x * TN_;
    const int n_w = gated ? 2 * N : N;
    const bf16* We = W + (size_t)e * n_w * K;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][TN_ / 16];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < TN_ / 16; ++j) wmma::fill_fragment(acc[h][j], 0.0f);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int k0 = 0; k0 < K; k0 += TK_) {
        // 64 rows x 32 k of A and of each W half: 256 pieces of 8 elements each, two per thread
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int i = tid * 2 + q, r = i >> 2, kc = (i & 3) * 8, k = k0 + kc;
            const int src = src_rows[r];
            if (a_scale && src >= 0 && k < K) {
                float av[8];
                load8(A + (size_t)src * lda + k, av);
#pragma unroll
                for (int t = 0; t < 8; ++t) av[t] *= src_scale[r];
                store8(&As[r][kc], av);
            } else {
                *reinterpret_cast<uint4*>(&As[r][kc]) =
                    (src >= 0 && k < K) ? *reinterpret_cast<const uint4*>(A + (size_t)src * lda + k) : zero;
            }
            const int n = n0 + r;
            const bool ok = n < N && k < K;
            *reinterpret_cast<uint4*>(&Ws[0][r][kc]) = ok ? *reinterpret_cast<const uint4*>(We + (size_t)n * K + k) : zero;
            if (gated)
                *reinterpret_cast<uint4*>(&Ws[1][r][kc]) = ok ? *reinterpret_cast<const uint4*>(We + (size_t)(N + n) * K + k) : zero;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK_; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
            wmma::load_matrix_sync(a, &As[warp * 16][kk], TK_ + 8);
#pragma unroll
            for (int j = 0; j < TN_ / 16; ++j) {
                wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b;
                wmma::load_matrix_sync(b, &Ws[0][j * 16][kk], TK_ + 8);
                wmma::mma_sync(acc[0][j], a, b, acc[0][j]);
                if (gated) {
                    wmma::load_matrix_sync(b, &Ws[1][j * 16][kk], TK_ + 8);
                    wmma::mma_sync(acc[1][j], a, b, acc[1][j]);
                }
            }
        }
        __syncthreads();
    }
    // Epilogue through shared memory: each warp owns its 16 rows, a lane two columns of each.  With the activation
    // the up half goes first and is parked, rounded to the storage type, in the output element it belongs to; the
    // same thread reads it back when the gate half follows.
    for (int h = gated ? 1 : 0; h >= 0; --h) {
#pragma unroll
        for (int j = 0; j < TN_ / 16; ++j) wmma::store_matrix_sync(&Cs[warp][0][j * 16], acc[h][j], TN_ + 4, wmma::mem_row_major);
        __syncwarp();
        for (int rr = 0; rr < 16; ++rr) {
            const int r = r0 + warp * 16 + rr;
            if (r >= rend) break;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int col = lane * 2 + c, n = n0 + col;
                if (n >= N) continue;
                bf16* dst = C + (size_t)r * ldc + n;
                const float v = Cs[warp][rr][col];
                if (h == 0 && gated) {
                    const float g = to_f32<bf16>(from_f32<bf16>(v));
                    *dst = from_f32<bf16>(clamped_gate(g, to_f32<bf16>(*dst), limit, slope, up_offset));
                } else if (relu2) {
                    const float g = fmaxf(to_f32<bf16>(from_f32<bf16>(v)), 0.0f);
                    *dst = from_f32<bf16>(g * g);
                } else {
                    *dst = from_f32<bf16>(v);
                }
            }
        }
        __syncwarp();
    }
}

ZI_EXPORT int zi_moe_gemm(const void* A, int a_dtype, long long lda, const int* row_pair, int pairs_per_src,
                          const void* W, int w_dtype, const int* offsets, int n_experts, void* C, int c_dtype,
                          long long ldc, int n_rows, int N, int K, int gated, float limit, float slope, float up_offset,
                          int allow_tensor_cores, const float* a_scale, cudaStream_t stream) {
    if (n_rows <= 0 || N <= 0) return 0;
    if (gated < 0 || gated > 2) return zi_fail("moe_gemm: unknown activation %d", gated);
    if (K <= 0 || n_experts <= 0) return zi_fail("moe_gemm: K=%d experts=%d", K, n_experts);
    if (row_pair && pairs_per_src <= 0) return zi_fail("moe_gemm: pairs_per_src=%d", pairs_per_src);
    // few rows: the weight-streaming form (allow_tensor_cores & 2 switches it off)
    // ... and so does a product all in float32: the SIMT form below adds every output's terms in rising k whatever the
    // number of rows, so float32 results do not depend on how a step was cut
    const bool all_f32 = a_dtype == ZI_F32 && w_dtype == ZI_F32 && c_dtype == ZI_F32;
    if (n_rows <= 64 && !(allow_tensor_cores & 2) && !all_f32 && (size_t)GV_ROWS * K * sizeof(float) <= 160 * 1024) {
        const size_t smem = (size_t)GV_ROWS * K * sizeof(float);
        const int cols = GV_WARPS * (gated == 1 ? 2 : 4);         // GV_COLS of the kernel that runs
        dim3 grid((N + cols - 1) / cols, n_experts);
        if (grid.y > 65535) return zi_fail("moe_gemm: %d experts are too many for one launch", n_experts);
        ZI_DISPATCH(a_dtype, TA, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(c_dtype, TC, {
            if (gated == 1) {
                auto fn = moe_gemv_kernel<TA, TW, TC, true>;
                if (smem > 48 * 1024 && cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                    return zi_fail("moe_gemm: cannot reserve %zu bytes of shared memory", smem);
                fn<<<grid, GV_WARPS * 32, smem, stream>>>((const TA*)A, lda, row_pair, pairs_per_src, (const TW*)W, offsets, (TC*)C,
                                                          ldc, N, K, limit, slope, up_offset, a_scale, gated == 2 ? 1 : 0);
            } else {
                auto fn = moe_gemv_kernel<TA, TW, TC, false>;
                if (smem > 48 * 1024 && cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                    return zi_fail("moe_gemm: cannot reserve %zu bytes of shared memory", smem);
                fn<<<grid, GV_WARPS * 32, smem, stream>>>((const TA*)A, lda, row_pair, pairs_per_src, (const TW*)W, offsets, (TC*)C,
                                                          ldc, N, K, limit, slope, up_offset, a_scale, gated == 2 ? 1 : 0);
            }
        });););
        return zi_check_launch("moe_gemm");
    }
    const bool tc = (allow_tensor_cores & 1) && a_dtype == ZI_BF16 && w_dtype == ZI_BF16 && c_dtype == ZI_BF16 && K % 8 == 0 &&
                    lda % 8 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
    if (tc) {
        dim3 grid((N + TN_ - 1) / TN_, (n_rows + TM_ - 1) / TM_ + n_experts);
        if (grid.y > 65535) return zi_fail("moe_gemm: %d rows are too many for one launch", n_rows);
        moe_gemm_mma_kernel<<<grid, 128, 0, stream>>>((const bf16*)A, lda, row_pair, pairs_per_src, (const bf16*)W, offsets,
                                                      n_experts, (bf16*)C, ldc, N, K, gated, limit, slope, up_offset, a_scale);
        return zi_check_launch("moe_gemm");
    }
    dim3 grid((N + GN - 1) / GN, (n_rows + GM - 1) / GM + n_experts);
    if (grid.y > 65535) return zi_fail("moe_gemm: %d rows are too many for one launch", n_rows);
    ZI_DISPATCH(a_dtype, TA, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(c_dtype, TC, {
        moe_gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, lda, row_pair, pairs_per_src, (const TW*)W,
                                                                  offsets, n_experts, (TC*)C, ldc, N, K, gated, limit, slope,
                                                                  up_offset, a_scale);
    });););
    return zi_check_launch("moe_gemm");
}

// ---------------------------------------------------------------------------------------
// Combine: out[t, :] = sum_j wts[t, j] * Y[pair_row[t * top + j], :]  (+ shared_gate[t] * shared[t, :]), j rising, float32, one
// rounding.  A pair without a sorted row (pair_row -1: an expert that returns its input) contributes wts[t, j] * x[t, :].
// shared_gate null: 1.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ Y, const int* __restrict__ pair_row, const float* __restrict__ wts,
                                   const T* __restrict__ shared, T* __restrict__ out, int top, int hidden,
                                   const T* __restrict__ x, long long ldx, const float* __restrict__ shared_gate) {
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float acc = 0.0f;
        for (int c = 0; c < top; ++c) {
            const int r = pair_row[(size_t)t * top + c];
            const float y = r >= 0 ? to_f32<T>(Y[(size_t)r * hidden + j]) : to_f32<T>(x[(size_t)t * ldx + j]);
            acc = fmaf(wts ? wts[(size_t)t * top + c] : 1.0f, y, acc);
        }
        if (shared) acc = fmaf(shared_gate ? shared_gate[t] : 1.0f, to_f32<T>(shared[(size_t)t * hidden + j]), acc);
        out[(size_t)t * hidden + j] = from_f32<T>(acc);
    }
}

// The same, eight columns per thread with 16- or 32-byte accesses (hidden % 8 == 0, aligned rows); the same sums.
template <typename T>
__global__ void moe_combine_vec8_kernel(const T* __restrict__ Y, const int* __restrict__ pair_row, const float* __restrict__ wts,
                                        const T* __restrict__ shared, T* __restrict__ out, int top, int hidden,
                                        const T* __restrict__ x, long long ldx, const float* __restrict__ shared_gate) {
    const int t = blockIdx.x;
    for (int j = threadIdx.x * 8; j < hidden; j += blockDim.x * 8) {
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        for (int c = 0; c < top; ++c) {
            const int r = pair_row[(size_t)t * top + c];
            const float wt = wts ? wts[(size_t)t * top + c] : 1.0f;
            float v[8];
            load8(r >= 0 ? Y + (size_t)r * hidden + j : x + (size_t)t * ldx + j, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(wt, v[i], acc[i]);
        }
        if (shared) {
            float v[8];
            load8(shared + (size_t)t * hidden + j, v);
            const float g = shared_gate ? shared_gate[t] : 1.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(g, v[i], acc[i]);
        }
        store8(out + (size_t)t * hidden + j, acc);
    }
}

ZI_EXPORT int zi_moe_combine(const void* Y, const int* pair_row, const float* wts, const void* shared, void* out, int dtype,
                             int n_tokens, int top, int hidden, const void* x, long long ldx, const float* shared_gate,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top <= 0 || hidden <= 0) return zi_fail("moe_combine: top=%d hidden=%d", top, hidden);
    if (hidden % 8 == 0 && (((uintptr_t)Y | (uintptr_t)shared | (uintptr_t)out | (uintptr_t)x) & 31) == 0 && ldx % 16 == 0) {
        ZI_DISPATCH(dtype, T, {
            moe_combine_vec8_kernel<T><<<n_tokens, hidden >= 2048 ? 256 : 128, 0, stream>>>((const T*)Y, pair_row, wts, (const T*)shared,
                                                                                           (T*)out, top, hidden, (const T*)x, ldx, shared_gate);
        });
        return zi_check_launch("moe_combine");
    }
    ZI_DISPATCH(dtype, T, {
        moe_combine_kernel<T><<<n_tokens, hidden >= 1024 ? 256 : 128, 0, stream>>>((const T*)Y, pair_row, wts, (const T*)shared,
                                                                                  (T*)out, top, hidden, (const T*)x, ldx, shared_gate);
    });
    return zi_check_launch("moe_combine");
}
