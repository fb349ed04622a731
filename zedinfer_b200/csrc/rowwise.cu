// Row-wise kernels beside those of elementwise.cu: embedding with a learned position table, the logit cap,
// two feed-forward activations (squared ReLU; a clamped, sigmoid-gated product), and an RMSNorm whose output
// rows go straight into the pages of a paged cache (the latent of a latent-attention layer).
// All arithmetic is float32; storage types are float32 or bfloat16 per tensor.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(rowwise)

// ---------------------------------------------------------------------------------------
// Embedding with learned absolute positions: out[n, :] = table[ids[n], :] + pos_table[pos[n], :]
// ---------------------------------------------------------------------------------------
template <typename TT, typename TO>
__global__ void embedding_pos_kernel(const TT* __restrict__ table, const TT* __restrict__ pos_table,
                                     const int* __restrict__ ids, const int* __restrict__ pos, TO* __restrict__ out,
                                     int hidden, int vocab, int max_pos) {
    const int n = blockIdx.x;
    int id = ids[n], p = pos[n];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);       // the host refuses ids and positions outside the tables
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    const TT* src = table + (size_t)id * hidden;
    const TT* ps = pos_table + (size_t)p * hidden;
    TO* dst = out + (size_t)n * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) dst[j] = from_f32<TO>(to_f32<TT>(src[j]) + to_f32<TT>(ps[j]));
}

ZI_EXPORT int zi_embedding_pos(const void* table, const void* pos_table, int table_dtype, const int* ids, const int* pos,
                               void* out, int out_dtype, int n_tokens, int hidden, int vocab, int max_pos,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || max_pos <= 0)
        return zi_fail("embedding: hidden=%d vocab=%d positions=%d must be positive", hidden, vocab, max_pos);
    const int threads = hidden >= 1024 ? 256 : 128;
    ZI_DISPATCH(table_dtype, TT, ZI_DISPATCH(out_dtype, TO, {
        embedding_pos_kernel<TT, TO><<<n_tokens, threads, 0, stream>>>((const TT*)table, (const TT*)pos_table, ids, pos,
                                                                      (TO*)out, hidden, vocab, max_pos);
    }););
    return zi_check_launch("embedding_pos");
}

// ---------------------------------------------------------------------------------------
// Logit cap, in place on float32: x = cap * tanh(x / cap)
// ---------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

ZI_EXPORT int zi_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.0f)) return zi_fail("softcap: cap=%g must be positive", (double)cap);
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    softcap_kernel<<<(int)(want > 148 * 16 ? 148 * 16 : want), threads, 0, stream>>>(x, (size_t)total, cap);
    return zi_check_launch("softcap");
}

// ---------------------------------------------------------------------------------------
// Squared ReLU: out = max(x, 0)^2
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32<T>(x[i]), 0.0f);
        out[i] = from_f32<T>(v * v);
    }
}
template <typename T>
__global__ void relu2_vec8_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        float v[8];
        load8(x + i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[e] = fmaxf(v[e], 0.0f); v[e] = v[e] * v[e]; }
        store8(out + i * 8, v);
    }
}

ZI_EXPORT int zi_relu2(const void* x, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    if (total % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 31) == 0) {
        const long long want = (total / 8 + threads - 1) / threads;
        ZI_DISPATCH(dtype, T, { relu2_vec8_kernel<T><<<(int)(want > 148 * 32 ? 148 * 32 : want), threads, 0, stream>>>((const T*)x, (T*)out, (size_t)(total / 8)); });
        return zi_check_launch("relu2");
    }
    const long long want = (total + threads - 1) / threads;
    ZI_DISPATCH(dtype, T, { relu2_kernel<T><<<(int)(want > 148 * 16 ? 148 * 16 : want), threads, 0, stream>>>((const T*)x, (T*)out, (size_t)total); });
    return zi_check_launch("relu2");
}

// ---------------------------------------------------------------------------------------
// Clamped gated product.  x [rows, 2 * inter]: gate = x[n, j], up = x[n, inter + j];
//   g = min(gate, limit);  u = clamp(up, -limit, limit);  out[n, j] = g * sigmoid(slope * g) * (u + up_offset)
// limit <= 0: no clamping.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float clamped_gate(float g, float u, float limit, float slope, float up_offset) {
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return (g / (1.0f + expf(-slope * g))) * (u + up_offset);
}

template <typename T>
__global__ void gated_clamp_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, size_t total,
                                       float limit, float slope, float up_offset) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / inter, j = i - n * inter;
        out[i] = from_f32<T>(clamped_gate(to_f32<T>(x[n * 2 * inter + j]), to_f32<T>(x[n * 2 * inter + inter + j]),
                                          limit, slope, up_offset));
    }
}
template <typename T>
__global__ void gated_clamp_mul_vec8_kernel(const T* __restrict__ x, T* __restrict__ out, int inter8, size_t total8,
                                            float limit, float slope, float up_offset) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / inter8, j = (i - n * inter8) * 8;
        const size_t inter = (size_t)inter8 * 8;
        float g[8], u[8], r[8];
        load8(x + n * 2 * inter + j, g);
        load8(x + n * 2 * inter + inter + j, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = clamped_gate(g[e], u[e], limit, slope, up_offset);
        store8(out + n * inter + j, r);
    }
}

ZI_EXPORT int zi_gated_clamp_mul(const void* gate_up, void* out, int dtype, int rows, int inter, float limit, float slope,
                                 float up_offset, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0) return zi_fail("gated_clamp_mul: width %d must be positive", inter);
    const size_t total = (size_t)rows * inter;
    const int threads = 256;
    if (inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 31) == 0) {
        const size_t total8 = total / 8;
        const size_t want = (total8 + threads - 1) / threads;
        ZI_DISPATCH(dtype, T, {
            gated_clamp_mul_vec8_kernel<T><<<(int)(want > 148 * 32 ? 148 * 32 : want), threads, 0, stream>>>(
                (const T*)gate_up, (T*)out, inter / 8, total8, limit, slope, up_offset);
        });
        return zi_check_launch("gated_clamp_mul");
    }
    const size_t want = (total + threads - 1) / threads;
    ZI_DISPATCH(dtype, T, {
        gated_clamp_mul_kernel<T><<<(int)(want > 148 * 16 ? 148 * 16 : want), threads, 0, stream>>>(
            (const T*)gate_up, (T*)out, inter, total, limit, slope, up_offset);
    });
    return zi_check_launch("gated_clamp_mul");
}

// ---------------------------------------------------------------------------------------
// RMSNorm of `width` columns of each row of x, written into the pages of a paged cache with one
// plane and one head per token (a latent):  y = (w * x) * rstd,  rstd = 1/sqrt(mean(x^2) + eps).
//   x      [n_tokens, row_stride]; the first `width` columns of a row are normed
//   cache  one call's slice of the pool: row (page, off) is at cache + page*page_stride + off*width
//   tables [n_segments, max_blocks] page ids; tok_seg[n] = segment of token n; pos[n] = its position
// One warp per token; the sum's order depends on the width alone.
// ---------------------------------------------------------------------------------------
#define NA_WARPS 4
template <typename TX, typename TW, typename TC>
__global__ void __launch_bounds__(NA_WARPS * 32)
rmsnorm_append_kernel(const TX* __restrict__ x, long long row_stride, const TW* __restrict__ w, float eps,
                      TC* __restrict__ cache, const int* __restrict__ tables, const int* __restrict__ tok_seg,
                      const int* __restrict__ pos, int n_tokens, int width, int page_size, int max_blocks,
                      long long page_stride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * NA_WARPS + warp;
    if (n >= n_tokens) return;
    const TX* xr = x + (size_t)n * row_stride;
    float ss = 0.0f;
    for (int j = lane; j < width; j += 32) {
        const float v = to_f32<TX>(xr[j]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
    const int p = pos[n];
    const int seg = tok_seg ? tok_seg[n] : n;
    const int page = tables[(size_t)seg * max_blocks + p / page_size];
    TC* dst = cache + (long long)page * page_stride + (long long)(p % page_size) * width;
    for (int j = lane; j < width; j += 32) dst[j] = from_f32<TC>((to_f32<TW>(w[j]) * to_f32<TX>(xr[j])) * rstd);
}

ZI_EXPORT int zi_rmsnorm_append(const void* x, int x_dtype, long long row_stride, const void* w, int w_dtype, float eps,
                                void* cache, int cache_dtype, const int* tables, const int* tok_seg, const int* pos,
                                int n_tokens, int width, int page_size, int max_blocks, long long page_stride,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || row_stride < width) return zi_fail("rmsnorm_append: width=%d row_stride=%lld", width, row_stride);
    if (page_size <= 0 || max_blocks <= 0) return zi_fail("rmsnorm_append: page_size=%d max_blocks=%d", page_size, max_blocks);
    const int blocks = (n_tokens + NA_WARPS - 1) / NA_WARPS;
    ZI_DISPATCH(x_dtype, TX, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(cache_dtype, TC, {
        rmsnorm_append_kernel<TX, TW, TC><<<blocks, NA_WARPS * 32, 0, stream>>>(
            (const TX*)x, row_stride, (const TW*)w, eps, (TC*)cache, tables, tok_seg, pos, n_tokens, width, page_size,
            max_blocks, page_stride);
    });););
    return zi_check_launch("rmsnorm_append");
}

// ---------------------------------------------------------------------------------------
// Rotation by position of a span of every head, in either pairing, with the cache append of keys and values.
//   x       [n_tokens, ldx]: n_q query heads, then n_k key heads, then (v_mode 1) n_k value heads, head_dim each
//   span    entries rot_offset .. rot_offset + rot_dims - 1 of a head turn, the rest pass unchanged
//   pairing interleaved 0: entry i pairs with i + rot_dims / 2;  1: entry 2i with 2i + 1  (i < rot_dims / 2)
//           (lo, hi) -> (lo cos a - hi sin a, hi cos a + lo sin a),  a = float(pos) * inv_freq[i]
//   q_out   [n_tokens, ldq] receives the query heads (may be x itself: a pair is read and written by one thread)
//   cache   null, or a paged cache with two planes: rotated keys go to the first; the second receives the value heads
//           (v_mode 1) or the keys as they were before the rotation (v_mode 2: the values are the unrotated keys)
// One block per token; a thread takes a pair of the span or a single entry outside it.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void rotate_pair(float lo, float hi, float c, float s, float* olo, float* ohi) {
    *olo = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s));
    *ohi = __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s));
}

template <typename T>
__global__ void __launch_bounds__(256)
rotary_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ q_out, long long ldq, T* __restrict__ cache,
              const int* __restrict__ tables, const int* __restrict__ tok_seg, const int* __restrict__ pos,
              const float* __restrict__ inv_freq, int n_q, int n_k, int head_dim, int rot_offset, int rot_dims,
              int interleaved, int v_mode, int page_size, int max_blocks, long long page_stride, long long kv_stride) {
    extern __shared__ float cs[];            // cos[half], sin[half]
    const int n = blockIdx.x;
    const int half = rot_dims >> 1;
    const int p = pos[n];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)p * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    T* page_base = nullptr;
    if (cache) {
        const int seg = tok_seg ? tok_seg[n] : n;
        const int page = tables[(size_t)seg * max_blocks + p / page_size];
        page_base = cache + (size_t)page * page_stride + (size_t)(p % page_size) * head_dim;
    }
    const T* row = x + (size_t)n * ldx;
    const int per_head = head_dim - half;                      // pairs of the span, then the singles outside it
    const int heads = n_q + (cache ? n_k * (v_mode == 1 ? 2 : 1) : 0);
    for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
        const int h = idx / per_head, it = idx - h * per_head;
        const T* src = row + (size_t)h * head_dim;
        T* dst;
        T* raw = nullptr;                                      // where the unrotated copy of a key goes (v_mode 2)
        bool turn = true;
        if (h < n_q) {
            dst = q_out + (size_t)n * ldq + (size_t)h * head_dim;
        } else if (h < n_q + n_k) {
            dst = page_base + (size_t)(h - n_q) * page_size * head_dim;
            if (v_mode == 2) raw = dst + kv_stride;
        } else {
            dst = page_base + kv_stride + (size_t)(h - n_q - n_k) * page_size * head_dim;
            turn = false;
        }
        if (it < half) {
            const int lo_at = rot_offset + (interleaved ? 2 * it : it), hi_at = rot_offset + (interleaved ? 2 * it + 1 : it + half);
            const T lo_raw = src[lo_at], hi_raw = src[hi_at];
            if (raw) { raw[lo_at] = lo_raw; raw[hi_at] = hi_raw; }
            if (turn) {
                float olo, ohi;
                rotate_pair(to_f32<T>(lo_raw), to_f32<T>(hi_raw), cs[it], cs[half + it], &olo, &ohi);
                dst[lo_at] = from_f32<T>(olo);
                dst[hi_at] = from_f32<T>(ohi);
            } else {
                dst[lo_at] = lo_raw;
                dst[hi_at] = hi_raw;
            }
        } else {
            int d = it - half;                                 // the (it - half)-th entry outside the span
            if (d >= rot_offset) d += rot_dims;
            const T v = src[d];
            if (raw) raw[d] = v;
            if (dst != src) dst[d] = v;
        }
    }
}

// The same with 8 entries per access, where head size, span and its offset are multiples of 8 (16 for the span in the
// rotate-half pairing) and every row is aligned for it: a thread takes 8 neighbouring entries (interleaved pairing: four
// pairs inside them), or 8 entries of the span's first half and the 8 that pair with them, or 8 entries outside the span.
// The arithmetic per pair is rotate_pair as above: the same bits.
template <typename T>
__global__ void __launch_bounds__(256)
rotary_vec8_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ q_out, long long ldq, T* __restrict__ cache,
                   const int* __restrict__ tables, const int* __restrict__ tok_seg, const int* __restrict__ pos,
                   const float* __restrict__ inv_freq, int n_q, int n_k, int head_dim, int rot_offset, int rot_dims,
                   int interleaved, int v_mode, int page_size, int max_blocks, long long page_stride, long long kv_stride) {
    extern __shared__ float cs[];            // cos[half], sin[half]
    const int n = blockIdx.x;
    const int half = rot_dims >> 1;
    const int p = pos[n];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)p * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    T* page_base = nullptr;
    if (cache) {
        const int seg = tok_seg ? tok_seg[n] : n;
        const int page = tables[(size_t)seg * max_blocks + p / page_size];
        page_base = cache + (size_t)page * page_stride + (size_t)(p % page_size) * head_dim;
    }
    const T* row = x + (size_t)n * ldx;
    const int span_units = interleaved ? rot_dims >> 3 : half >> 3;
    const int units = span_units + ((head_dim - rot_dims) >> 3);
    const int heads = n_q + (cache ? n_k * (v_mode == 1 ? 2 : 1) : 0);
    for (int idx = threadIdx.x; idx < heads * units; idx += blockDim.x) {
        const int h = idx / units, u = idx - h * units;
        const T* src = row + (size_t)h * head_dim;
        T* dst;
        T* raw = nullptr;
        bool turn = true;
        if (h < n_q) {
            dst = q_out + (size_t)n * ldq + (size_t)h * head_dim;
        } else if (h < n_q + n_k) {
            dst = page_base + (size_t)(h - n_q) * page_size * head_dim;
            if (v_mode == 2) raw = dst + kv_stride;
        } else {
            dst = page_base + kv_stride + (size_t)(h - n_q - n_k) * page_size * head_dim;
            turn = false;
        }
        if (u >= span_units) {                                  // 8 entries outside the span
            int d = (u - span_units) * 8;
            if (d >= rot_offset) d += rot_dims;
            float v[8];
            load8(src + d, v);
            if (raw) store8(raw + d, v);
            if (dst != src) store8(dst + d, v);
        } else if (interleaved) {                               // four pairs inside 8 neighbouring entries
            const int d = rot_offset + u * 8, i0 = u * 4;
            float v[8], o[8];
            load8(src + d, v);
            if (raw) store8(raw + d, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (turn) rotate_pair(v[2 * k], v[2 * k + 1], cs[i0 + k], cs[half + i0 + k], &o[2 * k], &o[2 * k + 1]);
                else { o[2 * k] = v[2 * k]; o[2 * k + 1] = v[2 * k + 1]; }
            }
            // what the scalar kernel stores is the rounded value; store8 rounds the same way
            store8(dst + d, o);
        } else {                                                // 8 entries of the first half and their partners
            const int lo_at = rot_offset + u * 8, hi_at = lo_at + half, i0 = u * 8;
            float a[8], b[8], lo[8], hi[8];
            load8(src + lo_at, a);
            load8(src + hi_at, b);
            if (raw) { store8(raw + lo_at, a); store8(raw + hi_at, b); }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (turn) rotate_pair(a[k], b[k], cs[i0 + k], cs[half + i0 + k], &lo[k], &hi[k]);
                else { lo[k] = a[k]; hi[k] = b[k]; }
            }
            store8(dst + lo_at, lo);
            store8(dst + hi_at, hi);
        }
    }
}

ZI_EXPORT int zi_rotary(const void* x, int dtype, long long ldx, void* q_out, long long ldq, void* cache, const int* tables,
                        const int* tok_seg, const int* pos, const float* inv_freq, int n_tokens, int n_q, int n_k, int head_dim,
                        int rot_offset, int rot_dims, int interleaved, int v_mode, int page_size, int max_blocks,
                        long long page_stride, long long kv_stride, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_offset < 0 || rot_offset + rot_dims > head_dim)
        return zi_fail("rotary: a span of %d entries from %d does not fit a head of %d (or is odd)", rot_dims, rot_offset, head_dim);
    if (n_q < 0 || n_k < 0 || v_mode < 0 || v_mode > 2) return zi_fail("rotary: bad head counts or value mode");
    if (cache && (page_size <= 0 || max_blocks <= 0 || !tables)) return zi_fail("rotary: the cache append needs tables and a page size");
    if (cache && v_mode == 2 && kv_stride == 0) return zi_fail("rotary: unrotated keys as values need a second plane");
    const size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float);
    const size_t align = dtype == ZI_BF16 ? 16 : 32;
    const bool vec8 = head_dim % 8 == 0 && rot_offset % 8 == 0 && rot_dims % (interleaved ? 8 : 16) == 0 && ldx % 8 == 0 && ldq % 8 == 0 &&
                      ((uintptr_t)x % align) == 0 && ((uintptr_t)q_out % align) == 0 &&
                      (!cache || (((uintptr_t)cache % align) == 0 && page_stride % 8 == 0 && kv_stride % 8 == 0));
    if (vec8) {
        ZI_DISPATCH(dtype, T, {
            rotary_vec8_kernel<T><<<n_tokens, 128, smem, stream>>>((const T*)x, ldx, (T*)q_out, ldq, (T*)cache, tables, tok_seg, pos,
                                                                   inv_freq, n_q, n_k, head_dim, rot_offset, rot_dims, interleaved, v_mode,
                                                                   page_size, max_blocks, page_stride, kv_stride);
        });
        return zi_check_launch("rotary");
    }
    ZI_DISPATCH(dtype, T, {
        rotary_kernel<T><<<n_tokens, 256, smem, stream>>>((const T*)x, ldx, (T*)q_out, ldq, (T*)cache, tables, tok_seg, pos, inv_freq,
                                                          n_q, n_k, head_dim, rot_offset, rot_dims, interleaved, v_mode, page_size,
                                                          max_blocks, page_stride, kv_stride);
    });
    return zi_check_launch("rotary");
}

// ---------------------------------------------------------------------------------------
// The latents of a latent-attention layer whose keys carry a rotated part, from one row of a stacked product:
//   cq_out[n, :]              = rmsnorm(x[n, q_off .. q_off + q_rank)) * gq               (q_rank 0: no query latent)
//   cache row of token n      = [ rmsnorm(x[n, c_off .. c_off + rank)) * gc | turn(x[n, c_off + rank .. + rot_dim)) | 0 .. ]
// The cache has one plane and one head of `row_width` >= rank + rot_dim entries per token; what lies behind rank + rot_dim is
// never written (the pool is zeroed when it is made).  The turned part: the first rot_dims of its rot_dim entries, paired as
// in rotary_kernel.  One block per token.
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ x, long long ldx, int q_off, int q_rank, const TW* __restrict__ gq,
                      T* __restrict__ cq_out, int c_off, int rank, const TW* __restrict__ gc, int rot_dim, int rot_dims,
                      int interleaved, const float* __restrict__ inv_freq, float eps, T* __restrict__ cache, int row_width,
                      const int* __restrict__ tables, const int* __restrict__ tok_seg, const int* __restrict__ pos,
                      int page_size, int max_blocks, long long page_stride) {
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    const T* xr = x + (size_t)n * ldx;
    if (q_rank > 0) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < q_rank; j += blockDim.x) {
            const float v = to_f32<T>(xr[q_off + j]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
            cq_out[(size_t)n * q_rank + j] = from_f32<T>((to_f32<TW>(gq[j]) * to_f32<T>(xr[q_off + j])) * rstd);
    }
    if (!cache) return;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) {
        const float v = to_f32<T>(xr[c_off + j]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)rank + eps);
    const int p = pos[n];
    const int seg = tok_seg ? tok_seg[n] : n;
    const int page = tables[(size_t)seg * max_blocks + p / page_size];
    T* dst = cache + (long long)page * page_stride + (long long)(p % page_size) * row_width;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) dst[j] = from_f32<T>((to_f32<TW>(gc[j]) * to_f32<T>(xr[c_off + j])) * rstd);
    const int half = rot_dims >> 1;
    const T* kr = xr + c_off + rank;
    for (int it = threadIdx.x; it < rot_dim - half; it += blockDim.x) {
        if (it < half) {
            const int lo_at = interleaved ? 2 * it : it, hi_at = interleaved ? 2 * it + 1 : it + half;
            float s, c, olo, ohi;
            sincosf((float)p * inv_freq[it], &s, &c);
            rotate_pair(to_f32<T>(kr[lo_at]), to_f32<T>(kr[hi_at]), c, s, &olo, &ohi);
            dst[rank + lo_at] = from_f32<T>(olo);
            dst[rank + hi_at] = from_f32<T>(ohi);
        } else {
            const int d = it - half + rot_dims;
            dst[rank + d] = kr[d];
        }
    }
}

ZI_EXPORT int zi_latent_prepare(const void* x, int dtype, long long ldx, int q_off, int q_rank, const void* gq, void* cq_out,
                                int c_off, int rank, const void* gc, int w_dtype, int rot_dim, int rot_dims, int interleaved,
                                const float* inv_freq, float eps, void* cache, int row_width, const int* tables,
                                const int* tok_seg, const int* pos, int n_tokens, int page_size, int max_blocks,
                                long long page_stride, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (q_rank < 0 || rank <= 0 || rot_dim < 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > rot_dim)
        return zi_fail("latent_prepare: q_rank=%d rank=%d rot_dim=%d rot_dims=%d", q_rank, rank, rot_dim, rot_dims);
    if (cache && (row_width < rank + rot_dim || page_size <= 0 || max_blocks <= 0))
        return zi_fail("latent_prepare: a cache row of %d entries cannot hold %d + %d", row_width, rank, rot_dim);
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        latent_prepare_kernel<T, TW><<<n_tokens, 128, 0, stream>>>((const T*)x, ldx, q_off, q_rank, (const TW*)gq, (T*)cq_out, c_off,
                                                                   rank, (const TW*)gc, rot_dim, rot_dims, interleaved, inv_freq, eps,
                                                                   (T*)cache, row_width, tables, tok_seg, pos, page_size, max_blocks,
                                                                   page_stride);
    }););
    return zi_check_launch("latent_prepare");
}

// ---------------------------------------------------------------------------------------
// Output gate: a[n, j] *= sigmoid(g[n, j]), float32 inside; the rows of g may be strided (a slice of a wider product).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ a, const T* __restrict__ g, long long ldg, int width, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / width;
        const int j = (int)(i - n * width);
        const float gv = to_f32<T>(g[n * ldg + j]);
        a[i] = from_f32<T>(to_f32<T>(a[i]) / (1.0f + expf(-gv)));
    }
}

ZI_EXPORT int zi_sigmoid_mul(void* a, const void* g, int dtype, long long ldg, int rows, int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    const size_t total = (size_t)rows * width;
    const size_t want = (total + 255) / 256;
    ZI_DISPATCH(dtype, T, {
        sigmoid_mul_kernel<T><<<(int)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>((T*)a, (const T*)g, ldg, width, total);
    });
    return zi_check_launch("sigmoid_mul");
}

// ---------------------------------------------------------------------------------------
// Rotation by position of the first rot_dims entries of every query and key head, with a factor on cosines and sines,
// then (unit_norm) every query and key head divided by its root mean square over its qk_dim entries, then the append
// of keys and values to a paged cache whose rows are row_dim wide (row_dim >= qk_dim, v_dim; what lies past a head's own
// entries is written as zero).
//   x       [n_tokens, ldx]: n_q query heads and n_k key heads of qk_dim entries, then n_k value heads of v_dim entries
//   pairing as in rotary_kernel;  the angle of pair i is float(pos) * inv_freq[i], cos and sin are multiplied by mag
//   q_out   [n_tokens, n_q * row_dim]
//   cache   null (queries alone: n_k is then 0), or two planes: keys after turn and norm, and the values
// One block per token, one warp per head at a time; a head passes through the warp's stretch of shared memory, so the
// sum of squares has one order whatever the step.
// ---------------------------------------------------------------------------------------
#define RN_WARPS 8
template <typename T>
__global__ void __launch_bounds__(RN_WARPS * 32)
rotary_norm_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ tables,
                   const int* __restrict__ tok_seg, const int* __restrict__ pos, const float* __restrict__ inv_freq, float mag,
                   const float* __restrict__ q_head_scale, int n_q, int n_k, int qk_dim, int v_dim, int row_dim, int rot_dims, int interleaved, int unit_norm, float eps,
                   int page_size, int max_blocks, long long page_stride, long long kv_stride) {
    extern __shared__ float rn_smem[];       // cos[half], sin[half], then a head per warp
    const int n = blockIdx.x, half = rot_dims >> 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* cs = rn_smem;
    float* head = rn_smem + rot_dims + warp * qk_dim;
    const int p = pos[n];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)p * inv_freq[i], &s, &c);
        cs[i] = c * mag;
        cs[half + i] = s * mag;
    }
    __syncthreads();
    T* page_base = nullptr;
    if (cache) {
        const int seg = tok_seg ? tok_seg[n] : n;
        const int page = tables[(size_t)seg * max_blocks + p / page_size];
        page_base = cache + (size_t)page * page_stride + (size_t)(p % page_size) * row_dim;
    }
    const T* row = x + (size_t)n * ldx;
    const int heads = n_q + (cache ? 2 * n_k : 0);
    for (int h = warp; h < heads; h += RN_WARPS) {
        if (h >= n_q + n_k) {                                   // a value head: copied, padded with zeros
            const int g = h - n_q - n_k;
            const T* src = row + (size_t)(n_q + n_k) * qk_dim + (size_t)g * v_dim;
            T* dst = page_base + kv_stride + (size_t)g * page_size * row_dim;
            for (int d = lane; d < row_dim; d += 32) dst[d] = d < v_dim ? src[d] : from_f32<T>(0.0f);
            continue;
        }
        const T* src = row + (size_t)h * qk_dim;
        T* dst = h < n_q ? q_out + ((size_t)n * n_q + h) * row_dim : page_base + (size_t)(h - n_q) * page_size * row_dim;
        float ss = 0.0f;
        for (int it = lane; it < qk_dim - half; it += 32) {
            if (it < half) {
                const int lo_at = interleaved ? 2 * it : it, hi_at = interleaved ? 2 * it + 1 : it + half;
                float olo, ohi;
                rotate_pair(to_f32<T>(src[lo_at]), to_f32<T>(src[hi_at]), cs[it], cs[half + it], &olo, &ohi);
                head[lo_at] = olo;
                head[hi_at] = ohi;
            } else {
                const int d = it - half + rot_dims;
                head[d] = to_f32<T>(src[d]);
            }
        }
        __syncwarp();
        float r = 1.0f;
        if (unit_norm) {
            for (int d = lane; d < qk_dim; d += 32) ss = fmaf(head[d], head[d], ss);
            ss = warp_sum(ss);
            r = 1.0f / sqrtf(ss / (float)qk_dim + eps);
        }
        if (q_head_scale && h < n_q) r *= q_head_scale[h];         // a query head's own factor on its scores
        for (int d = lane; d < row_dim; d += 32) dst[d] = from_f32<T>(d < qk_dim ? head[d] * r : 0.0f);
        __syncwarp();
    }
}

ZI_EXPORT int zi_rotary_norm(const void* x, int dtype, long long ldx, void* q_out, void* cache, const int* tables, const int* tok_seg,
                             const int* pos, const float* inv_freq, float mag, const float* q_head_scale, int n_tokens, int n_q, int n_k,
                             int qk_dim, int v_dim,
                             int row_dim, int rot_dims, int interleaved, int unit_norm, float eps, int page_size, int max_blocks,
                             long long page_stride, long long kv_stride, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (qk_dim <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > qk_dim)
        return zi_fail("rotary_norm: a span of %d entries does not fit a head of %d (or is odd)", rot_dims, qk_dim);
    if (row_dim < qk_dim || (cache && row_dim < v_dim)) return zi_fail("rotary_norm: rows of %d entries cannot hold heads of %d and %d", row_dim, qk_dim, v_dim);
    if (n_q < 0 || n_k < 0) return zi_fail("rotary_norm: bad head counts");
    if (cache && (page_size <= 0 || max_blocks <= 0 || !tables || kv_stride == 0))
        return zi_fail("rotary_norm: the cache append needs tables, a page size and two planes");
    if (rot_dims > 0 && !inv_freq) return zi_fail("rotary_norm: a turned span needs its frequencies");
    const size_t smem = (size_t)(rot_dims + RN_WARPS * qk_dim) * sizeof(float);
    if (smem > 48 * 1024) return zi_fail("rotary_norm: heads of %d entries are too wide", qk_dim);
    ZI_DISPATCH(dtype, T, {
        rotary_norm_kernel<T><<<n_tokens, RN_WARPS * 32, smem, stream>>>((const T*)x, ldx, (T*)q_out, (T*)cache, tables, tok_seg, pos,
                                                                         inv_freq, mag, q_head_scale, n_q, n_k, qk_dim, v_dim, row_dim, rot_dims,
                                                                         interleaved, unit_norm, eps, page_size, max_blocks, page_stride,
                                                                         kv_stride);
    });
    return zi_check_launch("rotary_norm");
}

// ---------------------------------------------------------------------------------------
// A branch's output, normed, joins the float32 residual stream:  h[n, :] += y[n, :] / sqrt(mean(y[n]^2) + eps) * w.
// rounded (optional, of the step's type) receives the new h, which the next sublayer reads.  One block per row.
// ---------------------------------------------------------------------------------------
#define NA_THREADS 256
template <typename T, typename TW>
__global__ void __launch_bounds__(NA_THREADS)
norm_add_kernel(float* __restrict__ h, const T* __restrict__ y, const TW* __restrict__ w, T* __restrict__ rounded, float eps, int hidden) {
    extern __shared__ float na_row[];
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    const T* yr = y + n * hidden;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = to_f32<T>(yr[j]);
        na_row[j] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    float* hr = h + n * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = hr[j] + (na_row[j] * r) * to_f32<TW>(w[j]);
        hr[j] = v;
        if (rounded) rounded[n * hidden + j] = from_f32<T>(v);
    }
}

// The same with eight entries per access; hidden a multiple of 8 and every pointer on a 16-byte boundary.
template <typename T, typename TW>
__global__ void __launch_bounds__(NA_THREADS)
norm_add_vec8_kernel(float* __restrict__ h, const T* __restrict__ y, const TW* __restrict__ w, T* __restrict__ rounded, float eps, int hidden) {
    extern __shared__ float na_row[];
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    const T* yr = y + n * hidden;
    float ss = 0.0f;
    for (int j = threadIdx.x * 8; j < hidden; j += NA_THREADS * 8) {
        float v[8];
        load8(yr + j, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
        store8(na_row + j, v);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    float* hr = h + n * hidden;
    for (int j = threadIdx.x * 8; j < hidden; j += NA_THREADS * 8) {
        float v[8], a[8], g[8];
        load8(na_row + j, v);
        load8(hr + j, a);
        load8(w + j, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] + (v[e] * r) * g[e];
        store8(hr + j, a);
        if (rounded) store8(rounded + n * hidden + j, a);
    }
}

ZI_EXPORT int zi_norm_add(float* h, const void* y, int dtype, const void* w, int w_dtype, void* rounded, float eps, int rows, int hidden,
                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || (size_t)hidden * sizeof(float) > 48 * 1024) return zi_fail("norm_add: hidden=%d is not supported", hidden);
    // which form runs depends on the sizes and on where the buffers start, never on the rows of the step
    const bool vec = hidden % 8 == 0 && (((size_t)h | (size_t)y | (size_t)w | (size_t)rounded) & 15) == 0;
    if (vec) {
        ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
            norm_add_vec8_kernel<T, TW><<<rows, NA_THREADS, (size_t)hidden * sizeof(float), stream>>>(h, (const T*)y, (const TW*)w, (T*)rounded,
                                                                                                    eps, hidden);
        }););
        return zi_check_launch("norm_add");
    }
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        norm_add_kernel<T, TW><<<rows, NA_THREADS, (size_t)hidden * sizeof(float), stream>>>(h, (const T*)y, (const TW*)w, (T*)rounded, eps,
                                                                                           hidden);
    }););
    return zi_check_launch("norm_add");
}

// ---------------------------------------------------------------------------------------
// A gate on a token's own table entry:  out[n, j] = gelu_tanh(t[n, j]) * table[ids[n], col0 + j],  j < width, with
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), float32 inside.  Rows of t may be strided.
// ---------------------------------------------------------------------------------------
template <typename T, typename TT>
__global__ void gelu_mul_rows_kernel(const T* __restrict__ t, long long ldt, const TT* __restrict__ table, long long ld_table, int col0,
                                     const int* __restrict__ ids, int vocab, T* __restrict__ out, int width, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / width;
        const int j = (int)(i - n * width);
        int id = ids[n];
        id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
        const float z = to_f32<T>(t[n * ldt + j]);
        const float g = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        out[i] = from_f32<T>(g * to_f32<TT>(table[(size_t)id * ld_table + col0 + j]));
    }
}

ZI_EXPORT int zi_gelu_mul_rows(const void* t, int dtype, long long ldt, const void* table, int table_dtype, long long ld_table, int col0,
                               const int* ids, int vocab, void* out, int rows, int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    if (vocab <= 0 || col0 < 0 || col0 + width > ld_table) return zi_fail("gelu_mul_rows: columns %d .. %d do not lie in a table row of %lld", col0, col0 + width, ld_table);
    const size_t total = (size_t)rows * width;
    const size_t want = (total + 255) / 256;
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(table_dtype, TT, {
        gelu_mul_rows_kernel<T, TT><<<(int)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>((const T*)t, ldt, (const TT*)table, ld_table,
                                                                                                 col0, ids, vocab, (T*)out, width, total);
    }););
    return zi_check_launch("gelu_mul_rows");
}

// ---------------------------------------------------------------------------------------
// The tanh norm  N(v; a, w, b) = tanh(a v) * w + b  (a scalar a, vectors w and b; no mean, no variance) around the float32
// residual stream, for layers with a norm before and a norm after every sublayer:
//     v = h[row] + N(y[row]; post)        where a branch's output y is pending (y null: v = h[row])
//     h[row] = v                          where write_h is set
//     out[r] = N(v; pre)                  where out is given
// row = row_idx[r] where row_idx is given (then h is not written), else r.  h float32; y and out of the step's type; w, b
// float32.  Entry by entry, so a row's result depends on nothing else.
// ---------------------------------------------------------------------------------------
// Three block sums at once; scratch holds at least 96 floats.  The order of additions depends on the block size alone.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    __syncthreads();
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; scratch[64 + warp] = c; }
    __syncthreads();
    a = warp_sum(lane < nwarps ? scratch[lane] : 0.0f);
    b = warp_sum(lane < nwarps ? scratch[32 + lane] : 0.0f);
    c = warp_sum(lane < nwarps ? scratch[64 + lane] : 0.0f);
}

struct TanhNormArgs { float a; const float* w; const float* b; };

template <typename T>
__global__ void __launch_bounds__(256)
tanh_norm_fold_kernel(float* __restrict__ h, const T* __restrict__ y, TanhNormArgs post, TanhNormArgs pre, T* __restrict__ out,
                      const int* __restrict__ row_idx, int write_h, int hidden) {
    const size_t r = blockIdx.x, row = row_idx ? (size_t)row_idx[r] : r;
    float* hr = h + row * hidden;
    const T* yr = y ? y + row * hidden : nullptr;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = hr[j];
        if (yr) v += tanhf(post.a * to_f32<T>(yr[j])) * post.w[j] + post.b[j];
        if (write_h) hr[j] = v;
        if (out) out[r * hidden + j] = from_f32<T>(tanhf(pre.a * v) * pre.w[j] + pre.b[j]);
    }
}

// The same with eight entries per access; hidden a multiple of 8 and every pointer on a 32-byte boundary.
template <typename T>
__global__ void __launch_bounds__(256)
tanh_norm_fold_vec8_kernel(float* __restrict__ h, const T* __restrict__ y, TanhNormArgs post, TanhNormArgs pre, T* __restrict__ out,
                           const int* __restrict__ row_idx, int write_h, int hidden) {
    const size_t r = blockIdx.x, row = row_idx ? (size_t)row_idx[r] : r;
    float* hr = h + row * hidden;
    const T* yr = y ? y + row * hidden : nullptr;
    for (int j = threadIdx.x * 8; j < hidden; j += blockDim.x * 8) {
        float v[8];
        load8(hr + j, v);
        if (yr) {
            float t[8], w[8], b[8];
            load8(yr + j, t); load8(post.w + j, w); load8(post.b + j, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] += tanhf(post.a * t[e]) * w[e] + b[e];
        }
        if (write_h) store8(hr + j, v);
        if (out) {
            float w[8], b[8], o[8];
            load8(pre.w + j, w); load8(pre.b + j, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = tanhf(pre.a * v[e]) * w[e] + b[e];
            store8(out + r * hidden + j, o);
        }
    }
}

ZI_EXPORT int zi_tanh_norm_fold(float* h, const void* y, int dtype, float post_a, const float* post_w, const float* post_b, float pre_a,
                                const float* pre_w, const float* pre_b, void* out, const int* row_idx, int rows, int hidden, int write_h,
                                cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0) return zi_fail("tanh_norm_fold: hidden=%d", hidden);
    if (y && (!post_w || !post_b)) return zi_fail("tanh_norm_fold: a pending branch needs the norm that follows it");
    if (out && (!pre_w || !pre_b)) return zi_fail("tanh_norm_fold: an output needs the norm that makes it");
    if (row_idx && write_h) return zi_fail("tanh_norm_fold: chosen rows leave the stream as it is");
    const TanhNormArgs post{post_a, post_w, post_b}, pre{pre_a, pre_w, pre_b};
    const int threads = hidden >= 2048 ? 256 : 128;
    // which form runs depends on the sizes and on where the buffers start, never on the rows of the step
    const bool vec = hidden % 8 == 0 && (((size_t)h | (size_t)y | (size_t)out | (size_t)post_w | (size_t)post_b | (size_t)pre_w | (size_t)pre_b) & 31) == 0;
    ZI_DISPATCH(dtype, T, {
        if (vec) tanh_norm_fold_vec8_kernel<T><<<rows, threads, 0, stream>>>(h, (const T*)y, post, pre, (T*)out, row_idx, write_h, hidden);
        else tanh_norm_fold_kernel<T><<<rows, threads, 0, stream>>>(h, (const T*)y, post, pre, (T*)out, row_idx, write_h, hidden);
    });
    return zi_check_launch("tanh_norm_fold");
}

// The same fold for a pending output of two branches that read the same input and are joined on the way:
//     y = (U(y1) * w1 + U(y2) * w2) / 2,   U(v) = v / sqrt(mean(v^2) + eps) over the row;   v = h[row] + N(y; post);  ...
// One block per row; the joined row never leaves the chip.
template <typename T>
__global__ void __launch_bounds__(256)
tanh_norm_fold_pair_kernel(float* __restrict__ h, const T* __restrict__ y1, const T* __restrict__ y2, const float* __restrict__ w1,
                           const float* __restrict__ w2, float eps, TanhNormArgs post, TanhNormArgs pre, T* __restrict__ out,
                           const int* __restrict__ row_idx, int write_h, int hidden) {
    extern __shared__ float fp_row[];                    // y1's row, then y2's
    __shared__ float scratch[96];
    const size_t r = blockIdx.x, row = row_idx ? (size_t)row_idx[r] : r;
    float s1 = 0.0f, s2 = 0.0f, unused = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float a = to_f32<T>(y1[row * hidden + j]), b = to_f32<T>(y2[row * hidden + j]);
        fp_row[j] = a; fp_row[hidden + j] = b;
        s1 = fmaf(a, a, s1); s2 = fmaf(b, b, s2);
    }
    block_sum3(s1, s2, unused, scratch);
    const float r1 = 1.0f / sqrtf(s1 / (float)hidden + eps), r2 = 1.0f / sqrtf(s2 / (float)hidden + eps);
    float* hr = h + row * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float joined = 0.5f * ((fp_row[j] * r1) * w1[j] + (fp_row[hidden + j] * r2) * w2[j]);
        const float v = hr[j] + (tanhf(post.a * joined) * post.w[j] + post.b[j]);
        if (write_h) hr[j] = v;
        if (out) out[r * hidden + j] = from_f32<T>(tanhf(pre.a * v) * pre.w[j] + pre.b[j]);
    }
}

// The same with eight entries per access and C such groups per thread (hidden <= 2048 C, a multiple of 8; every pointer on a
// 32-byte boundary).  Everything a thread needs (its entries of both branches, of the stream and of the five vectors) is asked
// for before the block's sums are taken, so the sums wait for memory once and the rest finds its operands on the chip.
template <typename T, int C>
__global__ void __launch_bounds__(256)
tanh_norm_fold_pair_vec8_kernel(float* __restrict__ h, const T* __restrict__ y1, const T* __restrict__ y2, const float* __restrict__ w1,
                                const float* __restrict__ w2, float eps, TanhNormArgs post, TanhNormArgs pre, T* __restrict__ out,
                                const int* __restrict__ row_idx, int write_h, int hidden) {
    __shared__ float scratch[96];
    const size_t r = blockIdx.x, row = row_idx ? (size_t)row_idx[r] : r;
    float a[C][8], b[C][8], hv[C][8], g1[C][8], g2[C][8], pw[C][8], pb[C][8];
    float s1 = 0.0f, s2 = 0.0f, unused = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int j = (c * 256 + threadIdx.x) * 8;
        if (j < hidden) {
            load8(y1 + row * hidden + j, a[c]); load8(y2 + row * hidden + j, b[c]); load8(h + row * hidden + j, hv[c]);
            load8(w1 + j, g1[c]); load8(w2 + j, g2[c]); load8(post.w + j, pw[c]); load8(post.b + j, pb[c]);
#pragma unroll
            for (int e = 0; e < 8; ++e) { s1 = fmaf(a[c][e], a[c][e], s1); s2 = fmaf(b[c][e], b[c][e], s2); }
        }
    }
    block_sum3(s1, s2, unused, scratch);
    const float r1 = 1.0f / sqrtf(s1 / (float)hidden + eps), r2 = 1.0f / sqrtf(s2 / (float)hidden + eps);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int j = (c * 256 + threadIdx.x) * 8;
        if (j < hidden) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float joined = 0.5f * ((a[c][e] * r1) * g1[c][e] + (b[c][e] * r2) * g2[c][e]);
                v[e] = hv[c][e] + (tanhf(post.a * joined) * pw[c][e] + pb[c][e]);
            }
            if (write_h) store8(h + row * hidden + j, v);
            if (out) {
                float qw[8], qb[8], o[8];
                load8(pre.w + j, qw); load8(pre.b + j, qb);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = tanhf(pre.a * v[e]) * qw[e] + qb[e];
                store8(out + r * hidden + j, o);
            }
        }
    }
}

ZI_EXPORT int zi_tanh_norm_fold_pair(float* h, const void* y1, const void* y2, int dtype, const float* w1, const float* w2, float eps, float post_a,
                                     const float* post_w, const float* post_b, float pre_a, const float* pre_w, const float* pre_b, void* out,
                                     const int* row_idx, int rows, int hidden, int write_h, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || (size_t)hidden * 2 * sizeof(float) > 48 * 1024) return zi_fail("tanh_norm_fold_pair: hidden=%d is not supported", hidden);
    if (!y1 || !y2 || !w1 || !w2 || !post_w || !post_b) return zi_fail("tanh_norm_fold_pair: two branches, their weights and the norm that follows are needed");
    if (out && (!pre_w || !pre_b)) return zi_fail("tanh_norm_fold_pair: an output needs the norm that makes it");
    if (row_idx && write_h) return zi_fail("tanh_norm_fold_pair: chosen rows leave the stream as it is");
    const TanhNormArgs post{post_a, post_w, post_b}, pre{pre_a, pre_w, pre_b};
    // which form runs depends on the sizes and on where the buffers start, never on the rows of the step
    const bool vec = hidden % 8 == 0 && hidden <= 3 * 2048 &&
                     (((size_t)h | (size_t)y1 | (size_t)y2 | (size_t)out | (size_t)w1 | (size_t)w2 | (size_t)post_w | (size_t)post_b |
                       (size_t)pre_w | (size_t)pre_b) & 31) == 0;
    ZI_DISPATCH(dtype, T, {
        if (vec && hidden <= 2048)
            tanh_norm_fold_pair_vec8_kernel<T, 1><<<rows, 256, 0, stream>>>(h, (const T*)y1, (const T*)y2, w1, w2, eps, post, pre, (T*)out, row_idx, write_h, hidden);
        else if (vec && hidden <= 4096)
            tanh_norm_fold_pair_vec8_kernel<T, 2><<<rows, 256, 0, stream>>>(h, (const T*)y1, (const T*)y2, w1, w2, eps, post, pre, (T*)out, row_idx, write_h, hidden);
        else if (vec)
            tanh_norm_fold_pair_vec8_kernel<T, 3><<<rows, 256, 0, stream>>>(h, (const T*)y1, (const T*)y2, w1, w2, eps, post, pre, (T*)out, row_idx, write_h, hidden);
        else
            tanh_norm_fold_pair_kernel<T><<<rows, hidden >= 2048 ? 256 : 128, (size_t)hidden * 2 * sizeof(float), stream>>>(
                h, (const T*)y1, (const T*)y2, w1, w2, eps, post, pre, (T*)out, row_idx, write_h, hidden);
    });
    return zi_check_launch("tanh_norm_fold_pair");
}

// out = tanh(a x) * w + b for rows of any of the two types (a norm called on its own).
template <typename TX, typename T>
__global__ void tanh_norm_kernel(const TX* __restrict__ x, TanhNormArgs nm, T* __restrict__ out, int hidden, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % hidden);
        out[i] = from_f32<T>(tanhf(nm.a * to_f32<TX>(x[i])) * nm.w[j] + nm.b[j]);
    }
}

ZI_EXPORT int zi_tanh_norm(const void* x, int x_dtype, float a, const float* w, const float* b, void* out, int dtype, int rows, int hidden,
                           cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || !w || !b) return zi_fail("tanh_norm: hidden=%d, weight and bias are needed", hidden);
    const size_t total = (size_t)rows * hidden, want = (total + 255) / 256;
    const TanhNormArgs nm{a, w, b};
    ZI_DISPATCH(x_dtype, TX, ZI_DISPATCH(dtype, T, {
        tanh_norm_kernel<TX, T><<<(int)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>((const TX*)x, nm, (T*)out, hidden, total);
    }););
    return zi_check_launch("tanh_norm");
}

// ---------------------------------------------------------------------------------------
// Two branches that read the same input, joined:  out = (U(x) * wx + U(z) * wz) / 2  with U(v) = v / sqrt(mean(v^2) + eps)
// over a row, float32 inside; wx, wz float32.  One block per row.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rms_pair_mean_kernel(const T* __restrict__ x, const T* __restrict__ z, const float* __restrict__ wx, const float* __restrict__ wz,
                     T* __restrict__ out, float eps, int hidden) {
    extern __shared__ float pm_row[];                    // x's row, then z's
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    float sx = 0.0f, sz = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float a = to_f32<T>(x[n * hidden + j]), b = to_f32<T>(z[n * hidden + j]);
        pm_row[j] = a; pm_row[hidden + j] = b;
        sx = fmaf(a, a, sx); sz = fmaf(b, b, sz);
    }
    sx = block_sum(sx, scratch);
    sz = block_sum(sz, scratch);
    const float rx = 1.0f / sqrtf(sx / (float)hidden + eps), rz = 1.0f / sqrtf(sz / (float)hidden + eps);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        out[n * hidden + j] = from_f32<T>(0.5f * ((pm_row[j] * rx) * wx[j] + (pm_row[hidden + j] * rz) * wz[j]));
}

ZI_EXPORT int zi_rms_pair_mean(const void* x, const void* z, int dtype, const float* wx, const float* wz, void* out, float eps, int rows,
                               int hidden, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || (size_t)hidden * 2 * sizeof(float) > 48 * 1024) return zi_fail("rms_pair_mean: hidden=%d is not supported", hidden);
    ZI_DISPATCH(dtype, T, {
        rms_pair_mean_kernel<T><<<rows, hidden >= 2048 ? 256 : 128, (size_t)hidden * 2 * sizeof(float), stream>>>(
            (const T*)x, (const T*)z, wx, wz, (T*)out, eps, hidden);
    });
    return zi_check_launch("rms_pair_mean");
}

// ---------------------------------------------------------------------------------------
// A feed-forward activation from powers of its input, each divided by its own root mean square over the row:
//     out = c1 U(z) + c2 U(z^2) + c3 U(z^3) + c0,   U(v) = v / sqrt(mean(v^2) + eps),  powers entry by entry
// float32 inside.  One block per row; rows of z may be strided.
// ---------------------------------------------------------------------------------------
// Eight entries per access: width and ldz multiples of 8, pointers on 16-byte boundaries.  The sums run per thread over its
// own entries in rising order and then over the block, as in the scalar form but dealt otherwise: which form runs depends on
// the sizes and on where the buffers start, never on the rows of the step.
template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_vec8_kernel(const T* __restrict__ z, long long ldz, T* __restrict__ out, int width, float c1, float c2, float c3, float c0, float eps) {
    extern __shared__ __align__(16) float pn_row[];
    __shared__ float scratch[96];
    const size_t n = blockIdx.x;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int j = threadIdx.x * 8; j < width; j += blockDim.x * 8) {
        float v[8];
        load8(z + n * ldz + j, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v2 = v[e] * v[e], v3 = v2 * v[e];
            s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6);
        }
        store8(pn_row + j, v);
    }
    block_sum3(s2, s4, s6, scratch);
    const float r1 = 1.0f / sqrtf(s2 / (float)width + eps), r2 = 1.0f / sqrtf(s4 / (float)width + eps), r3 = 1.0f / sqrtf(s6 / (float)width + eps);
    for (int j = threadIdx.x * 8; j < width; j += blockDim.x * 8) {
        float v[8], o[8];
        load8(pn_row + j, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v2 = v[e] * v[e], v3 = v2 * v[e];
            o[e] = c1 * (v[e] * r1) + c2 * (v2 * r2) + c3 * (v3 * r3) + c0;
        }
        store8(out + n * width + j, o);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_kernel(const T* __restrict__ z, long long ldz, T* __restrict__ out, int width, float c1, float c2, float c3, float c0, float eps) {
    extern __shared__ __align__(16) float pn_row[];
    __shared__ float scratch[96];
    const size_t n = blockIdx.x;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = to_f32<T>(z[n * ldz + j]), v2 = v * v, v3 = v2 * v;
        pn_row[j] = v;
        s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6);
    }
    block_sum3(s2, s4, s6, scratch);
    const float r1 = 1.0f / sqrtf(s2 / (float)width + eps), r2 = 1.0f / sqrtf(s4 / (float)width + eps), r3 = 1.0f / sqrtf(s6 / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = pn_row[j], v2 = v * v, v3 = v2 * v;
        out[n * width + j] = from_f32<T>(c1 * (v * r1) + c2 * (v2 * r2) + c3 * (v3 * r3) + c0);
    }
}

ZI_EXPORT int zi_poly_norm(const void* z, int dtype, long long ldz, void* out, int rows, int width, float c1, float c2, float c3, float c0,
                           float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (width <= 0 || smem > 200 * 1024) return zi_fail("poly_norm: width=%d is not supported", width);
    const bool vec = width % 8 == 0 && ldz % 8 == 0 && (((size_t)z | (size_t)out) & 31) == 0;
    ZI_DISPATCH(dtype, T, {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(vec ? poly_norm_vec8_kernel<T> : poly_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return zi_fail("poly_norm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        }
        if (vec) poly_norm_vec8_kernel<T><<<rows, 256, smem, stream>>>((const T*)z, ldz, (T*)out, width, c1, c2, c3, c0, eps);
        else poly_norm_kernel<T><<<rows, 256, smem, stream>>>((const T*)z, ldz, (T*)out, width, c1, c2, c3, c0, eps);
    });
    return zi_check_launch("poly_norm");
}

// ---------------------------------------------------------------------------------------
// One gate per row:  g[n] = sigmoid(x[n, :] . w)  in float32 (x, w of any of the two types).  One warp per row, eight rows
// per block; a lane's terms in rising k, the lanes' sums in a fixed order.  VEC: eight entries per access (K and ldx multiples
// of 8, pointers on 16- and 32-byte boundaries); which form runs depends on sizes and addresses, never on the rows.
// ---------------------------------------------------------------------------------------
#define RG_WARPS 8
template <typename T, typename TW, bool VEC>
__global__ void __launch_bounds__(RG_WARPS * 32)
row_gate_kernel(const T* __restrict__ x, long long ldx, const TW* __restrict__ w, float* __restrict__ g, int rows, int K) {
    const int lane = threadIdx.x & 31;
    const size_t n = (size_t)blockIdx.x * RG_WARPS + (threadIdx.x >> 5);
    if (n >= (size_t)rows) return;
    float acc = 0.0f;
    if (VEC) {
        for (int k = lane * 8; k < K; k += 256) {
            float a[8], b[8];
            load8(x + n * ldx + k, a); load8(w + k, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(a[e], b[e], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(to_f32<T>(x[n * ldx + k]), to_f32<TW>(w[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) g[n] = 1.0f / (1.0f + expf(-acc));
}

ZI_EXPORT int zi_row_gate(const void* x, int dtype, long long ldx, const void* w, int w_dtype, float* g, int rows, int K, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (K <= 0) return zi_fail("row_gate: K=%d", K);
    const bool vec = K % 8 == 0 && ldx % 8 == 0 && (((size_t)x | (size_t)w) & 31) == 0;
    const int blocks = (rows + RG_WARPS - 1) / RG_WARPS;
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        if (vec) row_gate_kernel<T, TW, true><<<blocks, RG_WARPS * 32, 0, stream>>>((const T*)x, ldx, (const TW*)w, g, rows, K);
        else row_gate_kernel<T, TW, false><<<blocks, RG_WARPS * 32, 0, stream>>>((const T*)x, ldx, (const TW*)w, g, rows, K);
    }););
    return zi_check_launch("row_gate");
}
