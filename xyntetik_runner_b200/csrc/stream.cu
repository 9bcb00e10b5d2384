// Kernels on the float32 residual stream that models with other layer arrangements than the pre-norm block need:
// an embedding with a hashed pair table, a norm on a sublayer's OUTPUT added into the stream, a weighted average over the
// streams that all earlier layers left, a cast of the stream for sublayers that read it without a norm, and a rotation of
// head rows by their token's position (values turned before they are cached, an attention's sums turned back).
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------------------
// Embedding plus a pair table: x[t] = E[id_t] + P[row_t], row_t = (prev_t * mul_prev + id_t * mul_cur) mod buckets, where
// prev_t is the token before t in its request; a request's first token (position 0) reads row `buckets`, the table's last.
// The token before a portion's first comes from last[slot], which k_last_token sets after every step.
// ids below zero stand for fed tokens as in k_embed.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int sk_token(const int* ids, const int* feed, int n_feed, int t, int vocab) {
    int id = ids[t];
    if (feed != nullptr && id < 0 && -(id + 1) < n_feed) id = feed[-(id + 1)];
    return (id < 0 || id >= vocab) ? 0 : id;
}

template <typename TW>
__global__ void k_embed_pair(const TW* __restrict__ table, const TW* __restrict__ pairs, const int* __restrict__ ids,
                             const int* __restrict__ feed, const int* __restrict__ positions, const int* __restrict__ tok_seg,
                             const int* __restrict__ seg_start, const int* __restrict__ seg_slot, const int* __restrict__ last,
                             float* __restrict__ x, int d, int vocab, int n_feed, long long buckets, long long mul_prev, long long mul_cur) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int t = blockIdx.x;
    const int id = sk_token(ids, feed, n_feed, t, vocab);
    long long row = buckets;
    if (positions[t] > 0) {
        const int seg = tok_seg[t];
        const int prev = t > seg_start[seg] ? sk_token(ids, feed, n_feed, t - 1, vocab) : last[seg_slot[seg]];
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const TW* e = table + (size_t)id * d;
    const TW* p = pairs + (size_t)row * d;
    float* out = x + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = xr_to_f32<TW>(e[i]) + xr_to_f32<TW>(p[i]);
}

XR_EXPORT int xr_embed_pair(const void* table, const void* pairs, int table_dtype, const int* ids, const int* feed, int n_feed,
                            const int* positions, const int* tok_seg, const int* seg_start, const int* seg_slot, const int* last,
                            float* x, int n, int d, int vocab, long long buckets, long long mul_prev, long long mul_cur,
                            cudaStream_t stream) {
    if (n < 1 || d < 1 || vocab < 1 || n_feed < 0 || buckets < 1) return XR_ERR_ARG;
#define EP(T) xr_launch((k_embed_pair<T>), dim3(n), dim3(256), 0, stream, (const T*)table, (const T*)pairs, ids, feed, positions, tok_seg, \
                        seg_start, seg_slot, last, x, d, vocab, n_feed, buckets, mul_prev, mul_cur)
    if (table_dtype == XR_F32) EP(float);
    else if (table_dtype == XR_BF16) EP(__nv_bfloat16);
    else return XR_ERR_ARG;
#undef EP
    return xr_launch_status();
}

// last[slot of portion s] = the portion's last token.  A launch of its own behind k_embed_pair: within one launch the block of a
// portion's last token could write before the block of its first token has read.
__global__ void k_last_token(const int* __restrict__ ids, const int* __restrict__ feed, int n_feed, const int* __restrict__ seg_start,
                             const int* __restrict__ seg_len, const int* __restrict__ seg_slot, int* __restrict__ last, int n_seg, int vocab) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seg || seg_len[s] < 1) return;
    last[seg_slot[s]] = sk_token(ids, feed, n_feed, seg_start[s] + seg_len[s] - 1, vocab);
}

XR_EXPORT int xr_last_token(const int* ids, const int* feed, int n_feed, const int* seg_start, const int* seg_len, const int* seg_slot,
                            int* last, int n_seg, int vocab, cudaStream_t stream) {
    if (n_seg < 1 || vocab < 1 || n_feed < 0) return XR_ERR_ARG;
    xr_launch(k_last_token, dim3((n_seg + 127) / 128), dim3(128), 0, stream, ids, feed, n_feed, seg_start, seg_len, seg_slot, last, n_seg, vocab);
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Norm on a sublayer's output, added into the stream: x[t] += d[t] / sqrt(mean(d[t]^2) + eps) * g, g ONE number (read from the
// device).  With `cast` the updated row is also written in the activation dtype, for a sublayer that reads the stream as it is.
// With `clear`, d[t] is zeroed behind the read, ready for the next sublayer's products to add into.
// `partial` (float32 [splits][n][width], or null): the sublayer's last products were cut along K and left their partial sums;
// the row is then d[t] plus the partial sums in split order (plus `bias` [width], if any).
// One block per row; the row is held in registers between the two passes (columns beyond what the threads own are read again);
// float32 throughout; the order of the sums depends on the width and the cut only.
// ---------------------------------------------------------------------------
// Two shapes: many rows, 256 threads a row with up to 16 columns each, one split's loads in flight at a time; few rows (a step of
// single tokens, where the partial sums are many and nothing else hides their latency), 1,024 threads a row with up to 4 columns
// each and eight splits' loads in flight together.  The sums are added in split order in both.
template <typename T, int OWN, int BATCH>
__global__ void __launch_bounds__(OWN <= 4 ? 1024 : 256)
k_norm_add(float* __restrict__ d, float* __restrict__ x, const float* __restrict__ g, T* __restrict__ cast, int width, float eps, int clear,
           const float* __restrict__ partial, const float* __restrict__ bias, int splits, int n) {
    xr_pdl_launch();
    __shared__ float scratch[33];
    const float gain = g[0];
    xr_pdl_wait();
    const int nt = blockDim.x;
    const size_t row = (size_t)blockIdx.x * width, split_stride = (size_t)n * width;
    float* dr = d + row;
    float* xr = x + row;
    auto value = [&](int i) -> float {
        float v = dr[i];
        if (partial != nullptr) {
            for (int s2 = 0; s2 < splits; s2++) v += __ldcg(partial + (size_t)s2 * split_stride + row + i);
            if (bias != nullptr) v += bias[i];
        }
        return v;
    };
    float own[OWN];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < OWN; k++) {
        const int i = threadIdx.x + k * nt;
        own[k] = i < width ? dr[i] : 0.f;
    }
    if (partial != nullptr) {
        for (int s0 = 0; s0 < splits; s0 += BATCH) {
            float v[BATCH][OWN];
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const float* ps = partial + (size_t)(s0 + b) * split_stride + row;
#pragma unroll
                for (int k = 0; k < OWN; k++) {
                    const int i = threadIdx.x + k * nt;
                    v[b][k] = (s0 + b < splits && i < width) ? xr_ld_now(ps + i) : 0.f;
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
#pragma unroll
                for (int k = 0; k < OWN; k++) { xr_ld_fence(v[b][k]); own[k] += v[b][k]; }
            }
        }
        if (bias != nullptr) {
#pragma unroll
            for (int k = 0; k < OWN; k++) {
                const int i = threadIdx.x + k * nt;
                if (i < width) own[k] += bias[i];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < OWN; k++) ss = fmaf(own[k], own[k], ss);
    for (int i = threadIdx.x + OWN * nt; i < width; i += nt) { const float v = value(i); ss = fmaf(v, v, ss); }
    ss = xr_block_sum(ss, scratch);
    const float inv = gain / sqrtf(ss / (float)width + eps);
    auto finish = [&](int i, float dv) {
        const float v = fmaf(dv, inv, xr[i]);
        xr[i] = v;
        if (cast != nullptr) cast[row + i] = xr_from_f32<T>(v);
        if (clear) dr[i] = 0.f;
    };
#pragma unroll
    for (int k = 0; k < OWN; k++) {
        const int i = threadIdx.x + k * nt;
        if (i < width) finish(i, own[k]);
    }
    for (int i = threadIdx.x + OWN * nt; i < width; i += nt) finish(i, value(i));
}

XR_EXPORT int xr_norm_add(float* d, float* x, const float* g, void* cast, int cast_dtype, int n, int width, float eps, int clear,
                          const float* partial, const float* bias, int splits, cudaStream_t stream) {
    if (n < 1 || width < 1 || (partial != nullptr && splits < 1)) return XR_ERR_ARG;
    const bool few = n <= 32;
#define NA(T)                                                                                                                                \
    do {                                                                                                                                     \
        if (few) xr_launch((k_norm_add<T, 4, 8>), dim3(n), dim3(1024), 0, stream, d, x, g, (T*)cast, width, eps, clear, partial, bias, splits, n); \
        else xr_launch((k_norm_add<T, 16, 1>), dim3(n), dim3(256), 0, stream, d, x, g, (T*)cast, width, eps, clear, partial, bias, splits, n);   \
    } while (0)
    if (cast == nullptr || cast_dtype == XR_F32) NA(float);
    else if (cast_dtype == XR_BF16) NA(__nv_bfloat16);
    else return XR_ERR_ARG;
#undef NA
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// A norm over a whole row with a weight per column, times a sigmoid gate: y[t][i] = o[t][i] / sqrt(mean(o[t]^2) + eps) * w[i] *
// sigmoid(g[t][i]) * scale; o, g float32 (g at g + t * ld_g), y in the activation dtype.  One block per row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
k_row_norm_gate(const float* __restrict__ o, const float* __restrict__ g, long long ld_g, const float* __restrict__ w, T* __restrict__ y,
                int width, float eps, float scale) {
    xr_pdl_launch();
    __shared__ float scratch[33];
    xr_pdl_wait();
    const float* src = o + (size_t)blockIdx.x * width;
    const float* gate = g + (size_t)blockIdx.x * ld_g;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = src[i]; ss = fmaf(v, v, ss); }
    ss = xr_block_sum(ss, scratch);
    const float inv = scale / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        y[(size_t)blockIdx.x * width + i] = xr_from_f32<T>(src[i] * inv * w[i] / (1.0f + expf(-gate[i])));
}

XR_EXPORT int xr_row_norm_gate(const float* o, const float* g, long long ld_g, const float* w, void* y, int dtype, int n, int width, float eps,
                               float scale, cudaStream_t stream) {
    if (n < 1 || width < 1) return XR_ERR_ARG;
    if (dtype == XR_F32) xr_launch((k_row_norm_gate<float>), dim3(n), dim3(256), 0, stream, o, g, ld_g, w, (float*)y, width, eps, scale);
    else if (dtype == XR_BF16) xr_launch((k_row_norm_gate<__nv_bfloat16>), dim3(n), dim3(256), 0, stream, o, g, ld_g, w, (__nv_bfloat16*)y, width, eps, scale);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// out[i] = x[i] in the activation dtype
template <typename T>
__global__ void k_cast_rows(const float* __restrict__ x, T* __restrict__ out, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) out[i] = xr_from_f32<T>(x[i]);
}

XR_EXPORT int xr_cast_rows(const float* x, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total < 1) return XR_ERR_ARG;
    const int blocks = (int)((total + 255) / 256 < (long long)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (dtype == XR_F32) xr_launch((k_cast_rows<float>), dim3(blocks), dim3(256), 0, stream, x, (float*)out, (size_t)total);
    else if (dtype == XR_BF16) xr_launch((k_cast_rows<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, (size_t)total);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Depth average: with X_0 = x0 (the embedding's output), X_1 .. X_(k-1) in hist [k-1][total] and X_k = x (what the layer just
// left), keep x in hist[k-1] and set x <- sum_(j=0..k) w[j] X_j, added in ascending j.  With `cast`, x is also written in the
// activation dtype.  float32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void k_depth_average(float* __restrict__ x, const float* __restrict__ x0, float* __restrict__ hist, const float* __restrict__ w,
                                T* __restrict__ cast, int k, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float cur = x[i];
        float acc = w[0] * x0[i];
        for (int j = 1; j < k; j++) acc = fmaf(w[j], hist[(size_t)(j - 1) * total + i], acc);
        acc = fmaf(w[k], cur, acc);
        hist[(size_t)(k - 1) * total + i] = cur;
        x[i] = acc;
        if (cast != nullptr) cast[i] = xr_from_f32<T>(acc);
    }
}

XR_EXPORT int xr_depth_average(float* x, const float* x0, float* hist, const float* w, void* cast, int cast_dtype, int k, long long total,
                               cudaStream_t stream) {
    if (total < 1 || k < 1) return XR_ERR_ARG;
    const int blocks = (int)((total + 255) / 256 < (long long)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (cast == nullptr || cast_dtype == XR_F32) xr_launch((k_depth_average<float>), dim3(blocks), dim3(256), 0, stream, x, x0, hist, w, (float*)cast, k, (size_t)total);
    else if (cast_dtype == XR_BF16) xr_launch((k_depth_average<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, x, x0, hist, w, (__nv_bfloat16*)cast, k, (size_t)total);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Rotation of head rows by their token's position, in place: for every token t and head h, the first `dims` of the head's
// elements at rows[t * ld + col0 + h * head_stride] are turned in pairs, pair m by sign * position_t * freq[m] (the angle a float64
// product), cosine and sine in float32; "half" pairs element m with m + dims/2, "adjacent" 2m with 2m + 1.  Every element of the
// head's first `live` (>= dims) is then multiplied by `scale`.  A block per token, a warp per head.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
k_rotate_heads(T* __restrict__ rows, long long ld, int col0, int heads, int head_stride, int dims, int live, int adjacent,
               const double* __restrict__ freq, const int* __restrict__ positions, float sign, float scale) {
    xr_pdl_launch();
    extern __shared__ float rh_cs[];                 // [half] cosines, [half] sines
    const int t = blockIdx.x, half = dims >> 1;
    const double pos = (double)positions[t] * (double)sign;
    for (int j = threadIdx.x; j < half; j += blockDim.x) xr_sincos_angle(pos * freq[j], &rh_cs[half + j], &rh_cs[j]);
    __syncthreads();
    xr_pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = warp; h < heads; h += nw) {
        T* p = rows + (size_t)t * ld + col0 + (size_t)h * head_stride;
        for (int m = lane; m < half; m += 32) {
            const int ia = adjacent ? 2 * m : m, ib = adjacent ? 2 * m + 1 : m + half;
            const float a = xr_to_f32<T>(p[ia]), b = xr_to_f32<T>(p[ib]);
            const float c = rh_cs[m], s = rh_cs[half + m];
            p[ia] = xr_from_f32<T>((a * c - b * s) * scale);
            p[ib] = xr_from_f32<T>((b * c + a * s) * scale);
        }
        if (scale != 1.0f)
            for (int e = dims + lane; e < live; e += 32) p[e] = xr_from_f32<T>(xr_to_f32<T>(p[e]) * scale);
    }
}

XR_EXPORT int xr_rotate_heads(void* rows, int dtype, long long ld, int col0, int heads, int head_stride, int dims, int live, int adjacent,
                              const double* freq, const int* positions, float sign, float scale, int n, cudaStream_t stream) {
    if (n < 1 || heads < 1 || dims < 0 || (dims & 1) || live < dims || live > head_stride || (dims > 0 && freq == nullptr)) return XR_ERR_ARG;
    const size_t smem = (size_t)dims * sizeof(float);
    if (smem > 48 * 1024) return XR_ERR_ARG;
    if (dtype == XR_F32) xr_launch((k_rotate_heads<float>), dim3(n), dim3(256), smem, stream, (float*)rows, ld, col0, heads, head_stride, dims, live, adjacent, freq, positions, sign, scale);
    else if (dtype == XR_BF16) xr_launch((k_rotate_heads<__nv_bfloat16>), dim3(n), dim3(256), smem, stream, (__nv_bfloat16*)rows, ld, col0, heads, head_stride, dims, live, adjacent, freq, positions, sign, scale);
    else return XR_ERR_ARG;
    return xr_launch_status();
}
