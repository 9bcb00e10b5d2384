// Memory-bound kernels of the step: embedding gather, RMSNorm, rotation + paged
// key/value store, SwiGLU.  The residual stream is float32 in both precisions;
// "activation dtype" below is what matrix products read and write (bfloat16 in
// the serving path, float32 in the true 32-bit path).
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[t] = E[id_t], ids outside [0, vocab) read row 0
// (the reference does the same on the host, src/model.c:6148-6162).
// ---------------------------------------------------------------------------
// `feed` (optional): ids[t] = -(1 + j) stands for feed[j], a token that an earlier step of the same stream left
// on the device (the one it sampled), so that the host need not have seen it when it describes this step.
template <typename TW>
__global__ void k_embed(const TW* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ feed,
                        float* __restrict__ x, int d, int vocab, int n_feed, float scale) {
    xr_pdl_launch();
    // The token ids are part of the step's description and the table is a weight: the row is read before the kernel
    // ahead is complete, sixteen values a thread in one run of loads; only the stores wait.  (A fed token is another
    // matter: it is what the step before sampled, so it is read after the wait.)
    int t = blockIdx.x;
    int id = ids[t];
    const bool fed = feed != nullptr && id < 0 && -(id + 1) < n_feed;
    if (fed) {
        xr_pdl_wait();
        id = feed[-(id + 1)];
    }
    if (id < 0 || id >= vocab) id = 0;
    const TW* row = table + (size_t)id * d;
    float* out = x + (size_t)t * d;
    for (int i0 = threadIdx.x; i0 < d; i0 += 16 * blockDim.x) {
        TW v[16];
#pragma unroll
        for (int k = 0; k < 16; k++) {
            int i = i0 + k * blockDim.x;
            v[k] = row[i < d ? i : d - 1];
        }
        if (i0 == (int)threadIdx.x && !fed) xr_pdl_wait();
#pragma unroll
        for (int k = 0; k < 16; k++) {
            int i = i0 + k * blockDim.x;
            if (i < d) out[i] = xr_to_f32<TW>(v[k]) * scale;
        }
    }
}

// x[t] = E[id_t] * scale (scale 1 for a model without an embedding multiplier: the product is then exact)
XR_EXPORT int xr_embed(const void* table, int table_dtype, const int* ids, const int* feed, int n_feed, float* x, int n, int d,
                       int vocab, float scale, cudaStream_t stream) {
    if (n < 1 || d < 1 || vocab < 1 || n_feed < 0) return XR_ERR_ARG;
    if (table_dtype == XR_F32) xr_launch((k_embed<float>), dim3(n), dim3(256), 0, stream, (const float*)table, ids, feed, x, d, vocab, n_feed, scale);
    else if (table_dtype == XR_BF16) xr_launch((k_embed<__nv_bfloat16>), dim3(n), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, feed, x, d, vocab, n_feed, scale);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm of float32 rows: y = x * rsqrt(mean(x^2) + eps) * w
// (src/model.c:3386-3392; the reference's kernel is src/kernels.cu:32-48).
// `rows` (optional) picks the rows to normalise: out[i] = norm(x[rows[i]]).
// One block per row; the reduction order depends on the width only.
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void k_rmsnorm(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                          TO* __restrict__ out, const float* __restrict__ w2, TO* __restrict__ out2, int d, float eps) {
    xr_pdl_launch();
    xr_pdl_wait();
    __shared__ float scratch[33];
    int r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + (size_t)r * d;
    TO* o = out + (size_t)blockIdx.x * d;
    constexpr int PER = 16;                     // elements a thread can keep: rows up to 16 * blockDim.x stay in registers
    if (d <= PER * (int)blockDim.x) {
        float v[PER];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < PER; k++) {
            int i = threadIdx.x + k * blockDim.x;
            v[k] = i < d ? xr[i] : 0.f;
            ss += v[k] * v[k];
        }
        ss = xr_block_sum(ss, scratch);
        float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int k = 0; k < PER; k++) {
            int i = threadIdx.x + k * blockDim.x;
            if (i < d) {
                o[i] = xr_from_f32<TO>(v[k] * scale * w[i]);
                if (w2) out2[(size_t)blockIdx.x * d + i] = xr_from_f32<TO>(v[k] * scale * w2[i]);
            }
        }
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    ss = xr_block_sum(ss, scratch);
    float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        o[i] = xr_from_f32<TO>(xr[i] * scale * w[i]);
        if (w2) out2[(size_t)blockIdx.x * d + i] = xr_from_f32<TO>(xr[i] * scale * w2[i]);
    }
}

// Rows whose width is a multiple of four: a thread keeps up to eight float4 of the row, so a row needs few
// threads (width / 32) and many rows are in flight on an SM at once.  The block size, and with it the order
// of the sum, is a function of the width alone.
__device__ __forceinline__ void rms_store4(float* o, float4 v) { *reinterpret_cast<float4*>(o) = v; }
__device__ __forceinline__ void rms_store4(__nv_bfloat16* o, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(o) = u;
}
template <typename TO>
__global__ void k_rmsnorm_vec(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                              TO* __restrict__ out, const float* __restrict__ w2, TO* __restrict__ out2, int d, float eps) {
    xr_pdl_launch();
    xr_pdl_wait();
    __shared__ float scratch[33];
    constexpr int PER = 8;
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * d);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    TO* o = out + (size_t)blockIdx.x * d;
    const int quads = d >> 2;
    float4 v[PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = threadIdx.x + k * blockDim.x;
        v[k] = i < quads ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < PER; k++) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = xr_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = threadIdx.x + k * blockDim.x;
        if (i < quads) {
            float4 g = w4[i];
            rms_store4(o + 4 * (size_t)i, make_float4(v[k].x * scale * g.x, v[k].y * scale * g.y, v[k].z * scale * g.z, v[k].w * scale * g.w));
            if (w2) {
                g = reinterpret_cast<const float4*>(w2)[i];
                rms_store4(out2 + (size_t)blockIdx.x * d + 4 * (size_t)i,
                           make_float4(v[k].x * scale * g.x, v[k].y * scale * g.y, v[k].z * scale * g.z, v[k].w * scale * g.w));
            }
        }
    }
}

// `w2`, `out2` (both or neither): a second norm of the same rows with a weight of its own, written beside the first.
XR_EXPORT int xr_rmsnorm(const float* x, const int* rows, const float* w, void* out, const float* w2, void* out2, int out_dtype, int n, int d,
                         float eps, cudaStream_t stream) {
    if (n < 1 || d < 1 || (w2 == nullptr) != (out2 == nullptr)) return XR_ERR_ARG;
    if (out_dtype != XR_F32 && out_dtype != XR_BF16) return XR_ERR_ARG;
    if ((d & 3) == 0 && d <= 32 * 1024 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)w2 | (uintptr_t)out2) & 15) == 0) {
        int threads = (((d / 4 + 7) / 8 + 31) / 32) * 32;          // eight float4 per thread cover the row
        if (out_dtype == XR_F32) xr_launch((k_rmsnorm_vec<float>), dim3(n), dim3(threads), 0, stream, x, rows, w, (float*)out, w2, (float*)out2, d, eps);
        else xr_launch((k_rmsnorm_vec<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, x, rows, w, (__nv_bfloat16*)out, w2, (__nv_bfloat16*)out2, d, eps);
        return xr_launch_status();
    }
    int threads = d >= 2048 ? 512 : 256;
    if (out_dtype == XR_F32) xr_launch((k_rmsnorm<float>), dim3(n), dim3(threads), 0, stream, x, rows, w, (float*)out, w2, (float*)out2, d, eps);
    else if (out_dtype == XR_BF16) xr_launch((k_rmsnorm<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, x, rows, w, (__nv_bfloat16*)out, w2, (__nv_bfloat16*)out2, d, eps);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Rotation of Q and K and the store of K, V into their pages.
//
// qkv: [n, (H + 2K) * hd] rows as the fused projection wrote them (Q heads,
// then K heads, then V heads).  For the token at position p and pair index
// j < rotary_dim/2: a = p * inv_freq[j] in float32, then
// (x0, x1) -> (x0 c - x1 s, x0 s + x1 c) on elements (j, j + rotary_dim/2)
// (src/model.c:3514-3532, the half-split pairing).  Q is rotated in place; K
// is rotated and written to the cache, V copied (src/model.c:6276-6310).
// The cache of a layer group is [page][layer][K|V][kv head][token in page][hd];
// `cache_k` points at this layer's K block of page 0.
// ---------------------------------------------------------------------------
struct RopeStoreArgs {
    void* qkv;
    const int* positions;
    const int* tok_seg;
    const int* block_tables;     // [n_seg][max_pages]
    const float* inv_freq;       // [rotary_dim / 2] or null when rotary_dim == 0
    void* cache_k;               // null: this layer stores nothing (it reads another layer's cache)
    long long page_stride;       // elements between pages
    long long v_offset;          // elements from a layer's K block to its V block
    int n, H, K, hd, rotary_dim, max_pages, page_size;
    int adjacent;                // 0: pair j is elements (j, j + rotary_dim/2); 1: elements (2j, 2j + 1)
    float mscale;                // factor on the cosines and sines (1 unless the position encoding scales magnitudes)
};

// One block per token.  A thread owns pair index j (and every `blockDim.x / half`-th head): the angle
// pos * inv_freq[j] and its cosine and sine are computed once and used for all the Q and K heads.
template <typename T>
__global__ void k_rope_store(RopeStoreArgs a) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int t = blockIdx.x;
    const int qkv_dim = (a.H + 2 * a.K) * a.hd;
    T* row = (T*)a.qkv + (size_t)t * qkv_dim;
    const int pos = a.positions[t];
    const int half = a.rotary_dim >> 1;
    T* kdst = nullptr;
    if (a.cache_k != nullptr) {
        int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        kdst = (T*)a.cache_k + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * a.hd;
    }
    const size_t head_step = (size_t)a.page_size * a.hd;          // between kv heads inside a page
    // rotated pairs of the Q and K heads
    if (half > 0) {
        const int lanes = blockDim.x / half > 0 ? blockDim.x / half : 1;      // heads handled side by side
        const int j = threadIdx.x % half, h0 = threadIdx.x / half;
        if (threadIdx.x < lanes * half) {
            float ang = (float)pos * a.inv_freq[j];
            float c = cosf(ang) * a.mscale, s = sinf(ang) * a.mscale;
            const int i0 = a.adjacent ? 2 * j : j, i1 = a.adjacent ? 2 * j + 1 : j + half;
            for (int head = h0; head < a.H + a.K; head += lanes) {
                T* src = row + (size_t)head * a.hd;
                float x0 = xr_to_f32<T>(src[i0]), x1 = xr_to_f32<T>(src[i1]);
                T y0 = xr_from_f32<T>(x0 * c - x1 * s), y1 = xr_from_f32<T>(x0 * s + x1 * c);
                if (head < a.H) { src[i0] = y0; src[i1] = y1; }
                else if (kdst) { T* d = kdst + (size_t)(head - a.H) * head_step; d[i0] = y0; d[i1] = y1; }
            }
        }
    }
    if (kdst == nullptr) return;
    // the part of K beyond the rotated dimensions, and V, are copied
    const int tail = a.hd - 2 * half;
    for (int i = threadIdx.x; i < a.K * tail; i += blockDim.x) {
        int kvh = i / tail, e = 2 * half + i % tail;
        kdst[(size_t)kvh * head_step + e] = row[(size_t)(a.H + kvh) * a.hd + e];
    }
    T* vdst = kdst + a.v_offset;
    for (int i = threadIdx.x; i < a.K * a.hd; i += blockDim.x) {
        int kvh = i / a.hd, e = i % a.hd;
        vdst[(size_t)kvh * head_step + e] = row[(size_t)(a.H + a.K + kvh) * a.hd + e];
    }
}

// bfloat16 rows whose head size and rotated width are multiples of eight and sixteen: every access is a
// 16-byte vector of eight elements.  The cosines and sines of the token's angles are computed once, in
// shared memory; a thread then takes (head, group of eight pairs) units.
struct __align__(16) Bf16x8 { __nv_bfloat162 p[4]; };
__global__ void __launch_bounds__(256)
k_rope_store_vec(RopeStoreArgs a) {
    xr_pdl_launch();
    // positions, block tables and frequencies do not change while the step runs: the token's page and the table of
    // its angles are worked out before the kernel ahead (the product that writes the rows) is complete
    extern __shared__ float rope_cs[];                 // [half] cosines, [half] sines
    const int t = blockIdx.x;
    const int qkv_dim = (a.H + 2 * a.K) * a.hd;
    __nv_bfloat16* row = (__nv_bfloat16*)a.qkv + (size_t)t * qkv_dim;
    const int pos = a.positions[t];
    const int half = a.rotary_dim >> 1;
    __nv_bfloat16* kdst = nullptr;
    if (a.cache_k != nullptr) {
        int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        kdst = (__nv_bfloat16*)a.cache_k + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * a.hd;
    }
    const size_t head_step = (size_t)a.page_size * a.hd;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float ang = (float)pos * a.inv_freq[j];
        rope_cs[j] = cosf(ang) * a.mscale;
        rope_cs[half + j] = sinf(ang) * a.mscale;
    }
    __syncthreads();
    xr_pdl_wait();
    const int groups = half >> 3;                      // groups of eight pairs per head
    const int rot_heads = kdst ? a.H + a.K : a.H;      // without a cache to write, K is not needed
    for (int u = threadIdx.x; u < rot_heads * groups; u += blockDim.x) {
        int head = u / groups, j0 = (u % groups) << 3;
        if (a.adjacent) {
            // eight pairs are sixteen consecutive elements: two vectors, each bfloat162 one pair
            __nv_bfloat16* src = row + (size_t)head * a.hd + 2 * j0;
            Bf16x8 v[2] = {*reinterpret_cast<const Bf16x8*>(src), *reinterpret_cast<const Bf16x8*>(src + 8)};
#pragma unroll
            for (int k = 0; k < 8; k++) {
                float2 x = __bfloat1622float2(v[k >> 2].p[k & 3]);
                float c = rope_cs[j0 + k], sn = rope_cs[half + j0 + k];
                v[k >> 2].p[k & 3] = __floats2bfloat162_rn(x.x * c - x.y * sn, x.x * sn + x.y * c);
            }
            __nv_bfloat16* dst = head < a.H ? src : kdst + (size_t)(head - a.H) * head_step + 2 * j0;
            *reinterpret_cast<Bf16x8*>(dst) = v[0];
            *reinterpret_cast<Bf16x8*>(dst + 8) = v[1];
            continue;
        }
        __nv_bfloat16* src = row + (size_t)head * a.hd + j0;
        Bf16x8 lo = *reinterpret_cast<const Bf16x8*>(src), hi = *reinterpret_cast<const Bf16x8*>(src + half);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float2 x0 = __bfloat1622float2(lo.p[k]), x1 = __bfloat1622float2(hi.p[k]);
            float c0 = rope_cs[j0 + 2 * k], c1 = rope_cs[j0 + 2 * k + 1];
            float s0 = rope_cs[half + j0 + 2 * k], s1 = rope_cs[half + j0 + 2 * k + 1];
            lo.p[k] = __floats2bfloat162_rn(x0.x * c0 - x1.x * s0, x0.y * c1 - x1.y * s1);
            hi.p[k] = __floats2bfloat162_rn(x0.x * s0 + x1.x * c0, x0.y * s1 + x1.y * c1);
        }
        __nv_bfloat16* dst = head < a.H ? src : kdst + (size_t)(head - a.H) * head_step + j0;
        *reinterpret_cast<Bf16x8*>(dst) = lo;
        *reinterpret_cast<Bf16x8*>(dst + half) = hi;
    }
    if (kdst == nullptr) return;
    const int tail8 = (a.hd - 2 * half) >> 3, hd8 = a.hd >> 3;
    for (int i = threadIdx.x; i < a.K * tail8; i += blockDim.x) {
        int kvh = i / tail8, e = 2 * half + ((i % tail8) << 3);
        *reinterpret_cast<Bf16x8*>(kdst + (size_t)kvh * head_step + e) = *reinterpret_cast<const Bf16x8*>(row + (size_t)(a.H + kvh) * a.hd + e);
    }
    __nv_bfloat16* vdst = kdst + a.v_offset;
    for (int i = threadIdx.x; i < a.K * hd8; i += blockDim.x) {
        int kvh = i / hd8, e = (i % hd8) << 3;
        *reinterpret_cast<Bf16x8*>(vdst + (size_t)kvh * head_step + e) = *reinterpret_cast<const Bf16x8*>(row + (size_t)(a.H + a.K + kvh) * a.hd + e);
    }
}

XR_EXPORT int xr_rope_store(void* qkv, int dtype, const int* positions, const int* tok_seg, const int* block_tables,
                            const float* inv_freq, void* cache_k, long long page_stride, long long v_offset,
                            int n, int H, int K, int hd, int rotary_dim, int max_pages, int page_size,
                            int adjacent_pairs, float mscale, cudaStream_t stream) {
    if (n < 1 || H < 1 || K < 1 || hd < 1 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) ||
        page_size < 1 || H + 2 * K > 65535)
        return XR_ERR_ARG;
    RopeStoreArgs a{qkv, positions, tok_seg, block_tables, inv_freq, cache_k, page_stride, v_offset,
                    n, H, K, hd, rotary_dim, max_pages, page_size, adjacent_pairs ? 1 : 0, mscale};
    int threads = 256;
    if (dtype == XR_BF16 && (hd & 7) == 0 && (rotary_dim & 15) == 0 && ((uintptr_t)qkv & 15) == 0 &&
        (cache_k == nullptr || ((((uintptr_t)cache_k) & 15) == 0 && (page_stride & 7) == 0 && (v_offset & 7) == 0))) {
        xr_launch(k_rope_store_vec, dim3(n), dim3(threads), (size_t)rotary_dim * sizeof(float), stream, a);
        return xr_launch_status();
    }
    if (dtype == XR_F32) xr_launch((k_rope_store<float>), dim3(n), dim3(threads), 0, stream, a);
    else if (dtype == XR_BF16) xr_launch((k_rope_store<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, a);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm of rows in the activation dtype (a projection's output that is normed before the next product):
// out[t] = in[t] * rsqrt(mean(in[t]^2) + eps) * w, float32 arithmetic; rows may be strided.  One block per row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
k_rmsnorm_act(const T* __restrict__ in, long long ld_in, const float* __restrict__ w, T* __restrict__ out, long long ld_out, int d, float eps) {
    xr_pdl_launch();
    __shared__ float scratch[33];
    const T* src = in + (size_t)blockIdx.x * ld_in;
    T* dst = out + (size_t)blockIdx.x * ld_out;
    xr_pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) { const float v = xr_to_f32<T>(src[i]); ss = fmaf(v, v, ss); }
    ss = xr_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = xr_from_f32<T>(xr_to_f32<T>(src[i]) * inv * w[i]);
}

XR_EXPORT int xr_rmsnorm_act(const void* in, int dtype, long long ld_in, const float* w, void* out, long long ld_out, int n, int d, float eps,
                             cudaStream_t stream) {
    if (n < 1 || d < 1) return XR_ERR_ARG;
    if (dtype == XR_F32) xr_launch((k_rmsnorm_act<float>), dim3(n), dim3(128), 0, stream, (const float*)in, ld_in, w, (float*)out, ld_out, d, eps);
    else if (dtype == XR_BF16)
        xr_launch((k_rmsnorm_act<__nv_bfloat16>), dim3(n), dim3(128), 0, stream, (const __nv_bfloat16*)in, ld_in, w, (__nv_bfloat16*)out, ld_out, d, eps);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Queries and keys with a norm per head before the rotation, and value heads of another size than the key heads.
//
// in: [n, ld_in] rows as one projection wrote them: Q heads [H][D], then K heads [K][D], then V heads [K][Vd].
// Every Q and K head is divided by its root mean square (eps inside the root) and multiplied by a weight of D values
// that all heads share (q_w, k_w; null: no norm, or with `unit` a norm without a weight), in float32; the Q heads are
// then multiplied by a factor that grows with the position p, 1 + q_coef ln(floor((p + 1) / q_every) + 1) (q_every 0:
// no factor); then the first rotary_dim elements are rotated, pair
// (2j, 2j + 1) or (j, j + rotary_dim/2), by angle = position * freq[j] (a float64 product brought into [-pi, pi] in
// float64, cosine and sine in float32).  The attention kernels take one head size hd >= max(D, Vd) for keys and
// values: Q goes to q_out [n, q_ld] (head h at h * hd), K and V to the token's cache rows, each head filled up to hd
// with zeros, which change neither a score nor a sum.  One block per token, a warp per head.
// ---------------------------------------------------------------------------
struct QkNormStoreArgs {
    const void* in;
    long long ld_in;
    void* q_out;
    long long q_ld;
    const int* positions;
    const int* tok_seg;
    const int* block_tables;
    const double* freq;          // [rotary_dim / 2] or null when rotary_dim == 0
    const float* q_w;
    const float* k_w;
    void* cache_k;               // null: this layer stores nothing
    long long page_stride, v_offset;
    int H, K, D, Vd, hd, rotary_dim, max_pages, page_size, adjacent;
    float eps;
    int pairs;                   // every size, stride and base address is even in elements (set by the launcher)
    int unit;                    // with null weights: divide by the root mean square all the same
    float q_coef; int q_every;   // the queries' factor by position (q_every 0: none)
    // The projection as the partial sums of a product that was cut along K, [splits][n][cols] float32 (null: `in` holds the rows):
    // the kernel first sums a row's partials in split order, adds the bias and writes the row to `in`, all `cols` columns (columns
    // behind the values, such as gates that a later kernel reads, are finished with them).
    const float* partial; const float* bias; int splits, cols, n;
    float mscale;                // factor on every cosine and sine
    int norm_after;              // the unit norm is taken of the ROTATED head (with mscale other than one the order matters)
};

template <typename T>
__global__ void __launch_bounds__(256)
k_qk_norm_rope_store(QkNormStoreArgs a) {
    xr_pdl_launch();
    extern __shared__ __align__(16) float qk_sm[];     // [half] cosines, [half] sines, then D floats per warp
    const int t = blockIdx.x, half = a.rotary_dim >> 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int pos = a.positions[t];
    float* cs = qk_sm;
    float* mine = qk_sm + 2 * half + (size_t)warp * a.D;
    const int part = blockIdx.y, parts = gridDim.y;        // a token's heads and columns may be shared out over several blocks
    if (part * nw < a.H + a.K)                             // (a block that only finishes columns behind the heads needs no angles)
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            xr_sincos_angle((double)pos * a.freq[j], &cs[half + j], &cs[j]);
            cs[half + j] *= a.mscale; cs[j] *= a.mscale;
        }
    T* kdst = nullptr;
    if (a.cache_k != nullptr) {
        const int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        kdst = (T*)a.cache_k + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * a.hd;
    }
    const size_t head_step = (size_t)a.page_size * a.hd;
    const float q_factor = a.q_every > 0 ? 1.0f + a.q_coef * logf((float)((pos + 1) / a.q_every) + 1.0f) : 1.0f;
    // A turn by an angle keeps a pair's sum of squares, and cosines and sines times mscale multiply it by mscale^2: the sum of
    // squares of the rotated head is that of the head as it is, the rotated elements weighted by mscale^2.
    const float rot_weight = a.norm_after ? a.mscale * a.mscale : 1.0f;
    __syncthreads();
    xr_pdl_wait();
    const T* row = (const T*)a.in + (size_t)t * a.ld_in;
    // Rows that are still a product's partial sums: whoever reads a column sums it first (split order, then the bias), rounds it
    // as the product's own epilogue would and writes it to the row; nobody reads a column that another thread finished.
    T* wr = (T*)a.in + (size_t)t * a.ld_in;
    const size_t split_stride = (size_t)a.n * a.cols;
    const float* psum = a.partial != nullptr ? a.partial + (size_t)t * a.cols : nullptr;
    auto finished = [&](int c) -> T {
        float acc = 0.f;
#pragma unroll 8
        for (int s2 = 0; s2 < a.splits; s2++) acc += __ldcg(psum + (size_t)s2 * split_stride + c);
        const T r = xr_from_f32<T>(a.bias ? acc + a.bias[c] : acc);
        wr[c] = r;
        return r;
    };
    const int heads = kdst ? a.H + a.K : a.H;
    // bfloat16 rows whose sizes and strides are even: elements are read and written two at a time
    const bool pairs = sizeof(T) == 2 && a.pairs;
    // with more blocks than the heads take, the first ones take the heads and the others the columns behind them
    const int head_parts = min(parts, (heads + nw - 1) / nw), tail_parts = parts - head_parts;
    for (int head = part * nw + warp; head < heads && part < head_parts; head += head_parts * nw) {
        const T* src = row + (size_t)head * a.D;
        const float* w = head < a.H ? a.q_w : a.k_w;
        float ss = 0.f;
        if (psum != nullptr) {
            // a lane's columns (up to eight: heads have at most 256 elements), all of a split's loads in flight together
            float acc[8];
#pragma unroll
            for (int k = 0; k < 8; k++) acc[k] = 0.f;
            const float* ph = psum + (size_t)head * a.D + lane;
#pragma unroll 8
            for (int s2 = 0; s2 < a.splits; s2++) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = lane + 32 * k < a.D ? __ldcg(ph + (size_t)s2 * split_stride + 32 * k) : 0.f;
#pragma unroll
                for (int k = 0; k < 8; k++) acc[k] += v[k];
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int e = lane + 32 * k;
                if (e < a.D) {
                    const int c = head * a.D + e;
                    const T r = xr_from_f32<T>(a.bias ? acc[k] + a.bias[c] : acc[k]);
                    wr[c] = r;
                    const float x = xr_to_f32<T>(r);
                    mine[e] = x; ss = fmaf(x * (e < a.rotary_dim ? rot_weight : 1.0f), x, ss);
                }
            }
        } else if (pairs) {
            for (int e = 2 * lane; e < a.D; e += 64) {
                const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(src) + e));
                mine[e] = x.x; mine[e + 1] = x.y;
                ss = fmaf(x.x * (e < a.rotary_dim ? rot_weight : 1.0f), x.x, fmaf(x.y * (e + 1 < a.rotary_dim ? rot_weight : 1.0f), x.y, ss));
            }
        } else {
            for (int e = lane; e < a.D; e += 32) {
                const float x = xr_to_f32<T>(src[e]);
                mine[e] = x; ss = fmaf(x * (e < a.rotary_dim ? rot_weight : 1.0f), x, ss);
            }
        }
        ss = xr_warp_sum(ss);
        const bool normed = w != nullptr || a.unit;
        float inv = normed ? 1.0f / sqrtf(ss / (float)a.D + a.eps) : 1.0f;
        if (head < a.H) inv *= q_factor;
        __syncwarp();
        T* dst = head < a.H ? (T*)a.q_out + (size_t)t * a.q_ld + (size_t)head * a.hd : kdst + (size_t)(head - a.H) * head_step;
        auto value = [&](int e) -> float {
            if (e >= a.D) return 0.f;
            float y = w != nullptr ? mine[e] * inv * w[e] : mine[e] * inv;
            if (e < a.rotary_dim) {
                int j, other; bool first;
                if (a.adjacent) { j = e >> 1; first = !(e & 1); other = e ^ 1; }
                else { first = e < half; j = first ? e : e - half; other = first ? e + half : e - half; }
                const float z = w != nullptr ? mine[other] * inv * w[other] : mine[other] * inv;
                y = first ? y * cs[j] - z * cs[half + j] : y * cs[j] + z * cs[half + j];
            }
            return y;
        };
        if (pairs) {
            // two elements a lane, one 4-byte store
            for (int e = 2 * lane; e < a.hd; e += 64)
                *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(dst) + e) = __floats2bfloat162_rn(value(e), value(e + 1));
        } else {
            for (int e = lane; e < a.hd; e += 32) dst[e] = xr_from_f32<T>(value(e));
        }
        __syncwarp();
    }
    const int v_at = (a.H + a.K) * a.D;
    if (psum != nullptr) {
        // the columns behind the values (gates that a later kernel reads), then the values, a thread a column
        const int behind = a.cols - v_at - a.K * a.Vd, n_v = kdst ? a.K * a.hd : 0;
        T* vdst = kdst ? kdst + a.v_offset : nullptr;
        if (tail_parts > 0 && part < head_parts) return;
        const int first = tail_parts > 0 ? part - head_parts : part, step = (tail_parts > 0 ? tail_parts : parts) * blockDim.x;
        for (int i = first * blockDim.x + threadIdx.x; i < behind + n_v; i += step) {
            if (i < behind) { finished(v_at + a.K * a.Vd + i); continue; }
            const int kvh = (i - behind) / a.hd, e = (i - behind) % a.hd;
            vdst[(size_t)kvh * head_step + e] = e < a.Vd ? finished(v_at + kvh * a.Vd + e) : xr_from_f32<T>(0.f);
        }
        return;
    }
    if (kdst == nullptr) return;
    T* vdst = kdst + a.v_offset;
    const T* vsrc = row + (size_t)v_at;
    if (pairs && !(a.Vd & 1) && !(a.v_offset & 1) && !(((a.H + a.K) * a.D) & 1)) {
        const int hd2 = a.hd >> 1;
        for (int i = threadIdx.x; i < a.K * hd2; i += blockDim.x) {
            const int kvh = i / hd2, e = (i % hd2) * 2;
            uint32_t two = 0;                    // (two zeros)
            if (e < a.Vd) two = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(vsrc) + (size_t)kvh * a.Vd + e);
            *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(vdst) + (size_t)kvh * head_step + e) = two;
        }
        return;
    }
    for (int i = threadIdx.x; i < a.K * a.hd; i += blockDim.x) {
        const int kvh = i / a.hd, e = i % a.hd;
        vdst[(size_t)kvh * head_step + e] = e < a.Vd ? vsrc[(size_t)kvh * a.Vd + e] : xr_from_f32<T>(0.f);
    }
}

// The same for bfloat16 rows of whole prompts when every size, stride and address falls on a 16-byte border.  A block brings its
// token's row (queries, keys, values) into shared memory, 16 bytes a thread and all loads in flight together; then SUB lanes share a
// head, eight consecutive elements a lane (SUB * 8 >= hd), so that a warp takes 32 / SUB heads at a time: one 16-byte read, the sum
// of squares over the SUB lanes by shuffles, the rotation's partner as a second 16-byte read of the row, one 16-byte store.
template <int SUB>
__global__ void __launch_bounds__(256)
k_qk_norm_rope_store_vec(QkNormStoreArgs a) {
    xr_pdl_launch();
    extern __shared__ __align__(16) float qk_sm[];     // [half] cosines, [half] sines, then (on a 16-byte border) the row
    const int t = blockIdx.x, half = a.rotary_dim >> 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int pos = a.positions[t];
    float* cs = qk_sm;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        xr_sincos_angle((double)pos * a.freq[j], &cs[half + j], &cs[j]);
        cs[half + j] *= a.mscale; cs[j] *= a.mscale;
    }
    const float rot_weight = a.norm_after ? a.mscale * a.mscale : 1.0f;     // (see k_qk_norm_rope_store)
    __nv_bfloat16* kdst = nullptr;
    if (a.cache_k != nullptr) {
        const int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        kdst = (__nv_bfloat16*)a.cache_k + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * a.hd;
    }
    const size_t head_step = (size_t)a.page_size * a.hd;
    const float q_factor = a.q_every > 0 ? 1.0f + a.q_coef * logf((float)((pos + 1) / a.q_every) + 1.0f) : 1.0f;
    const int v_at = (a.H + a.K) * a.D;
    Bf16x8* staged = reinterpret_cast<Bf16x8*>(qk_sm + ((2 * half + 3) & ~3));
    xr_pdl_wait();
    {
        const Bf16x8* g = reinterpret_cast<const Bf16x8*>((const __nv_bfloat16*)a.in + (size_t)t * a.ld_in);
        const int n16 = (v_at + a.K * a.Vd) >> 3;
#pragma unroll 4
        for (int i = threadIdx.x; i < n16; i += blockDim.x) staged[i] = g[i];
    }
    __syncthreads();
    const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(staged);
    const int heads = kdst ? a.H + a.K : a.H;
    const int e0 = (lane & (SUB - 1)) << 3;
    const bool normed = a.q_w != nullptr || a.unit;
    for (int h0 = warp * (32 / SUB); h0 < heads; h0 += nw * (32 / SUB)) {
        const int head = h0 + lane / SUB;
        const bool live = head < heads && e0 < a.D;
        float x[8];
#pragma unroll
        for (int k = 0; k < 8; k++) x[k] = 0.f;
        if (live) {
            const Bf16x8 v = *reinterpret_cast<const Bf16x8*>(row + (size_t)head * a.D + e0);
#pragma unroll
            for (int k = 0; k < 4; k++) { const float2 f = __bfloat1622float2(v.p[k]); x[2 * k] = f.x; x[2 * k + 1] = f.y; }
        }
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) ss = fmaf(x[k], x[k], ss);
        if (e0 < a.rotary_dim) ss *= rot_weight;              // (a lane's eight elements are all rotated or all not)
#pragma unroll
        for (int o = SUB >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (head >= heads || e0 >= a.hd) continue;
        float inv = normed ? 1.0f / sqrtf(ss / (float)a.D + a.eps) : 1.0f;
        if (head < a.H) inv *= q_factor;
        const float* w = head < a.H ? a.q_w : a.k_w;
        float y[8];
        if (w != nullptr && live) {
            const float4 w0 = *reinterpret_cast<const float4*>(w + e0), w1 = *reinterpret_cast<const float4*>(w + e0 + 4);
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int k = 0; k < 8; k++) y[k] = x[k] * inv * ww[k];
        } else {
#pragma unroll
            for (int k = 0; k < 8; k++) y[k] = x[k] * inv;
        }
        if (live && e0 < a.rotary_dim) {
            if (a.adjacent) {
                const int j0 = e0 >> 1;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float c = cs[j0 + k], sn = cs[half + j0 + k], u = y[2 * k], v = y[2 * k + 1];
                    y[2 * k] = u * c - v * sn;
                    y[2 * k + 1] = v * c + u * sn;
                }
            } else {
                const bool first = e0 < half;
                const int other = first ? e0 + half : e0 - half, j0 = first ? e0 : e0 - half;
                const Bf16x8 v = *reinterpret_cast<const Bf16x8*>(row + (size_t)head * a.D + other);
                float z[8];
#pragma unroll
                for (int k = 0; k < 4; k++) { const float2 f = __bfloat1622float2(v.p[k]); z[2 * k] = f.x * inv; z[2 * k + 1] = f.y * inv; }
                if (w != nullptr) {
#pragma unroll
                    for (int k = 0; k < 8; k++) z[k] *= w[other + k];
                }
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float c = cs[j0 + k], sn = cs[half + j0 + k];
                    y[k] = first ? y[k] * c - z[k] * sn : y[k] * c + z[k] * sn;
                }
            }
        }
        Bf16x8 out;
#pragma unroll
        for (int k = 0; k < 4; k++) out.p[k] = __floats2bfloat162_rn(y[2 * k], y[2 * k + 1]);
        __nv_bfloat16* dst = head < a.H ? (__nv_bfloat16*)a.q_out + (size_t)t * a.q_ld + (size_t)head * a.hd : kdst + (size_t)(head - a.H) * head_step;
        *reinterpret_cast<Bf16x8*>(dst + e0) = out;
    }
    if (kdst == nullptr) return;
    __nv_bfloat16* vdst = kdst + a.v_offset;
    const int hd8 = a.hd >> 3;
    for (int i = threadIdx.x; i < a.K * hd8; i += blockDim.x) {
        const int kvh = i / hd8, e = (i % hd8) << 3;
        Bf16x8 v;
#pragma unroll
        for (int k = 0; k < 4; k++) v.p[k] = __floats2bfloat162_rn(0.f, 0.f);
        if (e < a.Vd) v = *reinterpret_cast<const Bf16x8*>(row + (size_t)v_at + (size_t)kvh * a.Vd + e);
        *reinterpret_cast<Bf16x8*>(vdst + (size_t)kvh * head_step + e) = v;
    }
}

XR_EXPORT int xr_qk_norm_rope_store(const void* in, int dtype, long long ld_in, void* q_out, long long q_ld, const int* positions,
                                    const int* tok_seg, const int* block_tables, const double* freq, const float* q_w, const float* k_w,
                                    void* cache_k, long long page_stride, long long v_offset, int n, int H, int K, int D, int Vd, int hd,
                                    int rotary_dim, int max_pages, int page_size, int adjacent_pairs, float eps, int unit_norm,
                                    float q_coef, int q_every, const float* partial, int splits, const float* bias, int cols,
                                    float mscale, int norm_after, cudaStream_t stream) {
    if (partial != nullptr && (splits < 1 || D > 256 || cols < (H + K) * D + K * Vd || cols > ld_in)) return XR_ERR_ARG;
    if (n < 1 || H < 1 || K < 1 || D < 1 || Vd < 1 || hd < D || hd < Vd || rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) ||
        page_size < 1 || (rotary_dim > 0 && freq == nullptr) || (q_w == nullptr) != (k_w == nullptr) || q_every < 0 ||
        (unit_norm && q_w != nullptr) || (norm_after && !unit_norm))
        return XR_ERR_ARG;
    const int pairs = !((D | hd | ld_in | q_ld | page_stride) & 1) && !(((uintptr_t)in | (uintptr_t)q_out | (uintptr_t)cache_k) & 3);
    QkNormStoreArgs a{in, ld_in, q_out, q_ld, positions, tok_seg, block_tables, freq, q_w, k_w, cache_k, page_stride, v_offset,
                      H, K, D, Vd, hd, rotary_dim, max_pages, page_size, adjacent_pairs ? 1 : 0, eps, pairs, unit_norm ? 1 : 0,
                      q_coef, q_every, partial, bias, splits, cols, n, mscale, norm_after ? 1 : 0};
    const size_t smem = ((size_t)rotary_dim + 8 * (size_t)D) * sizeof(float);
    if (smem > 48 * 1024) return XR_ERR_ARG;
    // bfloat16 rows of whole prompts whose sizes, strides and addresses all fall on 16-byte borders: eight elements a lane
    const int row_cols = (H + K) * D + K * Vd;
    const size_t vec_smem = (((size_t)rotary_dim * sizeof(float) + 15) & ~(size_t)15) + (size_t)row_cols * 2;
    const int rot_ok = adjacent_pairs ? !(rotary_dim & 7) : !(rotary_dim & 15);
    if (dtype == XR_BF16 && partial == nullptr && rot_ok && hd <= 256 && vec_smem <= 48 * 1024 &&
        !((D | Vd | hd | ld_in | q_ld | page_stride | v_offset) & 7) &&
        !(((uintptr_t)in | (uintptr_t)q_out | (uintptr_t)cache_k | (uintptr_t)q_w | (uintptr_t)k_w) & 15)) {
        if (hd <= 32) xr_launch((k_qk_norm_rope_store_vec<4>), dim3(n), dim3(256), vec_smem, stream, a);
        else if (hd <= 64) xr_launch((k_qk_norm_rope_store_vec<8>), dim3(n), dim3(256), vec_smem, stream, a);
        else if (hd <= 128) xr_launch((k_qk_norm_rope_store_vec<16>), dim3(n), dim3(256), vec_smem, stream, a);
        else xr_launch((k_qk_norm_rope_store_vec<32>), dim3(n), dim3(256), vec_smem, stream, a);
        return xr_launch_status();
    }
    // rows as partial sums come from few tokens: a warp a head, a thread a column behind the heads (values, gates), over as many
    // blocks as that takes, so that the sums' loads spread and no thread sums more than one column after the other
    int parts = 1;
    if (partial != nullptr) {
        const int behind = cols - (H + K) * D - K * Vd + K * hd;
        parts = (H + K + 7) / 8 + (behind + 255) / 256;
        if (parts > 64) parts = 64;
    }
    if (dtype == XR_F32) xr_launch((k_qk_norm_rope_store<float>), dim3(n, parts), dim3(256), smem, stream, a);
    else if (dtype == XR_BF16) xr_launch((k_qk_norm_rope_store<__nv_bfloat16>), dim3(n, parts), dim3(256), smem, stream, a);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Activation of a feed-forward: gated, h = act(g) * u with g, u the two halves of each row of gu [n, 2F]
// (src/model.c:4425-4452, `gated_act`); ungated, h = act(x) of x [n, F] (src/model.c:6380-6396).
// act 1: SiLU, g / (1 + exp(-g)), 0 for g < -80 (src/model.c:4451-4452; the reference's kernel is
// src/kernels.cu:2868-2874); act 2: tanh-GELU, 0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3)))
// (src/model.c:4438-4441); act 0: none.  Full-precision expf and tanhf: this is the kernel of the true 32-bit path.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float xr_activation(int act, float g) {
    if (act == 1) return g < -80.0f ? 0.0f : g / (1.0f + expf(-g));
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
    return g;
}

// act 3 (gated only): with g' = min(g, limit) and u' = u clamped to [-limit, limit], h = g' sigmoid(1.702 g') (u' + 1).
__device__ __forceinline__ float xr_gate(int act, float limit, float g, float u) {
    if (act == 3) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return xr_activation(act, g) * u;
}

template <typename T>
__global__ void k_act_mul(const T* gu, T* h, int n, int F, int act, int gated, float limit) {       // (h may be gu: no __restrict__)
    xr_pdl_launch();
    xr_pdl_wait();
    size_t total = (size_t)n * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i / F, f = i % F;
        float v;
        if (gated) v = xr_gate(act, limit, xr_to_f32<T>(gu[t * 2 * F + f]), xr_to_f32<T>(gu[t * 2 * F + F + f]));
        else v = xr_activation(act, xr_to_f32<T>(gu[i]));
        h[i] = xr_from_f32<T>(v);
    }
}

// gated: gu [n, 2F] -> h [n, F]; ungated: gu [n, F] -> h [n, F] (h may be gu)
XR_EXPORT int xr_act_mul(const void* gu, void* h, int dtype, int n, int F, int act, int gated, float limit, cudaStream_t stream) {
    if (n < 1 || F < 1 || act < 0 || act > 3 || (act == 3 && !gated)) return XR_ERR_ARG;
    size_t total = (size_t)n * F;
    int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (dtype == XR_F32) xr_launch((k_act_mul<float>), dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)h, n, F, act, gated, limit);
    else if (dtype == XR_BF16) xr_launch((k_act_mul<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, n, F, act, gated, limit);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// y[t][i] += d[t][i] on the float32 residual stream (src/kernels.cu:2903-2906),
// for parts whose last product cannot add into the stream itself.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void k_residual_add(float* __restrict__ x, const T* __restrict__ dlt, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] += xr_to_f32<T>(dlt[i]);
}

XR_EXPORT int xr_residual_add(float* x, const void* dlt, int dtype, int n, int d, cudaStream_t stream) {
    if (n < 1 || d < 1) return XR_ERR_ARG;
    size_t total = (size_t)n * d;
    int blocks = (int)((total + 255) / 256 < xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (dtype == XR_F32) xr_launch((k_residual_add<float>), dim3(blocks), dim3(256), 0, stream, x, (const float*)dlt, total);
    else if (dtype == XR_BF16) xr_launch((k_residual_add<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, x, (const __nv_bfloat16*)dlt, total);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// x[t][i] += m * d[t][i] on float32 streams: a block that runs its sublayers side by side collects their sum in d
// and adds it to the residual stream once, times the model's residual multiplier.
// ---------------------------------------------------------------------------
__global__ void k_scaled_add(float* __restrict__ x, const float* __restrict__ d, float m, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = fmaf(m, d[i], x[i]);
}

XR_EXPORT int xr_scaled_add(float* x, const float* d, float m, int n, int width, cudaStream_t stream) {
    if (n < 1 || width < 1) return XR_ERR_ARG;
    size_t total = (size_t)n * width;
    int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    xr_launch(k_scaled_add, dim3(blocks), dim3(256), 0, stream, x, d, m, total);
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// x[t][i] += x0[t][i] + v[i] on float32 streams (x0 null: the vector alone): the start of a pass of a model that runs a
// span of layers several times, where the embedding's output and a vector of the pass join the stream.
// ---------------------------------------------------------------------------
__global__ void k_stream_step(float* __restrict__ x, const float* __restrict__ x0, const float* __restrict__ v, int width, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float add = v != nullptr ? v[i % (size_t)width] : 0.f;
        if (x0 != nullptr) add += x0[i];
        x[i] += add;
    }
}

XR_EXPORT int xr_stream_step(float* x, const float* x0, const float* v, int n, int width, cudaStream_t stream) {
    if (n < 1 || width < 1 || (x0 == nullptr && v == nullptr)) return XR_ERR_ARG;
    size_t total = (size_t)n * width;
    int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    xr_launch(k_stream_step, dim3(blocks), dim3(256), 0, stream, x, x0, v, width, total);
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// An output gate on attention heads: o[t][h][d] *= sigmoid(g[t][h * Vd + d]) (a gate per element, `each`) or
// sigmoid(g[t][h]) (a gate per head), for d < Vd of every head's hd columns; the sigmoid and the product in float32.
// g are columns of the projection's rows (row stride ld_g).  bfloat16: eight elements a thread where sizes, strides and addresses
// fall on 16-byte borders (`two` = 8), two where they are even (`two` = 2).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void k_sigmoid_gate(T* __restrict__ o, long long ld_o, const T* __restrict__ g, long long ld_g, int H, int hd, int Vd, int each, int two) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int t = blockIdx.x;
    T* orow = o + (size_t)t * ld_o;
    const T* grow = g + (size_t)t * ld_g;
    if (sizeof(T) == 2 && two == 8) {
        const int v8 = Vd >> 3, per = H * v8;
        for (int i = threadIdx.x; i < per; i += blockDim.x) {
            const int h = i / v8, d = (i % v8) << 3;
            Bf16x8* dst = reinterpret_cast<Bf16x8*>(reinterpret_cast<__nv_bfloat16*>(orow) + (size_t)h * hd + d);
            Bf16x8 x = *dst;
            if (each) {
                const Bf16x8 gg = *reinterpret_cast<const Bf16x8*>(reinterpret_cast<const __nv_bfloat16*>(grow) + (size_t)h * Vd + d);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 a = __bfloat1622float2(x.p[k]), b = __bfloat1622float2(gg.p[k]);
                    x.p[k] = __floats2bfloat162_rn(a.x / (1.0f + expf(-b.x)), a.y / (1.0f + expf(-b.y)));
                }
            } else {
                const float den = 1.0f + expf(-xr_to_f32<T>(grow[h]));
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 a = __bfloat1622float2(x.p[k]);
                    x.p[k] = __floats2bfloat162_rn(a.x / den, a.y / den);
                }
            }
            *dst = x;
        }
        return;
    }
    if (sizeof(T) == 2 && two) {
        const int half_v = Vd >> 1, per = H * half_v;
        for (int i = threadIdx.x; i < per; i += blockDim.x) {
            const int h = i / half_v, d = (i % half_v) * 2;
            __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(orow) + (size_t)h * hd + d);
            const float2 x = __bfloat1622float2(*dst);
            float ga, gb;
            if (each) {
                const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(grow) + (size_t)h * Vd + d));
                ga = gg.x; gb = gg.y;
            } else {
                ga = gb = xr_to_f32<T>(grow[h]);
            }
            *dst = __floats2bfloat162_rn(x.x / (1.0f + expf(-ga)), x.y / (1.0f + expf(-gb)));
        }
        return;
    }
    for (int i = threadIdx.x; i < H * Vd; i += blockDim.x) {
        const int h = i / Vd, d = i % Vd;
        const float gv = xr_to_f32<T>(grow[each ? i : h]);
        T* dst = orow + (size_t)h * hd + d;
        *dst = xr_from_f32<T>(xr_to_f32<T>(*dst) / (1.0f + expf(-gv)));
    }
}

XR_EXPORT int xr_sigmoid_gate(void* o, long long ld_o, const void* g, long long ld_g, int dtype, int n, int H, int hd, int Vd, int each,
                              cudaStream_t stream) {
    if (n < 1 || H < 1 || Vd < 1 || hd < Vd) return XR_ERR_ARG;
    int two = !((hd | Vd | ld_o | ld_g) & 1) && !(((uintptr_t)o | (uintptr_t)g) & 3) ? 2 : 0;
    if (!((hd | Vd | ld_o) & 7) && !((uintptr_t)o & 15) && (!each || (!(ld_g & 7) && !((uintptr_t)g & 15)))) two = 8;
    const int work = H * Vd / (dtype == XR_BF16 && two ? two : 1);
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == XR_F32) xr_launch((k_sigmoid_gate<float>), dim3(n), dim3(threads), 0, stream, (float*)o, ld_o, (const float*)g, ld_g, H, hd, Vd, each ? 1 : 0, 0);
    else if (dtype == XR_BF16)
        xr_launch((k_sigmoid_gate<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, (__nv_bfloat16*)o, ld_o, (const __nv_bfloat16*)g, ld_g, H, hd, Vd,
                  each ? 1 : 0, two);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// out[t] = [a[t] ; b[t]] of two float32 streams, in the activation dtype: the input of a product over both.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void k_concat_cast(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int n, int width) {
    xr_pdl_launch();
    xr_pdl_wait();
    size_t total = (size_t)n * 2 * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i / (2 * (size_t)width), c = i % (2 * (size_t)width);
        out[i] = xr_from_f32<T>(c < (size_t)width ? a[t * width + c] : b[t * width + c - width]);
    }
}

XR_EXPORT int xr_concat_cast(const float* a, const float* b, void* out, int dtype, int n, int width, cudaStream_t stream) {
    if (n < 1 || width < 1) return XR_ERR_ARG;
    size_t total = (size_t)n * 2 * width;
    int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (dtype == XR_F32) xr_launch((k_concat_cast<float>), dim3(blocks), dim3(256), 0, stream, a, b, (float*)out, n, width);
    else if (dtype == XR_BF16) xr_launch((k_concat_cast<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, a, b, (__nv_bfloat16*)out, n, width);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Soft cap of float32 logits in place: z <- cap * tanh(z / cap).
// ---------------------------------------------------------------------------
__global__ void k_softcap(float* __restrict__ z, float cap, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    const float inv = 1.0f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        z[i] = cap * tanhf(z[i] * inv);
}

XR_EXPORT int xr_softcap(float* z, float cap, long long total, cudaStream_t stream) {
    if (total < 1 || !(cap > 0.f)) return XR_ERR_ARG;
    int blocks = (int)((total + 255) / 256 < (long long)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    xr_launch(k_softcap, dim3(blocks), dim3(256), 0, stream, z, cap, (size_t)total);
    return xr_launch_status();
}

#ifdef XR_TRACE
// ---------------------------------------------------------------------------
// Tracing build only: the records of all source files, one after another.
// host: [files][4096][4] (time resident, time the wait returned, grid packed 20 bits a dimension, block size);
// counts: [files] records written since the last call.  Returns the number of files.
// ---------------------------------------------------------------------------
static xr_tr_dump_fn g_tr_fns[32];
static int g_tr_nfns = 0;
extern "C" int xr_trace_add(xr_tr_dump_fn fn) { if (g_tr_nfns < 32) g_tr_fns[g_tr_nfns++] = fn; return g_tr_nfns; }
XR_EXPORT int xr_trace_dump(unsigned long long* host, unsigned int* counts) {
    for (int i = 0; i < g_tr_nfns; i++) g_tr_fns[i](host + (size_t)i * 4096 * 4, counts + i);
    return g_tr_nfns;
}
#endif
