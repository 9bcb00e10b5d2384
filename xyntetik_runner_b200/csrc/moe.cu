// Routed experts (mixture of experts): the choice of experts per token, the order of (token, choice) pairs by expert,
// the experts' products over the rows that chose them, and the weighted sum back into the token's stream.
//
//   z = W_router h (float32, a product of the caller);  the `top` largest z are chosen (ties: the lower index),
//   weights = softmax over the chosen z only;  out[t] += sum_j weight_j * expert_{e_j}(h[t]).
// An expert is a gated feed-forward: y = gate_act(W_gate h, W_up h), then W_down y (see xr_gate below for the
// activations).  No step reads anything back to the host: the plan of who computes what is made on the device, and
// the grids are sized for the worst case (every tile index beyond the plan's count returns at once).
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------------------------------------
// Choice: one warp per token.  ids [n][top] int32, wts [n][top] float32 (in the order of descending z).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
k_route_topk(const float* __restrict__ z, int* __restrict__ ids, float* __restrict__ wts, int n, int E, int top,
             const float* __restrict__ correction, int sigmoid_scores) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= n) return;
    const float* row = z + (size_t)t * E;
    float best0 = 0.f, sum = 0.f;
    int last_e = -1;
    float last_v = INFINITY;
    // the j-th choice: the largest value that comes after the (j-1)-th in the order (value descending, index ascending)
    for (int j = 0; j < top; j++) {
        float bv = -INFINITY;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            // (sigmoid scores: the choice is by score plus the expert's correction, where there is one)
            float v = row[e];
            if (sigmoid_scores) { v = 1.0f / (1.0f + expf(-v)); if (correction != nullptr) v += correction[e]; }
            const bool after = v < last_v || (v == last_v && e > last_e);
            if (after && (v > bv || (v == bv && e < be))) { bv = v; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        if (j == 0) best0 = bv;
        // the weight: softmax over the chosen logits, or the chosen expert's score itself, without its correction
        const float p = sigmoid_scores ? 1.0f / (1.0f + expf(-row[be < E ? be : 0])) : expf(bv - best0);
        sum += p;
        if (lane == 0) { ids[(size_t)t * top + j] = be; wts[(size_t)t * top + j] = p; }
        last_v = bv; last_e = be;
    }
    __syncwarp();
    if (sigmoid_scores) return;
    if (lane < top) wts[(size_t)t * top + lane] /= sum;
    for (int j = 32 + lane; j < top; j += 32) wts[(size_t)t * top + j] /= sum;
}

// sigmoid_scores: scores s = sigmoid(z); the `top` largest s + correction (correction [E] float32 or null) are chosen and their
// weights are s itself, not renormalised.  Otherwise the `top` largest z, weights their softmax.
XR_EXPORT int xr_route_topk(const float* z, int* ids, float* wts, int n, int E, int top, const float* correction, int sigmoid_scores,
                            cudaStream_t stream) {
    if (n < 1 || E < 1 || top < 1 || top > E || (correction != nullptr && !sigmoid_scores)) return XR_ERR_ARG;
    xr_launch(k_route_topk, dim3((n + 3) / 4), dim3(128), 0, stream, z, ids, wts, n, E, top, correction, sigmoid_scores ? 1 : 0);
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Plan, one block: rows = the n * top pairs sorted by expert, every expert's rows starting at a multiple of `align`
// (the row tile of the kernel that multiplies them), so that a tile of `align` rows meets one expert.
//   row_src [max_rows]: the pair (t * top + j) that row r computes, -1 for a row of padding;
//   pair_row [pairs]: the row of every pair;  tile_group [max_rows / align]: the tile's expert, -1 for a tile without rows.
//   max_rows = (pairs / align + E + 1) * align always suffices.
// Which row a pair gets among its expert's rows depends on the order in which threads arrive; a row's result does not.
// ---------------------------------------------------------------------------------------------
#define MOE_MAX_E 1024

__global__ void __launch_bounds__(1024)
k_moe_plan(const int* __restrict__ ids, int* __restrict__ row_src, int* __restrict__ pair_row, int* __restrict__ tile_group,
           int pairs, int E, int align, int max_tiles) {
    xr_pdl_launch();
    __shared__ int count[MOE_MAX_E], cursor[MOE_MAX_E], tile0[MOE_MAX_E + 1];
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    xr_pdl_wait();
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int tiles = 0;
        for (int e = 0; e < E; e++) {
            tile0[e] = tiles; cursor[e] = tiles * align;
            tiles += (count[e] + align - 1) / align;
        }
        tile0[E] = tiles;
    }
    __syncthreads();
    const int used = tile0[E];
    for (int r = threadIdx.x; r < max_tiles * align; r += blockDim.x) row_src[r] = -1;
    for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_group[t] = -1;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        for (int t = tile0[e]; t < tile0[e + 1]; t++) tile_group[t] = e;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int r = atomicAdd(&cursor[ids[p]], 1);
        row_src[r] = p;
        pair_row[p] = r;
    }
    (void)used;
}

XR_EXPORT int xr_moe_plan(const int* ids, int* row_src, int* pair_row, int* tile_group, int pairs, int E, int align, int max_tiles,
                          cudaStream_t stream) {
    if (pairs < 1 || E < 1 || E > MOE_MAX_E || align < 1 || max_tiles < pairs / align + E) return XR_ERR_ARG;
    xr_launch(k_moe_plan, dim3(1), dim3(1024), 0, stream, ids, row_src, pair_row, tile_group, pairs, E, align, max_tiles);
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// out[r] = h[row_src[r] / top] for the rows of tiles that hold any, zeros for rows of padding: the first product's
// input in the order of the plan, for the tensor-core product (which reads its rows through a tensor map).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
k_moe_gather(const T* __restrict__ h, long long ldh, T* __restrict__ out, const int* __restrict__ row_src,
             const int* __restrict__ tile_group, int top, int width, int align) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int r = blockIdx.x;
    if (tile_group[r / align] < 0) return;
    const int src = row_src[r];
    T* o = out + (size_t)r * width;
    if (src < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = xr_from_f32<T>(0.f);
        return;
    }
    const T* a = h + (size_t)(src / top) * ldh;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = a[i];
}

XR_EXPORT int xr_moe_gather(const void* h, int dtype, long long ldh, void* out, const int* row_src, const int* tile_group, int top,
                            int width, int align, int max_rows, cudaStream_t stream) {
    if (max_rows < 1 || width < 1 || top < 1 || align < 1) return XR_ERR_ARG;
    if (dtype == XR_F32) xr_launch((k_moe_gather<float>), dim3(max_rows), dim3(256), 0, stream, (const float*)h, ldh, (float*)out, row_src, tile_group, top, width, align);
    else if (dtype == XR_BF16) xr_launch((k_moe_gather<__nv_bfloat16>), dim3(max_rows), dim3(256), 0, stream, (const __nv_bfloat16*)h, ldh, (__nv_bfloat16*)out, row_src, tile_group, top, width, align);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// The experts' products over the planned tiles (align = 64 rows), float32 FMA, k in ascending order for every result:
// the products of the true 32-bit path and of sizes the tensor-core product does not take.
//  first product (gated = 1): rows gather their token's h (row_src[r] / top); W = [E][2F][K] (an expert's gate rows,
//    then its up rows); out Y [rows][F] in the activation dtype = gate_act(h . w_gate_f, h . w_up_f).
//  second product (gated = 0): rows read Y [rows][K = F]; W = [E][N][K]; out Z [rows][N] float32.
// Tile: 64 rows x 64 columns (gated: 32 features, gate and up side by side), 256 threads with 4 x 4 results each.
// ---------------------------------------------------------------------------------------------
#define MOE_TM 64
XR_EXPORT int xr_moe_tile_rows() { return MOE_TM; }

__device__ __forceinline__ float moe_gate(int act, float limit, float g, float u) {
    if (act == 3) {                  // g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit)
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    if (act == 1) return (g < -80.0f ? 0.0f : g / (1.0f + expf(-g))) * u;
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g))) * u;
    return g * u;
}

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
k_moe_gemm(const TA* __restrict__ A, long long lda, const TW* __restrict__ W, TO* __restrict__ out, long long ldo,
           const int* __restrict__ row_src, const int* __restrict__ tile_group, int top, int N, int K, int gated, int act, float limit) {
    xr_pdl_launch();
    __shared__ float As[16][64 + 1], Ws[16][64 + 1];
    __shared__ int src_row[64];
    xr_pdl_wait();
    const int e = tile_group[blockIdx.x];
    if (e < 0) return;
    const int r0 = blockIdx.x * MOE_TM;
    const int cols = gated ? 32 : 64;                 // output columns (features) per tile
    const int c0 = blockIdx.y * cols;
    const TW* We = W + (size_t)e * (gated ? 2 : 1) * N * K;
    if (threadIdx.x < 64) {
        const int r = threadIdx.x, s = row_src[r0 + r];
        src_row[r] = s < 0 ? -1 : (gated ? s / top : r0 + r);
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            const int kk = i & 15, r = i >> 4, k = k0 + kk, s = src_row[r];
            As[kk][r] = (s >= 0 && k < K) ? xr_to_f32<TA>(A[(size_t)s * lda + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            const int kk = i & 15, c = i >> 4, k = k0 + kk;
            // gated: columns 0..31 are gate rows c0 + c, columns 32..63 the up rows of the same features
            const int wrow = gated ? (c < 32 ? c0 + c : N + c0 + c - 32) : c0 + c;
            const bool ok = k < K && (gated ? (c0 + (c & 31) < N) : (c0 + c < N));
            Ws[kk][c] = ok ? xr_to_f32<TW>(We[(size_t)wrow * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = As[kk][ty + 16 * i]; b[i] = Ws[kk][tx + 16 * i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = ty + 16 * i;
        if (src_row[r] < 0) continue;
        TO* orow = out + (size_t)(r0 + r) * ldo;
        if (gated) {
            // this thread's columns tx, tx + 16 are gate sums, tx + 32, tx + 48 the up sums of the same two features
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int f = c0 + tx + 16 * j;
                if (f < N) orow[f] = xr_from_f32<TO>(moe_gate(act, limit, acc[i][j], acc[i][j + 2]));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int c = c0 + tx + 16 * j;
                if (c < N) orow[c] = xr_from_f32<TO>(acc[i][j]);
            }
        }
    }
}

// a_dtype: of A; w_dtype: of the experts' matrices; max_tiles: tiles of 64 rows the plan may use.
XR_EXPORT int xr_moe_gemm(const void* A, int a_dtype, long long lda, const void* W, int w_dtype, void* out, int out_dtype,
                          long long ldo, const int* row_src, const int* tile_group, int max_tiles,
                          int top, int N, int K, int gated, int act, float limit, cudaStream_t stream) {
    if (max_tiles < 1 || N < 1 || K < 1 || top < 1 || act < 0 || act > 3) return XR_ERR_ARG;
    const int cols = gated ? 32 : 64;
    dim3 grid(max_tiles, (N + cols - 1) / cols);
    if (grid.y > 65535) return XR_ERR_ARG;
    typedef __nv_bfloat16 bf;
#define MG(TA, TW, TO) xr_launch((k_moe_gemm<TA, TW, TO>), grid, dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, (TO*)out, ldo, \
                                 row_src, tile_group, top, N, K, gated, act, limit)
    const int key = a_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case XR_BF16 * 4 + XR_BF16 * 2 + XR_BF16: MG(bf, bf, bf); break;
        case XR_BF16 * 4 + XR_BF16 * 2 + XR_F32: MG(bf, bf, float); break;
        case XR_F32 * 4 + XR_BF16 * 2 + XR_F32: MG(float, bf, float); break;
        case XR_F32 * 4 + XR_F32 * 2 + XR_F32: MG(float, float, float); break;
        case XR_BF16 * 4 + XR_F32 * 2 + XR_BF16: MG(bf, float, bf); break;
        case XR_BF16 * 4 + XR_F32 * 2 + XR_F32: MG(bf, float, float); break;
        default: return XR_ERR_ARG;
    }
#undef MG
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// d[t][c] += sum_j wts[t][j] * Z[pair_row[t * top + j]][c], j ascending (float32).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_moe_combine(float* __restrict__ d, const float* __restrict__ Z, const float* __restrict__ wts, const int* __restrict__ pair_row,
              int n, int width, int top) {
    xr_pdl_launch();
    xr_pdl_wait();
    const size_t total = (size_t)n * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width, c = i % width;
        float s = 0.f;
        for (int j = 0; j < top; j++) s = fmaf(wts[t * top + j], Z[(size_t)pair_row[t * top + j] * width + c], s);
        d[i] += s;
    }
}

XR_EXPORT int xr_moe_combine(float* d, const float* Z, const float* wts, const int* pair_row, int n, int width, int top,
                             cudaStream_t stream) {
    if (n < 1 || width < 1 || top < 1) return XR_ERR_ARG;
    const size_t total = (size_t)n * width;
    int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    xr_launch(k_moe_combine, dim3(blocks), dim3(256), 0, stream, d, Z, wts, pair_row, n, width, top);
    return xr_launch_status();
}
