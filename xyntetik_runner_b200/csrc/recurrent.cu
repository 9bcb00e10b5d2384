// Two linear recurrences with a fixed-size float32 state per request slot.
//
// (1) The real-gated linear recurrent unit (the recurrence of Griffin's recurrent block).  With R channels in B blocks of
//     R / B, a short causal convolution per channel, and per token the projections' rows y' and x' (float32, biases included):
//       u   = conv_b + sum_j conv_w[c][taps-1-j] x'[t-j][c]           (zeros before the request's first token; no activation)
//       r   = sigmoid(Wa[b] u_b + ba),  i = sigmoid(Wi[b] u_b + bi)    per block b, Wa[b] and Wi[b] square
//       a   = exp(-c r softplus(lam)),  S <- a S + sqrt(1 - a^2) (i u)  c a constant of the design (an argument)
//       out = S * gelu_tanh(y')
//     State per slot: S [R], then the last taps - 1 rows x' [taps-1][R].
//     k_rglru_gates, a block per (tile of tokens, channel block): convolution into shared memory, then both gate products
//     with one output channel a thread (the matrices are given transposed, [b][in][out], so that a warp reads a row), then
//     a and the recurrence's input.  k_rglru_scan, a thread a channel: the walk over a portion's tokens, the read-out times
//     the gated branch, and the slot's new tail.
//
// (2) Linear attention with a constant decay per head ("lightning attention"): S [D][V] per head,
//       S <- decay_h S + k v^T,   o = S^T q,   q, k, v = silu of the projections' rows.
//     k_decay_scan, a block per (32 value columns, head, portion): the tile of S in shared memory, a warp a stripe of key
//     rows, a lane a value column; the next token's q and k are fetched while this one is computed.
//
// Everything here is float32 in both precisions, and both walks go token by token: the state after a token does not depend
// on how the tokens were cut into steps, bit for bit.
#include "common.cuh"
#include <math.h>

#define RG_TT 8                 // tokens a block of the gates kernel takes
#define RG_MAX_TAPS 16

__device__ __forceinline__ float rc_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_softplus(float z) { return z > 30.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rc_silu(float z) { return z < -80.0f ? 0.0f : z / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_gelu_tanh(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

__global__ void __launch_bounds__(128)
k_rglru_gates(const float* __restrict__ proj, long long ldp, int x_col, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
              const float* __restrict__ wa_t, const float* __restrict__ wi_t, const float* __restrict__ ba, const float* __restrict__ bi,
              const float* __restrict__ lam, const float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seg,
              const int* __restrict__ seg_start, const int* __restrict__ seg_slot, float* __restrict__ a_out, float* __restrict__ b_out,
              int n, int R, int Bs, int taps, float c) {
    xr_pdl_launch();
    extern __shared__ float rg_u[];                // [RG_TT][Bs]
    const int t0 = blockIdx.x * RG_TT, b = blockIdx.y, c0 = b * Bs;
    const int nt = min(RG_TT, n - t0);
    xr_pdl_wait();
    for (int idx = threadIdx.x; idx < nt * Bs; idx += blockDim.x) {
        const int tt = idx / Bs, e = idx % Bs, t = t0 + tt, ch = c0 + e;
        const int seg = tok_seg[t], i = t - seg_start[seg];
        const float* tail = state + (size_t)seg_slot[seg] * state_stride + R;
        const float* w = conv_w + (size_t)ch * taps;
        float acc = conv_b[ch];
        for (int j = taps - 1; j >= 0; j--) {                            // oldest input first
            const int ip = i - j;
            const float x = ip >= 0 ? proj[(size_t)(t - j) * ldp + x_col + ch] : tail[(size_t)(taps - 1 + ip) * R + ch];
            acc = fmaf(w[taps - 1 - j], x, acc);
        }
        rg_u[tt * Bs + e] = acc;
    }
    __syncthreads();
    const float* wa = wa_t + (size_t)b * Bs * Bs;
    const float* wi = wi_t + (size_t)b * Bs * Bs;
    for (int o = threadIdx.x; o < Bs; o += blockDim.x) {
        float ra[RG_TT], ri[RG_TT];
#pragma unroll
        for (int tt = 0; tt < RG_TT; tt++) { ra[tt] = ba[c0 + o]; ri[tt] = bi[c0 + o]; }
        for (int k = 0; k < Bs; k++) {
            const float va = wa[(size_t)k * Bs + o], vi = wi[(size_t)k * Bs + o];
#pragma unroll
            for (int tt = 0; tt < RG_TT; tt++) {
                const float u = rg_u[tt * Bs + k];
                ra[tt] = fmaf(va, u, ra[tt]);
                ri[tt] = fmaf(vi, u, ri[tt]);
            }
        }
        const float rate = -c * rc_softplus(lam[c0 + o]);
#pragma unroll
        for (int tt = 0; tt < RG_TT; tt++) {
            if (tt < nt) {
                const float log_a = rate * rc_sigmoid(ra[tt]);
                const float a = expf(log_a);
                const float mult = sqrtf(-expm1f(2.0f * log_a));          // sqrt(1 - a^2) without the cancellation near a = 1
                const size_t at = (size_t)(t0 + tt) * R + c0 + o;
                a_out[at] = a;
                b_out[at] = mult * (rc_sigmoid(ri[tt]) * rg_u[tt * Bs + o]);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
k_rglru_scan(const float* __restrict__ proj, long long ldp, int y_col, int x_col, const float* __restrict__ a_in, const float* __restrict__ b_in,
             float* __restrict__ state, long long state_stride, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
             const int* __restrict__ seg_slot, T* __restrict__ out, int R, int taps) {
    xr_pdl_launch();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x, seg = blockIdx.y;
    if (ch >= R) return;
    const int start = seg_start[seg], len = seg_len[seg];
    float* st = state + (size_t)seg_slot[seg] * state_stride;
    xr_pdl_wait();
    float S = st[ch];
#pragma unroll 4
    for (int i = 0; i < len; i++) {
        const size_t t = (size_t)(start + i);
        S = fmaf(a_in[t * R + ch], S, b_in[t * R + ch]);
        out[t * R + ch] = xr_from_f32<T>(S * rc_gelu_tanh(proj[t * ldp + y_col + ch]));
    }
    st[ch] = S;
    // the slot's tail becomes the last taps - 1 inputs of the convolution: rows of this portion, older ones from the tail as it was
    float keep[RG_MAX_TAPS];
    float* tail = st + R;
    for (int r = 0; r < taps - 1; r++) {
        const int i = len - (taps - 1) + r;
        keep[r] = i >= 0 ? proj[(size_t)(start + i) * ldp + x_col + ch] : tail[(size_t)(r + len) * R + ch];
    }
    for (int r = 0; r < taps - 1; r++) tail[(size_t)r * R + ch] = keep[r];
}

// proj [n][ldp] float32: the gated branch's pre-activations at y_col, the convolution's inputs at x_col, R columns each.
// conv_w [R][taps], conv_b [R]; wa_t, wi_t [B][R/B (in)][R/B (out)]; ba, bi, lam [R]; all float32.
// state [slots][state_stride] float32: S [R], tail [taps-1][R].  a_s, b_s [n][R] float32 scratch.  out [n][R] dtype `dtype`.
XR_EXPORT int xr_rglru(const float* proj, long long ldp, int y_col, int x_col, const float* conv_w, const float* conv_b, const float* wa_t,
                       const float* wi_t, const float* ba, const float* bi, const float* lam, float* state, long long state_stride,
                       const int* tok_seg, const int* seg_start, const int* seg_len, const int* seg_slot, float* a_s, float* b_s, void* out,
                       int dtype, int n, int n_seg, int R, int B, int taps, float c, cudaStream_t stream) {
    if (n < 1 || n_seg < 1 || R < 1 || B < 1 || R % B || taps < 1 || taps > RG_MAX_TAPS || n_seg > 65535 || B > 65535 ||
        state_stride < (long long)R * taps)
        return XR_ERR_ARG;
    const int Bs = R / B;
    const size_t smem = (size_t)RG_TT * Bs * sizeof(float);
    if (smem > 48 * 1024) return XR_ERR_ARG;
    xr_launch(k_rglru_gates, dim3((n + RG_TT - 1) / RG_TT, B), dim3(128), smem, stream, proj, ldp, x_col, conv_w, conv_b, wa_t, wi_t, ba, bi, lam,
              (const float*)state, state_stride, tok_seg, seg_start, seg_slot, a_s, b_s, n, R, Bs, taps, c);
    dim3 gs((R + 127) / 128, n_seg);
    if (dtype == XR_F32)
        xr_launch((k_rglru_scan<float>), gs, dim3(128), 0, stream, proj, ldp, y_col, x_col, (const float*)a_s, (const float*)b_s, state,
                  state_stride, seg_start, seg_len, seg_slot, (float*)out, R, taps);
    else if (dtype == XR_BF16)
        xr_launch((k_rglru_scan<__nv_bfloat16>), gs, dim3(128), 0, stream, proj, ldp, y_col, x_col, (const float*)a_s, (const float*)b_s, state,
                  state_stride, seg_start, seg_len, seg_slot, (__nv_bfloat16*)out, R, taps);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
#define DA_COLS 32
#define DA_WARPS 8

__global__ void __launch_bounds__(DA_COLS * DA_WARPS)
k_decay_scan(const float* __restrict__ proj, long long ldp, int q_col, int k_col, int v_col, const float* __restrict__ decay,
             float* __restrict__ state, long long state_stride, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
             const int* __restrict__ seg_slot, float* __restrict__ o, int H, int D, int V) {
    xr_pdl_launch();
    extern __shared__ float da_sm[];                     // S tile [D][32], k [D], q [D], partial sums [8][32]
    float* S = da_sm;
    float* ks = S + (size_t)D * DA_COLS;
    float* qs = ks + D;
    float* part = qs + D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int v0 = blockIdx.x * DA_COLS, h = blockIdx.y, seg = blockIdx.z;
    const int col = v0 + lane;
    const bool live = col < V;
    const int start = seg_start[seg], len = seg_len[seg];
    const float dec = decay[h];
    float* st = state + (size_t)seg_slot[seg] * state_stride + (size_t)h * D * V;
    xr_pdl_wait();
    for (int d = warp; d < D; d += DA_WARPS) S[d * DA_COLS + lane] = live ? st[(size_t)d * V + col] : 0.f;
    // D <= 2 * blockDim: a thread fetches up to two elements of q and of k per token
    const int e0 = threadIdx.x, e1 = threadIdx.x + blockDim.x;
    float nq0 = 0.f, nk0 = 0.f, nq1 = 0.f, nk1 = 0.f, nv = 0.f;
    auto fetch = [&](int i) {
        const float* row = proj + (size_t)(start + i) * ldp;
        if (e0 < D) { nq0 = row[q_col + h * D + e0]; nk0 = row[k_col + h * D + e0]; }
        if (e1 < D) { nq1 = row[q_col + h * D + e1]; nk1 = row[k_col + h * D + e1]; }
        nv = live ? row[v_col + h * V + col] : 0.f;
    };
    if (len > 0) fetch(0);
    for (int i = 0; i < len; i++) {
        if (e0 < D) { qs[e0] = rc_silu(nq0); ks[e0] = rc_silu(nk0); }
        if (e1 < D) { qs[e1] = rc_silu(nq1); ks[e1] = rc_silu(nk1); }
        const float v = rc_silu(nv);
        __syncthreads();
        if (i + 1 < len) fetch(i + 1);
        float acc = 0.f;
        for (int d = warp; d < D; d += DA_WARPS) {
            const float s = fmaf(dec, S[d * DA_COLS + lane], ks[d] * v);
            S[d * DA_COLS + lane] = s;
            acc = fmaf(s, qs[d], acc);
        }
        part[warp * DA_COLS + lane] = acc;
        __syncthreads();
        if (warp == 0 && live) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < DA_WARPS; w++) sum += part[w * DA_COLS + lane];
            o[(size_t)(start + i) * H * V + (size_t)h * V + col] = sum;
        }
    }
    __syncthreads();
    if (live)
        for (int d = warp; d < D; d += DA_WARPS) st[(size_t)d * V + col] = S[d * DA_COLS + lane];
}

// proj [n][ldp] float32: pre-activations of q at q_col [H][D], k at k_col [H][D], v at v_col [H][V]; decay [H] float32;
// state [slots][state_stride] float32, S [H][D][V];  o [n][H V] float32 receives the read-outs.
XR_EXPORT int xr_decay_attention(const float* proj, long long ldp, int q_col, int k_col, int v_col, const float* decay, float* state,
                                 long long state_stride, const int* seg_start, const int* seg_len, const int* seg_slot, float* o, int n_seg,
                                 int H, int D, int V, cudaStream_t stream) {
    if (n_seg < 1 || H < 1 || D < 1 || V < 1 || D > 2 * DA_COLS * DA_WARPS || n_seg > 65535 || H > 65535 || state_stride < (long long)H * D * V)
        return XR_ERR_ARG;
    const size_t smem = ((size_t)D * DA_COLS + 2 * (size_t)D + DA_WARPS * DA_COLS) * sizeof(float);
    if (smem > 200 * 1024) return XR_ERR_ARG;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k_decay_scan, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return XR_ERR_LAUNCH;
    xr_launch(k_decay_scan, dim3((V + DA_COLS - 1) / DA_COLS, H, n_seg), dim3(DA_COLS * DA_WARPS), smem, stream, proj, ldp, q_col, k_col, v_col,
              decay, state, state_stride, seg_start, seg_len, seg_slot, o, H, D, V);
    return xr_launch_status();
}
