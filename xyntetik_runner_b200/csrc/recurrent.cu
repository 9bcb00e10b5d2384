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
//     a, the recurrence's input and the gated branch's activation.  k_rglru_scan, a thread a channel: the walk over a
//     portion's tokens, the read-out times the gated branch, and the slot's new tail.
//
// (2) Linear attention with a constant decay per head ("lightning attention"): S [D][V] per head,
//       S <- decay_h S + k v^T,   o = S^T q,   q, k, v the projections' rows behind their activation.
//     k_decay_scan, a warp per eight value columns of a head: the state in registers, see there.
//
// Everything here is float32 in both precisions, and both walks go token by token: the state after a token does not depend
// on how the tokens were cut into steps, bit for bit.
#include "common.cuh"
#include <math.h>

#define RG_MAX_TAPS 16

// a weight through the read-only path (blocks of the same SM read the same rows), pinned where it is written like xr_ld_now
__device__ __forceinline__ float rc_ld_weight(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float rc_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_softplus(float z) { return z > 30.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rc_silu(float z) { return z < -80.0f ? 0.0f : z / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_gelu_tanh(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

#define RG_COLS 128              // output channels a block of the gates kernel takes (a thread each)

// The convolution of tokens t0 .. t0 + nt - 1 over the channels of block b into shared memory; u[e * stride_e + tt * stride_t].
__device__ __forceinline__ void rg_conv_tile(float* u, int stride_e, int stride_t, const float* __restrict__ proj, long long ldp, int x_col,
                                             const float* __restrict__ conv_w, const float* __restrict__ conv_b, const float* __restrict__ state,
                                             long long state_stride, const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                                             const int* __restrict__ seg_slot, int t0, int nt, int c0, int R, int Bs, int taps) {
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
        u[e * stride_e + tt * stride_t] = acc;
    }
}

// a and the recurrence's input from the gates' sums; the gated branch's activation in place (nothing else reads those columns)
__device__ __forceinline__ void rg_finish(float ra, float ri, float u, float rate, float* a_out, float* b_out, float* y) {
    *y = rc_gelu_tanh(*y);
    const float log_a = rate * rc_sigmoid(ra);
    *a_out = expf(log_a);
    *b_out = sqrtf(-expm1f(2.0f * log_a)) * (rc_sigmoid(ri) * u);          // sqrt(1 - a^2) without the cancellation near a = 1
}

// Many tokens: a block per (TT tokens, channel block, 64 output channels), a thread an output channel with TT sums of each gate.
// The tile of u lies in shared memory input-major, [in][TT], so that a thread reads four tokens' values at once.
template <int TT>
__global__ void __launch_bounds__(RG_COLS)
k_rglru_gates(float* __restrict__ proj, long long ldp, int y_col, int x_col, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
              const float* __restrict__ wa_t, const float* __restrict__ wi_t, const float* __restrict__ ba, const float* __restrict__ bi,
              const float* __restrict__ lam, const float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seg,
              const int* __restrict__ seg_start, const int* __restrict__ seg_slot, float* __restrict__ a_out, float* __restrict__ b_out,
              int n, int R, int Bs, int taps, float c) {
    xr_pdl_launch();
    extern __shared__ __align__(16) float rg_u[];                // [Bs][TT]
    const int t0 = blockIdx.x * TT, b = blockIdx.y, c0 = b * Bs;
    const int nt = min(TT, n - t0);
    xr_pdl_wait();
    if (nt < TT)
        for (int idx = threadIdx.x; idx < TT * Bs; idx += blockDim.x) rg_u[idx] = 0.f;
    __syncthreads();
    rg_conv_tile(rg_u, TT, 1, (const float*)proj, ldp, x_col, conv_w, conv_b, state, state_stride, tok_seg, seg_start, seg_slot, t0, nt, c0, R, Bs, taps);
    __syncthreads();
    const float* wa = wa_t + (size_t)b * Bs * Bs;
    const float* wi = wi_t + (size_t)b * Bs * Bs;
    for (int o = blockIdx.z * RG_COLS + threadIdx.x; o < Bs; o += gridDim.z * RG_COLS) {
        float ra[TT], ri[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) { ra[tt] = ba[c0 + o]; ri[tt] = bi[c0 + o]; }
        // eight inputs' weights are fetched in one run of loads ahead of their multiply-adds (they come from the L2 cache, and
        // the few warps an SM holds of this kernel do not hide that latency otherwise)
        for (int k0 = 0; k0 < Bs; k0 += 8) {
            float va[8], vi[8];
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                const int k = min(k0 + kk, Bs - 1);
                va[kk] = rc_ld_weight(wa + (size_t)k * Bs + o); vi[kk] = rc_ld_weight(wi + (size_t)k * Bs + o);
            }
#pragma unroll
            for (int kk = 0; kk < 8; kk++) { xr_ld_fence(va[kk]); xr_ld_fence(vi[kk]); }
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                if (k0 + kk < Bs) {
                    const float4* uk = reinterpret_cast<const float4*>(rg_u + (size_t)(k0 + kk) * TT);
#pragma unroll
                    for (int q4 = 0; q4 < TT / 4; q4++) {
                        const float4 u = uk[q4];
                        ra[4 * q4] = fmaf(va[kk], u.x, ra[4 * q4]); ri[4 * q4] = fmaf(vi[kk], u.x, ri[4 * q4]);
                        ra[4 * q4 + 1] = fmaf(va[kk], u.y, ra[4 * q4 + 1]); ri[4 * q4 + 1] = fmaf(vi[kk], u.y, ri[4 * q4 + 1]);
                        ra[4 * q4 + 2] = fmaf(va[kk], u.z, ra[4 * q4 + 2]); ri[4 * q4 + 2] = fmaf(vi[kk], u.z, ri[4 * q4 + 2]);
                        ra[4 * q4 + 3] = fmaf(va[kk], u.w, ra[4 * q4 + 3]); ri[4 * q4 + 3] = fmaf(vi[kk], u.w, ri[4 * q4 + 3]);
                    }
                }
            }
        }
        const float rate = -c * rc_softplus(lam[c0 + o]);
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            if (tt < nt) {
                const size_t at = (size_t)(t0 + tt) * R + c0 + o;
                rg_finish(ra[tt], ri[tt], rg_u[(size_t)o * TT + tt], rate, a_out + at, b_out + at, proj + (size_t)(t0 + tt) * ldp + y_col + c0 + o);
            }
        }
    }
}

// The convolution alone, a thread an element: u [n][R].  Ahead of k_rglru_gates_few, whose many small blocks would each compute
// the whole tile again behind a chain of dependent loads.
__global__ void k_rglru_conv(const float* __restrict__ proj, long long ldp, int x_col, const float* __restrict__ conv_w,
                             const float* __restrict__ conv_b, const float* __restrict__ state, long long state_stride,
                             const int* __restrict__ tok_seg, const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                             float* __restrict__ u, int n, int R, int taps) {
    xr_pdl_launch();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * R) return;
    const int t = idx / R, ch = idx % R;
    const int seg = tok_seg[t], i = t - seg_start[seg];
    const float* tail = state + (size_t)seg_slot[seg] * state_stride + R;
    const float* w = conv_w + (size_t)ch * taps;
    float acc = conv_b[ch];
    xr_pdl_wait();
    for (int j = taps - 1; j >= 0; j--) {                            // oldest input first
        const int ip = i - j;
        const float x = ip >= 0 ? proj[(size_t)(t - j) * ldp + x_col + ch] : tail[(size_t)(taps - 1 + ip) * R + ch];
        acc = fmaf(w[taps - 1 - j], x, acc);
    }
    u[idx] = acc;
}

// Few tokens (a step of single tokens): a warp an output channel, its lanes share the inputs, so that the matrices' rows (as
// stored, [b][out][in]) are read by whole warps and every load of a thread is in flight at once.  A block: 8 tokens, 8 channels.
__global__ void __launch_bounds__(256)
k_rglru_gates_few(float* __restrict__ proj, long long ldp, int y_col, int x_col, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                  const float* __restrict__ wa, const float* __restrict__ wi, const float* __restrict__ ba, const float* __restrict__ bi,
                  const float* __restrict__ lam, const float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seg,
                  const int* __restrict__ seg_start, const int* __restrict__ seg_slot, float* __restrict__ a_out, float* __restrict__ b_out,
                  int n, int R, int Bs, int taps, float c, int groups, const float* __restrict__ u_in) {
    xr_pdl_launch();
    extern __shared__ __align__(16) float rg_u[];                // [8][Bs]
    const int t0 = blockIdx.x * 8, b = blockIdx.y / groups, c0 = b * Bs;
    const int nt = min(8, n - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o = (blockIdx.y % groups) * 8 + warp;
    xr_pdl_wait();
    for (int idx = threadIdx.x; idx < nt * Bs; idx += blockDim.x) rg_u[idx] = u_in[(size_t)(t0 + idx / Bs) * R + c0 + idx % Bs];
    __syncthreads();
    if (o >= Bs) return;
    const float* rowa = wa + ((size_t)b * Bs + o) * Bs;
    const float* rowi = wi + ((size_t)b * Bs + o) * Bs;
    float ra[8], ri[8];
#pragma unroll
    for (int tt = 0; tt < 8; tt++) { ra[tt] = 0.f; ri[tt] = 0.f; }
#pragma unroll 4
    for (int k = lane; k < Bs; k += 32) {
        const float va = rowa[k], vi = rowi[k];
#pragma unroll
        for (int tt = 0; tt < 8; tt++) {
            const float u = tt < nt ? rg_u[tt * Bs + k] : 0.f;
            ra[tt] = fmaf(va, u, ra[tt]);
            ri[tt] = fmaf(vi, u, ri[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < 8; tt++) { ra[tt] = xr_warp_sum(ra[tt]); ri[tt] = xr_warp_sum(ri[tt]); }
    const float rate = -c * rc_softplus(lam[c0 + o]);
#pragma unroll
    for (int tt = 0; tt < 8; tt++) {
        if (lane == tt && tt < nt) {
            const size_t at = (size_t)(t0 + tt) * R + c0 + o;
            rg_finish(ra[tt] + ba[c0 + o], ri[tt] + bi[c0 + o], rg_u[tt * Bs + o], rate, a_out + at, b_out + at, proj + (size_t)(t0 + tt) * ldp + y_col + c0 + o);
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
    // The walk is a chain of dependent multiply-adds and nothing else hides the loads' latency: eight tokens' values are fetched in
    // one run of loads, and the next eight are on their way while these are walked.  (The gated branch's columns hold their
    // activation already: the gates kernel left it there.)
    float a[8], b[8], y[8], na[8], nb[8], ny[8];
    auto fetch = [&](int i0, float* fa, float* fb, float* fy) {
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const size_t t = (size_t)(start + min(i0 + k, len - 1));
            fa[k] = xr_ld_now(a_in + t * R + ch); fb[k] = xr_ld_now(b_in + t * R + ch); fy[k] = xr_ld_now(proj + t * ldp + y_col + ch);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) { xr_ld_fence(fa[k]); xr_ld_fence(fb[k]); xr_ld_fence(fy[k]); }
    };
    if (len > 0) fetch(0, na, nb, ny);
    for (int i0 = 0; i0 < len; i0 += 8) {
#pragma unroll
        for (int k = 0; k < 8; k++) { a[k] = na[k]; b[k] = nb[k]; y[k] = ny[k]; }
        if (i0 + 8 < len) fetch(i0 + 8, na, nb, ny);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (i0 + k < len) {
                S = fmaf(a[k], S, b[k]);
                out[(size_t)(start + i0 + k) * R + ch] = xr_from_f32<T>(S * y[k]);
            }
        }
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
// conv_w [R][taps], conv_b [R]; wa_t, wi_t [B][R/B (in)][R/B (out)] and wa, wi the same matrices as stored, [B][out][in]; ba, bi,
// lam [R]; all float32.
// state [slots][state_stride] float32: S [R], tail [taps-1][R].  a_s, b_s, u_s [n][R] float32 scratch.  out [n][R] dtype `dtype`.
XR_EXPORT int xr_rglru(float* proj, long long ldp, int y_col, int x_col, const float* conv_w, const float* conv_b, const float* wa_t,
                       const float* wi_t, const float* wa, const float* wi, const float* ba, const float* bi, const float* lam, float* state, long long state_stride,
                       const int* tok_seg, const int* seg_start, const int* seg_len, const int* seg_slot, float* a_s, float* b_s, float* u_s, void* out,
                       int dtype, int n, int n_seg, int R, int B, int taps, float c, cudaStream_t stream) {
    if (n < 1 || n_seg < 1 || R < 1 || B < 1 || R % B || taps < 1 || taps > RG_MAX_TAPS || n_seg > 65535 || B > 65535 ||
        state_stride < (long long)R * taps)
        return XR_ERR_ARG;
    const int Bs = R / B;
    // (a tile of eight tokens of one channel block in shared memory: wide blocks ask for more than the default 48 KB)
    const size_t smem8 = (size_t)8 * Bs * sizeof(float);
    if (smem8 > 200 * 1024) return XR_ERR_ARG;
    if (smem8 > 48 * 1024 &&
        (cudaFuncSetAttribute(k_rglru_gates_few, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem8) != cudaSuccess ||
         cudaFuncSetAttribute(k_rglru_gates<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem8) != cudaSuccess))
        return XR_ERR_LAUNCH;
#define RG_ARGS(A, I) proj, ldp, y_col, x_col, conv_w, conv_b, A, I, ba, bi, lam, (const float*)state, state_stride, tok_seg, seg_start, seg_slot, a_s, b_s, n, R, Bs, taps, c
    if (n <= 16) {
        const int groups = (Bs + 7) / 8;
        xr_launch(k_rglru_conv, dim3((n * R + 255) / 256), dim3(256), 0, stream, (const float*)proj, ldp, x_col, conv_w, conv_b, (const float*)state,
                  state_stride, tok_seg, seg_start, seg_slot, u_s, n, R, taps);
        xr_launch(k_rglru_gates_few, dim3((n + 7) / 8, B * groups), dim3(256), smem8, stream, RG_ARGS(wa, wi), groups, (const float*)u_s);
    } else if (n >= 64 && (size_t)32 * Bs * sizeof(float) <= 48 * 1024) {
        xr_launch((k_rglru_gates<32>), dim3((n + 31) / 32, B, (Bs + RG_COLS - 1) / RG_COLS), dim3(RG_COLS), (size_t)32 * Bs * sizeof(float), stream, RG_ARGS(wa_t, wi_t));
    } else {
        xr_launch((k_rglru_gates<8>), dim3((n + 7) / 8, B, (Bs + RG_COLS - 1) / RG_COLS), dim3(RG_COLS), smem8, stream, RG_ARGS(wa_t, wi_t));
    }
#undef RG_ARGS
    dim3 gs((R + 127) / 128, n_seg);
    // (a step with long portions is a few long-lived blocks: they start behind the gates kernel, not into its last wave)
    const bool walk = n > 4 * n_seg;
    if (walk && dtype == XR_F32)
        xr_launch_behind((k_rglru_scan<float>), gs, dim3(128), 0, stream, (const float*)proj, ldp, y_col, x_col, (const float*)a_s, (const float*)b_s, state,
                         state_stride, seg_start, seg_len, seg_slot, (float*)out, R, taps);
    else if (walk && dtype == XR_BF16)
        xr_launch_behind((k_rglru_scan<__nv_bfloat16>), gs, dim3(128), 0, stream, (const float*)proj, ldp, y_col, x_col, (const float*)a_s, (const float*)b_s, state,
                         state_stride, seg_start, seg_len, seg_slot, (__nv_bfloat16*)out, R, taps);
    else if (dtype == XR_F32)
        xr_launch((k_rglru_scan<float>), gs, dim3(128), 0, stream, (const float*)proj, ldp, y_col, x_col, (const float*)a_s, (const float*)b_s, state,
                  state_stride, seg_start, seg_len, seg_slot, (float*)out, R, taps);
    else if (dtype == XR_BF16)
        xr_launch((k_rglru_scan<__nv_bfloat16>), gs, dim3(128), 0, stream, (const float*)proj, ldp, y_col, x_col, (const float*)a_s, (const float*)b_s, state,
                  state_stride, seg_start, seg_len, seg_slot, (__nv_bfloat16*)out, R, taps);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// A block of eight warps owns VC * 8 value columns of one head, a warp VC of them; a warp's lanes share the key rows (lane l has rows l JD ..
// l JD + JD - 1), so a column's state lies in JD registers of every lane.  Per token a lane updates its JD x VC state elements
// and adds them, times q, into VC sums.  The sums of 32 / VC tokens are added over the lanes together: 32 numbers a lane, halved
// five times by an exchange with the lane 16, 8, 4, 2, 1 away, after which every lane holds one (token, column) sum and stores
// it: 31 shuffles for 32 / VC tokens, and one chain of five exchanges instead of one per token.
// The tokens' q, k and v come in chunks of CH tokens through shared memory, two buffers: the next chunk's values are fetched into
// registers before this chunk is walked and stored behind it (16 bytes a load where sizes and addresses allow: VEC).  A step of
// many tokens applies silu to the rows beforehand, in
// place (k_silu_cols); a step of few applies it on the way into shared memory.
#define DA_WARPS 8

__global__ void k_silu_cols(float* __restrict__ rows, long long ld, int cols, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float* p = rows + (i / cols) * ld + (i % cols);
        *p = rc_silu(*p);
    }
}

template <int JD, int VC, int CH, bool VEC>
__global__ void __launch_bounds__(32 * DA_WARPS)
k_decay_scan(const float* __restrict__ proj, long long ldp, int q_col, int k_col, int v_col, const float* __restrict__ decay,
             float* __restrict__ state, long long state_stride, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
             const int* __restrict__ seg_slot, float* __restrict__ o, int H, int D, int V, int activated) {
    xr_pdl_launch();
    constexpr int COLS = VC * DA_WARPS, DP = 32 * JD, RW = 2 * DP + COLS, TB = 32 / VC;
    constexpr int PER = (CH * RW + 32 * DA_WARPS - 1) / (32 * DA_WARPS);
    static_assert(CH % TB == 0, "a chunk is whole batches of tokens");
    __shared__ __align__(16) float da_sm[2 * CH * RW];       // a token's row: q [DP], k [DP] (zeros behind D), the block's v [COLS]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int vb = blockIdx.x * COLS, v0 = vb + warp * VC, h = blockIdx.y, seg = blockIdx.z;
    const int start = seg_start[seg], len = seg_len[seg];
    const float dec = decay[h];
    float* st = state + (size_t)seg_slot[seg] * state_stride + (size_t)h * D * V;
    xr_pdl_wait();
    float s[VC][JD];
#pragma unroll
    for (int j = 0; j < JD; j++) {
        const int d = lane * JD + j;
#pragma unroll
        for (int c = 0; c < VC; c++) s[c][j] = (d < D && v0 + c < V) ? st[(size_t)d * V + v0 + c] : 0.f;
    }
    constexpr int PER4 = (CH * RW / 4 + 32 * DA_WARPS - 1) / (32 * DA_WARPS);
    float stage[VEC ? 1 : PER];
    float4 stage4[VEC ? PER4 : 1];
    // (loads that stay where they are written: left alone, the compiler moves them down to their use behind the walk to save
    // registers, and the chunk then waits for them one after the other)
    auto load = [&](int chunk) {
        if constexpr (VEC) {
#pragma unroll
            for (int k = 0; k < PER4; k++) {
                const int e = 4 * (threadIdx.x + k * 32 * DA_WARPS);
                const int tok = e / RW, cc = e % RW, i = chunk * CH + tok;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (tok < CH && i < len) {
                    const float* row = proj + (size_t)(start + i) * ldp;
                    if (cc < DP) { if (cc < D) v = xr_ld_now4(reinterpret_cast<const float4*>(row + q_col + h * D + cc)); }
                    else if (cc < 2 * DP) { if (cc - DP < D) v = xr_ld_now4(reinterpret_cast<const float4*>(row + k_col + h * D + cc - DP)); }
                    else if (vb + cc - 2 * DP < V) v = xr_ld_now4(reinterpret_cast<const float4*>(row + v_col + h * V + vb + cc - 2 * DP));
                }
                stage4[k] = v;
            }
#pragma unroll
            for (int k = 0; k < PER4; k++) xr_ld_fence(stage4[k]);
        } else {
#pragma unroll
            for (int k = 0; k < PER; k++) {
                const int e = threadIdx.x + k * 32 * DA_WARPS;
                const int tok = e / RW, cc = e % RW, i = chunk * CH + tok;
                float v = 0.f;
                if (tok < CH && i < len) {
                    const float* row = proj + (size_t)(start + i) * ldp;
                    if (cc < DP) { if (cc < D) v = xr_ld_now(row + q_col + h * D + cc); }
                    else if (cc < 2 * DP) { if (cc - DP < D) v = xr_ld_now(row + k_col + h * D + cc - DP); }
                    else if (vb + cc - 2 * DP < V) v = xr_ld_now(row + v_col + h * V + vb + cc - 2 * DP);
                }
                stage[k] = v;
            }
#pragma unroll
            for (int k = 0; k < PER; k++) xr_ld_fence(stage[k]);
        }
    };
    auto store = [&](int buf) {
        if constexpr (VEC) {
#pragma unroll
            for (int k = 0; k < PER4; k++) {
                const int e = 4 * (threadIdx.x + k * 32 * DA_WARPS);
                float4 v = stage4[k];
                if (!activated) { v.x = rc_silu(v.x); v.y = rc_silu(v.y); v.z = rc_silu(v.z); v.w = rc_silu(v.w); }
                if (e < CH * RW) *reinterpret_cast<float4*>(da_sm + buf * CH * RW + e) = v;
            }
        } else {
#pragma unroll
            for (int k = 0; k < PER; k++) {
                const int e = threadIdx.x + k * 32 * DA_WARPS;
                if (e < CH * RW) da_sm[buf * CH * RW + e] = activated ? stage[k] : rc_silu(stage[k]);
            }
        }
    };
    const int chunks = (len + CH - 1) / CH;
    if (chunks > 0) { load(0); store(0); }
    __syncthreads();
    for (int ch = 0; ch < chunks; ch++) {
        if (ch + 1 < chunks) load(ch + 1);
        const float* base = da_sm + (ch & 1) * CH * RW;
        const int here = min(CH, len - ch * CH);
#pragma unroll 1
        for (int t0 = 0; t0 < here; t0 += TB) {
            float acc[TB * VC];
#pragma unroll
            for (int tb = 0; tb < TB; tb++) {
#pragma unroll
                for (int c = 0; c < VC; c++) acc[tb * VC + c] = 0.f;
                if (t0 + tb < here) {
                    const float* row = base + (t0 + tb) * RW;
                    float q[JD], k[JD], v[VC];
                    if constexpr (JD % 4 == 0) {
#pragma unroll
                        for (int j = 0; j < JD; j += 4) {
                            const float4 a = *reinterpret_cast<const float4*>(row + lane * JD + j);
                            const float4 b = *reinterpret_cast<const float4*>(row + DP + lane * JD + j);
                            q[j] = a.x; q[j + 1] = a.y; q[j + 2] = a.z; q[j + 3] = a.w;
                            k[j] = b.x; k[j + 1] = b.y; k[j + 2] = b.z; k[j + 3] = b.w;
                        }
                    } else if constexpr (JD == 2) {
                        const float2 a = *reinterpret_cast<const float2*>(row + lane * 2);
                        const float2 b = *reinterpret_cast<const float2*>(row + DP + lane * 2);
                        q[0] = a.x; q[1] = a.y; k[0] = b.x; k[1] = b.y;
                    } else {
#pragma unroll
                        for (int j = 0; j < JD; j++) { q[j] = row[lane * JD + j]; k[j] = row[DP + lane * JD + j]; }
                    }
                    if constexpr (VC % 4 == 0) {
#pragma unroll
                        for (int c = 0; c < VC; c += 4) {
                            const float4 a = *reinterpret_cast<const float4*>(row + 2 * DP + warp * VC + c);
                            v[c] = a.x; v[c + 1] = a.y; v[c + 2] = a.z; v[c + 3] = a.w;
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < VC; c++) v[c] = row[2 * DP + warp * VC + c];
                    }
#pragma unroll
                    for (int j = 0; j < JD; j++) {
#pragma unroll
                        for (int c = 0; c < VC; c++) {
                            s[c][j] = fmaf(dec, s[c][j], k[j] * v[c]);
                            acc[tb * VC + c] = fmaf(s[c][j], q[j], acc[tb * VC + c]);
                        }
                    }
                }
            }
            // 32 sums a lane -> one: a lane whose bit is set keeps the upper half of what it carries and hands over the lower one
#pragma unroll
            for (int w = 16, bit = 16; w > 0; w >>= 1, bit >>= 1) {
                const bool upper = lane & bit;
#pragma unroll
                for (int c = 0; c < w; c++) {
                    const float send = upper ? acc[c] : acc[c + w], keep = upper ? acc[c + w] : acc[c];
                    acc[c] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                }
            }
            // the sum this lane holds: bit 16 of the lane chose the upper 16 of 32, bit 8 the upper 8 of those, ...: the lane's number
            // read from its highest bit down is the sum's index
            const int mine = ((lane & 16) ? 16 : 0) + ((lane & 8) ? 8 : 0) + ((lane & 4) ? 4 : 0) + ((lane & 2) ? 2 : 0) + (lane & 1);
            const int tb = mine / VC, c = mine % VC;
            if (t0 + tb < here && v0 + c < V) o[(size_t)(start + ch * CH + t0 + tb) * H * V + (size_t)h * V + v0 + c] = acc[0];
        }
        if (ch + 1 < chunks) store((ch + 1) & 1);
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < JD; j++) {
        const int d = lane * JD + j;
#pragma unroll
        for (int c = 0; c < VC; c++)
            if (d < D && v0 + c < V) st[(size_t)d * V + v0 + c] = s[c][j];
    }
}

// proj [n][ldp] float32: pre-activations of q at q_col [H][D], k at k_col [H][D], v at v_col [H][V] (`cols` columns from the first
// of them to the last of v, which a step of many tokens activates in place); decay [H] float32; state [slots][state_stride]
// float32, S [H][D][V];  o [n][H V] float32 receives the read-outs.
XR_EXPORT int xr_decay_attention(float* proj, long long ldp, int q_col, int k_col, int v_col, const float* decay, float* state,
                                 long long state_stride, const int* seg_start, const int* seg_len, const int* seg_slot, float* o, int n, int n_seg,
                                 int H, int D, int V, cudaStream_t stream) {
    if (n < 1 || n_seg < 1 || H < 1 || D < 1 || V < 1 || D > 256 || n_seg > 65535 || H > 65535 || state_stride < (long long)H * D * V)
        return XR_ERR_ARG;
    // q, k, v lie side by side from q_col on (the caller's layout): one pass activates them all
    const bool many = n > 16 && k_col == q_col + H * D && v_col == k_col + H * D;
    if (many) {
        const size_t total = (size_t)n * (2 * H * D + H * V);
        const int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
        xr_launch(k_silu_cols, dim3(blocks), dim3(256), 0, stream, proj + q_col, ldp, 2 * H * D + H * V, total);
    }
    // (a step with long portions is a few long-lived blocks: they start behind the kernel ahead, not into its last wave)
    const bool walk = n > 4 * n_seg;
    // 16 bytes a load where every row, column offset and size falls on a 16-byte border
    const bool vec = !((D | V | ldp | q_col | k_col | v_col) & 3) && !((uintptr_t)proj & 15);
#define DS_ARGS(JD, VC, CH) dim3((V + VC * DA_WARPS - 1) / (VC * DA_WARPS), H, n_seg), dim3(32 * DA_WARPS), 0, stream,                      \
                            (const float*)proj, ldp, q_col, k_col, v_col, decay, state, state_stride, seg_start, seg_len, seg_slot, o, H, D, V, many ? 1 : 0
#define DS1(JD, VC, CH, VEC)                                                                                                                 \
    do {                                                                                                                                     \
        if (walk) xr_launch_behind((k_decay_scan<JD, VC, CH, VEC>), DS_ARGS(JD, VC, CH));                                                    \
        else xr_launch((k_decay_scan<JD, VC, CH, VEC>), DS_ARGS(JD, VC, CH));                                                                \
    } while (0)
#define DS(JD, VC, CH)                                                                                                                       \
    do {                                                                                                                                     \
        if (vec) DS1(JD, VC, CH, true);                                                                                                      \
        else DS1(JD, VC, CH, false);                                                                                                         \
    } while (0)
    if (D <= 32) DS(1, 2, 16);
    else if (D <= 64) DS(2, 2, 16);
    else if (D <= 128) DS(4, 2, 16);
    else DS(8, 4, 8);
#undef DS
#undef DS1
#undef DS_ARGS
    return xr_launch_status();
}
