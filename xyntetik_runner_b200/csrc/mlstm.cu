// Matrix-memory recurrence (the mLSTM cell of xLSTM) with a stabilising running maximum, per request and head.
//
// State per (request slot, head): S [D][V], n [D], m (float32, zero when the slot is assigned).  For a token with
// query q (times D^-1/2), key k, value v, pre-activations a_i, a_f of the gates and cap c:
//   li = c tanh(a_i / c)                      (log of the input gate)
//   lf = logsigmoid(c tanh(a_f / c))          (log of the forget gate)
//   m' = max(lf + m, li);  f = exp(lf + m - m');  i = exp(li - m')
//   S' = f S + i k v^T;    n' = f n + i k
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
// Everything above is float32; q, k, v come from the projections in the activation dtype.
//
// Three kernels.  k_mlstm_gates walks a request's tokens once per head: m, f, i, n and the denominator of every token
// (scalars per token and head), and leaves n and m in the state.  k_mlstm_scan walks them once per (head, slice of
// 32 value columns) with S in shared memory, each thread updating its own cells, and writes o.  k_mlstm_out divides
// each head's o by its root mean square, multiplies by the norm weight and the sigmoid of the output gate.
// The walk is token by token in both, so the state after a token does not depend on how the tokens were cut into
// steps, bit for bit.
#include "common.cuh"
#include <math.h>

#define ML_VS 32          // value columns per block of the scan
#define ML_RG 8           // row groups (warps) per block of the scan
#define ML_CHUNK 8        // tokens whose q, k, v are staged together (the register scan stages one token per warp: = ML_RG)

__device__ __forceinline__ float ml_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// state layout per slot: [H][D * V + D + 1]
__device__ __forceinline__ size_t ml_state_head(int D, int V) { return (size_t)D * V + D + 1; }

// Tokens are taken `stage` at a time, in four steps a chunk, so that nothing but a few scalar operations per token is
// serial: (1) the logarithms of the gates of the chunk's tokens, a thread a token; (2) one thread walks the chunk's
// scalars: m, f, i and exp(-m) of every token; (3) every thread owns elements of n and walks the chunk with them,
// n <- f n + i k, leaving n[d] q[d] of every token in shared memory; (4) the warps sum those products token by token
// (always in the same order) and write (f, i, denominator).
template <typename T>
__global__ void __launch_bounds__(256)
k_mlstm_gates(const T* __restrict__ proj, long long ldp, int q_col, int k_col, const float* __restrict__ gates,
              float* __restrict__ state, float* __restrict__ coef, const int* __restrict__ seg_start,
              const int* __restrict__ seg_len, const int* __restrict__ seg_slot, int H, int D, int V, float cap, int stage) {
    xr_pdl_launch();
    extern __shared__ float gsm[];
    float* prod = gsm;                          // [stage][D]: n[d] q[d] of the chunk's tokens
    float* lg = prod + (size_t)stage * D;       // [stage][2]: log input gate, log forget gate
    float* fi = lg + 2 * stage;                 // [stage][3]: f, i, exp(-m)
    __shared__ float m_run;
    const int h = blockIdx.x, seg = blockIdx.y;
    const int start = seg_start[seg], len = seg_len[seg], slot = seg_slot[seg];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    xr_pdl_wait();
    float* st = state + ((size_t)slot * H + h) * ml_state_head(D, V);
    float* n_g = st + (size_t)D * V;
    constexpr int OWN = 4;                      // elements of n per thread: D <= 4 * 256
    float nreg[OWN];
#pragma unroll
    for (int i = 0; i < OWN; i++) { const int d = threadIdx.x + i * blockDim.x; nreg[i] = d < D ? n_g[d] : 0.f; }
    if (threadIdx.x == 0) m_run = n_g[D];
    const float qs = 1.0f / sqrtf((float)D);
    for (int j0 = 0; j0 < len; j0 += stage) {
        const int cnt = min(stage, len - j0);
        for (int j = threadIdx.x; j < cnt; j += blockDim.x) {
            const int t = start + j0 + j;
            const float ai = gates[(size_t)t * 2 * H + h], af = gates[(size_t)t * 2 * H + H + h];
            lg[2 * j] = cap * tanhf(ai / cap);
            lg[2 * j + 1] = ml_logsigmoid(cap * tanhf(af / cap));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = m_run;
            for (int j = 0; j < cnt; j++) {
                const float li = lg[2 * j], lf = lg[2 * j + 1];
                const float m_new = fmaxf(lf + m, li);
                fi[3 * j] = expf(lf + m - m_new); fi[3 * j + 1] = expf(li - m_new); fi[3 * j + 2] = expf(-m_new);
                m = m_new;
            }
            m_run = m;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < OWN; i++) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d < D) {
                float nn = nreg[i];
#pragma unroll 8
                for (int j = 0; j < cnt; j++) {
                    const T* row = proj + (size_t)(start + j0 + j) * ldp + (size_t)h * D + d;
                    nn = fmaf(fi[3 * j], nn, fi[3 * j + 1] * xr_to_f32<T>(row[k_col]));
                    prod[j * D + d] = nn * (xr_to_f32<T>(row[q_col]) * qs);
                }
                nreg[i] = nn;
            }
        }
        __syncthreads();
        for (int j = warp; j < cnt; j += nw) {
            float part = 0.f;
            for (int d = lane; d < D; d += 32) part += prod[j * D + d];
            const float qn = xr_warp_sum(part);
            if (lane == 0) {
                float* c = coef + ((size_t)(start + j0 + j) * H + h) * 3;
                c[0] = fi[3 * j]; c[1] = fi[3 * j + 1]; c[2] = fmaxf(fabsf(qn), fi[3 * j + 2]) + 1e-6f;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < OWN; i++) { const int d = threadIdx.x + i * blockDim.x; if (d < D) n_g[d] = nreg[i]; }
    if (threadIdx.x == 0) n_g[D] = m_run;
}

template <typename T>
__global__ void __launch_bounds__(ML_VS * ML_RG)
k_mlstm_scan_wide(const T* __restrict__ proj, long long ldp, int q_col, int k_col, int v_col, const float* __restrict__ coef,
             float* __restrict__ state, float* __restrict__ out, const int* __restrict__ seg_start,
             const int* __restrict__ seg_len, const int* __restrict__ seg_slot, int H, int D, int V) {
    xr_pdl_launch();
    extern __shared__ float sm[];
    float* S = sm;                                   // [D][ML_VS]
    float* ks = S + (size_t)D * ML_VS;               // [ML_CHUNK][D]
    float* qsm = ks + (size_t)ML_CHUNK * D;          // [ML_CHUNK][D]
    float* vs = qsm + (size_t)ML_CHUNK * D;          // [ML_CHUNK][ML_VS]
    float* red = vs + ML_CHUNK * ML_VS;              // [ML_CHUNK][ML_RG][ML_VS]
    float* cf = red + ML_CHUNK * ML_RG * ML_VS;      // [ML_CHUNK][3]
    const int col = threadIdx.x & (ML_VS - 1), rg = threadIdx.x / ML_VS;
    const int v0 = blockIdx.x * ML_VS, h = blockIdx.y, seg = blockIdx.z;
    const int start = seg_start[seg], len = seg_len[seg], slot = seg_slot[seg];
    const bool col_ok = v0 + col < V;
    xr_pdl_wait();
    float* Sg = state + ((size_t)slot * H + h) * ml_state_head(D, V);
    for (int d = rg; d < D; d += ML_RG) S[d * ML_VS + col] = col_ok ? Sg[(size_t)d * V + v0 + col] : 0.f;
    const float qscale = 1.0f / sqrtf((float)D);
    for (int j0 = 0; j0 < len; j0 += ML_CHUNK) {
        const int cnt = min(ML_CHUNK, len - j0);
        __syncthreads();
        for (int e = threadIdx.x; e < cnt * D; e += blockDim.x) {
            const int j = e / D, d = e % D;
            const T* row = proj + (size_t)(start + j0 + j) * ldp;
            ks[j * D + d] = xr_to_f32<T>(row[k_col + h * D + d]);
            qsm[j * D + d] = xr_to_f32<T>(row[q_col + h * D + d]) * qscale;
        }
        for (int e = threadIdx.x; e < cnt * ML_VS; e += blockDim.x) {
            const int j = e / ML_VS, c = e % ML_VS;
            vs[e] = v0 + c < V ? xr_to_f32<T>(proj[(size_t)(start + j0 + j) * ldp + v_col + h * V + v0 + c]) : 0.f;
        }
        for (int e = threadIdx.x; e < cnt * 3; e += blockDim.x) cf[e] = coef[((size_t)(start + j0 + e / 3) * H + h) * 3 + e % 3];
        __syncthreads();
        for (int j = 0; j < cnt; j++) {
            const float f = cf[j * 3], iv = cf[j * 3 + 1] * vs[j * ML_VS + col];
            float num = 0.f;
            for (int d = rg; d < D; d += ML_RG) {
                const float s = fmaf(f, S[d * ML_VS + col], iv * ks[j * D + d]);
                S[d * ML_VS + col] = s;
                num = fmaf(s, qsm[j * D + d], num);
            }
            red[(j * ML_RG + rg) * ML_VS + col] = num;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < cnt * ML_VS; e += blockDim.x) {
            const int j = e / ML_VS, c = e % ML_VS;
            if (v0 + c >= V) continue;
            float num = 0.f;
#pragma unroll
            for (int r = 0; r < ML_RG; r++) num += red[(j * ML_RG + r) * ML_VS + c];
            out[(size_t)(start + j0 + j) * H * V + (size_t)h * V + v0 + c] = num / cf[j * 3 + 2];
        }
    }
    __syncthreads();
    if (col_ok)
        for (int d = rg; d < D; d += ML_RG) Sg[(size_t)d * V + v0 + col] = S[d * ML_VS + col];
}

// The same walk with S in registers, for key sizes up to 256: thread (row group rg, column) keeps rows
// rg * RPT .. rg * RPT + RPT - 1 of its column (RPT = rows per thread, 8 * RPT >= D; rows beyond D stay zero), and reads
// the staged k and q of a token as float4 that the whole warp shares.
template <typename T, int RPT>
__global__ void __launch_bounds__(ML_VS * ML_RG)
k_mlstm_scan(const T* __restrict__ proj, long long ldp, int q_col, int k_col, int v_col, const float* __restrict__ coef,
             float* __restrict__ state, float* __restrict__ out, const int* __restrict__ seg_start,
             const int* __restrict__ seg_len, const int* __restrict__ seg_slot, int H, int D, int V) {
    xr_pdl_launch();
    constexpr int DP = ML_RG * RPT;
    __shared__ __align__(16) float ks[ML_CHUNK][DP];
    __shared__ __align__(16) float qsm[ML_CHUNK][DP];
    __shared__ float vs[ML_CHUNK][ML_VS];
    __shared__ float red[ML_CHUNK][ML_RG][ML_VS];
    __shared__ float cf[ML_CHUNK][3];
    const int col = threadIdx.x & (ML_VS - 1), rg = threadIdx.x / ML_VS;
    const int v0 = blockIdx.x * ML_VS, h = blockIdx.y, seg = blockIdx.z;
    const int start = seg_start[seg], len = seg_len[seg], slot = seg_slot[seg];
    const bool col_ok = v0 + col < V;
    xr_pdl_wait();
    float* Sg = state + ((size_t)slot * H + h) * ml_state_head(D, V);
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int d = rg * RPT + i;
        S[i] = (col_ok && d < D) ? Sg[(size_t)d * V + v0 + col] : 0.f;
    }
    const float qscale = 1.0f / sqrtf((float)D);
    // the next chunk's k, q, v and scalars are on their way to registers while this chunk is computed
    constexpr int NL = ML_CHUNK * DP / (ML_VS * ML_RG);           // elements of k (and of q) per thread and chunk
    T kreg[NL], qreg[NL], vreg = xr_from_f32<T>(0.f);
    float creg = 0.f;
    auto prefetch = [&](int j0) {
        const int cnt = min(ML_CHUNK, len - j0);
#pragma unroll
        for (int i = 0; i < NL; i++) {
            const int e = threadIdx.x + i * (ML_VS * ML_RG), j = e / DP, d = e % DP;
            const bool ok = j < cnt && d < D;
            const T* row = proj + (size_t)(start + j0 + (ok ? j : 0)) * ldp + (size_t)h * D + (ok ? d : 0);
            kreg[i] = ok ? row[k_col] : xr_from_f32<T>(0.f);
            qreg[i] = ok ? row[q_col] : xr_from_f32<T>(0.f);
        }
        const int j = threadIdx.x / ML_VS;
        vreg = (j < cnt && col_ok) ? proj[(size_t)(start + j0 + j) * ldp + v_col + h * V + v0 + col] : xr_from_f32<T>(0.f);
        if ((int)threadIdx.x < cnt * 3) creg = coef[((size_t)(start + j0 + threadIdx.x / 3) * H + h) * 3 + threadIdx.x % 3];
    };
    prefetch(0);
    for (int j0 = 0; j0 < len; j0 += ML_CHUNK) {
        const int cnt = min(ML_CHUNK, len - j0);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NL; i++) {
            const int e = threadIdx.x + i * (ML_VS * ML_RG), j = e / DP, d = e % DP;
            ks[j][d] = xr_to_f32<T>(kreg[i]);
            qsm[j][d] = xr_to_f32<T>(qreg[i]) * qscale;
        }
        vs[threadIdx.x / ML_VS][col] = xr_to_f32<T>(vreg);
        if (threadIdx.x < ML_CHUNK * 3) cf[threadIdx.x / 3][threadIdx.x % 3] = creg;
        __syncthreads();
        if (j0 + ML_CHUNK < len) prefetch(j0 + ML_CHUNK);
        for (int j = 0; j < cnt; j++) {
            const float f = cf[j][0], iv = cf[j][1] * vs[j][col];
            const float4* k4 = reinterpret_cast<const float4*>(&ks[j][rg * RPT]);
            const float4* q4 = reinterpret_cast<const float4*>(&qsm[j][rg * RPT]);
            float num = 0.f;
#pragma unroll
            for (int i = 0; i < RPT / 4; i++) {
                const float4 kk = k4[i], qq = q4[i];
                S[4 * i] = fmaf(f, S[4 * i], iv * kk.x);         num = fmaf(S[4 * i], qq.x, num);
                S[4 * i + 1] = fmaf(f, S[4 * i + 1], iv * kk.y); num = fmaf(S[4 * i + 1], qq.y, num);
                S[4 * i + 2] = fmaf(f, S[4 * i + 2], iv * kk.z); num = fmaf(S[4 * i + 2], qq.z, num);
                S[4 * i + 3] = fmaf(f, S[4 * i + 3], iv * kk.w); num = fmaf(S[4 * i + 3], qq.w, num);
            }
            red[j][rg][col] = num;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < cnt * ML_VS; e += blockDim.x) {
            const int j = e / ML_VS, c = e % ML_VS;
            if (v0 + c >= V) continue;
            float num = 0.f;
#pragma unroll
            for (int r = 0; r < ML_RG; r++) num += red[j][r][c];
            out[(size_t)(start + j0 + j) * H * V + (size_t)h * V + v0 + c] = num / cf[j][2];
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int d = rg * RPT + i;
            if (d < D) Sg[(size_t)d * V + v0 + col] = S[i];
        }
    }
}

// o [n][H][V] float32 -> y [n][H * V] (activation dtype): o / rms(o over the head) * w * act(g); one warp per (token, head).
// The weight of head h starts at w + h * w_head (0: one weight of V values for all heads); act is the sigmoid, or SiLU
// with `gate_silu`.
// (TG: the gate's dtype, the activation dtype or float32)
template <typename T, typename TG = T>
__global__ void __launch_bounds__(128)
k_mlstm_out(const float* __restrict__ o, const TG* __restrict__ proj, long long ldp, int g_col, const float* __restrict__ w,
            T* __restrict__ y, int n, int H, int V, float eps, int w_head, int gate_silu) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 4 + warp;
    if (idx >= (long long)n * H) return;
    const int t = (int)(idx / H), h = (int)(idx % H);
    const float* src = o + ((size_t)t * H + h) * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = xr_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    const TG* g = proj + (size_t)t * ldp + g_col + (size_t)h * V;
    T* dst = y + (size_t)t * H * V + (size_t)h * V;
    for (int i = lane; i < V; i += 32) {
        const float z = xr_to_f32<TG>(g[i]);
        float gate = 1.0f / (1.0f + expf(-z));
        if (gate_silu) gate *= z;
        dst[i] = xr_from_f32<T>(src[i] * inv * w[(size_t)h * w_head + i] * gate);
    }
}

// proj [n][ldp] (activation dtype): q at q_col [H][D], k at k_col [H][D], v at v_col [H][V], output gate at g_col [H][V];
// gates [n][2H] float32 (input-gate pre-activations, then forget-gate ones, biases included);
// state [slots][H][D*V + D + 1] float32;  coef [n][H][3], o [n][H][V]: float32 scratch;  y [n][H*V] activation dtype.
XR_EXPORT int xr_mlstm(const void* proj, int dtype, long long ldp, int q_col, int k_col, int v_col, int g_col, const float* gates,
                       float* state, float* coef, float* o, const float* norm_w, void* y, const int* seg_start,
                       const int* seg_len, const int* seg_slot, int n, int n_seg, int H, int D, int V, float cap, float eps,
                       cudaStream_t stream) {
    if (n < 1 || n_seg < 1 || H < 1 || D < 1 || V < 1 || !(cap > 0.f) || n_seg > 65535 || H > 65535) return XR_ERR_ARG;
    // tokens a chunk of the gates kernel: what fits 44 KB of shared memory, at most 32; its threads own up to 4 elements of n each
    if (D > 1024) return XR_ERR_ARG;
    int stage = (int)((44 * 1024 / sizeof(float)) / ((size_t)D + 5));
    stage = stage > 32 ? 32 : stage;
    const size_t smem_g = (size_t)stage * (D + 5) * sizeof(float);
    const size_t smem_s = ((size_t)D * ML_VS + 2 * (size_t)ML_CHUNK * D + ML_CHUNK * ML_VS + ML_CHUNK * ML_RG * ML_VS + ML_CHUNK * 3) * sizeof(float);
    if (smem_g > 48 * 1024 || smem_s > 220 * 1024) return XR_ERR_ARG;
    dim3 gg(H, n_seg), gs((V + ML_VS - 1) / ML_VS, H, n_seg);
    const long long warps = (long long)n * H;
    const unsigned gb = (unsigned)((warps + 3) / 4);
#define SCAN_ARGS(T) gs, dim3(ML_VS * ML_RG), 0, stream, (const T*)proj, ldp, q_col, k_col, v_col, (const float*)coef, state, o, seg_start, seg_len, seg_slot, H, D, V
#define SCAN(T)                                                                                                                       \
    do {                                                                                                                              \
        if (D <= 32) xr_launch((k_mlstm_scan<T, 4>), SCAN_ARGS(T));                                                                   \
        else if (D <= 64) xr_launch((k_mlstm_scan<T, 8>), SCAN_ARGS(T));                                                              \
        else if (D <= 128) xr_launch((k_mlstm_scan<T, 16>), SCAN_ARGS(T));                                                            \
        else if (D <= 256) xr_launch((k_mlstm_scan<T, 32>), SCAN_ARGS(T));                                                            \
        else xr_launch((k_mlstm_scan_wide<T>), gs, dim3(ML_VS * ML_RG), smem_s, stream, (const T*)proj, ldp, q_col, k_col, v_col,      \
                       (const float*)coef, state, o, seg_start, seg_len, seg_slot, H, D, V);                                          \
    } while (0)
#define ML(T)                                                                                                                         \
    do {                                                                                                                              \
        if (D > 256 && smem_s > 48 * 1024 &&                                                                                                     \
            cudaFuncSetAttribute(k_mlstm_scan_wide<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s) != cudaSuccess)      \
            return XR_ERR_LAUNCH;                                                                                                     \
        xr_launch((k_mlstm_gates<T>), gg, dim3(D <= 128 ? 128 : 256), smem_g, stream, (const T*)proj, ldp, q_col, k_col, gates, state, coef, seg_start, \
                  seg_len, seg_slot, H, D, V, cap, stage);                                                                            \
        SCAN(T);                                                                                                                      \
        xr_launch((k_mlstm_out<T>), dim3(gb), dim3(128), 0, stream, (const float*)o, (const T*)proj, ldp, g_col, norm_w, (T*)y, n, H, \
                  V, eps, V, 0);                                                                                                         \
    } while (0)
    if (dtype == XR_F32) ML(float);
    else if (dtype == XR_BF16) ML(__nv_bfloat16);
    else return XR_ERR_ARG;
#undef ML
#undef SCAN
#undef SCAN_ARGS
    return xr_launch_status();
}

// The last step alone, for other recurrences: y [n][H * V] (dtype `dtype`) = o / rms(o per head) * w * act(gate), gate [n][ld_gate]
// (dtype `gate_dtype`: that of y, or float32) from column 0, head h at h * V; w_head: elements between the heads' weights (0: one
// weight for all heads).
XR_EXPORT int xr_head_norm_gate(const float* o, const void* gate, int gate_dtype, long long ld_gate, const float* w, int w_head, int gate_silu,
                                void* y, int dtype, int n, int H, int V, float eps, cudaStream_t stream) {
    if (n < 1 || H < 1 || V < 1 || w_head < 0) return XR_ERR_ARG;
    const long long warps = (long long)n * H;
    const unsigned gb = (unsigned)((warps + 3) / 4);
    typedef __nv_bfloat16 bf;
    if (dtype == XR_F32 && gate_dtype == XR_F32)
        xr_launch((k_mlstm_out<float, float>), dim3(gb), dim3(128), 0, stream, o, (const float*)gate, ld_gate, 0, w, (float*)y, n, H, V, eps, w_head, gate_silu);
    else if (dtype == XR_BF16 && gate_dtype == XR_BF16)
        xr_launch((k_mlstm_out<bf, bf>), dim3(gb), dim3(128), 0, stream, o, (const bf*)gate, ld_gate, 0, w, (bf*)y, n, H, V, eps, w_head, gate_silu);
    else if (dtype == XR_BF16 && gate_dtype == XR_F32)
        xr_launch((k_mlstm_out<bf, float>), dim3(gb), dim3(128), 0, stream, o, (const float*)gate, ld_gate, 0, w, (bf*)y, n, H, V, eps, w_head, gate_silu);
    else return XR_ERR_ARG;
    return xr_launch_status();
}
