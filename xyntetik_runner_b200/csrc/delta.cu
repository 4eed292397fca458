// The gated delta rule: a matrix memory per head that decays, is corrected towards the value at the key, and is read.
//
// Per request slot the state holds S [H][V][D] (float32; the D values of one value column lie together) and the last
// taps - 1 inputs of the short convolutions [taps - 1][CH], CH = 2 G D + H V channels (queries, keys, values; G
// query/key heads, H value heads, value head h reads query/key head h / (H / G)).  For a token with the projections'
// rows x (channels in the order q, k, v), gate pre-activations b and a per head:
//   y  = silu(sum_j w[c][taps-1-j] x[t-j][c])             (zeros before the request's first token)
//   q  = y_q / sqrt(sum y_q^2 + 1e-6) * D^-1/2,   k = y_k / sqrt(sum y_k^2 + 1e-6),   v = y_v
//   beta = sigmoid(b),   g = exp(-exp(A_log) softplus(a + dt_bias))
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// Everything after the projections is float32 in both precisions.
//
// Three kernels.  k_delta_prep, a block per token: the convolutions (earlier tokens of the portion from the rows,
// tokens of earlier steps from the slot's tail), the unit vectors and the two scalars per head.  k_delta_tail, a block
// per portion: the slot's tail becomes the last taps - 1 inputs.  k_delta_scan walks a portion's tokens once per
// (head, 16 value columns): a column's D state values live in the registers of eight lanes, so both sums of a token
// are shuffles inside a warp and the columns never wait for one another.  The walk is token by token, so the state
// after a token does not depend on how the tokens were cut into steps, bit for bit.
#include "common.cuh"
#include <math.h>

#define DL_LPC 8                              // lanes that share a value column
#define DL_WARPS 4
#define DL_COLS (DL_WARPS * 32 / DL_LPC)      // value columns per block of the scan
#define DL_CHUNK 8                            // tokens whose q, k, v are staged together

template <typename T>
__global__ void __launch_bounds__(256)
k_delta_prep(const T* __restrict__ proj, long long ldp, const float* __restrict__ conv_w, const float* __restrict__ gates,
             const float* __restrict__ neg_a, const float* __restrict__ dt_bias, const float* __restrict__ state,
             long long state_stride, long long tail_off, const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
             const int* __restrict__ seg_slot, float* __restrict__ qkv, float* __restrict__ coef, int H, int G, int D, int V, int taps) {
    xr_pdl_launch();
    extern __shared__ float ysm[];            // [CH]: the convolutions' outputs after the activation
    const int t = blockIdx.x, CH = 2 * G * D + H * V;
    const int seg = tok_seg[t], i = t - seg_start[seg];
    const float* tail = state + (size_t)seg_slot[seg] * state_stride + tail_off;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    xr_pdl_wait();
    for (int c = threadIdx.x; c < CH; c += blockDim.x) {
        const float* w = conv_w + (size_t)c * taps;
        float acc = 0.f;
        for (int j = taps - 1; j >= 0; j--) {                       // oldest input first
            const int ip = i - j;
            const float x = ip >= 0 ? xr_to_f32<T>(proj[(size_t)(t - j) * ldp + c]) : tail[(size_t)(taps - 1 + ip) * CH + c];
            acc = fmaf(w[taps - 1 - j], x, acc);
        }
        ysm[c] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    float* row = qkv + (size_t)t * CH;
    for (int u = warp; u < 2 * G; u += nw) {                        // the G query heads, then the G key heads
        const float* y = ysm + (size_t)u * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(y[d], y[d], ss);
        ss = xr_warp_sum(ss);
        float inv = 1.0f / sqrtf(ss + 1e-6f);
        if (u < G) inv *= 1.0f / sqrtf((float)D);
        for (int d = lane; d < D; d += 32) row[(size_t)u * D + d] = y[d] * inv;
    }
    for (int c = 2 * G * D + threadIdx.x; c < CH; c += blockDim.x) row[c] = ysm[c];
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float b = gates[(size_t)t * 2 * H + h], a = gates[(size_t)t * 2 * H + H + h] + dt_bias[h];
        const float softplus = fmaxf(a, 0.f) + log1pf(expf(-fabsf(a)));
        coef[((size_t)t * H + h) * 2] = expf(neg_a[h] * softplus);
        coef[((size_t)t * H + h) * 2 + 1] = 1.0f / (1.0f + expf(-b));
    }
}

// tail[j] <- the input at place len - (taps - 1) + j of the portion: a row of this step, or, where the portion is
// shorter than the tail, what the tail held len places further on (read before it is overwritten: j ascends)
template <typename T>
__global__ void __launch_bounds__(256)
k_delta_tail(const T* __restrict__ proj, long long ldp, float* __restrict__ state, long long state_stride, long long tail_off,
             const int* __restrict__ seg_start, const int* __restrict__ seg_len, const int* __restrict__ seg_slot, int CH, int taps) {
    xr_pdl_launch();
    const int seg = blockIdx.x;
    const int start = seg_start[seg], len = seg_len[seg];
    float* tail = state + (size_t)seg_slot[seg] * state_stride + tail_off;
    xr_pdl_wait();
    for (int c = threadIdx.x; c < CH; c += blockDim.x)
        for (int j = 0; j < taps - 1; j++) {
            const int src = len - (taps - 1) + j;
            tail[(size_t)j * CH + c] = src >= 0 ? xr_to_f32<T>(proj[(size_t)(start + src) * ldp + c]) : tail[(size_t)(j + len) * CH + c];
        }
}

// thread (column, row lane l) keeps rows l, l + 8, ... of its column: RPT of them, 8 RPT >= D (rows beyond D stay zero)
template <int RPT>
__global__ void __launch_bounds__(32 * DL_WARPS)
k_delta_scan(const float* __restrict__ qkv, const float* __restrict__ coef, float* __restrict__ state, long long state_stride,
             float* __restrict__ out, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
             const int* __restrict__ seg_slot, int H, int G, int D, int V) {
    xr_pdl_launch();
    constexpr int DP = DL_LPC * RPT;
    __shared__ float ks[DL_CHUNK][DP], qs[DL_CHUNK][DP], vs[DL_CHUNK][DL_COLS], cf[DL_CHUNK][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & (DL_LPC - 1), colb = warp * (32 / DL_LPC) + lane / DL_LPC;
    const int v0 = blockIdx.x * DL_COLS, v = v0 + colb, h = blockIdx.y, seg = blockIdx.z;
    const int kvh = h / (H / G), CH = 2 * G * D + H * V;
    const bool col_ok = v < V;
    const int start = seg_start[seg], len = seg_len[seg], slot = seg_slot[seg];
    xr_pdl_wait();
    float* Sg = state + (size_t)slot * state_stride + ((size_t)h * V + (col_ok ? v : 0)) * D;
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int d = l + DL_LPC * i;
        S[i] = (col_ok && d < D) ? Sg[d] : 0.f;
    }
    // the next chunk's rows are on their way to registers while this chunk is walked
    constexpr int NL = DL_CHUNK * DP / (32 * DL_WARPS);            // elements of k (and of q) per thread and chunk
    float kreg[NL], qreg[NL], vreg = 0.f, creg = 0.f;
    auto prefetch = [&](int j0) {
        const int cnt = min(DL_CHUNK, len - j0);
#pragma unroll
        for (int i = 0; i < NL; i++) {
            const int e = threadIdx.x + i * (32 * DL_WARPS), j = e / DP, d = e % DP;
            const bool ok = j < cnt && d < D;
            const float* row = qkv + (size_t)(start + j0 + (ok ? j : 0)) * CH + (size_t)kvh * D + (ok ? d : 0);
            qreg[i] = ok ? row[0] : 0.f;
            kreg[i] = ok ? row[(size_t)G * D] : 0.f;
        }
        {
            const int j = threadIdx.x / DL_COLS, c = threadIdx.x % DL_COLS;
            vreg = (j < cnt && v0 + c < V) ? qkv[(size_t)(start + j0 + j) * CH + 2 * (size_t)G * D + (size_t)h * V + v0 + c] : 0.f;
        }
        if (threadIdx.x < DL_CHUNK * 2) {
            const int j = threadIdx.x >> 1;
            creg = j < cnt ? coef[((size_t)(start + j0 + j) * H + h) * 2 + (threadIdx.x & 1)] : 0.f;
        }
    };
    prefetch(0);
    for (int j0 = 0; j0 < len; j0 += DL_CHUNK) {
        const int cnt = min(DL_CHUNK, len - j0);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NL; i++) {
            const int e = threadIdx.x + i * (32 * DL_WARPS);
            ks[e / DP][e % DP] = kreg[i];
            qs[e / DP][e % DP] = qreg[i];
        }
        vs[threadIdx.x / DL_COLS][threadIdx.x % DL_COLS] = vreg;
        if (threadIdx.x < DL_CHUNK * 2) cf[threadIdx.x >> 1][threadIdx.x & 1] = creg;
        __syncthreads();
        if (j0 + DL_CHUNK < len) prefetch(j0 + DL_CHUNK);
        for (int j = 0; j < cnt; j++) {
            const float g = cf[j][0], beta = cf[j][1];
            float kv = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                S[i] *= g;
                kv = fmaf(S[i], ks[j][l + DL_LPC * i], kv);
            }
            kv += __shfl_xor_sync(0xffffffffu, kv, 1);
            kv += __shfl_xor_sync(0xffffffffu, kv, 2);
            kv += __shfl_xor_sync(0xffffffffu, kv, 4);
            const float u = beta * (vs[j][colb] - kv);
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                S[i] = fmaf(ks[j][l + DL_LPC * i], u, S[i]);
                o = fmaf(S[i], qs[j][l + DL_LPC * i], o);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (l == 0 && col_ok) out[(size_t)(start + j0 + j) * H * V + (size_t)h * V + v] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int d = l + DL_LPC * i;
            if (d < D) Sg[d] = S[i];
        }
    }
}

static inline long long dl_state_floats(int H, int G, int D, int V, int taps) {
    return (long long)H * V * D + (long long)(taps - 1) * (2LL * G * D + (long long)H * V);
}

// proj [n][ldp] (activation dtype): the convolutions' channels (q [G][D], k [G][D], v [H][V]) from column 0;
// conv_w [CH][taps] float32, the last column the current token's; gates [n][2H] float32 (pre-activations of beta, then
// of the decay); neg_a [H] = -exp(A_log), dt_bias [H]; state [slots][state_stride] float32;
// qkv [n][CH] and coef [n][H][2]: float32 scratch;  o [n][H * V] float32: the read-outs.
XR_EXPORT int xr_delta(const void* proj, int dtype, long long ldp, const float* conv_w, const float* gates, const float* neg_a,
                       const float* dt_bias, float* state, long long state_stride, float* qkv, float* coef, float* o,
                       const int* tok_seg, const int* seg_start, const int* seg_len, const int* seg_slot, int n, int n_seg,
                       int H, int G, int D, int V, int taps, cudaStream_t stream) {
    if (n < 1 || n_seg < 1 || H < 1 || G < 1 || H % G || D < 1 || D > 256 || V < 1 || taps < 1 || taps > 64 || n_seg > 65535 || H > 65535)
        return XR_ERR_ARG;
    const long long CH = 2LL * G * D + (long long)H * V, tail_off = (long long)H * V * D;
    if (state_stride < dl_state_floats(H, G, D, V, taps) || CH * sizeof(float) > 200 * 1024) return XR_ERR_ARG;
    const size_t smem = (size_t)CH * sizeof(float);
    dim3 gs((V + DL_COLS - 1) / DL_COLS, H, n_seg);
#define DL_SCAN(RPT) xr_launch((k_delta_scan<RPT>), gs, dim3(32 * DL_WARPS), 0, stream, (const float*)qkv, (const float*)coef, state, \
                               state_stride, o, seg_start, seg_len, seg_slot, H, G, D, V)
#define DL(T)                                                                                                                        \
    do {                                                                                                                             \
        if (smem > 48 * 1024 && cudaFuncSetAttribute(k_delta_prep<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return XR_ERR_LAUNCH;                                                                                                    \
        xr_launch((k_delta_prep<T>), dim3(n), dim3(256), smem, stream, (const T*)proj, ldp, conv_w, gates, neg_a, dt_bias,           \
                  (const float*)state, state_stride, tail_off, tok_seg, seg_start, seg_slot, qkv, coef, H, G, D, V, taps);           \
        if (taps > 1)                                                                                                                \
            xr_launch((k_delta_tail<T>), dim3(n_seg), dim3(256), 0, stream, (const T*)proj, ldp, state, state_stride, tail_off,      \
                      seg_start, seg_len, seg_slot, (int)CH, taps);                                                                  \
    } while (0)
    if (dtype == XR_F32) DL(float);
    else if (dtype == XR_BF16) DL(__nv_bfloat16);
    else return XR_ERR_ARG;
    if (D <= 32) DL_SCAN(4);
    else if (D <= 64) DL_SCAN(8);
    else if (D <= 128) DL_SCAN(16);
    else DL_SCAN(32);
#undef DL
#undef DL_SCAN
    return xr_launch_status();
}
