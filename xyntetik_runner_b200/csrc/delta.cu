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
// Two kernels.  k_delta_prep, a block per token and head: the convolutions (earlier tokens of the portion from the rows,
// tokens of earlier steps from the slot's tail), the unit vectors and the two scalars per head.  k_delta_scan walks a
// portion's tokens once per (head, 16 value columns): a column's D state values live in the registers of eight lanes,
// so both sums of a token are shuffles inside a warp and the columns never wait for one another; a portion's blocks
// then make the slot's tail the last taps - 1 inputs.  The walk is token by token, so the state after a token
// does not depend on how the tokens were cut into steps, bit for bit.
#include "common.cuh"
#include <math.h>

#define DL_WARPS 4
#define DL_CHUNK 8                            // tokens whose q, k, v are staged together

// grid (tokens, 2 G + H): block y < 2 G takes one query or key head (convolution, activation, unit vector), block
// 2 G + h the values of head h and its two scalars.
template <typename T>
__global__ void __launch_bounds__(128)
k_delta_prep(const T* __restrict__ proj, long long ldp, const float* __restrict__ conv_w, const float* __restrict__ gates,
             const float* __restrict__ neg_a, const float* __restrict__ dt_bias, const float* __restrict__ state,
             long long state_stride, long long tail_off, const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
             const int* __restrict__ seg_slot, float* __restrict__ qkv, float* __restrict__ coef, int H, int G, int D, int V, int taps,
             int early) {
    // The walk that follows is a few long-lived blocks.  Let in while this kernel's many blocks still hold the machine, they
    // settle several to an SM wherever room appears first, and the walk, a chain of dependent operations, then takes twice as
    // long (measured); so only a step of few tokens releases it early.
    if (early) xr_pdl_launch();
    __shared__ float scratch[33];
    const int t = blockIdx.x, y = blockIdx.y, CH = 2 * G * D + H * V;
    const bool unit = y < 2 * G;
    const int c0 = unit ? y * D : 2 * G * D + (y - 2 * G) * V, cn = unit ? D : V;
    const int seg = tok_seg[t], i = t - seg_start[seg];
    const float* tail = state + (size_t)seg_slot[seg] * state_stride + tail_off;
    xr_pdl_wait();
    constexpr int OWN = 4;                        // channels per thread: D, V <= 4 * 128 (longer heads take more passes)
    float* row = qkv + (size_t)t * CH;
    for (int r0 = 0; r0 < cn; r0 += OWN * 128) {
        float yv[OWN];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < OWN; k++) {
            const int e = r0 + threadIdx.x + k * 128;
            yv[k] = 0.f;
            if (e < cn) {
                const int c = c0 + e;
                const float* w = conv_w + (size_t)c * taps;
                float acc = 0.f;
                for (int j = taps - 1; j >= 0; j--) {                       // oldest input first
                    const int ip = i - j;
                    const float x = ip >= 0 ? xr_to_f32<T>(proj[(size_t)(t - j) * ldp + c]) : tail[(size_t)(taps - 1 + ip) * CH + c];
                    acc = fmaf(w[taps - 1 - j], x, acc);
                }
                yv[k] = acc / (1.0f + expf(-acc));
                ss = fmaf(yv[k], yv[k], ss);
            }
        }
        float inv = 1.0f;
        if (unit) {                               // (a head of more than 512 elements would need its sum over all passes: refused by the launcher)
            ss = xr_block_sum(ss, scratch);
            inv = 1.0f / sqrtf(ss + 1e-6f);
            if (y < G) inv *= 1.0f / sqrtf((float)D);
        }
#pragma unroll
        for (int k = 0; k < OWN; k++) {
            const int e = r0 + threadIdx.x + k * 128;
            if (e < cn) row[c0 + e] = yv[k] * inv;
        }
    }
    if (!unit && threadIdx.x == 0) {
        const int h = y - 2 * G;
        const float b = gates[(size_t)t * 2 * H + h], a = gates[(size_t)t * 2 * H + H + h] + dt_bias[h];
        const float softplus = fmaxf(a, 0.f) + log1pf(expf(-fabsf(a)));
        coef[((size_t)t * H + h) * 2] = expf(neg_a[h] * softplus);
        coef[((size_t)t * H + h) * 2 + 1] = 1.0f / (1.0f + expf(-b));
    }
}

// tail[j] <- the input at place len - (taps - 1) + j of the portion: a row of this step, or, where the portion is
// shorter than the tail, what the tail held len places further on.  All blocks of the scan that walk a portion share
// its channels (block `part` of `parts`), after the kernel that read the old tail is complete; a thread reads all of a
// channel's values before it writes any (eight at a time: the reads of a pass lie ahead of its writes, j ascends).
template <typename T>
__device__ __forceinline__ void dl_tail_update(const T* __restrict__ proj, long long ldp, float* tail, int start, int len,
                                               int CH, int taps, int part, int parts) {
    for (int c = part * blockDim.x + threadIdx.x; c < CH; c += parts * blockDim.x)
        for (int j0 = 0; j0 < taps - 1; j0 += 8) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int j = j0 + i, src = len - (taps - 1) + j;
                x[i] = j >= taps - 1 ? 0.f : (src >= 0 ? xr_to_f32<T>(proj[(size_t)(start + src) * ldp + c]) : tail[(size_t)(j + len) * CH + c]);
            }
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (j0 + i < taps - 1) tail[(size_t)(j0 + i) * CH + c] = x[i];
        }
}

// LPC lanes (8 or 16) share a value column.  Thread (column, row lane l) keeps RPT rows of its column, four at a time:
// rows 4 (l + LPC m) .. 4 (l + LPC m) + 3 for m < RPT / 4 (LPC RPT >= D; rows beyond D stay zero), so that the lanes
// of a column read k and q of a token from shared memory as consecutive 16-byte vectors and the state from memory in
// runs of 128 bytes or more.  Per token the walk itself needs one sum over the column (S^T k, a few shuffles); the
// read-out's sums of a chunk's tokens are taken together after the chunk, off the walk's path.  The walk is a chain of
// dependent operations whose length the shuffles set.
template <typename T, int RPT, int LPC>
__global__ void __launch_bounds__(32 * DL_WARPS)
k_delta_scan(const float* __restrict__ qkv, const float* __restrict__ coef, float* __restrict__ state, long long state_stride,
             float* __restrict__ out, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
             const int* __restrict__ seg_slot, int H, int G, int D, int V, const T* __restrict__ proj, long long ldp, int taps) {
    constexpr int DP = LPC * RPT, R4 = RPT / 4, DL_COLS = DL_WARPS * 32 / LPC;
    __shared__ __align__(16) float ks[DL_CHUNK][DP];
    __shared__ __align__(16) float qs[DL_CHUNK][DP];
    __shared__ float vs[DL_CHUNK][DL_COLS], cf[DL_CHUNK][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & (LPC - 1), colb = warp * (32 / LPC) + lane / LPC;
    const int v0 = blockIdx.x * DL_COLS, v = v0 + colb, h = blockIdx.y, seg = blockIdx.z;
    const int kvh = h / (H / G), CH = 2 * G * D + H * V;
    const bool col_ok = v < V;
    const int start = seg_start[seg], len = seg_len[seg], slot = seg_slot[seg];
    xr_pdl_wait();
    float* Sg = state + (size_t)slot * state_stride + ((size_t)h * V + (col_ok ? v : 0)) * D;
    const bool vec = (D & 3) == 0 && (state_stride & 3) == 0 && ((uintptr_t)state & 15) == 0;
    float S[RPT];
#pragma unroll
    for (int m = 0; m < R4; m++) {
        const int d = 4 * (l + LPC * m);
        if (vec && col_ok && d < D) {
            const float4 x = *reinterpret_cast<const float4*>(Sg + d);
            S[4 * m] = x.x; S[4 * m + 1] = x.y; S[4 * m + 2] = x.z; S[4 * m + 3] = x.w;
        } else {
#pragma unroll
            for (int c = 0; c < 4; c++) S[4 * m + c] = (col_ok && d + c < D) ? Sg[d + c] : 0.f;
        }
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
            // (issued here and now: left alone, the compiler moves these loads down to where the chunk after this one is
            // staged, and every chunk then waits a trip to memory)
            qreg[i] = ok ? xr_ld_now(row) : 0.f;
            kreg[i] = ok ? xr_ld_now(row + (size_t)G * D) : 0.f;
        }
        {
            const int j = threadIdx.x / DL_COLS, c = threadIdx.x % DL_COLS;
            vreg = (j < DL_CHUNK && j < cnt && v0 + c < V) ? qkv[(size_t)(start + j0 + j) * CH + 2 * (size_t)G * D + (size_t)h * V + v0 + c] : 0.f;
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
        if (threadIdx.x < DL_CHUNK * DL_COLS) vs[threadIdx.x / DL_COLS][threadIdx.x % DL_COLS] = vreg;
        if (threadIdx.x < DL_CHUNK * 2) cf[threadIdx.x >> 1][threadIdx.x & 1] = creg;
        __syncthreads();
        if (j0 + DL_CHUNK < len) prefetch(j0 + DL_CHUNK);
        float part[DL_CHUNK];                                      // this thread's share of every token's read-out
#pragma unroll
        for (int j = 0; j < DL_CHUNK; j++) {
            part[j] = 0.f;
            if (j < cnt) {
                const float g = cf[j][0], beta = cf[j][1];
                const float4* k4 = reinterpret_cast<const float4*>(&ks[j][0]);
                const float4* q4 = reinterpret_cast<const float4*>(&qs[j][0]);
                float4 kk[R4];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int m = 0; m < R4; m++) {
                    kk[m] = k4[l + LPC * m];
                    S[4 * m] *= g; S[4 * m + 1] *= g; S[4 * m + 2] *= g; S[4 * m + 3] *= g;
                    a0 = fmaf(S[4 * m], kk[m].x, a0); a1 = fmaf(S[4 * m + 1], kk[m].y, a1);
                    a2 = fmaf(S[4 * m + 2], kk[m].z, a2); a3 = fmaf(S[4 * m + 3], kk[m].w, a3);
                }
                float kv = (a0 + a1) + (a2 + a3);
                kv += __shfl_xor_sync(0xffffffffu, kv, 1);
                kv += __shfl_xor_sync(0xffffffffu, kv, 2);
                kv += __shfl_xor_sync(0xffffffffu, kv, 4);
                if (LPC == 16) kv += __shfl_xor_sync(0xffffffffu, kv, 8);
                const float u = beta * (vs[j][colb] - kv);
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                for (int m = 0; m < R4; m++) {
                    const float4 qq = q4[l + LPC * m];
                    S[4 * m] = fmaf(kk[m].x, u, S[4 * m]); S[4 * m + 1] = fmaf(kk[m].y, u, S[4 * m + 1]);
                    S[4 * m + 2] = fmaf(kk[m].z, u, S[4 * m + 2]); S[4 * m + 3] = fmaf(kk[m].w, u, S[4 * m + 3]);
                    o0 = fmaf(S[4 * m], qq.x, o0); o1 = fmaf(S[4 * m + 1], qq.y, o1);
                    o2 = fmaf(S[4 * m + 2], qq.z, o2); o3 = fmaf(S[4 * m + 3], qq.w, o3);
                }
                part[j] = (o0 + o1) + (o2 + o3);
            }
        }
#pragma unroll
        for (int j = 0; j < DL_CHUNK; j++) {
            float o = part[j];
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (LPC == 16) o += __shfl_xor_sync(0xffffffffu, o, 8);
            if (j < cnt && l == 0 && col_ok) out[(size_t)(start + j0 + j) * H * V + (size_t)h * V + v] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int m = 0; m < R4; m++) {
            const int d = 4 * (l + LPC * m);
            if (vec && d < D) {
                *reinterpret_cast<float4*>(Sg + d) = make_float4(S[4 * m], S[4 * m + 1], S[4 * m + 2], S[4 * m + 3]);
            } else {
#pragma unroll
                for (int c = 0; c < 4; c++) if (d + c < D) Sg[d + c] = S[4 * m + c];
            }
        }
    }
    xr_pdl_launch();
    if (taps > 1)
        dl_tail_update<T>(proj, ldp, state + (size_t)slot * state_stride + (size_t)H * V * D, start, len, CH, taps,
                          blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y);
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
    const long long tail_off = (long long)H * V * D;
    if (state_stride < dl_state_floats(H, G, D, V, taps) || 2 * G + H > 65535) return XR_ERR_ARG;
    // eight lanes a column (sixteen above 128 key elements, to bound the registers): measured at 128 x 256 a head, a fourth
    // shuffle in the walk's sum costs more than the shorter runs of multiply-adds save
    const int lpc = D > 128 ? 16 : 8, cols = DL_WARPS * 32 / lpc;
    dim3 gs((V + cols - 1) / cols, H, n_seg);
#define DL_SCAN(T, RPT, LPC) xr_launch((k_delta_scan<T, RPT, LPC>), gs, dim3(32 * DL_WARPS), 0, stream, (const float*)qkv, (const float*)coef, state, \
                                       state_stride, o, seg_start, seg_len, seg_slot, H, G, D, V, (const T*)proj, ldp, taps)
#define DL(T)                                                                                                                        \
    do {                                                                                                                             \
        xr_launch((k_delta_prep<T>), dim3(n, 2 * G + H), dim3(128), 0, stream, (const T*)proj, ldp, conv_w, gates, neg_a, dt_bias,   \
                  (const float*)state, state_stride, tail_off, tok_seg, seg_start, seg_slot, qkv, coef, H, G, D, V, taps,            \
                  n <= 64 ? 1 : 0);                                                                                                  \
        if (D <= 32) DL_SCAN(T, 4, 8);                                                                                               \
        else if (D <= 64) DL_SCAN(T, 8, 8);                                                                                          \
        else if (D <= 128) DL_SCAN(T, 16, 8);                                                                                        \
        else DL_SCAN(T, 16, 16);                                                                                                     \
    } while (0)
    if (dtype == XR_F32) DL(float);
    else if (dtype == XR_BF16) DL(__nv_bfloat16);
    else return XR_ERR_ARG;
#undef DL
#undef DL_SCAN
    return xr_launch_status();
}
