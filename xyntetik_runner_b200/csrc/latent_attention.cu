// Attention whose keys and values are expanded from a small latent vector per token (one latent and one rotated
// key part per token, shared by all heads), over the paged cache.
//
// Per token the cache row holds [c (C values, RMS-normed) | r (R values, rotated)].  With per-head matrices
// Wuk [D, C] (key expansion) and Wuv [V, C] (value expansion), head h of the query at position p has
//   s_j = (q_h . Wuk_h c_j + qr_h . r_j) * scale,   a = softmax(s_j, j <= p),   o_h = Wuv_h sum_j a_j c_j.
// Nothing per head is ever expanded for the keys: the kernels use
//   q_h . Wuk_h c_j = (Wuk_h^T q_h) . c_j   and   sum_j a_j Wuv_h c_j = Wuv_h (sum_j a_j c_j),
// so a head's query is first taken into the latent space (xr_head_matmul), attention runs over the cached rows
// with one "key" of C + R values and one "value" of C values for all heads (xr_latent_attention), and the result
// is expanded by Wuv (xr_head_matmul again, times the head's output gate).  Scores, softmax weights and both
// latent-space vectors are float32 in both precisions.
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------------------------------------
// Preparation, one block per token.  proj row t (activation dtype): the heads' queries [H][D + R] from column 0
// and the down projection [C + R] from column `down_col`.
//  * the last R values of every head's query are rotated in place (the first `rot_dims` of them: pair (i, i + rot_dims/2),
//    angle = position * freq[i], cosine and sine from a float64 angle);
//  * c = down[:C] / sqrt(mean(down[:C]^2) + eps) * norm_w and r = rotate(down[C:]) go to the token's cache row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
k_latent_prep(T* __restrict__ proj, long long ldp, int down_col, const int* __restrict__ positions,
              const int* __restrict__ tok_seg, const int* __restrict__ block_tables, const double* __restrict__ freq,
              const float* __restrict__ norm_w, T* __restrict__ cache, long long page_stride, int H, int D, int R, int C,
              int rot_dims, int max_pages, int page_size, float eps) {
    xr_pdl_launch();
    __shared__ float scratch[33];
    extern __shared__ float cs[];            // cos [half], sin [half]
    const int t = blockIdx.x, half = rot_dims / 2;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)pos * freq[i], &s, &c);
        cs[i] = (float)c; cs[half + i] = (float)s;
    }
    xr_pdl_wait();
    __syncthreads();
    T* row = proj + (size_t)t * ldp;
    // queries
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        int h = idx / half, i = idx % half;
        T* qr = row + (size_t)h * (D + R) + D;
        float u = xr_to_f32<T>(qr[i]), v = xr_to_f32<T>(qr[i + half]);
        qr[i] = xr_from_f32<T>(u * cs[i] - v * cs[half + i]);
        qr[i + half] = xr_from_f32<T>(v * cs[i] + u * cs[half + i]);
    }
    if (cache == nullptr) return;
    const T* down = row + down_col;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { float v = xr_to_f32<T>(down[i]); ss += v * v; }
    ss = xr_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)C + eps);
    const int page = block_tables[(size_t)tok_seg[t] * max_pages + pos / page_size];
    T* dst = cache + (size_t)page * page_stride + (size_t)(pos % page_size) * (C + R);
    for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = xr_from_f32<T>(xr_to_f32<T>(down[i]) * inv * norm_w[i]);
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float out;
        if (i < half) out = xr_to_f32<T>(down[C + i]) * cs[i] - xr_to_f32<T>(down[C + i + half]) * cs[half + i];
        else if (i < rot_dims) out = xr_to_f32<T>(down[C + i]) * cs[i - half] + xr_to_f32<T>(down[C + i - half]) * cs[i];
        else out = xr_to_f32<T>(down[C + i]);
        dst[C + i] = xr_from_f32<T>(out);
    }
}

XR_EXPORT int xr_latent_prep(void* proj, int dtype, long long ldp, int down_col, const int* positions, const int* tok_seg,
                             const int* block_tables, const double* freq, const float* norm_w, void* cache,
                             long long page_stride, int n, int H, int D, int R, int C, int rot_dims, int max_pages,
                             int page_size, float eps, cudaStream_t stream) {
    if (n < 1 || H < 1 || D < 0 || R < 0 || C < 1 || rot_dims < 0 || rot_dims > R || (rot_dims & 1) || page_size < 1) return XR_ERR_ARG;
    size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float);
    if (smem > 40000) return XR_ERR_ARG;
    if (dtype == XR_F32)
        xr_launch((k_latent_prep<float>), dim3(n), dim3(256), smem, stream, (float*)proj, ldp, down_col, positions, tok_seg, block_tables,
                  freq, norm_w, (float*)cache, page_stride, H, D, R, C, rot_dims, max_pages, page_size, eps);
    else if (dtype == XR_BF16)
        xr_launch((k_latent_prep<__nv_bfloat16>), dim3(n), dim3(256), smem, stream, (__nv_bfloat16*)proj, ldp, down_col, positions, tok_seg,
                  block_tables, freq, norm_w, (__nv_bfloat16*)cache, page_stride, H, D, R, C, rot_dims, max_pages, page_size, eps);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// A small matrix per head: out[t][h][j] = sum_k in[t][h][k] * W_h(k, j) (* sigmoid(gate[t][h])), float32 sums.
// in row t, head h starts at in + t * ld_in + h * head_in; W_h(k, j) = W[h * w_head + k * w_k + j * w_j]
// (so both "W_h as stored" and its transpose are a choice of strides); out row t, head h at out + t * ld_out + h * J.
// Tile: 64 tokens x 64 columns, 256 threads with 4 x 4 results each, 16 values of k a round.
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TW, typename TO, typename TG>
__global__ void __launch_bounds__(256)
k_head_matmul(const TI* __restrict__ in, long long ld_in, int head_in, const TW* __restrict__ W, long long w_head, long long w_k,
              long long w_j, TO* __restrict__ out, long long ld_out, const TG* __restrict__ gate, long long ld_gate,
              int n, int Kd, int J) {
    xr_pdl_launch();
    __shared__ float As[16][64 + 1], Ws[16][64 + 1];
    const int h = blockIdx.z, t0 = blockIdx.x * 64, j0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const TW* Wh = W + (size_t)h * w_head;
    float acc[4][4] = {};
    // the weights of the first round need no earlier kernel
    xr_pdl_wait();
    for (int k0 = 0; k0 < Kd; k0 += 16) {
        for (int e = threadIdx.x; e < 16 * 64; e += 256) {
            int kk = e & 15, r = e >> 4;                    // A: consecutive threads along k (contiguous in memory)
            int t = t0 + r, k = k0 + kk;
            As[kk][r] = (t < n && k < Kd) ? xr_to_f32<TI>(in[(size_t)t * ld_in + (size_t)h * head_in + k]) : 0.f;
        }
        for (int e = threadIdx.x; e < 16 * 64; e += 256) {
            int kk, c;
            if (w_j == 1) { c = e & 63; kk = e >> 6; } else { kk = e & 15; c = e >> 4; }
            int k = k0 + kk, j = j0 + c;
            Ws[kk][c] = (k < Kd && j < J) ? xr_to_f32<TW>(Wh[(size_t)k * w_k + (size_t)j * w_j]) : 0.f;
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
        int t = t0 + ty + 16 * i;
        if (t >= n) continue;
        float g = 1.0f;
        if (gate != nullptr) g = 1.0f / (1.0f + expf(-xr_to_f32<TG>(gate[(size_t)t * ld_gate + h])));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int c = j0 + tx + 16 * j;
            if (c < J) out[(size_t)t * ld_out + (size_t)h * J + c] = xr_from_f32<TO>(acc[i][j] * g);
        }
    }
}

// in_dtype / w_dtype / out_dtype: XR_F32 or XR_BF16; the gate (optional) has the dtype `gate_dtype`.
XR_EXPORT int xr_head_matmul(const void* in, int in_dtype, long long ld_in, int head_in, const void* W, int w_dtype,
                             long long w_head, long long w_k, long long w_j, void* out, int out_dtype, long long ld_out,
                             const void* gate, int gate_dtype, long long ld_gate, int n, int H, int Kd, int J, cudaStream_t stream) {
    if (n < 1 || H < 1 || Kd < 1 || J < 1 || H > 65535) return XR_ERR_ARG;
    dim3 grid((n + 63) / 64, (J + 63) / 64, H);
    if (grid.y > 65535) return XR_ERR_ARG;
#define HM(TI, TW, TO, TG) xr_launch((k_head_matmul<TI, TW, TO, TG>), grid, dim3(256), 0, stream, (const TI*)in, ld_in, head_in, (const TW*)W, \
                                     w_head, w_k, w_j, (TO*)out, ld_out, (const TG*)gate, ld_gate, n, Kd, J)
    typedef __nv_bfloat16 bf;
    const int key = in_dtype * 8 + w_dtype * 4 + out_dtype * 2 + (gate ? gate_dtype : 0);
    switch (key) {
        // the four uses: (query -> latent) and (latent -> value) in each precision
        case XR_BF16 * 8 + XR_BF16 * 4 + XR_F32 * 2 + 0: HM(bf, bf, float, float); break;
        case XR_F32 * 8 + XR_BF16 * 4 + XR_BF16 * 2 + XR_BF16: HM(float, bf, bf, bf); break;
        case XR_F32 * 8 + XR_BF16 * 4 + XR_F32 * 2 + XR_F32: HM(float, bf, float, float); break;
        case XR_F32 * 8 + XR_F32 * 4 + XR_F32 * 2 + XR_F32: HM(float, float, float, float); break;
        case XR_F32 * 8 + XR_F32 * 4 + XR_BF16 * 2 + XR_BF16: HM(float, float, bf, bf); break;
        case XR_BF16 * 8 + XR_F32 * 4 + XR_F32 * 2 + 0: HM(bf, float, float, float); break;
        default: return XR_ERR_ARG;
    }
#undef HM
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Attention over the cached rows, one block per token, a warp per head (eight heads at a time).  Keys are taken in
// tiles of 32 in ascending order from position 0, with a running maximum: a query's result depends on its position
// and the cached rows alone, not on how the step was cut or what else is in the batch.  The tile of 32 rows is
// brought to shared memory once for the eight heads that share it.
//   ql [n][H][C] float32: the queries in the latent space;  qr: the rotated query parts, head h of token t at
//   qr + t * ld_qr + h * head_qr (activation dtype);  out [n][H][C] float32: sum_j a_j c_j.
// ---------------------------------------------------------------------------------------------
#define LA_WARPS 8
#define LA_MAX_ND 32       // C <= 1024

template <typename T>
__global__ void __launch_bounds__(32 * LA_WARPS)
k_latent_attention(const float* __restrict__ ql, const T* __restrict__ qr, long long ld_qr, int head_qr,
                   float* __restrict__ out, const T* __restrict__ cache, long long page_stride,
                   const int* __restrict__ positions, const int* __restrict__ tok_seg, const int* __restrict__ block_tables,
                   int H, int C, int R, int max_pages, int page_size, float scale) {
    xr_pdl_launch();
    extern __shared__ float sm[];
    const int W = C + R, ldw = W | 1;                       // odd row stride: lanes that read one column of 32 rows hit 32 banks
    float* tile = sm;                                        // [32][ldw]
    float* qs = sm + 32 * ldw;                               // [LA_WARPS][ldw]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int* bt = block_tables + (size_t)tok_seg[t] * max_pages;
    xr_pdl_wait();
    for (int h0 = 0; h0 < H; h0 += LA_WARPS) {
        const int h = h0 + warp;
        const bool live = h < H;
        __syncthreads();                                     // the round before is done with qs and tile
        if (live) {
            const float* a = ql + ((size_t)t * H + h) * C;
            for (int i = lane; i < C; i += 32) qs[warp * ldw + i] = a[i];
            const T* b = qr + (size_t)t * ld_qr + (size_t)h * head_qr;
            for (int i = lane; i < R; i += 32) qs[warp * ldw + C + i] = xr_to_f32<T>(b[i]);
        }
        float acc[LA_MAX_ND];
#pragma unroll
        for (int i = 0; i < LA_MAX_ND; i++) acc[i] = 0.f;
        float m = -INFINITY, l = 0.f;
        for (int k0 = 0; k0 <= pos; k0 += 32) {
            const int cnt = min(32, pos - k0 + 1);
            __syncthreads();
            for (int j = warp; j < cnt; j += LA_WARPS) {
                const int kp = k0 + j;
                const T* src = cache + (size_t)bt[kp / page_size] * page_stride + (size_t)(kp % page_size) * W;
                for (int i = lane; i < W; i += 32) tile[j * ldw + i] = xr_to_f32<T>(src[i]);
            }
            __syncthreads();
            if (!live) continue;
            float s = -INFINITY;
            if (lane < cnt) {
                const float* kr = tile + lane * ldw;
                const float* q = qs + warp * ldw;
                float dot = 0.f;
                for (int i = 0; i < W; i++) dot = fmaf(q[i], kr[i], dot);
                s = dot * scale;
            }
            const float m_new = fmaxf(m, xr_warp_max(s));
            const float corr = expf(m - m_new);
            const float p = lane < cnt ? expf(s - m_new) : 0.f;
            l = l * corr + xr_warp_sum(p);
#pragma unroll
            for (int i = 0; i < LA_MAX_ND; i++) acc[i] *= corr;
            for (int j = 0; j < cnt; j++) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                const float* vr = tile + j * ldw;
#pragma unroll
                for (int i = 0; i < LA_MAX_ND; i++) {
                    const int dd = lane + 32 * i;
                    if (dd < C) acc[i] = fmaf(pj, vr[dd], acc[i]);
                }
            }
            m = m_new;
        }
        if (live) {
            float* o = out + ((size_t)t * H + h) * C;
            const float inv = 1.0f / l;
#pragma unroll
            for (int i = 0; i < LA_MAX_ND; i++) {
                const int dd = lane + 32 * i;
                if (dd < C) o[dd] = acc[i] * inv;
            }
        }
    }
}

XR_EXPORT int xr_latent_attention(const float* ql, const void* qr, int dtype, long long ld_qr, int head_qr, float* out,
                                  const void* cache, long long page_stride, const int* positions, const int* tok_seg,
                                  const int* block_tables, int n, int H, int C, int R, int max_pages, int page_size,
                                  float scale, cudaStream_t stream) {
    if (n < 1 || H < 1 || C < 1 || C > 32 * LA_MAX_ND || R < 0 || page_size < 1) return XR_ERR_ARG;
    const size_t smem = (size_t)(32 + LA_WARPS) * ((C + R) | 1) * sizeof(float);
    if (smem > 220 * 1024) return XR_ERR_ARG;
    cudaError_t e = cudaSuccess;
    if (dtype == XR_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(k_latent_attention<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return XR_ERR_LAUNCH;
        xr_launch((k_latent_attention<float>), dim3(n), dim3(32 * LA_WARPS), smem, stream, ql, (const float*)qr, ld_qr, head_qr, out,
                  (const float*)cache, page_stride, positions, tok_seg, block_tables, H, C, R, max_pages, page_size, scale);
    } else if (dtype == XR_BF16) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(k_latent_attention<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return XR_ERR_LAUNCH;
        xr_launch((k_latent_attention<__nv_bfloat16>), dim3(n), dim3(32 * LA_WARPS), smem, stream, ql, (const __nv_bfloat16*)qr, ld_qr,
                  head_qr, out, (const __nv_bfloat16*)cache, page_stride, positions, tok_seg, block_tables, H, C, R, max_pages,
                  page_size, scale);
    } else return XR_ERR_ARG;
    return xr_launch_status();
}
