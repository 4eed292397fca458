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
// Preparation, one block per token.  q row t (activation dtype, ldq elements a row): the heads' queries [H][D + R];
// down row t (ldd elements a row; null with a null cache): the down projection [C + R].
//  * the last R values of every head's query are rotated in place: the first `rot_dims` of them, pair (i, i + rot_dims/2)
//    or, with `adjacent`, pair (2i, 2i + 1); angle = position * freq[i] as a float64 product, reduced to [-pi, pi] in float64, cosine and sine in float32;
//  * c = down[:C] / sqrt(mean(down[:C]^2) + eps) * norm_w and r = rotate(down[C:]) go to the token's cache row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
k_latent_prep(T* __restrict__ q, long long ldq, const T* __restrict__ down_all, long long ldd, const int* __restrict__ positions,
              const int* __restrict__ tok_seg, const int* __restrict__ block_tables, const double* __restrict__ freq,
              const float* __restrict__ norm_w, T* __restrict__ cache, long long page_stride, int H, int D, int R, int C,
              int rot_dims, int max_pages, int page_size, float eps, int adjacent) {
    xr_pdl_launch();
    __shared__ float scratch[33];
    extern __shared__ float cs[];            // cos [half], sin [half]
    const int t = blockIdx.x, half = rot_dims / 2;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        xr_sincos_angle((double)pos * freq[i], &cs[half + i], &cs[i]);
    }
    xr_pdl_wait();
    __syncthreads();
    // element indices of pair i
    const int step = adjacent ? 2 : 1, apart = adjacent ? 1 : half;
    T* row = q + (size_t)t * ldq;
    // queries
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        int h = idx / half, i = idx % half;
        T* qr = row + (size_t)h * (D + R) + D;
        float u = xr_to_f32<T>(qr[step * i]), v = xr_to_f32<T>(qr[step * i + apart]);
        qr[step * i] = xr_from_f32<T>(u * cs[i] - v * cs[half + i]);
        qr[step * i + apart] = xr_from_f32<T>(v * cs[i] + u * cs[half + i]);
    }
    if (cache == nullptr) return;
    const T* down = down_all + (size_t)t * ldd;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { float v = xr_to_f32<T>(down[i]); ss += v * v; }
    ss = xr_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)C + eps);
    const int page = block_tables[(size_t)tok_seg[t] * max_pages + pos / page_size];
    T* dst = cache + (size_t)page * page_stride + (size_t)(pos % page_size) * (C + R);
    for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = xr_from_f32<T>(xr_to_f32<T>(down[i]) * inv * norm_w[i]);
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float out = xr_to_f32<T>(down[C + i]);
        if (i < rot_dims) {
            int j, other; bool first;
            if (adjacent) { j = i >> 1; first = !(i & 1); other = i ^ 1; }
            else { first = i < half; j = first ? i : i - half; other = first ? i + half : i - half; }
            const float z = xr_to_f32<T>(down[C + other]);
            out = first ? out * cs[j] - z * cs[half + j] : out * cs[j] + z * cs[half + j];
        }
        dst[C + i] = xr_from_f32<T>(out);
    }
}

XR_EXPORT int xr_latent_prep(void* q, int dtype, long long ldq, const void* down, long long ldd, const int* positions, const int* tok_seg,
                             const int* block_tables, const double* freq, const float* norm_w, void* cache,
                             long long page_stride, int n, int H, int D, int R, int C, int rot_dims, int max_pages,
                             int page_size, float eps, int adjacent, cudaStream_t stream) {
    if (n < 1 || H < 1 || D < 0 || R < 0 || C < 1 || rot_dims < 0 || rot_dims > R || (rot_dims & 1) || page_size < 1) return XR_ERR_ARG;
    if (cache != nullptr && (down == nullptr || norm_w == nullptr)) return XR_ERR_ARG;
    size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float);
    if (smem > 40000) return XR_ERR_ARG;
    if (dtype == XR_F32)
        xr_launch((k_latent_prep<float>), dim3(n), dim3(256), smem, stream, (float*)q, ldq, (const float*)down, ldd, positions, tok_seg, block_tables,
                  freq, norm_w, (float*)cache, page_stride, H, D, R, C, rot_dims, max_pages, page_size, eps, adjacent ? 1 : 0);
    else if (dtype == XR_BF16)
        xr_launch((k_latent_prep<__nv_bfloat16>), dim3(n), dim3(256), smem, stream, (__nv_bfloat16*)q, ldq, (const __nv_bfloat16*)down, ldd, positions, tok_seg,
                  block_tables, freq, norm_w, (__nv_bfloat16*)cache, page_stride, H, D, R, C, rot_dims, max_pages, page_size, eps, adjacent ? 1 : 0);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// A small matrix per head: out[t][h][j] = sum_k in[t][h][k] * W_h(k, j) (* sigmoid(gate[t][h]), or, with `gate_each`,
// * sigmoid(gate[t][h * J + j])), float32 sums.
// in row t, head h starts at in + t * ld_in + h * head_in; W_h(k, j) = W[h * w_head + k * w_k + j * w_j]
// (so both "W_h as stored" and its transpose are a choice of strides); out row t, head h at out + t * ld_out + h * J.
// Tile: 64 tokens x 64 columns, 256 threads with 4 x 4 results each, 16 values of k a round.
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TW, typename TO, typename TG>
__global__ void __launch_bounds__(256)
k_head_matmul(const TI* __restrict__ in, long long ld_in, int head_in, const TW* __restrict__ W, long long w_head, long long w_k,
              long long w_j, TO* __restrict__ out, long long ld_out, const TG* __restrict__ gate, long long ld_gate,
              int n, int Kd, int J, int gate_each) {
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
        if (gate != nullptr && !gate_each) g = 1.0f / (1.0f + expf(-xr_to_f32<TG>(gate[(size_t)t * ld_gate + h])));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int c = j0 + tx + 16 * j;
            if (c >= J) continue;
            if (gate != nullptr && gate_each) g = 1.0f / (1.0f + expf(-xr_to_f32<TG>(gate[(size_t)t * ld_gate + (size_t)h * J + c])));
            out[(size_t)t * ld_out + (size_t)h * J + c] = xr_from_f32<TO>(acc[i][j] * g);
        }
    }
}

// in_dtype / w_dtype / out_dtype: XR_F32 or XR_BF16; the gate (optional) has the dtype `gate_dtype`.
XR_EXPORT int xr_head_matmul(const void* in, int in_dtype, long long ld_in, int head_in, const void* W, int w_dtype,
                             long long w_head, long long w_k, long long w_j, void* out, int out_dtype, long long ld_out,
                             const void* gate, int gate_dtype, long long ld_gate, int n, int H, int Kd, int J, int gate_each,
                             cudaStream_t stream) {
    if (n < 1 || H < 1 || Kd < 1 || J < 1 || H > 65535) return XR_ERR_ARG;
    dim3 grid((n + 63) / 64, (J + 63) / 64, H);
    if (grid.y > 65535) return XR_ERR_ARG;
#define HM(TI, TW, TO, TG) xr_launch((k_head_matmul<TI, TW, TO, TG>), grid, dim3(256), 0, stream, (const TI*)in, ld_in, head_in, (const TW*)W, \
                                     w_head, w_k, w_j, (TO*)out, ld_out, (const TG*)gate, ld_gate, n, Kd, J, gate_each)
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
        case XR_BF16 * 8 + XR_BF16 * 4 + XR_BF16 * 2 + 0: HM(bf, bf, bf, float); break;
        case XR_BF16 * 8 + XR_F32 * 4 + XR_BF16 * 2 + 0: HM(bf, float, bf, float); break;
        default: return XR_ERR_ARG;
    }
#undef HM
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Attention over the cached rows, one block per token, a warp per head (eight heads at a time).  Keys are taken in
// tiles of 32 in ascending order from the first visible position (0, or position - window + 1 with a window of
// `window` > 0 keys), with a running maximum: a query's result depends on its position
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
                   int H, int C, int R, int max_pages, int page_size, float scale, int window) {
    xr_pdl_launch();
    extern __shared__ float sm[];
    const int W = C + R, ldw = W | 1;                       // odd row stride: lanes that read one column of 32 rows hit 32 banks
    float* tile = sm;                                        // [32][ldw]
    float* qs = sm + 32 * ldw;                               // [LA_WARPS][ldw]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int* bt = block_tables + (size_t)tok_seg[t] * max_pages;
    const int kfirst = (window > 0 && pos >= window) ? pos - window + 1 : 0;     // the first key the token sees
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
        for (int k0 = kfirst; k0 <= pos; k0 += 32) {
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
                                  float scale, int window, cudaStream_t stream) {
    if (n < 1 || H < 1 || C < 1 || C > 32 * LA_MAX_ND || R < 0 || page_size < 1) return XR_ERR_ARG;
    const size_t smem = (size_t)(32 + LA_WARPS) * ((C + R) | 1) * sizeof(float);
    if (smem > 220 * 1024) return XR_ERR_ARG;
    cudaError_t e = cudaSuccess;
    if (dtype == XR_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(k_latent_attention<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return XR_ERR_LAUNCH;
        xr_launch((k_latent_attention<float>), dim3(n), dim3(32 * LA_WARPS), smem, stream, ql, (const float*)qr, ld_qr, head_qr, out,
                  (const float*)cache, page_stride, positions, tok_seg, block_tables, H, C, R, max_pages, page_size, scale, window);
    } else if (dtype == XR_BF16) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(k_latent_attention<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return XR_ERR_LAUNCH;
        xr_launch((k_latent_attention<__nv_bfloat16>), dim3(n), dim3(32 * LA_WARPS), smem, stream, ql, (const __nv_bfloat16*)qr, ld_qr,
                  head_qr, out, (const __nv_bfloat16*)cache, page_stride, positions, tok_seg, block_tables, H, C, R, max_pages,
                  page_size, scale, window);
    } else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// The same attention on tensor cores (bfloat16, mma.sync m16n8k16 with float32 accumulators), for latent sizes that
// are multiples of 64 up to 512 and rotated parts that are multiples of 8.
//
// A CTA of four warps takes one token and up to sixteen of its heads (the rows of the M = 16 tile: all heads read the
// same cached rows) over a range of keys, in tiles of 32 keys that cp.async brings to shared memory two deep.
//   scores   S [16 x 32] = Q [16 x Wp] K^T: warp w takes keys 8w .. 8w + 7 of the tile (Wp = C + R rounded up to 16,
//            the padding zero on both sides); the scores go to shared memory, times `scale`, keys beyond the range -inf;
//   softmax  every warp reads S in the layout of the A operand (rows g and g + 8, g = lane / 4), keeps the running
//            maximum and sum of its rows (the four lanes of a row agree through shuffles) and has P in registers;
//   sums     O [16 x C] += P [16 x 32] V [32 x C], warp w owning columns w C/4 .. (w+1) C/4; V is the first C columns
//            of the same rows, read through ldmatrix.trans.
// grid = (tokens, tiles of 16 heads, splits).  With one split a CTA writes out = O / l; with more, split s takes keys
// [first + s chunk, first + (s+1) chunk), first the first key the token sees (0, or position - window + 1), and leaves
// (m, l, O) in scratch for k_latent_merge, which combines them per (token, head).
// ---------------------------------------------------------------------------------------------
#define LT_KT 32
#define LT_NW 4
#define LT_MAX_NT 16         // n8 tiles of O per warp: C / 4 / 8 <= 16, so C <= 512

__device__ __forceinline__ uint32_t lt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lt_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lt_ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void lt_ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lt_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lt_cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t lt_pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
// bytes between rows of a tile in shared memory: an odd number of 16-byte units, so that the eight rows an ldmatrix
// reads lie in different banks
static __host__ __device__ inline int lt_row_bytes(int Wp) { int u = Wp / 8; return ((u & 1) ? u : u + 1) * 16; }

__global__ void __launch_bounds__(32 * LT_NW)
k_latent_attention_mma(const __nv_bfloat16* __restrict__ ql, long long ql_tok, long long ql_head,
                       const __nv_bfloat16* __restrict__ qr, long long ld_qr, int head_qr,
                       float* __restrict__ out, __nv_bfloat16* __restrict__ out_h, long long oh_tok, long long oh_head,
                       float* __restrict__ part_o, float* __restrict__ part_ml,
                       const __nv_bfloat16* __restrict__ cache, long long page_stride, const int* __restrict__ positions,
                       const int* __restrict__ tok_seg, const int* __restrict__ block_tables, int H, int C, int R, int max_pages,
                       int page_size, float scale, int chunk, int splits, int window) {
    xr_pdl_launch();
    extern __shared__ __align__(16) uint8_t lt_sm[];
    const int W = C + R, Wp = (W + 15) / 16 * 16, rb = lt_row_bytes(Wp);
    uint8_t* Qs = lt_sm;                                   // [16][rb]
    uint8_t* Ks = Qs + 16 * rb;                            // [2][32][rb]
    float* Ss = reinterpret_cast<float*>(Ks + 2 * LT_KT * rb);   // [16][33]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c2 = (lane & 3) * 2;
    const int t = blockIdx.x, h0 = blockIdx.y * 16, split = blockIdx.z;
    const int pos = positions[t];
    const int* bt = block_tables + (size_t)tok_seg[t] * max_pages;
    const int kfirst = (window > 0 && pos >= window) ? pos - window + 1 : 0;     // the first key the token sees
    const int kbeg = kfirst + split * chunk, kend = min(pos + 1, kbeg + chunk);  // keys [kbeg, kend)
    const int mt = gridDim.y;
    float* my_ml = part_ml + (((size_t)t * mt + blockIdx.y) * splits + split) * 32;
    float* my_o = part_o + (((size_t)t * mt + blockIdx.y) * splits + split) * 16 * (size_t)C;
    xr_pdl_wait();
    if (kend <= kbeg) {                                    // nothing for this split (only with splits > 1)
        if (threadIdx.x < 16) { my_ml[threadIdx.x * 2] = -INFINITY; my_ml[threadIdx.x * 2 + 1] = 0.f; }
        return;
    }
    // zeros everywhere first: the padding columns stay zero, and rows that a last, partial tile leaves alone hold
    // finite values (a weight of zero times them must be zero)
    for (int i = threadIdx.x; i < (16 + 2 * LT_KT) * rb / 16; i += blockDim.x) reinterpret_cast<uint4*>(lt_sm)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    const int n_tiles = (kend - kbeg + LT_KT - 1) / LT_KT;
    const int chunks16 = W / 8;                            // 16-byte pieces of a cached row
    auto fetch = [&](int tile, int buf) {
        // a warp per key (its page and row worked out once), the lanes over the row's 16-byte pieces
        const int k0 = kbeg + tile * LT_KT, cnt = min(LT_KT, kend - k0);
        for (int j = warp; j < cnt; j += LT_NW) {
            const int kp = k0 + j;
            const __nv_bfloat16* src = cache + (size_t)bt[kp / page_size] * page_stride + (size_t)(kp % page_size) * W;
            const uint32_t dst = lt_smem(Ks + ((size_t)buf * LT_KT + j) * rb);
            for (int piece = lane; piece < chunks16; piece += 32) lt_cp16(dst + piece * 16, src + piece * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, 0);
    // the queries: [latent part | rotated part] of heads h0 .. h0 + 15 (rows of heads that do not exist stay zero)
    for (int i = threadIdx.x; i < 16 * (W / 2); i += blockDim.x) {
        const int r = i / (W / 2), e = (i % (W / 2)) * 2, h = h0 + r;
        if (h >= H) continue;
        uint32_t v;
        if (e < C) v = *reinterpret_cast<const uint32_t*>(ql + (size_t)t * ql_tok + (size_t)h * ql_head + e);
        else v = *reinterpret_cast<const uint32_t*>(qr + (size_t)t * ld_qr + (size_t)h * head_qr + (e - C));
        *reinterpret_cast<uint32_t*>(Qs + (size_t)r * rb + e * 2) = v;
    }
    const int DW = C / LT_NW, NT = DW / 8;                 // this warp's columns of O and their n8 tiles
    float acc[LT_MAX_NT][4];
#pragma unroll
    for (int i = 0; i < LT_MAX_NT; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;       // rows g and g + 8
    const uint32_t q_addr = lt_smem(Qs) + (lane & 15) * rb + (lane >> 4) * 16;
    for (int tile = 0; tile < n_tiles; tile++) {
        const int buf = tile & 1;
        if (tile + 1 < n_tiles) {
            fetch(tile + 1, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t k_base = lt_smem(Ks + (size_t)buf * LT_KT * rb);
        // ---- scores of keys 8 warp .. 8 warp + 7
        {
            // four accumulators and four k steps a round: consecutive MMAs do not wait for one another
            float s[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f}, sc[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t k_addr = k_base + (8 * warp + (lane & 7)) * rb + ((lane >> 3) & 3) * 16;
            const int steps = Wp / 16;
            int ks = 0;
            for (; ks + 3 < steps; ks += 4) {
                uint32_t a0[4], a1[4], a2[4], a3[4], b01[4], b23[4];
                lt_ldsm_x4(b01, k_addr + ks * 32);               // this key tile's columns of two k steps
                lt_ldsm_x4(b23, k_addr + ks * 32 + 64);
                lt_ldsm_x4(a0, q_addr + ks * 32);
                lt_ldsm_x4(a1, q_addr + ks * 32 + 32);
                lt_ldsm_x4(a2, q_addr + ks * 32 + 64);
                lt_ldsm_x4(a3, q_addr + ks * 32 + 96);
                lt_mma(s, a0, b01[0], b01[1]);
                lt_mma(sb, a1, b01[2], b01[3]);
                lt_mma(sc, a2, b23[0], b23[1]);
                lt_mma(sd, a3, b23[2], b23[3]);
            }
            for (; ks < steps; ks++) {
                uint32_t a[4], b[2];
                lt_ldsm_x4(a, q_addr + ks * 32);
                lt_ldsm_x2(b, k_addr + ks * 32);
                lt_mma(s, a, b[0], b[1]);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) s[i] = (s[i] + sb[i]) + (sc[i] + sd[i]);
            const int key = kbeg + tile * LT_KT + 8 * warp + c2;
            const float s0 = key < kend ? s[0] * scale : -INFINITY, s1 = key + 1 < kend ? s[1] * scale : -INFINITY;
            const float s2 = key < kend ? s[2] * scale : -INFINITY, s3 = key + 1 < kend ? s[3] * scale : -INFINITY;
            Ss[g * 33 + 8 * warp + c2] = s0; Ss[g * 33 + 8 * warp + c2 + 1] = s1;
            Ss[(g + 8) * 33 + 8 * warp + c2] = s2; Ss[(g + 8) * 33 + 8 * warp + c2 + 1] = s3;
        }
        __syncthreads();
        // ---- softmax (every warp for itself): this thread's values of rows g and g + 8, in the A operand's layout
        float lo[8], hi[8];
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const int col = 16 * kk + c2;
            lo[4 * kk] = Ss[g * 33 + col]; lo[4 * kk + 1] = Ss[g * 33 + col + 1];
            lo[4 * kk + 2] = Ss[g * 33 + col + 8]; lo[4 * kk + 3] = Ss[g * 33 + col + 9];
            hi[4 * kk] = Ss[(g + 8) * 33 + col]; hi[4 * kk + 1] = Ss[(g + 8) * 33 + col + 1];
            hi[4 * kk + 2] = Ss[(g + 8) * 33 + col + 8]; hi[4 * kk + 3] = Ss[(g + 8) * 33 + col + 9];
        }
        float mx_lo = lo[0], mx_hi = hi[0];
#pragma unroll
        for (int i = 1; i < 8; i++) { mx_lo = fmaxf(mx_lo, lo[i]); mx_hi = fmaxf(mx_hi, hi[i]); }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);        // finite: a tile holds at least one key
        const float corr_lo = __expf(m_lo - mn_lo), corr_hi = __expf(m_hi - mn_hi);
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            lo[i] = __expf(lo[i] - mn_lo); hi[i] = __expf(hi[i] - mn_hi);
            sum_lo += lo[i]; sum_hi += hi[i];
        }
        sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1); sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
        sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1); sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
        l_lo = l_lo * corr_lo + sum_lo; l_hi = l_hi * corr_hi + sum_hi;
        m_lo = mn_lo; m_hi = mn_hi;
        uint32_t pa[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            pa[kk][0] = lt_pack(lo[4 * kk], lo[4 * kk + 1]); pa[kk][1] = lt_pack(hi[4 * kk], hi[4 * kk + 1]);
            pa[kk][2] = lt_pack(lo[4 * kk + 2], lo[4 * kk + 3]); pa[kk][3] = lt_pack(hi[4 * kk + 2], hi[4 * kk + 3]);
        }
        // ---- O = O corr + P V over this warp's columns
        const uint32_t v_addr = k_base + (lane & 15) * rb + (warp * DW + (lane >> 4) * 8) * 2;
#pragma unroll
        for (int nt = 0; nt < LT_MAX_NT; nt += 2) {
            if (nt < NT) {
                acc[nt][0] *= corr_lo; acc[nt][1] *= corr_lo; acc[nt][2] *= corr_hi; acc[nt][3] *= corr_hi;
                acc[nt + 1][0] *= corr_lo; acc[nt + 1][1] *= corr_lo; acc[nt + 1][2] *= corr_hi; acc[nt + 1][3] *= corr_hi;
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    uint32_t b[4];
                    lt_ldsm_x4_trans(b, v_addr + kk * 16 * rb + nt * 16);
                    lt_mma(acc[nt], pa[kk], b[0], b[1]);
                    lt_mma(acc[nt + 1], pa[kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();                                   // S and this buffer are free for the tile after next
    }
    // ---- results
    if (splits == 1) {
        const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
#pragma unroll
        for (int nt = 0; nt < LT_MAX_NT; nt++) {
            if (nt < NT) {
                const int col = warp * DW + nt * 8 + c2;
                if (out_h != nullptr) {
                    if (h0 + g < H) *reinterpret_cast<uint32_t*>(out_h + (size_t)t * oh_tok + (size_t)(h0 + g) * oh_head + col) = lt_pack(acc[nt][0] * inv_lo, acc[nt][1] * inv_lo);
                    if (h0 + g + 8 < H) *reinterpret_cast<uint32_t*>(out_h + (size_t)t * oh_tok + (size_t)(h0 + g + 8) * oh_head + col) = lt_pack(acc[nt][2] * inv_hi, acc[nt][3] * inv_hi);
                } else {
                    if (h0 + g < H) *reinterpret_cast<float2*>(out + ((size_t)t * H + h0 + g) * C + col) = make_float2(acc[nt][0] * inv_lo, acc[nt][1] * inv_lo);
                    if (h0 + g + 8 < H) *reinterpret_cast<float2*>(out + ((size_t)t * H + h0 + g + 8) * C + col) = make_float2(acc[nt][2] * inv_hi, acc[nt][3] * inv_hi);
                }
            }
        }
    } else {
        if (warp == 0 && (lane & 3) == 0) {
            my_ml[g * 2] = m_lo; my_ml[g * 2 + 1] = l_lo;
            my_ml[(g + 8) * 2] = m_hi; my_ml[(g + 8) * 2 + 1] = l_hi;
        }
#pragma unroll
        for (int nt = 0; nt < LT_MAX_NT; nt++) {
            if (nt < NT) {
                const int col = warp * DW + nt * 8 + c2;
                *reinterpret_cast<float2*>(my_o + (size_t)g * C + col) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(my_o + (size_t)(g + 8) * C + col) = make_float2(acc[nt][2], acc[nt][3]);
            }
        }
    }
}

// out[t][h] = sum_s O_s e^(m_s - M) / sum_s l_s e^(m_s - M), M = max_s m_s, over the splits that saw any key; one warp per
// (t, h): the lanes first hold one split each (its weight e^(m_s - M), zero for a split without keys), then one column each
__global__ void __launch_bounds__(128)
k_latent_merge(const float* __restrict__ part_o, const float* __restrict__ part_ml, float* __restrict__ out,
               __nv_bfloat16* __restrict__ out_h, long long oh_tok, long long oh_head, int n, int H, int C, int mt, int splits) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 4 + warp;
    if (idx >= (long long)n * H) return;
    const int t = (int)(idx / H), h = (int)(idx % H), tile = h / 16, row = h % 16;
    const float* ml = part_ml + ((size_t)t * mt + tile) * splits * 32 + row * 2;
    const float* po = part_o + ((size_t)t * mt + tile) * splits * 16 * (size_t)C + (size_t)row * C;
    float M = -INFINITY;
    for (int s = lane; s < splits; s += 32) if (ml[s * 32 + 1] > 0.f) M = fmaxf(M, ml[s * 32]);
    M = xr_warp_max(M);
    float L = 0.f;
    for (int s = lane; s < splits; s += 32) if (ml[s * 32 + 1] > 0.f) L += ml[s * 32 + 1] * __expf(ml[s * 32] - M);
    L = xr_warp_sum(L);
    const float inv = 1.0f / L;
    float acc[LT_MAX_NT];                       // columns lane, lane + 32, ... (C <= 512)
#pragma unroll
    for (int i = 0; i < LT_MAX_NT; i++) acc[i] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        const int mine = s0 + lane;
        const float w_mine = (mine < splits && ml[mine * 32 + 1] > 0.f) ? __expf(ml[mine * 32] - M) : 0.f;
        const int cnt = min(32, splits - s0);
        for (int j = 0; j < cnt; j++) {
            const float w = __shfl_sync(0xffffffffu, w_mine, j);
            if (w == 0.f) continue;                    // (the same for the whole warp)
            const float* src = po + (size_t)(s0 + j) * 16 * C;
#pragma unroll
            for (int i = 0; i < LT_MAX_NT; i++) {
                const int d = lane + 32 * i;
                if (d < C) acc[i] = fmaf(src[d], w, acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < LT_MAX_NT; i++) {
        const int d = lane + 32 * i;
        if (d >= C) continue;
        if (out_h != nullptr) out_h[(size_t)t * oh_tok + (size_t)h * oh_head + d] = __float2bfloat16_rn(acc[i] * inv);
        else out[((size_t)t * H + h) * C + d] = acc[i] * inv;
    }
}

XR_EXPORT int xr_latent_attention_mma_supported(int C, int R) {
    const int Wp = (C + R + 15) / 16 * 16;
    const size_t smem = (size_t)(16 + 2 * LT_KT) * lt_row_bytes(Wp) + 16 * 33 * sizeof(float);
    return C >= 64 && C % 64 == 0 && C <= 8 * LT_NW * LT_MAX_NT && R % 8 == 0 && smem <= 200 * 1024;
}

// ql: the queries in the latent space, bfloat16, head h of token t at ql + t * ql_tok + h * ql_head (elements); the result
// goes to out [n][H * C] float32, or, when out_h is given, as bfloat16 to out_h + t * oh_tok + h * oh_head.
// qr: rotated query parts (bfloat16, head h of token t at qr + t * ld_qr + h * head_qr);
// out [n][H * C] float32; part_o [n * ceil(H/16) * splits * 16 * C], part_ml [n * ceil(H/16) * splits * 32]: float32
// scratch (used when splits > 1); chunk: keys per split, a multiple of 32.
XR_EXPORT int xr_latent_attention_mma(const void* ql, long long ql_tok, long long ql_head, const void* qr, long long ld_qr, int head_qr,
                                      float* out, void* out_h, long long oh_tok, long long oh_head, float* part_o, float* part_ml, const void* cache, long long page_stride, const int* positions,
                                      const int* tok_seg, const int* block_tables, int n, int H, int C, int R, int max_pages,
                                      int page_size, float scale, int chunk, int splits, int window, cudaStream_t stream) {
    if (n < 1 || H < 1 || !xr_latent_attention_mma_supported(C, R) || page_size < 1 || splits < 1 || chunk < LT_KT || chunk % LT_KT) return XR_ERR_ARG;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return XR_ERR_ARG;
    if ((ql_tok | ql_head | oh_tok | oh_head) & 1) return XR_ERR_ARG;            // pairs of bfloat16 are read and written
    if (splits > 65535 || (H + 15) / 16 > 65535) return XR_ERR_ARG;
    const int Wp = (C + R + 15) / 16 * 16;
    const size_t smem = (size_t)(16 + 2 * LT_KT) * lt_row_bytes(Wp) + 16 * 33 * sizeof(float);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_latent_attention_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return XR_ERR_LAUNCH;
        configured = true;
    }
    const int mt = (H + 15) / 16;
    xr_launch(k_latent_attention_mma, dim3(n, mt, splits), dim3(32 * LT_NW), smem, stream, (const __nv_bfloat16*)ql, ql_tok, ql_head,
              (const __nv_bfloat16*)qr, ld_qr, head_qr, out, (__nv_bfloat16*)out_h, oh_tok, oh_head, part_o, part_ml, (const __nv_bfloat16*)cache, page_stride, positions, tok_seg, block_tables, H, C, R,
              max_pages, page_size, scale, chunk, splits, window);
    if (splits > 1) {
        const long long warps = (long long)n * H;
        xr_launch(k_latent_merge, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml, out, (__nv_bfloat16*)out_h, oh_tok, oh_head, n, H, C, mt, splits);
    }
    return xr_launch_status();
}


// ---------------------------------------------------------------------------------------------
// Head-major copies around the per-head products on tensor cores (the grouped product wants the rows of one head
// together, n_pad rows a head):
//   gather:   out[h * n_pad + t][k] = in[t][h * head_in + k], k < Kd (rows t >= n: zeros)
//   scatter:  y[t][h * J + j] = in[h * n_pad + t][j] * sigmoid(gate[t][h])     (in: the product's float32 sums, rounded once here;
//             with `gate_each` the gate is gate[t][h * J + j])
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
k_heads_gather(const __nv_bfloat16* __restrict__ in, long long ld_in, int head_in, __nv_bfloat16* __restrict__ out, int n, int n_pad, int Kd) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    __nv_bfloat16* o = out + ((size_t)h * n_pad + t) * Kd;
    if (t >= n) {
        for (int k = threadIdx.x; k < Kd; k += blockDim.x) o[k] = __float2bfloat16_rn(0.f);
        return;
    }
    const __nv_bfloat16* a = in + (size_t)t * ld_in + (size_t)h * head_in;
    for (int k = threadIdx.x; k < Kd; k += blockDim.x) o[k] = a[k];
}

__global__ void __launch_bounds__(128)
k_heads_scatter_gate(const float* __restrict__ in, __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ gate,
                     long long ld_gate, int n_pad, int H, int J, int gate_each) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    float g = (gate != nullptr && !gate_each) ? 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * ld_gate + h]))) : 1.0f;
    const float* a = in + ((size_t)h * n_pad + t) * J;
    __nv_bfloat16* o = y + ((size_t)t * H + h) * J;
    for (int j = threadIdx.x; j < J; j += blockDim.x) {
        if (gate != nullptr && gate_each) g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * ld_gate + (size_t)h * J + j])));
        o[j] = __float2bfloat16_rn(a[j] * g);
    }
}

XR_EXPORT int xr_heads_gather(const void* in, long long ld_in, int head_in, void* out, int n, int n_pad, int H, int Kd, cudaStream_t stream) {
    if (n < 1 || n_pad < n || H < 1 || H > 65535 || Kd < 1) return XR_ERR_ARG;
    xr_launch(k_heads_gather, dim3(n_pad, H), dim3(128), 0, stream, (const __nv_bfloat16*)in, ld_in, head_in, (__nv_bfloat16*)out, n, n_pad, Kd);
    return xr_launch_status();
}

XR_EXPORT int xr_heads_scatter_gate(const void* in, void* y, const void* gate, long long ld_gate, int n, int n_pad, int H, int J,
                                    int gate_each, cudaStream_t stream) {
    if (n < 1 || n_pad < n || H < 1 || H > 65535 || J < 1) return XR_ERR_ARG;
    xr_launch(k_heads_scatter_gate, dim3(n, H), dim3(128), 0, stream, (const float*)in, (__nv_bfloat16*)y, (const __nv_bfloat16*)gate,
              ld_gate, n_pad, H, J, gate_each);
    return xr_launch_status();
}
