// Latent attention around the attention kernel: what follows the stacked
// down-projection, and the per-head products between latents and heads.
//
//  * rfx_latent_post: a row of the stacked product [query latent | key/value
//    latent | gates] -> RMSNorm of the query latent (out, for the query
//    up-projection), RMSNorm of the key/value latent written into the paged
//    cache at the row's position (one "head" of kv_rank elements a position),
//    sigmoid of the per-head gates (32-bit).
//  * rfx_heads_linear: y[r, b, :] = x[r, b, :] W_b^T for every head b, W
//    [heads, N, K]; optionally times a per-(row, head) factor.  32-bit
//    accumulation, each output reduced over k in index order by one thread.
#include "common.cuh"
#include "paged.cuh"

namespace {

using namespace rfx;

template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
latent_post_kernel(const TI* __restrict__ proj, int stride, const float* __restrict__ q_w,
                   const float* __restrict__ kv_w, float eps, const int* __restrict__ row_pos,
                   const int* __restrict__ row_slot, TO* __restrict__ q_out, TO* __restrict__ pages,
                   PagedKV cache, float* __restrict__ gate_out, int q_rank, int kv_rank, int n_gate,
                   int write_cache) {
    __shared__ float scratch[32];
    pdl_prologue();
    const int r = blockIdx.x;
    const TI* row = proj + (size_t)r * stride;
    // query latent
    float ss = 0.0f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
        const float t = ld<TI>(row, c);
        ss = fmaf(t, t, ss);
    }
    float rr = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
        st<TO>(q_out + (size_t)r * q_rank, c, (ld<TI>(row, c) * rr) * q_w[c]);
    // key/value latent, into the cache
    if (write_cache) {
        const TI* kv = row + q_rank;
        ss = 0.0f;
        for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
            const float t = ld<TI>(kv, c);
            ss = fmaf(t, t, ss);
        }
        rr = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
        TO* dst = pages + kv_offset(cache, row_slot[r], row_pos[r], 0);
        for (int c = threadIdx.x; c < kv_rank; c += blockDim.x)
            st<TO>(dst, c, (ld<TI>(kv, c) * rr) * kv_w[c]);
    }
    // gates
    const TI* gt = row + q_rank + kv_rank;
    for (int c = threadIdx.x; c < n_gate; c += blockDim.x)
        gate_out[(size_t)r * n_gate + c] = 1.0f / (1.0f + expf(-ld<TI>(gt, c)));
}

constexpr int TM = 64, TN = 64, TK = 16;

// x [R, heads, K] (row stride ldx), W [heads, N, K], y [R, heads, N] (row stride ldy);
// scale [R, heads] or null.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
heads_linear_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ W, TO* __restrict__ y,
                    int ldy, const float* __restrict__ scale, int R, int N, int K, int heads) {
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[TK][TN + 1];
    pdl_prologue();
    const int b = blockIdx.z;
    const int r0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* xb = x + (size_t)b * K;
    const T* wb = W + (size_t)b * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int row = e / TK, kk = e % TK;
            const int k = k0 + kk;
            xs[kk][row] = (r0 + row < R && k < K) ? ld<T>(xb, (size_t)(r0 + row) * ldx + k) : 0.0f;
            ws[kk][row] = (n0 + row < N && k < K) ? ld<T>(wb, (size_t)(n0 + row) * K + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) c[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], c[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty * 4 + i;
        if (r >= R) continue;
        const float f = scale ? scale[(size_t)r * heads + b] : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) st<TO>(y + (size_t)r * ldy + (size_t)b * N, n, acc[i][j] * f);
        }
    }
}

// The same product for a few rows (decode): a block takes one head's rows into
// shared memory, a warp takes output columns one after another, reads the
// column's weights once (16 bytes a lane where the rows allow) and applies
// them to every row.  Sums are 32-bit; the order depends on K alone.
constexpr int GV_ROWS = 16;

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
heads_gemv_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ W, TO* __restrict__ y, int ldy,
                  const float* __restrict__ scale, int R, int N, int K, int heads) {
    extern __shared__ __align__(16) float xs[];  // [R][K]
    pdl_prologue();
    const int b = blockIdx.x;
    for (int e = threadIdx.x; e < R * K; e += blockDim.x)
        xs[e] = ld<T>(x, (size_t)(e / K) * ldx + (size_t)b * K + e % K);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const T* wb = W + (size_t)b * N * K;
    const bool vec = sizeof(T) == 2 && (K & 7) == 0 && (reinterpret_cast<uintptr_t>(wb) & 15) == 0;
    for (int n = blockIdx.y * nwarps + warp; n < N; n += gridDim.y * nwarps) {
        const T* wrow = wb + (size_t)n * K;
        float acc[GV_ROWS];
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) acc[r] = 0.0f;
        if (vec) {
            for (int v = lane; v < K / 8; v += 32) {
                const uint4 u = reinterpret_cast<const uint4*>(wrow)[v];
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
                float w[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(p[i]);
                    w[2 * i] = f.x;
                    w[2 * i + 1] = f.y;
                }
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r) {
                    if (r >= R) break;
                    const float* xr = xs + r * K + 8 * v;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r] = fmaf(xr[i], w[i], acc[r]);
                }
            }
        } else {
            for (int c = lane; c < K; c += 32) {
                const float w = ld<T>(wrow, c);
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r)
                    if (r < R) acc[r] = fmaf(xs[r * K + c], w, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
            if (r >= R) break;
            const float v = warp_sum(acc[r]);
            if (lane == 0) st<TO>(y + (size_t)r * ldy + (size_t)b * N, n, v * (scale ? scale[(size_t)r * heads + b] : 1.0f));
        }
    }
}

// y[r, b, :] *= scale[r, b]
template <typename T>
__global__ void scale_heads_kernel(T* __restrict__ y, const float* __restrict__ scale, size_t total,
                                   int N) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x)
        st<T>(y, i, ld<T>(y, i) * scale[i / N]);
}

}  // namespace

extern "C" int rfx_latent_post(const void* proj, int in_dt, int ld, const float* q_w, const float* kv_w,
                               float eps, const int* row_pos, const int* row_slot, void* q_out,
                               void* pages, int out_dt, const int* page_table, int max_pages,
                               int page_size, float* gate_out, int R, int q_rank, int kv_rank,
                               int n_gate, int write_cache, void* stream) {
    if (R <= 0) return 0;
    if (q_rank <= 0 || kv_rank <= 0 || ld < q_rank + kv_rank + n_gate) return RFX_ERR_BAD_ARG;
    PagedKV cache{page_table, max_pages, page_size, 1, kv_rank};
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(TI, TO)                                                                               \
    RFX_LAUNCH((latent_post_kernel<TI, TO>), R, 128, 0, s, (const TI*)proj, ld, q_w, kv_w, eps, row_pos, \
               row_slot, (TO*)q_out, (TO*)pages, cache, gate_out, q_rank, kv_rank, n_gate, write_cache)
    if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_F32) RFX_GO(float, float);
    else if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_BF16) RFX_GO(float, __nv_bfloat16);
    else if (in_dt == RFX_DT_BF16 && out_dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16, __nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}

extern "C" int rfx_heads_linear(const void* x, int ldx, const void* W, void* y, int ldy, int dt,
                                const float* scale, int R, int N, int K, int heads, void* stream) {
    if (R <= 0 || N <= 0 || heads <= 0) return 0;
    if (K <= 0) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (R <= GV_ROWS && (size_t)R * K * sizeof(float) <= 48 * 1024) {
        // a few rows: every weight is read once and meets all rows
        int gy = (N + 7) / 8;
        if (gy > 32) gy = 32;
        dim3 g(heads, gy);
        const size_t smem = (size_t)R * K * sizeof(float);
        if (dt == RFX_DT_F32)
            RFX_LAUNCH((heads_gemv_kernel<float, float>), g, 256, smem, s, (const float*)x, ldx, (const float*)W,
                       (float*)y, ldy, scale, R, N, K, heads);
        else if (dt == RFX_DT_BF16)
            RFX_LAUNCH((heads_gemv_kernel<__nv_bfloat16, __nv_bfloat16>), g, 256, smem, s,
                       (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, (__nv_bfloat16*)y, ldy, scale, R, N,
                       K, heads);
        else
            return RFX_ERR_BAD_ARG;
        return 0;
    }
    dim3 grid((N + TN - 1) / TN, (R + TM - 1) / TM, heads);
    if (grid.y > 65535 || grid.z > 65535) return RFX_ERR_UNSUPPORTED;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH((heads_linear_kernel<float, float>), grid, 256, 0, s, (const float*)x, ldx,
                   (const float*)W, (float*)y, ldy, scale, R, N, K, heads);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH((heads_linear_kernel<__nv_bfloat16, __nv_bfloat16>), grid, 256, 0, s,
                   (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, (__nv_bfloat16*)y, ldy, scale, R,
                   N, K, heads);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_scale_heads(void* y, int dt, const float* scale, long long total, int N, void* stream) {
    if (total <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int blocks = (int)((total + 255) / 256);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(scale_heads_kernel<float>, blocks, 256, 0, s, (float*)y, scale, (size_t)total, N);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(scale_heads_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)y, scale,
                   (size_t)total, N);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
