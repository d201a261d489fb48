// Mixture-of-experts feed-forward with top-k routing, for any number of rows.
//
//  * rfx_moe_route: router logits (32-bit, bias added here) -> the `top`
//    experts with the largest logits (ties: the lower index) and their weights,
//    the softmax over the chosen logits only.  One warp a row.
//  * rfx_moe_up: act[(r, k), :] = f(W_up[e] x[r]) for expert e = ids[r, k];
//    f = relu squared (act 0) or silu (act 1).  One warp an output element,
//    the row in shared memory.
//  * rfx_moe_down: y[r, :] = sum_k wts[r, k] W_down[ids[r, k]] act[(r, k), :],
//    the experts in the order of their rank, 32-bit sums: a row's result does
//    not depend on the batch.
// Expert weights are stacked: W_up [experts, ff, width], W_down [experts, width, ff].
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int MAX_PER_LANE = 8;  // up to 256 experts

__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 int* __restrict__ ids, float* __restrict__ wts, int R, int E, int top) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    float z[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = i * 32 + lane;
        z[i] = e < E ? logits[(size_t)r * E + e] + (bias ? bias[e] : 0.0f) : -INFINITY;
    }
    float zmax = 0.0f, sum = 0.0f, mine = 0.0f;  // lane k keeps the k-th choice's exponential
    int my_id = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (z[i] > best) { best = z[i]; best_e = e; }  // within a lane e rises: the lower index wins a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if ((k & 31) == lane && k < 32) { mine = p; my_id = best_e; }
        if (k >= 32 && lane == 0) {  // more than 32 choices: written unnormalised, scaled below
            ids[(size_t)r * top + k] = best_e;
            wts[(size_t)r * top + k] = p;
        }
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i)
            if (i * 32 + lane == best_e) z[i] = -INFINITY;
    }
    if (lane < top) {
        ids[(size_t)r * top + lane] = my_id;
        wts[(size_t)r * top + lane] = mine / sum;
    }
    if (lane == 0)
        for (int k = 32; k < top; ++k) wts[(size_t)r * top + k] /= sum;
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ x, const T* __restrict__ W, const int* __restrict__ ids,
              T* __restrict__ act, int top, int ff, int width, int kind) {
    extern __shared__ __align__(16) float xs[];  // the row
    pdl_prologue();
    const int pair = blockIdx.x;
    const int r = pair / top;
    const int e = ids[pair];
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = ld<T>(x, (size_t)r * width + c);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const T* We = W + (size_t)e * ff * width;
    for (int j = blockIdx.y * nwarps + warp; j < ff; j += gridDim.y * nwarps) {
        const T* wrow = We + (size_t)j * width;
        float dot = 0.0f;
        for (int c = lane; c < width; c += 32) dot = fmaf(xs[c], ld<T>(wrow, c), dot);
        dot = warp_sum(dot);
        if (lane == 0) {
            float a;
            if (kind == 0) { a = fmaxf(dot, 0.0f); a *= a; }
            else a = dot / (1.0f + expf(-dot));
            st<T>(act, (size_t)pair * ff + j, a);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ W, const int* __restrict__ ids,
                const float* __restrict__ wts, float* __restrict__ y, int top, int ff, int width) {
    extern __shared__ __align__(16) float as[];  // [top][ff]
    pdl_prologue();
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < top * ff; c += blockDim.x) as[c] = ld<T>(act, (size_t)r * top * ff + c);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int n = blockIdx.y * nwarps + warp; n < width; n += gridDim.y * nwarps) {
        float total = 0.0f;
        for (int k = 0; k < top; ++k) {
            const T* wrow = W + ((size_t)ids[(size_t)r * top + k] * width + n) * ff;
            float dot = 0.0f;
            for (int c = lane; c < ff; c += 32) dot = fmaf(as[k * ff + c], ld<T>(wrow, c), dot);
            total = fmaf(wts[(size_t)r * top + k], warp_sum(dot), total);
        }
        if (lane == 0) y[(size_t)r * width + n] = total;
    }
}

}  // namespace

extern "C" int rfx_moe_route(const float* logits, const float* bias, int* ids, float* wts, int R, int E,
                             int top, void* stream) {
    if (R <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E) return RFX_ERR_BAD_ARG;
    if (E > 32 * MAX_PER_LANE) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(moe_route_kernel, (R + 3) / 4, 128, 0, (cudaStream_t)stream, logits, bias, ids, wts, R, E, top);
    return 0;
}

extern "C" int rfx_moe_up(const void* x, const void* W, const int* ids, void* act, int dt, int R, int top,
                          int ff, int width, int kind, void* stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    int gy = (ff + 7) / 8;
    if (gy > 64) gy = 64;
    dim3 grid(R * top, gy);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(T)                                                                                        \
    do {                                                                                                 \
        if (smem > 48 * 1024) {                                                                          \
            cudaError_t e = cudaFuncSetAttribute(moe_up_kernel<T>,                                       \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                         \
        }                                                                                                \
        RFX_LAUNCH(moe_up_kernel<T>, grid, 256, smem, s, (const T*)x, (const T*)W, ids, (T*)act, top, ff,  \
                   width, kind);                                                                         \
    } while (0)
    if (dt == RFX_DT_F32) RFX_GO(float);
    else if (dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}

extern "C" int rfx_moe_down(const void* act, const void* W, const int* ids, const float* wts, float* y,
                            int dt, int R, int top, int ff, int width, void* stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)top * ff * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    int gy = (width + 7) / 8;
    if (gy > 64) gy = 64;
    dim3 grid(R, gy);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(T)                                                                                        \
    do {                                                                                                 \
        if (smem > 48 * 1024) {                                                                          \
            cudaError_t e = cudaFuncSetAttribute(moe_down_kernel<T>,                                     \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                         \
        }                                                                                                \
        RFX_LAUNCH(moe_down_kernel<T>, grid, 256, smem, s, (const T*)act, (const T*)W, ids, wts, y, top,   \
                   ff, width);                                                                           \
    } while (0)
    if (dt == RFX_DT_F32) RFX_GO(float);
    else if (dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}
