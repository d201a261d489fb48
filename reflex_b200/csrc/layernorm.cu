// Layer norm with a weight and no bias, with the residual add that precedes it.
//
// One block per output row, the same interface as the RMSNorm kernel:
//   src = rows ? rows[blockIdx.x] : blockIdx.x
//   t   = x[src] (+ delta[src])                     residual sum in 32-bit
//   if x_out: x_out[src] = t                        (only without `rows`; may be x)
//   if out:   out[blockIdx.x] = (t - mean(t)) / sqrt(var(t) + eps) * w
// with var the mean of the squared deviations (two passes over the row, which
// lies in shared memory).  Statistics are 32-bit; the reduction order depends
// on the row's size alone.
#include "common.cuh"

namespace {

using namespace rfx;

template <typename TD, typename TO>
__global__ void layernorm_kernel(const float* x, const TD* __restrict__ delta, float* x_out,
                                 const float* __restrict__ w, TO* __restrict__ out,
                                 const int* __restrict__ rows, int H, float eps) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float row_buf[];  // H floats
    pdl_prologue();
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + (size_t)src * H;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float t = xr[c];
        if (delta) t += ld<TD>(delta, (size_t)src * H + c);
        row_buf[c] = t;
        if (x_out) x_out[(size_t)src * H + c] = t;
        sum += t;
    }
    if (!out) return;
    const float mean = block_sum(sum, scratch) / (float)H;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float d = row_buf[c] - mean;
        sq = fmaf(d, d, sq);
    }
    const float var = block_sum(sq, scratch) / (float)H;
    const float r = 1.0f / sqrtf(var + eps);
    TO* orow = out + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) st<TO>(orow, c, ((row_buf[c] - mean) * r) * w[c]);
}

int ln_threads(int H) {
    int t = ((H + 3) / 4 + 31) / 32 * 32;
    if (t < 32) t = 32;
    if (t > 256) t = 256;
    return t;
}

}  // namespace

extern "C" int rfx_layernorm(const float* x, const void* delta, int delta_dt, float* x_out, const float* w,
                             float eps, void* out, int out_dt, const int* rows, int R_out, int H,
                             void* stream) {
    if (R_out <= 0) return 0;
    if (rows && x_out) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = ln_threads(H);
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
#define RFX_NORM(TD, TO)                                                                          \
    do {                                                                                          \
        if (smem > 48 * 1024) {                                                                   \
            cudaError_t e = cudaFuncSetAttribute(layernorm_kernel<TD, TO>,                        \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                                 (int)smem);                                      \
            if (e != cudaSuccess) return (int)e;                                                  \
        }                                                                                         \
        RFX_LAUNCH((layernorm_kernel<TD, TO>), R_out, threads, smem, s, x, (const TD*)delta, x_out, \
                   w, (TO*)out, rows, H, eps);                                                    \
    } while (0)
    const bool dbf = delta && delta_dt == RFX_DT_BF16;
    if (out_dt == RFX_DT_BF16) {
        if (dbf) RFX_NORM(__nv_bfloat16, __nv_bfloat16);
        else RFX_NORM(float, __nv_bfloat16);
    } else if (out_dt == RFX_DT_F32) {
        if (dbf) RFX_NORM(__nv_bfloat16, float);
        else RFX_NORM(float, float);
    } else {
        return RFX_ERR_BAD_ARG;
    }
#undef RFX_NORM
    return 0;
}
