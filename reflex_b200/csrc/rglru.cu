// A real-gated linear recurrence, channel by channel, across steps.
//
// With u the recurrence's input (a short convolution's output), r_pre and
// i_pre the two gates' pre-activations (block-diagonal products of u, made
// before this kernel; their biases are added here), lam a learned number a
// channel and y_pre the other branch's projection:
//   r = sigmoid(r_pre + rb),  i = sigmoid(i_pre + ib)
//   log a = -c * r * softplus(lam),  a = exp(log a)
//   S_t = a S_(t-1) + sqrt(1 - a^2) * (i * u)          S = 0 before the first token
//   out_t = S_t * gelu_tanh(y_pre + yb)
// All of it is 32-bit; sqrt(1 - a^2) is taken as sqrt(-expm1(2 log a)), which
// keeps its digits when a is close to one.  S lives in the cache's state
// ([slot][...], at `state_off`), read when a step begins and stored when it
// ends.
//
// Two kernels.  A few rows a sequence (decode): a thread owns one channel of
// one sequence and walks the step's rows in order.  Many rows (prompts): the
// recurrence is linear, S_t = a_t S_(t-1) + b_t, so a stretch of rows folds into
// one pair (P, B) with S_end = P S_begin + B; a block owns 8 channels of a
// sequence and takes 128 rows at a time, 32 groups of threads with 4 rows each:
// every thread loads its rows, does all the gates' arithmetic and folds its 4
// rows (keeping each row's own pair), the groups' pairs meet in shared memory,
// every thread folds the groups before it onto the carried S, and then writes
// its rows' outputs.  The loads and the exponentials of 128 rows run side by
// side, the next tile's loads are already under way, and only 32 multiply-adds
// a tile are in sequence.  Both kernels compute the same function, rounded
// differently.
#include "common.cuh"

namespace {

using namespace rfx;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
// For results that are rounded to bfloat16 anyway (the serving path): the fast
// exponential, division and hyperbolic tangent, a few units in the last place of
// 32 bits (the tangent 2^-11) off, far below that rounding.  The 32-bit path keeps
// the exact forms.
template <typename TO> __device__ __forceinline__ float sigmoid_for(float z) {
    if constexpr (sizeof(TO) == 2) return __fdividef(1.0f, 1.0f + __expf(-z));
    else return sigmoid_f(z);
}
template <typename TO> __device__ __forceinline__ float exp_for(float z) {
    if constexpr (sizeof(TO) == 2) return __expf(z);
    else return expf(z);
}
template <typename TO> __device__ __forceinline__ float gelu_tanh_for(float z) {
    if constexpr (sizeof(TO) == 2) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        return 0.5f * z * (1.0f + t);
    } else {
        return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    }
}
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The convolution before the recurrence keeps its last taps - 1 inputs (columns
// x_off.. of proj, plus x_bias) beside S, [taps - 1][W] at `tail`, oldest first.
// That convolution ran in the launch before this one, so this kernel may bring
// them up to date: place i takes the input at local time n - T + i, one of the
// step's rows or what the state held n places later (read before it is written:
// a thread owns its channel and goes through i upwards).
__device__ __forceinline__ void update_tail(const float* __restrict__ proj, int ld, int x_off,
                                            const float* __restrict__ x_bias, int taps, float* __restrict__ tail,
                                            int W, int c, int row0, int n) {
    const int T = taps - 1;
    if (T <= 0 || x_off < 0) return;
    const float b = x_bias ? x_bias[c] : 0.0f;
    for (int i = 0; i < T; ++i) {
        const int src = n - T + i;
        tail[(size_t)i * W + c] = src >= 0 ? proj[(size_t)(row0 + src) * ld + x_off + c] + b
                                           : tail[(size_t)(n + i) * W + c];
    }
}

// gates: [R][blocks][2 * K] (a block's r_pre, then its i_pre); channel c = b * K + k
template <typename TO>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const float* __restrict__ u, const float* __restrict__ gates,
                  const float* __restrict__ r_bias, const float* __restrict__ i_bias,
                  const float* __restrict__ lam, float decay_scale, const float* __restrict__ proj, int ld,
                  int y_off, const float* __restrict__ y_bias, float* __restrict__ state, size_t slot_stride,
                  size_t state_off, const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                  TO* __restrict__ out, int W, int K, int x_off, const float* __restrict__ x_bias, int taps,
                  size_t tail_off) {
    pdl_prologue();
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int row0 = seq_row0[s], n = seq_row0[s + 1] - row0;
    float* sp = state + (size_t)seq_slot[s] * slot_stride + state_off + c;
    const int b = c / K, k = c % K;
    const size_t g_r = (size_t)b * 2 * K + k, g_i = g_r + K;
    const float rb = r_bias ? r_bias[c] : 0.0f, ib = i_bias ? i_bias[c] : 0.0f;
    const float yb = y_bias ? y_bias[c] : 0.0f;
    const float rate = -decay_scale * softplus_f(lam[c]);
    float S = *sp;
#pragma unroll 4
    for (int t = 0; t < n; ++t) {
        const size_t row = (size_t)(row0 + t);
        const float uv = u[row * W + c];
        const float r = sigmoid_f(gates[row * 2 * W + g_r] + rb);
        const float i = sigmoid_f(gates[row * 2 * W + g_i] + ib);
        const float yv = gelu_tanh_f(proj[row * ld + y_off + c] + yb);
        const float log_a = rate * r;
        const float a = expf(log_a);
        const float step = sqrtf(-expm1f(2.0f * log_a));
        S = fmaf(a, S, step * (i * uv));
        st<TO>(out, row * W + c, S * yv);
    }
    *sp = S;
    update_tail(proj, ld, x_off, x_bias, taps, state + (size_t)seq_slot[s] * slot_stride + tail_off, W, c, row0, n);
}

constexpr int CH_CHANNELS = 8, CH_GROUPS = 32, CH_ROWS = 4;  // 128 rows a tile

struct RowIn {
    float u, r, i, y;
};

template <typename TO>
__global__ void __launch_bounds__(CH_CHANNELS * CH_GROUPS)
rglru_chunk_kernel(const float* __restrict__ u, const float* __restrict__ gates,
                   const float* __restrict__ r_bias, const float* __restrict__ i_bias,
                   const float* __restrict__ lam, float decay_scale, const float* __restrict__ proj, int ld,
                   int y_off, const float* __restrict__ y_bias, float* __restrict__ state, size_t slot_stride,
                   size_t state_off, const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                   TO* __restrict__ out, int W, int K, int x_off, const float* __restrict__ x_bias, int taps,
                   size_t tail_off) {
    __shared__ float fold_p[CH_GROUPS][CH_CHANNELS], fold_b[CH_GROUPS][CH_CHANNELS];
    __shared__ float carry[2][CH_CHANNELS];
    pdl_prologue();
    const int s = blockIdx.x;
    const int cl = threadIdx.x % CH_CHANNELS, grp = threadIdx.x / CH_CHANNELS;
    const int c = blockIdx.y * CH_CHANNELS + cl;
    const bool live = c < W;
    const int cc = live ? c : W - 1;  // idle threads follow a real channel and store nothing
    const int row0 = seq_row0[s], n = seq_row0[s + 1] - row0;
    float* sp = state + (size_t)seq_slot[s] * slot_stride + state_off + cc;
    const int b = cc / K, k = cc % K;
    const size_t g_r = (size_t)b * 2 * K + k, g_i = g_r + K;
    const float rb = r_bias ? r_bias[cc] : 0.0f, ib = i_bias ? i_bias[cc] : 0.0f;
    const float yb = y_bias ? y_bias[cc] : 0.0f;
    const float rate = -decay_scale * softplus_f(lam[cc]);
    if (grp == 0) carry[0][cl] = *sp;
    int cur = 0;
    // a tile's loads are issued one tile ahead, so that they travel during the tile before
    auto fetch = [&](int tile, RowIn (&in)[CH_ROWS]) {
#pragma unroll
        for (int j = 0; j < CH_ROWS; ++j) {
            const int t = tile + grp * CH_ROWS + j;
            if (t < n) {
                const size_t row = (size_t)(row0 + t);
                in[j].u = u[row * W + cc];
                in[j].r = gates[row * 2 * W + g_r];
                in[j].i = gates[row * 2 * W + g_i];
                in[j].y = proj[row * ld + y_off + cc];
            }
        }
    };
    RowIn ahead[CH_ROWS];
    fetch(0, ahead);
    for (int tile = 0; tile < n; tile += CH_GROUPS * CH_ROWS) {
        RowIn in[CH_ROWS];
#pragma unroll
        for (int j = 0; j < CH_ROWS; ++j) in[j] = ahead[j];
        if (tile + CH_GROUPS * CH_ROWS < n) fetch(tile + CH_GROUPS * CH_ROWS, ahead);
        float P[CH_ROWS], B[CH_ROWS], Y[CH_ROWS];
        float p = 1.0f, acc = 0.0f;
#pragma unroll
        for (int j = 0; j < CH_ROWS; ++j) {
            const int t = tile + grp * CH_ROWS + j;
            if (t < n) {
                const float r = sigmoid_for<TO>(in[j].r + rb);
                const float i = sigmoid_for<TO>(in[j].i + ib);
                Y[j] = gelu_tanh_for<TO>(in[j].y + yb);
                const float log_a = rate * r;
                const float a = exp_for<TO>(log_a);
                acc = fmaf(a, acc, sqrtf(-expm1f(2.0f * log_a)) * (i * in[j].u));
                p *= a;
            } else {
                Y[j] = 0.0f;
            }
            P[j] = p;
            B[j] = acc;
        }
        fold_p[grp][cl] = p;
        fold_b[grp][cl] = acc;
        __syncthreads();
        float S = carry[cur][cl];
        for (int g2 = 0; g2 < grp; ++g2) S = fmaf(fold_p[g2][cl], S, fold_b[g2][cl]);
        if (live) {
#pragma unroll
            for (int j = 0; j < CH_ROWS; ++j) {
                const int t = tile + grp * CH_ROWS + j;
                if (t < n) st<TO>(out, (size_t)(row0 + t) * W + c, fmaf(P[j], S, B[j]) * Y[j]);
            }
        }
        // the last group's end is the tile's; the other buffer, so that no thread still reads this one
        if (grp == CH_GROUPS - 1) carry[cur ^ 1][cl] = fmaf(p, S, acc);
        cur ^= 1;
        __syncthreads();
    }
    if (live && grp == 0) {
        *sp = carry[cur][cl];
        update_tail(proj, ld, x_off, x_bias, taps, state + (size_t)seq_slot[s] * slot_stride + tail_off, W, c, row0, n);
    }
}

}  // namespace

// `chunked` != 0: the form for many rows a sequence (above).  `x_off` >= 0 and `taps` > 1:
// the kernel also brings the preceding convolution's last inputs up to date (columns
// x_off.. of proj plus x_bias, kept at `tail_off` of a slot's state).
extern "C" int rfx_rglru_scan(const float* u, const float* gates, const float* r_bias, const float* i_bias,
                              const float* lam, float decay_scale, const float* proj, int ld, int y_off,
                              const float* y_bias, float* state, long long slot_stride, long long state_off,
                              const int* seq_slot, const int* seq_row0, int S, void* out, int out_dt, int W,
                              int blocks, int chunked, int x_off, const float* x_bias, int taps,
                              long long tail_off, void* stream) {
    if (S <= 0 || W <= 0) return 0;
    if (blocks <= 0 || W % blocks != 0) return RFX_ERR_BAD_ARG;
    dim3 grid(S, (W + 127) / 128);
    cudaStream_t s = (cudaStream_t)stream;
    const int K = W / blocks;
    if (chunked) {
        dim3 cgrid(S, (W + CH_CHANNELS - 1) / CH_CHANNELS);
        if (cgrid.y > 65535) return RFX_ERR_UNSUPPORTED;
        if (out_dt == RFX_DT_F32)
            RFX_LAUNCH(rglru_chunk_kernel<float>, cgrid, CH_CHANNELS * CH_GROUPS, 0, s, u, gates, r_bias, i_bias,
                       lam, decay_scale, proj, ld, y_off, y_bias, state, (size_t)slot_stride, (size_t)state_off,
                       seq_slot, seq_row0, (float*)out, W, K, x_off, x_bias, taps, (size_t)tail_off);
        else if (out_dt == RFX_DT_BF16)
            RFX_LAUNCH(rglru_chunk_kernel<__nv_bfloat16>, cgrid, CH_CHANNELS * CH_GROUPS, 0, s, u, gates, r_bias,
                       i_bias, lam, decay_scale, proj, ld, y_off, y_bias, state, (size_t)slot_stride,
                       (size_t)state_off, seq_slot, seq_row0, (__nv_bfloat16*)out, W, K, x_off, x_bias, taps,
                       (size_t)tail_off);
        else
            return RFX_ERR_BAD_ARG;
        return 0;
    }
    if (out_dt == RFX_DT_F32)
        RFX_LAUNCH(rglru_scan_kernel<float>, grid, 128, 0, s, u, gates, r_bias, i_bias, lam, decay_scale, proj,
                   ld, y_off, y_bias, state, (size_t)slot_stride, (size_t)state_off, seq_slot, seq_row0,
                   (float*)out, W, K, x_off, x_bias, taps, (size_t)tail_off);
    else if (out_dt == RFX_DT_BF16)
        RFX_LAUNCH(rglru_scan_kernel<__nv_bfloat16>, grid, 128, 0, s, u, gates, r_bias, i_bias, lam,
                   decay_scale, proj, ld, y_off, y_bias, state, (size_t)slot_stride, (size_t)state_off,
                   seq_slot, seq_row0, (__nv_bfloat16*)out, W, K, x_off, x_bias, taps, (size_t)tail_off);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
