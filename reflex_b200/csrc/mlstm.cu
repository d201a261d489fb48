// The mLSTM matrix memory: the recurrence over a step's rows, sequence by
// sequence, and what follows it.
//
// Per head, with log gates i_t and f_t and a running maximum m (m_0 = 0):
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = e^(f_t + m_{t-1} - m_t) S_{t-1} + e^(i_t - m_t) k_t v_t^T          [dim, vdim]
//   n_t = e^(f_t + m_{t-1} - m_t) n_{t-1} + e^(i_t - m_t) k_t                [dim]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
// where i_t = cap tanh(a_t / cap) and f_t = logsigmoid(cap tanh(b_t / cap)) for
// the gate pre-activations a_t, b_t (projection plus bias).  Everything here is
// 32-bit.  (S, n, m) is a sequence's state: [heads][dim * vdim + dim + slices]
// floats per slot (every slice of vdim columns, a block each, keeps its own copy
// of m, so no block reads what another writes), zero at a sequence's start,
// carried from step to step.
//
//  * rfx_mlstm_scan: a block owns (sequence, head, a slice of vdim columns): a
//    thread holds one column of S in shared memory and walks the sequence's
//    rows in order; n is one more column whose v is 1, so n . q falls out of
//    the same loop.  Rows are staged in tiles, so the block synchronises once
//    a tile, not once a row.  It writes the numerators S^T q and the
//    denominators.  Up to dim 256 the memory lies in registers.
//  * rfx_mlstm_out: o = numerator / denominator, each head's o divided by its
//    root mean square, times the norm weight, times sigmoid(gate).
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int VT = 64;   // columns of S a block owns
constexpr int TT = 16;   // rows staged at a time

constexpr int RT = 32;   // rows of a staged tile in the register kernel (two tiles take turns)

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(src)
                 : "memory");
}

__device__ __forceinline__ float log_sigmoid(float z) {
    return fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
}

// proj [R, ld]: columns q_off.. (heads * dim), k_off.. (heads * dim), v_off..
// (heads * vdim), i_off.. (heads), f_off.. (heads).
__global__ void mlstm_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                                  int i_off, int f_off, const float* __restrict__ bias_i,
                                  const float* __restrict__ bias_f, float cap, float q_scale,
                                  const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                                  float* __restrict__ state, float* __restrict__ num,
                                  float* __restrict__ den, int heads, int dim, int vdim) {
    extern __shared__ __align__(16) float smem[];
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int j0 = blockIdx.z * VT;
    const int nv = min(VT, vdim - j0);          // value columns of this block
    const bool has_n = blockIdx.z == 0;         // the block that also carries n (and stores m)
    const int ncol = nv + (has_n ? 1 : 0);
    const int W = VT + 1;                       // row length of the S tile
    float* S = smem;                            // [dim][W]
    float* qs = S + (size_t)dim * W;            // [TT][dim]
    float* ks = qs + TT * dim;                  // [TT][dim]
    float* vs = ks + TT * dim;                  // [TT][W]   (column nv of the n block: 1)
    float* gi = vs + TT * W;                    // [TT]
    float* gf = gi + TT;                        // [TT]
    const int tid = threadIdx.x;
    const int slot = seq_slot[seq];
    const int row0 = seq_row0[seq], n_rows = seq_row0[seq + 1] - row0;
    const size_t per_head = (size_t)dim * vdim + dim + gridDim.z;
    float* st_h = state + ((size_t)slot * heads + h) * per_head;

    for (int e = tid; e < dim * ncol; e += blockDim.x) {
        const int d = e / ncol, j = e % ncol;
        S[d * W + j] = j < nv ? st_h[(size_t)d * vdim + j0 + j] : st_h[(size_t)dim * vdim + d];
    }
    float m = st_h[(size_t)dim * vdim + dim + blockIdx.z];

    for (int t0 = 0; t0 < n_rows; t0 += TT) {
        const int nt = min(TT, n_rows - t0);
        __syncthreads();  // the tile before is done with; S is loaded
        for (int e = tid; e < nt * dim; e += blockDim.x) {
            const int t = e / dim, d = e % dim;
            const float* row = proj + (size_t)(row0 + t0 + t) * ld;
            qs[t * dim + d] = row[q_off + h * dim + d] * q_scale;
            ks[t * dim + d] = row[k_off + h * dim + d];
        }
        for (int e = tid; e < nt * ncol; e += blockDim.x) {
            const int t = e / ncol, j = e % ncol;
            vs[t * W + j] = j < nv ? proj[(size_t)(row0 + t0 + t) * ld + v_off + h * vdim + j0 + j] : 1.0f;
        }
        for (int t = tid; t < nt; t += blockDim.x) {
            const float* row = proj + (size_t)(row0 + t0 + t) * ld;
            const float a = row[i_off + h] + bias_i[h], b = row[f_off + h] + bias_f[h];
            gi[t] = cap * tanhf(a / cap);
            gf[t] = log_sigmoid(cap * tanhf(b / cap));
        }
        __syncthreads();
        if (tid < ncol) {
            for (int t = 0; t < nt; ++t) {
                const float fm = gf[t] + m;
                const float m_new = fmaxf(fm, gi[t]);
                const float a = expf(fm - m_new), b = expf(gi[t] - m_new);
                m = m_new;
                const float bv = b * vs[t * W + tid];
                const float* kt = ks + t * dim;
                const float* qt = qs + t * dim;
                float acc = 0.0f;
                for (int d = 0; d < dim; ++d) {
                    const float s = fmaf(a, S[d * W + tid], bv * kt[d]);
                    S[d * W + tid] = s;
                    acc = fmaf(s, qt[d], acc);
                }
                const size_t r = (size_t)(row0 + t0 + t);
                if (tid < nv) num[(r * heads + h) * vdim + j0 + tid] = acc;
                else den[r * heads + h] = fmaxf(fabsf(acc), expf(-m)) + 1e-6f;
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < dim * ncol; e += blockDim.x) {
        const int d = e / ncol, j = e % ncol;
        if (j < nv) st_h[(size_t)d * vdim + j0 + j] = S[d * W + j];
        else st_h[(size_t)dim * vdim + d] = S[d * W + j];
    }
    if (tid == 0) st_h[(size_t)dim * vdim + dim + blockIdx.z] = m;
}

// The same walk with S in registers: a column of S is shared by SPLIT
// neighbouring lanes, DPT elements each (dim <= DPT * SPLIT), so no element of S
// makes a trip through shared memory, k and q come four at a time, and the
// lanes' partial sums of S^T q meet in a butterfly.
template <int DPT, int SPLIT>
__global__ void __launch_bounds__(((VT + 1) * SPLIT + 31) / 32 * 32, 1)
mlstm_scan_reg_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int i_off,
                      int f_off, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                      float cap, float q_scale, const int* __restrict__ seq_slot,
                      const int* __restrict__ seq_row0, float* __restrict__ state, float* __restrict__ num,
                      float* __restrict__ den, int heads, int dim, int vdim) {
    constexpr int DMAX = DPT * SPLIT;
    extern __shared__ __align__(16) float smem[];
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int j0 = blockIdx.z * VT;
    const int nv = min(VT, vdim - j0);
    const bool has_n = blockIdx.z == 0;
    const int ncol = nv + (has_n ? 1 : 0);
    const int W = VT + 1;
    constexpr int TILE = 2 * RT * DMAX + RT * W + 2 * RT;  // floats of one staged tile of rows
    const int tid = threadIdx.x;
    // lane `part` of a column holds elements 4 (i SPLIT + part) .. + 3, i = 0 .. DPT / 4: the
    // lanes' 16-byte loads of k and q then fall side by side, in different banks
    const int col = tid / SPLIT, part = tid % SPLIT;
    const int slot = seq_slot[seq];
    const int row0 = seq_row0[seq], n_rows = seq_row0[seq + 1] - row0;
    const size_t per_head = (size_t)dim * vdim + dim + gridDim.z;
    float* st_h = state + ((size_t)slot * heads + h) * per_head;
    const bool mine = col < ncol;
    const bool is_n = mine && col >= nv;

    // Two tiles of rows take turns: while one is walked, the next one's q, k, v and
    // gate pre-activations arrive by 4-byte asynchronous copies.  What no copy
    // writes is set once: the padding of q and k beyond dim, and the 1 that the
    // n column has in place of a v.
    for (int e = tid; e < 2 * TILE; e += blockDim.x) smem[e] = 0.0f;
    __syncthreads();
    if (has_n)
        for (int e = tid; e < 2 * RT; e += blockDim.x) smem[(e / RT) * TILE + 2 * RT * DMAX + (e % RT) * W + nv] = 1.0f;
    auto issue = [&](int buf, int t0) {
        float* base = smem + buf * TILE;
        const int nt = min(RT, n_rows - t0);
        for (int e = tid; e < nt * dim; e += blockDim.x) {
            const int t = e / dim, d = e % dim;
            const float* row = proj + (size_t)(row0 + t0 + t) * ld;
            cp_async4(base + t * DMAX + d, row + q_off + h * dim + d);
            cp_async4(base + RT * DMAX + t * DMAX + d, row + k_off + h * dim + d);
        }
        for (int e = tid; e < nt * nv; e += blockDim.x) {
            const int t = e / nv, j = e % nv;
            cp_async4(base + 2 * RT * DMAX + t * W + j, proj + (size_t)(row0 + t0 + t) * ld + v_off + h * vdim + j0 + j);
        }
        for (int t = tid; t < nt; t += blockDim.x) {
            const float* row = proj + (size_t)(row0 + t0 + t) * ld;
            cp_async4(base + 2 * RT * DMAX + RT * W + t, row + i_off + h);
            cp_async4(base + 2 * RT * DMAX + RT * W + RT + t, row + f_off + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = 4 * ((i / 4) * SPLIT + part) + (i % 4);
        S[i] = (mine && d < dim) ? (is_n ? st_h[(size_t)dim * vdim + d] : st_h[(size_t)d * vdim + j0 + col]) : 0.0f;
    }
    float m = st_h[(size_t)dim * vdim + dim + blockIdx.z];
    const float bi = bias_i[h], bf = bias_f[h];

    if (n_rows > 0) issue(0, 0);
    for (int t0 = 0, buf = 0; t0 < n_rows; t0 += RT, buf ^= 1) {
        const int nt = min(RT, n_rows - t0);
        if (t0 + RT < n_rows) {
            issue(buf ^ 1, t0 + RT);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float* qs = smem + buf * TILE;    // [RT][DMAX]
        float* ks = qs + RT * DMAX;       // [RT][DMAX]
        float* vs = ks + RT * DMAX;       // [RT][W]
        float* gi = vs + RT * W;          // [RT]
        float* gf = gi + RT;              // [RT]
        for (int t = tid; t < nt; t += blockDim.x) {
            gi[t] = cap * tanhf((gi[t] + bi) / cap);
            gf[t] = log_sigmoid(cap * tanhf((gf[t] + bf) / cap));
        }
        __syncthreads();
        // every lane walks (lanes without a column carry zeros): the butterfly needs the whole warp
#pragma unroll 1
        for (int t = 0; t < nt; ++t) {
            const float fm = gf[t] + m;
            const float m_new = fmaxf(fm, gi[t]);
            const float a = expf(fm - m_new), b = expf(gi[t] - m_new);
            m = m_new;
            const float bv = mine ? b * vs[t * W + col] : 0.0f;
            const float4* kt = reinterpret_cast<const float4*>(ks + t * DMAX) + part;
            const float4* qt = reinterpret_cast<const float4*>(qs + t * DMAX) + part;
            float acc = 0.0f;
#pragma unroll
            for (int i4 = 0; i4 < DPT / 4; ++i4) {
                const float4 k4 = kt[i4 * SPLIT], q4 = qt[i4 * SPLIT];
                S[4 * i4] = fmaf(a, S[4 * i4], bv * k4.x);
                S[4 * i4 + 1] = fmaf(a, S[4 * i4 + 1], bv * k4.y);
                S[4 * i4 + 2] = fmaf(a, S[4 * i4 + 2], bv * k4.z);
                S[4 * i4 + 3] = fmaf(a, S[4 * i4 + 3], bv * k4.w);
                acc = fmaf(S[4 * i4], q4.x, acc);
                acc = fmaf(S[4 * i4 + 1], q4.y, acc);
                acc = fmaf(S[4 * i4 + 2], q4.z, acc);
                acc = fmaf(S[4 * i4 + 3], q4.w, acc);
            }
#pragma unroll
            for (int o = 1; o < SPLIT; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            acc *= q_scale;  // q is staged unscaled
            if (mine && part == 0) {
                const size_t r = (size_t)(row0 + t0 + t);
                if (!is_n) num[(r * heads + h) * vdim + j0 + col] = acc;
                else den[r * heads + h] = fmaxf(fabsf(acc), expf(-m)) + 1e-6f;
            }
        }
        __syncthreads();  // this tile's buffer is the target of the copies issued next
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = 4 * ((i / 4) * SPLIT + part) + (i % 4);
            if (d < dim) {
                if (is_n) st_h[(size_t)dim * vdim + d] = S[i];
                else st_h[(size_t)d * vdim + j0 + col] = S[i];
            }
        }
    }
    if (tid == 0) st_h[(size_t)dim * vdim + dim + blockIdx.z] = m;
}

// One warp per (row, head).
template <typename TO>
__global__ void mlstm_out_kernel(const float* __restrict__ num, const float* __restrict__ den,
                                 const float* __restrict__ proj, int ld, int g_off,
                                 const float* __restrict__ w, float eps, TO* __restrict__ out, int R,
                                 int heads, int vdim) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= R * heads) return;
    const int r = pair / heads, h = pair % heads;
    const float inv = 1.0f / den[pair];
    const float* nrow = num + (size_t)pair * vdim;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) {
        const float o = nrow[j] * inv;
        ss = fmaf(o, o, ss);
    }
    const float rr = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    const float* g = proj + (size_t)r * ld + g_off + h * vdim;
    for (int j = lane; j < vdim; j += 32) {
        const float o = nrow[j] * inv;
        const float gate = 1.0f / (1.0f + expf(-g[j]));
        st<TO>(out, (size_t)pair * vdim + j, ((o * rr) * w[h * vdim + j]) * gate);
    }
}

}  // namespace

// Floats of state per head and slot.
extern "C" int rfx_mlstm_state_floats(int dim, int vdim) { return dim * vdim + dim + (vdim + VT - 1) / VT; }

extern "C" int rfx_mlstm_scan(const float* proj, int ld, int q_off, int k_off, int v_off, int i_off,
                              int f_off, const float* bias_i, const float* bias_f, float cap,
                              float q_scale, const int* seq_slot, const int* seq_row0, int S,
                              float* state, float* num, float* den, int heads, int dim, int vdim,
                              void* stream) {
    if (S <= 0) return 0;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || cap <= 0.0f) return RFX_ERR_BAD_ARG;
    const int W = VT + 1;
    const size_t smem = ((size_t)dim * W + 2 * TT * dim + TT * W + 2 * TT) * sizeof(float);
    if (smem > 220 * 1024) return RFX_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(S, heads, (vdim + VT - 1) / VT);
    if (grid.y > 65535 || grid.z > 65535) return RFX_ERR_UNSUPPORTED;
    const int cols = (vdim < VT ? vdim : VT) + 1;
    const int threads = (cols + 31) / 32 * 32;
#define RFX_REG(DPT, SPLIT)                                                                                \
    do {                                                                                                   \
        const size_t sm = (size_t)2 * (2 * RT * DPT * SPLIT + RT * W + 2 * RT) * sizeof(float);            \
        const int th = (cols * SPLIT + 31) / 32 * 32;                                                      \
        if (sm > 48 * 1024) {                                                                              \
            cudaError_t e2 = cudaFuncSetAttribute(mlstm_scan_reg_kernel<DPT, SPLIT>,                       \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);   \
            if (e2 != cudaSuccess) return (int)e2;                                                         \
        }                                                                                                  \
        RFX_LAUNCH((mlstm_scan_reg_kernel<DPT, SPLIT>), grid, th, sm, (cudaStream_t)stream, proj, ld,      \
                   q_off, k_off, v_off, i_off, f_off, bias_i, bias_f, cap, q_scale, seq_slot, seq_row0,    \
                   state, num, den, heads, dim, vdim);                                                     \
        return 0;                                                                                          \
    } while (0)
    if (dim <= 32) RFX_REG(32, 1);
    if (dim <= 64) RFX_REG(32, 2);
    if (dim <= 128) RFX_REG(32, 4);
    if (dim <= 256) RFX_REG(64, 4);
#undef RFX_REG
    RFX_LAUNCH(mlstm_scan_kernel, grid, threads, smem, (cudaStream_t)stream, proj, ld, q_off, k_off, v_off,
               i_off, f_off, bias_i, bias_f, cap, q_scale, seq_slot, seq_row0, state, num, den, heads, dim,
               vdim);
    return 0;
}

extern "C" int rfx_mlstm_out(const float* num, const float* den, const float* proj, int ld, int g_off,
                             const float* w, float eps, void* out, int out_dt, int R, int heads, int vdim,
                             void* stream) {
    if (R <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (R * heads + 3) / 4;
    if (out_dt == RFX_DT_F32)
        RFX_LAUNCH(mlstm_out_kernel<float>, blocks, 128, 0, s, num, den, proj, ld, g_off, w, eps,
                   (float*)out, R, heads, vdim);
    else if (out_dt == RFX_DT_BF16)
        RFX_LAUNCH(mlstm_out_kernel<__nv_bfloat16>, blocks, 128, 0, s, num, den, proj, ld, g_off, w, eps,
                   (__nv_bfloat16*)out, R, heads, vdim);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
