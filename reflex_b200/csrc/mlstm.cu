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

// The chunkwise form for many rows a sequence (prefill).  With F_t the sum of
// the log forget gates from the chunk's first row to t, g_s = i_s - F_s and
// M_t = max(m_prev, max_{s<=t} g_s), the walk above gives m_t = F_t + M_t and
//   S_t^T q_t = e^(m_prev - M_t) S_prev^T q_t + sum_{s<=t} e^(g_s - M_t) (q_t . k_s) v_s
//   S_L = e^(m_prev - M_L) S_prev + sum_s e^(g_s - M_L) k_s v_s^T
// (every exponent is <= 0), and the same for n with v = 1.  A block owns
// (sequence, head, 64 value columns) and takes 32 rows at a time: the gates'
// sums and maxima by one warp's shuffles, then three small 32-bit products in
// registers over shared-memory tiles (the rows' scores, the read-out, the
// state's update).  dim <= 16 RD.  The rows' q, k, v and gate pre-activations
// arrive by 4-byte asynchronous copies, with NB = 2 a chunk ahead of their use.
template <int RD, int NB>
__global__ void __launch_bounds__(256)
mlstm_chunk_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int i_off,
                   int f_off, const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                   float q_scale, const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                   float* __restrict__ state, float* __restrict__ num, float* __restrict__ den, int heads,
                   int dim, int vdim) {
    constexpr int L = 32, DMAX = 16 * RD, DP = DMAX + 4, VP = VT + 4, LP = L + 1;
    extern __shared__ __align__(16) float smem[];
    constexpr int TILE = 2 * L * DP + L * VP + 2 * L;  // q, k, v and the two gates of a chunk
    float* Ss = smem + NB * TILE;   // [DMAX][VP]
    float* ns = Ss + DMAX * VP;     // [DMAX]
    float* Ps = ns + DMAX;          // [L][LP]
    float* Fs = Ps + L * LP;        // [L] each: F, g, M, e^(m_prev - M), e^(g - M_L)
    float* gs = Fs + L;
    float* Ms = gs + L;
    float* dec = Ms + L;
    float* wl = dec + L;
    float* two = wl + L;            // e^(m_prev - M_L), m_L
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int j0 = blockIdx.z * VT;
    const int nv = min(VT, vdim - j0);
    const bool has_n = blockIdx.z == 0;
    const int tid = threadIdx.x, lane = tid & 31;
    const int cg = tid & 15, rp = tid >> 4;
    const int slot = seq_slot[seq];
    const int row0 = seq_row0[seq], n_rows = seq_row0[seq + 1] - row0;
    const size_t per_head = (size_t)dim * vdim + dim + gridDim.z;
    float* st_h = state + ((size_t)slot * heads + h) * per_head;
    const float bi = bias_i[h], bf = bias_f[h];

    for (int e = tid; e < NB * TILE; e += 256) smem[e] = 0.0f;  // what no copy writes stays zero
    for (int e = tid; e < DMAX * VT; e += 256) {
        const int d = e / VT, j = e % VT;
        Ss[d * VP + j] = (d < dim && j < nv) ? st_h[(size_t)d * vdim + j0 + j] : 0.0f;
    }
    __syncthreads();
    auto issue = [&](int buf, int t0) {
        float* base = smem + buf * TILE;
        const int nt = min(L, n_rows - t0);
        for (int e = tid; e < nt * dim; e += 256) {
            const int t = e / dim, d = e % dim;
            const float* row = proj + (size_t)(row0 + t0 + t) * ld;
            cp_async4(base + t * DP + d, row + q_off + h * dim + d);
            cp_async4(base + L * DP + t * DP + d, row + k_off + h * dim + d);
        }
        for (int e = tid; e < nt * nv; e += 256) {
            const int t = e / nv, j = e % nv;
            cp_async4(base + 2 * L * DP + t * VP + j, proj + (size_t)(row0 + t0 + t) * ld + v_off + h * vdim + j0 + j);
        }
        for (int t = tid; t < nt; t += 256) {
            const float* row = proj + (size_t)(row0 + t0 + t) * ld;
            cp_async4(base + 2 * L * DP + L * VP + t, row + i_off + h);
            cp_async4(base + 2 * L * DP + L * VP + L + t, row + f_off + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (NB == 2 && n_rows > 0) issue(0, 0);
    for (int d = tid; d < DMAX; d += 256) ns[d] = d < dim ? st_h[(size_t)dim * vdim + d] : 0.0f;
    float m_prev = st_h[(size_t)dim * vdim + dim + blockIdx.z];

    for (int t0 = 0, buf = 0; t0 < n_rows; t0 += L, buf = (buf + 1) % NB) {
        const int nt = min(L, n_rows - t0);
        __syncthreads();  // the chunk before is done with the tiles
        if (NB == 2) {
            if (t0 + L < n_rows) {
                issue(buf ^ 1, t0 + L);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        } else {
            issue(0, t0);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        // rows beyond the chunk's may hold an earlier chunk's values: nothing below reads
        // them into a result (their weights are zero, their scores masked, their sums not stored)
        const float* Qs = smem + buf * TILE;  // [L][DP], unscaled: the results take q's scale
        const float* Ks = Qs + L * DP;        // [L][DP]
        const float* Vs = Ks + L * DP;        // [L][VP]
        const float* raw = Vs + L * VP;       // [2][L]
        if (tid < L) {  // one warp: the gates, their running sum and running maximum
            float gi = -INFINITY, F = 0.0f;
            if (lane < nt) {
                gi = cap * tanhf((raw[lane] + bi) / cap);
                F = log_sigmoid(cap * tanhf((raw[L + lane] + bf) / cap));
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xffffffffu, F, o);
                if (lane >= o) F += v;
            }
            const float g = gi - F;  // -inf beyond the chunk's rows
            float M = fmaxf(g, m_prev);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xffffffffu, M, o);
                if (lane >= o) M = fmaxf(M, v);
            }
            const float ML = __shfl_sync(0xffffffffu, M, nt - 1), FL = __shfl_sync(0xffffffffu, F, nt - 1);
            Fs[lane] = F;
            gs[lane] = g;
            Ms[lane] = M;
            dec[lane] = expf(m_prev - M);
            wl[lane] = expf(g - ML);
            if (lane == 0) {
                two[0] = expf(m_prev - ML);
                two[1] = FL + ML;
            }
        }
        __syncthreads();
        {   // scores of row t against rows s <= t, times their weights
            const int t = tid >> 3, si = tid & 7;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const float4* q4 = reinterpret_cast<const float4*>(Qs + t * DP);
#pragma unroll 4
            for (int d4 = 0; d4 < DMAX / 4; ++d4) {
                const float4 q = q4[d4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 k = reinterpret_cast<const float4*>(Ks + (si + 8 * j) * DP)[d4];
                    acc[j] = fmaf(q.x, k.x, acc[j]);
                    acc[j] = fmaf(q.y, k.y, acc[j]);
                    acc[j] = fmaf(q.z, k.z, acc[j]);
                    acc[j] = fmaf(q.w, k.w, acc[j]);
                }
            }
            const float Mt = Ms[t];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int sidx = si + 8 * j;
                Ps[t * LP + sidx] = sidx <= t ? acc[j] * expf(gs[sidx] - Mt) : 0.0f;
            }
        }
        __syncthreads();
        {   // read-out: rows 2 rp and 2 rp + 1, columns 4 cg .. 4 cg + 3
            float acc[2][4];
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] = 0.0f;
            const float4* qa = reinterpret_cast<const float4*>(Qs + (2 * rp) * DP);
            const float4* qb = reinterpret_cast<const float4*>(Qs + (2 * rp + 1) * DP);
#pragma unroll 2
            for (int d4 = 0; d4 < DMAX / 4; ++d4) {
                const float4 a = qa[d4], b = qb[d4];
                const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 sv = *reinterpret_cast<const float4*>(Ss + (4 * d4 + i) * VP + 4 * cg);
                    acc[0][0] = fmaf(av[i], sv.x, acc[0][0]);
                    acc[0][1] = fmaf(av[i], sv.y, acc[0][1]);
                    acc[0][2] = fmaf(av[i], sv.z, acc[0][2]);
                    acc[0][3] = fmaf(av[i], sv.w, acc[0][3]);
                    acc[1][0] = fmaf(bv[i], sv.x, acc[1][0]);
                    acc[1][1] = fmaf(bv[i], sv.y, acc[1][1]);
                    acc[1][2] = fmaf(bv[i], sv.z, acc[1][2]);
                    acc[1][3] = fmaf(bv[i], sv.w, acc[1][3]);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float dt = dec[2 * rp + r];
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] *= dt;
            }
            for (int sidx = 0; sidx <= 2 * rp + 1; ++sidx) {
                const float4 v = *reinterpret_cast<const float4*>(Vs + sidx * VP + 4 * cg);
                const float pa = Ps[(2 * rp) * LP + sidx], pb = Ps[(2 * rp + 1) * LP + sidx];
                acc[0][0] = fmaf(pa, v.x, acc[0][0]);
                acc[0][1] = fmaf(pa, v.y, acc[0][1]);
                acc[0][2] = fmaf(pa, v.z, acc[0][2]);
                acc[0][3] = fmaf(pa, v.w, acc[0][3]);
                acc[1][0] = fmaf(pb, v.x, acc[1][0]);
                acc[1][1] = fmaf(pb, v.y, acc[1][1]);
                acc[1][2] = fmaf(pb, v.z, acc[1][2]);
                acc[1][3] = fmaf(pb, v.w, acc[1][3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int t = 2 * rp + r;
                if (t < nt) {
                    float* dst = num + ((size_t)(row0 + t0 + t) * heads + h) * vdim + j0 + 4 * cg;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (4 * cg + c < nv) dst[c] = acc[r][c] * q_scale;
                }
            }
        }
        if (has_n) {  // n . q: eight lanes a row
            const int t = tid >> 3, l8 = tid & 7;
            float qn = 0.0f, ps = 0.0f;
            for (int d = l8; d < DMAX; d += 8) qn = fmaf(Qs[t * DP + d], ns[d], qn);
            for (int sidx = l8; sidx < L; sidx += 8) ps += Ps[t * LP + sidx];
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                qn += __shfl_xor_sync(0xffffffffu, qn, o);
                ps += __shfl_xor_sync(0xffffffffu, ps, o);
            }
            if (l8 == 0 && t < nt)
                den[(size_t)(row0 + t0 + t) * heads + h] =
                    fmaxf(fabsf(fmaf(dec[t], qn, ps) * q_scale), expf(-(Fs[t] + Ms[t]))) + 1e-6f;
        }
        __syncthreads();  // every read of S and n is done
        {   // the state: rows rp RD .. + RD - 1 of S, columns 4 cg .. + 3
            const float dl = two[0];
            float acc[RD][4];
#pragma unroll
            for (int i = 0; i < RD; ++i) {
                const float4 sv = *reinterpret_cast<const float4*>(Ss + (rp * RD + i) * VP + 4 * cg);
                acc[i][0] = dl * sv.x;
                acc[i][1] = dl * sv.y;
                acc[i][2] = dl * sv.z;
                acc[i][3] = dl * sv.w;
            }
            for (int sidx = 0; sidx < nt; ++sidx) {
                const float w = wl[sidx];
                float4 v = *reinterpret_cast<const float4*>(Vs + sidx * VP + 4 * cg);
                v.x *= w;
                v.y *= w;
                v.z *= w;
                v.w *= w;
                const float4* k4 = reinterpret_cast<const float4*>(Ks + sidx * DP + rp * RD);
#pragma unroll
                for (int i4 = 0; i4 < RD / 4; ++i4) {
                    const float4 k = k4[i4];
                    const float kv[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[4 * i4 + i][0] = fmaf(kv[i], v.x, acc[4 * i4 + i][0]);
                        acc[4 * i4 + i][1] = fmaf(kv[i], v.y, acc[4 * i4 + i][1]);
                        acc[4 * i4 + i][2] = fmaf(kv[i], v.z, acc[4 * i4 + i][2]);
                        acc[4 * i4 + i][3] = fmaf(kv[i], v.w, acc[4 * i4 + i][3]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < RD; ++i)
                *reinterpret_cast<float4*>(Ss + (rp * RD + i) * VP + 4 * cg) =
                    make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            for (int d = tid; d < DMAX; d += 256) {
                float a = dl * ns[d];
                for (int sidx = 0; sidx < nt; ++sidx) a = fmaf(wl[sidx], Ks[sidx * DP + d], a);
                ns[d] = a;
            }
            m_prev = two[1];
        }
    }
    __syncthreads();
    for (int e = tid; e < dim * nv; e += 256) {
        const int d = e / nv, j = e % nv;
        st_h[(size_t)d * vdim + j0 + j] = Ss[d * VP + j];
    }
    if (has_n)
        for (int d = tid; d < dim; d += 256) st_h[(size_t)dim * vdim + d] = ns[d];
    if (tid == 0) st_h[(size_t)dim * vdim + dim + blockIdx.z] = m_prev;
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

// The chunkwise form (many rows a sequence); RFX_ERR_UNSUPPORTED beyond dim 256.
extern "C" int rfx_mlstm_chunk(const float* proj, int ld, int q_off, int k_off, int v_off, int i_off,
                               int f_off, const float* bias_i, const float* bias_f, float cap,
                               float q_scale, const int* seq_slot, const int* seq_row0, int S,
                               float* state, float* num, float* den, int heads, int dim, int vdim,
                               void* stream) {
    if (S <= 0) return 0;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || cap <= 0.0f) return RFX_ERR_BAD_ARG;
    if (dim > 256) return RFX_ERR_UNSUPPORTED;
    dim3 grid(S, heads, (vdim + VT - 1) / VT);
    if (grid.y > 65535 || grid.z > 65535) return RFX_ERR_UNSUPPORTED;
#define RFX_CHUNK(RD, NB)                                                                                   \
    do {                                                                                                    \
        constexpr int L = 32, DMAX = 16 * RD, DP = DMAX + 4, VP = VT + 4, LP = L + 1;                       \
        const size_t sm = ((size_t)NB * (2 * L * DP + L * VP + 2 * L) + DMAX * VP + DMAX + L * LP + 5 * L + 2) * \
                          sizeof(float);                                                                    \
        cudaError_t e = cudaFuncSetAttribute((mlstm_chunk_kernel<RD, NB>),                                  \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);         \
        if (e != cudaSuccess) return (int)e;                                                                \
        RFX_LAUNCH((mlstm_chunk_kernel<RD, NB>), grid, 256, sm, (cudaStream_t)stream, proj, ld, q_off, k_off, \
                   v_off, i_off, f_off, bias_i, bias_f, cap, q_scale, seq_slot, seq_row0, state, num, den,  \
                   heads, dim, vdim);                                                                       \
        return 0;                                                                                           \
    } while (0)
    if (dim <= 64) RFX_CHUNK(4, 2);
    if (dim <= 128) RFX_CHUNK(8, 2);
    RFX_CHUNK(16, 1);  // two chunks of 256-wide rows beside the state do not fit shared memory
#undef RFX_CHUNK
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
