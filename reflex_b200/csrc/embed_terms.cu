// Terms added to the token embedding: a hashed bigram row and a sinusoidal
// position vector.  Both add into the 32-bit residual stream in place.
#include "common.cuh"

namespace {

using namespace rfx;

// hidden[r] += table[row(r)],  row = (prev * mul_prev + token * mul_cur) mod buckets,
// and row = buckets (the table's extra last row) at a sequence's first position.
// The previous token of a step's first row comes from the sequence's state word
// `prev_state[slot]`; the step's last token of every sequence is stored there.
// The block of a sequence's first row does both, the read before the write, so
// the launch needs no second pass; every other row takes the token of the row
// before it.  A step's rows of one sequence follow one another, and
// `seq_row0` [S + 1] gives each sequence's first row.
template <typename T>
__global__ void bigram_add_kernel(float* __restrict__ hidden, const T* __restrict__ table,
                                  const int* __restrict__ tokens, const int* __restrict__ row_pos,
                                  const int* __restrict__ row_slot, const int* __restrict__ seq_row0,
                                  int S, int* __restrict__ prev_state, int H, int buckets,
                                  long long mul_prev, long long mul_cur, int vocab) {
    __shared__ int s_row;
    pdl_prologue();
    const int r = blockIdx.x;
    if (threadIdx.x == 0) {
        const int slot = row_slot[r], tok = tokens[r];
        int prev;
        if (r > 0 && row_slot[r - 1] == slot) {
            prev = tokens[r - 1];
        } else {
            prev = prev_state[slot];
            int lo = 0, hi = S - 1;  // the sequence s with seq_row0[s] == r
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (seq_row0[mid] <= r) lo = mid;
                else hi = mid - 1;
            }
            prev_state[slot] = tokens[seq_row0[lo + 1] - 1];
        }
        int row = buckets;  // a sequence's first position: the extra row, whatever the state holds
        if (row_pos[r] != 0) {
            long long v = ((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets;
            if (v < 0) v += buckets;
            row = (prev < 0 || prev >= vocab) ? -1 : (int)v;
        }
        if (tok < 0 || tok >= vocab) row = -1;  // an id outside the vocabulary: the embedding reports it
        s_row = row;
    }
    __syncthreads();
    const int row = s_row;
    if (row < 0) return;
    const T* src = table + (size_t)row * H;
    float* dst = hidden + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] += ld<T>(src, c);
}

// hidden[r, 2i] += sin(p f_i), hidden[r, 2i + 1] += cos(p f_i), f_i = inv_freq[i]
// (base^(-2i / H), made on the host in double precision).  The angle and its
// sine and cosine are taken in double precision, so that the 32-bit sum sees
// correctly rounded terms at every position.
__global__ void sinusoid_add_kernel(float* __restrict__ hidden, const int* __restrict__ row_pos,
                                    const double* __restrict__ inv_freq, int H) {
    pdl_prologue();
    const int r = blockIdx.x;
    const double p = (double)row_pos[r];
    float* dst = hidden + (size_t)r * H;
    for (int i = threadIdx.x; 2 * i < H; i += blockDim.x) {
        double sn, cs;
        sincos(p * inv_freq[i], &sn, &cs);
        dst[2 * i] += (float)sn;
        if (2 * i + 1 < H) dst[2 * i + 1] += (float)cs;
    }
}

}  // namespace

extern "C" int rfx_bigram_add(float* hidden, const void* table, int table_dt, const int* tokens,
                              const int* row_pos, const int* row_slot, const int* seq_row0, int S,
                              int* prev_state, int R, int H, int buckets, long long mul_prev,
                              long long mul_cur, int vocab, void* stream) {
    if (R <= 0) return 0;
    if (S <= 0 || buckets <= 0) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dt == RFX_DT_F32)
        RFX_LAUNCH(bigram_add_kernel<float>, R, threads, 0, s, hidden, (const float*)table, tokens, row_pos,
                   row_slot, seq_row0, S, prev_state, H, buckets, mul_prev, mul_cur, vocab);
    else if (table_dt == RFX_DT_BF16)
        RFX_LAUNCH(bigram_add_kernel<__nv_bfloat16>, R, threads, 0, s, hidden, (const __nv_bfloat16*)table,
                   tokens, row_pos, row_slot, seq_row0, S, prev_state, H, buckets, mul_prev, mul_cur, vocab);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_sinusoid_add(float* hidden, const int* row_pos, const double* inv_freq, int R, int H,
                                void* stream) {
    if (R <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    RFX_LAUNCH(sinusoid_add_kernel, R, 128, 0, s, hidden, row_pos, inv_freq, H);
    return 0;
}
