// A short causal convolution over time on every channel of a projection's rows, with the last taps - 1 input rows of
// every sequence kept as its state:
//
//     y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c],   j = 0 .. taps - 1,   u = 0 before the sequence's start
//
//   short_conv       : one thread per (token, channel) - or, for 2 to 4 taps and rows of 16-byte packets, per run of up to 16
//                      tokens and packet of channels, the last rows kept in registers; an input row before the step's first
//                      token comes from the state [slot][taps - 1][C] (float32; the oldest row first), zeros for a new sequence.
//                      The products are summed in 32-bit in ascending j whatever the step, so a token's output is the
//                      same bits however the sequence was cut.
//   short_conv_state : afterwards, one thread per (sequence, channel) moves the state on: the last taps - 1 rows of
//                      (old state, the step's rows).
//
// u has `row_in` values per row (the convolved channels are its first C), y is dense [N, C]; w float32 [taps, C] (tap
// by tap, so that neighbouring channels' weights are neighbours).
#include "common.cuh"

namespace {

// VEC channels a thread (16 bytes of a row where the sizes allow it, else one).
template <typename T, int VEC>
__global__ void short_conv_kernel(const T* __restrict__ u, int64_t row_in, const float* __restrict__ w, const float* __restrict__ state,
                                  int64_t slot_stride, const int* __restrict__ token_seq, const int* __restrict__ seq_start,
                                  const int* __restrict__ seq_slots, T* __restrict__ y, int C, int taps, int64_t n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = C / VEC;
    const int64_t total = n_tokens * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / per_row;
        const int c = (int)(i % per_row) * VEC;
        const int seq = token_seq[t];
        const int64_t first = seq_start[seq];                  // the step's first row of this sequence
        const float* st = state + (int64_t)seq_slots[seq] * slot_stride;
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int64_t src = t - (taps - 1) + j;
            float x[VEC];
            if (src >= first) {
                if constexpr (VEC == 1) {
                    x[0] = to_f32<T>(u[src * row_in + c]);
                } else {
                    const Pack<T> pk = load_pack<T>(u + src * row_in + c);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) x[k] = pk.get(k);
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] = st[(int64_t)(taps - 1 + (src - first)) * C + c + k];
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] = fmaf(w[(int64_t)j * C + c + k], x[k], acc[k]);
        }
        if constexpr (VEC == 1) {
            y[t * C + c] = from_f32<T>(acc[0]);
        } else {
            Pack<T> pk;
#pragma unroll
            for (int k = 0; k < VEC; ++k) pk.set(k, acc[k]);
            store_pack<T>(y + t * C + c, pk);
        }
    }
}

// The same for TAPS known at compile time and 16-byte packets: a thread walks `run` consecutive tokens of its VEC channels
// with the last TAPS - 1 rows in registers, so that every row is read once (and TAPS - 1 more at the start of a run or of a
// sequence).  The sums run in the same order as above: the same bits.
template <typename T, int VEC, int TAPS>
__global__ void short_conv_walk_kernel(const T* __restrict__ u, int64_t row_in, const float* __restrict__ w, const float* __restrict__ state,
                                       int64_t slot_stride, const int* __restrict__ token_seq, const int* __restrict__ seq_start,
                                       const int* __restrict__ seq_slots, T* __restrict__ y, int C, int64_t n_tokens, int run) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c >= C) return;
    float wt[TAPS][VEC], win[TAPS > 1 ? TAPS - 1 : 1][VEC];
#pragma unroll
    for (int j = 0; j < TAPS; ++j)
#pragma unroll
        for (int k = 0; k < VEC; ++k) wt[j][k] = w[(int64_t)j * C + c + k];
    const int64_t t_begin = (int64_t)blockIdx.y * run, t_end = min(t_begin + run, n_tokens);
    int cur = -1;
    for (int64_t t = t_begin; t < t_end; ++t) {
        const int seq = token_seq[t];
        if (seq != cur) {                                      // the run's first token, or a sequence's first: fill the window
            cur = seq;
            const int64_t first = seq_start[seq];
            const float* st = state + (int64_t)seq_slots[seq] * slot_stride;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int64_t src = t - (TAPS - 1) + j;
                if (src >= first) {
                    const Pack<T> pk = load_pack<T>(u + src * row_in + c);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) win[j][k] = pk.get(k);
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) win[j][k] = st[(int64_t)(TAPS - 1 + (src - first)) * C + c + k];
                }
            }
        }
        const Pack<T> pk = load_pack<T>(u + t * row_in + c);
        float x[VEC], acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            x[k] = pk.get(k);
            acc[k] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j)
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] = fmaf(wt[j][k], win[j][k], acc[k]);
        Pack<T> out;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            acc[k] = fmaf(wt[TAPS - 1][k], x[k], acc[k]);
            out.set(k, acc[k]);
        }
        store_pack<T>(y + t * C + c, out);
#pragma unroll
        for (int j = 0; j + 1 < TAPS - 1; ++j)
#pragma unroll
            for (int k = 0; k < VEC; ++k) win[j][k] = win[j + 1][k];
        if (TAPS > 1) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) win[TAPS - 2 > 0 ? TAPS - 2 : 0][k] = x[k];
        }
    }
}

template <typename T, int TAPS>
int short_conv_walk_launch(const T* u, int64_t row_in, const float* w, const float* state, int64_t slot_stride, const int* token_seq,
                           const int* seq_start, const int* seq_slots, T* y, int C, int64_t n_tokens, cudaStream_t stream) {
    constexpr int V = Pack<T>::N;
    const int run = n_tokens >= 1024 ? 16 : (n_tokens >= 128 ? 4 : 1);
    const int64_t runs = (n_tokens + run - 1) / run;
    if (runs > 65535) return Q3_ERR_TOO_LARGE;
    const dim3 grid((unsigned)((C / V + 127) / 128), (unsigned)runs);
    return (int)q3_launch(short_conv_walk_kernel<T, V, TAPS>, grid, dim3(128), 0, stream, u, row_in, w, state, slot_stride, token_seq,
                          seq_start, seq_slots, y, C, n_tokens, run);
}

template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ u, int64_t row_in, float* __restrict__ state, int64_t slot_stride,
                                        const int* __restrict__ seq_start, const int* __restrict__ seq_slots, int C, int taps,
                                        int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = (int64_t)n_seqs * C;
    const int keep = taps - 1;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int seq = (int)(i / C), c = (int)(i % C);
        const int64_t first = seq_start[seq], n_new = seq_start[seq + 1] - first;
        float* st = state + (int64_t)seq_slots[seq] * slot_stride;
        // row r of the new state is row r + n_new of (old state, new rows): ascending r never reads what it wrote
        for (int r = 0; r < keep; ++r) {
            const int64_t src = r + n_new;
            st[(int64_t)r * C + c] = src < keep ? st[src * C + c] : to_f32<T>(u[(first + src - keep) * row_in + c]);
        }
    }
}

}  // namespace

#define Q3_CONV_EXPORTS(SUFFIX, T)                                                                                        \
    Q3_EXPORT int q3_short_conv_##SUFFIX(const void* u, int64_t row_in, const float* w, float* state, int64_t slot_stride, \
                                         const int* token_seq, const int* seq_start, const int* seq_slots, void* y,      \
                                         int channels, int taps, int64_t n_tokens, int n_seqs, void* stream) {           \
        if (n_tokens <= 0 || n_seqs <= 0) return 0;                                                                       \
        if (channels <= 0 || taps <= 0 || taps > 64 || row_in < channels) return Q3_ERR_BAD_SIZE;                         \
        constexpr int V = Pack<T>::N;                                                                                     \
        const bool vec = channels % V == 0 && row_in % V == 0 && aligned16(u) && aligned16(y);                            \
        const int64_t blocks = (n_tokens * (channels / (vec ? V : 1)) + 255) / 256;                                       \
        const dim3 grid((unsigned)(blocks < 65536 ? blocks : 65536));                                                     \
        const bool walk = vec && taps >= 2 && taps <= 4 && (n_tokens + 15) / 16 <= 65535;                                 \
        int code = walk ? (taps == 2 ? short_conv_walk_launch<T, 2>((const T*)u, row_in, w, state, slot_stride, token_seq, \
                                                                    seq_start, seq_slots, (T*)y, channels, n_tokens,      \
                                                                    (cudaStream_t)stream)                                 \
                           : taps == 3 ? short_conv_walk_launch<T, 3>((const T*)u, row_in, w, state, slot_stride,         \
                                                                      token_seq, seq_start, seq_slots, (T*)y, channels,   \
                                                                      n_tokens, (cudaStream_t)stream)                     \
                                       : short_conv_walk_launch<T, 4>((const T*)u, row_in, w, state, slot_stride,         \
                                                                      token_seq, seq_start, seq_slots, (T*)y, channels,   \
                                                                      n_tokens, (cudaStream_t)stream))                    \
                   : vec ? (int)q3_launch(short_conv_kernel<T, V>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)u,   \
                                        row_in, w, (const float*)state, slot_stride, token_seq, seq_start, seq_slots,    \
                                        (T*)y, channels, taps, n_tokens)                                                  \
                       : (int)q3_launch(short_conv_kernel<T, 1>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)u,   \
                                        row_in, w, (const float*)state, slot_stride, token_seq, seq_start, seq_slots,    \
                                        (T*)y, channels, taps, n_tokens);                                                 \
        if (code != 0 || taps == 1) return code;                                                                          \
        const int64_t sblocks = ((int64_t)n_seqs * channels + 255) / 256;                                                 \
        return (int)q3_launch(short_conv_state_kernel<T>, dim3((unsigned)(sblocks < 65536 ? sblocks : 65536)), dim3(256), \
                              0, (cudaStream_t)stream, (const T*)u, row_in, state, slot_stride, seq_start, seq_slots,     \
                              channels, taps, n_seqs);                                                                    \
    }

Q3_CONV_EXPORTS(f32, float)
Q3_CONV_EXPORTS(bf16, bf16)
