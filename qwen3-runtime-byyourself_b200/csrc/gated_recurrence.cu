// Linear attention whose forget gate also decides what is written (HGRN2), with a fixed-size state per sequence:
//
//     f_t = low + (1 - low) * sigmoid(z_t + bias)          per head and channel, low the gate's lower bound
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T            (S: [d, vd] per head, float32, one per cache slot)
//     o_t = S_t^T q_t,   q_t = SiLU(projection)
//
// A row of the projection holds, head by head, the H*d values of q, the H*d of z and the H*vd of v.
//
//   gated_scan    : one block per (head, sequence, tile of up to 64 columns of the state: columns do not depend
//                   on one another) walks the sequence's new tokens in order with its share of the state in
//                   registers: thread (j, r) owns column j of the tile and the rows r, r + R, r + 2R, ...; it reads
//                   the state from the slot's row before the first token and writes it back after the last.  The
//                   tokens arrive STAGE at a time: all threads fetch and activate q, f and v of a stage into shared
//                   memory, then every thread walks the stage by itself, so a token costs no barrier of its own.
//                   A decode step is the same kernel with one token.  Gate, state and o are 32-bit whatever T.
//   head_rms_norm : out = T( o / sqrt(mean(o^2) + eps) * w ) over the vd values of every (token, head); one weight
//                   vector for all heads.
#include "common.cuh"

namespace {

constexpr int COL_TILE = 64;      // columns of the state per block
constexpr int MAX_THREADS = 512;
constexpr int STAGE = 8;          // tokens fetched together

template <typename T, int ROWS>
__global__ void __launch_bounds__(MAX_THREADS)
gated_scan_kernel(const T* __restrict__ proj, float* __restrict__ state, const float* __restrict__ low, const float* __restrict__ bias,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_slots, float* __restrict__ out, int H, int d, int vd,
                  int R, int vt) {
    extern __shared__ float smem[];
    float* q_s = smem;                       // [STAGE][d]
    float* f_s = q_s + STAGE * d;            // [STAGE][d]
    float* v_s = f_s + STAGE * d;            // [STAGE][vt]
    float* red = v_s + STAGE * vt;           // [STAGE][R][vt]
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * vt;
    const int tid = threadIdx.x, nthreads = blockDim.x, jt = tid % vt, j = col0 + jt, r = tid / vt;
    const bool live = r < R && j < vd;
    const int64_t cols = 2 * (int64_t)H * d + (int64_t)H * vd;
    float* S_g = state + ((int64_t)seq_slots[seq] * H + head) * d * vd;
    float S[ROWS];
#pragma unroll
    for (int n = 0; n < ROWS; ++n) {
        const int i = r + n * R;
        S[n] = live && i < d ? S_g[(int64_t)i * vd + j] : 0.0f;
    }
    const int t_end = seq_start[seq + 1];
    for (int t0 = seq_start[seq]; t0 < t_end; t0 += STAGE) {
        const int n_stage = min(STAGE, t_end - t0);
        for (int x = tid; x < n_stage * d; x += nthreads) {
            const int tt = x / d, i = x % d;
            const T* row = proj + (int64_t)(t0 + tt) * cols;
            const float qz = to_f32<T>(row[(int64_t)head * d + i]), fz = to_f32<T>(row[(int64_t)(H + head) * d + i]);
            const float lo = low[head * d + i];
            q_s[x] = qz / (1.0f + expf(-qz));
            f_s[x] = lo + (1.0f - lo) / (1.0f + expf(-(fz + bias[head * d + i])));
        }
        for (int x = tid; x < n_stage * vt; x += nthreads) {
            const int tt = x / vt, c = x % vt;
            v_s[x] = col0 + c < vd ? to_f32<T>(proj[(int64_t)(t0 + tt) * cols + 2 * (int64_t)H * d + (int64_t)head * vd + col0 + c]) : 0.0f;
        }
        __syncthreads();
        if (live) {
            for (int tt = 0; tt < n_stage; ++tt) {
                const float v = v_s[tt * vt + jt];
                float part = 0.0f;
#pragma unroll
                for (int n = 0; n < ROWS; ++n) {
                    const int i = r + n * R;
                    if (i < d) {
                        const float f = f_s[tt * d + i];
                        S[n] = fmaf(f, S[n], (1.0f - f) * v);
                        part = fmaf(S[n], q_s[tt * d + i], part);
                    }
                }
                red[(tt * R + r) * vt + jt] = part;
            }
        }
        __syncthreads();
        for (int x = tid; x < n_stage * vt; x += nthreads) {
            const int tt = x / vt, c = x % vt;
            if (col0 + c < vd) {
                float o = 0.0f;
                for (int rr = 0; rr < R; ++rr) o += red[(tt * R + rr) * vt + c];
                out[((int64_t)(t0 + tt) * H + head) * vd + col0 + c] = o;
            }
        }
        // the next stage's fetch writes q_s, f_s and v_s, which nobody reads any more; `red` is written again
        // only after the barrier that follows that fetch
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < ROWS; ++n) {
            const int i = r + n * R;
            if (i < d) S_g[(int64_t)i * vd + j] = S[n];
        }
    }
}

template <typename T>
int gated_scan_launch(const T* proj, float* state, const float* low, const float* bias, const int* seq_start, const int* seq_slots,
                      float* out, int n_seqs, int H, int d, int vd, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || d <= 0 || vd <= 0 || d > 256 || vd > 256 || n_seqs > 65535) return Q3_ERR_BAD_SIZE;
    const int vt = min(vd, COL_TILE);
    const int R = min(d, MAX_THREADS / vt);            // row slices: as many as a block holds
    const int rows = (d + R - 1) / R;                  // at most 32: d <= 256, R >= 8 unless d is smaller
    const int threads = ((vt * R + 31) / 32) * 32;
    const size_t smem = (size_t)STAGE * (2 * d + vt + R * vt) * sizeof(float);      // at most 35 KB
    const dim3 grid(H, n_seqs, (vd + vt - 1) / vt);
#define Q3_SCAN(ROWS)                                                                                                       \
    return (int)q3_launch(gated_scan_kernel<T, ROWS>, grid, dim3(threads), smem, stream, proj, state, low, bias, seq_start, \
                          seq_slots, out, H, d, vd, R, vt)
    if (rows <= 1) Q3_SCAN(1);
    if (rows <= 2) Q3_SCAN(2);
    if (rows <= 4) Q3_SCAN(4);
    if (rows <= 8) Q3_SCAN(8);
    if (rows <= 16) Q3_SCAN(16);
    Q3_SCAN(32);
#undef Q3_SCAN
}

// One warp per (token, head).
template <typename T>
__global__ void head_rms_norm_kernel(const float* __restrict__ o, const float* __restrict__ w, T* __restrict__ out, int64_t n_rows, int vd,
                                     float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = o + row * vd;
    float sq = 0.0f;
    for (int c = lane; c < vd; c += 32) sq += x[c] * x[c];
    const float inv = rsqrtf(warp_sum(sq) / (float)vd + eps);
    for (int c = lane; c < vd; c += 32) out[row * vd + c] = from_f32<T>(x[c] * inv * w[c]);
}

}  // namespace

#define Q3_GATED_EXPORTS(SUFFIX, T)                                                                                         \
    Q3_EXPORT int q3_gated_scan_##SUFFIX(const void* proj, float* state, const float* low, const float* bias,              \
                                         const int* seq_start, const int* seq_slots, float* out, int n_seqs, int heads,    \
                                         int d, int vd, void* stream) {                                                    \
        return gated_scan_launch<T>((const T*)proj, state, low, bias, seq_start, seq_slots, out, n_seqs, heads, d, vd,      \
                                    (cudaStream_t)stream);                                                                 \
    }                                                                                                                       \
    Q3_EXPORT int q3_head_rms_norm_##SUFFIX(const float* o, const float* w, void* out, int64_t n_rows, int vd, float eps,   \
                                            void* stream) {                                                                \
        if (n_rows <= 0) return 0;                                                                                          \
        if (vd <= 0 || (n_rows + 7) / 8 > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                             \
        return (int)q3_launch(head_rms_norm_kernel<T>, dim3((unsigned)((n_rows + 7) / 8)), dim3(256), 0,                    \
                              (cudaStream_t)stream, o, w, (T*)out, n_rows, vd, eps);                                        \
    }

Q3_GATED_EXPORTS(f32, float)
Q3_GATED_EXPORTS(bf16, bf16)
