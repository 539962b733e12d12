// Linear attention whose forget gate also decides what is written (HGRN2), with a fixed-size state per sequence:
//
//     f_t = low + (1 - low) * sigmoid(z_t + bias)          per head and channel, low the gate's lower bound
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T            (S: [d, vd] per head, float32, one per cache slot)
//     o_t = S_t^T q_t,   q_t = SiLU(projection)
//
// A row of the projection holds, head by head, the H*d values of q, the H*d of z and the H*vd of v.
//
//   gated_scan    : one block per (head, sequence, tile of up to 16 columns of the state: columns do not depend
//                   on one another) walks the sequence's new tokens in order with its share of the state in
//                   registers: thread (j, r) owns column j of the tile and the rows r * ROWS .. r * ROWS + ROWS - 1 (up
//                   to 8 rows; the threads of a column add their partial outputs through shared memory); it reads the
//                   state from the slot's row before the first token and writes it back after the last.  The
//                   tokens arrive a stage (up to 16) at a time: while the threads walk a stage, each by itself,
//                   the projection rows of the next stage are already on their way into registers; they are activated
//                   into shared memory between the two barriers of a stage, so a token costs no barrier of its own
//                   and no wait for global memory.  The launch depends on the sizes only, never on the step: a
//                   token's output is the same bits however the sequence was cut.  A decode step is the same kernel
//                   with one token.  Gate, state and o are 32-bit whatever T.
//   head_rms_norm : out = T( o / sqrt(mean(o^2) + eps) * w ) over the vd values of every (token, head); one weight
//                   vector for all heads.
#include "common.cuh"

namespace {

constexpr int COL_TILE = 16;      // columns of the state per block
constexpr int MAX_ROWS = 8;       // rows of the state per thread
constexpr int MAX_STAGE = 16;     // tokens fetched together
constexpr int PRE_QF = 8;         // values of q and of the gate that a thread holds for the next stage
constexpr int PRE_V = 2;          // values of v

// Sigmoid for the gate and the query's SiLU: exact division and expf in the 32-bit path; with bfloat16 inputs the
// hardware's exponential and reciprocal (32-bit, a few units in the last place).
template <typename T> __device__ __forceinline__ float sigmoid_of(float z) { return 1.0f / (1.0f + expf(-z)); }
template <> __device__ __forceinline__ float sigmoid_of<bf16>(float z) { return __fdividef(1.0f, 1.0f + __expf(-z)); }

template <typename T, int ROWS>
__global__ void __launch_bounds__(512)
gated_scan_kernel(const T* __restrict__ proj, float* __restrict__ state, const float* __restrict__ low, const float* __restrict__ bias,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_slots, float* __restrict__ out, int H, int d, int vd,
                  int R, int vt, int stage) {
    extern __shared__ __align__(16) float smem[];
    const int dp = R * ROWS;                 // d rounded up to whole threads: the rows beyond d hold q = 0
    float* q_s = smem;                       // [stage][dp]
    float* f_s = q_s + stage * dp;           // [stage][dp]
    float* v_s = f_s + stage * dp;           // [stage][vt]
    float* red = v_s + stage * vt;           // [stage][R][vt]
    pdl_launch_dependents();
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * vt;
    const int tid = threadIdx.x, nthreads = blockDim.x, jt = tid % vt, j = col0 + jt, r = tid / vt;
    const bool live = r < R && j < vd;
    const int64_t cols = 2 * (int64_t)H * d + (int64_t)H * vd;
    // which values of a stage this thread fetches: x = tid + k * nthreads < stage * d (q and gate), < stage * vt (v);
    // the token and the channel of each, found once (token << 16 | channel; a token beyond the stage: none)
    float lo_r[PRE_QF], bias_r[PRE_QF];
    int at_qf[PRE_QF], at_v[PRE_V];
#pragma unroll
    for (int k = 0; k < PRE_QF; ++k) {
        const int x = tid + k * nthreads;
        const int i = x % d;
        at_qf[k] = x < stage * d ? (x / d) << 16 | i : MAX_STAGE << 16;
        lo_r[k] = x < stage * d ? low[head * d + i] : 0.0f;
        bias_r[k] = x < stage * d ? bias[head * d + i] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < PRE_V; ++k) {
        const int x = tid + k * nthreads;
        at_v[k] = x < stage * vt ? (x / vt) << 16 | (x % vt) : MAX_STAGE << 16;
    }
    for (int x = tid; x < 2 * stage * dp; x += nthreads) smem[x] = 0.0f;        // the padding rows stay 0
    pdl_wait();
    float* S_g = state + ((int64_t)seq_slots[seq] * H + head) * d * vd;
    float S[ROWS];
#pragma unroll
    for (int n = 0; n < ROWS; ++n) {
        const int i = r * ROWS + n;
        S[n] = live && i < d ? S_g[(int64_t)i * vd + j] : 0.0f;
    }
    const int t_begin = seq_start[seq], t_end = seq_start[seq + 1];
    T q_raw[PRE_QF], f_raw[PRE_QF], v_raw[PRE_V];
    auto fetch = [&](int t0) {
        const int n_stage = min(stage, t_end - t0);
#pragma unroll
        for (int k = 0; k < PRE_QF; ++k) {
            const int tt = at_qf[k] >> 16, i = at_qf[k] & 0xffff;
            if (tt < n_stage) {
                const T* row = proj + (int64_t)(t0 + tt) * cols + i;
                q_raw[k] = row[(int64_t)head * d];
                f_raw[k] = row[(int64_t)(H + head) * d];
            }
        }
#pragma unroll
        for (int k = 0; k < PRE_V; ++k) {
            const int tt = at_v[k] >> 16, c = at_v[k] & 0xffff;
            if (tt < n_stage && col0 + c < vd)
                v_raw[k] = proj[(int64_t)(t0 + tt) * cols + 2 * (int64_t)H * d + (int64_t)head * vd + col0 + c];
        }
    };
    auto activate = [&](int t0) {
        const int n_stage = min(stage, t_end - t0);
#pragma unroll
        for (int k = 0; k < PRE_QF; ++k) {
            const int tt = at_qf[k] >> 16, i = at_qf[k] & 0xffff;
            if (tt < n_stage) {
                const float qz = to_f32<T>(q_raw[k]), fz = to_f32<T>(f_raw[k]);
                q_s[tt * dp + i] = qz * sigmoid_of<T>(qz);
                f_s[tt * dp + i] = lo_r[k] + (1.0f - lo_r[k]) * sigmoid_of<T>(fz + bias_r[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < PRE_V; ++k) {
            const int tt = at_v[k] >> 16, c = at_v[k] & 0xffff;
            if (tt < n_stage) v_s[tt * vt + c] = col0 + c < vd ? to_f32<T>(v_raw[k]) : 0.0f;
        }
    };
    if (t_begin < t_end) fetch(t_begin);
    __syncthreads();                                     // the zeros are in place
    if (t_begin < t_end) activate(t_begin);
    __syncthreads();
    for (int t0 = t_begin; t0 < t_end; t0 += stage) {
        const int n_stage = min(stage, t_end - t0);
        if (t0 + stage < t_end) fetch(t0 + stage);       // on its way while this stage is walked
        if (live) {
#pragma unroll 2
            for (int tt = 0; tt < n_stage; ++tt) {
                const float v = v_s[tt * vt + jt];
                const float* fr = f_s + tt * dp + r * ROWS;
                const float* qr = q_s + tt * dp + r * ROWS;
                float part0 = 0.0f, part1 = 0.0f;
                if constexpr (ROWS % 4 == 0) {
#pragma unroll
                    for (int n = 0; n < ROWS; n += 4) {
                        const float4 f4 = *reinterpret_cast<const float4*>(fr + n), q4 = *reinterpret_cast<const float4*>(qr + n);
                        S[n] = fmaf(f4.x, S[n] - v, v);          // f S + (1 - f) v
                        S[n + 1] = fmaf(f4.y, S[n + 1] - v, v);
                        S[n + 2] = fmaf(f4.z, S[n + 2] - v, v);
                        S[n + 3] = fmaf(f4.w, S[n + 3] - v, v);
                        part0 = fmaf(S[n], q4.x, part0);
                        part1 = fmaf(S[n + 1], q4.y, part1);
                        part0 = fmaf(S[n + 2], q4.z, part0);
                        part1 = fmaf(S[n + 3], q4.w, part1);
                    }
                } else {
#pragma unroll
                    for (int n = 0; n < ROWS; ++n) {
                        S[n] = fmaf(fr[n], S[n] - v, v);
                        part0 = fmaf(S[n], qr[n], part0);
                    }
                }
                red[(tt * R + r) * vt + jt] = part0 + part1;
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
        if (t0 + stage < t_end) activate(t0 + stage);    // everybody has left the stage's q, gate and v
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < ROWS; ++n) {
            const int i = r * ROWS + n;
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
    const int R = (d + MAX_ROWS - 1) / MAX_ROWS;       // threads that share a column: up to 32
    const int need = (d + R - 1) / R;                  // rows a thread: up to 8
    const int rows = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
    const int threads = ((vt * R + 31) / 32) * 32;     // up to 512
    const int stage = max(1, min(MAX_STAGE, min(PRE_QF * threads / d, PRE_V * threads / vt)));
    const size_t smem = (size_t)stage * (2 * R * rows + vt + R * vt) * sizeof(float);      // at most 66 KB
    const dim3 grid(H, n_seqs, (vd + vt - 1) / vt);
#define Q3_SCAN(ROWS)                                                                                                        \
    do {                                                                                                                     \
        if (smem > 48 * 1024) {                                                                                              \
            const cudaError_t e = cudaFuncSetAttribute(gated_scan_kernel<T, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                       (int)smem);                                                           \
            if (e != cudaSuccess) return (int)e;                                                                             \
        }                                                                                                                    \
        return (int)q3_launch(gated_scan_kernel<T, ROWS>, grid, dim3(threads), smem, stream, proj, state, low, bias,         \
                              seq_start, seq_slots, out, H, d, vd, R, vt, stage);                                           \
    } while (0)
    if (rows == 1) Q3_SCAN(1);
    if (rows == 2) Q3_SCAN(2);
    if (rows == 4) Q3_SCAN(4);
    Q3_SCAN(8);
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
