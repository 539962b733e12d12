// Linear attention with keys: a state S [d, vdx] per head and sequence (float32, in the cache's state rows) that
// every token decays and writes an outer product into,
//
//     S_t = diag(a_t) S_(t-1) + k_t (b_t v_t)^T,        o_t = S_t^T (q_t * q_scale)
//
// in two forms that share one kernel:
//
//   per channel  : a_t [N, H*d] (float32), one decay per key channel, b = 1 (gated linear attention; `channel_decay`
//                  makes a_t = sigmoid(z_t + bias)^(1/tau) from 32-bit logits, once for all the blocks that read it).
//   per head     : a_t = keep[t, h], b_t = write[t, h], two 32-bit numbers per token and head that `memory_gates`
//                  prepares (a matrix memory with exponential gates).  With `ones` the state has one column more than
//                  the values, vdx = vd + 1, whose value is 1 for every token: that column is the normaliser
//                  n_t = a_t n_(t-1) + b_t k_t, and its output n_t . q_t.
//
//   decay_scan   : one block per (head, sequence, tile of up to 16 columns of the state: columns do not depend on
//                  one another) walks the sequence's new tokens in order with its share of the state in registers:
//                  thread (j, r) owns column j of the tile and the rows r * ROWS .. r * ROWS + ROWS - 1; the threads of
//                  a column add their partial outputs through shared memory.  It reads the state from the slot's row
//                  before the first token and writes it back after the last.  Tokens arrive a stage (up to 16) at a
//                  time: while a stage is walked, the rows of the next are on their way into registers, the decays of
//                  the one after it too, and the lines of q, k and v of the one after it are asked into L2 (a walk of
//                  16 tokens is about as long as a trip to DRAM and hides no more than that).  The launch
//                  depends on the sizes only, never on the step: a token's output is the same bits however the
//                  sequence was cut.  A decode step is the same kernel with one token.
//   memory_gates : for every (sequence, head) one warp turns the gate logits zi, zf [N, H] (float32, biases added here)
//                  into i = cap tanh(zi / cap), f = logsigmoid(cap tanh(zf / cap)), finds the running maximum
//                  m_t = max(f_t + m_(t-1), i_t) from the slot's stored m (0 for a new sequence), 32 tokens at a time by a
//                  scan over the warp, and writes keep = exp(f + m_(t-1) - m_t), write = exp(i - m_t) and low = exp(-m_t).
//   head_gated_norm : per (token, head): x = o (divided by max(|n . q|, low) + floor if the state has the normaliser
//                  column), y = x / sqrt(mean(x^2) + eps) * w * act(gate), act = sigmoid or SiLU; w one vector per
//                  head or one for all heads.
//
// Decays, gates, state and outputs are 32-bit whatever T; T is the type of q, k, v, the output gate and the result.
#include "common.cuh"

namespace {

constexpr int COL_TILE = 16;      // columns of the state per block
constexpr int MAX_ROWS = 8;       // rows of the state per thread
constexpr int MAX_STAGE = 16;     // tokens fetched together
constexpr int PRE_QK = 8;         // values of q, of k and of the decay logits that a thread holds for the next stage
constexpr int PRE_V = 2;          // values of v

// Asks for a line to be brought into L2; nothing waits for it.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

struct ScanArgs {
    const void* q;                 // T: q, k, v are columns of rows of `row` values, head h at q + h * d and so on
    const void* k;
    const void* v;
    int64_t row;
    const float* z;                // per channel: [N, H * d] decays; per head: null
    const float* keep;             // per head: [N, H]
    const float* write;
    float q_scale;
    int ones;                      // the state's last column takes the value 1
    float* state;                  // slot s, head h at state + s * slot_stride + h * d * vdx
    int64_t slot_stride;
    const int* seq_start;
    const int* seq_slots;
    float* out;                    // [N, H, vdx]
    int H, d, vd, vdx;
};

// MAXT: the most threads a block has (256 for keys up to 128 wide, which leaves a thread room for the values it holds for
// the stages to come)
template <typename T, int ROWS, bool PER_CHANNEL, int MAXT>
__global__ void __launch_bounds__(MAXT)
decay_scan_kernel(const ScanArgs p, int R, int vt, int stage) {
    extern __shared__ __align__(16) float smem[];
    const int dp = R * ROWS;                 // d rounded up to whole threads: the rows beyond d hold q = k = 0
    float* q_s = smem;                       // [stage][dp]
    float* k_s = q_s + stage * dp;           // [stage][dp]
    float* a_s = k_s + stage * dp;           // [stage][dp] per channel; per head [MAX_STAGE] keep, then [MAX_STAGE] write
    float* v_s = a_s + (PER_CHANNEL ? stage * dp : 2 * MAX_STAGE);   // [stage][vt]
    float* red = v_s + stage * vt;           // [stage][R][vt]
    pdl_launch_dependents();
    const int H = p.H, d = p.d, vd = p.vd, vdx = p.vdx;
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * vt;
    const int tid = threadIdx.x, nthreads = blockDim.x, jt = tid % vt, j = col0 + jt, r = tid / vt;
    const bool live = r < R && j < vdx;
    // nothing this kernel writes is read by it again: the inputs go through the read-only path
    const T* __restrict__ q_g = reinterpret_cast<const T*>(p.q) + (int64_t)head * d;
    const T* __restrict__ k_g = reinterpret_cast<const T*>(p.k) + (int64_t)head * d;
    const T* __restrict__ v_g = reinterpret_cast<const T*>(p.v) + (int64_t)head * vd;
    const float* __restrict__ z_g = p.z, * __restrict__ keep_g = p.keep, * __restrict__ write_g = p.write;
    float* __restrict__ out_g = p.out;
    const int64_t row_g = p.row;
    // which values of a stage this thread fetches: x = tid + n * nthreads < stage * d (q, k, decay), < stage * vt (v);
    // the token and the channel of each, found once (token << 16 | channel; a token beyond the stage: none)
    int at_qk[PRE_QK], at_v[PRE_V];
#pragma unroll
    for (int n = 0; n < PRE_QK; ++n) {
        const int x = tid + n * nthreads;
        at_qk[n] = x < stage * d ? (x / d) << 16 | (x % d) : MAX_STAGE << 16;
    }
#pragma unroll
    for (int n = 0; n < PRE_V; ++n) {
        const int x = tid + n * nthreads;
        at_v[n] = x < stage * vt ? (x / vt) << 16 | (x % vt) : MAX_STAGE << 16;
    }
    for (int x = tid; x < (PER_CHANNEL ? 3 : 2) * stage * dp; x += nthreads) smem[x] = 0.0f;    // the padding rows stay 0
    pdl_wait();
    float* S_g = p.state + (int64_t)p.seq_slots[seq] * p.slot_stride + (int64_t)head * d * vdx;
    float S[ROWS];
#pragma unroll
    for (int n = 0; n < ROWS; ++n) {
        const int i = r * ROWS + n;
        S[n] = live && i < d ? S_g[(int64_t)i * vdx + j] : 0.0f;
    }
    const int t_begin = p.seq_start[seq], t_end = p.seq_start[seq + 1];
    T q_raw[PRE_QK], k_raw[PRE_QK], v_raw[PRE_V];
    float z_raw[PER_CHANNEL ? PRE_QK : 1], z_ahead[PER_CHANNEL ? PRE_QK : 1], keep_raw = 0.0f, write_raw = 1.0f;
    // the decays are twice as many bytes as q or k, and asking them into L2 ahead did not hide them: they are loaded into
    // registers a stage earlier than the rest, two stages before they are walked
    auto load_decays = [&](int t0) {
        if constexpr (PER_CHANNEL) {
            const int n_stage = min(stage, t_end - t0);
#pragma unroll
            for (int n = 0; n < PRE_QK; ++n) {
                const int tt = at_qk[n] >> 16, i = at_qk[n] & 0xffff;
                if (tt < n_stage) z_ahead[n] = __ldg(z_g + ((int64_t)(t0 + tt) * H + head) * d + i);
            }
        }
    };
    auto fetch = [&](int t0) {
        const int n_stage = min(stage, t_end - t0);
        if constexpr (PER_CHANNEL) {
#pragma unroll
            for (int n = 0; n < PRE_QK; ++n) z_raw[n] = z_ahead[n];
            load_decays(t0 + stage);
        }
#pragma unroll
        for (int n = 0; n < PRE_QK; ++n) {
            const int tt = at_qk[n] >> 16, i = at_qk[n] & 0xffff;
            if (tt < n_stage) {
                q_raw[n] = __ldg(q_g + (int64_t)(t0 + tt) * row_g + i);
                k_raw[n] = __ldg(k_g + (int64_t)(t0 + tt) * row_g + i);
            }
        }
#pragma unroll
        for (int n = 0; n < PRE_V; ++n) {
            const int tt = at_v[n] >> 16, c = at_v[n] & 0xffff;
            if (tt < n_stage && col0 + c < vd) v_raw[n] = __ldg(v_g + (int64_t)(t0 + tt) * row_g + col0 + c);
        }
        if constexpr (!PER_CHANNEL) {
            if (tid < n_stage) {
                keep_raw = __ldg(keep_g + (int64_t)(t0 + tid) * H + head);
                write_raw = __ldg(write_g + (int64_t)(t0 + tid) * H + head);
            }
        }
        // the stage after that one: its lines are asked into L2 now (one request per 32 bytes), so that its loads, a stage
        // from now, find them there - a walk of 16 tokens is about as long as a trip to DRAM and hides no more
        const int n_ahead = min(stage, t_end - t0 - stage);
#pragma unroll
        for (int n = 0; n < PRE_QK; ++n) {
            const int tt = at_qk[n] >> 16, i = at_qk[n] & 0xffff;
            if (tt < n_ahead && (i & 7) == 0) {
                if ((i & 15) == 0 || sizeof(T) == 4) {
                    prefetch_l2(q_g + (int64_t)(t0 + stage + tt) * row_g + i);
                    prefetch_l2(k_g + (int64_t)(t0 + stage + tt) * row_g + i);
                }
            }
        }
#pragma unroll
        for (int n = 0; n < PRE_V; ++n) {
            const int tt = at_v[n] >> 16, c = at_v[n] & 0xffff;
            if (tt < n_ahead && c == 0) prefetch_l2(v_g + (int64_t)(t0 + stage + tt) * row_g + col0);
        }
    };
    auto activate = [&](int t0) {
        const int n_stage = min(stage, t_end - t0);
#pragma unroll
        for (int n = 0; n < PRE_QK; ++n) {
            const int tt = at_qk[n] >> 16, i = at_qk[n] & 0xffff;
            if (tt < n_stage) {
                q_s[tt * dp + i] = to_f32<T>(q_raw[n]) * p.q_scale;
                k_s[tt * dp + i] = to_f32<T>(k_raw[n]);
                if constexpr (PER_CHANNEL) a_s[tt * dp + i] = z_raw[n];
            }
        }
#pragma unroll
        for (int n = 0; n < PRE_V; ++n) {
            const int tt = at_v[n] >> 16, c = at_v[n] & 0xffff;
            if (tt < n_stage) v_s[tt * vt + c] = col0 + c < vd ? to_f32<T>(v_raw[n]) : (p.ones && col0 + c == vd ? 1.0f : 0.0f);
        }
        if constexpr (!PER_CHANNEL) {
            if (tid < n_stage) {
                a_s[tid] = keep_raw;
                a_s[MAX_STAGE + tid] = write_raw;
            }
        }
    };
    if (t_begin < t_end) {
        load_decays(t_begin);
        fetch(t_begin);
    }
    __syncthreads();                                     // the zeros are in place
    if (t_begin < t_end) activate(t_begin);
    __syncthreads();
    for (int t0 = t_begin; t0 < t_end; t0 += stage) {
        const int n_stage = min(stage, t_end - t0);
        if (t0 + stage < t_end) fetch(t0 + stage);       // on its way while this stage is walked
        if (live) {
#pragma unroll 2
            for (int tt = 0; tt < n_stage; ++tt) {
                const float v = PER_CHANNEL ? v_s[tt * vt + jt] : v_s[tt * vt + jt] * a_s[MAX_STAGE + tt];   // b_t v_t
                const float* kr = k_s + tt * dp + r * ROWS;
                const float* qr = q_s + tt * dp + r * ROWS;
                const float* ar = a_s + tt * dp + r * ROWS;
                const float a_head = PER_CHANNEL ? 0.0f : a_s[tt];
                float part0 = 0.0f, part1 = 0.0f;
                if constexpr (ROWS % 4 == 0) {
#pragma unroll
                    for (int n = 0; n < ROWS; n += 4) {
                        const float4 k4 = *reinterpret_cast<const float4*>(kr + n), q4 = *reinterpret_cast<const float4*>(qr + n);
                        float4 a4 = make_float4(a_head, a_head, a_head, a_head);
                        if constexpr (PER_CHANNEL) a4 = *reinterpret_cast<const float4*>(ar + n);
                        S[n] = fmaf(a4.x, S[n], k4.x * v);
                        S[n + 1] = fmaf(a4.y, S[n + 1], k4.y * v);
                        S[n + 2] = fmaf(a4.z, S[n + 2], k4.z * v);
                        S[n + 3] = fmaf(a4.w, S[n + 3], k4.w * v);
                        part0 = fmaf(S[n], q4.x, part0);
                        part1 = fmaf(S[n + 1], q4.y, part1);
                        part0 = fmaf(S[n + 2], q4.z, part0);
                        part1 = fmaf(S[n + 3], q4.w, part1);
                    }
                } else {
#pragma unroll
                    for (int n = 0; n < ROWS; ++n) {
                        S[n] = fmaf(PER_CHANNEL ? ar[n] : a_head, S[n], kr[n] * v);
                        part0 = fmaf(S[n], qr[n], part0);
                    }
                }
                red[(tt * R + r) * vt + jt] = part0 + part1;
            }
        }
        __syncthreads();
        for (int x = tid; x < n_stage * vt; x += nthreads) {
            const int tt = x / vt, c = x % vt;
            if (col0 + c < vdx) {
                float o = 0.0f;
                for (int rr = 0; rr < R; ++rr) o += red[(tt * R + rr) * vt + c];
                out_g[((int64_t)(t0 + tt) * H + head) * vdx + col0 + c] = o;
            }
        }
        if (t0 + stage < t_end) activate(t0 + stage);    // everybody has left the stage's q, k, decay and v
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < ROWS; ++n) {
            const int i = r * ROWS + n;
            if (i < d) S_g[(int64_t)i * vdx + j] = S[n];
        }
    }
}

template <typename T, bool PER_CHANNEL>
int decay_scan_launch(const ScanArgs& p, int n_seqs, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    const int d = p.d, vdx = p.vdx;
    if (p.H <= 0 || d <= 0 || p.vd <= 0 || d > 256 || vdx > 256 || vdx < p.vd || vdx > p.vd + 1 || n_seqs > 65535 || p.H > 65535)
        return Q3_ERR_BAD_SIZE;
    const int vt = min(vdx, COL_TILE);
    const int R = (d + MAX_ROWS - 1) / MAX_ROWS;       // threads that share a column: up to 32
    const int need = (d + R - 1) / R;                  // rows a thread: up to 8
    const int rows = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
    const int threads = ((vt * R + 31) / 32) * 32;     // up to 512
    const int stage = max(1, min(MAX_STAGE, min(PRE_QK * threads / d, PRE_V * threads / vt)));
    const size_t smem = ((size_t)stage * ((PER_CHANNEL ? 3 : 2) * R * rows + vt + R * vt) + (PER_CHANNEL ? 0 : 2 * MAX_STAGE)) * sizeof(float);
    const dim3 grid(p.H, n_seqs, (vdx + vt - 1) / vt);
#define Q3_SCAN(ROWS, MAXT)                                                                                                  \
    do {                                                                                                                     \
        if (smem > 48 * 1024) {                                                                                              \
            const cudaError_t e = cudaFuncSetAttribute(decay_scan_kernel<T, ROWS, PER_CHANNEL, MAXT>,                        \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
            if (e != cudaSuccess) return (int)e;                                                                             \
        }                                                                                                                    \
        return (int)q3_launch(decay_scan_kernel<T, ROWS, PER_CHANNEL, MAXT>, grid, dim3(threads), smem, stream, p, R, vt,    \
                              stage);                                                                                        \
    } while (0)
    if (rows == 1) Q3_SCAN(1, 256);                    // d <= 8: at most 128 threads
    if (rows == 2) Q3_SCAN(2, 256);
    if (rows == 4) Q3_SCAN(4, 256);
    if (threads <= 256) Q3_SCAN(8, 256);
    Q3_SCAN(8, 512);
#undef Q3_SCAN
}

// a = sigmoid(z + bias)^(1 / tau) = exp(logsigmoid(z + bias) / tau), in place.
__global__ void channel_decay_kernel(float* __restrict__ z, const float* __restrict__ bias, float inv_tau, int64_t n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        z[i] = expf(log_sigmoid(z[i] + (bias != nullptr ? bias[i % width] : 0.0f)) * inv_tau);
}

// One warp per (sequence, head); 32 tokens at a time: the gates' activations side by side, the running maximum by a
// scan over the lanes, the exponentials side by side again.
__global__ void memory_gates_kernel(const float* __restrict__ zi, const float* __restrict__ zf, const float* __restrict__ bias_i,
                                    const float* __restrict__ bias_f, float cap, float* __restrict__ m_state, int64_t slot_stride,
                                    const int* __restrict__ seq_start, const int* __restrict__ seq_slots, float* __restrict__ keep,
                                    float* __restrict__ write, float* __restrict__ low, int H, int64_t z_row, int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_seqs * H) return;
    const int seq = pair / H, head = pair % H;
    float* m_at = m_state + (int64_t)seq_slots[seq] * slot_stride + head;
    float m = *m_at;
    const float inv_cap = 1.0f / cap, bi = bias_i ? bias_i[head] : 0.0f, bf = bias_f ? bias_f[head] : 0.0f;
    const int t_begin = seq_start[seq], t_end = seq_start[seq + 1];
    for (int t0 = t_begin; t0 < t_end; t0 += 32) {
        const int t = t0 + lane, n = min(32, t_end - t0);
        float gi = 0.0f, gf = 0.0f;
        if (t < t_end) {
            gi = cap * tanhf((zi[(int64_t)t * z_row + head] + bi) * inv_cap);
            gf = log_sigmoid(cap * tanhf((zf[(int64_t)t * z_row + head] + bf) * inv_cap));
        }
        // m_t = max(f_t + m_(t-1), i_t) is the map m -> max(m + F, I) with (F, I) = (f_t, i_t); two such maps in a row
        // are one, (F1, I1) then (F2, I2) = (F1 + F2, max(I1 + F2, I2)): a scan over the warp gives every lane the map of
        // all tokens up to its own.  (The maximum only has to be the same number wherever it is used: keep, write and
        // low are made from the m computed here, so the order of these sums shows in no output beyond rounding.)
        float F = t < t_end ? gf : 0.0f, I = t < t_end ? gi : -INFINITY;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float Fp = __shfl_up_sync(0xffffffffu, F, off), Ip = __shfl_up_sync(0xffffffffu, I, off);
            if (lane >= off) {
                I = fmaxf(Ip + F, I);
                F = Fp + F;
            }
        }
        const float m_mine = fmaxf(m + F, I);
        float m_before = __shfl_up_sync(0xffffffffu, m_mine, 1);
        if (lane == 0) m_before = m;
        m = __shfl_sync(0xffffffffu, m_mine, n - 1);
        if (t < t_end) {
            keep[(int64_t)t * H + head] = expf(gf + m_before - m_mine);
            write[(int64_t)t * H + head] = expf(gi - m_mine);
            low[(int64_t)t * H + head] = expf(-m_mine);
        }
    }
    if (lane == 0) *m_at = m;
}

// One warp per (token, head).  act 0: sigmoid, 1: SiLU.
template <typename T>
__global__ void head_gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ low, float floor_add,
                                       const float* __restrict__ w, int w_per_head, const T* __restrict__ gate, int64_t gate_row,
                                       T* __restrict__ out, int64_t n_rows, int H, int vd, int vdx, float eps, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const int64_t t = row / H;
    const int head = (int)(row % H);
    const float* x = o + row * vdx;
    float inv_den = 1.0f;
    if (vdx > vd) inv_den = 1.0f / (fmaxf(fabsf(x[vd]), low[row]) + floor_add);
    float sq = 0.0f;
    for (int c = lane; c < vd; c += 32) {
        const float y = x[c] * inv_den;
        sq += y * y;
    }
    const float inv = rsqrtf(warp_sum(sq) / (float)vd + eps);
    const float* wh = w + (w_per_head ? (int64_t)head * vd : 0);
    const T* g = gate + t * gate_row + (int64_t)head * vd;
    for (int c = lane; c < vd; c += 32) {
        const float z = to_f32<T>(g[c]);
        const float s = 1.0f / (1.0f + expf(-z));
        out[row * vd + c] = from_f32<T>(x[c] * inv_den * inv * wh[c] * (act ? z * s : s));
    }
}

}  // namespace

#define Q3_SCAN_EXPORTS(SUFFIX, T)                                                                                           \
    Q3_EXPORT int q3_decay_scan_##SUFFIX(const void* q, const void* k, const void* v, int64_t row, const float* z,          \
                                         const float* keep, const float* write,                                             \
                                         float q_scale, int ones, float* state, int64_t slot_stride, const int* seq_start,  \
                                         const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd,           \
                                         void* stream) {                                                                   \
        ScanArgs p;                                                                                                         \
        p.q = q; p.k = k; p.v = v; p.row = row; p.z = z; p.keep = keep;                                                     \
        p.write = write; p.q_scale = q_scale; p.ones = ones; p.state = state; p.slot_stride = slot_stride;                  \
        p.seq_start = seq_start; p.seq_slots = seq_slots; p.out = out; p.H = heads; p.d = d; p.vd = vd;                     \
        p.vdx = vd + (ones ? 1 : 0);                                                                                        \
        if ((z == nullptr) == (keep == nullptr) || (keep != nullptr && write == nullptr)) return Q3_ERR_BAD_SIZE;           \
        if (z != nullptr) return decay_scan_launch<T, true>(p, n_seqs, (cudaStream_t)stream);                               \
        return decay_scan_launch<T, false>(p, n_seqs, (cudaStream_t)stream);                                                \
    }                                                                                                                       \
    Q3_EXPORT int q3_head_gated_norm_##SUFFIX(const float* o, const float* low, float floor_add, const float* w,            \
                                              int w_per_head, const void* gate, int64_t gate_row, void* out,               \
                                              int64_t n_tokens, int heads, int vd, int vdx, float eps, int act,            \
                                              void* stream) {                                                              \
        const int64_t n_rows = n_tokens * heads;                                                                            \
        if (n_rows <= 0) return 0;                                                                                          \
        if (vd <= 0 || vdx < vd || (vdx > vd && low == nullptr) || (n_rows + 7) / 8 > 0x7fffffffLL) return Q3_ERR_BAD_SIZE; \
        return (int)q3_launch(head_gated_norm_kernel<T>, dim3((unsigned)((n_rows + 7) / 8)), dim3(256), 0,                  \
                              (cudaStream_t)stream, o, low, floor_add, w, w_per_head, (const T*)gate, gate_row, (T*)out,    \
                              n_rows, heads, vd, vdx, eps, act);                                                            \
    }

Q3_SCAN_EXPORTS(f32, float)
Q3_SCAN_EXPORTS(bf16, bf16)

Q3_EXPORT int q3_channel_decay(float* z, const float* bias, float inv_tau, int64_t n_tokens, int width, void* stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0) return Q3_ERR_BAD_SIZE;
    const int64_t n = n_tokens * width, blocks = (n + 255) / 256;
    return (int)q3_launch(channel_decay_kernel, dim3((unsigned)(blocks < 65536 ? blocks : 65536)), dim3(256), 0, (cudaStream_t)stream, z,
                          bias, inv_tau, n, width);
}

Q3_EXPORT int q3_memory_gates(const float* zi, const float* zf, const float* bias_i, const float* bias_f, float cap,
                              float* m_state, int64_t slot_stride, const int* seq_start, const int* seq_slots, float* keep,
                              float* write, float* low, int heads, int64_t z_row, int n_seqs, void* stream) {
    if (n_seqs <= 0) return 0;
    if (heads <= 0 || !(cap > 0.0f)) return Q3_ERR_BAD_SIZE;
    const int64_t pairs = (int64_t)n_seqs * heads;
    if ((pairs + 3) / 4 > 0x7fffffffLL) return Q3_ERR_TOO_LARGE;
    return (int)q3_launch(memory_gates_kernel, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, zi, zf,
                          bias_i, bias_f, cap, m_state, slot_stride, seq_start, seq_slots, keep, write, low, heads, z_row, n_seqs);
}
