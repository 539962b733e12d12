// More kernels for a hidden state that is kept in 32-bit whatever the compute type T of the matrix products:
//
//   settle_norm : a sublayer's output y (T) is normalised and added to the stream, stream += post(y), and the sum
//                 is normalised for the next reader, out = pre(stream), in one pass over the row.  Each of the two
//                 norms is of one of these kinds:
//                     0  none (no branch / no output)
//                     1  unit rms with a weight:   x / sqrt(mean(x^2) + eps) * w
//                     2  dynamic tanh:             tanh(alpha x) * w + b      (no statistics)
//                     3  nothing but the rounding: x                          (the output only)
//                 `out` is T, or float for a reader that goes on in 32-bit (a token shift).  With a list of rows
//                 only those rows are read, nothing is written to the stream and out[r] belongs to rows[r] (the
//                 model's tail).
//   token_shift : out[t] = T( h[t] + (h[t-1] - h[t]) * mu ), row by row within a sequence; the row before a step's
//                 first row of a sequence is that sequence's saved row (zero for a new sequence), and the step's last
//                 row of every sequence is saved for the next step.  h is float.
//   side_gate   : out[t, j] = T( gelu_tanh(a[t, j]) * table[ids[t], col0 + j] ): a slice of a second embedding gated
//                 by a projection of the hidden state.
//
// Statistics, weights and sums are 32-bit; only `out` is rounded to T.
#include "common.cuh"
#include <initializer_list>

namespace {

struct NormSpec {
    const float* w;
    const float* b;
    float alpha;
    float eps;
    int kind;
};

// V values at a time: 4 when rows split into 16-byte packets of floats, else 1
template <int V> __device__ __forceinline__ void ld_f32(const float* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
        v[0] = *p;
    }
}
template <int V> __device__ __forceinline__ void st_f32(float* p, const float (&v)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
template <typename T, int V> __device__ __forceinline__ void ld_t(const T* p, float (&v)[V]) {
    if constexpr (V == 4 && sizeof(T) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
    } else if constexpr (V == 4) {
        ld_f32<4>(reinterpret_cast<const float*>(p), v);
    } else {
        v[0] = to_f32<T>(*p);
    }
}
template <typename T, int V> __device__ __forceinline__ void st_t(T* p, const float (&v)[V]) {
    if constexpr (V == 4 && sizeof(T) == 2) {
        uint2 raw;
        *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = raw;
    } else if constexpr (V == 4) {
        st_f32<4>(reinterpret_cast<float*>(p), v);
    } else {
        *p = from_f32<T>(v[0]);
    }
}

template <typename T, int V>
__global__ void settle_norm_kernel(float* __restrict__ stream, const T* __restrict__ branch, NormSpec post, NormSpec pre,
                                   void* __restrict__ out, int out_f32, const int* __restrict__ rows, int size) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    float* xr = stream + row * size;
    const T* yr = post.kind != 0 ? branch + row * size : nullptr;
    const int first = threadIdx.x * V, stride = blockDim.x * V;
    float inv_post = 0.0f;
    if (post.kind == 1) {
        float sq = 0.0f;
        for (int c = first; c < size; c += stride) {
            float y[V];
            ld_t<T, V>(yr + c, y);
#pragma unroll
            for (int i = 0; i < V; ++i) sq += y[i] * y[i];
        }
        inv_post = rsqrtf(block_sum(sq, scratch) / (float)size + post.eps);
    }
    // the sum of V elements: every thread forms the elements it owns the same way in both passes below
    auto settled = [&](int c, float (&x)[V]) {
        ld_f32<V>(xr + c, x);
        if (post.kind == 0) return;
        float y[V], w[V];
        ld_t<T, V>(yr + c, y);
        ld_f32<V>(post.w + c, w);
        if (post.kind == 1) {
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] += y[i] * inv_post * w[i];
        } else {
            float b[V];
            ld_f32<V>(post.b + c, b);
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] += tanhf(post.alpha * y[i]) * w[i] + b[i];
        }
    };
    float inv_pre = 0.0f;
    if (pre.kind == 1) {
        float sq = 0.0f;
        for (int c = first; c < size; c += stride) {
            float x[V];
            settled(c, x);
#pragma unroll
            for (int i = 0; i < V; ++i) sq += x[i] * x[i];
        }
        inv_pre = rsqrtf(block_sum(sq, scratch) / (float)size + pre.eps);
    }
    T* out_t = reinterpret_cast<T*>(out) + (int64_t)blockIdx.x * size;
    float* out_f = reinterpret_cast<float*>(out) + (int64_t)blockIdx.x * size;
    for (int c = first; c < size; c += stride) {
        float x[V];
        settled(c, x);
        if (post.kind != 0 && rows == nullptr) st_f32<V>(xr + c, x);
        if (pre.kind == 0) continue;
        float y[V];
        if (pre.kind == 1) {
            float w[V];
            ld_f32<V>(pre.w + c, w);
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = x[i] * inv_pre * w[i];
        } else if (pre.kind == 2) {
            float w[V], b[V];
            ld_f32<V>(pre.w + c, w);
            ld_f32<V>(pre.b + c, b);
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = tanhf(pre.alpha * x[i]) * w[i] + b[i];
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = x[i];
        }
        if (out_f32) st_f32<V>(out_f + c, y);
        else st_t<T, V>(out_t + c, y);
    }
}

template <typename T, int V>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                   T* __restrict__ out, const int* __restrict__ token_seq, const int* __restrict__ seq_start,
                                   const int* __restrict__ seq_slots, int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int seq = token_seq[t];
    const int first = seq_start[seq], last = seq_start[seq + 1] - 1;
    const bool opens = t == first;
    // the block of a sequence's first row in the step reads the saved row and then replaces it: one reader, one writer
    float* saved = state + (int64_t)seq_slots[seq] * size;
    const float* before = opens ? saved : h + (t - 1) * size;
    for (int c = threadIdx.x * V; c < size; c += blockDim.x * V) {
        float now[V], prev[V], m[V], y[V];
        ld_f32<V>(h + t * size + c, now);
        ld_f32<V>(before + c, prev);
        ld_f32<V>(mu + c, m);
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = now[i] + (prev[i] - now[i]) * m[i];
        st_t<T, V>(out + t * size + c, y);
        if (opens) {
            float keep[V];
            ld_f32<V>(h + (int64_t)last * size + c, keep);
            st_f32<V>(saved + c, keep);
        }
    }
}

// whether every row starts on a 16-byte boundary for 4 values at a time (null pointers pass)
bool packets4(int size, std::initializer_list<const void*> ptrs) {
    if (size % 4 != 0) return false;
    for (const void* p : ptrs)
        if (((uintptr_t)p & 15) != 0) return false;
    return true;
}

template <typename T>
__global__ void side_gate_kernel(const T* __restrict__ a, const int* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int64_t n_tokens, int dim, int col0, int table_cols, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = n_tokens * dim;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / dim;
        const int j = (int)(i % dim), id = ids[t];
        const float e = id >= 0 && id < vocab ? to_f32<T>(table[(int64_t)id * table_cols + col0 + j]) : 0.0f;   // an id outside the table: zero
        out[i] = from_f32<T>(gate_activation<2>(to_f32<T>(a[i])) * e);
    }
}

bool spec_ok(const NormSpec& s, bool is_output) {
    if (s.kind < 0 || s.kind > 3 || (s.kind == 3 && !is_output)) return false;
    if ((s.kind == 1 || s.kind == 2) && s.w == nullptr) return false;
    return s.kind != 2 || s.b != nullptr;
}

}  // namespace

#define Q3_SHIFT_EXPORTS(SUFFIX, T)                                                                                          \
    Q3_EXPORT int q3_settle_norm_##SUFFIX(float* stream_rows, const void* branch, int post_kind, const float* post_w,        \
                                          const float* post_b, float post_alpha, float post_eps, int pre_kind,              \
                                          const float* pre_w, const float* pre_b, float pre_alpha, float pre_eps, void* out, \
                                          int out_f32, const int* rows, int64_t n_rows, int size, void* stream) {           \
        if (n_rows <= 0) return 0;                                                                                           \
        NormSpec post = {post_w, post_b, post_alpha, post_eps, post_kind}, pre = {pre_w, pre_b, pre_alpha, pre_eps, pre_kind}; \
        if (size <= 0 || !spec_ok(post, false) || !spec_ok(pre, true) || (post.kind != 0 && branch == nullptr) ||            \
            (pre.kind != 0 && out == nullptr) || n_rows > 0x7fffffffLL)                                                      \
            return Q3_ERR_BAD_SIZE;                                                                                          \
        if (packets4(size, {stream_rows, branch, post_w, post_b, pre_w, pre_b, out})) {                                       \
            const int lanes = size >= 2048 ? 512 : (size >= 1024 ? 256 : 128);                                               \
            return (int)q3_launch(settle_norm_kernel<T, 4>, dim3((unsigned)n_rows), dim3(lanes), 0, (cudaStream_t)stream,    \
                                  stream_rows, (const T*)branch, post, pre, out, out_f32, rows, size);                       \
        }                                                                                                                    \
        const int threads = size >= 2048 ? 512 : (size >= 512 ? 256 : 128);                                                  \
        return (int)q3_launch(settle_norm_kernel<T, 1>, dim3((unsigned)n_rows), dim3(threads), 0, (cudaStream_t)stream,      \
                              stream_rows, (const T*)branch, post, pre, out, out_f32, rows, size);                           \
    }                                                                                                                        \
    Q3_EXPORT int q3_token_shift_##SUFFIX(const float* h, const float* mu, float* state, void* out, const int* token_seq,    \
                                          const int* seq_start, const int* seq_slots, int64_t n_tokens, int size,           \
                                          void* stream) {                                                                    \
        if (n_tokens <= 0) return 0;                                                                                         \
        if (size <= 0 || n_tokens > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                                    \
        if (packets4(size, {h, mu, state, out}))                                                                             \
            return (int)q3_launch(token_shift_kernel<T, 4>, dim3((unsigned)n_tokens), dim3(size >= 1024 ? 256 : 128), 0,     \
                                  (cudaStream_t)stream, h, mu, state, (T*)out, token_seq, seq_start, seq_slots, size);       \
        return (int)q3_launch(token_shift_kernel<T, 1>, dim3((unsigned)n_tokens), dim3(size >= 1024 ? 256 : 128), 0,         \
                              (cudaStream_t)stream, h, mu, state, (T*)out, token_seq, seq_start, seq_slots, size);           \
    }                                                                                                                        \
    Q3_EXPORT int q3_side_gate_##SUFFIX(const void* a, const int* ids, const void* table, void* out, int64_t n_tokens,       \
                                        int dim, int col0, int table_cols, int vocab, void* stream) {                       \
        if (n_tokens <= 0) return 0;                                                                                         \
        if (dim <= 0 || col0 < 0 || col0 + dim > table_cols || vocab <= 0) return Q3_ERR_BAD_SIZE;                           \
        int64_t blocks = (n_tokens * dim + 255) / 256;                                                                       \
        const int64_t resident = (int64_t)q3_device_sm_count() * 8;                                                          \
        if (blocks > resident) blocks = resident;                                                                            \
        return (int)q3_launch(side_gate_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)a,  \
                              ids, (const T*)table, (T*)out, n_tokens, dim, col0, table_cols, vocab);                       \
    }

Q3_SHIFT_EXPORTS(f32, float)
Q3_SHIFT_EXPORTS(bf16, bf16)
