// Attention whose keys and values are expanded from a small latent per token (a cache row is the latent c of `rank`
// values followed by one rotated key part of `rot` values that all heads share).  The expansion never happens: with
//
//     score_h(i, j) = ( q_plain_h(i) . W_uk_h c_j  +  q_rot_h(i) . k_rot_j ) * scale
//                   = ( (W_uk_h^T q_plain_h(i)) . c_j  +  q_rot_h(i) . k_rot_j ) * scale
//     out_h(i)      = W_uv_h ( sum_j p_h(i, j) c_j )
//
// the attention itself is multi-query attention over the cache rows [c | k_rot] with values c, and two products per
// head stand before and after it.  The kernels of this file do what is particular to that form:
//
//   latent_prepare : per token.  c = unit_rms(down[:rank]) * w_c, the rest of the row rotated by the token's position;
//                    both go to the token's key row in its page, c also to its value row.  With q_rank > 0 the
//                    latent of the queries, another stretch of the same projection row, is normalised with its own
//                    weight into `cq`.
//   latent_queries : per (token, head).  The rotated part of the query is rotated and put behind the absorbed part
//                    in the row the attention reads: q_full[t, h, rank:] = rotate(q[t, h, dim:]).
//   head_product   : out[t, h, out_off + j] = sum_i x[t, h, x_off + i] * W[h, i, j]  (* sigmoid(gate[t, h, j])), a product
//                    per head with 32-bit accumulation in ascending i: the absorption of W_uk into the query
//                    and the expansion of the attention's output by W_uv (with the output gate on the way).
//
// The rotation turns the first `rot_dims` values of the rotated part, in pairs (2i, 2i + 1) if `interleaved`, else
// (i, i + rot_dims / 2); pair i of a token at position p is turned by the angle p * f_i, whose cosine and sine come
// from tables [positions, rot_dims / 2] (float32).  Statistics, rotation and sums are 32-bit whatever T.
#include "common.cuh"

namespace {

constexpr int PAGE = Q3_PAGE_TOKENS;

// the rotated value at place i of a part of `rot` values, read from src
template <typename T>
__device__ __forceinline__ float rotated_at(const T* __restrict__ src, int i, int rot_dims, int interleaved,
                                            const float* __restrict__ cos_row, const float* __restrict__ sin_row) {
    if (i >= rot_dims) return to_f32<T>(src[i]);
    const int half = rot_dims >> 1;
    int pair, partner;
    bool first;
    if (interleaved) {
        pair = i >> 1;
        first = (i & 1) == 0;
        partner = first ? i + 1 : i - 1;
    } else {
        first = i < half;
        pair = first ? i : i - half;
        partner = first ? i + half : i - half;
    }
    const float a = to_f32<T>(src[i]), b = to_f32<T>(src[partner]);
    const float c = cos_row[pair], s = sin_row[pair];
    return first ? a * c - b * s : a * c + b * s;     // (u, v) -> (u cos - v sin, v cos + u sin)
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, int64_t proj_stride, int kv_off, int q_off, const float* __restrict__ w_c,
                      const float* __restrict__ w_q, T* __restrict__ cq, T* __restrict__ k_pages, T* __restrict__ v_pages,
                      const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, const int* __restrict__ token_seq,
                      const int* __restrict__ token_pos, const int* __restrict__ page_table, int pages_per_seq, int rank, int rot,
                      int rot_dims, int interleaved, int q_rank, float eps, int write_kv) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const T* row = proj + t * proj_stride;
    const int tid = threadIdx.x;
    if (q_rank > 0) {
        const T* qr = row + q_off;
        float sq = 0.0f;
        for (int i = tid; i < q_rank; i += blockDim.x) {
            const float v = to_f32<T>(qr[i]);
            sq += v * v;
        }
        const float inv = rsqrtf(block_sum(sq, scratch) / (float)q_rank + eps);
        for (int i = tid; i < q_rank; i += blockDim.x) cq[t * q_rank + i] = from_f32<T>(to_f32<T>(qr[i]) * inv * w_q[i]);
    }
    if (!write_kv) return;
    const T* kr = row + kv_off;
    float sq = 0.0f;
    for (int i = tid; i < rank; i += blockDim.x) {
        const float v = to_f32<T>(kr[i]);
        sq += v * v;
    }
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)rank + eps);
    const int pos = token_pos[t];
    const int page = page_table[(int64_t)token_seq[t] * pages_per_seq + pos / PAGE];
    T* key = k_pages + ((int64_t)page * PAGE + pos % PAGE) * (rank + rot);
    T* value = v_pages + ((int64_t)page * PAGE + pos % PAGE) * rank;
    for (int i = tid; i < rank; i += blockDim.x) {
        const T c = from_f32<T>(to_f32<T>(kr[i]) * inv * w_c[i]);
        key[i] = c;
        value[i] = c;
    }
    const int half = rot_dims >> 1;
    const float* cos_row = cos_tab + (int64_t)pos * half;
    const float* sin_row = sin_tab + (int64_t)pos * half;
    for (int i = tid; i < rot; i += blockDim.x)
        key[rank + i] = from_f32<T>(rotated_at<T>(kr + rank, i, rot_dims, interleaved, cos_row, sin_row));
}

template <typename T>
__global__ void latent_queries_kernel(const T* __restrict__ q, int64_t q_row, T* __restrict__ q_full, const float* __restrict__ cos_tab,
                                      const float* __restrict__ sin_tab, const int* __restrict__ token_pos, int64_t n_tokens, int H,
                                      int d, int rank, int rot, int rot_dims, int interleaved) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = n_tokens * H * rot;
    const int half = rot_dims >> 1;
    for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(x % rot);
        const int64_t th = x / rot, t = th / H;
        const int pos = token_pos[t];
        const T* src = q + t * q_row + (th - t * H) * (d + rot) + d;
        q_full[th * (rank + rot) + rank + i] =
            from_f32<T>(rotated_at<T>(src, i, rot_dims, interleaved, cos_tab + (int64_t)pos * half, sin_tab + (int64_t)pos * half));
    }
}

constexpr int TM = 32, TN = 64, TK = 32;

// One block per (tile of TM tokens, head, tile of TN outputs); 256 threads, each 2 tokens x 4 outputs.
template <typename T>
__global__ void __launch_bounds__(256)
head_product_kernel(const T* __restrict__ x, int64_t x_row, int x_head, int x_off, const T* __restrict__ w, T* __restrict__ out,
                    int64_t out_row, int out_head, int out_off, const T* __restrict__ gate, int64_t gate_row, int64_t n_tokens, int K,
                    int N) {
    __shared__ float xs[TM][TK + 1];
    __shared__ float ws[TK][TN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.y, col0 = blockIdx.z * TN;
    const int64_t row0 = (int64_t)blockIdx.x * TM;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const T* wh = w + (int64_t)head * K * N;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int e = tid; e < TM * TK; e += 256) {
            const int r = e / TK, k = e % TK;
            xs[r][k] = (row0 + r < n_tokens && k0 + k < K) ? to_f32<T>(x[(row0 + r) * x_row + (int64_t)head * x_head + x_off + k0 + k]) : 0.0f;
        }
        for (int e = tid; e < TK * TN; e += 256) {
            const int k = e / TN, c = e % TN;
            ws[k][c] = (k0 + k < K && col0 + c < N) ? to_f32<T>(wh[(int64_t)(k0 + k) * N + col0 + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < TK; ++k) {
            const float a0 = xs[ty * 2][k], a1 = xs[ty * 2 + 1][k];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float wv = ws[k][tx * 4 + b];
                acc[0][b] = fmaf(a0, wv, acc[0][b]);
                acc[1][b] = fmaf(a1, wv, acc[1][b]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        const int64_t r = row0 + ty * 2 + a;
        if (r >= n_tokens) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int c = col0 + tx * 4 + b;
            if (c >= N) continue;
            float v = acc[a][b];
            if (gate != nullptr) v = v / (1.0f + expf(-to_f32<T>(gate[r * gate_row + (int64_t)head * N + c])));
            out[r * out_row + (int64_t)head * out_head + out_off + c] = from_f32<T>(v);
        }
    }
}

}  // namespace

#define Q3_LATENT_EXPORTS(SUFFIX, T)                                                                                        \
    Q3_EXPORT int q3_latent_prepare_##SUFFIX(const void* proj, int64_t proj_stride, int kv_off, int q_off, const float* w_c, \
                                             const float* w_q, void* cq, void* k_pages, void* v_pages, const float* cos_tab, \
                                             const float* sin_tab, const int* token_seq, const int* token_pos,              \
                                             const int* page_table, int pages_per_seq, int64_t n_tokens, int rank, int rot, \
                                             int rot_dims, int interleaved, int q_rank, float eps, int write_kv,            \
                                             void* stream) {                                                                \
        if (n_tokens <= 0) return 0;                                                                                        \
        if (rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 != 0 || q_rank < 0 ||                     \
            (q_rank > 0 && (w_q == nullptr || cq == nullptr)) || (rot_dims > 0 && (cos_tab == nullptr || sin_tab == nullptr)) || \
            n_tokens > 0x7fffffffLL)                                                                                        \
            return Q3_ERR_BAD_SIZE;                                                                                         \
        return (int)q3_launch(latent_prepare_kernel<T>, dim3((unsigned)n_tokens), dim3(128), 0, (cudaStream_t)stream,       \
                              (const T*)proj, proj_stride, kv_off, q_off, w_c, w_q, (T*)cq, (T*)k_pages, (T*)v_pages, cos_tab, \
                              sin_tab, token_seq, token_pos, page_table, pages_per_seq, rank, rot, rot_dims, interleaved,    \
                              q_rank, eps, write_kv);                                                                       \
    }                                                                                                                       \
    Q3_EXPORT int q3_latent_queries_##SUFFIX(const void* q, int64_t q_row, void* q_full, const float* cos_tab, const float* sin_tab, \
                                             const int* token_pos, int64_t n_tokens, int heads, int d, int rank, int rot,   \
                                             int rot_dims, int interleaved, void* stream) {                                 \
        if (n_tokens <= 0 || rot <= 0) return 0;                                                                            \
        if (heads <= 0 || d < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 != 0 ||                       \
            (rot_dims > 0 && (cos_tab == nullptr || sin_tab == nullptr)))                                                   \
            return Q3_ERR_BAD_SIZE;                                                                                         \
        int64_t blocks = (n_tokens * heads * rot + 255) / 256;                                                              \
        const int64_t resident = (int64_t)q3_device_sm_count() * 8;                                                         \
        if (blocks > resident) blocks = resident;                                                                           \
        return (int)q3_launch(latent_queries_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream,         \
                              (const T*)q, q_row, (T*)q_full, cos_tab, sin_tab, token_pos, n_tokens, heads, d, rank, rot, rot_dims, \
                              interleaved);                                                                                 \
    }                                                                                                                       \
    Q3_EXPORT int q3_head_product_##SUFFIX(const void* x, int64_t x_row, int x_head, int x_off, const void* w, void* out,   \
                                           int64_t out_row, int out_head, int out_off, const void* gate, int64_t gate_row,  \
                                           int64_t n_tokens, int heads, int K, int N, void* stream) {                       \
        if (n_tokens <= 0) return 0;                                                                                        \
        if (heads <= 0 || heads > 65535 || K <= 0 || N <= 0 || (N + TN - 1) / TN > 65535 ||                                  \
            (n_tokens + TM - 1) / TM > 0x7fffffffLL)                                                                        \
            return Q3_ERR_BAD_SIZE;                                                                                         \
        const dim3 grid((unsigned)((n_tokens + TM - 1) / TM), heads, (N + TN - 1) / TN);                                     \
        return (int)q3_launch(head_product_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)x, x_row, x_head,  \
                              x_off, (const T*)w, (T*)out, out_row, out_head, out_off, (const T*)gate, gate_row, n_tokens, K, \
                              N);                                                                                           \
    }

Q3_LATENT_EXPORTS(f32, float)
Q3_LATENT_EXPORTS(bf16, bf16)
