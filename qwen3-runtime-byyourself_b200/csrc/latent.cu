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
//                    per head with 32-bit accumulation: the absorption of W_uk into the query and the expansion of
//                    the attention's output by W_uv (with the output gate on the way).  bfloat16 operands whose rows
//                    split into 16-byte packets take tensor-core tiles, everything else fmaf tiles.
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


// The same product on the tensor cores, for bfloat16 operands whose rows can be fetched in 16-byte packets.  One block per
// (64 tokens, head, 64 outputs); four warps of 16 tokens x 64 outputs each.  x and W pass through shared memory in chunks of
// 64 inner values (two stages of asynchronous copies), fragments come from ldmatrix (W transposed on the way), sums are
// 32-bit in mma.m16n8k16.  Packets beyond the last token, inner value or output are zero.
constexpr int CM = 64, CN = 64, CK = 64, C_ROW = CK * 2 + 16;       // padded rows: conflict-free ldmatrix

__device__ __forceinline__ void hp_cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void hp_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void hp_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void hp_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
head_product_tc_kernel(const bf16* __restrict__ x, int64_t x_row, int x_head, int x_off, const bf16* __restrict__ w,
                       bf16* __restrict__ out, int64_t out_row, int out_head, int out_off, const bf16* __restrict__ gate,
                       int64_t gate_row, int64_t n_tokens, int K, int N) {
    __shared__ __align__(16) unsigned char xs[2][CM * C_ROW];
    __shared__ __align__(16) unsigned char ws[2][CK * C_ROW];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.y, col0 = blockIdx.z * CN;
    const int64_t row0 = (int64_t)blockIdx.x * CM;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bf16* xh = x + (int64_t)head * x_head + x_off;
    const bf16* wh = w + (int64_t)head * K * N;
    const uint32_t xs_base = (uint32_t)__cvta_generic_to_shared(&xs[0][0]);
    const uint32_t ws_base = (uint32_t)__cvta_generic_to_shared(&ws[0][0]);

    auto issue = [&](int chunk, int stage) {
        const int k0 = chunk * CK;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int piece = tid + e * 128, r = piece >> 3, c = piece & 7;       // 8 packets of 8 values a row
            const uint32_t off = (uint32_t)(stage * CM * C_ROW + r * C_ROW + c * 16);
            if (row0 + r < n_tokens && k0 + c * 8 < K) hp_cp_async16(xs_base + off, xh + (row0 + r) * x_row + k0 + c * 8);
            else *reinterpret_cast<uint4*>(&xs[0][0] + off) = make_uint4(0, 0, 0, 0);
            if (k0 + r < K && col0 + c * 8 < N) hp_cp_async16(ws_base + off, wh + (int64_t)(k0 + r) * N + col0 + c * 8);
            else *reinterpret_cast<uint4*>(&ws[0][0] + off) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    const int chunks = (K + CK - 1) / CK;
    issue(0, 0);
    for (int c = 0; c < chunks; ++c) {
        const int stage = c & 1;
        if (c + 1 < chunks) {
            issue(c + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const uint32_t xa = xs_base + stage * CM * C_ROW + (warp * 16 + (lane & 15)) * C_ROW + (lane >> 4) * 16;
        const uint32_t wb = ws_base + stage * CK * C_ROW + ((lane & 7) + (((lane >> 3) & 1) << 3)) * C_ROW + (lane >> 4) * 16;
        const int steps = min(CK, K - c * CK + 15) >> 4;
        for (int kt = 0; kt < steps; ++kt) {
            uint32_t a[4];
            hp_ldmatrix_x4(a, xa + kt * 32);
#pragma unroll
            for (int n = 0; n < 8; n += 2) {
                uint32_t b[4];
                hp_ldmatrix_x4_trans(b, wb + kt * 16 * C_ROW + n * 16);
                hp_mma_bf16(acc[n], a, b[0], b[1]);
                hp_mma_bf16(acc[n + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();            // the stage may be overwritten by the next issue
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int64_t r = row0 + warp * 16 + (lane >> 2) + half * 8;
        if (r >= n_tokens) continue;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int cc = col0 + n * 8 + (lane & 3) * 2;
            if (cc >= N) continue;
            float v0 = acc[n][half * 2], v1 = acc[n][half * 2 + 1];
            if (gate != nullptr) {
                const bf16* g = gate + r * gate_row + (int64_t)head * N + cc;
                v0 = v0 / (1.0f + expf(-__bfloat162float(g[0])));
                v1 = v1 / (1.0f + expf(-__bfloat162float(g[1])));
            }
            *reinterpret_cast<__nv_bfloat162*>(out + r * out_row + (int64_t)head * out_head + out_off + cc) = __floats2bfloat162_rn(v0, v1);
        }
    }
}

// whether the tensor-core form can take these operands: 16-byte packets of x and W, pairs of outputs
template <typename T>
static bool head_product_tiles(const void*, int64_t, int, int, const void*, const void*, int64_t, int, int, int, int) { return false; }
template <>
bool head_product_tiles<bf16>(const void* x, int64_t x_row, int x_head, int x_off, const void* w, const void* out, int64_t out_row,
                              int out_head, int out_off, int K, int N) {
    return K % 8 == 0 && N % 8 == 0 && x_row % 8 == 0 && x_head % 8 == 0 && x_off % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
           ((uintptr_t)w & 15) == 0 && out_row % 2 == 0 && out_head % 2 == 0 && out_off % 2 == 0 && ((uintptr_t)out & 3) == 0;
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
        if (head_product_tiles<T>(x, x_row, x_head, x_off, w, out, out_row, out_head, out_off, K, N)) {                      \
            const dim3 tiles((unsigned)((n_tokens + CM - 1) / CM), heads, (N + CN - 1) / CN);                                \
            return (int)q3_launch(head_product_tc_kernel, tiles, dim3(128), 0, (cudaStream_t)stream, (const bf16*)x, x_row,  \
                                  x_head, x_off, (const bf16*)w, (bf16*)out, out_row, out_head, out_off, (const bf16*)gate,  \
                                  gate_row, n_tokens, K, N);                                                                 \
        }                                                                                                                   \
        const dim3 grid((unsigned)((n_tokens + TM - 1) / TM), heads, (N + TN - 1) / TN);                                     \
        return (int)q3_launch(head_product_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)x, x_row, x_head,  \
                              x_off, (const T*)w, (T*)out, out_row, out_head, out_off, (const T*)gate, gate_row, n_tokens, K, \
                              N);                                                                                           \
    }

Q3_LATENT_EXPORTS(f32, float)
Q3_LATENT_EXPORTS(bf16, bf16)
