// Grouped-query attention over the paged cache (bfloat16, dots on the tensor cores) for mixers whose
// scores are capped smoothly, whose queries read only the keys of their own chunk of positions, whose
// softmax has a sink, and whose values may have another size than their keys:
//
//     s_j = cap * tanh(q.k_j * scale / cap)         (cap = 0: s_j = q.k_j * scale)
//     j visible from i:  j <= i  and  floor(j / chunk) == floor(i / chunk)       (chunk = 0: j <= i)
//                        or, with a window: j <= i  and  (i - j < window  or  j < keep), keep the number of first keys
//                        of a sequence that stay visible (their pages are walked before the window's)
//     p_j = exp(s_j) / (sink + sum_visible exp(s_j)),  sink = 1 or 0
//     o   = sum_j p_j v_j
//
// Scores, the softmax and its weights are 32-bit.  The weights enter the P.V product as two bfloat16 terms,
// p = hi + lo with hi = bf16(p) and lo = bf16(p - hi), so that the product sees them to 16 bits of mantissa
// instead of 8: two tensor-core instructions per tile where a kernel with rounded weights needs one.
// The sink is a key of score 0 without a value: the running maximum starts at 0 and the running sum at 1.
//
// Two kernels share the tile code:
//   prompts  grid (query tile, query head, sequence): 64 new tokens of a sequence (16 rows a warp) walk the
//            pages from the first page of the tile's first chunk to the page of its last row; K and V panels
//            of a page are double-buffered through cp.async.
//   decode   grid (split, kv head, token): the query heads of a kv group are the rows of one m16n8k16 tile;
//            a block takes a range of the pages between the chunk's start and the token, each of its four
//            warps 16 keys of every page through its own cp.async pipeline; partial results (sums, maximum,
//            denominator) go to a float32 scratch and a second small kernel merges the splits, adds the sink
//            and divides.  The fused form takes the output of the q/k/v projection as it is: every block adds
//            the bias to the group's query heads and rotates them itself, and the block that holds the token's
//            own page does the same for the new key and value, writes them into the cache and adds their term
//            to its partial result directly (the page was asked for before they were written).
// Compiled for one pair of sizes: -DQ3_HEAD_DIM=<keys> -DQ3_VALUE_DIM=<values>, multiples of 16 up to 256.
#include "common.cuh"

#ifndef Q3_HEAD_DIM
#error "compile with -DQ3_HEAD_DIM=<head size>"
#endif
#ifndef Q3_VALUE_DIM
#define Q3_VALUE_DIM Q3_HEAD_DIM
#endif

namespace {

constexpr int D = Q3_HEAD_DIM, VD = Q3_VALUE_DIM;
constexpr int PAGE = Q3_PAGE_TOKENS;
static_assert(PAGE == 64, "the tiled attention takes pages of 64 keys");
static_assert(D % 16 == 0 && D >= 16 && D <= 256 && VD % 16 == 0 && VD >= 16 && VD <= 256, "head sizes: multiples of 16 up to 256");
constexpr int WARPS = 4;
constexpr int K_ROW = D * 2 + 16, V_ROW = VD * 2 + 16;       // padded rows: conflict-free ldmatrix
constexpr int KT = D / 16, NT = VD / 8;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two weights as the bfloat16 pair (hi) and what the rounding dropped (lo).
__device__ __forceinline__ void split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - __low2float(h), b - __high2float(h));
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The score in the softmax's base-2 scale: (cap * tanh(dot * scale / cap)) * log2(e).  tanh(x) = 1 - 2 / (e^2x + 1):
// absolute error about 1e-7 (of the cap), at both ends exactly +-1.
__device__ __forceinline__ float score_log2(float dot, float scale, float cap, float inv_cap) {
    float v = dot * scale;
    if (cap > 0.0f) {
        const float e = __expf(2.0f * v * inv_cap);
        v = cap * (1.0f - __fdividef(2.0f, e + 1.0f));
    }
    return v * LOG2E;
}

// The first key position `pos` sees.  `chunk` > 0: the start of its chunk; `chunk` < 0 stands for a sliding window of
// -chunk keys (itself and the -chunk - 1 before it); 0: every key.  It never decreases with `pos`.
__device__ __forceinline__ int chunk_start(int pos, int chunk) {
    return chunk > 0 ? pos / chunk * chunk : (chunk < 0 ? max(pos + chunk + 1, 0) : 0);
}

template <typename TO> __device__ __forceinline__ void store_pair(TO* p, float a, float b);
template <> __device__ __forceinline__ void store_pair<bf16>(bf16* p, float a, float b) {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16(a, b);
}
template <> __device__ __forceinline__ void store_pair<float>(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}

template <int ROWS, int COLS, int ROW_BYTES, int THREADS>
__device__ __forceinline__ void load_rows(uint32_t dst, const bf16* src, int tid) {
    constexpr int CHUNKS = COLS / 8;
#pragma unroll
    for (int i = tid; i < ROWS * CHUNKS; i += THREADS) {
        const int row = i / CHUNKS, c = i % CHUNKS;
        cp_async16(dst + row * ROW_BYTES + c * 16, src + row * COLS + c * 8);
    }
}

// ---------------------------------------------------------------------------------------------- prompts
constexpr int BM = 64;
constexpr int K_TILE = PAGE * K_ROW, V_TILE = PAGE * V_ROW;
constexpr int PREFILL_SMEM = 2 * (K_TILE + V_TILE);

template <typename TO>
__global__ void __launch_bounds__(WARPS * 32)
prefill_capped_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                      TO* __restrict__ out, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                      const int* __restrict__ page_table, int pages_per_seq, int nq, int nkv, float scale, float cap, int chunk,
                      int sink, int nv, const float* __restrict__ sink_values, int keep) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int t0 = seq_start[seq], n_new = seq_start[seq + 1] - t0;
    if (tile * BM >= n_new) return;
    const int kvh = head / (nq / nkv), vh = kvh / (nkv / nv);      // nv value heads, each shared by nkv / nv key heads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
    const int pos0 = seq_pos0[seq];
    const int* pages = page_table + (int64_t)seq * pages_per_seq;
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    // this warp's 16 rows; rows beyond the sequence's new tokens are computed on row 0's data and dropped
    const int r_lo = tile * BM + warp * 16 + quad, r_hi = r_lo + 8;
    const bool ok_lo = r_lo < n_new, ok_hi = r_hi < n_new;
    const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;                          // absolute positions
    const int c_lo = chunk_start(p_lo, chunk), c_hi = chunk_start(p_hi, chunk);   // first visible key of each row
    uint32_t qa[KT][4];
    {
        const bf16* q_lo = q + ((int64_t)(t0 + (ok_lo ? r_lo : 0)) * nq + head) * D;
        const bf16* q_hi = q + ((int64_t)(t0 + (ok_hi ? r_hi : 0)) * nq + head) * D;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            const int c = kt * 16 + tq * 2;
            qa[kt][0] = *reinterpret_cast<const uint32_t*>(q_lo + c);
            qa[kt][1] = *reinterpret_cast<const uint32_t*>(q_hi + c);
            qa[kt][2] = *reinterpret_cast<const uint32_t*>(q_lo + c + 8);
            qa[kt][3] = *reinterpret_cast<const uint32_t*>(q_hi + c + 8);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    const float m0 = sink ? (sink_values ? sink_values[head] * LOG2E : 0.0f) : -INFINITY, l0 = sink ? 1.0f : 0.0f;   // base-2 scale
    float m_run[2] = {m0, m0}, l_run[2] = {l0, l0};

    const int last_row = min(tile * BM + BM, n_new) - 1;
    const int pg_begin = chunk_start(pos0 + tile * BM, chunk) / PAGE, pg_end = (pos0 + last_row) / PAGE + 1;
    // with a window, the first `keep` keys of the sequence stay visible: the pages that hold them and lie before the
    // window's come first; step i of the walk is page i if i < n_keep, else page pg_begin + i - n_keep
    const int n_keep = min((keep + PAGE - 1) / PAGE, pg_begin), n_walk = n_keep + pg_end - pg_begin;
    const int warp_first_pos = pos0 + tile * BM + warp * 16;                   // lowest position of the warp's rows
    const int warp_first_key = chunk_start(warp_first_pos, chunk);             // no row of the warp sees a key before it
    const int warp_last_start = chunk_start(warp_first_pos + 15, chunk);       // from here on every row of the warp may see
    const uint32_t base = smem_u32(smem);

    auto issue = [&](int i) {
        if (i < n_walk) {
            const int pg = i < n_keep ? i : pg_begin + i - n_keep;
            const int64_t k_at = ((int64_t)pages[pg] * nkv + kvh) * PAGE, v_at = ((int64_t)pages[pg] * nv + vh) * PAGE;
            const uint32_t dst = base + (i & 1) * (K_TILE + V_TILE);
            load_rows<PAGE, D, K_ROW, WARPS * 32>(dst, k_pages + k_at * D, threadIdx.x);
            load_rows<PAGE, VD, V_ROW, WARPS * 32>(dst + K_TILE, v_pages + v_at * VD, threadIdx.x);
        }
        cp_async_commit();
    };
    issue(0);
    for (int i = 0; i < n_walk; ++i) {
        issue(i + 1);               // into the other stage, which every warp left before the last barrier
        cp_async_wait<1>();
        __syncthreads();
        const int pg = i < n_keep ? i : pg_begin + i - n_keep;
        const uint32_t kbuf = base + (i & 1) * (K_TILE + V_TILE), vbuf = kbuf + K_TILE;
        const int key_base = pg * PAGE;
        // a warp whose rows all lie before this page, or whose chunks all start behind it, has nothing to see in it
        // (but for the kept keys)
        if (key_base <= warp_first_pos + 15 && (key_base + PAGE > warp_first_key || key_base < keep)) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
            const int krow = (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
            for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {       // pairs of 8-key tiles
                    uint32_t b[4];
                    ldmatrix_x4(b, kbuf + (jp * 16 + krow) * K_ROW + (2 * kt + ((lane >> 3) & 1)) * 16);
                    mma_bf16(s[2 * jp], qa[kt], b[0], b[1]);
                    mma_bf16(s[2 * jp + 1], qa[kt], b[2], b[3]);
                }
            }
            const bool edge = key_base + PAGE - 1 > warp_first_pos || key_base < warp_last_start;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = score_log2(s[j][e], scale, cap, inv_cap);
                    if (edge) {
                        const int key = key_base + j * 8 + tq * 2 + (e & 1);
                        const bool seen = (e >> 1) ? (key <= p_hi && (key >= c_hi || key < keep)) : (key <= p_lo && (key >= c_lo || key < keep));
                        v = seen ? v : -INFINITY;
                    }
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                m_use[r] = m_new == -INFINITY ? 0.0f : m_new;
                alpha[r] = exp2f(m_run[r] - m_use[r]);
                m_run[r] = m_new;
            }
            float sum[2] = {0.0f, 0.0f};
            uint32_t pa[4][4], pb[4][4];               // the weights as hi and lo bfloat16 terms
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
                const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
                sum[0] += p0 + p1;
                sum[1] += p2 + p3;
                split_bf16(p0, p1, pa[j >> 1][(j & 1) * 2 + 0], pb[j >> 1][(j & 1) * 2 + 0]);
                split_bf16(p2, p3, pa[j >> 1][(j & 1) * 2 + 1], pb[j >> 1][(j & 1) * 2 + 1]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                l_run[r] = l_run[r] * alpha[r] + sum[r];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
            const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {            // 16 keys at a time
#pragma unroll
                for (int n = 0; n < NT; n += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vbuf + (kk * 16 + vrow) * V_ROW + (n + (lane >> 4)) * 16);
                    mma_bf16(o[n], pa[kk], b[0], b[1]);
                    mma_bf16(o[n + 1], pa[kk], b[2], b[3]);
                    mma_bf16(o[n], pb[kk], b[0], b[1]);
                    mma_bf16(o[n + 1], pb[kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();            // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();

    const float inv_lo = 1.0f / l_run[0], inv_hi = 1.0f / l_run[1];
    TO* o_lo = out + ((int64_t)(t0 + r_lo) * nq + head) * VD;
    TO* o_hi = out + ((int64_t)(t0 + r_hi) * nq + head) * VD;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int c = n * 8 + tq * 2;
        if (ok_lo) store_pair<TO>(o_lo + c, o[n][0] * inv_lo, o[n][1] * inv_lo);
        if (ok_hi) store_pair<TO>(o_hi + c, o[n][2] * inv_hi, o[n][3] * inv_hi);
    }
}

// ---------------------------------------------------------------------------------------------- decode
constexpr int KEYS_PER_WARP = PAGE / WARPS;        // 16
constexpr int K_PANEL = KEYS_PER_WARP * K_ROW, V_PANEL = KEYS_PER_WARP * V_ROW;
constexpr int STAGES = 3;
constexpr int DECODE_PIPE = WARPS * STAGES * (K_PANEL + V_PANEL);
constexpr int DECODE_MERGE = WARPS * 16 * (VD + 2) * 4;
constexpr int DECODE_SMEM = DECODE_PIPE > DECODE_MERGE ? DECODE_PIPE : DECODE_MERGE;

// the fused form keeps, behind the pipeline: the prepared queries [16][D], the new key [D] and value [VD] (bf16) and
// the new key's scores [16] (float32)
constexpr int DECODE_PREP = (16 * D + D + VD) * 2 + 16 * 4;
constexpr int DECODE_SMEM_FUSED = DECODE_SMEM + DECODE_PREP;

// What the fused form needs beyond the split form's arguments.
struct FusedArgs {
    const bf16* qkv;               // [tokens, (nq + nkv) * D + nkv * VD]: the projection output as it is
    const float* bias;             // one value per column of it, or null
    const float* cos_tab;          // [positions, rot / 2] or null
    const float* sin_tab;
    int rot;                       // the first `rot` values of a query or key head are rotated in pairs (i, i + rot/2)
};

// One head of the projection output with its bias added and (if `cos_tab`) rotated, by one warp, exactly as
// qkv_prepare does it (attention.cu), so that the cache holds the same values whichever kernel wrote them.
template <int SIZE>
__device__ __forceinline__ void prepare_head(const bf16* __restrict__ src, const float* __restrict__ bias, bf16* dst,
                                             const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int pos,
                                             int rot, int lane) {
    const int rhalf = cos_tab != nullptr ? rot >> 1 : 0;
    for (int i = lane; i < rhalf; i += 32) {
        float a = __bfloat162float(src[i]), b = __bfloat162float(src[i + rhalf]);
        if (bias != nullptr) {
            a = round_to<bf16>(a + bias[i]);
            b = round_to<bf16>(b + bias[i + rhalf]);
        }
        const float cs = cos_tab[(int64_t)pos * rhalf + i], sn = sin_tab[(int64_t)pos * rhalf + i];
        dst[i] = __float2bfloat16_rn(a * cs - b * sn);
        dst[i + rhalf] = __float2bfloat16_rn(b * cs + a * sn);
    }
    for (int i = 2 * rhalf + lane; i < SIZE; i += 32) {
        float c = __bfloat162float(src[i]);
        if (bias != nullptr) c = round_to<bf16>(c + bias[i]);
        dst[i] = __float2bfloat16_rn(c);
    }
}

// part: [tokens, nq, splits, VD + 2] float32: the unnormalised sums, then the maximum (base-2 scale) and the denominator.
// FUSED: `q` is unused; the pages are written by the block that holds the token's own page.
template <bool FUSED>
__global__ void __launch_bounds__(WARPS * 32)
decode_capped_split_kernel(const bf16* __restrict__ q, const bf16* k_pages, const bf16* v_pages,
                           float* __restrict__ part, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                           const int* __restrict__ page_table, int pages_per_seq, int nq, int nkv, float scale, float cap,
                           int chunk, const FusedArgs fused, int nv, int keep) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int split = blockIdx.x, n_splits = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int G = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
    const int pos = token_pos[t];
    const int* pages = page_table + (int64_t)token_seq[t] * pages_per_seq;
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    const int lo = chunk_start(pos, chunk);
    // with a window, the pages of the first `keep` keys that lie before the window's pages are walked first: step x of
    // the walk is page x if x < n_keep, else page first_page + x - n_keep; the splits share the steps
    const int first_page = lo / PAGE, n_keep = min((keep + PAGE - 1) / PAGE, first_page);
    const int n_pages = n_keep + pos / PAGE + 1 - first_page;
    const int per_split = (n_pages + n_splits - 1) / n_splits;
    const int pg_begin = split * per_split;
    const int pg_end = min(n_pages, pg_begin + per_split);
    const int count = max(pg_end - pg_begin, 0);
    auto page_of = [&](int x) { return x < n_keep ? x : first_page + x - n_keep; };

    const uint32_t pipe = smem_u32(smem) + warp * (STAGES * (K_PANEL + V_PANEL));
    auto issue = [&](int i) {
        if (i < count) {
            const int page = pages[page_of(pg_begin + i)];
            const int64_t at = ((int64_t)page * nkv + kvh) * PAGE + warp * KEYS_PER_WARP;
            const int64_t v_at = ((int64_t)page * nv + kvh / (nkv / nv)) * PAGE + warp * KEYS_PER_WARP;
            const uint32_t dst = pipe + (i % STAGES) * (K_PANEL + V_PANEL);
            load_rows<KEYS_PER_WARP, D, K_ROW, 32>(dst, k_pages + at * D, lane);
            load_rows<KEYS_PER_WARP, VD, V_ROW, 32>(dst + K_PANEL, v_pages + v_at * VD, lane);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);

    // the block that holds the token's own page owns the new key and value
    const bool owner = FUSED && count > 0 && pg_end == n_pages;
    bf16* prep_q = reinterpret_cast<bf16*>(smem + DECODE_SMEM);          // [16][D]
    bf16* new_k = prep_q + 16 * D;                                       // [D]
    bf16* new_v = new_k + D;                                             // [VD]
    float* new_s = reinterpret_cast<float*>(new_v + VD);                 // [16]: the new key's scores, base-2 scale
    if constexpr (FUSED) {
        const int64_t width = (int64_t)(nq + nkv) * D + (int64_t)nkv * VD;
        const bf16* row = fused.qkv + (int64_t)t * width;
        for (int r = warp; r < G; r += WARPS) {
            const int64_t col = (int64_t)(kvh * G + r) * D;
            prepare_head<D>(row + col, fused.bias ? fused.bias + col : nullptr, prep_q + r * D, fused.cos_tab, fused.sin_tab, pos,
                            fused.rot, lane);
        }
        if (owner) {
            if (warp == G % WARPS) {
                const int64_t col = (int64_t)(nq + kvh) * D;
                prepare_head<D>(row + col, fused.bias ? fused.bias + col : nullptr, new_k, fused.cos_tab, fused.sin_tab, pos,
                                fused.rot, lane);
            }
            if (warp == (G + 1) % WARPS) {
                const int64_t col = (int64_t)(nq + nkv) * D + (int64_t)kvh * VD;
                prepare_head<VD>(row + col, fused.bias ? fused.bias + col : nullptr, new_v, nullptr, nullptr, pos, 0, lane);
            }
        }
        __syncthreads();
        if (owner) {       // into the cache for the steps to come; this step takes them from shared memory
            const int64_t at = ((int64_t)pages[pos / PAGE] * nkv + kvh) * PAGE + pos % PAGE;
            for (int i = threadIdx.x; i < D; i += WARPS * 32) const_cast<bf16*>(k_pages)[at * D + i] = new_k[i];
            for (int i = threadIdx.x; i < VD; i += WARPS * 32) const_cast<bf16*>(v_pages)[at * VD + i] = new_v[i];
            for (int r = warp; r < G; r += WARPS) {                      // q.k of the new key, as the tensor core would sum it
                float dot = 0.0f;
                for (int i = lane; i < D; i += 32) dot = fmaf(__bfloat162float(prep_q[r * D + i]), __bfloat162float(new_k[i]), dot);
                dot = warp_sum(dot);
                if (lane == 0) new_s[r] = score_log2(dot, scale, cap, inv_cap);
            }
        }
    }
    // in the fused form the token's own key is not in the page that was asked for: it is added at the merge
    const int last_key = FUSED ? pos - 1 : pos;

    // query rows of the group as A fragments: row r = head kvh*G + r (rows >= G are zero)
    uint32_t qa[KT][4];
    {
        const bf16* q0 = FUSED ? prep_q : q + ((int64_t)t * nq + (int64_t)kvh * G) * D;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            const int c = kt * 16 + tq * 2;
            qa[kt][0] = quad < G ? *reinterpret_cast<const uint32_t*>(q0 + quad * D + c) : 0u;
            qa[kt][1] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (quad + 8) * D + c) : 0u;
            qa[kt][2] = quad < G ? *reinterpret_cast<const uint32_t*>(q0 + quad * D + c + 8) : 0u;
            qa[kt][3] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (quad + 8) * D + c + 8) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};   // rows quad and quad + 8

    for (int i = 0; i < count; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        issue(i + STAGES - 1);      // its stage was consumed in iteration i - 1
        const uint32_t kbuf = pipe + (i % STAGES) * (K_PANEL + V_PANEL), vbuf = kbuf + K_PANEL;
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const int krow = (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            uint32_t b[4];
            ldmatrix_x4(b, kbuf + krow * K_ROW + (2 * kt + ((lane >> 3) & 1)) * 16);
            mma_bf16(s[0], qa[kt], b[0], b[1]);
            mma_bf16(s[1], qa[kt], b[2], b[3]);
        }
        // key index of s[j][e]: page*64 + warp*16 + j*8 + tq*2 + (e & 1); keys outside [lo, pos] are not seen
        const int key0 = page_of(pg_begin + i) * PAGE + warp * KEYS_PER_WARP + tq * 2;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + j * 8 + (e & 1);
                const float v = ((key >= lo || key < keep) && key <= last_key) ? score_log2(s[j][e], scale, cap, inv_cap) : -INFINITY;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            m_use[r] = m_new == -INFINITY ? 0.0f : m_new;      // a row that has seen no key yet
            alpha[r] = exp2f(m_run[r] - m_use[r]);
            m_run[r] = m_new;
        }
        float sum[2] = {0.0f, 0.0f};
        uint32_t pa[4], pb[4];
        {
            float p[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
                    sum[e >> 1] += p[j][e];
                }
            split_bf16(p[0][0], p[0][1], pa[0], pb[0]);
            split_bf16(p[0][2], p[0][3], pa[1], pb[1]);
            split_bf16(p[1][0], p[1][1], pa[2], pb[2]);
            split_bf16(p[1][2], p[1][3], pa[3], pb[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
            l_run[r] = l_run[r] * alpha[r] + sum[r];
        }
        const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vbuf + vrow * V_ROW + (n + (lane >> 4)) * 16);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                o[n + h][0] *= alpha[0]; o[n + h][1] *= alpha[0];
                o[n + h][2] *= alpha[1]; o[n + h][3] *= alpha[1];
            }
            mma_bf16(o[n], pa, b[0], b[1]);
            mma_bf16(o[n + 1], pa, b[2], b[3]);
            mma_bf16(o[n], pb, b[0], b[1]);
            mma_bf16(o[n + 1], pb, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();     // every warp is done with the pipeline buffers: reuse them for the merge

    float* sm_o = reinterpret_cast<float*>(smem);             // [warp][row][VD]
    float* sm_ml = sm_o + WARPS * 16 * VD;                    // [warp][row][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = quad + 8 * r;
        if (tq == 0) {
            sm_ml[(warp * 16 + row) * 2 + 0] = m_run[r];
            sm_ml[(warp * 16 + row) * 2 + 1] = l_run[r];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n)
            *reinterpret_cast<float2*>(sm_o + (warp * 16 + row) * VD + n * 8 + tq * 2) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * VD; idx += WARPS * 32) {
        const int row = idx / VD, c = idx % VD;
        float m = owner ? new_s[row] : -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[(w * 16 + row) * 2]);
        float acc = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = sm_ml[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
            acc += f * sm_o[(w * 16 + row) * VD + c];
            l += f * sm_ml[(w * 16 + row) * 2 + 1];
        }
        if (owner) {                                   // the token's own key and value: one more term
            const float f = exp2f(new_s[row] - m);
            acc += f * __bfloat162float(new_v[c]);
            l += f;
        }
        float* dst = part + (((int64_t)t * nq + kvh * G + row) * n_splits + split) * (VD + 2);
        dst[c] = acc;
        if (c == 0) {
            dst[VD] = m;
            dst[VD + 1] = l;
        }
    }
}

// One block per (query head, token): the splits' partial results, the sink, the division.
template <typename TO>
__global__ void decode_capped_merge_kernel(const float* __restrict__ part, TO* __restrict__ out, int nq, int n_splits, int sink,
                                           const float* __restrict__ sink_values) {
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x;
    const int64_t t = blockIdx.y;
    const float* p = part + ((t * nq + head) * n_splits) * (VD + 2);
    const float sink_score = sink_values ? sink_values[head] * LOG2E : 0.0f;     // base-2 scale, as the splits' maxima
    float m = sink ? sink_score : -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, p[s * (VD + 2) + VD]);
    float l = sink ? exp2f(sink_score - m) : 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = p[s * (VD + 2) + VD];
        if (ms != -INFINITY) l += exp2f(ms - m) * p[s * (VD + 2) + VD + 1];
    }
    const float inv = 1.0f / l;
    for (int c = threadIdx.x; c < VD; c += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = p[s * (VD + 2) + VD];
            if (ms != -INFINITY) acc += exp2f(ms - m) * p[s * (VD + 2) + c];
        }
        out[(t * nq + head) * VD + c] = from_f32<TO>(acc * inv);
    }
}

}  // namespace

Q3_EXPORT int q3_attention_capped_head_dim() { return D; }
Q3_EXPORT int q3_attention_capped_value_dim() { return VD; }

// Prompts (or any mix of lengths): q [tokens, nq, D], out [tokens, nq, VD].
Q3_EXPORT int q3_attention_capped_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                               const int* seq_start, const int* seq_pos0, const int* page_table,
                                               int pages_per_seq, int n_seqs, int max_new, int nq, int nkv, float scale,
                                               float softcap, int chunk, int sink, int window, int value_heads, int out_f32,
                                               const float* sink_values, int keep_first, void* stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (keep_first < 0 || (keep_first > 0 && window <= 0)) return Q3_ERR_BAD_SIZE;
    if (value_heads <= 0) value_heads = nkv;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nkv % value_heads != 0 || softcap < 0.0f || chunk < 0 || window < 0 ||
        (chunk > 0 && window > 0))
        return Q3_ERR_BAD_SIZE;
    if (n_seqs > 65535 || nq > 65535) return Q3_ERR_TOO_LARGE;
    const int span = window > 0 ? -window : chunk;             // see chunk_start
    static Q3PerDevice configured[2];
    const dim3 grid((max_new + BM - 1) / BM, nq, n_seqs);
    if (out_f32) {
        cudaError_t e = q3_allow_shared_memory(prefill_capped_kernel<float>, PREFILL_SMEM, configured[1]);
        if (e != cudaSuccess) return (int)e;
        return (int)q3_launch(prefill_capped_kernel<float>, grid, dim3(WARPS * 32), PREFILL_SMEM, (cudaStream_t)stream, (const bf16*)q,
                              (const bf16*)k_pages, (const bf16*)v_pages, (float*)out, seq_start, seq_pos0, page_table,
                              pages_per_seq, nq, nkv, scale, softcap, span, sink, value_heads, sink_values, keep_first);
    }
    cudaError_t e = q3_allow_shared_memory(prefill_capped_kernel<bf16>, PREFILL_SMEM, configured[0]);
    if (e != cudaSuccess) return (int)e;
    return (int)q3_launch(prefill_capped_kernel<bf16>, grid, dim3(WARPS * 32), PREFILL_SMEM, (cudaStream_t)stream, (const bf16*)q,
                          (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, seq_start, seq_pos0, page_table,
                          pages_per_seq, nq, nkv, scale, softcap, span, sink, value_heads, sink_values, keep_first);
}

// One new token per sequence: scratch holds n_tokens * nq * n_splits * (VD + 2) float32.
Q3_EXPORT int q3_attention_capped_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, float* scratch,
                                              const int* token_seq, const int* token_pos, const int* page_table,
                                              int pages_per_seq, int64_t n_tokens, int nq, int nkv, float scale, float softcap,
                                              int chunk, int sink, int n_splits, int window, int value_heads, int out_f32,
                                              const float* sink_values, int keep_first, void* stream) {
    if (n_tokens <= 0) return 0;
    if (keep_first < 0 || (keep_first > 0 && window <= 0)) return Q3_ERR_BAD_SIZE;
    if (value_heads <= 0) value_heads = nkv;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || nkv % value_heads != 0 || softcap < 0.0f || chunk < 0 ||
        window < 0 || (chunk > 0 && window > 0) || n_splits <= 0)
        return Q3_ERR_BAD_SIZE;
    const int span = window > 0 ? -window : chunk;             // see chunk_start
    if (n_tokens > 65535 || nkv > 65535 || nq > 0x7fffffff / 2) return Q3_ERR_TOO_LARGE;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(decode_capped_split_kernel<false>, DECODE_SMEM, configured);
        if (e != cudaSuccess) return (int)e;
    }
    FusedArgs none = {};
    cudaError_t e = q3_launch(decode_capped_split_kernel<false>, dim3(n_splits, nkv, (unsigned)n_tokens), dim3(WARPS * 32), DECODE_SMEM,
                              (cudaStream_t)stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, scratch, token_seq,
                              token_pos, page_table, pages_per_seq, nq, nkv, scale, softcap, span, none, value_heads, keep_first);
    if (e != cudaSuccess) return (int)e;
    if (out_f32)
        return (int)q3_launch(decode_capped_merge_kernel<float>, dim3(nq, (unsigned)n_tokens), dim3(VD >= 128 ? 128 : 64), 0,
                              (cudaStream_t)stream, (const float*)scratch, (float*)out, nq, n_splits, sink, sink_values);
    return (int)q3_launch(decode_capped_merge_kernel<bf16>, dim3(nq, (unsigned)n_tokens), dim3(VD >= 128 ? 128 : 64), 0,
                          (cudaStream_t)stream, (const float*)scratch, (bf16*)out, nq, n_splits, sink, sink_values);
}

// The same from the output of the q/k/v projection as it is, qkv [tokens, (nq + nkv) * D + nkv * VD]: the bias (may be null),
// the rotation of the first rotary_dim values of the query and key heads (tables [positions, rotary_dim / 2], may be null) and
// the write of the new key and value into their pages happen in the attention's own kernel.
Q3_EXPORT int q3_attention_capped_decode_fused_bf16(const void* qkv, void* k_pages, void* v_pages, void* out, float* scratch,
                                                    const float* bias, const float* cos_tab, const float* sin_tab, int rotary_dim,
                                                    const int* token_seq, const int* token_pos, const int* page_table,
                                                    int pages_per_seq, int64_t n_tokens, int nq, int nkv, float scale,
                                                    float softcap, int chunk, int sink, int n_splits, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || softcap < 0.0f || chunk < 0 || n_splits <= 0) return Q3_ERR_BAD_SIZE;
    if ((cos_tab == nullptr) != (sin_tab == nullptr) || rotary_dim < 0 || rotary_dim % 2 != 0 || rotary_dim > D) return Q3_ERR_BAD_SIZE;
    if (n_tokens > 65535 || nkv > 65535 || nq > 0x7fffffff / 2) return Q3_ERR_TOO_LARGE;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(decode_capped_split_kernel<true>, DECODE_SMEM_FUSED, configured);
        if (e != cudaSuccess) return (int)e;
    }
    FusedArgs fused;
    fused.qkv = (const bf16*)qkv; fused.bias = bias; fused.cos_tab = cos_tab; fused.sin_tab = sin_tab;
    fused.rot = rotary_dim > 0 ? rotary_dim : D;
    cudaError_t e = q3_launch(decode_capped_split_kernel<true>, dim3(n_splits, nkv, (unsigned)n_tokens), dim3(WARPS * 32),
                              DECODE_SMEM_FUSED, (cudaStream_t)stream, (const bf16*)nullptr, (const bf16*)k_pages, (const bf16*)v_pages,
                              scratch, token_seq, token_pos, page_table, pages_per_seq, nq, nkv, scale, softcap, chunk, fused, nkv, 0);
    if (e != cudaSuccess) return (int)e;
    return (int)q3_launch(decode_capped_merge_kernel<bf16>, dim3(nq, (unsigned)n_tokens), dim3(VD >= 128 ? 128 : 64), 0,
                          (cudaStream_t)stream, (const float*)scratch, (bf16*)out, nq, n_splits, sink, (const float*)nullptr);
}
