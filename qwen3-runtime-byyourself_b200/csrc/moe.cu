// A routed feed-forward (mixture of experts) in five kernels, none of which needs the host to know how many
// tokens an expert received, so a step can be captured:
//
//   moe_route   : one block per token.  Router logits z = W_r h in 32-bit (ascending order of the sum),
//                 scores s = softmax(z) over all outputs, choice scores s + correction, restricted to the
//                 `keep` groups (of `count` equal groups of neighbours) whose best choice score is largest;
//                 the `top` largest choice scores win (ties: the lower index); the weights are their plain
//                 scores s.  The last `identity` outputs are experts without tensors whose output is the
//                 token itself: their weights are summed into id_weight[token].
//                 `by_logit` 1: the `top` largest logits win instead and the weights are the softmax over the chosen
//                 logits only; 2: the scores are sigmoid(z), each output by itself.  `group_pair`: a group's score is
//                 the sum of its two largest choice scores.  The weights are multiplied by `weight_scale`.  With `gate_out`, the router matrix has one more row after the outputs whose logit
//                 is no expert's: gate_out[token] = sigmoid(that logit), the weight of a shared expert.
//   moe_sort    : one block.  Counts the (token, choice) pairs of every real expert, lays the experts out one
//                 after the other (offsets) and gives every pair its place (slot_of_pair, pair_of_slot).
//   moe_up      : act[slot] = f(W_gate x, W_up x) for the pairs of each expert, a tile of TM pairs x 64
//                 columns per block; g = min(gate, limit), u = clamp(up, -limit, limit),
//                 f = g sigmoid(alpha g) (u + up_offset)  (limit = infinity, alpha = 1, up_offset = 0: SiLU(gate) * up).
//   moe_down    : y[slot] = W_down act[slot], the same tiling, 32-bit output.
//   moe_combine : out[token] = T( sum_k weight_k y[slot(token, k)] + id_weight h[token] + shared_w[token] shared[token] ),
//                 the last term for a shared expert that every token uses (may be absent).
//
// The products accumulate in 32-bit in ascending order of k whatever the tile a pair falls into, so a token's
// result does not depend on what else is in the step.  Float tiles run on fmaf; bfloat16 tiles on the tensor cores
// (mma.m16n8k16, see `mma` below) when the widths are multiples of 32, else on fmaf too.
#include "common.cuh"

namespace {

__device__ __forceinline__ bool aligned16_device(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int MAX_OUTPUTS = 1024;

template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, const T* __restrict__ w_router, const float* __restrict__ correction,
                 int* __restrict__ top_ids, float* __restrict__ top_w, float* __restrict__ id_weight, int hidden, int n_out,
                 int n_real, int top, int group_count, int group_keep, int by_logit, float* __restrict__ gate_out, int group_pair,
                 float weight_scale) {
    __shared__ float z[MAX_OUTPUTS];
    __shared__ float choice[MAX_OUTPUTS];
    __shared__ float group_best[MAX_OUTPUTS];
    __shared__ unsigned char group_kept[MAX_OUTPUTS];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const T* x = h + t * hidden;
    // a warp per router output; 16-byte packets when the rows allow it (the order of the sum is fixed either way)
    constexpr int VEC = Pack<T>::N;
    const bool packed = hidden % VEC == 0 && aligned16_device(x) && aligned16_device(w_router);
    const int n_rows = n_out + (gate_out != nullptr ? 1 : 0);
    for (int e = warp; e < n_rows; e += 8) {
        const T* w = w_router + (int64_t)e * hidden;
        float dot = 0.0f;
        if (packed) {
            for (int c = lane * VEC; c < hidden; c += 32 * VEC) {
                const Pack<T> wv = load_pack<T>(w + c), xv = load_pack<T>(x + c);
#pragma unroll
                for (int i = 0; i < VEC; ++i) dot = fmaf(wv.get(i), xv.get(i), dot);
            }
        } else {
            for (int c = lane; c < hidden; c += 32) dot = fmaf(to_f32<T>(w[c]), to_f32<T>(x[c]), dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) z[e] = dot;
    }
    __syncthreads();
    if (tid != 0) return;
    if (gate_out != nullptr) gate_out[t] = 1.0f / (1.0f + expf(-z[n_out]));
    if (by_logit == 1) {
        // the largest logits (ties: the lower index), weighted by the softmax over the chosen logits alone
        float best_z = 0.0f, sum = 0.0f;
        for (int e = 0; e < n_out; ++e) choice[e] = z[e];
        for (int k = 0; k < top; ++k) {
            int best = -1;
            for (int e = 0; e < n_out; ++e)
                if (choice[e] > -INFINITY && (best < 0 || choice[e] > choice[best])) best = e;
            if (best < 0) best = 0;
            if (k == 0) best_z = z[best];
            choice[best] = -INFINITY;
            const float w = expf(z[best] - best_z);
            top_ids[t * top + k] = best;
            top_w[t * top + k] = w;
            sum += w;
        }
        const float inv = 1.0f / sum;
        float idw = 0.0f;
        for (int k = 0; k < top; ++k) {
            top_w[t * top + k] *= inv;
            if (top_ids[t * top + k] >= n_real) idw += top_w[t * top + k];
        }
        id_weight[t] = idw;
        return;
    }
    if (by_logit == 2) {                         // every output's score by itself: sigmoid(z)
        for (int e = 0; e < n_out; ++e) {
            z[e] = 1.0f / (1.0f + expf(-z[e]));
            choice[e] = z[e] + correction[e];
        }
    } else {
        float m = -INFINITY, sum = 0.0f;
        for (int e = 0; e < n_out; ++e) m = fmaxf(m, z[e]);
        for (int e = 0; e < n_out; ++e) {
            z[e] = expf(z[e] - m);
            sum += z[e];
        }
        const float inv = 1.0f / sum;
        for (int e = 0; e < n_out; ++e) {
            z[e] *= inv;
            choice[e] = z[e] + correction[e];
        }
    }
    if (group_count > 1) {
        // a group's score is its best choice score, or (`group_pair`) the sum of its two best; the `keep` best groups
        // stay (of equal groups the earlier one)
        const int size = n_out / group_count;
        for (int g = 0; g < group_count; ++g) {
            float best = -INFINITY, second = -INFINITY;
            for (int e = 0; e < size; ++e) {
                const float c = choice[g * size + e];
                if (c > best) {
                    second = best;
                    best = c;
                } else if (c > second) {
                    second = c;
                }
            }
            group_best[g] = group_pair && size > 1 ? best + second : best;
            group_kept[g] = 0;
        }
        for (int k = 0; k < group_keep; ++k) {
            int best = -1;
            for (int g = 0; g < group_count; ++g)
                if (!group_kept[g] && (best < 0 || group_best[g] > group_best[best])) best = g;
            group_kept[best] = 1;
        }
        for (int e = 0; e < n_out; ++e)
            if (!group_kept[e / size]) choice[e] = -INFINITY;        // minus infinity, not 0: choice scores can be negative
    }
    float idw = 0.0f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        for (int e = 0; e < n_out; ++e)
            if (choice[e] > -INFINITY && (best < 0 || choice[e] > choice[best])) best = e;      // ties: the lower index
        if (best < 0) best = 0;                  // fewer candidates than `top` (the caller's sizes rule it out)
        choice[best] = -INFINITY;
        top_ids[t * top + k] = best;
        top_w[t * top + k] = z[best] * weight_scale;
        if (best >= n_real) idw += z[best] * weight_scale;
    }
    id_weight[t] = idw;
}

// counts [E + 1] (the last cell: pairs of identity experts), offsets [E + 1]
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ top_ids, int n_pairs, int n_real, int* __restrict__ offsets, int* __restrict__ slot_of_pair,
                int* __restrict__ pair_of_slot) {
    extern __shared__ int counts[];            // [n_real] counts, then [n_real + 1] running offsets
    int* start = counts + n_real;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < n_real; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_ids[p];
        if (e < n_real) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_real; ++e) {
            start[e] = run;
            offsets[e] = run;
            run += counts[e];
        }
        start[n_real] = run;
        offsets[n_real] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_real; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_ids[p];
        int slot = -1;
        if (e < n_real) {
            slot = start[e] + atomicAdd(&counts[e], 1);
            pair_of_slot[slot] = p;
        }
        slot_of_pair[p] = slot;
    }
}

// Which expert and which of its row tiles block `tile` works on; false: beyond the last tile.
template <int TM>
__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int n_real, int tile, int& expert, int& row0, int& rows) {
    int seen = 0;
    for (int e = 0; e < n_real; ++e) {
        const int n = offsets[e + 1] - offsets[e];
        const int tiles = (n + TM - 1) / TM;
        if (tile < seen + tiles) {
            expert = e;
            row0 = offsets[e] + (tile - seen) * TM;
            rows = min(TM, offsets[e + 1] - row0);
            return true;
        }
        seen += tiles;
    }
    return false;
}

constexpr int TN = 64, TK = 32;

// A tile of TM rows of X (gathered through `src_row`) times TN rows of W, accumulated over K in 32-bit on fmaf.
// 256 threads: thread (tx, ty) owns rows ty, ty + 16, ... (TM / 16 of them, at least 1 with TM = 8: ty < 8) and
// columns tx * 4 .. + 3.  DUAL: two weight matrices at once (gate and up).
template <typename T, int TM, bool DUAL>
__device__ __forceinline__ void tile_product(const T* __restrict__ X, int64_t x_stride, const int* src_row, int rows,
                                             const T* __restrict__ W0, const T* __restrict__ W1, int n_cols, int col0, int K,
                                             float (&acc0)[(TM + 15) / 16][4], float (&acc1)[(TM + 15) / 16][4], float* xs, float* ws0,
                                             float* ws1) {
    constexpr int RPT = (TM + 15) / 16;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
#pragma unroll
    for (int a = 0; a < RPT; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc0[a][b] = acc1[a][b] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += TK) {
        __syncthreads();
        for (int x = tid; x < TM * TK; x += 256) {
            const int rr = x / TK, kk = x % TK;
            xs[rr * (TK + 1) + kk] = (rr < rows && k0 + kk < K) ? to_f32<T>(X[(int64_t)src_row[rr] * x_stride + k0 + kk]) : 0.0f;
        }
        for (int x = tid; x < TN * TK; x += 256) {
            const int cc = x / TK, kk = x % TK;
            const bool ok = col0 + cc < n_cols && k0 + kk < K;
            ws0[cc * (TK + 1) + kk] = ok ? to_f32<T>(W0[(int64_t)(col0 + cc) * K + k0 + kk]) : 0.0f;
            if (DUAL) ws1[cc * (TK + 1) + kk] = ok ? to_f32<T>(W1[(int64_t)(col0 + cc) * K + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            float wv0[4], wv1[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                wv0[b] = ws0[(tx * 4 + b) * (TK + 1) + kk];
                if (DUAL) wv1[b] = ws1[(tx * 4 + b) * (TK + 1) + kk];
            }
#pragma unroll
            for (int a = 0; a < RPT; ++a) {
                const int rr = ty + a * 16;
                if (rr < TM) {
                    const float xv = xs[rr * (TK + 1) + kk];
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        acc0[a][b] = fmaf(xv, wv0[b], acc0[a][b]);
                        if (DUAL) acc1[a][b] = fmaf(xv, wv1[b], acc1[a][b]);
                    }
                }
            }
        }
    }
}

template <typename T, int TM>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gate_up, const int* __restrict__ offsets,
              const int* __restrict__ pair_of_slot, T* __restrict__ act, int n_real, int top, int hidden, int ff, float limit,
              float alpha, float up_offset) {
    __shared__ float xs[TM * (TK + 1)], ws0[TN * (TK + 1)], ws1[TN * (TK + 1)];
    __shared__ int src_row[TM];
    pdl_launch_dependents();
    pdl_wait();
    int expert, row0, rows;
    if (!find_tile<TM>(offsets, n_real, blockIdx.y, expert, row0, rows)) return;
    if (threadIdx.x < TM) src_row[threadIdx.x] = threadIdx.x < rows ? pair_of_slot[row0 + threadIdx.x] / top : 0;
    const int col0 = blockIdx.x * TN;
    const T* wg = w_gate_up + (int64_t)expert * 2 * ff * hidden;      // [gate rows; up rows] of the expert
    float g[(TM + 15) / 16][4], u[(TM + 15) / 16][4];
    tile_product<T, TM, true>(h, hidden, src_row, rows, wg, wg + (int64_t)ff * hidden, ff, col0, hidden, g, u, xs, ws0, ws1);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int a = 0; a < (TM + 15) / 16; ++a) {
        const int rr = ty + a * 16;
        if (rr >= rows || rr >= TM) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int c = col0 + tx * 4 + b;
            if (c >= ff) continue;
            const float gv = fminf(g[a][b], limit), uv = fminf(fmaxf(u[a][b], -limit), limit);
            act[(int64_t)(row0 + rr) * ff + c] = from_f32<T>(gv / (1.0f + expf(-alpha * gv)) * (uv + up_offset));
        }
    }
}

template <typename T, int TM>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ offsets, float* __restrict__ y,
                int n_real, int hidden, int ff) {
    __shared__ float xs[TM * (TK + 1)], ws0[TN * (TK + 1)];
    __shared__ int src_row[TM];
    pdl_launch_dependents();
    pdl_wait();
    int expert, row0, rows;
    if (!find_tile<TM>(offsets, n_real, blockIdx.y, expert, row0, rows)) return;
    if (threadIdx.x < TM) src_row[threadIdx.x] = row0 + min((int)threadIdx.x, rows - 1);
    const int col0 = blockIdx.x * TN;
    float acc[(TM + 15) / 16][4], unused[(TM + 15) / 16][4];
    tile_product<T, TM, false>(act, ff, src_row, rows, w_down + (int64_t)expert * hidden * ff, nullptr, hidden, col0, ff, acc, unused,
                               xs, ws0, nullptr);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int a = 0; a < (TM + 15) / 16; ++a) {
        const int rr = ty + a * 16;
        if (rr >= rows || rr >= TM) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int c = col0 + tx * 4 + b;
            if (c < hidden) y[(int64_t)(row0 + rr) * hidden + c] = acc[a][b];
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ h, const int* __restrict__ slot_of_pair,
                                   const float* __restrict__ top_w, const float* __restrict__ id_weight, T* __restrict__ out,
                                   int top, int hidden, const T* __restrict__ shared, const float* __restrict__ shared_w) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const float idw = id_weight[t];
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = idw != 0.0f ? idw * to_f32<T>(h[t * hidden + c]) : 0.0f;
        for (int k = 0; k < top; ++k) {
            const int slot = slot_of_pair[t * top + k];
            if (slot >= 0) v = fmaf(top_w[t * top + k], y[(int64_t)slot * hidden + c], v);
        }
        if (shared != nullptr) v = fmaf(shared_w[t], to_f32<T>(shared[t * hidden + c]), v);
        out[t * hidden + c] = from_f32<T>(v);
    }
}

// ---------------------------------------------------------------- the same two products on the tensor cores (bfloat16)
// A block of 8 warps owns 64 pairs x 64 columns (of gate AND up in the first product): warp w works on rows
// 16 (w % 4) .. + 15 and columns 32 (w / 4) .. + 31 with mma.m16n8k16 (bfloat16 in, 32-bit accumulators).  X rows
// (gathered through the pairs' token numbers) and W rows arrive as 16-byte asynchronous copies into a ring of four
// stages of 32 k-values, so a block keeps three stages in flight: with a handful of pairs per expert (a decode step)
// the kernel streams each chosen expert's weights once.  Widths in steps of 32.
namespace mma {
constexpr int BM = 64, BN = 64, BK = 32, STAGES = 4;
constexpr int ROW = (BK + 8) * 2;                       // bytes of a padded tile row: ldmatrix without bank conflicts
constexpr int TILE = BM * ROW;                          // one 64 x 32 tile
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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc0 (and acc1 with DUAL) [n-tile][4] of this warp: rows quad and quad + 8 of its 16, columns n * 8 + tq * 2, + 1 of its 32.
template <bool DUAL>
__device__ __forceinline__ void tile_product(const bf16* __restrict__ X, int64_t x_stride, const int* src_row, const bf16* __restrict__ W0,
                                             const bf16* __restrict__ W1, int n_cols, int col0, int K, unsigned char* smem,
                                             float (&acc0)[4][4], float (&acc1)[4][4]) {
    constexpr int MATS = DUAL ? 3 : 2;                  // tiles per stage: X, W0 (, W1)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = smem_u32(smem);
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc0[n][e] = acc1[n][e] = 0.0f;
    // this thread's copy per tile and stage: row tid / 4, 16-byte chunk tid % 4
    const int lr = tid >> 2, lc = tid & 3;
    const bf16* x_src = X + (int64_t)src_row[lr] * x_stride + lc * 8;
    const int w_row = min(col0 + lr, n_cols - 1);       // a row beyond the matrix reads the last one; its results are dropped
    const bf16* w0_src = W0 + (int64_t)w_row * K + lc * 8;
    const bf16* w1_src = DUAL ? W1 + (int64_t)w_row * K + lc * 8 : nullptr;
    const uint32_t dst = lr * ROW + lc * 16;
    const int nk = K / BK;
    auto issue = [&](int kb) {
        if (kb < nk) {
            const uint32_t stage = base + (kb % STAGES) * (MATS * TILE) + dst;
            cp_async16(stage, x_src + kb * BK);
            cp_async16(stage + TILE, w0_src + kb * BK);
            if (DUAL) cp_async16(stage + 2 * TILE, w1_src + kb * BK);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    const int m0 = (warp & 3) * 16, n0 = (warp >> 2) * 32;
    const int krow = (lane & 7) + ((lane >> 4) << 3);
    for (int kb = 0; kb < nk; ++kb) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                // stage kb has landed for every thread; stage kb - 1 is free
        issue(kb + STAGES - 1);
        const uint32_t xs = base + (kb % STAGES) * (MATS * TILE);
        const uint32_t ws0 = xs + TILE, ws1 = ws0 + TILE;
#pragma unroll
        for (int kt = 0; kt < BK / 16; ++kt) {
            uint32_t a[4];                              // rows 0-7 and 8-15 of the warp's 16, k 0-7 and 8-15 of the step
            ldmatrix_x4(a, xs + (m0 + (lane & 15)) * ROW + (kt * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                uint32_t b[4];
                const uint32_t off = (n0 + jp * 16 + krow) * ROW + (2 * kt + ((lane >> 3) & 1)) * 16;
                ldmatrix_x4(b, ws0 + off);
                mma_bf16(acc0[2 * jp], a, b[0], b[1]);
                mma_bf16(acc0[2 * jp + 1], a, b[2], b[3]);
                if (DUAL) {
                    ldmatrix_x4(b, ws1 + off);
                    mma_bf16(acc1[2 * jp], a, b[0], b[1]);
                    mma_bf16(acc1[2 * jp + 1], a, b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
}

__global__ void __launch_bounds__(256)
moe_up_kernel(const bf16* __restrict__ h, const bf16* __restrict__ w_gate_up, const int* __restrict__ offsets,
              const int* __restrict__ pair_of_slot, bf16* __restrict__ act, int n_real, int top, int hidden, int ff, float limit,
              float alpha, float up_offset) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int src_row[BM];
    pdl_launch_dependents();
    pdl_wait();
    int expert, row0, rows;
    if (!find_tile<BM>(offsets, n_real, blockIdx.y, expert, row0, rows)) return;
    if (threadIdx.x < BM) src_row[threadIdx.x] = pair_of_slot[row0 + min((int)threadIdx.x, rows - 1)] / top;
    __syncthreads();
    const int col0 = blockIdx.x * BN;
    const bf16* wg = w_gate_up + (int64_t)expert * 2 * ff * hidden;
    float g[4][4], u[4][4];
    tile_product<true>(h, hidden, src_row, wg, wg + (int64_t)ff * hidden, ff, col0, hidden, smem, g, u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int rr = (warp & 3) * 16 + quad + (e >> 1) * 8, c = col0 + (warp >> 2) * 32 + n * 8 + tq * 2 + (e & 1);
            if (rr < rows && c < ff) {
                const float gv = fminf(g[n][e], limit), uv = fminf(fmaxf(u[n][e], -limit), limit);
                act[(int64_t)(row0 + rr) * ff + c] = __float2bfloat16_rn(gv / (1.0f + expf(-alpha * gv)) * (uv + up_offset));
            }
        }
}

__global__ void __launch_bounds__(256)
moe_down_kernel(const bf16* __restrict__ act, const bf16* __restrict__ w_down, const int* __restrict__ offsets, float* __restrict__ y,
                int n_real, int hidden, int ff) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int src_row[BM];
    pdl_launch_dependents();
    pdl_wait();
    int expert, row0, rows;
    if (!find_tile<BM>(offsets, n_real, blockIdx.y, expert, row0, rows)) return;
    if (threadIdx.x < BM) src_row[threadIdx.x] = row0 + min((int)threadIdx.x, rows - 1);
    __syncthreads();
    const int col0 = blockIdx.x * BN;
    float acc[4][4], unused[4][4];
    tile_product<false>(act, ff, src_row, w_down + (int64_t)expert * hidden * ff, nullptr, hidden, col0, ff, smem, acc, unused);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int rr = (warp & 3) * 16 + quad + (e >> 1) * 8, c = col0 + (warp >> 2) * 32 + n * 8 + tq * 2 + (e & 1);
            if (rr < rows && c < hidden) y[(int64_t)(row0 + rr) * hidden + c] = acc[n][e];
        }
}

int experts_launch(const bf16* h, const bf16* w_gate_up, const bf16* w_down, const int* offsets, const int* pair_of_slot, bf16* act,
                   float* y, int n_pairs, int n_real, int top, int hidden, int ff, float limit, float alpha, float up_offset, cudaStream_t stream) {
    const int tiles = (n_pairs + BM - 1) / BM + n_real;          // an upper bound on the row tiles of all experts together
    if (tiles > 65535) return Q3_ERR_TOO_LARGE;
    static Q3PerDevice up_ok, down_ok;
    cudaError_t e = q3_allow_shared_memory(moe_up_kernel, STAGES * 3 * TILE, up_ok);
    if (e == cudaSuccess) e = q3_allow_shared_memory(moe_down_kernel, STAGES * 2 * TILE, down_ok);
    if (e != cudaSuccess) return (int)e;
    int code = (int)q3_launch(moe_up_kernel, dim3((ff + BN - 1) / BN, tiles), dim3(256), STAGES * 3 * TILE, stream, h, w_gate_up,
                              offsets, pair_of_slot, act, n_real, top, hidden, ff, limit, alpha, up_offset);
    if (code != 0) return code;
    return (int)q3_launch(moe_down_kernel, dim3((hidden + BN - 1) / BN, tiles), dim3(256), STAGES * 2 * TILE, stream, act, w_down,
                          offsets, y, n_real, hidden, ff);
}
}  // namespace mma

template <typename T, int TM>
int moe_experts_launch(const T* h, const T* w_gate_up, const T* w_down, const int* offsets, const int* pair_of_slot, T* act, float* y,
                       int n_pairs, int n_real, int top, int hidden, int ff, float limit, float alpha, float up_offset, cudaStream_t stream) {
    const int tiles = (n_pairs + TM - 1) / TM + n_real;         // an upper bound on the row tiles of all experts together
    if (tiles > 65535) return Q3_ERR_TOO_LARGE;
    int code = (int)q3_launch(moe_up_kernel<T, TM>, dim3((ff + TN - 1) / TN, tiles), dim3(256), 0, stream, h, w_gate_up, offsets,
                              pair_of_slot, act, n_real, top, hidden, ff, limit, alpha, up_offset);
    if (code != 0) return code;
    return (int)q3_launch(moe_down_kernel<T, TM>, dim3((hidden + TN - 1) / TN, tiles), dim3(256), 0, stream, act, w_down, offsets, y,
                          n_real, hidden, ff);
}

}  // namespace

#define Q3_MOE_EXPORTS(SUFFIX, T)                                                                                         \
    Q3_EXPORT int q3_moe_route_##SUFFIX(const void* h, const void* w_router, const float* correction, int* top_ids,       \
                                        float* top_w, float* id_weight, int64_t n_tokens, int hidden, int n_out, int n_real, \
                                        int top, int group_count, int group_keep, int by_logit, float* gate_out,           \
                                        int group_pair, float weight_scale, void* stream) {                                                                   \
        if (n_tokens <= 0) return 0;                                                                                      \
        if (n_out <= 0 || n_out >= MAX_OUTPUTS || top <= 0 || top > n_out || n_real < 0 || n_real > n_out || \
            group_count <= 0 || n_out % group_count != 0 || group_keep <= 0 || group_keep > group_count ||                \
            n_tokens > 0x7fffffffLL)                                                                                      \
            return Q3_ERR_BAD_SIZE;                                                                                       \
        return (int)q3_launch(moe_route_kernel<T>, dim3((unsigned)n_tokens), dim3(256), 0, (cudaStream_t)stream,          \
                              (const T*)h, (const T*)w_router, correction, top_ids, top_w, id_weight, hidden, n_out,      \
                              n_real, top, group_count, group_keep, by_logit, gate_out, group_pair, weight_scale);        \
    }                                                                                                                     \
    Q3_EXPORT int q3_moe_experts_##SUFFIX(const void* h, const void* w_gate_up, const void* w_down, const int* offsets,   \
                                          const int* pair_of_slot, void* act, float* y, int n_pairs, int n_real, int top, \
                                          int hidden, int ff, float limit, float alpha, float up_offset, void* stream) {                   \
        if (n_pairs <= 0 || n_real <= 0) return 0;                                                                        \
        if (n_pairs <= 64)                                                                                                \
            return moe_experts_launch<T, 8>((const T*)h, (const T*)w_gate_up, (const T*)w_down, offsets, pair_of_slot,    \
                                            (T*)act, y, n_pairs, n_real, top, hidden, ff, limit, alpha, up_offset,                   \
                                            (cudaStream_t)stream);                                                        \
        return moe_experts_launch<T, 32>((const T*)h, (const T*)w_gate_up, (const T*)w_down, offsets, pair_of_slot,       \
                                         (T*)act, y, n_pairs, n_real, top, hidden, ff, limit, alpha, up_offset, (cudaStream_t)stream); \
    }                                                                                                                     \
    Q3_EXPORT int q3_moe_combine_##SUFFIX(const float* y, const void* h, const int* slot_of_pair, const float* top_w,     \
                                          const float* id_weight, void* out, int64_t n_tokens, int top, int hidden,       \
                                          const void* shared, const float* shared_w, void* stream) {                      \
        if (n_tokens <= 0) return 0;                                                                                      \
        if (n_tokens > 0x7fffffffLL) return Q3_ERR_BAD_SIZE;                                                              \
        return (int)q3_launch(moe_combine_kernel<T>, dim3((unsigned)n_tokens), dim3(hidden >= 1024 ? 256 : 128), 0,       \
                              (cudaStream_t)stream, y, (const T*)h, slot_of_pair, top_w, id_weight, (T*)out, top, hidden, \
                              (const T*)shared, shared_w);                                                                \
    }

Q3_EXPORT int q3_moe_sort(const int* top_ids, int n_pairs, int n_real, int* offsets, int* slot_of_pair, int* pair_of_slot,
                          void* stream) {
    if (n_pairs <= 0) return 0;
    if (n_real < 0 || n_real > 4096) return Q3_ERR_BAD_SIZE;
    return (int)q3_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(2 * n_real + 1) * sizeof(int), (cudaStream_t)stream, top_ids,
                          n_pairs, n_real, offsets, slot_of_pair, pair_of_slot);
}

// bfloat16 with both widths in steps of 32 (and 16-byte aligned rows): the tensor-core tiles; else the fmaf tiles.
Q3_EXPORT int q3_moe_experts_tc_bf16(const void* h, const void* w_gate_up, const void* w_down, const int* offsets,
                                     const int* pair_of_slot, void* act, float* y, int n_pairs, int n_real, int top, int hidden, int ff,
                                     float limit, float alpha, float up_offset, void* stream) {
    if (n_pairs <= 0 || n_real <= 0) return 0;
    if (hidden % 32 != 0 || ff % 32 != 0 || hidden <= 0 || ff <= 0) return Q3_ERR_BAD_SIZE;
    if (!aligned16(h) || !aligned16(w_gate_up) || !aligned16(w_down) || !aligned16(act)) return Q3_ERR_MISALIGNED;
    return mma::experts_launch((const bf16*)h, (const bf16*)w_gate_up, (const bf16*)w_down, offsets, pair_of_slot, (bf16*)act, y, n_pairs,
                               n_real, top, hidden, ff, limit, alpha, up_offset, (cudaStream_t)stream);
}

Q3_MOE_EXPORTS(f32, float)
Q3_MOE_EXPORTS(bf16, bf16)
