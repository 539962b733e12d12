// qwen3/kernels.h - the C interface of the library's sm_100a kernels, for host programs that drive them
// without Python.  Each group of entry points lives in a shared library of its own, built from the source
// named beside it (csrc/, nvcc -gencode arch=compute_100a,code=sm_100a); the attention libraries are
// compiled for one head size (-DQ3_HEAD_DIM=<multiple of 16>).
//
// Conventions, the same everywhere:
//   * pointers are device pointers unless a comment says otherwise; `stream` is a cudaStream_t;
//   * nothing allocates: scratch is passed in (q3_attention_decode_bf16_static keeps its own, see
//     csrc/attention_decode_static.h);
//   * the result is 0, a cudaError_t of the launch, or one of the argument errors below - a size the kernel
//     does not take is refused, never computed wrongly;
//   * matrices are row-major; weights are [out, in] and used as x . W^T; bfloat16 values are passed as
//     `void*`; rows of activations are contiguous;
//   * the cache is paged: k_pages / v_pages [pages, kv heads, 64 tokens, head size]; page_table [sequences,
//     pages_per_seq] lists a sequence's pages in order; token_seq / token_pos give every token's sequence and
//     position; seq_start [sequences + 1] and seq_pos0 [sequences] describe packed prompts;
//   * `status` is one int32 word on the device into which a kernel whose bounded wait ran out writes where it
//     gave up (0 = none); read it where the host waits for the device anyway.
//
// The reference's counterparts: src/ops/{embedding,rms_norm,rope,elementwise,gqa_attention,argmax}.cu, the
// cublasGemmEx call of src/ops/linear.cpp:165-193, the CPU sampler of src/generation/sampler.cpp:137-247.
#pragma once

#include <stdint.h>

#define Q3_ERR_BAD_SIZE 10001        /* a size the kernel does not take */
#define Q3_ERR_TOO_LARGE 10002       /* more rows, heads or blocks than one launch takes */
#define Q3_ERR_MISALIGNED 10003      /* a pointer or stride that is not 16-byte aligned */

#ifdef __cplusplus
extern "C" {
#endif

/* ---- elementwise.cu: float32 (`f32`) and bfloat16 (`bf16`) forms ---------------------------------------- */
/* out[t] = table[ids[t]] (a zero row for an id outside [0, vocab)) */
int q3_embedding_f32(const int* ids, const void* table, void* out, int64_t n_tokens, int hidden, int vocab, void* stream);
int q3_embedding_bf16(const int* ids, const void* table, void* out, int64_t n_tokens, int hidden, int vocab, void* stream);
/* if delta: x += delta (32-bit sum, stored in x's type); y = round(x * rsqrt(mean(x^2) + eps)) * w */
int q3_rms_norm_f32(void* x, const void* delta, const float* w, void* y, int64_t rows, int size, float eps, int64_t x_stride,
                    int64_t y_stride, void* stream);
int q3_rms_norm_bf16(void* x, const void* delta, const float* w, void* y, int64_t rows, int size, float eps, int64_t x_stride,
                     int64_t y_stride, void* stream);
/* out = round(silu(gate)) * up; a row of gate_up holds the gate then the up values, or (interleaved) blocks of 8 + 8 */
int q3_silu_mul_f32(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, void* stream);
int q3_silu_mul_bf16(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, void* stream);
/* the same with the activation as a parameter: act 0 = SiLU, 1 = the tanh form of GELU */
int q3_act_mul_f32(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, int act, void* stream);
int q3_act_mul_bf16(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, int act, void* stream);
/* out = act(x) elementwise: act 0 = SiLU, 1 = the tanh form of GELU, 2 = GELU with the error function */
int q3_activation_f32(const void* x, void* out, int64_t n, int act, void* stream);
int q3_activation_bf16(const void* x, void* out, int64_t n, int act, void* stream);
/* out[r] = x[idx[r]] (+ delta[idx[r]]) */
int q3_gather_rows_f32(const void* x, const void* delta, const int* idx, void* out, int64_t rows, int size, void* stream);
int q3_gather_rows_bf16(const void* x, const void* delta, const int* idx, void* out, int64_t rows, int size, void* stream);
/* load time: rows of src into dst with conversion (kinds: 0 float32, 1 bfloat16); source row r goes to row
   dst_row0 + (r / block_rows) * dst_block_stride + r % block_rows */
int q3_place_rows(const void* src, int src_kind, void* dst, int dst_kind, int64_t rows, int64_t cols, int64_t block_rows,
                  int64_t dst_block_stride, int64_t dst_row0, void* stream);

/* ---- stream_f32.cu: a hidden state kept in float32 between parts that compute in float32 or bfloat16 -------- */
/* out[t] = table[ids[t]] * scale */
int q3_embedding_scaled_f32(const int* ids, const void* table, float* out, int64_t n_tokens, int hidden, int vocab, float scale, void* stream);
int q3_embedding_scaled_bf16(const int* ids, const void* table, float* out, int64_t n_tokens, int hidden, int vocab, float scale, void* stream);
/* stream += RMSNorm(branch) * w_post (branch and w_post may both be null), then out = RMSNorm(stream) * w_pre (out and
   w_pre may both be null), one pass over a row */
int q3_sandwich_norm_f32(float* stream_rows, const void* branch, const float* w_post, const float* w_pre, void* out, int64_t rows,
                         int size, float eps_post, float eps_pre, void* stream);
int q3_sandwich_norm_bf16(float* stream_rows, const void* branch, const float* w_post, const float* w_pre, void* out, int64_t rows,
                          int size, float eps_post, float eps_pre, void* stream);
/* out[t] = [a[t]; b[t]] in the compute type */
int q3_concat_cast_f32(const float* a, const float* b, void* out, int64_t rows, int size, void* stream);
int q3_concat_cast_bf16(const float* a, const float* b, void* out, int64_t rows, int size, void* stream);
/* out[r] = RMSNorm(stream_rows[idx[r]]) * w */
int q3_gather_rows_norm_f32(const float* stream_rows, const int* idx, const float* w, void* out, int64_t rows, int size, float eps, void* stream);
int q3_gather_rows_norm_bf16(const float* stream_rows, const int* idx, const float* w, void* out, int64_t rows, int size, float eps, void* stream);
/* x <- cap * tanh(x * scale / cap) in place, x * scale for cap = 0 */
int q3_scale_softcap_f32(float* x, int64_t n, float scale, float cap, void* stream);

/* ---- attention.cu: every head size in steps of 16 up to 256, float32 and bfloat16 ------------------------ */
/* per-head RMSNorm of q and k (weights may be null), rotation of the first rotary_dim values of a head (0: all of
   them; tables [positions, rotary_dim/2], may be null), and the write of k and v into their pages (write_kv = 0: q only);
   bias (may be null) is added to the row of the projection first; value_dim (0: d) is the size of a value head */
int q3_qkv_prepare_f32(const void* qkv, void* q_out, void* k_pages, void* v_pages, const float* q_norm_w, const float* k_norm_w,
                       const float* cos_tab, const float* sin_tab, const int* token_seq, const int* token_pos, const int* page_table,
                       int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d, float eps, int write_kv, int rotary_dim,
                       const float* bias, int value_dim, int value_heads, void* stream);
int q3_qkv_prepare_bf16(const void* qkv, void* q_out, void* k_pages, void* v_pages, const float* q_norm_w, const float* k_norm_w,
                        const float* cos_tab, const float* sin_tab, const int* token_seq, const int* token_pos, const int* page_table,
                        int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d, float eps, int write_kv, int rotary_dim,
                       const float* bias, int value_dim, int value_heads, void* stream);
/* (q3_qkv_prepare: value_heads 0 = nkv; fewer value heads than key heads: values that several key heads share)
   causal grouped-query attention of every token over its sequence's pages; window 0 = every key; value_dim 0 = d;
   value_heads 0 = nkv, else each value head serves nkv / value_heads key heads; out_f32: `out` is float whatever q is;
   softcap > 0: scores s <- softcap * tanh(s / softcap); chunk > 0: a query reads the keys of its own chunk of that many
   positions only; sink != 0: one more term exp(0) in the softmax's denominator, or exp(sink_values[head]) where sink_values
   (one float per query head) is given; keep_first (with window): the first so many keys of the sequence are seen too */
int q3_attention_generic_f32(const void* q, const void* k_pages, const void* v_pages, void* out, const int* token_seq,
                             const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d,
                             float scale, int window, int value_dim, float softcap, int chunk, int sink, int value_heads, int out_f32,
                             const float* sink_values, int keep_first, void* stream);
int q3_attention_generic_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* token_seq,
                              const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d,
                              float scale, int window, int value_dim, float softcap, int chunk, int sink, int value_heads, int out_f32,
                              const float* sink_values, int keep_first, void* stream);

/* the same from the q/k/v projection's output as it is: bias (may be null), rotation of the first rotary_dim values of q and k
   (tables may be null) and the write of the new key and value into their pages in the attention's own kernel */
int q3_attention_capped_decode_fused_bf16(const void* qkv, void* k_pages, void* v_pages, void* out, float* scratch, const float* bias,
                                          const float* cos_tab, const float* sin_tab, int rotary_dim, const int* token_seq,
                                          const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq,
                                          int nkv, float scale, float softcap, int chunk, int sink, int n_splits, void* stream);
/* attention_prefill_tc.cu compiled with -DQ3_CAPPED=1: the tcgen05 prompt attention with capped scores, chunks and a sink
   (head sizes 64 and 128, values as wide as keys); arguments as q3_attention_prefill_tc_bf16 plus softcap, chunk, sink */
int q3_attention_capped_prefill_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_start,
                                        const int* seq_pos0, const int* page_table, int pages_per_seq, int n_seqs, int max_new,
                                        int64_t n_tokens, int64_t n_cache_pages, int nq, int nkv, float scale, float softcap, int chunk,
                                        int sink, int* status, void* stream);

/* ---- attention_capped.cu (-DQ3_HEAD_DIM, -DQ3_VALUE_DIM): bfloat16 attention with scores capped by softcap * tanh(s / softcap)
   (0: none), chunked visibility (chunk 0: causal only), a sink term in the softmax's denominator, values of their own size */
int q3_attention_capped_head_dim(void);
int q3_attention_capped_value_dim(void);
int q3_attention_capped_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_start,
                                     const int* seq_pos0, const int* page_table, int pages_per_seq, int n_seqs, int max_new, int nq,
                                     int nkv, float scale, float softcap, int chunk, int sink, int window, int value_heads,
                                     int out_f32, const float* sink_values, int keep_first, void* stream);
/* (window > 0: a sliding window of that many keys instead of chunks, beside which the first keep_first keys of the sequence
   stay visible; value_heads 0 = nkv, else each value head serves nkv / value_heads key heads; out_f32: `out` is float;
   sink_values (may be null): the sink's score per query head) */
/* one new token per sequence; scratch: n_tokens * nq * n_splits * (value_dim + 2) float32 */
int q3_attention_capped_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, float* scratch,
                                    const int* token_seq, const int* token_pos, const int* page_table, int pages_per_seq,
                                    int64_t n_tokens, int nq, int nkv, float scale, float softcap, int chunk, int sink, int n_splits,
                                    int window, int value_heads, int out_f32, const float* sink_values, int keep_first, void* stream);

/* ---- attention_decode.cu (-DQ3_HEAD_DIM): one new token per sequence, bfloat16 ---------------------------- */
int q3_attention_decode_head_dim(void);
int64_t q3_attention_decode_scratch_floats(int64_t n_tokens, int nq, int n_splits);
/* split over the keys + merge; scratch: q3_attention_decode_scratch_floats(...) float32 */
int q3_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, float* scratch, const int* token_seq,
                             const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv,
                             float scale, int window, int n_splits, void* stream);
/* the whole attention of a decode step from the q/k/v projection's output: norm, rotation, cache write, attention,
   merge of up to 8 splits inside a thread-block cluster; no scratch */
int q3_attention_decode_fused_max_splits(void);   /* 16 where clusters of 16 blocks can be placed, else 8 */
int q3_attention_decode_fused_bf16(const void* qkv, void* k_pages, void* v_pages, void* out, const float* q_norm_w,
                                   const float* k_norm_w, const float* cos_tab, const float* sin_tab, float eps, const int* token_seq,
                                   const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv,
                                   float scale, int window, int n_splits, int write_kv, int rotary_dim, void* stream);

/* ---- attention_prefill.cu, attention_prefill_tc.cu (-DQ3_HEAD_DIM): prompts, bfloat16 --------------------- */
int q3_attention_prefill_head_dim(void);
int q3_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_start,
                              const int* seq_pos0, const int* page_table, int pages_per_seq, int n_seqs, int max_new, int nq, int nkv,
                              float scale, int window, void* stream);
int q3_attention_prefill_tc_head_dim(void);
/* both products on tcgen05 (head sizes 64 and 128, no window) */
int q3_attention_prefill_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_start,
                                 const int* seq_pos0, const int* page_table, int pages_per_seq, int n_seqs, int max_new,
                                 int64_t n_tokens, int64_t n_cache_pages, int nq, int nkv, float scale, int* status, void* stream);

/* ---- matrix products Y[M, N] = X[M, K] . W[N, K]^T -------------------------------------------------------- */
/* gemm_f32.cu: true 32-bit (fmaf, ascending k); and bfloat16 operands of any width on the CUDA cores */
int q3_gemm_tn_f32(const float* X, const float* W, float* Y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, void* stream);
int q3_gemm_tn_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, int out_is_f32,
                    void* stream);
/* gemm_skinny_bf16.cu: up to 64 rows, W streamed once; `gated`: W holds gate and up rows interleaved in blocks of
   eight and Y is [M, N / 2] = round(silu(g)) * u */
int q3_gemm_skinny_bf16(const void* X, const void* W, void* Y, int M, int N, int K, void* stream);
int q3_gemm_skinny_bf16_f32out(const void* X, const void* W, void* Y, int M, int N, int K, void* stream);
int q3_gemm_skinny_gated_bf16(const void* X, const void* W, void* Y, int M, int N, int K, void* stream);
/* the same with the activation as an argument: act 1 = SiLU, 2 = the tanh form of GELU */
int q3_gemm_skinny_act_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int act, void* stream);
/* gemm_tcgen05.cu: TMA + tcgen05; weights first with K split over a cluster (`mid`), tokens first on single SMs
   (`prompt`, tile_n 128 or 256) and on pairs of SMs (`pair`) */
int q3_gemm_tcgen05_mid_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated, int splits,
                             int* status, void* stream);
int q3_gemm_tcgen05_mid_splits(int N, int K, int M);
int q3_gemm_tcgen05_prompt_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int tile_n, int* status,
                                void* stream);
int q3_gemm_tcgen05_prompt_gated_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int* status, void* stream);
/* the q/k/v product of a prompt step with q3_qkv_prepare's work in its epilogue: W [(nq + 2 nkv) d, K]; q to q_out
   [M, nq d], k and v (write_kv) to the pages; d 64, 128 or 256; norm weights and whole-head tables may be null */
int q3_gemm_tcgen05_pair_qkv_bf16(const void* X, const void* W, int M, int K, void* q_out, void* k_pages, void* v_pages,
                                  const float* q_norm_w, const float* k_norm_w, const float* cos_tab, const float* sin_tab, float eps,
                                  const int* token_seq, const int* token_pos, const int* page_table, int pages_per_seq, int nq,
                                  int nkv, int d, int write_kv, int* status, void* stream);
/* splits 1..4: K split over that many pairs of SMs of one cluster (1: persistent pairs, no split) */
int q3_gemm_tcgen05_pair_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated, int splits,
                              int* status, void* stream);
int q3_gemm_tcgen05_pair_capacity(int splits);

/* ---- hyper.cu: a hidden state of several streams per token, float32 [token, streams, hidden] ------------------ */
/* out[t] = `copies` times table[ids[t]] * scale side by side */
int q3_embedding_streams_f32(const int* ids, const void* table, float* out, int64_t n_tokens, int hidden, int vocab, float scale,
                             int copies, void* stream);
int q3_embedding_streams_bf16(const int* ids, const void* table, float* out, int64_t n_tokens, int hidden, int vocab, float scale,
                              int copies, void* stream);
/* one pass: settle a pending sublayer output (x_to <- sum_from mix[from][to] x_from + out_coef[to] branch; branch may be
   null), u = sum_s in_coef[s] x_s (null: ones), out = u / sqrt(mean(u^2) + eps) * norm_w (normalize 0: u itself; out may be
   null).  rows != null: only those tokens, one output row each, the streams are not written */
int q3_hyper_norm_f32(float* streams, const void* branch, const float* mix, const float* out_coef, const float* in_coef,
                      const float* norm_w, float eps, void* out, int out_f32, const int* rows, int64_t n_rows, int n_streams,
                      int hidden, int normalize, void* stream);
int q3_hyper_norm_bf16(float* streams, const void* branch, const float* mix, const float* out_coef, const float* in_coef,
                       const float* norm_w, float eps, void* out, int out_f32, const int* rows, int64_t n_rows, int n_streams,
                       int hidden, int normalize, void* stream);

/* ---- lightning.cu: linear attention with a per-head decay and a float32 state [slot, heads, d, vd] ------------- */
/* proj [N, 2 heads d + 2 heads vd] = q, k, v (SiLU applied here), gate; S <- decay S + k v^T, out = S^T q, token by token */
int q3_lightning_scan_f32(const void* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots,
                          float* out, int n_seqs, int heads, int d, int vd, void* stream);
int q3_lightning_scan_bf16(const void* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots,
                           float* out, int n_seqs, int heads, int d, int vd, void* stream);
/* the same for prompts, 32 tokens at a time */
int q3_lightning_chunks_f32(const void* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots,
                            float* out, int n_seqs, int heads, int d, int vd, void* stream);
int q3_lightning_chunks_bf16(const void* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots,
                             float* out, int n_seqs, int heads, int d, int vd, void* stream);
/* the chunks' products on the tensor cores (operands as TF32 hi + lo terms): head sizes in steps of 8 */
int q3_lightning_chunks_tc_bf16(const void* proj, float* state, const float* decay, const int* seq_start, const int* seq_slots,
                                float* out, int n_seqs, int heads, int d, int vd, void* stream);
/* out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate), row by row; gate rows are gate_stride apart */
int q3_gated_norm_f32(const float* o, const void* gate, int64_t gate_stride, const float* w, float eps, void* out,
                      int64_t n_tokens, int size, void* stream);
int q3_gated_norm_bf16(const float* o, const void* gate, int64_t gate_stride, const float* w, float eps, void* out,
                       int64_t n_tokens, int size, void* stream);

/* ---- differential.cu ---------------------------------------------------------------------------------------- */
/* a float32 [token, group, 2 maps, per_group, vd]; out[t, h] = unit_rms(a1 - lambda a2) * gain */
int q3_diff_combine_f32(const float* a, void* out, int64_t n_tokens, int heads, int per_group, int vd, float lambda, float eps,
                        float gain, void* stream);
int q3_diff_combine_bf16(const float* a, void* out, int64_t n_tokens, int heads, int per_group, int vd, float lambda, float eps,
                         float gain, void* stream);

/* ---- moe.cu: a routed feed-forward ---------------------------------------------------------------------------- */
/* per token: float32 router logits, softmax, choice by score + correction within the kept groups, weights = scores;
   the outputs from n_real on are identity experts (their weights are summed into id_weight); by_logit: the largest logits
   are chosen, weighted by the softmax over the chosen logits alone; gate_out (may be null): the router matrix has one more
   row and gate_out[t] = sigmoid of its logit; by_logit 2: scores sigmoid(z) instead of the softmax; group_pair: a group's mark
   is the sum of its two best choice scores; the weights are multiplied by weight_scale */
int q3_moe_route_f32(const void* h, const void* w_router, const float* correction, int* top_ids, float* top_w, float* id_weight,
                     int64_t n_tokens, int hidden, int n_out, int n_real, int top, int group_count, int group_keep, int by_logit,
                     float* gate_out, int group_pair, float weight_scale, void* stream);
int q3_moe_route_bf16(const void* h, const void* w_router, const float* correction, int* top_ids, float* top_w, float* id_weight,
                      int64_t n_tokens, int hidden, int n_out, int n_real, int top, int group_count, int group_keep, int by_logit,
                      float* gate_out, int group_pair, float weight_scale, void* stream);
/* offsets [n_real + 1], slot_of_pair (-1: identity) and pair_of_slot of the (token, choice) pairs laid out by expert */
int q3_moe_sort(const int* top_ids, int n_pairs, int n_real, int* offsets, int* slot_of_pair, int* pair_of_slot, void* stream);
/* act[slot] = g sigmoid(alpha g) (u + up_offset), g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit); y[slot] = W_down act */
int q3_moe_experts_f32(const void* h, const void* w_gate_up, const void* w_down, const int* offsets, const int* pair_of_slot,
                       void* act, float* y, int n_pairs, int n_real, int top, int hidden, int ff, float limit, float alpha,
                       float up_offset, void* stream);
int q3_moe_experts_bf16(const void* h, const void* w_gate_up, const void* w_down, const int* offsets, const int* pair_of_slot,
                        void* act, float* y, int n_pairs, int n_real, int top, int hidden, int ff, float limit, float alpha,
                        float up_offset, void* stream);
/* the same on the tensor cores: bfloat16, hidden and ff multiples of 32 */
int q3_moe_experts_tc_bf16(const void* h, const void* w_gate_up, const void* w_down, const int* offsets, const int* pair_of_slot,
                           void* act, float* y, int n_pairs, int n_real, int top, int hidden, int ff, float limit, float alpha,
                           float up_offset, void* stream);
/* out[t] = sum_k top_w[t, k] y[slot_of_pair[t, k]] + id_weight[t] h[t] + shared_w[t] shared[t] (the last may be null) */
int q3_moe_combine_f32(const float* y, const void* h, const int* slot_of_pair, const float* top_w, const float* id_weight,
                       void* out, int64_t n_tokens, int top, int hidden, const void* shared, const float* shared_w, void* stream);
int q3_moe_combine_bf16(const float* y, const void* h, const int* slot_of_pair, const float* top_w, const float* id_weight,
                        void* out, int64_t n_tokens, int top, int hidden, const void* shared, const float* shared_w, void* stream);

/* ---- stream_shift.cu: a float32 hidden state with norms of several kinds, a token shift, a token side input ------ */
/* one pass over the rows: stream += post(branch), out = pre(stream).  Norm kinds: 0 none, 1 unit rms times w, 2 dynamic tanh
   tanh(alpha x) * w + b, 3 the rounded sum alone (pre only).  out_f32: `out` is float whatever the compute type.  With `rows`
   only those rows are read, nothing is written to the stream and out[r] belongs to rows[r] */
int q3_settle_norm_f32(float* stream_rows, const void* branch, int post_kind, const float* post_w, const float* post_b,
                       float post_alpha, float post_eps, int pre_kind, const float* pre_w, const float* pre_b, float pre_alpha,
                       float pre_eps, void* out, int out_f32, const int* rows, int64_t n_rows, int size, void* stream);
int q3_settle_norm_bf16(float* stream_rows, const void* branch, int post_kind, const float* post_w, const float* post_b,
                        float post_alpha, float post_eps, int pre_kind, const float* pre_w, const float* pre_b, float pre_alpha,
                        float pre_eps, void* out, int out_f32, const int* rows, int64_t n_rows, int size, void* stream);
/* out[t] = h[t] + (h[t-1] - h[t]) * mu within a sequence; the row before a step's first row is state[slot], which the step's
   last row replaces */
int q3_token_shift_f32(const float* h, const float* mu, float* state, void* out, const int* token_seq, const int* seq_start,
                       const int* seq_slots, int64_t n_tokens, int size, void* stream);
int q3_token_shift_bf16(const float* h, const float* mu, float* state, void* out, const int* token_seq, const int* seq_start,
                        const int* seq_slots, int64_t n_tokens, int size, void* stream);
/* out[t, j] = gelu_tanh(a[t, j]) * table[ids[t], col0 + j] */
int q3_side_gate_f32(const void* a, const int* ids, const void* table, void* out, int64_t n_tokens, int dim, int col0,
                     int table_cols, int vocab, void* stream);
int q3_side_gate_bf16(const void* a, const int* ids, const void* table, void* out, int64_t n_tokens, int dim, int col0,
                      int table_cols, int vocab, void* stream);

/* ---- gated_recurrence.cu: linear attention whose forget gate also writes, a float32 state [slot, heads, d, vd] --------- */
/* proj [tokens, heads (2 d + vd)]: q, gate logits and v head by head; f = low + (1 - low) sigmoid(z + bias),
   S = diag(f) S + (1 - f) v^T, out = S^T silu(q) (float32 [tokens, heads vd]) */
int q3_gated_scan_f32(const void* proj, float* state, const float* low, const float* bias, const int* seq_start,
                      const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd, void* stream);
int q3_gated_scan_bf16(const void* proj, float* state, const float* low, const float* bias, const int* seq_start,
                       const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd, void* stream);
/* out = o / sqrt(mean(o^2) + eps) * w over every run of vd values (n_rows runs) */
int q3_head_rms_norm_f32(const float* o, const float* w, void* out, int64_t n_rows, int vd, float eps, void* stream);
int q3_head_rms_norm_bf16(const float* o, const float* w, void* out, int64_t n_rows, int vd, float eps, void* stream);

/* ---- latent.cu: attention over a cache of latents [c | rotated key part] ---------------------------------------------- */
/* per token: c = unit_rms(proj[kv_off : kv_off + rank]) * w_c and the next `rot` values rotated go to the key row, c also to the
   value row; with q_rank > 0, cq = unit_rms(proj[q_off : q_off + q_rank]) * w_q */
int q3_latent_prepare_f32(const void* proj, int64_t proj_stride, int kv_off, int q_off, const float* w_c, const float* w_q, void* cq,
                          void* k_pages, void* v_pages, const float* cos_tab, const float* sin_tab, const int* token_seq,
                          const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int rank, int rot,
                          int rot_dims, int interleaved, int q_rank, float eps, int write_kv, void* stream);
int q3_latent_prepare_bf16(const void* proj, int64_t proj_stride, int kv_off, int q_off, const float* w_c, const float* w_q, void* cq,
                           void* k_pages, void* v_pages, const float* cos_tab, const float* sin_tab, const int* token_seq,
                           const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int rank, int rot,
                           int rot_dims, int interleaved, int q_rank, float eps, int write_kv, void* stream);
/* q_full[t, h, rank:] = rotate(q[t, h, d:]) */
int q3_latent_queries_f32(const void* q, int64_t q_row, void* q_full, const float* cos_tab, const float* sin_tab, const int* token_pos,
                          int64_t n_tokens, int heads, int d, int rank, int rot, int rot_dims, int interleaved, void* stream);
int q3_latent_queries_bf16(const void* q, int64_t q_row, void* q_full, const float* cos_tab, const float* sin_tab, const int* token_pos,
                           int64_t n_tokens, int heads, int d, int rank, int rot, int rot_dims, int interleaved, void* stream);
/* out[t, h, out_off + j] = sum_i x[t, h, x_off + i] * w[h, i, j] (* sigmoid(gate[t, h, j]) where gate is given) */
int q3_head_product_f32(const void* x, int64_t x_row, int x_head, int x_off, const void* w, void* out, int64_t out_row, int out_head,
                        int out_off, const void* gate, int64_t gate_row, int64_t n_tokens, int heads, int K, int N, void* stream);
int q3_head_product_bf16(const void* x, int64_t x_row, int x_head, int x_off, const void* w, void* out, int64_t out_row, int out_head,
                         int out_off, const void* gate, int64_t gate_row, int64_t n_tokens, int heads, int K, int N, void* stream);

/* ---- elementwise.cu: the clamped gated activation, a weighted sum, a bias ------------------------------------ */
/* out = g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); the layout of q3_act_mul */
int q3_clamped_mul_f32(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, float limit, float alpha, void* stream);
int q3_clamped_mul_bf16(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, float limit, float alpha, void* stream);
/* out = sa * a + sb * b */
int q3_scaled_sum_f32(const void* a, const void* b, float sa, float sb, void* out, int64_t n, void* stream);
int q3_scaled_sum_bf16(const void* a, const void* b, float sa, float sb, void* out, int64_t n, void* stream);
/* x[r, c] += bias[c] */
int q3_add_bias_f32(void* x, const float* bias, int64_t rows, int size, void* stream);
int q3_add_bias_bf16(void* x, const float* bias, int64_t rows, int size, void* stream);

/* ---- attention.cu: values blended across layers, a gate per head --------------------------------------------- */
/* on columns [v_off, v_off + width) of rows of `row` values: v += bias; save: first = v; else v = (1 - lambda) v + lambda first */
int q3_value_mix_f32(void* rows, int64_t row, int64_t v_off, int width, const float* bias, void* first, int save, float lambda,
                     int64_t n_tokens, void* stream);
int q3_value_mix_bf16(void* rows, int64_t row, int64_t v_off, int width, const float* bias, void* first, int save, float lambda,
                      int64_t n_tokens, void* stream);
/* x[t, h, :] *= sigmoid(gate[t, h]) */
int q3_head_gate_f32(void* x, const void* gate, int64_t gate_row, int heads, int vd, int64_t n_tokens, void* stream);
int q3_head_gate_bf16(void* x, const void* gate, int64_t gate_row, int heads, int vd, int64_t n_tokens, void* stream);

/* ---- short_conv.cu ------------------------------------------------------------------------------------------- */
/* y[t, c] = sum_j w[j, c] u[t - taps + 1 + j, c] (w [taps, channels]) within every sequence; rows before the step come from state
   [slot][taps - 1][channels] (float32), which is moved on afterwards */
int q3_short_conv_f32(const void* u, int64_t row_in, const float* w, float* state, int64_t slot_stride, const int* token_seq,
                      const int* seq_start, const int* seq_slots, void* y, int channels, int taps, int64_t n_tokens, int n_seqs,
                      void* stream);
int q3_short_conv_bf16(const void* u, int64_t row_in, const float* w, float* state, int64_t slot_stride, const int* token_seq,
                       const int* seq_start, const int* seq_slots, void* y, int channels, int taps, int64_t n_tokens, int n_seqs,
                       void* stream);

/* ---- linear_scan.cu: linear attention with keys ------------------------------------------------------------- */
/* z <- sigmoid(z + bias)^inv_tau in place: the decays per key channel from their logits [n_tokens, width] */
int q3_channel_decay(float* z, const float* bias, float inv_tau, int64_t n_tokens, int width, void* stream);
/* S_t = diag(a_t) S_(t-1) + k_t (b_t v_t)^T, o_t = S_t^T (q_t q_scale); z given: the decays a per (token, channel), b = 1;
   keep and write given: a and b per (token, head); ones: the state has a last column whose value is 1 */
int q3_decay_scan_f32(const void* q, const void* k, const void* v, int64_t row, const float* z,
                      const float* keep, const float* write, float q_scale, int ones, float* state, int64_t slot_stride,
                      const int* seq_start, const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd, void* stream);
int q3_decay_scan_bf16(const void* q, const void* k, const void* v, int64_t row, const float* z,
                       const float* keep, const float* write, float q_scale, int ones, float* state, int64_t slot_stride,
                       const int* seq_start, const int* seq_slots, float* out, int n_seqs, int heads, int d, int vd, void* stream);
/* i = cap tanh((zi + bias_i) / cap), f = logsigmoid(cap tanh((zf + bias_f) / cap)), m_t = max(f_t + m_(t-1), i_t) from and to
   m_state; keep = exp(f + m_(t-1) - m_t), write = exp(i - m_t), low = exp(-m_t) */
int q3_memory_gates(const float* zi, const float* zf, const float* bias_i, const float* bias_f, float cap, float* m_state,
                    int64_t slot_stride, const int* seq_start, const int* seq_slots, float* keep, float* write, float* low, int heads,
                    int64_t z_row, int n_seqs, void* stream);
/* per (token, head): x = o[:vd] (/ (max(|o[vd]|, low) + floor_add) if vdx > vd); out = x / sqrt(mean(x^2) + eps) * w * act(gate) */
int q3_head_gated_norm_f32(const float* o, const float* low, float floor_add, const float* w, int w_per_head, const void* gate,
                           int64_t gate_row, void* out, int64_t n_tokens, int heads, int vd, int vdx, float eps, int act, void* stream);
int q3_head_gated_norm_bf16(const float* o, const float* low, float floor_add, const float* w, int w_per_head, const void* gate,
                            int64_t gate_row, void* out, int64_t n_tokens, int heads, int vd, int vdx, float eps, int act, void* stream);

/* ---- sampling.cu ------------------------------------------------------------------------------------------ */
/* out[r] = index of the highest logit among the first `valid` (lowest id among equals, NaN as -inf) */
int q3_argmax_f32(const float* logits, int64_t stride, int rows, int valid, int* out, void* stream);
/* temperature -> top-k (ties stay) -> order by score then id -> softmax -> top-p -> inverse CDF; the uniform number of
   row r is a hash of (seed, seq_ids[r], steps ? steps[r] : step_all); out[r] = -1 for a row with a non-finite logit */
int q3_sample_f32(const float* logits, int64_t stride, int rows, int valid, float temperature, int top_k, float top_p, uint64_t seed,
                  const int64_t* seq_ids, const int* steps, int step_all, int* out, void* stream);

/* every library: programmatic dependent launch for its kernels on (1) or off (0, the default) */
void q3_set_pdl(int on);

#ifdef __cplusplus
}
#endif
