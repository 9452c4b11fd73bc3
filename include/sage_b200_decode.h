/*
 * sage_b200 — C ABI of the non-matmul steps of a Qwen3 decode step (one new token for each
 * of 1..16 sequences): embedding lookup, residual add + RMSNorm, per-head q/k RMSNorm +
 * rotate-half RoPE + KV-cache append, split-context attention, SwiGLU, FP16 lm_head and
 * argmax.  They let a whole decode step run as one CUDA graph with token ids and positions
 * kept in device memory.
 *
 * None of these has a counterpart in the reference's native code: there the same steps are
 * Hugging Face `transformers` Qwen3 modules and torch SDPA, driven by
 * benchmarks/model.py:43-133 (prefill, then one model call per token with a StaticCache).
 *
 * All pointers are device pointers, all tensors FP16 and contiguous unless noted; `stream`
 * is a cudaStream_t; every function returns 0, -1 (unsupported shape) or -5 (launch failed).
 * head_dim must be 128.
 */
#ifndef SAGE_B200_DECODE_H_
#define SAGE_B200_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* h[rows][hidden] = table[tokens[row]][:]; tokens are int64.  An id outside [0, vocab) reads
 * row 0 (never memory beyond the table). */
int sageb200_glue_embed(const void *table, const void *tokens, void *h, int rows, int hidden,
                        int vocab, void *stream);

/* residual += delta (skipped when delta is NULL); x = weight * rmsnorm(residual, eps). */
int sageb200_glue_add_rmsnorm(void *residual, const void *delta, const void *weight, void *x,
                              int rows, int hidden, float eps, void *stream);

/*
 * The same with the normalised row also written once per consumer in that consumer's quantised
 * channel order: outs[j][row][c] = x[row][perms[j][c]] for j < count <= 4 (int32 permutations and
 * outputs 16-byte aligned; x may be NULL).  The packed linears behind it then take their
 * activations as they lie (no permutation argument, no gather pre-pass).
 */
int sageb200_glue_add_rmsnorm_permuted(void *residual, const void *delta, const void *weight, void *x,
                                       const void *const *perms, void *const *outs, int count, int rows,
                                       int hidden, float eps, void *stream);

/* act[row][c] = silu(gate[row][perm[c]]) * up[row][perm[c]] (the rounding of sageb200_glue_swiglu). */
int sageb200_glue_swiglu_permuted(const void *gate, const void *up, const void *perm, void *act, int rows, int k,
                                  int sm_count, void *stream);

/*
 * q[rows][q_heads][128] is normalised and rotated in place; k is normalised, rotated and
 * written to k_cache[row][kv_head][positions[row]][:]; v is copied to v_cache likewise.
 * cos/sin tables are FP16 [max_seq][64]; positions are int32 [rows].
 */
int sageb200_glue_qk_norm_rope_cache(void *q, const void *k, const void *v, const void *q_weight,
                                     const void *k_weight, const void *cos_table,
                                     const void *sin_table, const void *positions, void *k_cache,
                                     void *v_cache, int rows, int q_heads, int kv_heads, int head_dim,
                                     int max_seq, float eps, void *stream);

/* FP32 scratch for sageb200_glue_attention_decode. */
size_t sageb200_glue_attention_scratch_bytes(int rows, int q_heads, int splits);

/*
 * out[rows][q_heads][128] = softmax(q . K^T / sqrt(128)) . V over cache positions
 * 0..positions[row] (the new token included), grouped-query heads, the context split over
 * `splits` CTAs per (row, kv head).
 */
int sageb200_glue_attention_decode(const void *q, const void *k_cache, const void *v_cache,
                                   const void *positions, void *out, void *scratch, int rows,
                                   int q_heads, int kv_heads, int head_dim, int max_seq, int splits,
                                   void *stream);

/*
 * The three calls above in ONE launch: q and the new k are normalised and rotated (q is left
 * untouched in memory), the new k/v go into the cache at positions[row] (bit-identical to
 * sageb200_glue_qk_norm_rope_cache), and each (row, kv head, block of four query heads) is
 * attended by a thread-block cluster of `splits` CTAs (1, 2, 4, 8 or - where the GPU can
 * co-schedule that many - 16; -1 otherwise) that combine their
 * partial results through distributed shared memory: no scratch.  Same FP32 arithmetic as
 * sageb200_glue_attention_decode, summed in another order.
 * The kernel is launched as a programmatic dependent and reads cache rows below `positions`
 * before it waits for the previous kernel of the stream: that kernel may produce q, k and v (as
 * the q/k/v projection does) but must not be the one that wrote those cache rows.
 */
int sageb200_glue_attention_step(const void *q, const void *k, const void *v, const void *q_weight,
                                 const void *k_weight, const void *cos_table, const void *sin_table,
                                 const void *positions, void *k_cache, void *v_cache, void *out, int rows,
                                 int q_heads, int kv_heads, int head_dim, int max_seq, int splits, float eps,
                                 void *stream);

/*
 * The same, with each output row written through `out_index` (int32 [q_heads * head_dim], or
 * null for the plain order): channel c of a row lands at out[row][out_index[c]].  Given the
 * inverse of the output projection's channel permutation, the rows arrive in that linear's
 * quantised channel order and it is called with an empty permutation (no gather of its own).
 */
int sageb200_glue_attention_step_permuted(const void *q, const void *k, const void *v, const void *q_weight,
                                          const void *k_weight, const void *cos_table, const void *sin_table,
                                          const void *positions, void *k_cache, void *v_cache, void *out,
                                          const void *out_index, int rows, int q_heads, int kv_heads, int head_dim,
                                          int max_seq, int splits, float eps, void *stream);

/*
 * Prompt processing (many tokens of each sequence at once).  Rows are [sequence][token]:
 * row s*tokens + t is token t of sequence s and sits at cache position positions[s] + t.
 * The first call is sageb200_glue_qk_norm_rope_cache for such rows (q normalised and rotated
 * in place, every token's k/v written to the cache); the second is causal attention of every
 * row over cache positions 0 .. its own, out[rows][q_heads][128].
 */
int sageb200_glue_prefill_qk_norm_rope_cache(void *q, const void *k, const void *v, const void *q_weight,
                                             const void *k_weight, const void *cos_table,
                                             const void *sin_table, const void *positions, void *k_cache,
                                             void *v_cache, int sequences, int tokens, int q_heads,
                                             int kv_heads, int head_dim, int max_seq, float eps, void *stream);
int sageb200_glue_prefill_attention(const void *q, const void *k_cache, const void *v_cache,
                                    const void *positions, void *out, int sequences, int tokens, int q_heads,
                                    int kv_heads, int head_dim, int max_seq, void *stream);

/* act[i] = fp16(silu(gate[i])) * up[i]. */
int sageb200_glue_swiglu(const void *gate, const void *up, void *act, long long count, void *stream);

/* logits[rows][vocab] = x[rows][hidden] . head[vocab][hidden]^T, FP32 accumulation. */
int sageb200_glue_lm_head(const void *head, const void *x, void *logits, int rows, int vocab,
                          int hidden, int sm_count, void *stream);

/*
 * tokens[row] = argmax(logits[row]) (int64, lowest index on ties); positions[row] += 1;
 * if log != NULL, log[row*log_stride + step[0]] = token and step[0] += 1 (int32).
 */
int sageb200_glue_argmax_advance(const void *logits, void *tokens, void *positions, void *log,
                                 void *step, int rows, int vocab, int log_stride, void *stream);

/*
 * The tail of a decode step in ONE launch: x = rmsnorm(residual + delta) * norm_weight (the
 * arithmetic of sageb200_glue_add_rmsnorm; `residual` itself is not updated, `delta` may be
 * NULL), logits = x . head^T, then what sageb200_glue_argmax_advance does.  `scratch` holds
 * sageb200_glue_lm_head_step_scratch_bytes() bytes whose first 256 (arrival and ticket counters) must
 * be zero before the first call; every call leaves them zero.
 */
size_t sageb200_glue_lm_head_step_scratch_bytes(int rows, int sm_count);
int sageb200_glue_lm_head_step(const void *head, const void *residual, const void *delta,
                               const void *norm_weight, void *x, void *logits, void *tokens,
                               void *positions, void *log, void *step, void *scratch, int rows, int vocab,
                               int hidden, float eps, int log_stride, int sm_count, void *stream);

/*
 * Mixture-of-experts routing of `rows` tokens in one launch: residual += delta (delta may be
 * NULL), x = rmsnorm(residual) * norm_weight (as sageb200_glue_add_rmsnorm), router logits =
 * fp16(x . router[experts][hidden]^T), softmax over all experts, the top_k experts per token
 * (lowest index on ties) as ids int32 [rows][top_k] with renormalised weights float
 * [rows][top_k] - the routing of Hugging Face Qwen3-MoE.  experts <= 256, top_k <= 32.
 */
int sageb200_glue_moe_route(void *residual, const void *delta, const void *norm_weight, const void *router,
                            void *x, void *ids, void *weights, int rows, int hidden, int experts, int top_k,
                            float eps, void *stream);

/*
 * The sorted expert compute behind an all-to-all dispatch (or any batch beyond one grouped launch):
 * `received` (token, expert) slots with global expert ids int32 `ids` (-1 = none) are packed into
 * blocks of rows_per_block rows, every block belonging to one of this rank's experts
 * [first_expert, first_expert + local_experts), the slots of an expert in received order.
 *   dispatch_plan  target[j] = row of the block buffer slot j takes (blocks * rows_per_block = "dump"
 *                  for a slot without a local expert), block_experts[b] = global expert id of block b
 *                  (-1 unused); one launch; received <= 4096, local_experts <= 256; `blocks` at least
 *                  local_experts + ceil(received / rows_per_block) places every slot
 *   dispatch_rows  rows[target[j]][:] = x[j / source_div][:]       (source_div = top_k when x holds tokens)
 *   combine_rows   back[j][:] = outputs[target[j]][:], zeros for a slot without a row
 * No counterpart in the reference (no packed mixture of experts there).
 */
int sageb200_glue_dispatch_plan(const void *ids, void *target, void *block_experts, int received,
                                int first_expert, int local_experts, int rows_per_block, int blocks, void *stream);
int sageb200_glue_dispatch_rows(const void *x, const void *target, void *rows, int received, int hidden, int dump,
                                int source_div, void *stream);
int sageb200_glue_combine_rows(const void *outputs, const void *target, void *back, int received, int hidden,
                               int dump, void *stream);

/* out[rows][hidden] = fp16(sum_s weights[row][s] * slot_outputs[row*top_k + s][:]) (FP32 sum). */
int sageb200_glue_moe_mix(const void *slot_outputs, const void *weights, void *out, int rows, int hidden,
                          int top_k, void *stream);

/* ---------------------------------------------------------------------------------------
 * One decoded token as ONE persistent kernel (batch 1, one GPU, dense-MLP Qwen3).
 *
 * A cooperative grid of one CTA per SM runs the whole token: per layer residual add + RMSNorm
 * + q/k/v, attention over the KV cache, o_proj, residual add + RMSNorm + gate/up + SwiGLU,
 * down_proj; then the final norm, the FP16 lm_head and the greedy argmax, with a grid barrier
 * between dependent phases and the next phase's packed weights streaming into shared memory
 * through the barriers.  Same arithmetic as the per-launch calls above and as
 * sageb200_linear_grouped_fused; sums associate in another (fixed) order.
 *
 * The reference has no counterpart (there a token is ~250 kernel launches driven by Hugging
 * Face modules, benchmarks/model.py:112-116 and weight_vq/inference/linear.py:289-309).
 *
 * All pointers are device pointers.  Packed buffers are the five buffers of sage_b200.h; the
 * four big ones and the permutation must be 16-byte aligned here.
 */
typedef struct sageb200_mega_linear {
  const void *codes, *radii, *grid, *book;
  const int32_t *perm;          /* NULL: identity */
  int n, k, entries;
} sageb200_mega_linear;

typedef struct sageb200_mega_layer {
  sageb200_mega_linear q, k, v, o, gate, up, down;
  const void *input_norm, *post_norm, *q_norm, *k_norm;   /* FP16 norm weights */
  void *k_cache, *v_cache;                                /* FP16 [kv_heads][max_seq][128] */
} sageb200_mega_layer;

typedef struct sageb200_mega_model {
  int layers, hidden, heads, kv_heads, head_dim, intermediate, vocab, max_seq;
  float eps;
  const void *embed, *lm_head, *final_norm;               /* FP16 [vocab][hidden] x2, [hidden] */
  const void *cos_table, *sin_table;                      /* FP16 [max_seq][64] */
} sageb200_mega_model;

/*
 * Bytes of device workspace a model needs (0: the model does not fit this kernel - head_dim
 * other than 128, more than 8 query heads per kv head, rows too long for shared memory, fewer
 * SMs than heads - and the caller stays on the per-launch path).  sm_count <= 0: the current
 * device's.  Pure host arithmetic.
 */
size_t sageb200_mega_workspace_bytes(const sageb200_mega_model *model, int sm_count);

/*
 * Writes the launch plan (per-CTA work ranges, layer tables, scratch pointers) into the
 * 256-byte aligned `workspace` and zeroes its barrier words and partial-sum slots; synchronises
 * `stream`.  Call once per model (and again after a SAGEB200_ERR_TIMEOUT, whose barrier words
 * are left as they were).  `layers` is a host array of model->layers entries.
 */
int sageb200_mega_prepare(const sageb200_mega_model *model, const sageb200_mega_layer *layers,
                          void *workspace, size_t workspace_bytes, void *stream);

/*
 * One decode step: reads tokens[0] (int64) and positions[0] (int32), appends the token's key and
 * value to every layer's cache, writes logits[vocab] (FP16), tokens[0] = argmax (lowest index
 * on ties), log[step[0]] = token if step[0] < log_stride, positions[0] += 1, step[0] += 1.
 * Enqueues one cooperative kernel on `stream`; no host synchronisation.  Every device-side
 * wait is bounded: one that runs out is recorded as SAGEB200_ERR_TIMEOUT (see
 * sageb200_clear_status in sage_b200.h).  Steps of one workspace must not overlap.
 */
int sageb200_mega_step(const sageb200_mega_model *model, void *workspace, void *tokens, void *positions,
                       void *log, void *step, void *logits, int log_stride, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_DECODE_H_ */
