/*
 * b200_mixers.h — C ABI of the ragged-batch sequence mixers and feed-forward pieces (libb200_mixers.so, sm_100a).
 *
 * Same conventions as b200_kv.h: extern "C", device pointers owned by the caller, work queued on `stream`
 * (a cudaStream_t passed as void*), nothing allocates or synchronises, 0 on success, negative B200_E* or a positive
 * cudaError_t otherwise with the text in b200_mixers_last_error().  `dtype` is the storage type T of activations,
 * weights and pools (0 = float16, 1 = float32, 2 = bfloat16).  The residual stream, norm statistics, attention
 * scores and weights, recurrence gates and state are fp32 for every T.
 *
 * A step's tokens are PACKED: row n of every activation is one token; the tokens of a sequence are consecutive and
 * in order.  tok_pos[n] is the token's position in its sequence.
 */
#ifndef B200_MIXERS_H_
#define B200_MIXERS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_MIXERS_ABI_VERSION 1

int b200_mixers_abi_version(void);
const char* b200_mixers_last_error(void);

/* out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * (1 + weight);  x fp32 [rows, width], out T [rows, width]. */
int b200_offset_rmsnorm(void* out, const float* x, const void* weight, float eps, int rows, int width, int dtype,
                        void* stream);

/* x[r] += mult * offset_norm(y[r]; w_post) in fp32 (x is updated in place); when w_next is given, out_next[r] =
 * offset_norm(x[r]; w_next) in T — the next sublayer's input.  y is T, or fp32 when y_is_f32. */
int b200_postnorm_residual(float* x, const void* y, int64_t y_stride, int y_is_f32, const void* w_post, float mult,
                           const void* w_next, void* out_next, float eps, int rows, int width, int dtype, void* stream);

/* Per token and kv head: v <- v / rms(v) (eps inside the root); with v_prev [n_tok, G*dv]: v <- (1 - lam) v + lam
 * v_prev.  The result (rounded to T) is scattered with k through slot_mapping (slot = block * block_size + offset,
 * negative = skip) into k_pool [max_blocks, G, block_size, dk] and v_pool [max_blocks, G, block_size, dv], and
 * copied to v_keep [n_tok, G*dv] when given. */
int b200_value_prep_append(const void* k, int64_t k_stride, const void* v, int64_t v_stride, const void* v_prev,
                           void* v_keep, float lam, float eps, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                           int n_tok, int G, int dk, int dv, int block_size, int64_t max_blocks, int dtype, void* stream);

/* Tokens of one sequence that a CTA of b200_biased_paged_attn serves at most (cut portions into tiles of this). */
int b200_biased_attn_tile_tokens(int n_tokens_in_portion, int H, int G);

/* Causal attention of packed query rows over the paged cache (which already holds this step's keys and values).
 *   score(i, j) = (q_i . k_j) * scale * (1 + temp_coef * ln(floor((i + 1) / temp_every) + 1)) + bias_lut[h][min(i - j, lut_len - 1)]
 *   out[n, h, :] = sigmoid(gate[n, h]) * softmax_j(score) . v_j          (gate may be NULL)
 * tiles: int32 [n_tiles, 3] = (first packed row, token count <= max_tile_tokens, block-table row); a tile's tokens
 * belong to one sequence.  bias_lut: fp32 [H, lut_len].  q: T rows of H*dk with row stride q_stride; out: T
 * [n_tok, H*dv] contiguous. */
int b200_biased_paged_attn(void* out, const void* q, int64_t q_stride, const void* gate, int64_t gate_stride,
                           const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                           const int32_t* tiles, int n_tiles, int max_tile_tokens, const int32_t* tok_pos,
                           const float* bias_lut, int lut_len, float scale, float temp_coef, int temp_every, int H, int G,
                           int dk, int dv, int block_size, int dtype, void* stream);

/* The same attention on the tensor cores (16-bit dtypes; dk a multiple of 16 up to 256, dv a multiple of 8 up to
 * 128 — b200_biased_prompt_attn_supported says whether a layer qualifies).  A CTA serves 64 rows = the tokens of a tile
 * times the query heads of one kv head, so tiles hold up to b200_biased_prompt_attn_tile_tokens(H, G) = 64 / (H / G)
 * tokens; a tile's tokens have consecutive positions.  Prompt portions and single decoded tokens alike: when no tile
 * has more than max_tile_tokens tokens and that many tokens are at most 16 rows, the warps of a CTA split the keys
 * instead of the rows (pass 0 when unknown).  Scores, bias and softmax are fp32; the softmax
 * weights are rounded to the storage type only as the operand of the P.V product.  Rows written: the tiles' tokens. */
int b200_biased_prompt_attn_supported(int dk, int dv, int dtype);
int b200_biased_prompt_attn_tile_tokens(int H, int G);
int b200_biased_prompt_attn(void* out, const void* q, int64_t q_stride, const void* gate, int64_t gate_stride,
                            const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                            const int32_t* tiles, int n_tiles, int max_tile_tokens, const int32_t* tok_pos,
                            const float* bias_lut, int lut_len, float scale, float temp_coef, int temp_every, int H, int G,
                            int dk, int dv, int block_size, int dtype, void* stream);

/* Gated linear recurrence per (sequence, head) over the sequence's tokens of this step, in order:
 *   q = silu(zq), f = lower + (1 - lower) * sigmoid(zf + f_bias), S <- diag(f) S + (1 - f) v^T, o = S^T q.
 * state: fp32 [slots, H, dk, dv]; seqs: int32 [n_seqs, 4] = (first packed row, token count, state slot, fresh);
 * fresh != 0 starts from a zero state.  The final state is written back.  o_raw: fp32 [n_tok, H, dv].  max_count: the
 * largest token count among seqs (a hint: portions of 8 tokens or more and key sizes up to 128 take the kernel that
 * keeps the state in registers, steps of single tokens the one that keeps it in shared memory). */
int b200_gated_scan(float* o_raw, const void* zq, const void* zf, const void* v, int64_t in_stride, const void* f_bias,
                    const void* lower, float* state, const int32_t* seqs, int n_seqs, int max_count, int H, int dk, int dv,
                    int dtype, void* stream);

/* out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * weight;  x fp32 [rows, dv], weight T [dv], out T. */
int b200_head_rmsnorm(void* out, const float* x, const void* weight, float eps, int64_t rows, int dv, int dtype,
                      void* stream);

/* out[r] = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u * rsqrt(mean(u^2) + eps) over the row; coef = (a, b, c, e). */
int b200_polynorm(void* out, const void* z, int64_t z_stride, const void* coef, float eps, int rows, int ff, int dtype,
                  void* stream);

/* The `top` largest of E fp32 logits per token (ties: lowest index); weights = sigmoid(logit). */
int b200_sigmoid_topk(int32_t* ids, float* weights, const float* logits, int n_tok, int E, int top, void* stream);

/* xs[r] = T(weights[src[r]] * h[src[r] / top]): the expert-sorted, input-scaled rows. */
int b200_scaled_gather(void* xs, const void* h, const float* weights, const int64_t* src, int64_t n_rows, int top,
                       int width, int dtype, void* stream);

/* Grouped linear over expert-sorted rows (16-bit dtypes, K a multiple of 8): out[r] = xs[r] . w[e]^T for
 * offsets[e] <= r < offsets[e + 1].  xs T [rows, K], w T [E, N, K], offsets int32 [E + 1] ON THE DEVICE, out T [rows, N].
 * max_rows: a bound on the rows of any one expert (the total row count will do); it sizes the grid only. */
int b200_grouped_linear_supported(int K, int dtype);
int b200_grouped_linear(void* out, const void* xs, const void* w, const int32_t* offsets, int64_t max_rows, int E, int N,
                        int K, int dtype, void* stream);

/* y = g' * sigmoid(alpha * g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit); gu rows = g | u. */
int b200_clamped_glu(void* y, const void* gu, int64_t rows, int ff, float limit, float alpha, int dtype, void* stream);

/* out[n] = sum over k (ascending) of ys[where[n * top + k]], fp32. */
int b200_expert_combine(float* out, const void* ys, const int64_t* where, int64_t n_tok, int top, int width, int dtype,
                        void* stream);

/* ---- pieces for hybrid designs: one norm per layer, mixer and feed-forward added to the residual together ---------- */

/* SeqSpan rows used below: int32 [n_seqs, 4] = (first packed row, token count, state slot, fresh); fresh != 0: the
 * sequence starts in this step and its carried state counts as zero. */

/* out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * (weight_offset + weight); x rows are fp32 (x_is_f32) or T, with row
 * strides in elements; out T. */
int b200_rms_norm(void* out, int64_t out_stride, const void* x, int64_t x_stride, int x_is_f32, const void* weight,
                  float weight_offset, float eps, int rows, int width, int dtype, void* stream);

/* x[r] += (a[r] + b[r]) in fp32, in place (b may be NULL); with w_next, out_next[r] = rms_norm(x[r]; w_next) in T. */
int b200_residual_add2_norm(float* x, const void* a, int64_t a_stride, const void* b, int64_t b_stride, const void* w_next,
                            float weight_offset, void* out_next, float eps, int rows, int width, int dtype, void* stream);

/* xIELU: z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2;  pq = (p, q) in T. */
int b200_xielu(void* out, const void* z, int64_t z_stride, const void* pq, int rows, int ff, int dtype, void* stream);

/* Rotary positions on the first rot_dims dimensions of every q head (in place) and k head, pair (i, i + rot_dims/2)
 * (interleaved: (2i, 2i + 1)) turned by pos * rot_base^(-2i / rot_dims); with rotate_values, the values are turned the
 * same way over their whole width dv by pos * rot_base^(-2m / dv).  k and v go to the pools ([max_blocks, G, block_size,
 * dk | dv]) at slot_mapping (negative = skip).  Angles are formed in double precision.  value_rot (may be NULL): fp32
 * [n_tok, dv / 2, 2] receives (cos, sin) of every value pair's angle, for the attention kernel that turns outputs back. */
int b200_rotary_kv_append(void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                          void* k_pool, void* v_pool, const int64_t* slot_mapping, const int32_t* tok_pos, int n_tok, int H,
                          int G, int dk, int dv, int rot_dims, float rot_base, int rotate_values, int interleaved,
                          int block_size, int64_t max_blocks, float* value_rot, int dtype, void* stream);

/* pool[slot] = rms_norm(x[n]; weight): latent rows of `width` into a one-head pool [max_blocks, 1, block_size, width]. */
int b200_norm_append(const void* x, int64_t x_stride, const void* weight, float weight_offset, float eps, void* pool,
                     const int64_t* slot_mapping, int n_tok, int width, int dtype, void* stream);

/* Softmax attention of packed query rows over the paged cache (which already holds this step's keys and values).
 *   raw(h, i, j)   = (q_ih . k_j) * scale                      k of kv head h / (H / G)
 *   score(h, i, j) = sum_g talk[h][g] raw(g, i, j)              (talk NULL: score = raw)
 *   softcap > 0    : score <- softcap * tanh(score / softcap)
 *   visible        : j <= i and (window <= 0 or i - j < window or j < keep_first)
 *   out(i, h)      = sum_j exp(score) v_j / (sum_j exp(score) + exp(sink[h]))     (sink NULL: no extra term)
 * With unrotate, pair m of out(i, h) is turned by -pos_i * rot_base^(-2m / dv) (the inverse of the rotation the
 * values were stored with); with gate, out(i, h) *= sigmoid(gate[i][h]).  q element (n, h, d) is at
 * n * q_tok_stride + h * q_head_stride + d, the output likewise; tok_row[n] is the token's row of block_tables. */
int b200_mixed_paged_attn(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q, int64_t q_tok_stride,
                          int64_t q_head_stride, const void* gate, int64_t gate_stride, const void* k_pool,
                          const void* v_pool, const int32_t* block_tables, int table_stride, const int32_t* tok_row,
                          const int32_t* tok_pos, int n_tok, const float* talk, const float* sink, float scale,
                          float softcap, int window, int keep_first, int unrotate, int interleaved, float rot_base, int H,
                          int G, int dk, int dv, int block_size, int dtype, void* stream);

/* The same with three more parameters.  chunk > 0: a position also sees only keys j with j / chunk == i / chunk (blocks
 * counted from position 0 of the sequence).  v_row: elements between value rows of v_pool, so that the values may be the
 * first dv columns of wider rows (v_pool == k_pool with one kv head: a latent row serves as key over its whole width dk
 * and as value over its first dv columns).  v_div: value head = key head / v_div; v_pool holds G / v_div heads per block
 * (several score maps over the same values).  out_f32 != 0: `out` is fp32 whatever T is (strides in elements; not with
 * unrotate), for results that are combined before they are rounded. */
int b200_mixed_paged_attn_ext(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q,
                              int64_t q_tok_stride, int64_t q_head_stride, const void* gate, int64_t gate_stride,
                              const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                              const int32_t* tok_row, const int32_t* tok_pos, int n_tok, const float* talk,
                              const float* sink, float scale, float softcap, int window, int keep_first, int chunk,
                              int unrotate, int interleaved, float rot_base, int H, int G, int dk, int dv, int v_row,
                              int v_div, int out_f32, int block_size, int dtype, void* stream);

/* The same attention on the tensor cores (16-bit T; dk a multiple of 16, dv a multiple of 8 up to 256, and a shared-
 * memory budget that b200_mixed_prompt_attn_supported checks; same_pool: keys and values are one pool).  tiles: int32
 * [n_tiles, 3] = (first packed row, token count <= 16, block-table row); a tile's tokens are consecutive positions of
 * one sequence.  Outputs are turned back when value_rot (the table b200_rotary_kv_append wrote for these tokens) is
 * given.  Scores, mask and softmax are fp32; the weights are rounded to T only as the operand of the P.V product. */
int b200_mixed_prompt_attn_supported(int H, int G, int dk, int dv, int has_talk, int same_pool, int unrotate, int dtype);
/* Steps of few tokens leave most SMs idle: with n_splits > 1 the key tiles of every query tile are divided over
 * n_splits CTAs, which leave (max, sum, unnormalised output) in `workspace` (fp32, b200_mixed_prompt_attn_workspace
 * bytes), and a second launch merges them.  b200_mixed_prompt_attn_splits proposes n_splits for a step of n_tiles
 * query tiles whose longest walk is key_tiles tiles of 32 keys.  n_tok: packed rows of the step (every row lies in
 * exactly one tile). */
int b200_mixed_prompt_attn_splits(int n_tiles, int key_tiles, int H, int G, int dk, int dv, int has_talk, int same_pool,
                                  int unrotate, int dtype);
size_t b200_mixed_prompt_attn_workspace(int n_splits, int n_tok, int H, int dv);
int b200_mixed_prompt_attn(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q, int64_t q_tok_stride,
                           int64_t q_head_stride, const void* gate, int64_t gate_stride, const void* k_pool,
                           const void* v_pool, const int32_t* block_tables, int table_stride, const int32_t* tiles,
                           int n_tiles, const int32_t* tok_pos, int n_tok, const float* talk, const float* sink,
                           float scale, float softcap, int window, int keep_first, const float* value_rot, int interleaved,
                           int H, int G, int dk, int dv, int block_size, int n_splits, float* workspace, int dtype,
                           void* stream);

/* b200_mixed_prompt_attn with chunk, v_row and v_div as in b200_mixed_paged_attn_ext (v_row a multiple of 8).
 * heads_as_rows != 0 (steps of single tokens over ONE kv head, G == 1, no talk / gate / value_rot): every tile is one
 * token (count 1) and the 16 rows of a tensor-core tile are 16 consecutive query heads instead of 16 tokens, so a warp
 * serves 16 heads against the staged keys.  For b200_mixed_prompt_attn_splits such a step counts (H + 15) / 16 heads.
 * out_f32 as in b200_mixed_paged_attn_ext (not with value_rot). */
int b200_mixed_prompt_attn_ext(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q,
                               int64_t q_tok_stride, int64_t q_head_stride, const void* gate, int64_t gate_stride,
                               const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                               const int32_t* tiles, int n_tiles, const int32_t* tok_pos, int n_tok, const float* talk,
                               const float* sink, float scale, float softcap, int window, int keep_first, int chunk,
                               const float* value_rot, int interleaved, int H, int G, int dk, int dv, int v_row, int v_div,
                               int heads_as_rows, int out_f32, int block_size, int n_splits, float* workspace, int dtype,
                               void* stream);

/* out[t, c] = silu(sum_i w[c][i] * x[t - (taps - 1 - i), c]) per sequence (SeqSpan rows); inputs before the portion
 * come from tail [slots, taps - 1, C] (fp32, oldest first), which then receives the portion's last taps - 1 inputs. */
int b200_causal_conv_silu(void* out, int64_t out_stride, const void* x, int64_t x_stride, const void* w, float* tail,
                          const int32_t* seqs, int n_seqs, int max_count, int C, int taps, int dtype, void* stream);

/* Gated delta rule per (sequence, head) over the sequence's tokens of this step, in order:
 *   q <- q / sqrt(sum q^2 + unit_eps) * q_scale, k <- k / sqrt(sum k^2 + unit_eps)          (per head)
 *   g = exp(-exp(a_log[h]) * softplus(a_logit + dt_bias)) [dk], beta = sigmoid(beta_logit)
 *   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
 * q, k: T rows of G*dk (value head h reads head h / (H / G)), v: T rows of H*dv, all with row stride in_stride;
 * a_logit: T [n, H*dk]; state fp32 [slots, H, dk, dv]; o_raw fp32 [n_tok, H, dv]. */
int b200_delta_scan(float* o_raw, const void* q, const void* k, const void* v, int64_t in_stride, const void* beta_logit,
                    int64_t beta_stride, const void* a_logit, int64_t a_stride, const void* dt_bias, const void* a_log,
                    float* state, const int32_t* seqs, int n_seqs, int H, int G, int dk, int dv, float unit_eps,
                    float q_scale, int dtype, void* stream);

/* out[n, h, :] = x[n, h, :] * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate[n, h, :]); x fp32 [n_tok, H, dv],
 * gate T rows of H*dv (NULL: no gate), out T [n_tok, H*dv]. */
int b200_head_rmsnorm_gated(void* out, const float* x, const void* weight, const void* gate, int64_t gate_stride, float eps,
                            int64_t n_tok, int H, int dv, int dtype, void* stream);

/* ---- pieces for designs with side-by-side mixers, post-norm sublayers and grouped softmax routing ------------------ */

/* Per-head RMS norm of q (in place) and k with weights q_norm / k_norm (T [dk]; NULL: no norm), then rotary positions on
 * the first rot_dims dimensions of every head, pair (i, i + rot_dims/2) (interleaved: (2i, 2i + 1)) turned by
 * pos * freqs[i]; freqs: rot_dims / 2 doubles ON THE DEVICE (any frequency rescaling is the caller's).  k and v go to the
 * pools ([max_blocks, G, block_size, dk | dv]) at slot_mapping (negative = skip). */
int b200_qknorm_rotary_append(void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                              const void* q_norm, const void* k_norm, float eps, const double* freqs, int rot_dims,
                              int interleaved, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                              const int32_t* tok_pos, int n_tok, int H, int G, int dk, int dv, int block_size,
                              int64_t max_blocks, int dtype, void* stream);

/* The same with Gv value heads in v [n_tok, Gv*dv] and v_pool [max_blocks, Gv, block_size, dv] (layouts whose key heads
 * outnumber the value heads: several score maps over the same values). */
int b200_qknorm_rotary_append_ext(void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                  int64_t v_stride, const void* q_norm, const void* k_norm, float eps, const double* freqs,
                                  int rot_dims, int interleaved, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                                  const int32_t* tok_pos, int n_tok, int H, int G, int Gv, int dk, int dv, int block_size,
                                  int64_t max_blocks, int dtype, void* stream);

/* Retention per (sequence, head) over the sequence's tokens of this step, in order (SeqSpan rows as above):
 *   S <- decay[h] S + (k_scale k_t) v_t^T;   o_t = S^T q_t
 * q, k T [n, H*dk] and v T [n, H*dv] are column slices of one tensor (row stride in_stride); decay fp32 [H]; state fp32
 * [slots, H, dk, dv], read unless the sequence is fresh and written back; o_raw fp32 [n, H, dv].  dk <= 512. */
int b200_retention_scan(float* o_raw, const void* q, const void* k, const void* v, int64_t in_stride, const float* decay,
                        float k_scale, float* state, const int32_t* seqs, int n_seqs, int H, int dk, int dv, int dtype,
                        void* stream);

/* Long portions in parallel.  Run b200_retention_scan over SEGMENTS of a portion as if each were a fresh sequence with a
 * slot of its own in a scratch state tensor seg_state [n_segs, H, dk, dv]; then
 *   b200_retention_carry        walks every parent's segments (parents int32 [n_parents, 4] = first segment, segments,
 *                               state slot, fresh): P_0 = the carried state (0 if fresh), P_(j+1) = decay^(n_j) P_j + E_j;
 *                               seg_state[j] becomes P_j, the parent's slot the final state;
 *   b200_retention_apply_carry  o_t += decay^(t - t0 + 1) P_j^T q_t for every token of every segment.
 * seg_spans are the SeqSpan rows the scan ran with. */
int b200_retention_carry(float* state, float* seg_state, const int32_t* parents, int n_parents, const int32_t* seg_spans,
                         const float* decay, int H, int dk, int dv, void* stream);
int b200_retention_apply_carry(float* o_raw, const void* q, int64_t in_stride, const float* seg_state,
                               const int32_t* seg_spans, int n_segs, const float* decay, int H, int dk, int dv, int dtype,
                               void* stream);

/* out[n, h*dv + i] = x[n][h][i] * rsqrt(mean_i x^2 + eps) * weight[i] * act(gate[n, h*dv + i]) * out_scale; weight and
 * gate may be NULL; gate_act 0: sigmoid, 1: SiLU.  x fp32 [n, H, dv]; out T with row stride out_stride. */
int b200_head_norm_act_gate(void* out, int64_t out_stride, const float* x, const void* weight, const void* gate,
                            int64_t gate_stride, int gate_act, float out_scale, float eps, int64_t n_tok, int H, int dv,
                            int dtype, void* stream);

/* y = sa a + sb b (b may be NULL);  x += layer_scale * w_norm * y * rsqrt(mean(y^2) + eps)  in place on the fp32
 * residual (layer_scale T [width] may be NULL); x_out (T, may be NULL) receives the new x.  a is fp32 (a_is_f32) or T. */
int b200_branch_postnorm_residual(float* x, const void* a, int64_t a_stride, int a_is_f32, float sa, const void* b,
                                  int64_t b_stride, float sb, const void* w_norm, const void* layer_scale, void* x_out,
                                  float eps, int rows, int width, int dtype, void* stream);

/* out[i] = T(x[i]) for n fp32 numbers. */
int b200_cast_rows(void* out, const float* x, int64_t n, int dtype, void* stream);

/* Routing with softmax scores s over E router outputs: choice scores c = s + correction (NULL: c = s); the experts form
 * `groups` equal groups of neighbours, only the `keep` groups with the largest best c can be chosen; the `top` largest c
 * among them are chosen (ties: lowest index); weights = their s over (the sum of their s + sum_floor). */
int b200_softmax_group_topk(int32_t* ids, float* weights, const float* logits, const float* correction, float sum_floor,
                            int n_tok, int E, int top, int groups, int keep, void* stream);

/* xs[r] = h[src[r] / top]: the expert-sorted rows, unscaled. */
int b200_gather_rows(void* xs, const void* h, const int64_t* src, int64_t n_rows, int top, int width, int dtype,
                     void* stream);

/* out[n] = sum over k (ascending) of weights[n][k] * (ids[n][k] < n_real ? ys[where[n * top + k]] : x_self[n])
 *          + shared_rows[n] (may be NULL), fp32.  Experts numbered n_real and up return the token's own fp32 row. */
int b200_weighted_expert_combine(float* out, const void* ys, const int64_t* where, const int32_t* ids, const float* weights,
                                 const float* x_self, const void* shared_rows, int64_t n_tok, int top, int n_real,
                                 int width, int dtype, void* stream);

/* ---- pieces for designs with token shift, sigmoid-gated post-norm sublayers, a decoupled rotated key part --------- */

/* out[t] = T(x[t] + (x[t - 1] - x[t]) * mu) per channel over each sequence's tokens (SeqSpan rows); the row before a
 * portion's first token comes from state [slots, width] (fp32; zero when the sequence is fresh), which then receives the
 * portion's last row.  x fp32 [n_tok, width] contiguous; out T rows with stride out_stride; x_cast (may be NULL) T
 * [n_tok, width] receives the unshifted rows rounded to T.  max_count: the largest token count among seqs. */
int b200_token_shift(void* out, int64_t out_stride, void* x_cast, const float* x, const void* mu, float* state,
                     const int32_t* seqs, int n_seqs, int max_count, int width, int dtype, void* stream);

/* Latent attention with a decoupled rotated key part.  dkv rows (T, stride dkv_stride) hold rank + rot_width columns:
 * pool[slot] = [rms_norm(dkv[:rank]; c_norm) | turn(dkv[rank:])] (a one-head pool of rows rank + rot_width; negative slot =
 * skip), and q_out[n, h, :] = turn(q_rot[n, h, :]) for the rot_width rotated columns of every query head (element (n, h, i)
 * at n * tok_stride + h * head_stride + i; q_out must not overlap q_rot).  turn: pairs (2i, 2i + 1), i < rot_dims / 2, go to
 * (u c - v s, v c + u s) with c, s = gain * cos, sin(pos * freqs[i]); columns from rot_dims on pass unchanged.  freqs:
 * rot_dims / 2 doubles ON THE DEVICE. */
int b200_latent_rotary_append(const void* q_rot, int64_t q_tok_stride, int64_t q_head_stride, void* q_out,
                              int64_t qo_tok_stride, int64_t qo_head_stride, const void* dkv, int64_t dkv_stride,
                              const void* c_norm, float eps, const double* freqs, float gain, int rot_dims, void* pool,
                              const int64_t* slot_mapping, const int32_t* tok_pos, int n_tok, int H, int rot_width,
                              int rank, int dtype, void* stream);

/* Two score maps per head over the same values: with a1, a2 = a[n, (h / rep) * 2 rep + (h % rep) (+ rep), :],
 * out[n, h * dv + i] = o_i * rsqrt(mean_i o^2 + eps) * out_scale, o = a1 - lam * a2.  a: T or fp32 (a_is_f32), element (n, head, i) at
 * n * a_tok_stride + head * a_head_stride + i; out T rows with stride out_stride. */
int b200_head_diff_norm(void* out, int64_t out_stride, const void* a, int64_t a_tok_stride, int64_t a_head_stride,
                        int a_is_f32, float lam, float out_scale, float eps, int64_t n_tok, int H, int rep, int dv, int dtype,
                        void* stream);

/* y = a * sigmoid(gate) (gate T rows, may be NULL);  x += (weight_offset + w_norm) * y * rsqrt(mean(y^2) + eps)  in place
 * on the fp32 residual; x_out (T, may be NULL) receives the new x.  a is fp32 (a_is_f32) or T. */
int b200_gated_postnorm_residual(float* x, const void* a, int64_t a_stride, int a_is_f32, const void* gate,
                                 int64_t gate_stride, const void* w_norm, float weight_offset, void* x_out, float eps,
                                 int rows, int width, int dtype, void* stream);

/* out[r, c] = max(z[r, c], 0)^2; z rows with stride z_stride, out contiguous [rows, ff]. */
int b200_relu_squared(void* out, const void* z, int64_t z_stride, int64_t rows, int ff, int dtype, void* stream);

/* out[n, c] = gelu_tanh(z[n, c]) * table[tokens[n]][col0 + c], c < d; gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z +
 * 0.044715 z^3))).  table T rows with stride table_stride, tokens int64. */
int b200_gated_table_rows(void* out, const void* z, int64_t z_stride, const void* table, int64_t table_stride, int col0,
                          const int64_t* tokens, int64_t n_tok, int d, int dtype, void* stream);

/* logits[n, e] = sum_i x[n, i] * w[e, i] + bias[e] in fp32 (bias may be NULL): x fp32 [n_tok, width] and w fp32 [E, width]
 * contiguous.  Meant for routers (few outputs); every sum runs in an order fixed by the width, whatever n_tok is. */
int b200_router_logits(float* logits, const float* x, const float* w, const float* bias, int64_t n_tok, int E, int width,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MIXERS_H_ */
