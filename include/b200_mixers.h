/*
 * b200_mixers.h -- C ABI of libb200mix.so: sequence mixers and feed-forward pieces of hybrid decoders on B200 (sm_100a):
 * latent attention with a softmax sink over a paged cache of compressed keys, grouped-query attention with a sliding
 * window (optionally with kept first tokens and mixed heads) and a linear distance bias, recurrences with per-sequence state
 * slots (selective scan, gated diagonal recurrence, gated delta rule), routed experts, and the row-wise ops around them
 * (embedding into an fp32 residual stream, residual update + weight-only layer norm, norm on a sublayer's output, RMS norm,
 * feed-forward activations).
 *
 * Conventions are those of b200_paged_attn.h: 0 or a negative B200_E* code; the caller owns every buffer; nothing
 * synchronises the host and every launch goes to the stream passed in, so a step can be captured in a CUDA graph;
 * per-step variation flows through device-resident metadata only.
 *
 * `is32` selects the activation / weight / cache element type: 0 = bf16 (serving), 1 = fp32 (everything in 32 bits).
 * Norm statistics, softmax, router scores, the residual stream and the recurrent state are fp32 in both.
 *
 * Step metadata.  A varlen step (prompt portions, single tokens, or both) passes cu_q / cu_k, int32 [num_seqs + 1]
 * cumulative counts of this step's tokens and of the tokens each sequence holds after the step, and ctx_lens = NULL.
 * A decode step passes cu_q = cu_k = NULL and ctx_lens, int32 [num_seqs]: one token per row, ctx_lens[s] tokens after the
 * step, 0 marking a padding row that is skipped.  Token i of a sequence with q tokens in the step and k after it sits at
 * position k - q + i.
 */
#ifndef B200_MIXERS_H
#define B200_MIXERS_H

#include <stddef.h>
#include <stdint.h>

#include "b200_paged_attn.h" /* the B200_E* codes */

#ifdef __cplusplus
extern "C" {
#endif

int b200m_abi_version(void);

/* out[i, :] = table[ids[i], :] as fp32 (the residual stream); copy (optional) receives the same rows in the table's type. */
int b200m_embed(const int64_t* ids, const void* table, float* out, void* copy, int n, int width, int64_t vocab, int is32,
                void* stream);

/* Token embedding times a constant plus a hashed embedding of the (previous token, token) pair (pair = NULL: none):
 * out = table[id] * scale + pair[(prev * mul_prev + id * mul_cur) mod buckets]; a sequence's first token takes row `buckets`.
 * The token before a portion comes from prev_tok[state_slots[s]] (int64 per state slot), which a second launch leaves holding
 * the portion's last token.  A padding row of a decode step (ctx_lens = 0) is zeroed. */
int b200m_embed_pair(const int64_t* ids, const void* table, float scale, const void* pair, int64_t buckets, int64_t mul_prev,
                     int64_t mul_cur, int64_t* prev_tok, const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                     const int32_t* ctx_lens, float* out, void* copy, int num_seqs, int max_q, int width, int64_t vocab, int is32,
                     void* stream);

/* Norm on a sublayer's output, then the residual update: x[r, :] += mult * y / sqrt(mean(y^2) + eps) * (w_offset + w), y =
 * y[r, :] (activation type) or y32[r, :] (fp32).  copy (optional): the updated rows in the activation type. */
int b200m_add_normed(float* x, const void* y, const float* y32, const void* w, float mult, float w_offset, void* copy, int rows,
                     int cols, float eps, int is32, void* stream);

/* b200m_add_normed, then (out_next != NULL) out_next[r, :] = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * (next_offset + w_next) of the
 * updated rows: the norm that closes one sublayer, the residual update and the norm that opens the next, in one pass. */
int b200m_add_normed_norm(float* x, const void* y, const float* y32, const void* w, float mult, float w_offset, void* copy,
                          const void* w_next, float next_offset, void* out_next, int rows, int cols, float eps, int is32,
                          void* stream);

/* out[i, :] = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * (w_offset + w), r = rows_idx[i] (or i when NULL), x the fp32 stream. */
int b200m_rmsnorm_rows(const float* x, const int32_t* rows_idx, const void* w, float w_offset, void* out, int rows, int cols,
                       float eps, int is32, void* stream);

/* x[r, :] += a[r, :] + b[r, :] + b32[r, :] (each optional; the terms are summed first), then, unless out is NULL,
 * out[r, :] = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w.  With rows_idx (int32 [rows]) nothing is added and
 * out[i, :] is the norm of row rows_idx[i]. */
int b200m_add_layernorm(float* x, const void* a, const void* b, const float* b32, const void* w, void* out,
                        const int32_t* rows_idx, int rows, int cols, float eps, int is32, void* stream);

/* out = x / sqrt(mean(x^2) + eps) * w over the first `cols` elements of each (strided) row. */
int b200m_rmsnorm(const void* x, int64_t x_stride, const void* w, void* out, int64_t out_stride, int rows, int cols,
                  float eps, int is32, void* stream);

/* kind 0: x = [gate | up] (2n per row), out = gelu_tanh(gate) * up;  1: out = relu(x)^2 (n per row);  2: silu(gate) * up;
 * 3: out = gelu_tanh(x) (n per row). */
int b200m_ff_act(const void* x, void* out, int64_t rows, int n, int kind, int is32, void* stream);

/* Gated unit with clamped branches: x = [gate | up] (2n of x_stride elements per row), g = min(gate, limit), u = clamp(up, -limit, limit),
 * out = g * sigmoid(alpha * g) * (u + 1). */
int b200m_ff_glu_clamped(const void* x, int64_t x_stride, void* out, int64_t rows, int n, float limit, float alpha, int is32, void* stream);

/* One sublayer's close in a layer that gates and norms the sublayer's result and scales it per column:
 *   t = y * sigmoid(gate)  (gate NULL: t = y);   x += t / sqrt(mean(t^2) + eps) * w_out;
 *   out_next (optional) = x / sqrt(mean(x^2) + eps) * next_scale * w_next   (w_next NULL: 1).
 * x fp32 [rows, cols] in place; y in the activation type (or y32, fp32), contiguous; gate in the activation type with row stride
 * gate_stride (a column slice of a wider projection); w_out, w_next fp32 [cols]; out_next in the activation type. */
int b200m_gated_add_normed_norm(float* x, const void* y, const float* y32, const void* gate, int64_t gate_stride,
                                const float* w_out, const float* w_next, float next_scale, void* out_next, int rows, int cols,
                                float eps, int is32, void* stream);

/* x <- cap * tanh(x / cap), fp32, in place (n elements). */
int b200m_softcap(float* x, int64_t n, float cap, void* stream);

/* ---- latent attention ---------------------------------------------------------------------------------------------- */

/* Per token: cache[slot] = [ rms_norm(dkv[:rank]) * norm_w | rotate(dkv[rank : rank + rot_dim]) ].  The rotation turns the
 * pairs (2i, 2i+1), i < rope_dims / 2, by cos_sin[position] = [cos (rope_dims/2) | sin (rope_dims/2)] (fp32, any magnitude
 * factor folded in); elements past rope_dims pass unchanged.  layout 1: the pairs are (i, i + rope_dims / 2) instead.
 * slot < 0 skips the token. */
int b200m_latent_store(const void* dkv, int64_t stride, const void* norm_w, const float* cos_sin, int rope_dims,
                       const int64_t* positions, const int32_t* slots, void* cache, int n, int rank, int rot_dim, float eps,
                       int layout, int is32, void* stream);

/* Multi-query attention of every head over the cached rows, causal, with a per-head sink logit in the softmax denominator
 * (sink NULL: an ordinary softmax).  window > 0: position i sees the keys j with 0 <= i - j < window only.  layout: the pairing of
 * the rotated query part, as for b200m_latent_store.
 * q_lat [H, total_q, rank]: queries already mapped into the latent space; q_raw: the raw query projection (token t, head h at
 * t * q_tok_stride + h * q_head_stride), whose rot_dim elements from q_rot_off on are rotated here by the token's position.  out [H, total_q, rank].
 * bf16 runs on the tensor cores (mma.sync over staged key tiles); fp32, or flags & 1, on the fp32 FMA pipe.
 * splits > 1 (bf16 decode steps only, ignored elsewhere): the keys of every sequence are shared out over `splits` CTAs whose
 * partial results, fp32 [num_seqs, 4 * splits, num_heads, rank + 2] in `part`, a second launch merges. */
int b200m_latent_attention(const void* q_lat, const void* q_raw, int64_t q_tok_stride, int q_head_stride, int q_rot_off, const void* cache,
                           const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q,
                           const int32_t* cu_k, const int32_t* ctx_lens, const float* sink, const float* cos_sin,
                           int rope_dims, void* out, int total_q, int num_seqs, int max_q, int num_heads, int rank,
                           int rot_dim, float scale, int window, int layout, int is32, int flags, int splits, float* part,
                           void* stream);

/* ---- windowed grouped-query attention ------------------------------------------------------------------------------ */

/* Per token of qkv = [q (q_cols) | k (k_cols) | v (v_cols)] (row stride `stride`): q <- q / rms(q) * q_norm_w over ALL q_cols
 * at once, in place (skipped when q_norm_w is NULL); cache[slot] = [k / rms(k) * k_norm_w | v] (k copied as is when
 * k_norm_w is NULL).  k_cols = v_cols = 0: queries only.  slot < 0 skips the store. */
int b200m_qk_norm_store(void* qkv, int64_t stride, int q_cols, int k_cols, int v_cols, const void* q_norm_w,
                        const void* k_norm_w, const int32_t* slots, void* cache, int n, float eps, int is32, void* stream);

/* Per token and head of x (row stride `stride`; q heads at q_off, key heads at k_off, value heads at v_off): q <- q / rms(q) *
 * q_norm_w with ONE weight vector of `dim` elements for all heads (NULL: no norm), then the pairs (2i, 2i+1), i < rope_dims / 2,
 * turned by cos_sin[position] = [cos (rope_dims/2) | sin (rope_dims/2)] (fp32; NULL: no rotation), in place; keys the same with
 * k_norm_w into cache[slot] = [k (G * dim) | v (G * vdim)]; values divided by their root mean square per head (v_unit_norm) or
 * copied; v_cos_sin (optional, fp32 [positions, v_rope_dims]): the value pairs (2m, 2m+1), m < v_rope_dims / 2, are turned by the
 * token's position before the store.  cache NULL or slot < 0: queries only. */
int b200m_headnorm_rope_store(void* x, int64_t stride, int q_off, int k_off, int v_off, int num_heads, int num_kv_heads, int dim,
                              int vdim, const void* q_norm_w, const void* k_norm_w, int v_unit_norm, const float* cos_sin,
                              int rope_dims, const float* v_cos_sin, int v_rope_dims, const int64_t* positions, const int32_t* slots,
                              void* cache, int n, float eps, int is32, void* stream);

/* out[t, h, :] = rotate(acc[t, h, :], sign * position[t]) * sigmoid(gate[t, h, :]): per-head attention results turned (back) by
 * the query's position and gated.  acc element (t, h, c) at t * acc_tok_stride + h * acc_head_stride + c (fp32 when acc_f32, else
 * the activation type); cos_sin fp32 [positions, rope_dims] = [cos | sin] (NULL: no rotation), pairs (2m, 2m+1) for layout 0,
 * (m, m + rope_dims / 2) for layout 1, elements past rope_dims unchanged; gate (optional) with row stride gate_stride; out
 * [n, num_heads * vdim] in the activation type with row stride out_stride. */
int b200m_head_rotate_gate(const void* acc, int acc_f32, int64_t acc_tok_stride, int64_t acc_head_stride, const float* cos_sin,
                           int rope_dims, int layout, float sign, const int64_t* positions, const void* gate, int64_t gate_stride,
                           void* out, int64_t out_stride, int n, int num_heads, int vdim, int is32, void* stream);

/* out[t, h, :] = out_scale * sigmoid(gate[t, h, :]) * sum_g mix[h, g] * acc[t, g, h / (H / G), :]: the heads' attention weights mixed after
 * the softmax, for acc [n, H, G, vdim] from b200m_window_attention with all_values (fp32 when acc_f32, else the activation
 * type).  mix fp32 [H, H]; gate (optional) with row stride gate_stride; out with row stride out_stride. */
int b200m_head_mix_gate(const void* acc, int acc_f32, const float* mix, const void* gate, int64_t gate_stride, void* out,
                        int64_t out_stride, float out_scale, int n, int num_heads, int num_kv_heads, int vdim, int is32, void* stream);

/* Causal attention of num_heads query heads over num_kv_heads cached key/value heads (head h reads h / (num_heads /
 * num_kv_heads)): score = q . k * scale - slopes[h] * (i - j) (slopes NULL: no bias), visible keys 0 <= i - j < window
 * or j < keep_first (window <= 0: all j <= i), ordinary softmax.  all_values: every query head's weights are applied to the
 * values of EVERY value head, out [total_q, num_heads, num_kv_heads, vdim] (for b200m_head_mix_gate).  flags & 2: out is fp32.  A cache row is row_elems long: key head g at g * dim, value head g at
 * v_off + g * vdim.  q [total_q, >= num_heads * dim] with row stride q_stride; out [total_q, num_heads * vdim].
 * bf16 with dim and vdim in {32, 64, 128} runs on the tensor cores unless flags & 1; everything else on the fp32 FMA pipe.
 * splits > 1 (bf16 tensor-core decode steps only): the visible keys of every row are shared out over `splits` CTAs whose
 * partials, fp32 [num_seqs, splits, num_heads (x num_kv_heads with all_values), vdim + 2] in `part`, a second launch merges. */
int b200m_window_attention(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off,
                           const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q,
                           const int32_t* cu_k, const int32_t* ctx_lens, const float* slopes, int window, int keep_first,
                           int all_values, void* out, int total_q, int num_seqs, int max_q, int num_heads, int num_kv_heads,
                           int dim, int vdim, float scale, int is32, int flags, int splits, float* part, void* stream);

/* ---- selective scan ------------------------------------------------------------------------------------------------ */

/* Depthwise causal convolution (w [channels, taps], last tap on the current token) + bias, then SiLU when act = 1 (act = 0:
 * nothing); the taps - 1 inputs before
 * a portion come from conv_state [slots, taps - 1, channels] (fp32) when the sequence has tokens behind it, zeros
 * otherwise; afterwards the slot holds the last taps - 1 inputs. */
int b200m_causal_conv(const void* x, int64_t x_stride, const void* w, const void* bias, float* conv_state,
                      const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens, void* out,
                      int num_seqs, int max_q, int channels, int taps, int act, int is32, void* stream);

/* S <- exp(dt A) S + dt u B;  y = (S C + D u) * silu(z), dt = softplus(dt_raw + dt_bias); A [channels, nstate] fp32;
 * state [slots, channels, nstate] fp32, started from zero when the sequence has no tokens behind it.
 * With a workspace (ws: fp32, num_seqs * ceil(max_q / chunk_len) * channels * (nstate + 1)) portions longer than chunk_len
 * run as chunks in parallel (local pass, carry pass, output pass: three launches); ws = NULL: one launch, serial per sequence. */
int b200m_selective_scan(const void* u, const void* dt_raw, const void* dt_bias, const float* A, const void* Bm, const void* Cm,
                         int64_t bc_stride, const void* Dv, const void* z, int64_t z_stride, float* state,
                         const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens, void* y,
                         int num_seqs, int channels, int nstate, int chunk_len, int max_q, float* ws, int is32, void* stream);

/* ---- gated diagonal recurrence and gated delta rule ------------------------------------------------------------------ */

/* Per channel c (block b = c / block_channels, j = c % block_channels), with gates fp32 [channels / block_channels, rows, 2 *
 * block_channels] holding for every token row the block's pre-activations of r, then of i, and gate_bias laid out alike:
 *     r = sigmoid(gates_r + bias_r), i = sigmoid(gates_i + bias_i), a = exp(rate[c] * r)   (rate <= 0)
 *     S <- a S + sqrt(1 - a^2) * i * u;   out = S * gelu_tanh(y)
 * state fp32 [slots, channels], started from zero when the sequence has no tokens behind it.  With a workspace (ws: fp32,
 * num_seqs * ceil(max_q / chunk_len) * channels * 2) portions longer than chunk_len run as chunks in parallel (three
 * launches); ws = NULL: one launch, serial per sequence. */
int b200m_diag_scan(const void* u, int64_t u_stride, const float* gates, int64_t rows, const float* gate_bias, const float* rate,
                    const void* y, int64_t y_stride, float* state, const int32_t* state_slots, const int32_t* cu_q,
                    const int32_t* cu_k, const int32_t* ctx_lens, void* out, int num_seqs, int max_q, int channels,
                    int block_channels, int chunk_len, float* ws, int is32, void* stream);

/* Gated delta rule.  Per token x holds q and k ([num_kv_heads, dim] at q_off / k_off) and v ([num_heads, vdim] at v_off);
 * ba fp32 holds num_heads write-strength inputs, then num_heads decay inputs.  Per head h (q/k head h / (H / G)):
 *     q <- q / sqrt(|q|^2 + 1e-6) * q_scale;  k <- k / sqrt(|k|^2 + 1e-6);  beta = sigmoid(b);  g = exp(rate[h] * softplus(a + dt_bias[h]))
 *     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  out = S^T q            (S fp32 [dim, vdim], from zero for a new sequence)
 * state fp32 [slots, num_heads, vdim, dim]; out fp32 [n, num_heads, vdim].  dim <= 256. */
int b200m_gated_delta(const void* x, int64_t stride, int q_off, int k_off, int v_off, const float* ba, int64_t ba_stride,
                      const float* rate, const float* dt_bias, float* state, const int32_t* state_slots, const int32_t* cu_q,
                      const int32_t* cu_k, const int32_t* ctx_lens, float* out, int num_seqs, int num_heads, int num_kv_heads, int dim,
                      int vdim, float q_scale, int is32, void* stream);

/* out[t, h, :] = out_scale * x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * w * act(gate[t, h, :]); x fp32 [n, num_heads, vdim];
 * w [vdim] shared by the heads (NULL: none); gate with row stride gate_stride (NULL: none); act 0 = sigmoid, 1 = silu; out with
 * row stride out_stride. */
int b200m_head_rmsnorm_gate(const float* x, const void* w, const void* gate, int64_t gate_stride, int act, void* out,
                            int64_t out_stride, float out_scale, int n, int num_heads, int vdim, float eps, int is32, void* stream);

/* ---- routed experts ------------------------------------------------------------------------------------------------ */

int b200m_moe_tile_rows(void);

/* idx / wgt [n, top]: the experts with the largest logits and sigmoid(logit) of each. */
int b200m_moe_route(const float* logits, int64_t ld, int n, int num_experts, int top, int32_t* idx, float* wgt, void* stream);

/* Router with a choice correction, group-limited choice and identity experts.  s = softmax (score_kind 0) or sigmoid (1) of
 * the num_outputs logits; the choice is made on s + correction (NULL: s) among the experts of the `keep` best of n_groups
 * equal groups of neighbours (a group's score: its largest choice score; n_groups <= 1: no limit).  wgt = s of the chosen,
 * divided by their sum + 1e-20 when renorm, times scale.  Outputs e >= num_real are identity experts: idx = -1. */
int b200m_moe_route_grouped(const float* logits, int64_t ld, int n, int num_outputs, int top, const float* correction,
                            int n_groups, int keep, int num_real, int score_kind, int renorm, float scale, int32_t* idx,
                            float* wgt, void* stream);

/* Groups the n * top (token, choice) pairs by expert (pairs with idx < 0 take part in no GEMM: pos_of = -1), each expert's run padded to a multiple of b200m_moe_tile_rows().
 * cap >= round_up(pairs + num_experts * (tile - 1), tile); counts: 2 * num_experts ints of scratch. */
int b200m_moe_align(const int32_t* idx, int pairs, int num_experts, int32_t* sorted_rows, int cap, int32_t* pos_of,
                    int32_t* tile_expert, int32_t* num_tiles, int32_t* counts, void* stream);

/* C[i, :] = act(A_i . W[expert of i]^T) for every grouped row i.  gather: A_i = A[pair / top] * wgt[pair] (the expert's
 * weighted input; wgt NULL: unweighted); else A_i = A[i].  W [experts, N, K].  act 1 = relu^2; act 2 = gated: W holds N/2
 * gate rows, then N/2 up rows, and C[i, o] = silu(gate_o) * up_o has N/2 columns.  C is T, or fp32 when out_f32. */
int b200m_moe_gemm(const void* A, int64_t a_stride, const int32_t* sorted_rows, const float* wgt, int top, int gather,
                   const int32_t* tile_expert, const int32_t* num_tiles, int max_tiles, const void* W, int N, int K, void* C,
                   int out_f32, int act, int is32, void* stream);

/* out[t, :] = sum_k wgt[t, k] * rows[pos_of[t, k], :] + sigmoid(gate_logit[t]) * shared[t, :]  (fp32 out; wgt NULL: 1; shared
 * optional; gate_logit NULL: gate 1).  A choice with pos_of < 0 adds wgt[t, k] * ident[t, :] instead (ident NULL: nothing). */
int b200m_moe_combine(const float* rows, const int32_t* pos_of, int top, const void* shared, const float* gate_logit,
                      int64_t gate_ld, const float* wgt, const float* ident, float* out, int n, int width, int is32,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif
