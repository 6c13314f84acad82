/*
 * trtllm_b200_ragged.h — C ABI of the operators that run a RAGGED in-flight batch: every call works on N token
 * rows that belong to E sequences, each sequence bringing any number of new tokens (a portion of a prompt or one
 * generated token) on top of what its pages of the cache pool and its state slot already hold.
 *
 * Conventions (as in trtllm_b200.h): device pointers, asynchronous on `stream`, 0 on success, negative for a
 * rejected argument, positive cudaError_t.  Element types are named by TB_DT_*; "T" below is the model's storage
 * type (bf16, or fp32 for the all-32-bit mode).  The residual stream, every normalisation, softmax, the recurrent
 * state and everything that feeds a recurrence are fp32 in both modes.
 *
 * Batch description (device int32 arrays, built by the scheduler once per step):
 *   tok_seq[N]   index of the row's sequence in this step        tok_pos[N]   position of the row in its sequence
 *   seq_start[E] first row of the sequence                       seq_len[E]   rows it brings
 *   seq_past[E]  positions it already holds (= tok_pos of its first row)
 *   seq_slot[E]  its recurrent-state slot                        block_table[E, max_blocks] its pages of the pool
 */
#ifndef TRTLLM_B200_RAGGED_H
#define TRTLLM_B200_RAGGED_H

#include "trtllm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { TB_DT_F32 = 1, TB_DT_BF16 = 2 };
enum { TB_ACT_NONE = 0, TB_ACT_GELU_TANH = 1, TB_ACT_GATED = 2 /* tb_linear_gated only */, TB_ACT_RELU_SQUARED = 3 /* max(z, 0)^2 */ };
/* tb_linear compute paths: AUTO = tensor cores for bf16 weights, FMA for fp32 weights; FMA32 = fp32 multiply-add in a
 * fixed k order whatever the storage type (the all-32-bit mode, and the small products that feed a recurrence). */
enum { TB_COMPUTE_AUTO = 0, TB_COMPUTE_FMA32 = 1, TB_COMPUTE_TILES = 2 /* bf16: the warp-MMA tiles at any row count (A/B) */ };
/* gated activations of a feed-forward's (gate, up) pair: SIGMOID = g' * sigmoid(alpha g') * (u' + up_shift) with g' = min(g, limit),
 * u' = clamp(u, -limit, limit) (limit <= 0: no clamp; alpha 1, shift 0 is silu(g) * u); GELU_TANH = gelu_tanh(g) * u. */
enum { TB_GATE_SIGMOID = 0, TB_GATE_GELU_TANH = 1 };
/* which elements of a head a rotation pairs: (2i, 2i + 1), or (i, i + dims / 2) */
enum { TB_ROPE_INTERLEAVED = 0, TB_ROPE_HALF = 1 };

/* C[b][m, n] = act( sum_k A[b][m, k] * W[b][n, k] + bias[b][n] ),  b < batch.
 * A: a_dtype, row stride lda, batch stride a_bs (elements).  W: w_dtype, [N, K] rows contiguous, batch stride w_bs.
 * bias: w_dtype or NULL, batch stride bias_bs.  C: c_dtype, row stride ldc, batch stride c_bs.
 * The sum over k runs in the same order for every row, whatever M is and wherever the row stands in the batch. */
int tb_linear(void* c, int c_dtype, int64_t ldc, int64_t c_bs, const void* a, int a_dtype, int64_t lda, int64_t a_bs,
              const void* w, int w_dtype, int64_t w_bs, const void* bias, int64_t bias_bs, int M, int N, int K, int batch,
              int act, int compute, tb_stream_t stream);

/* Gated feed-forward input side in one kernel, for generation steps (<= 8 rows, bf16 weights, 8 | K):
 * out[m, j] = the gated activation `gate` (TB_GATE_*) of g = a[m] . w[j] and u = a[m] . w[ff + j],
 * w [2 ff, K] = gate rows, then up rows.  Returns -3 when the shape is not one the streaming kernel takes; the caller
 * then runs tb_linear + tb_gated_act, which compute the same. */
int tb_linear_gated(void* c, int c_dtype, int64_t ldc, const void* a, int a_dtype, int64_t lda, const void* w, int w_dtype,
                    int M, int ff, int K, int gate, float alpha, float limit, float up_shift, tb_stream_t stream);

/* Prompt-sized products of bf16 operands on the 5th-generation tensor cores (tcgen05 / TMEM / TMA, the kernel of
 * tb_gemm_tc with bf16 formats): c = act(x w^T + bias); x [M, K], w [N, K] bf16 contiguous, 8 | K, both 16-byte aligned;
 * c [M, N] contiguous fp32 (out_type 1) or bf16 (out_type 3); bias bf16 [N] or NULL; act TB_ACT_*.
 * workspace / counters as for tb_gemm_tc (used only when M <= 16 splits K). */
int tb_gemm_tc_bf16(void* c, int out_type, const void* x, const void* w, const void* bias, int act, int M, int N, int K,
                    void* workspace, size_t workspace_bytes, int* counters, tb_stream_t stream);
/* out bf16 [rows, cols] contiguous = x fp32 (row stride ld): the residual stream as a tensor-core operand. */
int tb_cast_rows_bf16(void* out, const float* x, int64_t ld, int rows, int cols, tb_stream_t stream);

/* out[n, :] = table[ids[n], :] * scale  (fp32 residual stream; ids clamped into [0, vocab)). */
int tb_embed_scaled(float* out, const void* table, int t_dtype, const int* ids, float scale, int rows, int width,
                    int vocab, tb_stream_t stream);
/* The same plus a hashed embedding of the (previous, current) token pair: out[n, :] += pair[r, :] with
 * r = (prev_ids[n] * mul_prev + ids[n] * mul_cur) mod buckets, or r = buckets (the last row of pair [buckets + 1, width]) for a
 * token without a predecessor (prev_ids[n] < 0).  pair has the table's type. */
int tb_embed_bigram(float* out, const void* table, const void* pair, int t_dtype, const int* ids, const int* prev_ids, float scale,
                    int rows, int width, int vocab, int buckets, int mul_prev, int mul_cur, tb_stream_t stream);

/* y = out_scale * x / sqrt(mean(x^2) + eps) * (w + w_offset) over `cols` columns of each row; x fp32 with row stride ldi.
 * accumulate != 0: out (fp32) += y — the residual update of a layer that normalises the sublayer's OUTPUT (out_scale is
 * then the layer's residual multiplier); else out = y in out_dtype.  w == NULL: no weight.  rows_idx != NULL: row r of out
 * comes from row rows_idx[r] of x. */
int tb_rmsnorm_rows(void* out, int out_dtype, int64_t ldo, const float* x, int64_t ldi, const void* w, int w_dtype,
                    float w_offset, float eps, const int* rows_idx, int rows, int cols, int accumulate, float out_scale,
                    tb_stream_t stream);

/* The residual step of a layer that normalises before AND after its sublayers, with the next sublayer's input, in one
 * pass: x <- x + out_scale * y / rms(y) * (w_post + w_offset), then h = x / rms(x) * (w_pre + w_offset) stored as h_dtype.
 * x fp32 in place (row stride ldx), y fp32 (ldy); both weights of type w_dtype.  Computes what tb_rmsnorm_rows with
 * accumulate followed by tb_rmsnorm_rows computes. */
int tb_residual_norm_rows(float* x, int64_t ldx, const float* y, int64_t ldy, const void* w_post, const void* w_pre,
                          int w_dtype, float w_offset, float eps, float out_scale, void* h, int h_dtype, int64_t ldh, int rows,
                          int cols, tb_stream_t stream);

/* Layer normalisation with weight and bias: out = (x - mean) / sqrt(var + eps) * w + b over `cols` columns of each fp32 row
 * (row stride ldi), var = mean of the squared deviations; w, b of type w_dtype (b may be NULL); out in out_dtype.
 * rows_idx != NULL: row r of out comes from row rows_idx[r] of x. */
int tb_layernorm_rows(void* out, int out_dtype, int64_t ldo, const float* x, int64_t ldi, const void* w, const void* b, int w_dtype,
                      float eps, const int* rows_idx, int rows, int cols, tb_stream_t stream);
/* The residual step of a layer whose sublayers all read one normalised input and are summed, with the next layer's input, in
 * one pass: x <- x + out_scale * (y1 + y2) (y2 may be NULL), then h = layer_norm(x; w, b) stored as h_dtype.  w == NULL: only
 * the residual step.  Computes what the sum followed by tb_layernorm_rows computes. */
int tb_residual_layernorm_rows(float* x, int64_t ldx, const float* y1, int64_t ldy1, const float* y2, int64_t ldy2, float out_scale,
                               const void* w, const void* b, int w_dtype, float eps, void* h, int h_dtype, int64_t ldh, int rows,
                               int cols, tb_stream_t stream);
/* The residual step of a sublayer that sits between two layer norms, with the next sublayer's input, in one pass:
 * x <- x + out_scale * LN(y; w_post, b_post), then h = LN(x; w_pre, b_pre) stored as h_dtype (w_pre == NULL: only the residual
 * step).  Biases may be NULL.  Computes what tb_layernorm_rows, the sum and tb_layernorm_rows compute. */
int tb_residual_sandwich_layernorm_rows(float* x, int64_t ldx, const float* y, int64_t ldy, const void* w_post, const void* b_post,
                                        const void* w_pre, const void* b_pre, int w_dtype, float eps, float out_scale, void* h,
                                        int h_dtype, int64_t ldh, int rows, int cols, tb_stream_t stream);
/* Per-layer token input, one kernel per layer: e = side_embed[ids[n], e_off : e_off + sd] (row stride lde), g = gelu_tanh(w_gate x)
 * * e (w_gate [sd, width]), y = w_proj g (w_proj [width, sd]), x <- x + y / sqrt(mean(y^2) + eps) * norm_w.  The operands of the two
 * products are rounded to the storage type w_dtype; sums, norm and residual are fp32.  With w_pre the next layer's input leaves the
 * same kernel: h = LN(x; w_pre, b_pre), or x / rms(x) * w_pre when pre_rms != 0.
 * y_in != NULL (fp32 [rows, width], row stride ldy): y has been computed by the caller — prompt-sized steps run the two products
 * as projections with tb_side_gate_mul between them — and the kernel does the norm, the residual step and the next norm. */
int tb_token_side_input(float* x, int64_t ldx, const float* y_in, int64_t ldy, const void* side_embed, int64_t lde, int e_off,
                        const int* ids, int vocab, const void* w_gate, const void* w_proj, const void* norm_w, int w_dtype, float eps,
                        int rows, int width, int sd, const void* w_pre, const void* b_pre, int pre_rms, void* h, int h_dtype,
                        int64_t ldh, tb_stream_t stream);
/* g[n, j] = gelu_tanh(z[n, j]) * side_embed[ids[n], e_off + j], j < sd, stored as g_dtype [rows, sd] contiguous; z fp32 (row stride ldz). */
int tb_side_gate_mul(void* g, int g_dtype, const float* z, int64_t ldz, const void* side_embed, int e_dtype, int64_t lde, int e_off,
                     const int* ids, int vocab, int rows, int sd, tb_stream_t stream);
/* out fp32 = out_scale * (a / rms(a) * wa + b / rms(b) * wb): two mixers side by side, each RMS-normalised over the row with its
 * own weight (a, b fp32 rows). */
int tb_rmsnorm_pair_sum(float* out, int64_t ldo, const float* a, int64_t lda, const float* b, int64_t ldb, const void* wa,
                        const void* wb, int w_dtype, float eps, float out_scale, int rows, int cols, tb_stream_t stream);
/* out[r] = [a[r, :cols_a] | b[r, :cols_b]] (fp32 inputs with row strides lda / ldb) in out_dtype, contiguous: the operand of a
 * projection that reads two streams side by side. */
int tb_concat_rows(void* out, int out_dtype, const float* a, int64_t lda, int cols_a, const float* b, int64_t ldb, int cols_b,
                   int rows, tb_stream_t stream);

/* x[r, :cols] += vec (fp32 rows with stride ld; vec fp32 or bf16): the vector a pass of a looped block of layers adds to
 * the residual stream. */
int tb_add_row_vector(float* x, int64_t ld, const void* vec, int v_dtype, int rows, int cols, tb_stream_t stream);

/* x <- cap * tanh(x / cap), in place over n fp32 values (soft cap of the logits). */
int tb_tanh_cap(float* x, int64_t n, float cap, tb_stream_t stream);

/* Gated feed-forward activation `gate` (TB_GATE_*) of g = gu[n, j], u = gu[n, ff + j]; gu fp32 [rows, 2 ff].
 * row_scale != NULL: g and u of row n are first multiplied by row_scale[row_index ? row_index[n] : n] (0 where the index is
 * negative): an expert whose router score weighs its input — the projections are linear, so the score moves behind them. */
int tb_gated_act(void* out, int out_dtype, const float* gu, int rows, int ff, int gate, float alpha, float limit, float up_shift,
                 const float* row_scale, const int* row_index, tb_stream_t stream);

/* cos / sin of pos * base^(-2 i / dims), i < dims / 2, for every row: table fp32 [N, dims / 2, 2] (angles in fp64). */
int tb_rope_table(float* table, const int* tok_pos, int rows, int dims, double base, tb_stream_t stream);
/* The same with scaled frequencies (factor > 0): with wavelength lambda = 2 pi / f, frequencies with lambda above
 * original / low are divided by factor, those with lambda below original / high are kept, and in the band between a share
 * keep = (original / lambda - low) / (high - low) of the frequency is kept: f' = f * (keep + (1 - keep) / factor). */
int tb_rope_table_scaled(float* table, const int* tok_pos, int rows, int dims, double base, double factor, double low,
                         double high, double original, tb_stream_t stream);

/* Rotated tail of the queries into the attention operand: for head h of row n the `rot_dim` elements of q (fp32,
 * [N, H, dim + rot_dim]) behind the first `dim` are rotated pairwise (2i, 2i + 1) over their first `dims` elements by
 * the row's table entry and stored as T at qa[n, h, lat + j], qa being [N, H, lat + rot_dim]. */
int tb_rope_query_tail(void* qa, int dtype, const float* q, const float* table, int rows, int heads, int dim,
                       int rot_dim, int dims, int lat, tb_stream_t stream);

/* Latent KV append: row n of kv (fp32, stride ldkv) holds `lat` latent values and `rot_dim` shared rotary key
 * values.  The latent is RMS-normalised (weight w, eps), the key part rotated by the row's table entry, and both are
 * stored as one entry [lat + rot_dim] of type T at the row's position in its sequence's pages:
 * pool[(block_table[seq, pos / page] * page + pos % page) * (lat + rot_dim)]. */
int tb_latent_kv_append(void* pool, int dtype, const float* kv, int64_t ldkv, const void* w, int w_dtype, float eps,
                        const float* table, int dims, const int* tok_seq, const int* tok_pos, const int* block_table,
                        int max_blocks, int page, int rows, int lat, int rot_dim, tb_stream_t stream);

/* Causal attention of every row over its sequence's cached latent entries 0..pos (multi-query form: one entry serves
 * all heads).  qa T [N, H, lat + rot_dim]: per head the query absorbed into latent space, then its rotated tail.
 * score = scale * <qa, entry>; softmax in fp32 over the visible entries; out T [N, H, lat] = sum_j p_j * entry_j[:lat].
 * Keys are visited in blocks of 32 positions from 0, so a row's result does not depend on how its prompt was cut
 * or on what else is in the batch.
 * bf16 with 32 | lat, 16 | rot_dim runs on tensor cores (tb_latent_attention_tensor_cores tells): one CTA per (row,
 * 16 heads, key range).  nsplit > 1 deals every row's key blocks to nsplit CTAs whose partial results (workspace: fp32
 * [rows, heads, nsplit, lat + 2]) a second kernel merges — for steps with few rows and long contexts; other
 * configurations ignore it; nsplit < 0 keeps any configuration on the warp-per-head kernel (A/B). */
int tb_latent_attention_tensor_cores(int dtype, int lat, int rot_dim);
int tb_latent_attention(void* out, const void* qa, const void* pool, int dtype, const int* tok_seq, const int* tok_pos,
                        const int* block_table, int max_blocks, int page, int rows, int heads, int lat, int rot_dim,
                        float scale, int nsplit, float* workspace, tb_stream_t stream);

/* Per-channel causal convolution over a ragged batch with carried inputs: out[n, c] = bias[c] + sum_k w[c, k] *
 * x(pos - (taps - 1 - k)), where positions before the sequence's portion come from state[slot] (fp32
 * [slots, taps - 1, C], oldest first) and positions before the sequence's start are zero.  x, out fp32 [N, C]. */
int tb_causal_conv1d(float* out, const float* x, const void* w, const void* bias, int w_dtype, const float* state,
                     const int* tok_seq, const int* tok_pos, const int* seq_start, const int* seq_past,
                     const int* seq_slot, int rows, int channels, int taps, tb_stream_t stream);
/* state[slot] <- the last taps - 1 inputs of (what it held ++ this step's rows); run after the convolution.  x has row
 * stride ldx (its first `channels` columns are the convolution's inputs).  skip_single != 0: sequences that bring one row
 * are left alone (tb_qkv_conv_rope_append has moved them on). */
int tb_causal_conv1d_update(float* state, const float* x, int64_t ldx, const int* seq_start, const int* seq_len, const int* seq_past,
                            const int* seq_slot, int seqs, int channels, int taps, int skip_single, tb_stream_t stream);

/* Real-gated linear recurrent unit over a ragged batch.  gates fp32 [N, blocks, 2, C / blocks]: per block the
 * recurrence-gate logits, then the input-gate logits (biases already added).  Per channel, in sequence order:
 *   r = sigmoid(gr), i = sigmoid(gi), log a = -c * r * softplus(lam), S <- exp(log a) * S + sqrt(1 - exp(2 log a)) * i * u
 * with S read from / written to state[slot] (fp32 [slots, C]; zero at a sequence's first position), and
 * out[n, ch] = S * y[n, ch] stored as T.  u fp32 [N, C], y T [N, C], lam w_dtype [C].
 * max_len: the longest seq_len (host); with workspace (fp32, 3 * seqs * ceil(max_len / 32) * C) and max_len > 32 the rows
 * of a sequence are scanned in parallel chunks of 32 whose summaries are carried in order. */
int tb_rglru_scan(void* out, int dtype, const float* u, const float* gates, const void* lam, int w_dtype, const void* y,
                  float* state, const int* seq_start, const int* seq_len, const int* seq_past, const int* seq_slot,
                  int seqs, int channels, int blocks, float c, int max_len, float* workspace, tb_stream_t stream);

/* ---- windowed grouped-query attention with short convolutions, a softmax sink and output gates ------------------
 * Pool entry of one position (type T): [kv_heads][dim] rotated keys, then [kv_heads][vdim] values.
 *
 * tb_qkv_conv_rope_append: proj fp32 [N, ldp] holds per row q (heads * dim) | k (kv_heads * dim) | v (kv_heads * vdim)
 * = C channels (further columns are ignored).  Each channel runs a causal convolution of `taps` taps (conv_w [C, taps],
 * no bias; tap j weighs the input taps - 1 - j positions back) over the row's portion and the carried inputs state[slot] (fp32
 * [slots, taps - 1, C], oldest first; zeros before the sequence's start); then the first `dims` elements of every query
 * and key head are rotated as interleaved pairs (2i, 2i + 1) by the row's table entry.  Queries go to q_out T [N, heads,
 * dim]; keys and values to the row's position in its sequence's pages.  Carry the state on with
 * tb_causal_conv1d_update(state, proj, ldp, ..., C, taps, skip_single) afterwards.  state_rw == state with seq_len given: a
 * sequence that brings ONE row has its carried inputs moved on by this kernel (the thread that read a channel's inputs
 * rewrites them), the update is then called with skip_single = 1 — or not at all when every sequence brings one row. */
int tb_qkv_conv_rope_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* conv_w,
                            int w_dtype, const float* state, const float* table, int dims, const int* tok_seq,
                            const int* tok_pos, const int* seq_start, const int* seq_past, const int* seq_slot,
                            const int* block_table, int max_blocks, int page, int rows, int heads, int kv_heads, int dim,
                            int vdim, int taps, float* state_rw, const int* seq_len, tb_stream_t stream);

/* The same step for an attention that RMS-normalises queries and keys over the WHOLE projection: proj holds q (heads * dim) | k
 * (kv_heads * dim) [| v (kv_heads * vdim) unless tied_values].  After the convolution (conv_w [C, taps] or NULL: none) the q part
 * and the k part are each divided by their root mean square over all their channels (eps inside the root) and multiplied by
 * norm_q [heads * dim] / norm_k [kv_heads * dim] (both NULL: no norm), then rotated and stored as above.  tied_values != 0: the
 * values are the keys as they leave the convolution, before norm and rotation (vdim == dim; C = (heads + kv_heads) * dim).
 * The carried inputs are [slots, taps - 1, C]; carry them on as above. */
int tb_qk_conv_norm_rope_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* conv_w,
                                const void* norm_q, const void* norm_k, int w_dtype, float eps, const float* state, const float* table,
                                int dims, const int* tok_seq, const int* tok_pos, const int* seq_start, const int* seq_past,
                                const int* seq_slot, const int* block_table, int max_blocks, int page, int rows, int heads,
                                int kv_heads, int dim, int vdim, int taps, int tied_values, float* state_rw, const int* seq_len,
                                tb_stream_t stream);

/* Attention of every row over the cached positions j of its sequence with 0 <= pos - j < window (window 0: all of
 * 0..pos).  Query head h uses key/value head h / (heads / kv_heads).  score = scale * <q, k>; the softmax denominator
 * also holds exp(sink[h]) (sink fp32 or bf16 [heads], or NULL for none): a term without key or value, not scaled.
 * out T [N, heads, vdim] = softmax-weighted values, times sigmoid(gate[n, h]) when gate (fp32 logits, row stride ldg) is
 * given.  Softmax in fp32; keys are visited in blocks of 32 absolute positions from the window's first block, so a row's
 * result does not depend on how its prompt was cut or on the batch around it.  vdim <= 512.
 * bf16 with a (dim, vdim) pair the tensor-core kernel is built for (tb_window_attention_tensor_cores tells) runs on
 * tensor cores when the per-sequence description is given: seq_start / seq_len / seq_past [seqs] and max_len >= the longest
 * seq_len (host; it sizes the grid).  nsplit > 1 (tensor-core form only) deals every row block's key tiles to nsplit CTAs
 * whose partial results (workspace: fp32 [rows, heads, nsplit, vdim + 2]) a second kernel merges in index order — for steps
 * with few rows (generation), so that more than a handful of SMs read the cache.  mode 1 keeps any configuration on the
 * SIMT kernel (A/B). */
int tb_window_attention_tensor_cores(int dtype, int heads, int kv_heads, int dim, int vdim);
int tb_window_attention(void* out, const void* q, const void* pool, int dtype, const float* gate, int64_t ldg,
                        const void* sink, int sink_dtype, const int* tok_seq, const int* tok_pos, const int* block_table,
                        const int* seq_start, const int* seq_len, const int* seq_past, int seqs, int max_len,
                        int max_blocks, int page, int rows, int heads, int kv_heads, int dim, int vdim, float scale,
                        int window, int mode, int nsplit, float* workspace, tb_stream_t stream);

/* The same attention with value heads shared by neighbouring key heads: there are kv_heads key heads but only kv_heads / v_share
 * value heads, key head g reads value head g / v_share, and a pool entry is [kv_heads][dim] keys, then [kv_heads / v_share][vdim]
 * values (several attention maps over one set of values).  out_f32 != 0: the result is stored as fp32 [N, heads, vdim] whatever
 * the storage type (for a step that combines maps before anything is rounded).  keep_first > 0 (with a window): positions
 * j < keep_first stay visible to every later row as well (they keep their true positions).  v_share = 1, out_f32 = 0,
 * keep_first = 0 is tb_window_attention. */
int tb_window_attention_shared_values(void* out, int out_f32, const void* q, const void* pool, int dtype, const float* gate,
                                      int64_t ldg, const void* sink, int sink_dtype, const int* tok_seq, const int* tok_pos,
                                      const int* block_table, const int* seq_start, const int* seq_len, const int* seq_past,
                                      int seqs, int max_len, int max_blocks, int page, int rows, int heads, int kv_heads,
                                      int v_share, int dim, int vdim, float scale, int window, int keep_first, int mode,
                                      int nsplit, float* workspace, tb_stream_t stream);

/* ---- differential attention: two attention maps per head over one set of values ---------------------------------------
 * tb_qk_norm_append: proj fp32 [N, ldp] holds per row q_vectors query vectors, k_vectors key vectors (each of `dim`) and
 * v_channels value channels.  Every query and key vector is RMS-normalised over dim (x / sqrt(mean(x^2) + eps)) and multiplied
 * by wq / wk ([dim], shared by all vectors; NULL: none); queries are also multiplied by the position's temperature
 * 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1) (temp_every <= 0: none).  Queries go to q_out T [N, q_vectors, dim]; keys
 * and values to the row's position in its pages (entry = [k_vectors][dim] keys, then v_channels values). */
int tb_qk_norm_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* wq, const void* wk, int w_dtype,
                      float eps, float temp_coef, int temp_every, const int* tok_seq, const int* tok_pos, const int* block_table,
                      int max_blocks, int page, int rows, int q_vectors, int k_vectors, int dim, int v_channels, tb_stream_t stream);
/* maps fp32 [N, kv_heads, 2, per, vdim]: for every key/value head the first and the second map of its `per` query heads.
 * out T [N, kv_heads * per, vdim] = o / sqrt(mean(o^2) + eps) * mult with o = map1 - lambda * map2 and
 * lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (the four vectors of ldim elements, type w_dtype).  All fp32. */
int tb_diff_combine(void* out, int dtype, const float* maps, const void* lq1, const void* lk1, const void* lq2, const void* lk2,
                    int w_dtype, int ldim, float diff, float eps, float mult, int rows, int kv_heads, int per, int vdim,
                    tb_stream_t stream);

/* ---- gated delta rule -----------------------------------------------------------------------------------------------------
 * Per head a state S [dim, vdim] (fp32): S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  `heads` value heads,
 * `kv_heads` query / key heads (head h uses query / key head h / (heads / kv_heads)).
 *
 * tb_delta_prepare: proj fp32 [N, ldp]; its first C = 2 kv_heads dim + heads vdim columns are q | k | v.  Each of these channels
 * runs a causal convolution of `taps` taps (conv_w [C, taps], no bias; the last tap weighs the current input) over the row's portion
 * and the carried inputs state[slot] (fp32 [slots, taps - 1, C], oldest first; zeros before the sequence's start), then SiLU.
 * Queries and keys are then divided by sqrt(sum(x^2) + eps_unit) per head, queries also by sqrt(dim).  u fp32 [N, C] receives
 * q | k | v.  bg fp32 [N, 2 heads] receives beta = sigmoid(proj[col_b + h]) and g = exp(-exp(a_log[h]) * softplus(proj[col_a + h]
 * + dt_bias[h])).  state_rw == state: a sequence that brings ONE row has its carried inputs moved on here; run
 * tb_causal_conv1d_update(state, proj, ldp, ..., C, taps, 1) afterwards for the others. */
int tb_delta_prepare(float* u, float* bg, const float* proj, int64_t ldp, const void* conv_w, const void* a_log, const void* dt_bias,
                     int w_dtype, int col_b, int col_a, const float* state, float* state_rw, const int* tok_seq, const int* tok_pos,
                     const int* seq_start, const int* seq_len, const int* seq_past, const int* seq_slot, int rows, int heads,
                     int kv_heads, int dim, int vdim, int taps, float eps_unit, tb_stream_t stream);
/* The recurrence over every sequence's rows in order, from state[slot] (fp32 [slots, heads, vdim, dim]: S transposed, a value
 * column's elements contiguous; zeros at a sequence's first position) and back into it.  out fp32 [N, heads, vdim].  dim <= 512.
 * rows = N; max_len: the longest seq_len (host).  With workspace (fp32, rows * (16 kv_heads + 20 heads) values, 16-byte aligned)
 * and max_len >= 3 the rows of a sequence are resolved eight at a time (one reduction round per eight rows; the same recurrence
 * up to fp32 rounding); otherwise row by row. */
int tb_delta_rule_scan(float* out, const float* u, const float* bg, float* state, const int* seq_start, const int* seq_len,
                       const int* seq_past, const int* seq_slot, int rows, int seqs, int heads, int kv_heads, int dim, int vdim,
                       int max_len, float* workspace, tb_stream_t stream);
/* A/B switch for measurements: which prompt kernel tb_delta_rule_scan takes.  0: by the number of value columns (default);
 * 1: four columns per warp whenever dim <= 256; 3: one column per warp. */
int tb_delta_scan_set_mode(int mode);
/* out T [N, heads, vdim] = o / sqrt(mean_vdim(o^2) + eps) * w * silu(gate): o fp32 [N, heads, vdim]; w [vdim] shared by the heads
 * (NULL: none); gate fp32 logits [N, >= heads * vdim] with row stride ldg (NULL: none). */
int tb_gated_rmsnorm_heads(void* out, int dtype, const float* o, const float* gate, int64_t ldg, const void* w, int w_dtype, float eps,
                           int rows, int heads, int vdim, tb_stream_t stream);

/* ---- linear attention with a scalar decay per head and token ------------------------------------------------------------
 * Per (sequence, head) a state S [dim, vcols] (fp32):  S_t = a_t S_(t-1) + b_t k_t v_t^T,  o_t = S_t^T q_t.
 * q, k fp32 rows of [heads, dim] (row strides ldq, ldk), v fp32 rows of [heads, vdim] (ldv).  log_ab fp32 [N, heads, 2] = ln a_t
 * (<= 0), ln b_t; or NULL, then a_t = head_decay[h] (fp32 [heads]) and b_t = 1.  ones_col != 0: one more value column follows
 * the values whose v is 1 at every row (its state is sum of weighted keys: the normaliser of an mLSTM), vcols = vdim + 1.
 * state: slot s at state + s * state_stride, [heads, vcols, dim] (a column's dim elements contiguous); zeros at a sequence's
 * first position.  q_scale: a factor on every query (1: none).  out fp32 [N, heads, vcols].  max_len: the longest seq_len
 * (host): from 4 rows on (dim <= 256) the rows are
 * resolved 32 at a time from the portion's first row (the same recurrence up to fp32 rounding), else row by row.
 * segments > 1 with workspace (fp32, seqs * segments * (heads * vcols * dim + heads) values, 16-byte aligned): a
 * long portion is cut into that many segments (whole blocks of 32 rows) that run side by side — every segment's own end state
 * from zero, the states carried from segment to segment in order, then every segment from its carried state.
 * tb_decay_scan_segments tells how many segments fill the chip (1: none). */
int tb_decay_attention_scan(float* out, const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                            const float* log_ab, const float* head_decay, float* state, int64_t state_stride, const int* seq_start,
                            const int* seq_len, const int* seq_past, const int* seq_slot, int rows, int seqs, int heads, int dim,
                            int vdim, int ones_col, float q_scale, int max_len, float* workspace, int segments, tb_stream_t stream);
int tb_decay_scan_segments(int seqs, int heads, int vcols, int max_len);
/* A/B switch for tests and measurements: 1 keeps tb_decay_attention_scan row by row; 2 keeps long portions in one segment; 0: by
 * max_len (default). */
int tb_decay_scan_set_mode(int mode);
/* Gates of an mLSTM matrix memory.  Per row and head, from proj (fp32, row stride ldp): i = cap * tanh((proj[col_i + h] + bias_i[h])
 * / cap), f = logsigmoid(cap * tanh((proj[col_f + h] + bias_f[h]) / cap)) (cap <= 0: no cap); running maximum m_t = max(f_t +
 * m_(t-1), i_t) with m = 0 before a sequence's first row, carried in m_state[slot * m_stride + h].
 * log_ab [N, heads, 2] = (f_t + m_(t-1) - m_t, i_t - m_t);  m_out [N, heads] = m_t. */
int tb_mlstm_gates(float* log_ab, float* m_out, const float* proj, int64_t ldp, int col_i, int col_f, const void* bias_i,
                   const void* bias_f, int w_dtype, float cap, float* m_state, int64_t m_stride, const int* seq_start,
                   const int* seq_len, const int* seq_past, const int* seq_slot, int seqs, int heads, tb_stream_t stream);
/* out fp32 rows of [heads, dim] (row stride ldo) = x (ldx) with the first `dims` elements of every head rotated by the row's table
 * entry (tb_rope_table), pairs by `layout` (TB_ROPE_*), the rest copied; heads below `split` times scale_lo, the others times
 * scale_hi.  out may be x. */
int tb_rope_heads(float* out, int64_t ldo, const float* x, int64_t ldx, const float* table, int rows, int heads, int dim, int dims,
                  int layout, int split, float scale_lo, float scale_hi, tb_stream_t stream);
/* out T [N, heads, vdim] from o fp32 [N, heads, vcols] (the first vdim columns): with m (fp32 [N, heads]) first o / (max(|o[vdim]|,
 * exp(-m)) + den_eps); then o / sqrt(mean_vdim(o^2) + eps) * w (w [vdim] shared, or [heads * vdim] when w_per_head; NULL: none)
 * * act(gate) (gate fp32 logits [N, >= heads * vdim], row stride ldg; gate_act 0 none, 1 silu, 2 sigmoid). */
int tb_head_norm_gate(void* out, int dtype, const float* o, int vcols, const float* m, float den_eps, const float* gate, int64_t ldg,
                      int gate_act, const void* w, int w_dtype, int w_per_head, float eps, int rows, int heads, int vdim,
                      tb_stream_t stream);

/* ---- routed-expert feed-forward ------------------------------------------------------------------------------------
 * tb_moe_route: logits fp32 [N, experts].  s = sigmoid(logit); choice = s + correction (fp32 or bf16 [experts], NULL:
 * none).  Experts form `groups` equal groups of neighbours; a group scores the sum of its two largest choices and only the
 * `keep` best groups stay eligible.  The `top` largest eligible choices are taken (ties: lower index):
 * ids int32 [N, top], weights fp32 [N, top] = s of the chosen experts (not renormalised). */
int tb_moe_route(int* ids, float* weights, const float* logits, const void* correction, int c_dtype, int rows, int experts,
                 int top, int groups, int keep, tb_stream_t stream);
/* Softmax router: s = softmax(logits) over all experts (fp32); the `top` largest s are taken (ties: lower index);
 * weights = s / (sum of the chosen s + 1e-20) * scale when renorm != 0, else s * scale. */
int tb_moe_route_softmax(int* ids, float* weights, const float* logits, int rows, int experts, int top, int renorm, float scale,
                         tb_stream_t stream);
/* Plan: the N * top (token, choice) pairs sorted by expert, every expert's range padded to whole tiles of `tile` rows.
 * tb_moe_plan_tiles = the number of tiles that is always enough; slot_pair int32 [max_tiles * tile] (pair index, -1 in
 * the padding), tile_expert int32 [max_tiles] (-1: unused tile), pair_slot int32 [pairs] (the inverse map; may be NULL). */
enum { TB_MOE_TILE = 64 };
int tb_moe_plan_tiles(int pairs, int experts, int tile);
int tb_moe_plan(int* slot_pair, int* tile_expert, int* pair_slot, const int* ids, int pairs, int experts, int tile,
                int max_tiles, tb_stream_t stream);
/* c = act(a w_e^T) tile by tile over the plan (tile height TB_MOE_TILE): w [experts, N, K].  a_div > 0: a [tokens, K] and
 * slot s reads row slot_pair[s] / a_div; a_div == 0: a [slots, K].  c_by_pair != 0: C row = pair index, else the slot.
 * compute as tb_linear (AUTO: tensor cores for bf16 weights). */
int tb_moe_linear(void* c, int c_dtype, int64_t ldc, const void* a, int a_dtype, int64_t lda, const void* w, int w_dtype,
                  const int* slot_pair, const int* tile_expert, int max_tiles, int a_div, int c_by_pair, int N, int K, int act,
                  int compute, tb_stream_t stream);
/* The same products on the 5th-generation tensor cores (the kernel of tb_gemm_tc_bf16), for plans with tiles of 128 rows:
 * x bf16 [max_tiles * 128, K] contiguous in plan order (tb_moe_gather_rows makes it from token rows), w bf16
 * [experts, N, K], c fp32 (out_type 1) or bf16 (3) [max_tiles * 128, N] in plan order; 8 | K. */
int tb_gemm_tc_bf16_grouped(void* c, int out_type, const void* x, const void* w, const int* tile_expert, int max_tiles,
                            int experts, int act, int N, int K, tb_stream_t stream);
/* xs bf16 [slots, cols] = x[slot_pair[s] / top, :] (x fp32 or bf16 with row stride ldx; zeros where slot_pair[s] < 0). */
int tb_moe_gather_rows(void* xs, const void* x, int x_dtype, int64_t ldx, const int* slot_pair, int slots, int top, int cols,
                       tb_stream_t stream);
/* Expert products for few pairs (generation steps) without a plan: pair b = one row of the streaming kernel against the
 * weights of expert ids[b].  a_div > 0: a [tokens, K], pair b reads row b / a_div; a_div == 0: a [pairs, K].  c [pairs, N].
 * act TB_ACT_GATED: w [experts, 2 N, K] (gate rows, then up rows), c = the gated activation `gate` (TB_GATE_*) of them, both
 * first multiplied by pair_scale[b] when that is given (a score that weighs the expert's input).
 * Returns -3 when the streaming kernel does not take the shape (bf16 weights, 8 | K, 16-byte aligned rows). */
int tb_moe_gemv(void* c, int c_dtype, int64_t ldc, const void* a, int a_dtype, int64_t lda, const void* w, int w_dtype,
                const int* ids, int pairs, int a_div, int N, int K, int act, int gate, float alpha, float limit, float up_shift,
                const float* pair_scale, tb_stream_t stream);
/* out fp32 [N, width] = sum_k weights[n, k] * y[r(n * top + k), :], k in index order; r(p) = pair_slot[p] (rows of y in
 * plan order) or p itself when pair_slot is NULL (y fp32 in pair order).  weights == NULL: a plain sum. */
int tb_moe_combine(float* out, const float* y, const float* weights, const int* pair_slot, int rows, int width, int top,
                   tb_stream_t stream);

/* tb_moe_combine plus a term every token has: out = add + sum_k ... (add fp32 [N, width], e.g. a shared expert's output; NULL: none). */
int tb_moe_combine_add(float* out, const float* y, const float* weights, const int* pair_slot, const float* add, int rows, int width,
                       int top, tb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRTLLM_B200_RAGGED_H */
