// hybrid_ops.cuh -- launchers of the mechanisms the layer-list decoder (hybrid.cu) is assembled from.  Each returns a b200_status_t.
#pragma once
#include "common.cuh"

namespace b200 {

// attention_chunked.cu
int launch_attn_qk_norm_cache(int dtype, const void *proj, int ld, void *q_out, void *k_pool, void *v_pool, const float *q_norm,
                              const float *k_norm, float eps, const int *tok_seq, const int *tok_pos, const int *block_table, int mpps,
                              int tokens, int heads, int kv_heads, int dim, cudaStream_t st);
int launch_chunked_attention(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in,
                             int gate_ld, void *out, const int *tok_seq, const int *tok_pos, const int *block_table, int mpps, int tokens,
                             int heads, int kv_heads, int dim, float scale, int chunk, int max_keys, cudaStream_t st, const int *tok_list = nullptr);
// tensor-core prefill variant over tiles of <= 64 consecutive tokens of one sequence: int4 {sequence, first packed row, rows, first position}
bool chunked_attention_tiles_supported(int dtype, int dim, int gate_ld);
int launch_chunked_attention_tiles(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in,
                                   int gate_ld, void *out, const int *tiles, int n_tiles, const int *block_table, int mpps, int heads,
                                   int kv_heads, int dim, float scale, int chunk, cudaStream_t st);

// attention_latent.cu (layouts in the file's header): proj [tokens, ld] holds q at column q_col and, when kv_col >= 0, the down-projection
int launch_latent_prep(int dtype, const void *proj, int ld, int q_col, int kv_col, void *qn, void *qr, void *pool, const float *kv_norm,
                       float eps, const int *tok_seq, const int *tok_pos, const int *block_table, int mpps, int tokens, int t_pad, int heads,
                       int dim, int rot_dim, int kv_rank, int rot_dims, float rot_base, cudaStream_t st);
int launch_latent_attention(int dtype, const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tok_seq,
                            const int *tok_pos, const int *block_table, int mpps, int tokens, int t_pad, int heads, int kv_rank, int rot_dim,
                            float scale, int window, int max_keys, cudaStream_t st, const int *tok_list = nullptr);
// tensor-core form over tiles of <= 64 query rows that share their keys: int4 {sequence, first packed row, rows, first position};
// by_head == 0: consecutive tokens of one sequence x one head; by_head == 1: one token x 64 consecutive heads.  part (optional, by_head):
// fp32 [part_tiles, heads, kv_rank + 2] for the partial results when few tiles share out their keys over several CTAs
bool latent_attention_tiles_supported(int dtype, int kv_rank, int rot_dim);
int launch_latent_attention_tiles(int dtype, const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tiles,
                                  int n_tiles, const int *block_table, int mpps, int t_pad, int heads, int kv_rank, int rot_dim, float scale,
                                  int window, int by_head, float *part, int part_tiles, cudaStream_t st);
int launch_latent_gate(int dtype, const void *ov, const void *gate_in, int gate_ld, void *out, int tokens, int t_pad, int heads, int vdim,
                       cudaStream_t st);

// attention_scored.cu: proj [tokens, ld] holds q (heads*dim), k (kv_heads*dim), v (kv_heads*vdim) from column col0 on; b_in (optional) is
// counted from the same row.  q_out [tokens, heads*dim]; pools K [pages, kv_heads, page, dim], V [pages, kv_heads, page, vdim]
// options of the prep step: rot_half: rotating pairs (i, i + rot_dims/2) instead of (2i, 2i+1); rot_factor > 0: long wavelengths are slowed
// down (b200_hybrid_layer_t); v_norm: value heads are cached divided by their root mean square
struct ScoredPrepOptions { int rot_half = 0; float rot_factor = 0.0f, rot_low = 0.0f, rot_high = 0.0f, rot_original = 0.0f; int v_norm = 0; };
int launch_scored_prep(int dtype, const void *proj, int ld, int col0, const float *b_in, void *q_out, void *k_pool, void *v_pool,
                       const float *q_norm, const float *k_norm, float eps, const int *tok_seq, const int *tok_pos, const int *block_table,
                       int mpps, int tokens, int heads, int kv_heads, int dim, int vdim, int rot_dims, float rot_base, cudaStream_t st,
                       ScoredPrepOptions opt = ScoredPrepOptions());
int launch_scored_attention(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *dist_r1,
                            const float *dist_r2, const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale, const int *tok_seq,
                            const int *tok_pos, const int *block_table, int mpps, int tokens, int heads, int kv_heads, int dim, int vdim,
                            float scale, int window, int sigmoid, int max_keys, cudaStream_t st, const int *tok_list = nullptr,
                            float softcap = 0.0f);
bool scored_attention_tiles_supported(int dtype, int dim, int vdim, int gate_ld, int out_ld, int window, bool penalty);
int launch_scored_attention_tiles(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *dist_r1,
                                  const float *dist_r2, const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale,
                                  const int *tiles, int n_tiles, const int *block_table, int mpps, int heads, int kv_heads, int dim, int vdim,
                                  float scale, int window, int sigmoid, cudaStream_t st, float softcap = 0.0f);

// recurrent.cu: column offsets of the fp32 row per token that the prep kernels write and the recurrences read.
// launch_delta_prep scratch: lr (engine dtype) of tokens * (rank + gate_rank) elements + 256 bytes, za fp32 [tokens, heads*dim], zg fp32
// [tokens, heads*vdim]
struct DeltaRow { int q, k, v, decay, gate, beta, ld; };
struct MlstmRow { int q, k, v, gi, gf, ld; };
struct DecayRow { int q, k, v, skip, decay, ld; };  // q, k [kv_heads*dim] | v, skip [heads*vdim] | decay [heads]
DecayRow decay_row(int heads, int kv_heads, int dim, int vdim);
DeltaRow delta_row(int heads, int kv_heads, int dim, int vdim);
MlstmRow mlstm_row(int heads, int dim, int vdim);
int launch_delta_prep(int dtype, const void *proj, int ld, int col0, const float *conv_w, int taps, float *conv_state, const void *w_decay,
                      const float *decay_bias, const float *a_log, int rank, const void *w_gate2, int gate_rank, void *lr, float *za, float *zg,
                      float *rec, const int *tok_seq, const int *tok_pos, const int *seq_pos0, const int *seq_slot, int tokens, int heads,
                      int kv_heads, int dim, int vdim, cudaStream_t st);
int launch_conv_state_update(int dtype, const void *proj, int ld, int col0, float *conv_state, int taps, int channels, const int *seq_start,
                             const int *seq_pos0, const int *seq_slot, int n_seqs, cudaStream_t st);
// one_token: the host knows that every portion of the batch is a single token (a decode batch)
int launch_delta_recurrent(const float *rec, float *S, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs,
                           int heads, int kv_heads, int dim, int vdim, cudaStream_t st, int one_token = 0);
int launch_mlstm_prep(int dtype, const void *proj, int ld, int col0, const float *b_in, float cap, float *rec, int tokens, int heads, int dim,
                      int vdim, cudaStream_t st);
int launch_mlstm_recurrent(const float *rec, float *S, float *n_state, float *m_state, float *o, float *nq, float *m_out, const int *seq_start,
                           const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, cudaStream_t st, int one_token = 0);
// out[t, h*vdim + j] = out_scale * y * rsqrt(mean_j y^2 + eps) * w[h*w_stride + j] * sigmoid(gate); y = o, or o / (max(|nq|, exp(-m)) + 1e-6)
int launch_head_output(int dtype, const float *o, const float *nq, const float *m_in, const float *w, int w_stride, float eps,
                       const float *gate_f, int gate_f_ld, const void *gate_t, int gate_t_ld, void *out, int out_ld, float out_scale, int tokens,
                       int heads, int vdim, cudaStream_t st, int gate_act = 0);
// the delta rule with one decay per head and full-rank gates: proj row q | k | v | step (heads) | decay-in (heads) | gate (heads*vdim)
int launch_delta_prep_direct(int dtype, const void *proj, int ld, int col0, const float *conv_w, int taps, float *conv_state,
                             const float *decay_bias, const float *a_log, float *rec, const int *tok_seq, const int *tok_pos,
                             const int *seq_pos0, const int *seq_slot, int tokens, int heads, int kv_heads, int dim, int vdim, cudaStream_t st);
// the state-space mixer: proj row z | x (heads*vdim each) | B | C (groups*state each) | dt (heads); conv_state [slots, taps - 1, channels]
// over the channels x | B | C; writes the tokens' DecayRow (kv_heads = groups, dim = state)
int launch_ssd_prep(int dtype, const void *proj, int ld, int col0, const float *conv_w, const float *conv_b, int taps, float *conv_state,
                    const float *dt_bias, const float *a_log, const float *skip_w, float *rec, const int *tok_seq, const int *tok_pos,
                    const int *seq_pos0, const int *seq_slot, int tokens, int heads, int groups, int state, int vdim, cudaStream_t st);
// linear attention with a constant decay per head: proj row q | k (heads*dim each) | v | gate (heads*vdim each); writes the DecayRow
int launch_linear_prep(int dtype, const void *proj, int ld, int col0, const float *head_decay, float *rec, int tokens, int heads, int dim, int vdim,
                       cudaStream_t st);
// S <- decay S + k v^T;  o = S^T q over every sequence's portion, from the tokens' DecayRow
int launch_decay_recurrent(const float *rec, float *S, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs,
                           int heads, int kv_heads, int dim, int vdim, cudaStream_t st, int one_token = 0);
// out[t, c] = T((o + skip)[t, c] (* act(gate) if gate_first) * rsqrt(mean over the column's group + eps) * w[c] (* act(gate) if not)),
// `groups` equal groups of the `cols` columns; act = sigmoid (gate_act 0) or silu (1); skip may be NULL
int launch_group_output(int dtype, const float *o, const float *skip, int skip_ld, const float *w, float eps, const void *gate, int gate_ld,
                        int gate_act, int gate_first, void *out, int out_ld, int tokens, int cols, int groups, cudaStream_t st);

// gla.cu
// decay[t, c] = sigmoid(z)^(1/tau), z = w_decay[c, :] . proj[t, col0 : col0 + rank] + bias[c]   (fp32 from the projection on)
int launch_gla_decay(int dtype, const void *proj, int ld, int col0, const void *w_decay, const float *bias, float tau, float *decay,
                     int tokens, int rank, int channels, cudaStream_t st);
// kinds: which portions the batch holds, when the host knows (one-token portions have a kernel of their own; the default launches both)
constexpr int kGlaOneToken = 1, kGlaManyTokens = 2;
int launch_gla_recurrent(int dtype, const void *proj, int ld, const float *decay, float *state, float *o, const int *seq_start,
                         const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, cudaStream_t st,
                         int kinds = kGlaOneToken | kGlaManyTokens);
// out[t, h*vdim + j] = o[t,h,j] * rsqrt(mean_j o^2 + eps) * w[j] * silu(gate[t*gate_ld + h*vdim + j])
int launch_gla_output(int dtype, const float *o, const float *w, float eps, const void *gate_in, int gate_ld, void *out, int tokens,
                      int heads, int vdim, cudaStream_t st);

// moe.cu
int launch_moe_route_sigmoid(const float *logits, int ld, int *sel_expert, float *sel_weight, float *shared_gate, int tokens,
                             int experts, int top, cudaStream_t st);
// scores = softmax over `outputs` router outputs; choice by score + bias (NULL: none); weights = chosen scores / (their sum + 1e-20)
int launch_moe_route_softmax(const float *logits, int ld, const float *bias, int *sel_expert, float *sel_weight, int tokens, int outputs,
                             int top, cudaStream_t st);
constexpr int kMoeTileM = 64;  // rows of one expert are padded to whole tiles of this many (128 when the tcgen05 grouped GEMM runs)
// Groups the (token, choice) pairs by expert.  row_token / row_weight [max_rows]: token of every padded row (-1: padding) and its routing
// weight; tile_expert [max_tiles]; pair_row [tokens*top]: the row each pair landed in (-1 for a choice >= experts: an identity expert);
// n_tiles: device int.
int launch_moe_plan(const int *sel_expert, const float *sel_weight, int *row_token, float *row_weight, int *tile_expert, int *pair_row,
                    int *n_tiles, int tokens, int experts, int top, int tile, cudaStream_t st);
// xg[row, :] = T(weight[row] * x[token[row], :]) (zeros for padding rows): the routing weight multiplies the expert's INPUT
int launch_moe_gather(int dtype, const float *x, const int *row_token, const float *row_weight, void *xg, const int *n_tiles,
                      int max_rows, int width, int tile, cudaStream_t st);
// xg[row, :] = h[token[row], :] of the engine dtype (zeros for padding rows)
int launch_moe_gather_rows(int dtype, const void *h, const int *row_token, void *xg, const int *n_tiles, int max_rows, int width, int tile,
                           cudaStream_t st);
// out[r, c] = act(in[r, c]) * in[r, inner + c], in [rows, 2 * inner]; n_tiles (optional, device): only rows < *n_tiles * tile are live
int launch_gated_activation(int dtype, const void *in, void *out, int rows, int inner, int act, const int *n_tiles, int tile, cudaStream_t st);
// in place: x[r, c] = act(x[r, c] + bias[c]); bias NULL: none; act < 0: none
int launch_bias_activation(int dtype, void *x, const float *bias, size_t rows, int cols, int act, cudaStream_t st);
// gemm_tc.cu: the same product on tcgen05 for row tiles of 128 (16-bit dtypes, K >= 64 and a multiple of 8; B200_ERR_UNSUPPORTED otherwise)
int launch_gemm_tc_grouped(const void *a, const void *w, void *c, int max_rows, int N, int K, int experts, const int *tile_expert,
                           const int *n_live, int act, int dtype, cudaStream_t st);
// c[row, n] = act?(sum_k a[row, k] * w[tile_expert[row / kMoeTileM]][n, k]);  rows >= n_tiles * kMoeTileM are skipped
int launch_moe_grouped_gemm(int dtype, const void *a, const void *w, void *c, const int *tile_expert, const int *n_tiles, int max_tiles,
                            int N, int K, int act, cudaStream_t st);
// y fp32 [M, N] = x [M, K] * w[N, K]^T for 16-bit x and w on the tensor cores (fp32 accumulation, fp32 result); B200_ERR_UNSUPPORTED for
// fp32 engines and K not a multiple of 8 (the caller falls back to launch_proj_f32)
int launch_dense_f32out(int dtype, const void *x, const void *w, float *y, int M, int N, int K, cudaStream_t st);
// in place: x = act(x)
int launch_activation(int dtype, void *x, size_t n, int act, cudaStream_t st);

// hybrid.cu
// y[m, n] (fp32) = sum_k x[m*ldx + k] * w[n*K + k] (+ bias[n]);  x of type TX (fp32 when x_dtype == B200_F32), w of `w_dtype`
int launch_proj_f32(int x_dtype, const void *x, int ldx, int w_dtype, const void *w, const float *bias, float *y, int ldy, int M, int N,
                    int K, cudaStream_t st);

}  // namespace b200
