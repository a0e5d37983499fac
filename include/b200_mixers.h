/* C ABI of libb200mixers.so: sequence-mixing and normalisation kernels for decoder layers that are not plain softmax
 * attention -- Dynamic-Tanh normalisation fused with the residual update, sliding-window attention with sigmoid weights,
 * short causal convolutions, the gated delta rule and gated linear attention recurrences, PolyNorm, gated RMS output norm,
 * soft-capped logits.  All pointers are device pointers; every function enqueues on `stream` and returns 0 or a cudaError_t.
 *
 * dtype: 0 = float, 1 = bfloat16, 2 = half: the type of activations AND of parameters (a model lives in one type).
 * Whatever the dtype, the residual stream, attention scores and weights, every normalisation and everything inside a
 * recurrence (state, decays, gates, unit vectors) are 32-bit floats.
 *
 * Batches: a row holds S new tokens that follow the tokens of earlier calls; `slot0` numbers the first new token's slot
 * (the same for all rows) and `pad[b]` is row b's left padding: its token in slot c has position c - pad[b] and does not
 * exist when that is negative. */
#ifndef B200_MIXERS_H
#define B200_MIXERS_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct CUstream_st* mixers_stream_t;

/* x[n, :] = float(table[ids[n], :]) */
int mixers_embed_rows(int dtype, const void* table, const int64_t* ids, long n_rows, int width, float* x, mixers_stream_t stream);

/* x += tanh(post_alpha * y) * post_w + post_b   (if y);   x += add (if add);   out = tanh(pre_alpha * x) * pre_w + pre_b (if out).
 * x: float [n_rows, width], updated in place; y, out: dtype [n_rows, width]; vectors [width]; alphas: one element each. */
int mixers_dyt_residual_norm(int dtype, float* x, long n_rows, int width, const void* y, const void* post_w, const void* post_b,
                             const void* post_alpha, const void* add, const void* pre_w, const void* pre_b, const void* pre_alpha,
                             void* out, mixers_stream_t stream);

/* Queries, keys and values of new tokens taken from the columns of one projection output `proj` [B, S, ld]: per-head RMS norm
 * (weights q_w / k_w [dim]), rotation of the pairs (2i, 2i+1), i < rot_dims / 2, by position * inv_freq[i] (doubles: the angle is formed and its sine / cosine taken in double precision); queries go to
 * q_out float [B, S, heads, dim], keys and values into the caches k_store [B, kv_heads, cap, dim] / v_store [.., vdim] at
 * storage index held + t.  The token at storage index j sits in slot j + shift.  dyn (may be null): a device word that holds
 * `held` instead of the argument, for a step that is replayed from a CUDA graph while the cache grows. */
int mixers_window_qk_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads,
                             int kv_heads, int dim, int vdim, const void* q_w, const void* k_w, float eps, const double* inv_freq,
                             int rot_dims, float* q_out, void* k_store, void* v_store, int cap, int held, int shift,
                             const int32_t* pad, const int32_t* dyn, mixers_stream_t stream);

/* out[b, t, out_col + h * vdim + :] = out_scale * sum_j sigmoid(q . k_j * scale + head_bias[h]) v_j over the keys j of the same
 * row with 0 <= c - j < window (c = held + t the query's own storage index) that are not padding.  out: dtype [B * S, ld_out]. */
int mixers_sigmoid_window_attention(int dtype, const float* q, const void* k_store, const void* v_store, int B, int S, int heads,
                                    int kv_heads, int dim, int vdim, int cap, int held, int shift, const int32_t* pad, int window,
                                    float scale, const void* head_bias, void* out, int ld_out, int out_col, float out_scale,
                                    const int32_t* dyn, mixers_stream_t stream);

/* y[b, t, c] = silu(sum_j w[c, j] * in(t - taps + 1 + j)): in(t') = proj[b, t', off + c] for a new token, tail[b, taps-1+t', c]
 * for t' < 0, zero for padding.  tail_next receives the last taps-1 inputs (for S == 1 it may be `tail` itself: a thread
 * then owns its channel's whole tail).  w: [C, taps]; tails: [B, max(taps-1,1), C].  In this and the two recurrences `pad` may
 * be null: none of the new tokens is padding (true for every call but a batch's first). */
int mixers_short_conv_silu(int dtype, const void* proj, int B, int S, int ld, int off, int C, int taps, const void* w,
                           const void* tail, void* tail_next, int slot0, const int32_t* pad, void* y, mixers_stream_t stream);

/* Gated delta rule.  conv [B, S, C]: q | k (kv_heads x dim each) | v (heads x vdim) after the short convolution; q and k are
 * made unit vectors here (q also times dim^-1/2).  beta = sigmoid(proj[.., off_b + h]), decay = exp(-exp(A_log[h]) *
 * softplus(proj[.., off_a + h] + dt_bias[h])).  Per head:  M <- decay M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q.
 * state: float [B, heads, dim, vdim], updated in place; o: float [B, S, heads, vdim]. */
int mixers_gated_delta_rule(int dtype, const void* conv, int B, int S, int kv_heads, int heads, int dim, int vdim,
                            const void* proj, int ld, int off_b, int off_a, const void* A_log, const void* dt_bias, float* state,
                            int slot0, const int32_t* pad, float* o, mixers_stream_t stream);

/* Gated linear attention.  proj [B, S, ld]: q | k (heads x dim each) | v (heads x vdim) from column 0; z [B, S, heads * dim]:
 * decay logits, alpha = sigmoid(z)^(1/tau).  Per head:  M <- diag(alpha) M + k v^T;  o = M^T (q dim^-1/2). */
int mixers_gated_linear_attention(int dtype, const void* proj, int B, int S, int ld, int heads, int dim, int vdim, const void* z,
                                  float tau, float* state, int slot0, const int32_t* pad, float* o, mixers_stream_t stream);

/* out[n, out_col + h * vdim + c] = out_scale * o[n, h, c] / rms(o[n, h, :]) * w[c] * silu(gate[n, off_g + h * vdim + c]) */
int mixers_gated_rms_norm(int dtype, const float* o, long n_rows, int heads, int vdim, const void* gate, int ld_gate, int off_g,
                          const void* w, float eps, void* out, int ld_out, int out_col, float out_scale, mixers_stream_t stream);

/* out = a N(z) + b N(z^2) + c N(z^3) + e, N(v) = v / rms(v) over a row; coef = {a, b, c, e} */
int mixers_poly_norm(int dtype, const void* z, long n_rows, int width, const void* coef, float eps, void* out, mixers_stream_t stream);

/* out = cap * tanh(x / cap) as floats (cap <= 0: a plain conversion) */
int mixers_soft_cap(int dtype, const void* x, long n, float cap, float* out, mixers_stream_t stream);

/* ---- designs that normalise a sublayer's OUTPUT, cache a key/value latent and route tokens to experts ---- */

/* x[n, :] = table[ids[n], :] * scale + pair[row(n), :] as floats (x_copy, if given, gets the same; h, if given, the same in
 * dtype).  row(n) = (previous id * mul_prev + ids[n] * mul_cur) mod buckets; `buckets` itself for a sequence's first token
 * (position 0); the token before a call's first token is prev[b].  pair may be null (no second table).  ids: [B, S]; padding
 * slots (position < 0) give zeros.  pad may be null when slot0 > 0 (no new token is padding or a first token then): a step that
 * is replayed from a CUDA graph has no current slot0 to give. */
int mixers_embed_pair(int dtype, const void* table, float scale, const void* pair, long buckets, long mul_prev, long mul_cur,
                      const int64_t* ids, const int64_t* prev, int B, int S, int width, int slot0, const int32_t* pad, float* x,
                      float* x_copy, void* h, mixers_stream_t stream);

/* x += y / rms(y) * gain[0] * vec[:]  (gain, vec: dtype, either may be null; y: dtype, or float if y_is_float; rms over a row
 * with eps inside the root).  With `stack` (float [streams, n_rows, width], stack_stride = n_rows * width) the new x is stored
 * as stream `index`, and with `coef` (dtype [index + 1]) x becomes sum_{j <= index} coef[j] * stack[j].  h (may be null): x in dtype. */
int mixers_rms_residual(int dtype, float* x, long n_rows, int width, const void* y, int y_is_float, const void* gain, const void* vec,
                        float eps, float* stack, long stack_stride, int index, const void* coef, void* h, mixers_stream_t stream);

/* out = x / rms(x) * gain[0] * vec[:]   (x float, out dtype; gain, vec may be null) */
int mixers_rms_norm_rows(int dtype, const float* x, long n_rows, int width, const void* gain, const void* vec, float eps, void* out,
                         mixers_stream_t stream);

/* xIELU with pq = {p, q}; with a = softplus(p) and c = 1/2 + softplus(q): f(z) = a z^2 + z/2 where z is positive, c (expm1(z) - z) + z/2 elsewhere */
int mixers_xielu(int dtype, const void* z, long n, const void* pq, void* out, mixers_stream_t stream);

/* out[n, c] = silu(in[n, off_gate + c]) * in[n, off_up + c], c < cols; in: [n_rows, ld] */
int mixers_silu_mul(int dtype, const void* in, long n_rows, int ld, int off_gate, int off_up, int cols, void* out, mixers_stream_t stream);

/* out[n, c] = gelu_tanh(g[n, c]) * table[ids[n], col0 + c], c < cols */
int mixers_gelu_table_mul(int dtype, const void* g, long n_rows, int cols, const void* table, int ld_table, int col0, const int64_t* ids,
                          void* out, mixers_stream_t stream);

/* RMS norms (plain weights q_w [q_rank], c_w [kv_rank]) of two column ranges of proj [B, S, ld]: columns off_q.. -> cq_out
 * [B * S, q_rank]; columns off_c.. -> store [B, cap, kv_rank] at storage index held + t (zeros for padding).  dyn as above. */
int mixers_latent_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int q_rank, const void* q_w, int off_c,
                          int kv_rank, const void* c_w, float eps, void* cq_out, void* store, int cap, int held, int shift,
                          const int32_t* pad, const int32_t* dyn, mixers_stream_t stream);

/* Causal softmax attention of S new tokens per row.  q: head h of token n at q + n * q_ld + h * q_hs.  Key (value) of storage
 * index j, row b, kv head g at k + b * k_bs + j * k_ps + g * k_hs (strides in elements).  The query at storage index c = held
 * + t sees the keys j <= c of its row that are not padding (j + shift >= pad[b]) and, if window > 0, c - j < window.  Scores
 * (q . k) * scale and the softmax weights are 32-bit.  out[n, out_col + h * vdim + :] in dtype (zeros for padding queries).
 * allow_tensor_cores: 16-bit models may take the tensor-core kernels: for S >= 16 one block per 64 tokens of a head (head sizes
 * multiples of 16, <= 256); for S <= 16 and at least 4 query heads per kv head one pass over the keys for all heads of a
 * group, the keys split over blocks (dim a multiple of 16, <= 512; vdim 128, 256 or 512), which needs `ws`:
 * mixers_softmax_attention_workspace(...) floats (0: these sizes never take that kernel).  dyn as above. */
int mixers_softmax_attention(int dtype, const void* q, long q_ld, long q_hs, const void* k, long k_bs, long k_ps, long k_hs, const void* v,
                             long v_bs, long v_ps, long v_hs, int B, int S, int heads, int kv_heads, int dim, int vdim, int held,
                             int shift, const int32_t* pad, int window, float scale, void* out, long ld_out, int out_col,
                             const int32_t* dyn, int allow_tensor_cores, float* ws, mixers_stream_t stream);
long mixers_softmax_attention_workspace(int dtype, int B, int S, int heads, int kv_heads, int dim, int vdim);

/* Router of a mixture of experts.  z = router h (32-bit; router [n_out, width], h [n_rows, width] in dtype), s = softmax(z) over
 * all n_out outputs, choice = s + correction.  Outputs [g * n_out / groups, (g + 1) * n_out / groups) are group g; groups are
 * ranked by max(choice) over their members, the `keep` first groups stay eligible (every other output is out of the running,
 * whatever its sign), and the `top` eligible outputs of highest choice win.
 * idx_out int32 [n_rows, top] (n_out where nothing was left to choose), w_out float [n_rows, top] = s of the chosen. */
int mixers_grouped_router(int dtype, const void* h, long n_rows, int width, const void* router, const void* correction, int n_out,
                          int groups, int keep, int top, int32_t* idx_out, float* w_out, mixers_stream_t stream);

/* The chosen experts of a few tokens without host work.  gate_up[e] / down[e]: addresses of expert e's [2 ff_e, width] (gate rows,
 * then up rows) and [width, ff_e] matrices in dtype; ffs[e] = ff_e (null: `ff` for all; `ff` is the largest).  always_on != 0:
 * table entry n_experts is an expert that every token runs with weight 1 (a shared expert).  act: scratch dtype [n_rows, top +
 * (always_on ? 1 : 0), ff].  y float [n_rows, width] = sum_k w_k * down_e (silu(gate_e h) * (up_e h)) for chosen e < n_experts,
 * w_k * h for n_experts <= e < n_out, + the always-on expert, + shared_out (dtype [n_rows, width], may be null). */
int mixers_moe_small(int dtype, const void* h, long n_rows, int width, int ff, int top, int n_experts, int n_out, const int32_t* idx,
                     const float* wgt, const int64_t* gate_up, const int64_t* down, const int32_t* ffs, int always_on,
                     const void* shared_out, void* act, float* y, mixers_stream_t stream);

/* Counting sort of n_pairs = n_rows * top (token, choice) pairs by chosen output idx[i] in [0, n_keys): counts[e] = pairs of e;
 * pos[i] = row of pair i among the sorted pairs; token_of[row] = i / top. */
int mixers_moe_sort(const int32_t* idx, long n_pairs, int top, int n_keys, int32_t* counts, int32_t* pos, int64_t* token_of,
                    mixers_stream_t stream);

/* y float [n_rows, width] = sum_k w[n, k] * rows[pos[n, k], :] for chosen e < n_experts, w * h[n, :] for identity experts,
 * + shared_out; rows: dtype [*, width], the experts' outputs on rows sorted by expert. */
int mixers_moe_combine(int dtype, const void* rows, const int32_t* pos, const int32_t* idx, const float* wgt, const void* h,
                       const void* shared_out, long n_rows, int width, int top, int n_experts, int n_out, float* y, mixers_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
