// C launch API of the kernels behind hybrid (attention + recurrent-state) decoders: stream_ops.cu, recurrent.cu,
// attention_window.cu.  Every size is a runtime argument.  "Step plan" arrays describe one engine step of E entries
// (each a run of consecutive tokens of one sequence) packed into T tokens:
//   cu[E+1]        token offset of every entry        tok_entry[T]   entry of every token
//   pos[T]         position of the token in its sequence            kv_slot[T]  physical KV slot (page * PAGE + offset)
//   start[E]       tokens the sequence held before this step (0 = fresh state)
//   state_slot[E]  recurrent-state slot of the entry's sequence     block_table[E, max_blocks]  KV pages
// Storage types: `f32` flags select float (1) or bf16 (0) for a typed operand; everything that is accumulated,
// normalised, exponentiated or carried from token to token is float.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Optional terms of the paged attention kernels: the mask's form, per-head score terms and a per-head output gate.
typedef struct {
  int chunked;               // 0: sliding window, key j seen from position p when p - window < j <= p
                             // 1: chunks of `window` positions counted from position 0: floor(j / window) == floor(p / window), j <= p
  const float* head_scale;   // [Hq] or null: the score multiplier of head h is scale * head_scale[h]
  const float* head_slope;   // [Hq] or null: head_slope[h] * (p - j) is taken off the score
  const float* gate;         // [T, Hq] float (row stride gate_stride) or null: head h's output is multiplied by sigmoid(gate[t, h])
  long gate_stride;
  const float* head_sink;    // [Hq] or null: the softmax denominator also holds exp(head_sink[h]), a score without key or value
                             // (it is not multiplied by the scale and counts once)
  int kv_shared;             // 1: values are the first Dv columns of the key rows (v_cache == k_cache, rows of D): latent attention
  long q_head_stride;        // 0: head h of token t starts at q[t * sq + h * D]; else at q[t * sq + h * q_head_stride] (queries stored
                             // head-major, as a batched GEMM leaves them); scalar and latent kernels only
  float softcap;             // > 0: score <- softcap * tanh(score / softcap), after the scale and before the terms below
  int keep_first;            // > 0 (window form): keys at positions < keep_first stay visible however far back they lie
  const float* dist_bias;    // [dist_max + 1, Hq] or null: dist_bias[min(p - j, dist_max), h] is added to the score (not scaled)
  int dist_max;
  int v_div;                 // > 1: key head g reads the values of head g / v_div of a value cache with Hkv / v_div heads (several
                             // score maps over one set of values)
  float* out_float;          // non-null: the result goes here as float ([T, Hq * Dv], row stride out_float_stride) whatever the pages'
  long out_float_stride;     // type, and `out` is not written (results that are combined further before they are rounded)
} NrlAttnMods;

extern "C" {
// x0[t] = table[tok[t]] + pos_table[pos[t]]  (float out)
cudaError_t nrl_embed_pos(const void* embed, const void* pos_table, int w_f32, const int* tok, const int* pos, float* out,
                          int T, int W, cudaStream_t s);

// x0[t] = embed[tok[t]] * scale + pair[row] (float out): a hashed row per (previous token, token) pair,
//   row = (prev * mul_prev + tok * mul_cur) mod buckets, row `buckets` for the first token of a sequence; pair == nullptr: no
// such term.  The previous token of an entry's first token is read from prev_state[state_slot] (int [slots]); a second launch
// stores every entry's last token there.
cudaError_t nrl_embed_hashed(const void* embed, const void* pair, int w_f32, const int* tok, const int* cu, const int* tok_entry,
                             const int* start, const int* state_slot, int* prev_state, float scale, long mul_prev, long mul_cur,
                             long buckets, float* out, int T, int E, int W, cudaStream_t s);

// Sublayer boundary of a stream with a norm before and after every sublayer and a gated residual; norms are RMS norms over
// `groups` equal consecutive parts of the vector with a weight per column.
//   if (o)  y = o * sigmoid(gate + gate_bias)   (gate float, row stride sg, null: y = o);   x += y / rms_part(y) * w_post
//   if (h)  h (typed) = x / rms_part(x) * w_pre
cudaError_t nrl_group_norm_residual(float* x, const float* o, const float* gate, long sg, const float* gate_bias, const float* w_post,
                                    const float* w_pre, int groups, float eps, void* h, int h_f32, int T, int W, cudaStream_t s);

// Mixture-of-experts routing.  router float [T, E] (row stride sr) + router_bias [E]; the `top` largest logits (ties: lowest
// index) are chosen, weights = softmax over the chosen logits.  ids int [T, top], wts float [T, top] (either may be null).
// Dense form (act != nullptr): gu float (row stride sgu) holds per expert ff gate columns then ff up columns;
//   act[t, e*ff + c] (typed, row stride sa) = weight_e * silu(gate) * up, 0 for experts that were not chosen.
cudaError_t nrl_moe_route(const float* router, long sr, const float* router_bias, int E, int top, const float* gu, long sgu, int ff,
                          void* act, long sa, int act_f32, int* ids, float* wts, int T, cudaStream_t s);

// Grouped (sorted by expert) form of a mixture of experts, moe.cu.  ids int [R = T * top] from nrl_moe_route.
//   nrl_moe_plan: slot_of[R] = row of every (token, choice) pair in expert order, row_token[R] = token of every row,
//     seg[E + 1] = first row of every expert, tiles [*, 3] = (expert, first row, end row of the expert) per `tile_rows` rows of
//     an expert (at most ceil(R / tile_rows) + E of them), num_tiles[1]: the table of the grouped GEMM (gemm_tc.h).
//   nrl_gather_rows16: out[r] = in[row_token[r]] for rows of W 16-bit elements.
//   nrl_swiglu_rows: act[r, c] (bf16) = silu(gu[r, c]) * gu[r, ff + c].
//   nrl_moe_combine: out[t] (float) = sum_k wts[t, k] * y[slot_of[t * top + k]] in the order of k.
// n_real <= E: experts n_real .. E-1 get rows but no tiles (identity experts); nrl_moe_combine skips pairs of weight 0.
cudaError_t nrl_moe_plan(const int* ids, int R, int top, int E, int n_real, int tile_rows, int* slot_of, int* row_token, int* seg, int* tiles,
                         int* num_tiles, cudaStream_t s);
cudaError_t nrl_gather_rows16(const void* in, long in_stride, const int* row_token, void* out, int R, int W, cudaStream_t s);
cudaError_t nrl_swiglu_rows(const float* gu, long sg, void* act, long sa, int R, int ff, cudaStream_t s);
cudaError_t nrl_moe_combine(const float* y, long sy, const int* slot_of, const float* wts, int top, float* out, long so, int T, int W,
                            cudaStream_t s);

// Stream with the norm on the sublayer's output only (sublayers read x itself).
//   nrl_embed_norm:          x[t] = e / sqrt(mean(e^2) + eps) * w, e = embed[tok[t]] (typed table);  h = x (typed)
//   nrl_post_norm_residual:  y = o + self_w[t] * x (self_w [T] or null: y = o);  x += y / sqrt(mean(y^2) + eps) * w_post;
//                            h (typed, may be null) = w_pre ? x / sqrt(mean(x^2) + eps) * w_pre : x
cudaError_t nrl_embed_norm(const void* embed, int w_f32, const int* tok, const float* w, float eps, float* x, void* h, int h_f32, int T,
                           int W, cudaStream_t s);
cudaError_t nrl_post_norm_residual(float* x, const float* o, const float* self_w, const float* w_post, const float* w_pre, float eps,
                                   void* h, int h_f32, int T, int W, cudaStream_t s);
// Gated token-side input: out[t, c] (typed, row stride so) = gelu_tanh(u[t, c]) * table[tok[t], col0 + c] for c < C, 0 for C <= c < Cpad
// (u float, row stride su; table typed, row stride st_).
cudaError_t nrl_side_gate(const float* u, long su, const void* table, long st_, int w_f32, int col0, const int* tok, void* out, long so,
                          int out_f32, int T, int C, int Cpad, cudaStream_t s);
// out[t, c] (typed) = silu(in[t, c]) * in[t, C + c] * (rgate ? sigmoid(rgate[t * srg]) : 1)
cudaError_t nrl_swiglu_cols(const float* in, long si, const float* rgate, long srg, void* out, long so, int out_f32, int T, int C,
                            cudaStream_t s);
// Routing by a softmax over all E router outputs; the last E - n_real are identity experts.  The `top` largest
// softmax + correction (correction [E] or null; ties: lowest index) are chosen; weight = softmax / (sum over the chosen + 1e-20)
// * route_scale.  ids [T, top]; wts [T, top] (0 for a chosen identity expert); self_w [T] = summed weights of the chosen
// identity experts (needed when n_real < E).  Dense form as nrl_moe_route, over the n_real experts.
// groups > 1: the E outputs form `groups` equal groups of neighbours; a group's score is its largest choice score (score +
// correction) and only experts of the `keep` best groups can be chosen (the others count as -inf; ties: the lower group).
cudaError_t nrl_moe_route_all(const float* router, long sr, const float* correction, int E, int n_real, int top, float route_scale,
                              int groups, int keep, const float* gu, long sgu, int ff, void* act, long sa, int act_f32, int* ids,
                              float* wts, float* self_w, int T, cudaStream_t s);

// Layer boundary of a depth-weighted residual stream.  results: float [n_results_cap, stride_r] with rows of W.
//   if (o)  results[i] = xprev + o                      (closes the previous layer)
//   x = sum_{j <= i} dw[j] * results[j]   (dw == nullptr: x = results[i])      -> xcur (float)
//   h = x / sqrt(mean(x^2) + eps) * g[0]                                        -> h (typed)
cudaError_t nrl_stream_norm(float* results, long stride_r, int i, const float* o, const float* xprev, const float* dw,
                            const float* g, float eps, float* xcur, void* h, int h_f32, int T, int W, cudaStream_t s);

// out[t, c] (typed, row stride so, pre-offset) = act(in[t, c]) (float, row stride si);  act: 0 copy, 1 relu^2
cudaError_t nrl_act_cols(const float* in, long si, void* out, long so, int out_f32, int act, int T, int C, cudaStream_t s);

// Part-wise gated RMS norm:  y [T, n] float (row stride sy), gate float (row stride sg).  Parts of `part` columns.
//   gate_first: v = y * act(gate); v /= rms_part(v); v *= w        else: v = y / rms_part(y) * w * act(gate)
//   w index = shared_w ? (c % part) : c.   gate_act: 0 silu, 1 sigmoid.   out typed = scale * v
cudaError_t nrl_gated_part_rmsnorm(const float* y, long sy, const float* gate, long sg, const float* w, int shared_w, int part,
                                   int gate_act, int gate_first, float eps, float scale, void* out, long so, int out_f32,
                                   int T, int n, cudaStream_t s);

// Depthwise causal convolution over time with carried taps.  in float [T, C] (row stride si) plus in_bias float [C] or null
// (a bias of the projection that produced `in`: it is part of the convolution's input and of the carried taps, while the
// time before a sequence's start is zero), w float [C, taps], bias float [C] or null (added after the convolution),
// state float [slots, taps-1, C] (oldest first).  out float [T, C] (row stride so) = act ? silu(y) : y.
// nrl_causal_conv reads the old state; nrl_causal_conv_carry (launched after it) stores the step's last taps-1 inputs.
cudaError_t nrl_causal_conv(const float* in, long si, const float* in_bias, int act, const float* w, const float* bias,
                            const float* state, float* out, long so, const int* cu, const int* tok_entry, const int* start,
                            const int* state_slot, int T, int E, int C, int taps, cudaStream_t s);
cudaError_t nrl_causal_conv_carry(const float* in, long si, const float* in_bias, float* state, const int* cu, const int* start,
                                  const int* state_slot, int E, int C, int taps, cudaStream_t s);

// State-space scan (scalar decay per head).  xbc float [T, *] (row stride sx): x at column 0 (heads*P), B at col_b, C at col_c
// (groups*N each).  dt_raw float (row stride sd) [T, heads].  state float [slots, heads, N, P].
//   dt = softplus(dt_raw + dt_bias);  S = exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x      -> y float [T, heads*P]
cudaError_t nrl_ssd_scan(const float* xbc, long sx, int col_b, int col_c, const float* dt_raw, long sd, const float* dt_bias,
                         const float* A_log, const float* Dskip, float* state, float* y, const int* cu, const int* start,
                         const int* state_slot, int E, int heads, int groups, int N, int P, int impl, cudaStream_t s);
// `impl` of both scans: 0 picks by size; 1 a state column per thread (rows <= 128); 2 row groups of a column per thread;
// 3 the state in shared memory.  A kernel that does not fit the sizes returns cudaErrorInvalidValue.

// Gated delta rule inputs.  qkv float [T, *] (row stride sq): q at column 0, k at col_k (kv_heads*D each); both are made unit
// vectors per head in place (x / sqrt(sum x^2 + 1e-6)), q also times D^-1/2.  beta = sigmoid(b_raw).
// decay = exp(-exp(A_log[h]) * softplus(a_raw + dt_bias)) with a_raw / dt_bias / decay [heads] or, per_channel, [heads*D].
cudaError_t nrl_delta_prep(float* qkv, long sq, int col_k, const float* b_raw, long sb, const float* a_raw, long sa,
                           const float* dt_bias, const float* A_log, float* beta, float* decay, int T, int heads, int kv_heads,
                           int D, int per_channel, cudaStream_t s);

// Gated linear attention inputs.  qkv float [T, *] (row stride sq): q at column 0 (heads*D) is multiplied by D^-1/2 in place.
// decay [T, heads*D] = sigmoid(a_raw + a_bias)^(1 / tau) per key channel (a_raw float, row stride sa; a_bias [heads*D] or null).
cudaError_t nrl_gla_prep(float* qkv, long sq, const float* a_raw, long sa, const float* a_bias, float tau, float* decay, int T,
                         int heads, int D, cudaStream_t s);

// Gated delta rule scan.  Per head: S = g S (rows);  u = beta (v - S^T k);  S += k u^T;  o = S^T q.
// beta == nullptr: plain accumulation, u = v (gated linear attention: S = diag(g) S + k v^T).
// state float [slots, heads, D, Dv];  o float [T, heads*Dv].
cudaError_t nrl_delta_scan(const float* qkv, long sq, int col_k, int col_v, const float* beta, const float* decay, float* state,
                           float* o, const int* cu, const int* start, const int* state_slot, int E, int heads, int kv_heads, int D,
                           int Dv, int per_channel, int impl, cudaStream_t s);

// Per-head RMS norm (weight [D], shared by heads) of q in place and of k into the paged cache; v into the paged cache.
// q float [T, Hq*D] (row stride sq), k float [T, Hkv*D], v float [T, Hkv*Dv] (row strides sk, sv).
// k_cache typed [pages, Hkv, page, D], v_cache typed [pages, Hkv, page, Dv].
cudaError_t nrl_qknorm_kv_write(float* q, long sq, const float* k, long sk, const float* v, long sv, const float* qw, const float* kw,
                                float eps, void* k_cache, void* v_cache, int cache_f32, const int* kv_slot, int T, int Hq, int Hkv,
                                int D, int Dv, int page, cudaStream_t s);

// Latent attention, write side.  dkv float [T, rank + dr] (row stride sd): the first `rank` columns are RMS-normed with weight w
// [rank] (eps inside the root), the last dr are one key part shared by all heads; both go into the token's row of `cache`
// (typed [pages, 1, page, rank + dr]).  q float [T, H * (dn + dr)]: every head's last dr columns go to qa [T, H, rank + dr]
// (row stride sqa, head stride sha) behind the head's `rank` absorbed columns, which the caller fills; qn (bf16 [H, T, dn]) or
// null: the heads' first dn columns as the operand of that batched GEMM.  The first `rdims` of the dr columns
// of keys and queries are rotated by the angles pos * freq[i] (freq double [rdims / 2]), cos and sin times `mult`;
// interleaved = 1 pairs column 2i with 2i + 1, 0 pairs i with i + rdims / 2.
cudaError_t nrl_latent_kv_write(const float* q, long sq, int H, int dn, int dr, const float* dkv, long sd, int rank, const float* w,
                                float eps, const double* freq, int rdims, float mult, int interleaved, const int* pos, const int* kv_slot,
                                void* cache, int cache_f32, int page, float* qa, long sqa, long sha, void* qn, int T, cudaStream_t s);

// Keys and values of a step's tokens into their pages, the values optionally blended with another layer's values of the
// same tokens:  v <- (1 - lambda[0]) v + lambda[0] v_other  (v_other float, row stride svo, null: plain copy; lambda on device).
// k float [T, Hkv*D] (row stride sk), v float [T, Hkv*Dv] (row stride sv); v is also updated in place when blended.
cudaError_t nrl_kv_write_blend(const float* k, long sk, float* v, long sv, const float* v_other, long svo, const float* lambda,
                               void* k_cache, void* v_cache, int cache_f32, const int* kv_slot, int T, int Hkv, int D, int Dv, int page,
                               cudaStream_t s);

// Softmax attention over the paged cache: token at position p sees keys p-window+1 .. p (or, mods->chunked, the keys of its
// chunk up to p).  out typed (row stride so) = out_scale * softmax(scale q.k) v, with the optional terms of `mods` (null: none).
// single_token: every entry of the step holds one token.
cudaError_t nrl_window_attention(const float* q, long sq, const void* k_cache, const void* v_cache, int cache_f32,
                                 const int* block_table, int max_blocks, const int* tok_entry, const int* pos, int window,
                                 float scale, float out_scale, void* out, long so, int out_f32, int T, int Hq, int Hkv, int D,
                                 int Dv, int page, int single_token, int impl, int nsplit, float* part, const NrlAttnMods* mods,
                                 cudaStream_t s);
// `nsplit` >= 1 with `part` float [T, Hq, 4 nsplit, Dv + 2] (steps of single tokens over bf16 pages): every warp of nsplit
// blocks per (token, key/value head) walks its own pages and a second launch merges the parts; nrl_window_attention_splits
// proposes the count (0: the shape does not fit).
// `impl`: 0 picks by shape and step kind, 1 the scalar tile kernel, 2 one block per (token, head), 3 the tensor-core kernel.

// Latent attention on the tensor cores (attention_latent_mma.cu): causal attention of H absorbed queries per token (q float
// [T, H * D]) over bf16 pages [pages, 1, 16, D] whose rows are key and, in their first Dv columns, value of every head; sink
// and gate from `mods`.  `_fits`: D, Dv multiples of 8, Dv <= D <= 576.  Single-token steps with nsplit >= 1 and `part` float
// [T, H, 4 nsplit, Dv + 2] use the per-warp page walk + merge; `_splits` proposes the count.
int nrl_latent_attention_mma_fits(const void* out, long so, int D, int Dv, int page);
int nrl_latent_attention_splits(int T, int H, int Dv, int max_blocks);
cudaError_t nrl_latent_attention_mma(const float* q, long sq, const void* cache, const int* block_table, int max_blocks,
                                     const int* tok_entry, const int* pos, float scale, float out_scale, void* out, long so, int T, int H,
                                     int D, int Dv, int page, int single_token, int nsplit, float* part, const NrlAttnMods* mods,
                                     cudaStream_t s);

// Tensor-core kernel for prompt portions over bf16 pages of 16 tokens (attention_window_mma.cu); `_fits` says whether the
// shapes and the output's alignment allow it.
int nrl_window_attention_mma_fits(const void* out, long so, int Hq, int Hkv, int D, int Dv, int page);
int nrl_window_attention_splits(int T, int Hq, int Hkv, int window, int max_blocks, int page);
cudaError_t nrl_window_attention_decode(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table,
                                        int max_blocks, const int* tok_entry, const int* pos, int window, float scale,
                                        float out_scale, void* out, long so, int T, int Hq, int Hkv, int D, int Dv, int page,
                                        int nsplit, float* part, const NrlAttnMods* mods, cudaStream_t s);
cudaError_t nrl_window_attention_mma(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table,
                                     int max_blocks, const int* tok_entry, const int* pos, int window, float scale, float out_scale,
                                     void* out, long so, int T, int Hq, int Hkv, int D, int Dv, int page, int single_token,
                                     const NrlAttnMods* mods, cudaStream_t s);
// Several residual streams mixed by learned weights (hyper-connections), layer norms with weight and bias.  xs float [T, S, W].
//   nrl_embed_streams:   xs[t, s] = embed[tok[t]] * scale for every stream s
//   nrl_hyper_boundary:  if (o)  y = o + o_bias + self_w[t] * h[t]  (o float [T, W]; o_bias [W], self_w [T] or null; h still holds
//                                the closing sublayer's input);  x_t <- sum_s mix[s, t] x_s + outw[t] y for all t at once
//                                (mix [S, S] indexed [from, to], outw [S]; null: identity / ones)
//                        if (h)  u = sum_s inw[s] x_s (inw null: the plain sum);  h (typed) = (u - mean) / sqrt(var + eps) * ln_w + ln_b
cudaError_t nrl_embed_streams(const void* embed, int w_f32, const int* tok, float scale, float* xs, int T, int S, int W, cudaStream_t s);
cudaError_t nrl_hyper_boundary(float* xs, int S, const float* o, const float* o_bias, const float* self_w, const float* mix,
                               const float* outw, const float* inw, const float* ln_w, const float* ln_b, float eps, void* h, int h_f32,
                               int T, int W, cudaStream_t s);

// Matrix memory with exponential gates (mLSTM).  qkv float [T, *] (row stride sq): q at col_q, k at col_k (heads * D each), v at
// col_v (heads * Dv), raw gates at col_i / col_f (heads each; i_bias / f_bias [heads] or null are added).
//   i = cap tanh(raw_i / cap);  f = logsigmoid(cap tanh(raw_f / cap))  (cap <= 0: no cap);  m' = max(f + m, i)
//   S = exp(f + m - m') S + exp(i - m') k [v, 1]^T      state float [slots, heads, D, Cs], Cs >= Dv + 1 (column Dv is the normaliser n;
//                                                       rows padded to a multiple of 8 floats keep the accesses on sector borders)
//   o [T, heads, Dv + 1] = S^T (q * q_scale)            mstate float [slots, heads] carries m (0 for a new sequence); m_out [T, heads]
// `impl`: 0 picks by size, 1 a state column per thread in registers (D <= 128), 2 the state in global memory.  single_token: every
// entry holds one token (two threads then share a column of a 128-row state).
//   nrl_mlstm_out:  y = o[:Dv] / (max(|o[Dv]|, exp(-m)) + 1e-6);  out (typed) = scale * y / rms_head(y) * w * sigmoid(gate)
//                   (gate float [T, heads * Dv], row stride sg; w [heads * Dv])
cudaError_t nrl_mlstm_scan(const float* qkv, long sq, int col_q, int col_k, int col_v, int col_i, int col_f, const float* i_bias,
                           const float* f_bias, float cap, float q_scale, float* state, float* mstate, float* o, float* m_out,
                           const int* cu, const int* start, const int* state_slot, int E, int heads, int D, int Dv, int Cs,
                           int single_token, int impl, cudaStream_t s);
cudaError_t nrl_mlstm_out(const float* o, const float* m, const float* gate, long sg, const float* w, float eps, float scale, void* out,
                          long so, int out_f32, int T, int heads, int Dv, cudaStream_t s);

// Write side of rotated attention.  q float [T, Hq * D] (in place), k float [T, Hk * D], v float [T, Hv * Dv] or null (the values
// are then the keys as projected, bias included: Hv == Hk, Dv == D); biases [heads * D] or null.  The first `rdims` columns of every
// head turn by pos * freq[i] (freq double [rdims / 2]; cos and sin times mult; interleaved 1: pairs (2i, 2i + 1), 0: (i, i + rdims / 2));
// unit_norm: q and k are then divided by their root mean square per head (eps inside the root; times q_norm_w / k_norm_w [D] when
// given).  k == nullptr: queries only.  Caches typed [pages, heads, page, D or Dv].
cudaError_t nrl_rot_kv_write(float* q, long sq, const float* q_bias, const float* k, long sk, const float* k_bias, const float* v, long sv,
                             const double* freq, int rdims, float mult, int interleaved, int unit_norm, const float* q_norm_w,
                             const float* k_norm_w, float eps, const int* pos, const int* kv_slot, void* k_cache, void* v_cache,
                             int cache_f32, int page, int T, int Hq, int Hk, int Hv, int D, int Dv, cudaStream_t s);
// Differential attention, read side.  a typed [T, 2 H, Dv] (row stride sa): outputs of the two score maps, heads ordered (key/value
// head, map, query head of the group).  o = a_1 - lambda a_2;  out (typed, [T, H * Dv] in the order key/value head, query head)
// = out_scale * post * o / rms_head(o) * sigmoid(gate)   (gate float [T, H * Dv], row stride sg, or null)
cudaError_t nrl_diff_combine(const void* a, long sa, int a_f32, float lambda, float post, float eps, const float* gate, long sg,
                             float out_scale, void* out, long so, int out_f32, int T, int H, int Hkv, int Dv, cudaStream_t s);
}
