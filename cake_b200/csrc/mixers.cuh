// mixers.cuh — launch interface of the sequence mixers and the routed feed-forward of mixer-list blocks
// (cake_b200_block_load_mixer): latent attention (keys and values expanded from a cached low-rank latent), gated linear
// recurrences (a fixed decay per head, input-dependent decays of a state-space layer, or per-token factors of a matrix memory
// with exponential gates), the gated delta rule, softmax attention whose heads are mixed after the softmax, short causal
// convolutions, grouped unit norms with gates, norms and merges of sublayer outputs on the fp32 stream, embeddings with pair and
// position tables, and a mixture of experts with identity experts.  The kernels live in mixers.cu, a
// translation unit of its own; the entry points below take plain device pointers and a stream, so that any block
// structure can combine them.  Every function returns a cudaError_t cast to int and adds its launches to *launches.
//
// Nothing here follows a reference file: the reference has none of these layers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cake {
namespace mx {

// dtype codes are those of include/cake_b200.h (0 bf16, 1 f16, 2 f32): the type D of projections, caches and weights.
// Scores, softmax, norms, recurrent state, decays, routers and residual sums are fp32 whatever D is.

// ---- latent attention ------------------------------------------------------------------------------------------------
// Row m = (b, t) of a step of S tokens per batch row that starts at absolute position pos0.
struct LatentPrep {
  const void *proj;      // [M, ld] D: per head [dim | rot] query entries from column 0, then [rank | rot] at column kv_col
  int ld, kv_col;
  const void *norm_w;    // [rank] D
  const float *cos_t, *sin_t;  // [positions, rope_dims / 2]
  int rope_dims;         // <= rot: leading entries of the rotated part that are rotated (pairs i, i + rope_dims / 2)
  void *cache;           // [B, cap, rank + rot] D: the normed latent and the rotated shared key part
  void *cache_t;         // nullptr, or [B, rank, cap_t] D: the latent once more with the positions innermost (the second
  int cap_t;             // operand of the weights-times-latent product when it runs as a plain matrix product)
  void *qa;              // [M, heads, rank + rot] D: the rotated query part lands in columns rank..; columns 0..rank-1 are
                         // filled afterwards by the product of the unrotated query with the key expansion
  int B, S, heads, dim, rot, rank, cap, pos0;
  float eps;
};
int latent_prep(cudaStream_t, int dtype, const LatentPrep &, uint64_t *launches);

// softmax((qa . row_j) * scale over j <= position) weighted sum of the first `rank` columns of the cached rows
struct LatentAttn {
  const void *qa;        // [M, heads, rank + rot] D
  const void *cache;     // [B, cap, rank + rot] D
  void *lat;             // [M, heads, rank] D
  int B, S, heads, rank, rot, cap, pos0;
  float scale;
  // steps of a few rows: the keys of a (row, head) are split over nsplit CTAs whose partial (max, sum, weighted latent)
  // land in part [M * heads, nsplit, rank + 2] fp32 and are merged by a second kernel; nsplit <= 1: one warp per (row, head)
  float *part = nullptr;
  int nsplit = 0;
};
int latent_attention(cudaStream_t, int dtype, const LatentAttn &, uint64_t *launches);

// The same attention as matrix products for long portions in 16-bit D: scores [rows, kp] fp32 (rows = (t, head) pairs of `n_tok`
// tokens starting at step offset t0, kp keys padded to the product's tile) -> masked, scaled softmax -> the weights as
// w_hi + w_lo in D, [rows, 2 * kp]: hi in columns [0, kp), lo in [kp, 2 kp), zeros where row t sees no key.
struct LatentSoftmax {
  const float *scores;
  void *w;
  int n_tok, heads, kp, pos_first;   // pos_first: absolute position of the block's first token (it sees keys 0..pos_first)
  float scale;
};
int latent_softmax(cudaStream_t, int dtype, const LatentSoftmax &, uint64_t *launches);

// ---- batched small products: C[z][m, n] = sum_k A[z][m, k] * W[z][n, k]  (w_kn: W[z][k, n]) -------------------------------
struct HeadGemm {
  const void *A, *W;
  void *C;               // D
  int M, N, K, Z;
  long a_zs, w_zs, c_zs; // element offsets per z
  int lda, ldw, ldc;
  int w_kn;              // 1: W[z] is stored [K, N] row-major
};
int head_gemm(cudaStream_t, int dtype, const HeadGemm &, uint64_t *launches);

// out[z][c][r] = in[z][r][c] for Z matrices of [rows, cols] in D (weight layouts for the tensor-core products, at load)
int transpose_batched(cudaStream_t, int dtype, const void *in, void *out, int Z, int rows, int cols, uint64_t *launches);

// ---- gated linear recurrence -----------------------------------------------------------------------------------------
//   S_t = a_t S_{t-1} + b_t k_t v_t^T   (S: [dk, dv] fp32 per batch row and head),   o_t = S_t^T q_t + skip_h v_t
// fixed decay:      a_t = decay[h], b_t = kscale           (dt == nullptr)
// state space:      d = softplus(dt[m, h] + dt_bias[h]),  a_t = exp(-exp(a_log[h]) d),  b_t = d
// q and k of head h are read at column (h / group_div) * dk of their rows; with a rotation table the first rope_dims
// entries of q and k are rotated in fp32 on the way in.  The state is read unless pos0 == 0 and written back at the end.
struct Recurrence {
  const void *q, *k, *v; // D
  int ldq, ldk, ldv;
  int group_div;
  const void *dt;        // D [M, lddt] or nullptr
  int lddt;
  const void *dt_bias, *a_log, *skip;  // D [heads]; skip may be nullptr
  const float *decay;    // [heads] fp32
  float kscale;
  const float *cos_t, *sin_t;
  int rope_dims;
  float *state;          // [B, heads, dk, dv]
  float *o;              // [M, heads * dv] fp32
  int B, S, heads, dk, dv, pos0;
  // per-token factors computed elsewhere: a_t = a_tok[m, h], b_t = b_tok[m, h] (fp32 [M, heads]); they override decay / dt
  const float *a_tok = nullptr, *b_tok = nullptr;
};
int recurrence(cudaStream_t, int dtype, const Recurrence &, uint64_t *launches);

// ---- short causal convolution per channel + silu -----------------------------------------------------------------------
struct ShortConv {
  const void *in;        // [M, ld] D, channels from column col0
  int ld, col0;
  const void *w, *bias;  // [channels, taps] (last tap = current token), [channels] D (bias may be nullptr)
  void *hist;            // [B, taps - 1, channels] D: the inputs before the step; updated to the step's last ones
  void *out;             // [M, channels] D
  int B, S, channels, taps, pos0;
};
int short_conv(cudaStream_t, int dtype, const ShortConv &, uint64_t *launches);

// ---- unit norm over equal parts of a row, with a gate before or after ------------------------------------------------
//   val = o * (gate_first ? silu(gate) : 1);  out = val / rms(val over its part) * (w ? w : 1) * (gate_first ? 1 : silu(gate))
struct GateNorm {
  const float *o;        // [M, n] fp32
  const void *gate;      // [M, ldg] D from column 0
  int ldg;
  const void *w;         // [n] D or nullptr
  void *out;             // [M, n] D
  int M, n, parts, gate_first;
  float eps;
  int gate_sigmoid = 0;            // 1: the gate is sigmoid(gate) instead of silu(gate)
  int w_period = 0;                // > 0: w has w_period entries and repeats (one gain vector shared by every part)
  const float *row_div = nullptr;  // [M, parts] fp32: o of a part is divided by its entry before anything else
};
int gate_norm(cudaStream_t, int dtype, const GateNorm &, uint64_t *launches);

// ---- routed feed-forward ---------------------------------------------------------------------------------------------
// Router: z = Wr h (fp32, a matrix product done by the caller), s = softmax(z); the `top` largest s + correction are chosen; weights = s / (sum of chosen + 1e-20)
// * scale.  Experts [0, experts) are gated feed-forwards, [experts, experts + identity) return their input.
struct MoePlan {
  const float *logits;   // [M, ld] fp32: router logits in columns [0, experts + identity); with has_shared_gate the logit of the
  int ld;                // shared expert's gate in the next column (sigmoid of it -> sgate[m])
  const void *correction;// [experts + identity] D
  int has_shared_gate;
  int M, W, experts, identity, top;
  float scale;
  int *ids;              // [M, top]
  float *wts;            // [M, top]
  float *sgate;          // [M]
  // grouping of the (token, slot) pairs by expert: every expert's pairs start on a multiple of `tile` sorted rows
  int tile;
  int *counts;           // [experts + 1] scratch
  int *perm;             // [max_tiles * tile]: sorted row -> m * top + slot, or -1 (padding)
  int *pos_of;           // [M * top]: m * top + slot -> sorted row (pairs of identity experts: untouched)
  int *tile_expert;      // [max_tiles]: the expert of a block of `tile` sorted rows, or -1 (unused block)
  int max_tiles;
  // 1: `correction` is a bias of the logits (z = Wr h + correction); the `top` largest z are chosen and their weights are the
  // softmax over the chosen z alone (times scale)
  int logit_bias = 0;
};
int moe_route(cudaStream_t, int dtype, const MoePlan &, uint64_t *launches);

// sorted[r] = h[perm[r] / top] (zeros for padding rows): the operand of a grouped product on the tensor cores
int moe_gather(cudaStream_t, int dtype, const void *h, const int *perm, void *sorted, int rows, int W, int top, uint64_t *launches);

// CUDA-core experts for every shape and D = float: act = f(Wg h) * (Wu h), then y[sorted row] = Wd act
struct MoeExperts {
  const void *h;         // [M, W] D
  const void *wgu;       // [experts, 2 * ff, W] D: row 2i = gate_i, row 2i + 1 = up_i
  const void *wd;        // [experts, W, ff] D
  void *act;             // [max_tiles * tile, ff] D scratch
  float *y;              // [max_tiles * tile, W] fp32: expert outputs in sorted order, not yet weighted
  int M, W, ff, top, act_kind;
  const int *perm, *tile_expert;
  int tile, max_tiles;
  float limit = 0.f;     // act_kind 2 (the clamped form): its limit
};
int moe_experts(cudaStream_t, int dtype, const MoeExperts &, uint64_t *launches);

// x_out[m] = x[m] + sum over slots of wts * (expert: y[pos_of[m * top + slot]]; identity: h[m]), slots in order
// (x == nullptr: the sum alone)
struct MoeCombine {
  const float *x;
  float *x_out;
  const void *h;         // [M, W] D
  const float *y, *wts;
  const int *ids, *pos_of;
  int M, W, top, experts;
};
int moe_combine(cudaStream_t, int dtype, const MoeCombine &, uint64_t *launches);

// ---- RMS norm of rows of the fp32 stream, gain = w + w_add --------------------------------------------------------------
struct RmsRows {
  const float *x;        // [M, n] fp32
  const void *w;         // [n] D
  float w_add;
  float *out32;          // one of the two outputs: [M, n] fp32 ...
  void *outD;            // ... or [M, n] D
  int M, n;
  float eps;
};
int rms_rows(cudaStream_t, int dtype, const RmsRows &, uint64_t *launches);

// ---- h + conv(h): causal convolution over time per channel of an fp32 activation, no bias, no activation -----------------
struct CanonConv {
  const float *h;        // [M, n] fp32
  const void *w;         // [n, taps] D, last tap = the current token
  float *hist;           // [B, taps - 1, n] fp32: the inputs before the step; updated to the step's last ones
  void *out;             // [M, n] D
  int B, S, n, taps, pos0;
};
int canon_conv(cudaStream_t, int dtype, const CanonConv &, uint64_t *launches);

// ---- sublayer output -> residual stream -----------------------------------------------------------------------------------
//   one branch:   y = a + a_bias
//   two branches: y = ( rms(a + a_bias) * wa + rms(b + b_bias) * wb ) / 2        (rms over the row, plain gains)
//   x_out = x + (post ? rms(y) * (post + post_add) : y)
struct BranchMerge {
  const float *a, *b;    // [M, n] fp32; b may be nullptr
  const void *a_bias, *b_bias, *wa, *wb, *post;  // [n] D, nullable (wa / wb: required with two branches)
  float post_add;
  const float *x;
  float *x_out;          // may alias x
  int M, n;
  float eps;
};
int branch_merge(cudaStream_t, int dtype, const BranchMerge &, uint64_t *launches);

// ---- gated delta rule -----------------------------------------------------------------------------------------------------
// Prep: q and k of every key head become unit vectors (x / sqrt(sum x^2 + 1e-6); q also times qscale) in fp32, and per head
// beta = sigmoid(braw), g = exp(-exp(a_log[h]) * softplus(araw + dt_bias[h])).
struct DeltaPrep {
  const void *q, *k;     // [M, ld] D (after convolution and silu), kv_heads * dk entries each
  int ld;
  const void *braw, *araw;  // [M, ldg] D, heads entries each
  int ldg;
  const void *a_log, *dt_bias;  // [heads] D
  float *qn, *kn;        // [M, kv_heads * dk] fp32
  float *beta, *g;       // [M, heads] fp32
  int M, heads, kv_heads, dk;
  float qscale;
};
int delta_prep(cudaStream_t, int dtype, const DeltaPrep &, uint64_t *launches);
// S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q     (S: [dk, dv] fp32 per batch row and head)
struct DeltaRule {
  const float *qn, *kn;  // [M, kv_heads * dk] fp32
  const void *v;         // [M, ldv] D, heads * dv entries
  int ldv;
  const float *beta, *g; // [M, heads]
  float *state;          // [B, heads, dk, dv]; read unless pos0 == 0, written back at the end
  float *o;              // [M, heads * dv] fp32
  int B, S, heads, kv_heads, dk, dv, pos0;
};
int delta_rule(cudaStream_t, int dtype, const DeltaRule &, uint64_t *launches);

// ---- exponential gates of a matrix memory -----------------------------------------------------------------------------------
// Per (batch row, head), in token order: li = cap tanh((iraw + i_b) / cap), lf = logsigmoid(cap tanh((fraw + f_b) / cap)),
// m' = max(lf + m, li), a = exp(lf + m - m'), b = exp(li - m'), n <- a n + b k, div = (max(|qscale n . q|, exp(-m')) + 1e-6) / qscale.
// a and b drive `recurrence` (S <- a S + b k v^T, o = S^T q); o / div is the read-out.  aux = [n (dk) | m] per (batch row, head).
struct GatePrep {
  const void *q, *k;     // [M, ld] D, heads * dk entries each
  int ld;
  const void *iraw, *fraw;  // [M, ldg] D, heads entries each
  int ldg;
  const void *i_b, *f_b; // [heads] D
  float *aux;            // [B, heads, dk + 1] fp32; read unless pos0 == 0
  float *a, *b, *div;    // [M, heads] fp32
  int B, S, heads, dk, pos0;
  float cap, qscale;
};
int gate_prep(cudaStream_t, int dtype, const GatePrep &, uint64_t *launches);

// ---- softmax attention whose heads' weights are mixed after the softmax ----------------------------------------------------
//   s_g(i, j) = (q_g(i) . k_c(g)(j)) * scale + bias[i - j, g]     for j <= i, c(g) = g / (heads / kv_heads)
//   w_g = softmax_j s_g;   w'_h = sum_g talk[h, g] w_g   (talk == nullptr: w' = w);   o_h(i) = sum_j w'_h(i, j) v_c(h)(j)
//   out = o * sigmoid(gate)  (gate == nullptr: o)
struct TalkAttn {
  const void *q;         // [M, ldq] D, heads * dim entries
  int ldq;
  const void *kc, *vc;   // [B, kv_heads, cap, dim], [B, kv_heads, cap, vdim] D; positions 0 .. pos0 + S - 1 are valid
  const void *gate;      // [M, ldg] D, heads * vdim entries, or nullptr
  int ldg;
  const float *bias;     // [bias_len, heads] fp32 by distance (distances >= bias_len read the last row), or nullptr
  int bias_len;
  const void *talk;      // [heads, heads] D or nullptr
  void *out;             // [M, heads * vdim] D
  int B, S, heads, kv_heads, dim, vdim, cap, pos0;
  float scale;
  // steps of a few rows over many keys: the keys are split over nsplit CTAs per row; part holds
  // [M, nsplit, heads, 2] running (max, sum) and then [M, nsplit, heads * vdim] partial outputs (fp32)
  float *part = nullptr;
  int nsplit = 0;
};
int talk_attention(cudaStream_t, int dtype, const TalkAttn &, uint64_t *launches);
// The same attention as matrix products for long portions in 16-bit D.  Rows are (head, token) pairs of a block of n_tok tokens
// of one batch row, row = head * n_tok + token, so that the rows of a key head's query heads are contiguous:
//   rows_by_head   q [n_tok, ld] (heads * dim entries from column 0) -> [heads * n_tok, dim]
//   (product)      scores [heads * n_tok, kp] fp32 = q rows . keys^T, per key head, kp = the visible keys padded to the tile
//   talk_softmax   scale, distance bias, causal mask, softmax per row; then the heads' weights of a token are mixed and
//                  leave as w_hi + w_lo in D, [heads * n_tok, 2 * kp]: hi in columns [0, kp), lo in [kp, 2 kp), zeros where
//                  the token sees no key
//   (product)      o [heads * n_tok, vdim] = [w_hi | w_lo] . values (the cache keeps the values once more, positions innermost)
//   rows_to_tokens out[token, head * vdim + e] = o[head * n_tok + token, e] * sigmoid(gate[token, head * vdim + e])
struct TalkSoftmax {
  const float *scores;
  void *w;
  float *stats;          // [heads * n_tok, 2] scratch: row maximum and sum
  const float *bias;     // as TalkAttn
  int bias_len;
  const void *talk;      // [heads, heads] D or nullptr
  int n_tok, heads, kp, pos_first;   // pos_first: absolute position of the block's first token
  float scale;
};
int talk_softmax(cudaStream_t, int dtype, const TalkSoftmax &, uint64_t *launches);
int rows_by_head(cudaStream_t, int dtype, const void *src, int ld, void *dst, int n_tok, int heads, int dim, uint64_t *launches);
int rows_to_tokens(cudaStream_t, int dtype, const void *o, const void *gate, int ldg, void *out, int ldo, int n_tok, int heads, int vdim,
                   uint64_t *launches);
// vt[b, g, e, pos0 + t] = src[(b, t), col0 + g * vdim + e]: the values of a step appended with the positions innermost
int values_transposed_append(cudaStream_t, int dtype, const void *src, int ld, int col0, void *vt, int B, int S, int kv_heads, int vdim, int cap_t,
                             int pos0, uint64_t *launches);

// bias[d, h] = rel[bucket[d], h] for d < len (bucket: device ints): the per-distance form TalkAttn reads
int distance_bias_table(cudaStream_t, int dtype, const void *rel, const int *bucket, float *bias, int len, int heads, uint64_t *launches);

// ---- x[t] = E[id] * scale + bigram[(prev * mul_prev + id * mul_cur) mod buckets  |  buckets for a first token] + pos[p] ------
struct EmbedTables {
  const void *E;         // [vocab, W] D
  const uint32_t *ids;   // [B * S] then [B] previous tokens of every batch row's first token (ignored when pos0 == 0)
  const void *bigram;    // [buckets + 1, W] D or nullptr
  const void *pos;       // [positions, W] D or nullptr
  float *x;              // [B * S, W] fp32
  int B, S, W, vocab, buckets, mul_prev, mul_cur, pos0;
  float scale;           // 0 = none
};
int embed_tables(cudaStream_t, int dtype, const EmbedTables &, uint64_t *launches);

// ---- x[m] += (x0 ? x0[m] : 0) + vec   (fp32 stream; vec [W] in D) --------------------------------------------------------
int stream_inject(cudaStream_t, int dtype, float *x, const float *x0, const void *vec, int M, int W, uint64_t *launches);

// ---- element-wise squashing norm: out = tanh(alpha * y) * w + b  (no statistics of the row) ---------------------------------
// Output row i reads input row rows[i] (rows != nullptr) or i * row_mul + row_add.  With x the result is added to it:
// out32 = x + norm(y) (the sublayer's way back into the residual stream; out32 may alias x).
struct TanhNorm {
  const float *y;        // [*, n] fp32
  const int *rows;
  int row_mul, row_add;
  const void *w, *b;     // [n] D
  float alpha;
  const float *x;        // [M, n] fp32 or nullptr
  float *out32;          // one of the two outputs: [M, n] fp32 ...
  void *outD;            // ... or [M, n] D
  int M, n;
};
int tanh_norm(cudaStream_t, int dtype, const TanhNorm &, uint64_t *launches);

// ---- RMS norm with a plain gain over a column range of rows in D (a low-rank latent) ------------------------------------------
// Row m = (b, t) of a step of S tokens lands in output row b * out_rows + out_row0 + t: a scratch buffer (out_rows = S,
// out_row0 = 0) or a cache of `cap` positions per batch row (out_rows = cap, out_row0 = the step's first position).
struct RmsCols {
  const void *in;        // [M, ld] D, n entries from column col
  int ld, col;
  const void *w;         // [n] D
  void *out;             // [*, ldo] D
  int ldo, out_rows, out_row0;
  int M, S, n;
  float eps;
};
int rms_cols(cudaStream_t, int dtype, const RmsCols &, uint64_t *launches);

// ---- queries and keys of a step: rotation of the leading entries of every head, unit RMS per head, keys and values appended ----
// q_h <- rot(q_h), k_g <- rot(k_g) on the first rope_dims entries (pairs i, i + rope_dims / 2; table row = position), then with
// unit_norm x / sqrt(mean(x^2) + eps) over the head; q leaves in D, k and v join the caches at positions pos0 ..
struct QkPrep {
  const void *proj;      // [M, ld] D
  int ld, q_col, k_col, v_col;
  const float *cos_t, *sin_t;   // [positions, rope_dims / 2] or nullptr
  int rope_dims, unit_norm;
  float eps;
  void *q_out;           // [M, heads * dim] D
  void *kc, *vc;         // [B, kv_heads, cap, dim], [B, kv_heads, cap, vdim] D
  int B, S, heads, kv_heads, dim, vdim, cap, pos0;
};
int qk_prep(cudaStream_t, int dtype, const QkPrep &, uint64_t *launches);

// ---- softmax attention over cached keys and values with a sliding window, kept first tokens and a sink -----------------------
// Row i (absolute position) of head h sees key j of key head h / (heads / kv_heads) when j <= i and (window == 0 or i - j < window
// or j < keep_first).  s = (q . k_j) * scale; w_j = exp(s_j) / (sum over visible exp(s) + (sink ? exp(sink[h]) : 0)); the sink has
// no value.  out_h = (sum_j w_j v_j) * sigmoid(gate) with one gate per entry (gate_per_head 0: column h * vdim + e) or per head
// (gate_per_head 1: column h).  Keys and values may be the same rows (a shared latent: kv_heads 1, vc == kc, vdim == dim).
struct WindowAttn {
  const void *q;         // [M, ldq] D, head h at column h * dim
  int ldq;
  const void *kc, *vc;   // [B, kv_heads, cap, dim], [B, kv_heads, cap, vdim] D
  const void *gate;      // [M, ldg] D or nullptr
  int ldg, gate_per_head;
  const void *sink;      // [heads] D or nullptr
  void *out;             // [M, ldo] D, head h at column h * vdim
  int ldo;
  int B, S, heads, kv_heads, dim, vdim, cap, pos0, window, keep_first;
  float scale;
  // steps of a few rows over many keys: the visible keys of a (row, head) are split over nsplit CTAs whose partial (max, sum,
  // weighted values) land in part [M * heads, nsplit, vdim + 2] fp32 and are merged by a second kernel
  float *part = nullptr;
  int nsplit = 0;
};
int window_attention(cudaStream_t, int dtype, const WindowAttn &, uint64_t *launches);
// The tiled form for portions in 16-bit D (tensor-core products, a CTA per 64 rows of a head): true when the shapes fit it.
bool window_attention_tiled_ok(int dtype, const WindowAttn &);
int window_attention_tiled(cudaStream_t, int dtype, const WindowAttn &, uint64_t *launches);

// ---- per-layer token input: x += rms(P (gelu_tanh(G x) * e)) * w,  e = table[id, col .. col + dim) ----------------------------
// The two products run on the GEMMs of the caller; these are the steps around them: the stream's rows rounded to D (the first
// product's operand in 16-bit D), and g <- gelu_tanh(g) * e in place on the first product's result.
int rows_to_d(cudaStream_t, int dtype, const float *x, void *out, size_t n, uint64_t *launches);
struct SideGate {
  void *g;               // [M, ld] D, in place
  int ld;
  const uint32_t *ids;   // [M]
  const void *table;     // [vocab, table_ld] D
  int table_ld, col;
  int M, dim;
};
int side_gate(cudaStream_t, int dtype, const SideGate &, uint64_t *launches);

// ---- out[m] = [x[m] | x0[m]] in D  (the operand of a projection of the stream and the embedding output back into the stream) --
int concat_rows(cudaStream_t, int dtype, const float *x, const float *x0, void *out, int M, int W, uint64_t *launches);

}  // namespace mx
}  // namespace cake
