/*
 * cake_b200.h — C ABI of libcake_b200.so: the B200-native (sm_100a) implementation of cake's
 * sharded transformer-block forward path.
 *
 * This is the drop-in boundary.  A Rust `B200Transformer: Forwarder` (see INTEGRATION.md and
 * rust/b200_transformer.rs) binds exactly these entry points; nothing here mentions torch or candle
 * types — only opaque handles, plain pointers and sizes.  Conventions follow the reference's two
 * existing FFI surfaces (cake-core/src/backends/rocm/ffi.rs:12-51 function table with int status
 * returns; cake-mobile's cake_mobile_c.h explicit free functions):
 *   - every function returns CAKE_B200_OK (0) or a negative CAKE_B200_E*; the message of the last
 *     failure on the calling thread is available from cake_b200_last_error();
 *   - all handles are thread-compatible: any thread may call (the device is bound inside every call, as
 *     worker.rs:412-418 has to), but calls on ONE ctx share its stream and scratch buffers, so concurrent callers
 *     must serialise them (cake_worker / wire.py hold one lock per ctx); a cake_b200_block is immutable after load and
 *     may be shared by several caches/sessions (worker.rs:60-75 shares blocks across connections, each with its own
 *     Cache); a cake_b200_cache belongs to one session; null handles are reported as CAKE_B200_EINVAL, never
 *     dereferenced;
 *   - "_dev" pointers are device memory on the ctx's GPU, everything is enqueued on the ctx's
 *     stream and is asynchronous unless the name ends in _host or the doc says it synchronises.
 *
 * Reference interface each entry replaces (paths relative to /root/reference/cake-core/src):
 *   cake_b200_ctx_create      Context::from_args device/dtype/config part        cake/mod.rs:114-392
 *   cake_b200_block_load      Forwarder::load -> Transformer::load               cake/mod.rs:513-515, models/common/transformer.rs:79-101,
 *                             (qkv / gate_up fusion done here)                   attention.rs:76-149, mlp.rs:34-59
 *   cake_b200_cache_create    Cache::new / Cache::as_new                         models/common/cache.rs:31-114,241-245
 *   cake_b200_cache_clear     Cache::clear / Message::Goodbye handling           cache.rs:247-253, sharding/worker.rs:364-371
 *   cake_b200_forward_batch   Forwarder::forward / forward_mut / forward_batch   cake/mod.rs:517-543, transformer.rs:103-135
 *   cake_b200_head_load       TextModelBase::load embed/ln_f/lm_head             models/common/text_model.rs:159-193
 *   cake_b200_embed           backend.embedding (index_select)                   text_model.rs:271, backends/mod.rs:513-528
 *   cake_b200_logits          ln_f -> last position -> lm_head (-> ArgMax)       text_model.rs:336-352,102-118
 *   cake_b200_comm_* / send / recv   Client::forward_batch <-> Worker loop tensor hand-off,
 *                             replaced on this path by NCCL p2p over NVLink      sharding/client.rs:79-115,165-174, worker.rs:358-575
 *   cake_b200_decode_*        the per-token hot loop                              sharding/master.rs:131-155, text_model.rs:397-495
 */
#ifndef CAKE_B200_H
#define CAKE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CAKE_B200_OK 0
#define CAKE_B200_EINVAL (-1)  /* bad argument / unsupported configuration */
#define CAKE_B200_ECUDA (-2)   /* CUDA runtime error */
#define CAKE_B200_ENCCL (-3)   /* NCCL error or libnccl not loadable */
#define CAKE_B200_ESTATE (-4)  /* call sequence error (e.g. index_pos != cache length) */
#define CAKE_B200_ENOMEM (-5)

/* model dtype D (cake/mod.rs:75 --dtype): weights, activations and KV cache are stored in D */
#define CAKE_B200_BF16 0
#define CAKE_B200_F16 1
#define CAKE_B200_F32 2 /* layer-list models only (cake_b200_config.layer_list): weights, activations and cache in true fp32 */

typedef struct cake_b200_ctx cake_b200_ctx;     /* per (process, device): stream, workspaces, graphs, NCCL comm, head weights */
typedef struct cake_b200_block cake_b200_block; /* immutable weights of one transformer layer */
typedef struct cake_b200_cache cake_b200_cache; /* KV cache of one session (== reference Cache); RoPE tables live in the ctx */

/* models/common/config.rs:87-150, the fields the dense Llama-family block reads */
typedef struct cake_b200_config {
  int hidden, inter, n_heads, n_kv_heads, head_dim, n_layers, vocab, max_seq;
  float rms_eps, rope_theta, partial_rotary;
  int qkv_bias, qk_norm, tie_embeddings;
  int rope_llama3; /* cache.rs:49-80 */
  float rope_factor, rope_low, rope_high;
  int rope_orig_max;
  int dtype; /* CAKE_B200_BF16 | CAKE_B200_F16 */
  int sliding_window; /* config.rs:121 + cache.rs:173-205: attention sees the last `sliding_window` positions (0 = full
                         context).  The cache stays append-only in place; a call at index_pos P with s tokens attends from
                         position max(0, P + s - window) when P > 0 and over everything when P == 0 — exactly what the
                         reference's "cat, then keep the last `window`" leaves visible (first call stores everything,
                         test_cache.rs:99-124). */
  int use_gelu_mlp;   /* mlp.rs:25-26: gelu_tanh(gate) * up instead of silu(gate) * up */
  float embed_scale;  /* text_model.rs:274-276: x = embedding * scale (0 = none) */
  int pre_reshape_qk_norm; /* config.rs:116, attention.rs:176-192 (OLMo2): QK-norm over the whole q / k projection (weights
                              [n_heads*head_dim] / [n_kv_heads*head_dim]) before the head reshape, instead of per head */
  /* ---- layer-list models: the checkpoint's config lists its layers one by one, each with its own geometry ----
   * layer_list = 1: only hidden, n_layers, vocab, max_seq, rms_eps and dtype above are read; every other size comes with
   * the layer (cake_b200_block_load_spec).  The residual stream of such a model is FP32: x_dev / y_dev of
   * cake_b200_forward_batch and the output of cake_b200_embed are float, norms and the residual sum are computed in
   * fp32, and only the operands of the matrix products are in D. */
  int layer_list;
  float logit_softcap;   /* logits <- cap * tanh(logits / cap) after the head (0 = none) */
  int scalar_final_norm; /* the final norm's gain is ONE number (ln_f points to a single element) instead of [hidden] */
} cake_b200_config;

const char *cake_b200_last_error(void); /* thread-local; valid until the next call on this thread */
const char *cake_b200_version(void);

/* ---- context ---------------------------------------------------------------------------------- */
int cake_b200_ctx_create(int device, const cake_b200_config *cfg, cake_b200_ctx **out);
void cake_b200_ctx_destroy(cake_b200_ctx *);
int cake_b200_sync(cake_b200_ctx *);              /* cudaStreamSynchronize(ctx stream) */
void *cake_b200_stream(cake_b200_ctx *);          /* the cudaStream_t everything is enqueued on */
int cake_b200_launch_count(cake_b200_ctx *, uint64_t *kernels); /* kernels of this library launched so far (graph replays included) */

/* Device buffers for hosts that have no allocator of their own (the C++ host, tests); synchronous. */
int cake_b200_dev_alloc(cake_b200_ctx *, size_t bytes, void **out);
int cake_b200_dev_free(cake_b200_ctx *, void *p);

/* ---- blocks ----------------------------------------------------------------------------------- */
/* Pointers are HF-layout [out,in] row-major tensors in dtype D, in host OR device memory (copied
 * with cudaMemcpyDefault).  bias / norm pointers may be NULL when the config does not use them.
 * Fuses q,k,v -> Wqkv and gate,up -> Wgu (row-interleaved) into the device layout. */
int cake_b200_block_load(cake_b200_ctx *, int layer_idx, const void *q, const void *k, const void *v, const void *o,
                         const void *gate, const void *up, const void *down, const void *ln1, const void *ln2,
                         const void *q_bias, const void *k_bias, const void *v_bias, const void *q_norm,
                         const void *k_norm, cake_b200_block **out);
void cake_b200_block_free(cake_b200_block *);
int cake_b200_block_layer(const cake_b200_block *); /* global layer index given at load */

/* The sibling block structures — models/olmo2/block.rs:62-90, models/gemma3/block.rs:60-135, models/exaone4/block.rs:50-110 —
 * are the same attention and MLP with a different norm placement and a per-layer attention mode
 * (CausalSelfAttention::load_custom(vb, cfg, use_qk_norm, sliding_window, use_rope), attention.rs:76-149):
 *   - cake_b200_block_load accepts ln1 == NULL and/or ln2 == NULL: no pre-attention / pre-MLP norm (OLMo2);
 *   - post_attention_norm / post_feedforward_norm, when non-NULL ([hidden], D, host or device): RmsNorm of the attention /
 *     MLP output BEFORE the residual add (OLMo2, Gemma3);
 *   - sliding_window: -1 = the config's, 0 = none (a global layer), > 0 = this layer's window (cache.rs:173-205);
 *   - use_rope: 0 = q and k are not rotated on this layer (EXAONE4 global layers, Gemma3 local layers; attention.rs:242-253).
 * Part of loading: call it right after cake_b200_block_load, before the block is used.  A block with any of these set
 * runs its single-token steps through the batched path as well (cake_b200_forward_batch works for every shape);
 * cake_b200_decode_build refuses such blocks with CAKE_B200_EINVAL — hosts step them with cake_b200_forward_batch. */
typedef struct cake_b200_block_variant {
  int sliding_window;
  int use_rope;
  const void *post_attention_norm;
  const void *post_feedforward_norm;
} cake_b200_block_variant;
int cake_b200_block_set_variant(cake_b200_block *, const cake_b200_block_variant *);

/* ---- layer-list blocks ---------------------------------------------------------------------------
 * One layer of a model with cake_b200_config.layer_list: a PARALLEL block
 *     h = norm(x);   x <- x + ( mixer(shift(h)) + ff(h) )
 * whose mixer is grouped-query attention with the switches below.  Every constant is a parameter so that other
 * layer lists can combine them differently; a combination that is not built is refused with CAKE_B200_EINVAL.
 *   norm         RMS norm in fp32, x / sqrt(mean(x^2) + eps) * g, with g one number (scalar_norm) or a [hidden] vector
 *   token shift  the mixer reads h + (h_prev - h) * shift[hidden] where h_prev is the previous position's h (zeros at
 *                position 0); the last h of a call is kept per layer in the cache so that a prompt may be cut anywhere
 *   scores       s = (q . k) * scale;  softcap > 0: s <- softcap * tanh(s / softcap);  distance bias (r1, r2 non-NULL,
 *                one number per query head): s <- s - r1[h] * ln(1 + r2[h] * (i - j));  window > 0: row i attends to
 *                the keys j with i - window < j <= i (0 = every j <= i);  a plain softmax over the keys that row i sees, all in fp32
 *   values       values_are_keys: there is no V projection and no V cache; the output is the p-weighted sum of the keys
 *   head gate    gate non-NULL ([heads, hidden]): the output of head h is scaled by sigmoid(gate_h . shift(h))
 *   ff           ff > 0: down( act(gate_proj h) * (up h) ), act 0 = silu, 1 = tanh-gelu; ff == 0: no feed-forward
 * Weights are [out, in] row-major in D (host or device memory), q [heads*head_dim, hidden], k [kv_heads*head_dim, hidden],
 * o [hidden, heads*head_dim]. */
typedef struct cake_b200_layer_spec {
  int heads, kv_heads, head_dim;
  int window;
  float scale, softcap;
  int values_are_keys;
  int ff, act;
  int scalar_norm;
} cake_b200_layer_spec;
typedef struct cake_b200_layer_tensors {
  const void *norm;               /* [1] or [hidden] */
  const void *shift;              /* [hidden] or NULL */
  const void *q, *k, *v, *o;      /* v must be NULL with values_are_keys */
  const void *r1, *r2;            /* [heads] or both NULL */
  const void *gate;               /* [heads, hidden] or NULL */
  const void *ff_gate, *ff_up, *ff_down; /* [ff, hidden] x2, [hidden, ff]; NULL when ff == 0 */
} cake_b200_layer_tensors;
int cake_b200_block_load_spec(cake_b200_ctx *, int layer_idx, const cake_b200_layer_spec *, const cake_b200_layer_tensors *,
                              cake_b200_block **out);

/* ---- mixer-list blocks ----------------------------------------------------------------------------
 * One layer of a model with cake_b200_config.layer_list whose block is SEQUENTIAL and pre-normed,
 *     x <- x + mixer(norm1(x));   x <- x + ff(norm2(x))          (RMS norms with [hidden] gains, fp32)
 * with one of the sequence mixers below and an optional routed feed-forward (the structure switches further down change the
 * block: norms behind the sublayers, gains stored as offsets, an input convolution, a side mixer, a dense feed-forward).  Every size and constant is a parameter; a
 * combination that is not built is refused with CAKE_B200_EINVAL.  Scores, softmax, norms, rotations, recurrent state,
 * decays, the router and the residual sums are fp32; projections, caches and weights are in D.
 *   CAKE_B200_MIX_LATENT     attention whose keys and values are expanded from a cached low-rank latent: per head
 *                            [dim | rot] query entries; dkv h = [kv_rank | rot]: the first part RMS-normed (dkv_norm) is
 *                            the latent c, the second, rotated, is a key part shared by all heads; keys uk c, values uv c;
 *                            score = (q . uk c + q_rot . k_rot) * scale, causal softmax.  The cache holds [c | k_rot] only:
 *                            the query is taken through uk and the weighted latent through uv.
 *   CAKE_B200_MIX_RETENTION  linear attention with a fixed decay per head, S_t = decay_h S_{t-1} + k_t v_t^T,
 *                            o_t = S_t^T q_t; q and k rotated, k scaled by dim^-1/2; o of every head divided by its root
 *                            mean square, times silu(g h), then o.
 *   CAKE_B200_MIX_STATE_SPACE  `in` h = [z | x | B | C | dt] (inner = heads * vdim, groups * state each for B and C, heads);
 *                            x, B, C pass a causal convolution per channel (conv [channels, taps], last tap = the current
 *                            token) + silu; dt <- softplus(dt + dt_bias); S_t = exp(-exp(a_log_h) dt) S_{t-1} + dt B_t x_t^T,
 *                            y_t = S_t^T C_t + d_h x_t (head h reads group h / (heads / groups)); y * silu(z), RMS-normed in
 *                            norm_groups equal parts, times norm, then o.
 * The rotation pairs entry i with i + dims / 2 over the first `dims` entries of a head (the rotated part, for the latent
 * mixer): angle = position * f_i, f_i = base^(-2i/dims); with yarn_factor > 0 the frequency is blended towards f_i / factor
 * by a linear ramp between the pair indices that complete `yarn_fast` and `yarn_slow` turns over `yarn_original` positions,
 * and cos / sin are multiplied by 0.1 ln(factor) + 1.  Tables are computed in double precision at load.
 * Recurrent state (fp32) and the convolution's last taps - 1 inputs live in the cache, per block_idx: a block that is run
 * several times per token (a looped range of layers) is given one block_idx per run.
 * The feed-forward (moe.experts + moe.identity > 0): router logits router h in fp32, s = softmax over all experts; the `top`
 * largest s + correction are chosen; their weights are s / (sum of the chosen s + 1e-20) * scale.  Experts [0, experts) are
 * down(act(gate h) * (up h)); the last `identity` router outputs return h itself.  shared_ff > 0: one more expert of that
 * width runs for every token, times sigmoid(s_sg . h).
 *   CAKE_B200_MIX_DELTA      gated delta rule.  q, k ([kv_heads * dim, hidden]; head h reads q / k head h / (heads / kv_heads)) and
 *                            v ([heads * vdim, hidden]) pass a causal convolution per channel (q_conv / k_conv / v_conv [channels, conv],
 *                            last tap = the current token, no bias) + silu; q and k become unit vectors per head,
 *                            x / sqrt(sum x^2 + 1e-6), q times dim^-1/2; beta = sigmoid(beta h), decay g = exp(-exp(a_log_h)
 *                            softplus(a_proj h + dt_bias_h)) per head; S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q;
 *                            o of every head divided by its root mean square, times norm [vdim], times silu(g h), then o.
 *   CAKE_B200_MIX_TALKING_ATTENTION  grouped-query softmax attention without rotation, causal over every cached key; q / k / v / o
 *                            with biases (q_b, k_b, v_b, o_b); score = (q . k) * scale + rel[bucket(i - j), head], where with
 *                            R = bias_rows, h = R / 2: bucket(n) = n for n < h, else min(R - 1, h + floor(ln(n / h) /
 *                            ln(bias_max / h) * (R - h))); after the softmax the heads' weights are mixed, w_h <- sum_g
 *                            talk[h, g] w_g, and head h applies its mixed weights to the values of its own kv head; the
 *                            concatenated heads are multiplied by sigmoid(g h); then o.
 *   CAKE_B200_MIX_MATRIX_MEMORY  a matrix memory with exponential gates.  q (times dim^-1/2), k [heads * dim, hidden], v
 *                            [heads * vdim, hidden]; log gates per head i = cap tanh((i_proj h + i_b) / cap), f = logsigmoid(cap
 *                            tanh((f_proj h + f_b) / cap)), cap = gate_cap; running maximum m (0 at the start): m' = max(f + m, i);
 *                            S <- exp(f + m - m') S + exp(i - m') k v^T, n likewise with k alone; o = S^T q / (max(|n . q|,
 *                            exp(-m')) + 1e-6); o of every head divided by its root mean square, times norm [heads * vdim], times
 *                            sigmoid(g h), then o.  S, n and m live in the cache in fp32.
 *   CAKE_B200_MIX_SINK_ATTENTION  grouped-query softmax attention with a sliding window that keeps the sequence's first tokens and a
 *                            learned sink.  q / k / v with biases (q_b, k_b, v_b); the first rot.dims entries of every q and k head are
 *                            rotated (pairs i, i + dims / 2; optional frequency blend), then, with qk_unit, every head of q and k is
 *                            divided by its root mean square (eps of the ctx); score = (q . k) * scale; row i sees key j <= i when
 *                            window == 0, i - j < window or j < keep_first; the softmax's denominator also holds exp(sink_h) (sink
 *                            [heads], no key, no value; NULL = none); the concatenated heads are multiplied by sigmoid(g h)
 *                            (g [heads * vdim, hidden]; NULL = none); then o.  K and V rows live in the cache.
 *   CAKE_B200_MIX_LATENT_WINDOW  latent attention without positions: c_q = rms(dq h) * dq_norm ([q_rank]), q = uq c_q ([heads * dim,
 *                            q_rank]); c = rms(dkv h) * dkv_norm ([kv_rank]) is the only cached row; per head k = uk c, v = uv c
 *                            (steps of a few rows in the absorbed form: the query goes through uk, the weighted latent through
 *                            uv; portions with key and value size 128 in 16-bit D expand k and v for the rows the step sees);
 *                            score = (q . k) * scale over the window (as above, keep_first included); head h's output is
 *                            multiplied by sigmoid(g h)_h (g [heads, hidden]; NULL = none); then o.
 * Block structure switches (all 0 / NULL for the plain pre-norm block above):
 *   norm_kind    0: RMS norms; 1: the element-wise squashing norm tanh(alpha x) * w + b for norm1 / post1 / norm2 / post2, alpha =
 *                norm_alpha[0..3] in that order, offsets norm1_b / post1_b / norm2_b / post2_b ([hidden])
 *   side_dim     > 0: after the feed-forward the stream receives a per-layer token input: e = columns [side_col, side_col +
 *                side_dim) of the token's row of the ctx's side table (cake_b200_embed_tables.side), g = gelu_tanh(side_gate x) * e
 *                (side_gate [side_dim, hidden]), y = side_proj g ([hidden, side_dim]), x += y / rms(y) * side_norm ([hidden]).
 *                The ids are those of the step's cake_b200_embed call
 *   With these two, or with the two mixers above, the routed feed-forward (moe) may follow post-norm blocks as well; moe.logit_bias
 *   1: `correction` is added to the router's logits, the `top` largest logits are chosen and weighted by the softmax over the
 *   chosen alone; moe.act 2 is the clamped form with moe.limit (routed experts) / moe.shared_limit (shared expert)
 *   norm_offset  the gains of norm1 / norm2 / post1 / post2 are stored as offsets: gain = stored + norm_offset (computed in fp32)
 *   post1, post2 an RMS norm of the mixer's / feed-forward's output before it is added to the stream
 *   canon_taps   >= 1: the mixer reads h + conv(h), a causal convolution over time per channel of the normed input (canon
 *                [hidden, canon_taps], last tap = the current token, no bias, fp32); its last canon_taps - 1 inputs live in the cache
 *   side         a second mixer that reads the same input: both outputs are RMS-normed over the width with plain gains
 *                (branch_norm of each mixer's tensors) and averaged; the side mixer's spec / tensors use the mixer fields only
 *   dense_ff     > 0: a dense gated feed-forward of that width instead of the routed one (ff_gate, ff_up [dense_ff, hidden],
 *                ff_down [hidden, dense_ff]); dense_act 0 silu(g) u, 1 tanh-gelu(g) u, 2: g' = min(g, dense_limit), u' = clamp(u,
 *                -dense_limit, dense_limit), g' sigmoid(1.702 g') (u' + 1) */
#define CAKE_B200_MIX_LATENT 1
#define CAKE_B200_MIX_RETENTION 2
#define CAKE_B200_MIX_STATE_SPACE 3
#define CAKE_B200_MIX_DELTA 4
#define CAKE_B200_MIX_TALKING_ATTENTION 5
#define CAKE_B200_MIX_MATRIX_MEMORY 6
#define CAKE_B200_MIX_SINK_ATTENTION 7
#define CAKE_B200_MIX_LATENT_WINDOW 8
typedef struct cake_b200_rotary_spec {
  int dims;            /* 0 = no rotation */
  double base;
  double yarn_factor;  /* 0 = plain */
  double yarn_fast, yarn_slow;
  int yarn_original;
} cake_b200_rotary_spec;
typedef struct cake_b200_moe_spec {
  int experts, identity, top;
  float scale;
  int ff, shared_ff;
  int act;             /* 0 silu, 1 tanh-gelu, 2 clamped (limit / shared_limit) */
  float limit, shared_limit;
  int logit_bias;
} cake_b200_moe_spec;
typedef struct cake_b200_mixer_spec {
  int kind;
  int heads, dim, vdim;
  int rot_dim, kv_rank;   /* latent */
  float scale;            /* latent */
  cake_b200_rotary_spec rot;
  const float *decay;     /* retention: [heads], host */
  int state, groups, conv, norm_groups;  /* state space; dim is ignored (state is the key size); conv also: delta */
  cake_b200_moe_spec moe;
  int kv_heads;           /* delta, talking attention (0 = heads) */
  int bias_rows;          /* talking attention: rows of rel (0 = no distance bias) */
  float bias_max;
  float gate_cap;         /* matrix memory */
  float norm_offset;
  int canon_taps;
  int dense_ff, dense_act;
  float dense_limit;
  const struct cake_b200_mixer_spec *side;
  int window, keep_first; /* sink attention, windowed latent attention: 0 = every earlier key */
  int qk_unit;            /* sink attention: unit-RMS q and k heads */
  int q_rank;             /* windowed latent attention */
  int norm_kind;
  float norm_alpha[4];
  int side_dim, side_col;
} cake_b200_mixer_spec;
typedef struct cake_b200_mixer_tensors {
  const void *norm1, *norm2;                 /* [hidden]; norm2 NULL without a feed-forward */
  const void *q, *k, *v, *g, *o;             /* retention: all; latent: q [heads*(dim+rot_dim), hidden] and o */
  const void *dkv, *dkv_norm, *uk, *uv;      /* latent: [kv_rank+rot_dim, hidden], [kv_rank], [heads*dim, kv_rank], [heads*vdim, kv_rank] */
  const void *in, *conv, *conv_b, *dt_bias, *a_log, *d, *norm;  /* state space */
  const void *router, *correction;           /* [experts+identity, hidden], [experts+identity] */
  const void *const *e_gate, *const *e_up, *const *e_down;  /* `experts` pointers each: [ff, hidden] x2, [hidden, ff] */
  const void *s_gate, *s_up, *s_down, *s_sg; /* shared expert; s_sg [hidden] */
  const void *post1, *post2, *canon;         /* [hidden], [hidden], [hidden, canon_taps] */
  const void *q_conv, *k_conv, *v_conv, *beta, *a_proj;  /* delta: [kv_heads*dim, conv] x2, [heads*vdim, conv], [heads, hidden] x2 */
  const void *q_b, *k_b, *v_b, *o_b, *rel, *talk;        /* talking attention: biases, [bias_rows, heads], [heads, heads] */
  const void *i_proj, *i_b, *f_proj, *f_b;   /* matrix memory: [heads, hidden], [heads] each */
  const void *ff_gate, *ff_up, *ff_down;     /* dense feed-forward */
  const void *branch_norm;                   /* [hidden]: with a side mixer, the gain of this mixer's output norm */
  const struct cake_b200_mixer_tensors *side;
  const void *sink;                          /* sink attention: [heads] */
  const void *dq, *dq_norm, *uq;             /* windowed latent attention: [q_rank, hidden], [q_rank], [heads * dim, q_rank] */
  const void *norm1_b, *post1_b, *norm2_b, *post2_b;  /* norm_kind 1: [hidden] each */
  const void *side_gate, *side_proj, *side_norm;      /* side_dim > 0: [side_dim, hidden], [hidden, side_dim], [hidden] */
} cake_b200_mixer_tensors;
int cake_b200_block_load_mixer(cake_b200_ctx *, int layer_idx, const cake_b200_mixer_spec *, const cake_b200_mixer_tensors *,
                               cake_b200_block **out);
/* Between blocks of a looped range: x <- x + (x0 ? x0 : 0) + vec, rows of [hidden] fp32; vec [hidden] in D, host or device
 * memory on the first call with that pointer (it is uploaded once and kept by the ctx under `slot`, 0 <= slot < 64). */
int cake_b200_stream_inject(cake_b200_ctx *, float *x_dev, const float *x0_dev, const void *vec, int slot, int rows);
/* In front of a pass of a looped range: x <- W [x; x0], rows of [hidden] fp32, W [hidden, 2 * hidden] in D (x's half first), host
 * or device memory on the first call with that pointer (uploaded once and kept by the ctx). */
int cake_b200_stream_project(cake_b200_ctx *, float *x_dev, const float *x0_dev, const void *w, int rows);

/* ---- cache ------------------------------------------------------------------------------------ */
int cake_b200_cache_create(cake_b200_ctx *, int batch, int max_seq, cake_b200_cache **out);
int cake_b200_cache_clear(cake_b200_cache *);
void cake_b200_cache_free(cake_b200_cache *);
int cake_b200_cache_len(const cake_b200_cache *, int block_idx); /* tokens stored for that layer, or <0 */
/* Debug / parity access: copies layer `block_idx`'s K or V, positions [0,len), to host as
 * (batch, n_kv, len, head_dim) in dtype D.  Synchronises. */
int cake_b200_cache_read(cake_b200_cache *, int block_idx, int which /*0=K,1=V*/, void *out_host, size_t bytes);
/* Fill positions [0,len) of every layer this process owns with a deterministic pseudo-random pattern
 * (bench only: lets the decode benchmark start at a given context length without a long prefill). */
int cake_b200_cache_fill_synthetic(cake_b200_cache *, const int *block_idx, int n_blocks, int len, uint32_t seed);

/* ---- the block forward ------------------------------------------------------------------------ */
/* == Forwarder::forward_batch over `n_blocks` consecutive local layers (n_blocks == 1 == forward).
 * x_dev, y_dev: (batch, seq, hidden) in D; may alias.  index_pos: absolute position of x[:,0]
 * and it must equal the cache length of each block (CAKE_B200_ESTATE otherwise — the reference
 * only ever calls it that way, text_model.rs:401-412,454). */
int cake_b200_forward_batch(cake_b200_ctx *, cake_b200_block *const *blocks, const int *block_idx, int n_blocks,
                            cake_b200_cache *, const void *x_dev, void *y_dev, int batch, int seq, int index_pos);
/* Same with HOST buffers: H2D copy of x, forward, D2H copy of y, synchronises (the e2e path). */
int cake_b200_forward_batch_host(cake_b200_ctx *, cake_b200_block *const *blocks, const int *block_idx, int n_blocks,
                                 cake_b200_cache *, const void *x_host, void *y_host, int batch, int seq,
                                 int index_pos);

/* ---- head / tail (master role) ---------------------------------------------------------------- */
int cake_b200_head_load(cake_b200_ctx *, const void *embed, const void *ln_f, const void *lm_head /* NULL if tied */);
int cake_b200_embed(cake_b200_ctx *, const uint32_t *ids_host, int batch, int seq, void *x_dev);
/* Embeddings that depend on the place of a token in its sequence (layer-list models, fp32 stream), added to the scaled token
 * embedding:  a hashed pair embedding, row (previous token * mul_prev + token * mul_cur) mod (bigram_rows - 1) of bigram
 * [bigram_rows, hidden], the last row for a sequence's first token;  and a learned vector per position, pos [pos_rows, hidden].
 * Either pointer may be NULL.  final_norm_offset: the final norm's gain is stored as an offset from this number.  Call after
 * cake_b200_head_load.  With tables loaded, the stream starts with cake_b200_embed_at: the cache supplies the previous token
 * of every batch row and checks index_pos against the position the embedding has reached in it. */
typedef struct cake_b200_embed_tables {
  const void *bigram;
  int bigram_rows, mul_prev, mul_cur;
  const void *pos;
  int pos_rows;
  float final_norm_offset;
  const void *side;         /* [vocab, side_cols]: the per-layer token inputs of every layer side by side, or NULL */
  int side_cols;
  int final_norm_kind;      /* 1: the final norm is tanh(final_alpha x) * ln_f + final_bias ([hidden]) */
  float final_alpha;
  const void *final_bias;
} cake_b200_embed_tables;
int cake_b200_head_load_tables(cake_b200_ctx *, const cake_b200_embed_tables *);
int cake_b200_embed_at(cake_b200_ctx *, cake_b200_cache *, const uint32_t *ids_host, int batch, int seq, int index_pos, void *x_dev);
/* ln_f on the last position of each batch row, lm_head, logits (batch, vocab) in D written to
 * logits_dev (nullable); if argmax_host != NULL also computes the greedy token per row
 * (first maximum wins), copies it to argmax_host and synchronises. */
int cake_b200_logits(cake_b200_ctx *, const void *x_dev, int batch, int seq, void *logits_dev, uint32_t *argmax_host);
/* The same for ANY rows of x_dev ((n_rows_total, hidden), row = b * seq + t), in FP32: final norm -> lm_head -> logit
 * soft cap, logits_f32_dev[(i, vocab)] for i < n.  Layer-list models (fp32 residual stream) only.  Asynchronous. */
int cake_b200_logits_rows(cake_b200_ctx *, const void *x_dev, int n_rows_total, const int *rows_host, int n,
                          float *logits_f32_dev);
/* text_model.rs:60-99 repeat penalty on device over logits_dev (vocab) in D, then greedy token. */
int cake_b200_repeat_penalty_argmax(cake_b200_ctx *, void *logits_dev, float penalty, const uint32_t *ctx_tokens_host,
                                    int n_tokens, uint32_t *argmax_host);

/* ---- activation hand-off between shards (NCCL p2p over NVLink, in-stream) ---------------------- */
int cake_b200_comm_unique_id(void *out128); /* ncclGetUniqueId; 128 bytes */
int cake_b200_comm_init(cake_b200_ctx *, const void *unique_id128, int rank, int world);
int cake_b200_send(cake_b200_ctx *, const void *x_dev, size_t bytes, int peer);
int cake_b200_recv(cake_b200_ctx *, void *x_dev, size_t bytes, int peer);

/* Optional, after comm_init: hand-off fused into the decode kernels over NVLink peer memory instead of NCCL kernels.
 * Every rank exports a 64-byte IPC handle of its inbox and imports the handle of rank (r+1) % world; decode_build then
 * makes the last kernel of a shard write the next shard's inbox directly and release it (red.release.sys), and the
 * first kernel of a shard acquire its own inbox.  Without these calls the decode graph uses ncclSend/ncclRecv. */
int cake_b200_ring_export(cake_b200_ctx *, void *handle64);
int cake_b200_ring_import(cake_b200_ctx *, const void *next_rank_handle64);

/* ---- the decode hot loop (master.rs:131-155), one CUDA graph per shard ------------------------- */
/* Builds the per-token step for this rank's contiguous layer range (batch 1, seq 1):
 *   rank 0          : embed(token) -> its blocks -> [send -> ... -> recv from last rank] -> ln_f/lm_head/argmax -> token
 *   ranks 1..world-1: recv -> its blocks -> send to (rank+1) % world
 * Position and token are device-resident, so `n` steps replay back-to-back without host work.
 * world == 1 needs no communicator.  Greedy only (temperature <= 0 and repeat_penalty == 1). */
int cake_b200_decode_build(cake_b200_ctx *, cake_b200_block *const *blocks, const int *block_idx, int n_blocks,
                           cake_b200_cache *, int rank, int world);
/* first_token: token fed at the first step (ignored on ranks > 0); index_pos: its position. */
int cake_b200_decode_begin(cake_b200_ctx *, uint32_t first_token, int index_pos);
int cake_b200_decode_run(cake_b200_ctx *, int n_steps);                    /* async: enqueue n graph replays */
int cake_b200_decode_tokens(cake_b200_ctx *, uint32_t *out_host, int n);   /* last n generated tokens; synchronises (rank 0) */
/* One step driven from the host like TextModelBase::next_token: H2D of the token id, one replay,
 * D2H of the sampled token, synchronise.  (rank 0; other ranks call cake_b200_decode_run(ctx,1).) */
int cake_b200_decode_step_host(cake_b200_ctx *, uint32_t token_in, uint32_t *token_out);
int cake_b200_decode_logits(cake_b200_ctx *, void *logits_host, size_t bytes); /* logits (vocab) of the last step, D; synchronises */

/* ---- sampling on the device (text_model.rs:102-118 create_logits_processor, :429-460) ------------------------------
 * The reference picks a candle_transformers::generation::Sampling from (temperature, top_k, top_p): temperature <= 0
 * -> ArgMax; else (None, None) -> GumbelSoftmax, (k, None) -> TopK, (None, p) -> TopP, (k, p) -> TopKThenTopP ("All" =
 * plain multinomial is what TopK/TopP degrade to for k >= vocab / p outside (0,1)).  Only the 4-byte token leaves the GPU.
 * kind: 0 ArgMax, 1 All, 2 TopK, 3 TopP, 4 TopKThenTopP, 5 GumbelSoftmax.  top_k <= 1024. */
typedef struct cake_b200_sampling {
  int kind, top_k;
  float temperature, top_p;
  uint64_t seed; /* LogitsProcessor::from_sampling(seed, ..): keys a counter-based Philox stream (candle's own RNG stream
                    cannot be reproduced; see csrc/sample.cuh) */
} cake_b200_sampling;
/* next_token's tail in one call: repeat penalty over ctx_tokens_host (text_model.rs:60-99; skipped when penalty == 1 or
 * n_tokens == 0, applied IN PLACE to logits_dev), then one draw.  `step` selects the random numbers of this draw;
 * noise_host (nullable) supplies the uniforms in [0,1) instead — vocab floats for GumbelSoftmax, one float otherwise
 * (how the parity tests pin the arithmetic).  Synchronises. */
int cake_b200_sample(cake_b200_ctx *, void *logits_dev, const cake_b200_sampling *, float repeat_penalty,
                     const uint32_t *ctx_tokens_host, int n_tokens, uint64_t step, const float *noise_host,
                     uint32_t *token_host);
/* Sampler of the graph-captured decode loop (call before cake_b200_decode_build; NULL or kind 0 = greedy, the default):
 * a sampler kernel runs behind the decode kernel of rank 0, reads the logits it left in HBM/L2 and overwrites the greedy
 * token; the draw of step s uses (seed, s).  No repeat penalty inside the graph. */
int cake_b200_decode_set_sampling(cake_b200_ctx *, const cake_b200_sampling *);

/* ---- measurement aid (bench.py roofline leg) ---------------------------------------------------- */
/* Times ONE of the decode kernels of the given blocks in isolation with CUDA events on the ctx stream:
 * `reps` rounds over the blocks, back to back (which: 0 qkv GEMV, 1 o_proj GEMV, 2 gate_up GEMV,
 * 3 down GEMV, 4 attention at the cache's current length).  Different blocks hold distinct weights, so
 * with >= 2 blocks whose matrices exceed L2 no launch is served from cache.  Returns the mean
 * milliseconds per launch.  Synchronises.  Outputs go to scratch buffers; the cache is not advanced. */
int cake_b200_bench_kernel(cake_b200_ctx *, cake_b200_block *const *blocks, const int *block_idx, int n_blocks,
                           cake_b200_cache *, int which, int reps, float *ms_per_launch);

/* Weight upload statistics of this ctx (utils/mod.rs:255-384 is the reference's loader): block_load / head_load stage host
 * tensors through two pinned 64 MB buffers (filled by a few host threads) and copy them with cudaMemcpy(2D)Async on a
 * copy stream straight into the fused qkv / row-interleaved gate_up layouts; compute entry points wait for the uploads
 * issued so far.  bytes = host bytes uploaded, seconds = time spent staging + enqueueing them.  Synchronises the copy
 * stream. */
int cake_b200_load_stats(cake_b200_ctx *, double *bytes, double *seconds);

/* Per-step timeline of this rank's decode kernels for the last `n_steps` steps since cake_b200_decode_begin
 * (n_steps <= 2048): 8 u64 per step = {entry, input acquired, exit, 0} of the layer launch followed by the same for
 * rank 0's head-only launch when sharded (zeros otherwise); %globaltimer nanoseconds of CTA 0.  "input acquired"
 * is when the hidden state of the previous shard arrived (== entry on a single GPU).  Replaces eyeballing the
 * reference's per-hop log lines (worker.rs:505-530 ops/s + read/write stats).  Synchronises. */
int cake_b200_decode_trace(cake_b200_ctx *, uint64_t *out_host, int n_steps);

#ifdef __cplusplus
}
#endif
#endif /* CAKE_B200_H */
