/*
 * xotb200_lm.h — C ABI of libxotb200_lm.so: the layered-model engine of xotorch_b200 (sm_100a).
 *
 * libxotb200.so (xotb200.h) runs Llama-style shards through one persistent kernel.  This library runs decoders that are given as
 * a LIST of layers — each a token mixer and an optional feed-forward between grouped RMS norms — where the mixers differ from
 * layer to layer and keep different per-request state:
 *   XOTB200_LM_MIX_LATENT_ATTN  attention over a compressed (latent) key/value row per token + one rotated key part shared by
 *                               all heads; options: query through a normed latent, rotation layout, sliding window, output gate;
 *                               state = the paged latent cache;
 *   XOTB200_LM_MIX_DELTA_RULE   generalised delta-rule recurrence with per-channel decay and removal rate;
 *                               state = one fp32 matrix per head, request and layer;
 *   XOTB200_LM_MIX_ATTENTION    grouped-query attention over a paged cache of (normed) keys and values; options: projection
 *                               biases, query/key norm (per head or over the whole projection), soft cap, logarithmic distance
 *                               penalty, learned bias per distance bucket, query temperature, softmax sink, sliding window,
 *                               block-local mask, output gate per head or per entry, keys/values borrowed from an earlier layer;
 *   XOTB200_LM_MIX_GATED_DELTA  delta rule with one decay per head behind short causal convolutions;
 *                               state = fp32 matrix per head + the convolutions' last inputs;
 *   XOTB200_LM_MIX_MATRIX_LSTM  matrix memory with exponential input gate, sigmoid forget gate and a running maximum that keeps both
 *                               in range; state = fp32 matrix + normaliser vector + maximum per head;
 *   XOTB200_LM_MIX_MAMBA2       state-space layer with one decay per head, input-dependent step size, short convolution on its
 *                               inputs, gate before a grouped RMS norm; state = fp32 matrix per head + the convolution's last inputs.
 * A layer whose mixer is one of the last four kinds may carry a SECOND, recurrent mixer (par_on: gated delta rule, matrix LSTM or
 * state-space): both read the same input (one product for all their projections) and the layer's mixer output is
 * mix_scale * first + par_scale * second.
 * A layer wraps its sublayers in grouped RMS norms before and after them, or reads the stream itself and closes with a layer norm
 * or an RMS norm, or — pre-norm with one-number weights — reads `streams` copies of the residual stream through hyper-connections
 * and passes every sublayer input through a short causal convolution that is added to it (xotb200_lm_cfg.block); its feed-forward is dense (relu^2 or xIELU) or a mixture of experts (gated silu or relu^2
 * experts, two routing rules, an optional shared expert: xotb200_lm_layer.ff_kind and the fields after it).
 * Every size and constant of a layer is a field of xotb200_lm_layer, so a model family is a table of layers, not code.
 *
 * Serving model: requests live in SLOTS (0 .. max_requests-1).  A step (xotb200_lm_step) takes a packed batch — for each
 * participating slot its next n >= 1 tokens — appends them to the slot's cache / state and returns the logits of the rows asked
 * for.  Prompts, portions of prompts and single decoded tokens are the same call.  The latent cache is PAGED: one pool of pages
 * per attention layer, a page table per slot, pages handed out as a request grows and returned by xotb200_lm_clear_request.
 *
 * Conventions as in xotb200.h: 0 on success, negative XOTB200_E* on failure (message: xotb200_lm_last_error(), thread-local);
 * host pointers are caller-owned; calls on one engine are serialised by the caller.
 */
#ifndef XOTB200_LM_H
#define XOTB200_LM_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef XOTB200_OK
#define XOTB200_OK 0
#define XOTB200_EINVAL (-1)
#define XOTB200_ECUDA (-2)
#define XOTB200_EIO (-3)
#define XOTB200_ESTRICT (-4)
#endif

#define XOTB200_LM_DTYPE_BF16 0 /* weights, GEMM inputs and latent cache in bfloat16; fp32 accumulation, residual, norms, state */
#define XOTB200_LM_DTYPE_F32 2  /* everything in true fp32 (FMA products, no reduced-precision matrix mode)                       */

#define XOTB200_LM_MIX_LATENT_ATTN 0
#define XOTB200_LM_MIX_DELTA_RULE 1
#define XOTB200_LM_MIX_ATTENTION 2   /* grouped-query attention over a paged key/value cache (see xotb200_lm_layer)            */
#define XOTB200_LM_MIX_GATED_DELTA 3 /* delta rule with one decay per head behind short causal convolutions                    */
#define XOTB200_LM_MIX_MATRIX_LSTM 4 /* matrix memory: S <- e^(f + m' - m) S + e^(i - m) k v^T with running maximum m              */
#define XOTB200_LM_MIX_MAMBA2 5      /* state-space layer: S <- e^(-e^A dt) S + dt B x^T, y = S^T C + D x                          */

#define XOTB200_LM_FF_RELU2 0  /* W_down relu(W_up h)^2                                                                         */
#define XOTB200_LM_FF_XIELU 1  /* W_down act(W_up h), act(z) = softplus(p) z^2 + z/2 (z > 0), (1/2 + softplus(q))(e^z - 1 - z) + z/2 (z <= 0);
                                  p, q = the two entries of l<i>.mlp.act                                                         */
#define XOTB200_LM_FF_GELU 3   /* W_down gelu(W_up h), the exact gelu z (1 + erf(z / sqrt 2)) / 2                               */
#define XOTB200_LM_FF_MOE 2    /* mixture of experts; expert form, routing rule and shared expert: expert_act, router_kind, shared_ff */

#define XOTB200_LM_EXPERT_SILU_GATED 0 /* expert = W_down (silu(W_gate h) * W_up h)                                              */
#define XOTB200_LM_EXPERT_RELU2 1      /* expert = W_down relu(W_up h)^2  (no gate matrix)                                       */

#define XOTB200_LM_ROUTER_SOFTMAX_ALL 0 /* scores = softmax over all experts; group-limited top-k; weights = the chosen scores     */
#define XOTB200_LM_ROUTER_TOPK_SOFTMAX 1 /* the `top` largest logits (W_router h + router.b) are chosen; weights = softmax over them */

#define XOTB200_LM_BLOCK_GROUP_RMS 0  /* x += norm1b(mixer(norm1(x))): grouped RMS norms before and after every sublayer          */
#define XOTB200_LM_BLOCK_POST_LN 1    /* x += LN(mixer(x)): the sublayer reads the stream itself, layer norm (weight + bias) on its output */
#define XOTB200_LM_BLOCK_POST_RMS 2   /* x += rms(mixer(x)) * (1 + w): the same with an RMS norm whose weight is stored around zero     */

#define XOTB200_LM_BLOCK_PRE_SCALAR 3  /* x += mult * sublayer(c(rms(x) * g)): pre-norm whose weight is ONE number, c(h) = h + causal
                                         convolution of h over time (canon_taps; 0 = none); with streams > 0 the stream is kept in
                                         `streams` copies mixed by hyper-connections (below); embedding and final norm of the same kind */

#define XOTB200_LM_QKNORM_NONE 0
#define XOTB200_LM_QKNORM_HEAD 1      /* RMS norm of every query / key head, one weight of size dim shared by the heads                 */
#define XOTB200_LM_QKNORM_HEAD_PLAIN 3 /* every query / key head divided by its root mean square, no weight                            */
#define XOTB200_LM_QKNORM_ROW 2       /* ONE RMS norm over the whole query (key) projection, weights of size heads * dim (kv_heads * dim) */

#define XOTB200_LM_ROT_INTERLEAVED 0 /* pairs (2i, 2i+1)        */
#define XOTB200_LM_ROT_HALF 1        /* pairs (i, i + dims / 2) */

typedef struct xotb200_lm_layer {
  int32_t mixer;      /* XOTB200_LM_MIX_*                                                                   */
  int32_t heads;
  int32_t dim;        /* latent attention: unrotated query/key size per head; delta rule: key size per head  */
  int32_t vdim;       /* value size per head (delta rule: = dim)                                              */
  int32_t rot_dim;    /* latent attention: size of the rotated query part / shared key part                   */
  int32_t kv_rank;    /* latent attention: latent size                                                        */
  int32_t q_rank;     /* latent attention: > 0 = queries through a normed latent of this size, 0 = direct     */
  int32_t rot_dims;   /* how many leading entries of the rotated part are turned (<= rot_dim, even)           */
  int32_t rot_layout; /* XOTB200_LM_ROT_*                                                                     */
  int32_t window;     /* > 0: a query at position i sees i - window < j <= i; 0: every j <= i                 */
  int32_t out_gate;   /* attention: 1 = one sigmoid gate per head on the mixer output, 2 = one per output entry (heads * vdim) */
  int32_t low_rank;   /* delta rule: inner size of the decay branch                                           */
  int32_t ff;         /* feed-forward inner size (relu^2 between up and down); 0 = the layer has none         */
  float rot_base;
  float scale;        /* score scale                                                                          */
  /* -- grouped-query attention (MIX_ATTENTION) and gated delta rule (MIX_GATED_DELTA) -------------------------------------
   * MIX_ATTENTION: `heads` query heads of size `dim` share `kv_heads` key/value heads (query head a reads a / (heads / kv_heads)),
   * values of size `vdim`; the cache holds per token [keys after their norm | values].  score = q.k * scale, then
   * softcap * tanh(score / softcap) when softcap > 0, then - r1[a] * ln(1 + r2[a] * (i - j)) when dist_bias, then + rel[bucket(i - j), a]
   * when rel_buckets > 0; visible keys: j <= i, i - j < window when window > 0, floor(i / chunk) == floor(j / chunk) when chunk > 0;
   * softmax, whose denominator also holds exp(sink[a]) when `sink` (a term without key or value).
   * MIX_GATED_DELTA: `kv_heads` query/key heads of size `dim`, `heads` value heads of size `vdim`; q, k, v pass a causal
   * per-channel filter of `conv_taps` taps and silu; q, k unit vectors (q also / sqrt(dim)); per head S <- g S,
   * S += k (beta (v - S^T k))^T, o = S^T q with g = exp(-exp(A_log) softplus(W_a h + dt_bias)), beta = sigmoid(W_b h);
   * o / rms(o) * norm * silu(W_g h).  State: fp32 S [dim, vdim] per head + the last conv_taps - 1 filter inputs. */
  int32_t kv_heads;
  int32_t kv_from;    /* attention: -1 = own keys/values; else the (global) index of the earlier layer whose cache it reads */
  int32_t chunk;      /* attention: > 0 = block-local causal mask with blocks of this many positions          */
  int32_t qk_norm;    /* attention: XOTB200_LM_QKNORM_* (weights q.norm / k.norm)                              */
  int32_t proj_bias;  /* attention: 1 = q, k, v projections have biases (q.b, k.b, v.b)                       */
  int32_t dist_bias;  /* attention: 1 = logarithmic distance penalty with per-head r1, r2                     */
  int32_t conv_taps;  /* gated delta rule: taps of the short convolutions                                     */
  int32_t ff_kind;    /* XOTB200_LM_FF_*  (`ff` = inner size of the dense forms)                              */
  int32_t experts;    /* FF_MOE: number of experts, each of inner size expert_ff                              */
  int32_t expert_ff;
  int32_t top;        /* FF_MOE: experts per token (their weights: router_kind)                                       */
  int32_t groups;     /* FF_MOE: experts form `groups` equal groups of neighbours (<= 1: no groups) ...        */
  int32_t groups_keep;/* ... and only experts of the groups_keep groups with the largest best score can be chosen */
  float softcap;
  /* -- further options of MIX_ATTENTION -------------------------------------------------------------------------------- */
  int32_t out_bias;     /* 1 = the output projection has a bias (o.b)                                            */
  int32_t sink;         /* 1 = one learned logit per query head (sink) joins the softmax denominator            */
  int32_t rel_buckets;  /* B > 0: learned bias rel[B, heads] per distance bucket.  With h = B / 2 (integer): distances n < h have a
                           bucket each (n); the other B - h buckets divide [h, rel_max] in equal steps of ln(n):
                           bucket = min(B - 1, h + floor((B - h) * ln(n / h) / ln(rel_max / h)))                 */
  float rel_max;        /* distance at which the last bucket is reached at the latest                            */
  float q_temp_coef;    /* != 0: the query at position p is multiplied by 1 + q_temp_coef * ln(1 + (p + 1) / q_temp_every), the
                           quotient taken as an integer                                                          */
  int32_t q_temp_every;
  /* -- further options of FF_MOE ---------------------------------------------------------------------------------------- */
  int32_t expert_act;   /* XOTB200_LM_EXPERT_*                                                                   */
  int32_t router_kind;  /* XOTB200_LM_ROUTER_*                                                                   */
  int32_t router_bias;  /* 1 = the router logits have a bias (router.b)                                          */
  int32_t shared_ff;    /* > 0: a shared expert of this inner size (same form as the experts) runs for every token and is added */
  /* -- further options of MIX_ATTENTION: rotation of queries and keys, kept first tokens, pooled far blocks --------------------
   * rot_dims > 0: the first rot_dims entries of every query and key head are rotated by the token's position (rot_layout, rot_base;
   * the cache holds rotated keys).  rot_scale_factor > 0: with wavelength l = 2 pi / f, f stays where l < original / high, becomes
   * f / factor where l > original / low, and in between (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
   * keep_first > 0 (with a window): the first keep_first tokens of the request stay visible whatever the distance.
   * pool > 0 (with a window): every block of `pool` consecutive tokens (blocks counted from position 0) that lies wholly before a
   * row's window, b * pool + pool - 1 <= i - window, is seen as ONE key and value: the means of the block's cached keys and values. */
  float rot_scale_factor;
  float rot_scale_low;
  float rot_scale_high;
  float rot_scale_original;
  int32_t keep_first;
  int32_t pool;
  /* -- MIX_MATRIX_LSTM: heads x (dim, vdim); q = W_q h / sqrt(dim), k, v; log gates i = cap tanh((W_i h + b) / cap),
   * f = logsigmoid(cap tanh((W_f h + b) / cap)); m <- max(f + m, i) (m starts at 0); S <- e^(f + m_old - m) S + e^(i - m) k v^T, n likewise
   * with k alone; o = S^T q / (max(|n.q|, e^-m) + 1e-6); o / rms(o) * norm (heads * vdim) * sigmoid(W_g h).
   * MIX_MAMBA2: heads x vdim channels, state size `dim`, `kv_heads` groups of B / C; W_in h = [z | x | B | C | dt]; x, B, C through a
   * causal filter of conv_taps taps with bias and silu; dt <- softplus(dt + dt_bias); per head S <- e^(-e^A_log dt) S + dt B x^T,
   * y = S^T C + D x; (y * silu(z)) RMS-normed in out_norm_groups equal parts, times norm; W_o. */
  float gate_cap;
  int32_t out_norm_groups;
  /* -- a second mixer in the same layer (par_on = 1): tensors l<i>.mix.left.* (this mixer) and l<i>.mix.right.* (the second) ------ */
  int32_t par_on;
  int32_t par_mixer;    /* a recurrent kind: XOTB200_LM_MIX_GATED_DELTA, MIX_MATRIX_LSTM or MIX_MAMBA2                           */
  int32_t par_heads;    /* the second mixer's sizes, under the names its kind gives them as a first mixer             */
  int32_t par_kv_heads;
  int32_t par_dim;
  int32_t par_vdim;
  int32_t par_conv_taps;
  int32_t par_out_norm_groups;
  float par_gate_cap;
  float mix_scale;      /* the layer's mixer output = mix_scale * this mixer (0 = 1) + par_scale * the second                    */
  float par_scale;
} xotb200_lm_layer;

typedef struct xotb200_lm_cfg {
  int32_t n_layers;    /* of the whole model                                   */
  int32_t start_layer; /* inclusive layer range this engine runs (a shard)     */
  int32_t end_layer;
  int32_t width;
  int32_t vocab;
  int32_t norm_groups;
  int32_t dtype;       /* XOTB200_LM_DTYPE_*                                   */
  float norm_eps;
  int32_t block;         /* XOTB200_LM_BLOCK_*: how a layer wraps its sublayers; the final norm is of the same kind        */
  int32_t max_positions; /* > 0: a learned position vector pos[p] is added to the embedding; requests hold at most this many tokens */
  int32_t pos_sinusoid;  /* 1 = a computed position vector is added to the embedding: entry 2i = sin(p f_i), 2i + 1 = cos(p f_i),
                            f_i = sinusoid_base^(-2i / width)                                                                     */
  float sinusoid_base;
  int32_t embed_norm;    /* 1 = the block's closing norm (weight embed.norm) is applied to the embedding sum before the first layer */
  float logit_scale;     /* logits are multiplied by this (0 = 1)                                                                   */
  float logit_softcap;   /* > 0: logits <- cap * tanh(logits / cap), after the scale                                                */
  /* -- BLOCK_PRE_SCALAR ------------------------------------------------------------------------------------------------------
   * streams > 0: hyper-connections.  The stream is kept in `streams` copies X_1 .. X_s (all equal to the embedding output at the
   * start); sublayer q of a layer reads u = sum_s in[s] X_s and writes X_t <- sum_s mix[s, t] X_s + mult * out[t] * y for all t at
   * once (tensors l<i>.hc<q>.in / out / mix); the model's output stream is the sum of the copies.  streams = 0: x += mult * y. */
  int32_t streams;
  int32_t canon_taps;    /* > 0: taps of the convolution on every sublayer input (l<i>.canon<q> [width, taps], last tap = current token) */
  float residual_mult;   /* 0 = 1                                                                                                   */
} xotb200_lm_cfg;

typedef struct xotb200_lm xotb200_lm;

const char* xotb200_lm_last_error(void);
const char* xotb200_lm_version(void);

/* `layers` has cfg->n_layers entries (the engine keeps those of its range). */
int xotb200_lm_create(const xotb200_lm_cfg* cfg, const xotb200_lm_layer* layers, int device, xotb200_lm** out);
int xotb200_lm_destroy(xotb200_lm* e);

/* Weights.  Tensor names: embed, head, final.norm, l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.<t>, l<i>.mlp.up / down with
 * <t> in {dq, dq.norm, uq | q, dkv, dkv.norm, uk, uv, g, o} or {r, k, v, g, a, a.b, w1, w2, w0, norm, o}; linear weights [out, in].
 * BLOCK_POST_LN models: pos, final.norm.b, l<i>.norm1 / norm1.b / norm2 / norm2.b; MIX_ATTENTION <t> in {q, q.b, q.norm, k, k.b,
 * k.norm, v, v.b, r1, r2, g, o}; MIX_GATED_DELTA <t> in {q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, norm, g, o};
 * l<i>.mlp.act (FF_XIELU); l<i>.mlp.router, l<i>.mlp.e<n>.gate / up / down (FF_MOE).
 * BLOCK_POST_RMS models: l<i>.norm1 / norm2, embed.norm; further MIX_ATTENTION tensors: o.b, sink [heads], rel [buckets, heads]; with
 * QKNORM_ROW q.norm / k.norm have the projection's size; further FF_MOE tensors: router.b, shared.up / shared.down; relu^2 experts
 * have no gate matrix.
 * BLOCK_PRE_SCALAR models: embed.norm, final.norm, l<i>.norm1 / norm2 (one number each), l<i>.canon1 / canon2, l<i>.hc1 / hc2 .in / .out /
 * .mix; MIX_ATTENTION with QKNORM_HEAD_PLAIN has no norm weights; MIX_MATRIX_LSTM <t> in {q, k, v, g, i, i.b, f, f.b, norm, o};
 * MIX_MAMBA2 <t> in {in, conv, conv.b, dt_bias, A_log, D, norm, o}; a layer with two mixers names them l<i>.mix.left.<t> / .right.<t>.
 * xotb200_lm_load_dir reads every *.safetensors of the directory (BF16 tensors) and is STRICT: a tensor of this shard that is
 * missing, has another shape or dtype, or an unknown tensor of an owned layer, is an error. */
int xotb200_lm_load_dir(xotb200_lm* e, const char* dir);
/* one tensor from host memory as bf16 bit patterns; returns 1 when the tensor belongs to another shard (ignored) */
int xotb200_lm_load_tensor(xotb200_lm* e, const char* name, const void* bf16_bits, const int64_t* shape, int ndim);
int xotb200_lm_check_loaded(xotb200_lm* e);
/* random weights made on the device (benchmarks, smoke runs): matrices ~ U with deviation 1/sqrt(inputs), norm weights near 1 */
int xotb200_lm_init_synthetic(xotb200_lm* e, uint64_t seed);

/* Request state: (re)creates the cache for at most max_requests live requests holding at most max_tokens tokens together.
 * page_size tokens per page (0 = 64).  All slots start empty. */
int xotb200_lm_begin(xotb200_lm* e, int max_tokens, int max_requests, int page_size);
/* Empty a slot: its pages return to the pool, its recurrent states are zeroed, its length becomes 0. */
int xotb200_lm_clear_request(xotb200_lm* e, int slot);
int xotb200_lm_request_len(xotb200_lm* e, int slot, int* len);

/* The step.  n_seq requests; request i is slot slots[i] and brings counts[i] >= 1 rows, which continue it at its current length.
 * First shard: tokens[sum counts] (int32 ids); other shards: hidden_f32[sum counts, width] (the fp32 residual stream).
 * want_rows[n_want]: indices into the packed rows whose output is asked for.
 *   last shard : logits_f32[n_want, vocab] and/or argmax_i32[n_want] (lowest-index argmax) — either may be NULL;
 *   other shards: hidden_out_f32[sum counts, width] (want_rows ignored).
 * A slot may appear once per step.  Fails without touching any state when the pool has too few free pages. */
int xotb200_lm_step(xotb200_lm* e, int n_seq, const int32_t* slots, const int32_t* counts, const int32_t* tokens,
                    const float* hidden_f32, const int32_t* want_rows, int n_want, float* logits_f32, int32_t* argmax_i32,
                    float* hidden_out_f32);

/* Debug / tests: the fp32 residual stream after every layer of the most recent step is kept when enabled (trace = 1) and copied
 * out as [local layers, rows, width]. */
int xotb200_lm_set_trace(xotb200_lm* e, int on);
int xotb200_lm_read_trace(xotb200_lm* e, float* out, int64_t n_floats);
/* Projection kernel choice: 0 = automatic (<= 8 rows: the one-warp-per-output decode kernel; more rows: tcgen05 tensor-core tiles for
 * bf16 operands that TMA can describe, else fp32 FMA tiles), 1 = always FMA tiles, 2 = tensor-core tiles at any row count. */
int xotb200_lm_set_gemm_mode(xotb200_lm* e, int mode);

int xotb200_lm_kernel_launches(xotb200_lm* e, int64_t* count);
/* Decode steps (every request brings one row) are captured into CUDA graphs and replayed: 1 = on (default), 0 = off. */
int xotb200_lm_set_graphs(xotb200_lm* e, int on);
int xotb200_lm_graph_replays(xotb200_lm* e, int64_t* count);
/* Attention kernel choice in the bf16 mode: 0 = automatic (a request that brings 16 rows or more: expanded keys / values and the
 * tensor-core streaming-softmax kernel; fewer rows: the absorbed kernel over the latent rows), 1 = always the absorbed kernel. */
int xotb200_lm_set_attention_mode(xotb200_lm* e, int mode);
int xotb200_lm_prompt_attention_launches(xotb200_lm* e, int64_t* count);
/* how many of the launches were tensor-core (tcgen05) products */
int xotb200_lm_tensor_core_launches(xotb200_lm* e, int64_t* count);
int xotb200_lm_weight_bytes(xotb200_lm* e, int64_t* bytes);
int xotb200_lm_cache_stats(xotb200_lm* e, int* pages_total, int* pages_free, int* page_size);
/* device time (CUDA events) of the most recent step, ms */
int xotb200_lm_last_step_ms(xotb200_lm* e, float* ms);

#ifdef __cplusplus
}
#endif
#endif /* XOTB200_LM_H */
