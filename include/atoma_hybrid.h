/*
 * atoma_hybrid.h — operators and the step executor for models whose layers mix attention with
 * recurrent (state-carrying) mixers, run on MIXED batches: portions of prompts beside single decoded
 * tokens, keys and values in a paged cache, recurrent state in per-sequence slots.
 *
 * The first design served through it is Lilovik: sandwich RMS norms (weights stored as offsets from
 * one), a sinusoidal position signal on the embedding, sigmoid attention (no softmax) with a
 * whole-projection q/k norm, a position-dependent query temperature, a tanh soft cap, a linear
 * distance bias and a talking-heads mix of the attention weights, minGRU layers, and a ReLU-gated
 * feed-forward.  Every constant of those mechanisms is an argument, so that another design can use
 * the operator with other values.
 *
 * The second design is Patadra: a learned position table, pre-norm layers with RMS norms taken over
 * equal consecutive groups of the row, sublayer results gated by a sigmoid of a projection of the
 * sublayer's input before they join the residual stream, latent attention (queries, keys and values
 * expanded from low-rank latents; only the key/value latent is cached) under a sliding window with a
 * per-head softmax sink, a mixture-of-experts feed-forward with a sigmoid router whose score scales the
 * expert's INPUT, a clamped gated activation, an always-on shared expert, a per-layer token input
 * looked up in a side table, and a tanh cap on the logits.  A span of layers may run several times
 * with the same weights; every run is one entry of the layer list with a cache of its own.
 *
 * The third design is Nemasun: a scaled embedding without a position signal, several residual LANES
 * (copies of the residual stream; every sublayer reads a weighted sum of them and writes its result
 * back through a lane-mixing matrix — the arrangement known as hyper-connections), softmax attention
 * with grouped key/value heads whose values are the un-normed key projections, a per-head q/k RMS
 * norm, a learned bias looked up by query-key distance, a sliding window that also keeps the first
 * tokens of the sequence, and a sigmoid gate on the heads' outputs; a clamped gated feed-forward with
 * biases; and a mixture of experts with a softmax router whose choice (not its weights) carries a
 * per-output correction and is restricted to the best groups of neighbouring outputs, with identity
 * experts (router outputs that hand the token's input through) and an ungated shared expert.
 *
 * The fourth design is Surinex: PARALLEL blocks (one RMS norm per layer whose output both the mixer and the
 * feed-forward read, each through its own causal tap filter over time whose last inputs are carried as state;
 * x <- x + mixer + feed-forward), three mixers — gated linear attention (a matrix state per head whose rows decay
 * by a data-dependent factor per key channel), latent attention with one rotated key part shared by all heads
 * beside the cached latent, and a PAIR of mixers on the same input: sigmoid attention with rotary positions on
 * queries, keys AND values (a head's sum is turned back by the query's position) beside a gated delta rule
 * (short causal filters with silu on q / k / v, unit-length q and k, a scalar decay and a write strength per
 * head), each result RMS-normed over the model width before the two are averaged — and a span of layers that
 * runs several times with the embedding added again and a per-pass vector at the start of every pass.
 *
 * Conventions: row-major; `dtype` is the number format of activations, large weights and the caches:
 * 1 = bfloat16, 2 = float32 (true 32-bit arithmetic: no reduced-precision matrix mode).  Whatever the
 * dtype, the residual stream, norm statistics, attention scores and weights, recurrent state and all
 * small per-channel parameters (norm weights, biases, per-head tables) are float32.  Everything is
 * stream-ordered and allocates nothing (library workspaces excepted).  Errors: atoma_last_status()
 * / atoma_last_error() (atoma_flash.h).
 */
#ifndef ATOMA_HYBRID_H_
#define ATOMA_HYBRID_H_

#include <stdint.h>

#include "atoma_flash.h"

#ifdef __cplusplus
extern "C" {
#endif

#define ATOMA_DTYPE_BF16 1u
#define ATOMA_DTYPE_F32 2u

/* out[t, 2i] = table[tokens[t], 2i] + sin(positions[t] * inv_freq[i]), out[t, 2i+1] = ... + cos(same); the angle is
 * formed and reduced in double precision (inv_freq [ceil(width/2)] is a device table of doubles). */
void atoma_embed_sinusoid(const uint32_t *tokens, const int64_t *positions, const void *table, const double *inv_freq,
                          float *out, int64_t T, int64_t width, int64_t vocab, uint32_t dtype, atoma_stream_t stream);

/* out[r, :] = x[rows ? rows[r] : r, :] / sqrt(mean(x^2) + eps) * (weight_offset + weight); x float32, out `dtype`. */
void atoma_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float weight_offset, void *out,
                        int64_t R, int64_t width, float eps, uint32_t dtype, atoma_stream_t stream);

/* Sandwich-norm residual update and the next sublayer's input norm in ONE kernel:
 *   x[t, :] += rms(y[t, :]) * (weight_offset + w_post);   h[t, :] = rms(x[t, :]) * (weight_offset + w_pre)
 * y, h in `dtype`, x float32 in place; w_pre / h may be NULL (no following norm). */
void atoma_postnorm_add_prenorm(const void *y, float *x, const float *w_post, const float *w_pre, void *h, int64_t T,
                                int64_t width, float eps, float weight_offset, uint32_t dtype, atoma_stream_t stream);

/* After the fused q/k/v projection qkv [T, H dim + G dim + G vdim] (+ bias, float32, may be NULL):
 *   q <- rms over the WHOLE q part * q_weight * (1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)) -> q_out [T, H dim]
 *   k <- rms over the WHOLE k part * k_weight -> key cache row slot_mapping[t];   v -> value cache row
 * caches: [num_blocks * block_size, G, dim] and [.., G, vdim] in `dtype`; slot < 0 is skipped. */
void atoma_qk_norm_cache(const void *qkv, const float *bias, const float *q_weight, const float *k_weight,
                         const int64_t *positions, const int64_t *slot_mapping, void *q_out, void *k_cache, void *v_cache,
                         int64_t T, int64_t H, int64_t G, int64_t dim, int64_t vdim, float eps, float temp_coef,
                         int64_t temp_every, uint32_t dtype, atoma_stream_t stream);

/*
 * Sigmoid attention over a paged cache for a mixed batch.  For query token t of sequence b at position p and every
 * cached key j <= p of that sequence:
 *   s = (q_g . k_j) * scale;  s = softcap * tanh(s / softcap) (softcap > 0);  s -= slopes[g] * (p - j)
 *   a_g = sigmoid(s + head_bias[g]);   a'_h = sum_g talk[h, g] a_g  (talk NULL = identity)
 *   out[t, h, :] = sum_j a'_h(j) v_j[kv head of h, :]
 * Scores, weights and the sums are float32; keys are visited in position order whatever the batch looks like.
 */
typedef struct atoma_sigmoid_attn_args {
    const void *q;                /* [T, H dim] */
    const void *k_cache, *v_cache;
    void *out;                    /* [T, H vdim] */
    const int64_t *positions;     /* [T] */
    const int32_t *token_seq;     /* [T] batch row of every token */
    const int32_t *query_start;   /* [B + 1] first token of every batch row (rows are contiguous, positions ascending) */
    const int32_t *block_tables;  /* [B, max_blocks] */
    const float *slopes, *head_bias, *talk; /* [H] (NULL: no distance term), [H], [H, H] (NULL: the heads do not talk) */
    int64_t T, B, max_blocks, H, G, dim, vdim, block_size;
    float scale, softcap;
    uint32_t dtype;
    int32_t max_query_len;        /* longest portion of the batch (1 = decode only): selects the kernel */
    int32_t max_seq_len;          /* longest sequence (context + portion) of the batch; 0 = unknown (keys are not split) */
} atoma_sigmoid_attn_args;
void atoma_sigmoid_attention_paged(const atoma_sigmoid_attn_args *args, atoma_stream_t stream);

/*
 * minGRU over a mixed batch.  zxg [T, 3 S] = the fused projections (rows: update gate, candidate, output gate) with
 * bias [3 S] (may be NULL) added here.  Per sequence b (tokens query_start[b] .. query_start[b+1]) and channel c:
 *   z = sigmoid(zpre), cand = u >= 0 ? u + 1/2 : sigmoid(u),  s <- (1 - z) s + z cand,  out = s * silu(g)
 * s starts from state[state_slots[b], c] — from zero when context_lens[b] == 0 — and is stored back.  float32 state.
 */
void atoma_mingru_scan(const void *zxg, const float *bias, float *state, const int32_t *state_slots,
                       const int32_t *query_start, const int32_t *context_lens, void *out, int64_t T, int64_t B, int64_t S,
                       int32_t max_query_len, uint32_t dtype, atoma_stream_t stream);

/* out[t, j] = act(gu[t, j]) * gu[t, ff + j]; act: 0 = silu, 1 = relu, 2 = gelu (tanh form). */
void atoma_glu(const void *gu, void *out, int64_t T, int64_t ff, int32_t act, uint32_t dtype, atoma_stream_t stream);

/* y[T, N] = x[T, K] w[N, K]^T.  bfloat16 with 16-byte aligned rows runs the tcgen05 kernels of atoma_gemm_tn;
 * float32 (and whatever those kernels do not take) runs a plain float32-FMA tile kernel. */
void atoma_linear(const void *x, const void *w, void *y, int64_t T, int64_t N, int64_t K, uint32_t dtype,
                  atoma_stream_t stream);

/* logits_f32[r, :] = logits[r, :] * scale and token_out[r] = the last index of the row's maximum. */
void atoma_scale_logits_greedy(const void *logits, float *logits_f32, uint32_t *token_out, int64_t R, int64_t vocab,
                               float scale, uint32_t dtype, atoma_stream_t stream);

/* ------------------------------------------------------------------------------------------ */
/* Pre-norm designs with gated residuals, latent attention and mixtures of experts             */
/* ------------------------------------------------------------------------------------------ */

/* out[t, :] = table[tokens[t], :] + pos_table[positions[t], :] (float32 sum; positions beyond max_positions - 1 are an
 * error the caller must exclude: the kernel clamps). */
void atoma_embed_learned(const uint32_t *tokens, const int64_t *positions, const void *table, const void *pos_table, float *out,
                         int64_t T, int64_t width, int64_t vocab, int64_t max_positions, uint32_t dtype, atoma_stream_t stream);

/* RMS norm in `groups` equal consecutive parts of the row, each divided by its own sqrt(mean(part^2) + eps); the whole
 * row is then multiplied by (weight_offset + weight).  groups = 1 is atoma_rmsnorm_rows.  width % groups == 0. */
void atoma_group_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float weight_offset, int64_t groups,
                              void *out, int64_t R, int64_t width, float eps, uint32_t dtype, atoma_stream_t stream);

/*
 * Residual update of a pre-norm layer and the next sublayer's input norm in ONE kernel.  Per token t and channel c:
 *   v = (y ? y[t, c] * (row_scale ? row_scale[t] : 1) : 0) + sum_{k < top} expert_out[pair_row[t top + k], c]
 *   x[t, c] += gate ? v * sigmoid(gate[t, c] + gate_bias[c]) : v
 *   h[t, :]  = group_rmsnorm(x[t, :]) * (weight_offset + w_next)      (w_next NULL: no norm)
 *   x_cast[t, :] = x[t, :] in `dtype`                                  (x_cast NULL: not written)
 * y, gate, expert_out, h, x_cast in `dtype` with row strides ld_y, ld_gate, width, width, width; x float32 in place.
 * The experts' rows are added in the order k = 0 .. top - 1.
 */
typedef struct atoma_gated_residual_args {
    const void *y;
    int64_t ld_y;
    const float *row_scale;       /* [T] or NULL */
    const void *expert_out;       /* [rows, width] or NULL */
    const int32_t *pair_row;      /* [T top] row of expert_out that holds pair (t, k) */
    int64_t top;
    const void *gate;             /* pre-activation of the residual gate, or NULL */
    int64_t ld_gate;
    const float *gate_bias;       /* [width] */
    float *x;                     /* [T, width] */
    const float *w_next;          /* [width] or NULL */
    void *h;                      /* [T, width] */
    void *x_cast;                 /* [T, width] or NULL */
    int64_t T, width, groups;
    float eps, weight_offset;
    uint32_t dtype;
} atoma_gated_residual_args;
void atoma_gated_residual_norm(const atoma_gated_residual_args *args, atoma_stream_t stream);

/* Token side input, gate part: out[t, j] = gelu_tanh(a[t, j]) * side_table[tokens[t], part * dim + j], j < dim.
 * a (row stride ld_a) and out [T, dim] in `dtype`; side_table [vocab, table_width] in `dtype`. */
void atoma_side_gate(const void *a, int64_t ld_a, const uint32_t *tokens, const void *side_table, int64_t table_width, int64_t part,
                     void *out, int64_t T, int64_t dim, int64_t vocab, uint32_t dtype, atoma_stream_t stream);

/* x[t, :] += y[t, :] / sqrt(mean(y^2) + eps) * w_unit;  h[t, :] = group_rmsnorm(x[t, :]) * (weight_offset + w_next) (NULL: none). */
void atoma_unitnorm_add_norm(const void *y, float *x, const float *w_unit, const float *w_next, void *h, int64_t T, int64_t width,
                             int64_t groups, float eps, float weight_offset, uint32_t dtype, atoma_stream_t stream);

/* After the fused down projections proj[t, :] = [c_q (q_rank) | c (kv_rank) | ...] (row stride ld):
 *   cq_out[t, :] = rms(c_q) * q_weight  (q_rank = 0: no query latent)      latent_cache[slot_mapping[t], :] = rms(c) * kv_weight
 * plain weights; cq_out and the cache [num_blocks * block_size, kv_rank] in `dtype`; slot < 0 is skipped. */
void atoma_latent_norm_cache(const void *proj, int64_t ld, const float *q_weight, const float *kv_weight, const int64_t *slot_mapping,
                             void *cq_out, void *latent_cache, int64_t T, int64_t q_rank, int64_t kv_rank, float eps, uint32_t dtype,
                             atoma_stream_t stream);

/* Per-head projection between a head's own space and a shared latent, w [H n, R] (stored [out, in], as the checkpoint has it):
 *   absorb = 1:  out[t, h, r] = sum_j in[t, h n + j] w[h n + j, r]     in [T, H n] `dtype`      -> out [T, H, R] float32
 *   absorb = 0:  out[t, h n + j] = sum_r in[t, h, r] w[h n + j, r]     in [T, H, R] float32    -> out [T, H n] `dtype`
 * The first moves a query into the latent space of the keys (so that q . (W c) = (W^T q) . c needs no expanded keys);
 * the second expands a head's weighted sum of latents into its values. */
void atoma_head_project(const void *in, const void *w, void *out, int64_t T, int64_t H, int64_t n, int64_t R, int32_t absorb,
                        uint32_t dtype, atoma_stream_t stream);

/*
 * Softmax attention of H heads over ONE shared cached latent per token (keys = values = the latent), paged, mixed batch.
 * For query token t of sequence b at position p and keys j with 0 <= p - j < window (window <= 0: every j <= p):
 *   s_h(j) = (q_lat[t, h, :] . c_j) * scale
 *   w_h(j) = exp(s_h(j)) / (sum_j' exp(s_h(j')) + (sink ? exp(sink[h]) : 0))
 *   out[t, h, :] = sum_j w_h(j) c_j
 * q_lat and out float32 [T, H, R]; scores, weights and sums float32.
 */
typedef struct atoma_latent_attn_args {
    const float *q_lat;
    const void *latent_cache;     /* [num_blocks * block_size, R] `dtype` */
    float *out;
    const int64_t *positions;     /* [T] */
    const int32_t *token_seq;     /* [T] */
    const int32_t *query_start;   /* [B + 1] */
    const int32_t *block_tables;  /* [B, max_blocks] */
    const float *sink;            /* [H] or NULL */
    int64_t T, B, max_blocks, H, R, block_size, window;
    float scale;
    uint32_t dtype;
    int32_t max_query_len, max_seq_len;
    int32_t skip_min_q;           /* > 0: sequences with at least this many query tokens in the step are left alone */
    int64_t out_cols;             /* > 0: only the first out_cols entries of every row of `out` are read by the caller (a cached row whose
                                   * tail takes part in the scores only, like a rotated key part); the rest may be left unwritten */
} atoma_latent_attn_args;
void atoma_latent_attention_paged(const atoma_latent_attn_args *args, atoma_stream_t stream);

/*
 * The same attention for LONG prompt portions, on expanded keys and values (bfloat16, dim = vdim of 64 or 128): for every
 * sequence with at least min_q query tokens in the step, the latents its queries can see (window + portion) are gathered
 * from the paged cache, k = w_uk c and v = w_uv c are formed by two dense products, and softmax attention with the window
 * and the sink runs per head on the 5th-generation tensor cores; out[t, h dim ..] is written for those sequences' tokens
 * only.  A (query, key, head) pair costs 2 (dim + vdim) multiply-adds here instead of 4 kv_rank in the latent space.
 * max_keys: an upper bound of the gathered rows (sum over the long sequences of min(context, window - 1) + tokens).
 */
typedef struct atoma_latent_expanded_args {
    const void *q;                /* [T, H dim] */
    const void *latent_cache;
    const void *w_uk, *w_uv;      /* [H dim, R], [H dim, R] */
    void *out;                    /* [T, H dim] */
    const int32_t *query_start;   /* [B + 1] */
    const int32_t *context_lens;  /* [B] */
    const int32_t *block_tables;  /* [B, max_blocks] */
    const float *sink;            /* [H] or NULL */
    int64_t T, B, max_blocks, H, dim, R, block_size, window, max_keys;
    float scale;
    int32_t min_q, max_query_len, max_seq_len;
} atoma_latent_expanded_args;
void atoma_latent_attention_expanded(const atoma_latent_expanded_args *args, atoma_stream_t stream);

/* Router of a mixture of experts, float32: z = w_router h (h [T, width] `dtype`, w_router [experts, width] float32),
 * s = sigmoid(z) (score_fn 0) ; the `top` largest scores (ties: the lower index) -> top_expert [T, top] int32 and
 * top_weight [T, top] float32 = the chosen scores as they are (renormalize 0) or divided by their sum (1).
 * w_row_gate (float32 [width], may be NULL): row_gate[t] = sigmoid(w_row_gate . h[t]) — the shared expert's gate. */
void atoma_moe_route(const void *h, const float *w_router, const float *w_row_gate, int32_t *top_expert, float *top_weight,
                     float *row_gate, int64_t T, int64_t width, int64_t experts, int64_t top, int32_t renormalize, uint32_t dtype,
                     atoma_stream_t stream);

/* y = act(g, u) of a gated feed-forward with clamps: g = min(gu[t, j], limit), u = clamp(gu[t, ff + j], -limit, limit),
 * out[t, j] = g * sigmoid(alpha g) * (u + up_shift).  limit <= 0: no clamp.  gu row stride ld. */
void atoma_glu_clamped(const void *gu, int64_t ld, void *out, int64_t T, int64_t ff, float limit, float alpha, float up_shift,
                       uint32_t dtype, atoma_stream_t stream);

/*
 * The routed experts of a step: every (token, k) pair is sorted by its expert on the device (no host read), its input row
 * h[t] * top_weight[t, k] is gathered (scale_input 1; with 0 the weight multiplies the expert's output instead), and the
 * experts run as two grouped products with the clamped gated activation between them:
 *   expert_out[pair_row[t top + k], :] = w_down[e] act(w_gate_up[e] (weight * h[t]))
 * w_gate_up [experts, 2 ff, width] (gate rows, then up rows), w_down [experts, width, ff], all `dtype`.
 * workspace: atoma_moe_workspace_bytes(T, top, experts, width, ff, dtype) bytes; expert_out and pair_row point into it
 * and are returned through *expert_out / *pair_row for atoma_gated_residual_norm.
 */
typedef struct atoma_moe_args {
    const void *h;                /* [T, width] */
    const int32_t *top_expert;    /* [T, top] */
    const float *top_weight;      /* [T, top] */
    const void *w_gate_up, *w_down;
    void *workspace;
    int64_t workspace_bytes;
    int64_t T, width, experts, top, ff;
    float limit, alpha, up_shift;
    int32_t scale_input;
    uint32_t dtype;
} atoma_moe_args;
int64_t atoma_moe_workspace_bytes(int64_t T, int64_t top, int64_t experts, int64_t width, int64_t ff, uint32_t dtype);
void atoma_moe_experts(const atoma_moe_args *args, const void **expert_out, const int32_t **pair_row, atoma_stream_t stream);

/* logits_f32[r, :] = cap(logits[r, :] * scale), cap(v) = softcap * tanh(v / softcap) (softcap <= 0: identity), and
 * token_out[r] = the last index of the row's maximum. */
void atoma_finish_logits_greedy(const void *logits, float *logits_f32, uint32_t *token_out, int64_t R, int64_t vocab, float scale,
                                float softcap, uint32_t dtype, atoma_stream_t stream);

/* ------------------------------------------------------------------------------------------ */
/* Residual lanes, softmax attention with a distance table, grouped routing                     */
/* ------------------------------------------------------------------------------------------ */

/* x[t, s, :] = table[tokens[t], :] * scale for every lane s < lanes; x float32 [T, lanes, width]. */
void atoma_embed_scaled_lanes(const uint32_t *tokens, const void *table, float scale, float *x, int64_t T, int64_t lanes, int64_t width,
                              int64_t vocab, uint32_t dtype, atoma_stream_t stream);

/* A sublayer's input from the lanes: u = sum_s w_in[s] x[r, s, :] (w_in NULL: the plain sum), r = rows ? rows[i] : i;
 * out[i, :] = u / sqrt(mean(u^2) + eps) * (weight_offset + weight) in `dtype`; sum_out (float32 [R, width], may be NULL) = u. */
void atoma_lanes_read_norm(const float *x, const float *w_in, const int32_t *rows, const float *weight, float weight_offset, void *out,
                           float *sum_out, int64_t R, int64_t lanes, int64_t width, float eps, uint32_t dtype, atoma_stream_t stream);

/*
 * A sublayer's result written back to the lanes, fused with the NEXT sublayer's read and norm.  Per token t, channel c:
 *   v = (y ? y[t, c] : 0) + (y_bias ? y_bias[c] : 0)
 *       + sum_{k < top} (top_expert[t, k] in [0, experts):  expert_out[pair_row[t top + k], c]
 *                        top_expert[t, k] >= experts:        top_weight[t, k] * h_in[t, c]       (identity expert)
 *                        top_expert[t, k] < 0:               nothing)
 *   x'[t, s2, c] = sum_s w_mix[s, s2] x[t, s, c] + w_out[s2] v           (all lanes from the old ones)
 *   u = sum_s w_in_next[s] x'[t, s, c];  h[t, :] = u / sqrt(mean(u^2) + eps) * (weight_offset + w_next)    (w_next NULL: no read)
 *   lane_sum[t, c] = sum_s x'[t, s, c]                                                                    (NULL: not written)
 * y, expert_out, h_in, h in `dtype`; x float32 [T, lanes, width] in place.  h_in and h may be the same buffer.
 * The experts' rows are added in the order k = 0 .. top - 1.
 */
typedef struct atoma_lanes_update_args {
    const void *y;                /* [T, width] or NULL */
    const float *y_bias;          /* [width] or NULL */
    const void *expert_out;       /* rows of the routed experts' results, or NULL */
    const int32_t *pair_row;      /* [T top] */
    const int32_t *top_expert;    /* [T top] */
    const float *top_weight;      /* [T top] */
    const void *h_in;             /* [T, width]: what identity experts hand through */
    int64_t top, experts;
    float *x;                     /* [T, lanes, width] */
    const float *w_mix, *w_out;   /* [lanes, lanes] indexed [from, to]; [lanes] */
    const float *w_in_next;       /* [lanes] or NULL (plain sum) */
    const float *w_next;          /* [width] or NULL */
    void *h;                      /* [T, width] */
    float *lane_sum;              /* [T, width] or NULL */
    int64_t T, lanes, width;
    float eps, weight_offset;
    uint32_t dtype;
} atoma_lanes_update_args;
void atoma_lanes_update_norm(const atoma_lanes_update_args *args, atoma_stream_t stream);

/* After a fused projection proj[t, :] (row stride ld) that holds the queries at column q_off (H heads of dim), the keys at
 * k_off (G heads of dim) and the values at v_off (G heads of vdim; v_off = k_off: the values ARE the key projections):
 *   q_out[t, h, :] = proj_q / sqrt(mean over the head's dim + eps) * (weight_offset + q_weight)     (one weight [dim] for all heads)
 *   k_cache[slot_mapping[t], g, :] = the same with k_weight;   v_cache[slot, g, :] = the values as projected (no norm)
 * caches [num_blocks * block_size, G, dim] / [.., G, vdim] in `dtype`; slot < 0 is skipped. */
void atoma_qk_headnorm_cache(const void *proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, const float *q_weight,
                             const float *k_weight, float weight_offset, const int64_t *slot_mapping, void *q_out, void *k_cache,
                             void *v_cache, int64_t T, int64_t H, int64_t G, int64_t dim, int64_t vdim, float eps, uint32_t dtype,
                             atoma_stream_t stream);

/*
 * Softmax attention over a paged cache for a mixed batch, grouped key/value heads (head h reads kv head h / (H / G)).
 * Query token t of sequence b at position p sees key j <= p if p - j < window (window <= 0: no limit) or j < keep_first.
 *   s_h(j) = (q_h . k_j) * scale + (dist_bias ? dist_bias[min(p - j, dist_rows - 1), h] : 0)
 *   out[t, h, :] = softmax_j(s_h) v_j * (gate ? sigmoid(gate[t, h vdim ..]) : 1)
 * Scores, weights, maxima and sums are float32.  gate (row stride ld_gate) and out in `dtype`.
 */
typedef struct atoma_softmax_attn_args {
    const void *q;                /* [T, H dim] */
    const void *k_cache, *v_cache;
    void *out;                    /* [T, H vdim] */
    const void *gate;             /* pre-activation of the output gate, [T, >= H vdim], or NULL */
    int64_t ld_gate;
    const float *dist_bias;       /* [dist_rows, H] or NULL */
    int64_t dist_rows;
    const int64_t *positions;     /* [T] */
    const int32_t *token_seq;     /* [T] */
    const int32_t *query_start;   /* [B + 1] */
    const int32_t *block_tables;  /* [B, max_blocks] */
    int64_t T, B, max_blocks, H, G, dim, vdim, block_size, window, keep_first;
    float scale;
    uint32_t dtype;
    int32_t max_query_len, max_seq_len;
    int32_t skip_min_q;           /* > 0: sequences with at least this many query tokens in the step are left alone */
    /* long prompt portions (all zero = none): sequences with at least long_min_q (>= 32) tokens in the step, how many there are,
     * the sum of their tokens and of their contexts.  bfloat16 heads of 64 or 128 with dim = vdim run them on the tensor-memory
     * prefill kernel: the keys and values their queries can see through the window are gathered from the pages, the distance
     * term is added inside that kernel's softmax, the kept first tokens behind the window are a second short pass merged through
     * the log-sum-exp, and the gate is applied in the merge. */
    int32_t long_min_q, long_seqs;
    int64_t long_tokens, long_ctx_sum;
} atoma_softmax_attn_args;
void atoma_softmax_attention_paged(const atoma_softmax_attn_args *args, atoma_stream_t stream);

/* Router with a restricted choice, float32.  z = w_router h over `outputs` router rows (experts, then identity experts);
 * s = softmax(z) (score_fn 1) or sigmoid(z) (0); choice score c = s + correction (NULL: none).  The outputs form `groups`
 * equal groups of neighbours (groups <= 1: no restriction); a group's score is its largest c; only outputs of the `keep`
 * best groups can be chosen (ties: the lower group).  The `top` largest c among them (ties: the lower index) ->
 * top_expert [T, top] (an index >= the caller's expert count is an identity expert; -1 where fewer than `top` could be
 * chosen) and top_weight = their s divided by (their sum + 1e-20) (renormalize 1) or as they are (0). */
void atoma_moe_route_grouped(const void *h, const float *w_router, const float *correction, int32_t *top_expert, float *top_weight,
                             int64_t T, int64_t width, int64_t outputs, int64_t top, int64_t groups, int64_t keep, int32_t score_fn,
                             int32_t renormalize, uint32_t dtype, atoma_stream_t stream);

/* act_out[T, ff] = clamped gated activation (atoma_glu_clamped_bias) of the projection x [T, K] w_gate_up [2 ff, K]^T (gate rows,
 * then up rows).  Decode-sized bfloat16 steps (T <= 128, K % 64 == 0) run ONE kernel, the activation in the tcgen05 product's
 * epilogue; everything else atoma_linear into proj [T, 2 ff] and atoma_glu_clamped_bias. */
void atoma_linear_glu_clamped(const void *x, const void *w_gate_up, const float *bias, void *proj, void *act_out, int64_t T, int64_t ff,
                              int64_t K, float limit, float alpha, float up_shift, uint32_t dtype, atoma_stream_t stream);

/* atoma_glu_clamped with biases added first: g = gu[t, j] + bias[j], u = gu[t, ff + j] + bias[ff + j] (bias float32 [2 ff]). */
void atoma_glu_clamped_bias(const void *gu, int64_t ld, const float *bias, void *out, int64_t T, int64_t ff, float limit, float alpha,
                            float up_shift, uint32_t dtype, atoma_stream_t stream);

/* ------------------------------------------------------------------------------------------ */
/* Parallel blocks: tap filters with carried inputs, matrix-state recurrences, rotary operators */
/* ------------------------------------------------------------------------------------------ */

/*
 * Residual update of a parallel block fused with what precedes the next layer and with that layer's input norm.
 * Per token t and channel c, all in float32:
 *   a = y_a ? (norm_a ? y_a[t, :] / sqrt(mean(y_a[t, :]^2) + eps) * norm_a : y_a[t, :]) : 0        (b likewise)
 *   x[t, c] += mix_scale * (a[c] + b[c]) + (y_ff ? y_ff[t, c] : 0);     trace[t, c] = x[t, c]          (trace NULL: not written)
 *   x[t, c] += (add_rows ? add_rows[t, c] : 0) + (add_vec ? add_vec[c] : 0)
 *   h[t, :]  = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * (weight_offset + w_next)                       (w_next NULL: no norm)
 * y_a, y_b, y_ff, h in `dtype` [T, width]; x, trace, add_rows float32 [T, width].  With no addends it is the first
 * layer's input norm.
 */
typedef struct atoma_parallel_residual_args {
    const void *y_a, *y_b, *y_ff;
    const float *norm_a, *norm_b; /* [width] or NULL */
    float mix_scale;
    float *x;
    float *trace;
    const float *add_rows, *add_vec;
    const float *w_next;
    void *h;
    int64_t T, width;
    float eps, weight_offset;
    uint32_t dtype;
} atoma_parallel_residual_args;
void atoma_parallel_residual_norm(const atoma_parallel_residual_args *args, atoma_stream_t stream);

/*
 * Causal tap filter over time per channel, on a mixed batch, with the inputs that precede a portion carried as state.
 * in [T, channels] (row stride ld_in, `dtype`); w1, w2 [channels, taps] float32, the LAST column weighs the current token
 * (w2 / out2 may be NULL: one filter).  For token t of sequence b at position p:
 *   f_k(t, c) = sum_{j < taps} w_k[c, j] * in(position p - (taps - 1) + j, c)       zero before the sequence's start
 *   out_k[t, c] = act(residual ? in[t, c] + f_k : f_k)        act: 0 = none, 1 = silu        (`dtype`, row stride ld_out)
 * history [slots, history_stride] float32 holds, at the slot of the sequence, its last taps - 1 inputs as
 * [taps - 1, channels]; it is read for positions before the portion (never when they lie before the sequence's start)
 * and rewritten with the portion's last inputs.  taps <= 16.
 */
typedef struct atoma_tap_filter_args {
    const void *in;
    int64_t ld_in;
    const float *w1, *w2;
    void *out1, *out2;
    int64_t ld_out;
    float *history;
    int64_t history_stride;
    const int32_t *state_slots;   /* [B] */
    const int32_t *token_seq;     /* [T] */
    const int32_t *query_start;   /* [B + 1] */
    const int32_t *context_lens;  /* [B] */
    int64_t T, B, channels, taps;
    int32_t residual, act;
    uint32_t dtype;
} atoma_tap_filter_args;
void atoma_tap_filter(const atoma_tap_filter_args *args, atoma_stream_t stream);

/*
 * Matrix-state recurrences on a mixed batch.  Every head keeps S [dim, vdim] float32 at the sequence's state slot
 * (state [slots, state_stride], head h at h dim vdim); it starts from zero when context_lens[b] == 0 and is stored back.
 * Tokens of a sequence are visited in order, so the result does not depend on how the sequence was cut into steps.
 *   kind 0, gated linear attention (q, k [T, H dim], v [T, H vdim]; decay pre-activation z [T, H dim] + z_bias):
 *     alpha = exp(log(sigmoid(z)) / tau);  S <- diag(alpha) S + k v^T;  o = S^T (q * q_scale)
 *   kind 1, gated delta rule (q, k [T, G dim] shared by H / G heads, v [T, H vdim]; per head b_pre, a_pre [T, H]):
 *     q, k <- x / sqrt(sum(x^2) + unit_eps) (q also times q_scale);  beta = sigmoid(b_pre);
 *     g = exp(-exp(a_log[h]) * softplus(a_pre + dt_bias[h]));
 *     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
 * q, k, v, z, b_pre, a_pre are columns of `dtype` matrices with their own row strides; out float32 [T, H vdim].
 */
typedef struct atoma_state_scan_args {
    int32_t kind;
    const void *q, *k, *v, *z, *b_pre, *a_pre;
    int64_t ld_q, ld_k, ld_v, ld_z, ld_b, ld_a;
    const float *z_bias;          /* [H dim] (kind 0) */
    const float *a_log, *dt_bias; /* [H] (kind 1) */
    float tau, q_scale, unit_eps;
    float *state;
    int64_t state_stride;
    const int32_t *state_slots, *query_start, *context_lens;
    float *out;
    int64_t T, B, H, G, dim, vdim;
    uint32_t dtype;
} atoma_state_scan_args;
void atoma_state_scan(const atoma_state_scan_args *args, atoma_stream_t stream);

/* out[t, h vdim + j] = o[t, h, j] / sqrt(mean_j(o[t, h, :]^2) + eps) * weight[j] * silu(gate[t, h vdim + j]);
 * o float32 [T, H vdim], gate (row stride ld_gate) and out [T, H vdim] in `dtype`; gate NULL: no gate. */
void atoma_headnorm_gate(const float *o, const float *weight, const void *gate, int64_t ld_gate, void *out, int64_t T, int64_t H,
                         int64_t vdim, float eps, uint32_t dtype, atoma_stream_t stream);

/*
 * After a fused projection proj[t, :] (row stride ld): queries at q_off (H heads of dim), keys at k_off (G of dim), values
 * at v_off (G of vdim).  Per head: RMS norm over dim with q_weight / k_weight ([dim], NULL: none), then the first
 * 2 rot_pairs entries are turned by position * qk_freq[i] (float32 angle) in pairs (2i, 2i + 1) (interleaved = 1) or
 * (i, i + rot_pairs) (0); the values' first 2 v_pairs entries likewise by v_freq (v_freq NULL: stored as projected).
 * q -> q_out [T, H dim]; k, v -> cache rows slot_mapping[t] (slot < 0 is skipped).
 */
typedef struct atoma_qkv_rope_args {
    const void *proj;
    int64_t ld, q_off, k_off, v_off;
    const float *q_weight, *k_weight;
    const float *qk_freq, *v_freq;
    int64_t rot_pairs, v_pairs;
    int32_t interleaved;
    const int64_t *positions, *slot_mapping;
    void *q_out, *k_cache, *v_cache;
    int64_t T, H, G, dim, vdim;
    float eps;
    uint32_t dtype;
} atoma_qkv_rope_args;
void atoma_qkv_headnorm_rope_cache(const atoma_qkv_rope_args *args, atoma_stream_t stream);

/* In place on x [T, H, n] (`dtype`): the first 2 pairs entries of every head turned by sign * position * freq[i]. */
void atoma_rotate_heads(void *x, const int64_t *positions, const float *freq, int64_t T, int64_t H, int64_t n, int64_t pairs,
                        int32_t interleaved, float sign, uint32_t dtype, atoma_stream_t stream);

/*
 * Latent attention with a rotated key part.  proj[t, :] (row stride ld) = [c_q (q_rank) | c (kv_rank) | k_rot (rot_dim)]:
 *   cq_out[t, :] = rms(c_q) * q_weight;   cache[slot_mapping[t], :] = [rms(c) * kv_weight | rotate(k_rot, position)]
 * rotation in pairs (i, i + pairs) (interleaved 0) or (2i, 2i + 1); cache rows of kv_rank + rot_dim in `dtype`.
 */
void atoma_latent_norm_rope_cache(const void *proj, int64_t ld, const float *q_weight, const float *kv_weight, const float *freq,
                                  int64_t pairs, int32_t interleaved, const int64_t *positions, const int64_t *slot_mapping,
                                  void *cq_out, void *cache, int64_t T, int64_t q_rank, int64_t kv_rank, int64_t rot_dim, float eps,
                                  uint32_t dtype, atoma_stream_t stream);

/* Queries q [T, H, dim + rot_dim] (`dtype`) into the space of the cached rows, q_lat float32 [T, H, kv_rank + rot_dim]:
 *   q_lat[t, h, :kv_rank] = w_uk_h^T q[t, h, :dim]  (w_uk [H dim, kv_rank]);   q_lat[t, h, kv_rank:] = rotate(q[t, h, dim:], position) */
void atoma_latent_query_absorb_rope(const void *q, const void *w_uk, const float *freq, int64_t pairs, int32_t interleaved,
                                    const int64_t *positions, float *q_lat, int64_t T, int64_t H, int64_t dim, int64_t rot_dim,
                                    int64_t kv_rank, uint32_t dtype, atoma_stream_t stream);

/* Values of every head from its weighted sum of cached rows: out[t, h vdim + j] = sum_{r < kv_rank} o_lat[t, h, r] w_uv[h vdim + j, r];
 * o_lat float32 [T, H, row] with row >= kv_rank (what lies behind kv_rank is not read). */
void atoma_latent_expand_values(const float *o_lat, const void *w_uv, void *out, int64_t T, int64_t H, int64_t vdim, int64_t kv_rank,
                                int64_t row, uint32_t dtype, atoma_stream_t stream);

/* ------------------------------------------------------------------------------------------ */
/* Step executor                                                                                */
/* ------------------------------------------------------------------------------------------ */
enum { ATOMA_MIXER_SIGMOID_ATTENTION = 0, ATOMA_MIXER_MINGRU = 1, ATOMA_MIXER_LATENT_ATTENTION = 2, ATOMA_MIXER_SOFTMAX_ATTENTION = 3,
       ATOMA_MIXER_GLA = 4, ATOMA_MIXER_PAIR = 5 };
enum { ATOMA_BLOCK_SANDWICH = 0, ATOMA_BLOCK_PRENORM = 1, ATOMA_BLOCK_LANES = 2, ATOMA_BLOCK_PARALLEL = 3 };
enum { ATOMA_SCORE_SIGMOID = 0, ATOMA_SCORE_SOFTMAX = 1 };
enum { ATOMA_FF_DENSE = 0, ATOMA_FF_MOE = 1 };
enum { ATOMA_ACT_SILU = 0, ATOMA_ACT_RELU = 1, ATOMA_ACT_GELU_TANH = 2 };

typedef struct atoma_hybrid_layer {
    int32_t mixer, has_mlp;
    const float *norm1, *norm1b, *norm2, *norm2b; /* [width] offsets from one */
    /* attention */
    int64_t heads, kv_heads, dim, vdim, temp_every;
    float scale, softcap, temp_coef;
    const void *w_qkv;      /* [H dim + G dim + G vdim, width] */
    const float *b_qkv;
    const float *q_norm, *k_norm, *talk, *head_bias, *slopes;
    void *k_cache, *v_cache;
    /* minGRU */
    int64_t state_width;
    const void *w_zxg;      /* [3 S, width] */
    const float *b_zxg;
    float *state;           /* [slots, S] */
    /* both mixers */
    const void *w_o;        /* [width, H vdim] or [width, S] */
    /* feed-forward */
    int64_t ff;
    int32_t act;
    const void *w_gate_up;  /* [2 ff, width] */
    const void *w_down;     /* [width, ff] */
    /* ---- pre-norm blocks (model.block_style = ATOMA_BLOCK_PRENORM) ---- */
    /* latent attention (uses heads, dim, vdim, scale above) */
    int64_t q_rank, kv_rank, window;   /* window <= 0: every earlier token is visible */
    const void *w_down_in;  /* [q_rank + kv_rank (+ width with a gated residual), width]: query latent, key/value latent, residual gate */
    const float *dq_norm, *dkv_norm, *sink;
    const void *w_uq, *w_uk, *w_uv;    /* [H dim, q_rank], [H dim, kv_rank], [H vdim, kv_rank] */
    void *latent_cache;     /* [num_blocks * block_size, kv_rank] */
    /* gated residuals: bias of the gate, NULL = the sublayer's result is added as it is */
    const float *gate1_bias, *gate2_bias;
    /* mixture of experts (ff_kind = ATOMA_FF_MOE): ff above = the shared expert's size (0: none) */
    int32_t ff_kind, renormalize;
    int64_t experts, top, expert_ff;
    float expert_limit, shared_limit, act_alpha, act_up_shift;
    const float *w_router;  /* [experts, width] float32 */
    const float *w_shared_gate; /* [width] float32 or NULL */
    const void *w_expert_gate_up, *w_expert_down;
    const void *w_ff_in;    /* [2 ff (+ width with a gated residual), width]: shared gate rows, up rows, residual gate */
    /* token side input after the feed-forward (side_gate NULL: none) */
    int64_t side_part;
    const void *side_gate, *side_proj; /* [side_dim, width], [width, side_dim] */
    const float *side_norm;
    /* ---- blocks on residual lanes (model.block_style = ATOMA_BLOCK_LANES) ---- */
    /* softmax attention (uses heads, kv_heads, dim, vdim, scale, window, q_norm / k_norm [dim], k_cache, v_cache, w_o above;
     * w_qkv = the stacked projections [H dim queries | G dim keys | G vdim values unless values_are_keys | H vdim gate if out_gate]) */
    int64_t keep_first, dist_rows;
    const float *dist_bias; /* [dist_rows, heads] or NULL */
    int32_t values_are_keys, out_gate;
    /* lane weights of the mixer (1) and the feed-forward (2): read [lanes], write [lanes], mix [lanes, lanes] as [from, to] */
    const float *lanes_in1, *lanes_out1, *lanes_mix1, *lanes_in2, *lanes_out2, *lanes_mix2;
    /* feed-forward biases (dense kind; NULL: none) and what the router adds */
    const float *b_gate_up, *b_down; /* [2 ff], [width] */
    const float *router_correction;  /* [experts + identity_experts] or NULL */
    int64_t route_groups, route_keep, identity_experts;
    int32_t score_fn, scale_input;   /* ATOMA_SCORE_*; 1: the router's weight scales the expert's input, 0: its output */
    /* ---- parallel blocks (model.block_style = ATOMA_BLOCK_PARALLEL): x += mixer(f1(h)) + ff(f2(h)), h = norm1(x) ---- */
    /* what precedes the layer: the embedding rows and / or a vector added to the stream (the start of a pass over a looped span) */
    int32_t add_embedding;
    const float *add_vec;            /* [width] or NULL */
    /* tap filters of the two sublayers' inputs (taps <= 0: none); the layer's state row = [input history | mixer state] */
    int64_t taps;
    const float *tap_w1, *tap_w2;    /* [width, taps] */
    float *layer_state;              /* [slots, layer_state_stride] float32 */
    int64_t layer_state_stride;
    /* stacked projection of the mixer: w_qkv [proj_cols, width]; columns of its parts (-1: absent) */
    int64_t proj_cols;
    /* gated linear attention (heads, dim, vdim): q, k, v, g columns, the decay's low-rank projection (w_a1 [a_rank, width] as
     * columns a_off .. of the stacked projection, w_a2 [heads dim, a_rank], bias), head norm weight, tau */
    int64_t q_off, k_off, v_off, g_off, a_off, a_rank;
    const void *w_a2;
    const float *a2_bias, *head_norm;
    float tau;
    /* pair of mixers: left = sigmoid attention with rotary positions (heads, kv_heads, dim, vdim, scale, q_norm, k_norm, head_bias,
     * k_cache, v_cache, w_o above), right = gated delta rule */
    const float *qk_freq, *v_freq;   /* [rot_pairs], [v_pairs] float32 */
    int64_t rot_pairs, v_pairs;
    int32_t rot_interleaved;
    int64_t r_heads, r_kv_heads, r_dim, r_vdim, r_taps;
    int64_t rq_off, rk_off, rv_off, rg_off, rb_off, ra_off;
    const float *r_tap_w;            /* [2 r_kv_heads r_dim + r_heads r_vdim, r_taps] */
    const float *r_a_log, *r_dt_bias, *r_head_norm;
    const void *r_w_o;               /* [width, r_heads r_vdim] */
    const float *out_norm_a, *out_norm_b; /* [width] */
    /* latent attention with a rotated key part (q_rank, kv_rank, dq_norm, dkv_norm, w_uq [heads (dim + rot_dim), q_rank], w_uk, w_uv,
     * latent_cache rows of kv_rank + rot_dim; qk_freq / rot_pairs / rot_interleaved above) */
    int64_t rot_dim;
} atoma_hybrid_layer;

typedef struct atoma_hybrid_model {
    int64_t width, vocab, num_layers, block_size;
    float eps, logit_scale, norm_offset;
    uint32_t dtype;
    const void *embed;      /* [vocab, width] */
    const double *inv_freq; /* [ceil(width / 2)] */
    const float *final_norm;
    const void *head;       /* [vocab, width] */
    const atoma_hybrid_layer *layers; /* host array */
    /* ---- pre-norm designs ---- */
    int32_t block_style;    /* ATOMA_BLOCK_* */
    int32_t norm_groups;    /* 0 or 1: whole-row norms */
    const void *pos_table;  /* [max_positions, width] learned positions (then inv_freq may be NULL) */
    int64_t max_positions;
    float logit_softcap;    /* <= 0: none */
    const void *side_table; /* [vocab, side_table_width] */
    int64_t side_dim, side_table_width;
    /* ---- designs on residual lanes ---- */
    int32_t lanes;          /* copies of the residual stream (ATOMA_BLOCK_LANES: >= 1) */
    float embed_scale;      /* the embedding row times this; no position signal is added */
} atoma_hybrid_model;

typedef struct atoma_hybrid_batch {
    int64_t num_tokens, num_seqs, num_selected, max_blocks;
    int32_t max_query_len, max_seq_len;
    const uint32_t *tokens;       /* [T] */
    const int64_t *positions;     /* [T] */
    const int64_t *slot_mapping;  /* [T] */
    const int32_t *token_seq;     /* [T] */
    const int32_t *query_start;   /* [B + 1] */
    const int32_t *context_lens;  /* [B] tokens already in the cache / state */
    const int32_t *block_tables;  /* [B, max_blocks] */
    const int32_t *state_slots;   /* [B] */
    const int32_t *selected;      /* [num_selected] token rows whose logits are wanted */
    void *scratch;
    int64_t scratch_bytes;
    float *logits;                /* out [num_selected, vocab] */
    uint32_t *next_tokens;        /* out [num_selected] greedy */
    float *residual_trace;        /* optional out [num_layers, T, width]: the residual stream (the sum of the lanes) after every layer */
    /* long prompt portions (pre-norm designs; all zero = none): sequences with at least long_min_q tokens in the step, how many
     * there are, the sum of their tokens and of their contexts (tokens already cached) */
    int32_t long_seqs, long_min_q;
    int64_t long_tokens, long_ctx_sum;
} atoma_hybrid_batch;

int64_t atoma_hybrid_abi_sizeof(int which); /* 0 layer, 1 model, 2 batch, 3 attention args, 4 gated residual args, 5 latent attention args, 6 expert args, 7 expanded attention args, 8 lanes update args, 9 softmax attention args, 10 parallel residual args, 11 tap filter args, 12 state scan args, 13 rotary cache args */
int64_t atoma_hybrid_scratch_bytes(const atoma_hybrid_model *model, int64_t num_tokens, int64_t num_selected);
void atoma_hybrid_step(const atoma_hybrid_model *model, const atoma_hybrid_batch *batch, atoma_stream_t stream);

/* Diagnostics: bit 0 = every projection through the plain float32-FMA kernel; bit 1 = the general attention kernel
 * for every batch (no tensor-core prefill / split decode kernels); bit 2 = the sequential minGRU scan; bit 3 = the routed
 * experts' tensor-memory (tcgen05) products for steps of any size (they normally serve steps of 1024 pairs and more);
 * bit 4 = the matrix-state scans with many rows per lane whatever the step's size (they normally take 8 rows per lane when a
 * step has few CTAs; both add in the same order). */
void atoma_debug_hybrid(int flags);

#ifdef __cplusplus
}
#endif
#endif /* ATOMA_HYBRID_H_ */
