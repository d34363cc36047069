// Step executor for hybrid (attention + recurrent) models on a mixed batch — include/atoma_hybrid.h.
//
// One call enqueues the whole forward pass of the step's tokens on one stream, without host
// synchronisation: embedding + position signal, then per layer
//   attention: fused q/k/v projection -> q/k norm + temperature + cache write -> paged sigmoid attention -> o
//   minGRU:    fused z/x/g projection -> scan over each sequence's tokens from its state slot -> o
//   x += norm(mixer out) fused with the next sublayer's input norm; the gated feed-forward likewise;
// and at the end the wanted rows only: final norm, head, logit scale and the greedy choice.
// Keys, values and recurrent state left by earlier steps are read from / written to the paged caches and
// the state slots the batch names; nothing else survives the call.
#include "common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>
#include <nvtx3/nvToolsExt.h>

namespace atoma {

bool hyb_embed_sinusoid(const uint32_t *, const int64_t *, const void *, const double *, float *, int64_t, int64_t, int64_t, uint32_t,
                        cudaStream_t);
bool hyb_rmsnorm_rows(const float *, const int32_t *, const float *, float, void *, int64_t, int64_t, float, uint32_t, cudaStream_t);
bool hyb_postnorm_add_prenorm(const void *, float *, const float *, const float *, void *, int64_t, int64_t, float, float, uint32_t,
                              cudaStream_t);
bool hyb_qk_norm_cache(const void *, const float *, const float *, const float *, const int64_t *, const int64_t *, void *, void *,
                       void *, int64_t, int64_t, int64_t, int64_t, int64_t, float, float, int64_t, uint32_t, cudaStream_t);
bool hyb_attention(const atoma_sigmoid_attn_args &, cudaStream_t);
bool hyb_mingru_scan(const void *, const float *, float *, const int32_t *, const int32_t *, const int32_t *, void *, int64_t, int64_t,
                     int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_glu(const void *, void *, int64_t, int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_gate_up_act(const void *, const void *, void *, void *, int64_t, int64_t, int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_linear(const void *, const void *, void *, int64_t, int64_t, int64_t, uint32_t, cudaStream_t);
bool hyb_scale_greedy(const void *, float *, uint32_t *, int64_t, int64_t, float, float, uint32_t, cudaStream_t);
bool hyb_embed_learned(const uint32_t *, const int64_t *, const void *, const void *, float *, int64_t, int64_t, int64_t, int64_t, uint32_t,
                       cudaStream_t);
bool hyb_group_rmsnorm_rows(const float *, const int32_t *, const float *, float, int64_t, void *, int64_t, int64_t, float, uint32_t,
                            cudaStream_t);
bool hyb_gated_residual_norm(const atoma_gated_residual_args &, cudaStream_t);
bool hyb_side_gate(const void *, int64_t, const uint32_t *, const void *, int64_t, int64_t, void *, int64_t, int64_t, int64_t, uint32_t,
                   cudaStream_t);
bool hyb_unitnorm_add_norm(const void *, float *, const float *, const float *, void *, int64_t, int64_t, int64_t, float, float, uint32_t,
                           cudaStream_t);
bool hyb_glu_clamped(const void *, int64_t, void *, int64_t, int64_t, float, float, float, uint32_t, cudaStream_t);
bool hyb_latent_norm_cache(const void *, int64_t, const float *, const float *, const int64_t *, void *, void *, int64_t, int64_t, int64_t,
                           float, uint32_t, cudaStream_t);
bool hyb_head_project(const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int32_t, uint32_t, cudaStream_t);
bool hyb_latent_attention(const atoma_latent_attn_args &, cudaStream_t);
bool hyb_latent_expanded_ok(int64_t, int64_t, int64_t, uint32_t);
bool hyb_latent_attention_expanded(const atoma_latent_expanded_args &, cudaStream_t);
bool hyb_moe_route(const void *, const float *, const float *, int32_t *, float *, float *, int64_t, int64_t, int64_t, int64_t, int32_t,
                   uint32_t, cudaStream_t);
bool hyb_moe_route_grouped(const void *, const float *, const float *, int32_t *, float *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                           int32_t, int32_t, uint32_t, cudaStream_t);
bool hyb_embed_scaled_lanes(const uint32_t *, const void *, float, float *, int64_t, int64_t, int64_t, int64_t, uint32_t, cudaStream_t);
bool hyb_lanes_read_norm(const float *, const float *, const int32_t *, const float *, float, void *, float *, int64_t, int64_t, int64_t, float,
                         uint32_t, cudaStream_t);
bool hyb_lanes_update_norm(const atoma_lanes_update_args &, cudaStream_t);
bool hyb_qk_headnorm_cache(const void *, int64_t, int64_t, int64_t, int64_t, const float *, const float *, float, const int64_t *, void *, void *,
                           void *, int64_t, int64_t, int64_t, int64_t, int64_t, float, uint32_t, cudaStream_t);
bool hyb_softmax_attention(const atoma_softmax_attn_args &, cudaStream_t);
bool hyb_glu_clamped_bias(const void *, int64_t, const float *, void *, int64_t, int64_t, float, float, float, uint32_t, cudaStream_t);
bool hyb_gate_up_clamped(const void *, const void *, const float *, void *, void *, int64_t, int64_t, int64_t, float, float, float, uint32_t,
                         cudaStream_t);
bool hyb_parallel_residual_norm(const atoma_parallel_residual_args &, cudaStream_t);
bool hyb_tap_filter(const atoma_tap_filter_args &, cudaStream_t);
bool hyb_state_scan(const atoma_state_scan_args &, cudaStream_t);
bool hyb_headnorm_gate(const float *, const float *, const void *, int64_t, void *, int64_t, int64_t, int64_t, float, uint32_t, cudaStream_t);
bool hyb_qkv_headnorm_rope_cache(const atoma_qkv_rope_args &, cudaStream_t);
bool hyb_rotate_heads(void *, const int64_t *, const float *, int64_t, int64_t, int64_t, int64_t, int32_t, float, uint32_t, cudaStream_t);
bool hyb_latent_norm_rope_cache(const void *, int64_t, const float *, const float *, const float *, int64_t, int32_t, const int64_t *,
                                const int64_t *, void *, void *, int64_t, int64_t, int64_t, int64_t, float, uint32_t, cudaStream_t);
bool hyb_latent_query_absorb_rope(const void *, const void *, const float *, int64_t, int32_t, const int64_t *, float *, int64_t, int64_t, int64_t,
                                  int64_t, int64_t, uint32_t, cudaStream_t);
bool hyb_latent_expand_values(const float *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, uint32_t, cudaStream_t);
int64_t hyb_moe_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int64_t, uint32_t);
bool hyb_moe_experts(const atoma_moe_args &, const void **, const int32_t **, cudaStream_t);

namespace {

inline int64_t up256(int64_t x) { return (x + 255) / 256 * 256; }

struct Widths {
    int64_t proj = 0, q = 0, act = 0;   // widest projection output, query row, mixer / feed-forward activation row
    int64_t cq = 0, lat = 0, route = 0, side = 0;   // query latent row, heads x latent row, router outputs per token, side input row
    int64_t moe = 0;                    // bytes of the routed experts' workspace
    int64_t conv = 0, of32 = 0;         // parallel blocks: filtered q / k / v row of a delta-rule mixer, float32 read-out row of a recurrence
    bool parallel = false, keep_embedding = false;
};

inline bool gated(const float *bias) { return bias != nullptr; }

// columns of the stacked projection of a softmax-attention layer: queries, keys, values (unless they are the keys), output gate
inline int64_t softmax_proj_cols(const atoma_hybrid_layer &l) {
    return l.heads * l.dim + l.kv_heads * l.dim + (l.values_are_keys ? 0 : l.kv_heads * l.vdim) + (l.out_gate ? l.heads * l.vdim : 0);
}

Widths widths(const atoma_hybrid_model &m, int64_t T) {
    Widths w;
    for (int64_t i = 0; i < m.num_layers; ++i) {
        const atoma_hybrid_layer &l = m.layers[i];
        if (m.block_style == ATOMA_BLOCK_PARALLEL) {
            w.parallel = true;
            w.keep_embedding = w.keep_embedding || l.add_embedding;
            w.proj = std::max(w.proj, l.proj_cols);
            if (l.has_mlp) {
                w.proj = std::max(w.proj, 2 * l.ff);
                w.act = std::max(w.act, l.ff);
            }
            if (l.mixer == ATOMA_MIXER_GLA) {
                w.q = std::max(w.q, l.heads * l.dim);
                w.cq = std::max(w.cq, l.a_rank);
                w.act = std::max(w.act, l.heads * l.vdim);
                w.of32 = std::max(w.of32, l.heads * l.vdim);
            } else if (l.mixer == ATOMA_MIXER_LATENT_ATTENTION) {
                w.q = std::max(w.q, l.heads * (l.dim + l.rot_dim));
                w.cq = std::max(w.cq, l.q_rank);
                w.act = std::max(w.act, l.heads * l.vdim);
                w.lat = std::max(w.lat, l.heads * (l.kv_rank + l.rot_dim));
            } else if (l.mixer == ATOMA_MIXER_PAIR) {
                w.q = std::max(w.q, l.heads * l.dim);
                w.act = std::max(w.act, std::max(l.heads * l.vdim, l.r_heads * l.r_vdim));
                w.conv = std::max(w.conv, 2 * l.r_kv_heads * l.r_dim + l.r_heads * l.r_vdim);
                w.of32 = std::max(w.of32, l.r_heads * l.r_vdim);
            }
            continue;
        }
        if (l.mixer == ATOMA_MIXER_LATENT_ATTENTION) {
            w.proj = std::max(w.proj, l.q_rank + l.kv_rank + (gated(l.gate1_bias) ? m.width : 0));
            w.q = std::max(w.q, l.heads * l.dim);
            w.act = std::max(w.act, l.heads * l.vdim);
            w.cq = std::max(w.cq, l.q_rank);
            w.lat = std::max(w.lat, l.heads * l.kv_rank);
            if (l.has_mlp) {
                w.proj = std::max(w.proj, 2 * l.ff + (gated(l.gate2_bias) ? m.width : 0));
                w.act = std::max(w.act, l.ff);
                if (l.ff_kind == ATOMA_FF_MOE) {
                    w.route = std::max(w.route, l.top);
                    w.moe = std::max(w.moe, hyb_moe_workspace_bytes(T, l.top, l.experts, m.width, l.expert_ff, m.dtype));
                }
            }
            if (l.side_gate) w.side = std::max(w.side, m.side_dim);
            continue;
        }
        if (l.mixer == ATOMA_MIXER_SOFTMAX_ATTENTION) {
            w.proj = std::max(w.proj, softmax_proj_cols(l));
            w.q = std::max(w.q, l.heads * l.dim);
            w.act = std::max(w.act, l.heads * l.vdim);
            if (l.has_mlp) {
                w.act = std::max(w.act, l.ff);
                w.proj = std::max(w.proj, 2 * l.ff);
                if (l.ff_kind == ATOMA_FF_MOE) {
                    w.route = std::max(w.route, l.top);
                    w.moe = std::max(w.moe, hyb_moe_workspace_bytes(T, l.top, l.experts, m.width, l.expert_ff, m.dtype));
                }
            }
            continue;
        }
        if (l.mixer == ATOMA_MIXER_SIGMOID_ATTENTION) {
            w.proj = std::max(w.proj, (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim);
            w.q = std::max(w.q, l.heads * l.dim);
            w.act = std::max(w.act, l.heads * l.vdim);
        } else {
            w.proj = std::max(w.proj, 3 * l.state_width);
            w.act = std::max(w.act, l.state_width);
        }
        if (l.has_mlp) {
            w.proj = std::max(w.proj, 2 * l.ff);
            w.act = std::max(w.act, l.ff);
        }
    }
    return w;
}

struct Scratch {
    float *x;
    char *h, *proj, *q, *act, *y, *hs, *lg;
    // pre-norm designs
    char *cq, *xc, *side_a, *side_g, *moe;
    float *qlat, *olat, *top_weight, *row_gate;
    int32_t *top_expert;
    int64_t moe_bytes;
    // parallel blocks
    float *x0, *of32;
    char *h1, *h2, *y2, *yf, *conv;
    int64_t total;
};

Scratch carve(const atoma_hybrid_model &m, int64_t T, int64_t S, void *base) {
    const int64_t es = m.dtype == ATOMA_DTYPE_F32 ? 4 : 2;
    const Widths w = widths(m, T);
    Scratch s{};
    int64_t off = 0;
    char *b = static_cast<char *>(base);
    auto take = [&](int64_t bytes) {
        char *p = b ? b + off : nullptr;
        off += up256(bytes);
        return p;
    };
    s.x = reinterpret_cast<float *>(take(T * std::max<int64_t>(1, m.lanes) * m.width * 4));
    s.h = take(T * m.width * es);
    s.proj = take(T * w.proj * es);
    s.q = take(T * w.q * es);
    s.act = take(T * w.act * es);
    s.y = take(T * m.width * es);
    s.hs = take(S * m.width * es);
    s.lg = take(S * m.vocab * es);
    s.cq = take(T * w.cq * es);
    s.qlat = reinterpret_cast<float *>(take(T * w.lat * 4));
    s.olat = reinterpret_cast<float *>(take(T * w.lat * 4));
    s.top_expert = reinterpret_cast<int32_t *>(take(T * w.route * 4));
    s.top_weight = reinterpret_cast<float *>(take(T * w.route * 4));
    s.row_gate = reinterpret_cast<float *>(take(T * 4));
    s.xc = take(w.side ? T * m.width * es : 0);
    s.side_a = take(T * w.side * es);
    s.side_g = take(T * w.side * es);
    s.moe = take(w.moe);
    s.moe_bytes = w.moe;
    s.x0 = reinterpret_cast<float *>(take(w.keep_embedding ? T * m.width * 4 : 0));
    s.of32 = reinterpret_cast<float *>(take(T * w.of32 * 4));
    s.h1 = take(w.parallel ? T * m.width * es : 0);
    s.h2 = take(w.parallel ? T * m.width * es : 0);
    s.y2 = take(w.parallel ? T * m.width * es : 0);
    s.yf = take(w.parallel ? T * m.width * es : 0);
    s.conv = take(T * w.conv * es);
    s.total = off;
    return s;
}

// One layer of a pre-norm design: x += gate1 * mixer(norm1 x); x += gate2 * ff(norm2 x); x += unit-normed side input.
// s.h holds norm1(x) on entry and the next layer's norm1(x) (next_norm, may be NULL) on return.
bool prenorm_layer(const atoma_hybrid_model &m, const atoma_hybrid_batch &b, const atoma_hybrid_layer &l, const Scratch &s,
                   const float *next_norm, cudaStream_t stream) {
    const uint32_t dt = m.dtype;
    const int64_t es = dt == ATOMA_DTYPE_F32 ? 4 : 2;
    const int64_t T = b.num_tokens, W = m.width;
    const int64_t groups = m.norm_groups > 0 ? m.norm_groups : 1;
    const float off = m.norm_offset;
    if (l.mixer != ATOMA_MIXER_LATENT_ATTENTION) {
        set_status(kErrUnsupported, "atoma_hybrid_step: pre-norm layers take the latent-attention mixer, got %d", l.mixer);
        return false;
    }
    // ---- mixer: one product makes the query latent, the key/value latent and the residual gate ----
    const int64_t n_in = l.q_rank + l.kv_rank + (gated(l.gate1_bias) ? W : 0);
    if (!hyb_linear(s.h, l.w_down_in, s.proj, T, n_in, W, dt, stream)) return false;
    if (!hyb_latent_norm_cache(s.proj, n_in, l.dq_norm, l.dkv_norm, b.slot_mapping, s.cq, l.latent_cache, T, l.q_rank, l.kv_rank, m.eps, dt,
                               stream))
        return false;
    if (!hyb_linear(s.cq, l.w_uq, s.q, T, l.heads * l.dim, l.q_rank, dt, stream)) return false;
    // long prompt portions run on expanded keys and values (4x fewer multiply-adds per pair at usual sizes); decoded tokens and
    // short portions run in the latent space (the cache is read once for all heads)
    const bool expanded = b.long_seqs > 0 && b.long_min_q >= 32 && hyb_latent_expanded_ok(l.dim, l.vdim, l.kv_rank, dt);
    const bool latent_too = !expanded || b.long_seqs < b.num_seqs;
    if (latent_too && !hyb_head_project(s.q, l.w_uk, s.qlat, T, l.heads, l.dim, l.kv_rank, 1, dt, stream)) return false;
    atoma_latent_attn_args a{};
    a.q_lat = s.qlat;
    a.latent_cache = l.latent_cache;
    a.out = s.olat;
    a.positions = b.positions;
    a.token_seq = b.token_seq;
    a.query_start = b.query_start;
    a.block_tables = b.block_tables;
    a.sink = l.sink;
    a.T = T;
    a.B = b.num_seqs;
    a.max_blocks = b.max_blocks;
    a.H = l.heads;
    a.R = l.kv_rank;
    a.block_size = m.block_size;
    a.window = l.window;
    a.scale = l.scale;
    a.dtype = dt;
    a.max_query_len = b.max_query_len;
    a.max_seq_len = b.max_seq_len;
    a.skip_min_q = expanded ? b.long_min_q : 0;
    if (latent_too) {
        if (!hyb_latent_attention(a, stream)) return false;
        if (!hyb_head_project(s.olat, l.w_uv, s.act, T, l.heads, l.vdim, l.kv_rank, 0, dt, stream)) return false;
    }
    if (expanded) {   // after the latent path: it rewrites the long sequences' rows of s.act
        atoma_latent_expanded_args e{};
        e.q = s.q;
        e.latent_cache = l.latent_cache;
        e.w_uk = l.w_uk;
        e.w_uv = l.w_uv;
        e.out = s.act;
        e.query_start = b.query_start;
        e.context_lens = b.context_lens;
        e.block_tables = b.block_tables;
        e.sink = l.sink;
        e.T = T;
        e.B = b.num_seqs;
        e.max_blocks = b.max_blocks;
        e.H = l.heads;
        e.dim = l.dim;
        e.R = l.kv_rank;
        e.block_size = m.block_size;
        e.window = l.window;
        e.max_keys = b.long_tokens + (l.window > 0 ? std::min<int64_t>(b.long_ctx_sum, static_cast<int64_t>(b.long_seqs) * (l.window - 1))
                                                   : b.long_ctx_sum);
        e.scale = l.scale;
        e.min_q = b.long_min_q;
        e.max_query_len = b.max_query_len;
        e.max_seq_len = b.max_seq_len;
        if (!hyb_latent_attention_expanded(e, stream)) return false;
    }
    if (!hyb_linear(s.act, l.w_o, s.y, T, W, l.heads * l.vdim, dt, stream)) return false;
    const bool side = l.side_gate != nullptr;
    atoma_gated_residual_args r{};
    r.y = s.y;
    r.ld_y = W;
    r.gate = gated(l.gate1_bias) ? s.proj + (l.q_rank + l.kv_rank) * es : nullptr;
    r.ld_gate = n_in;
    r.gate_bias = l.gate1_bias;
    r.x = s.x;
    r.w_next = l.has_mlp ? l.norm2 : (side ? nullptr : next_norm);
    r.h = s.h;
    r.x_cast = (!l.has_mlp && side) ? s.xc : nullptr;
    r.T = T;
    r.width = W;
    r.groups = groups;
    r.eps = m.eps;
    r.weight_offset = off;
    r.dtype = dt;
    if (!hyb_gated_residual_norm(r, stream)) return false;
    // ---- feed-forward ----
    if (l.has_mlp) {
        atoma_gated_residual_args f{};
        const int64_t n_ff = 2 * l.ff + (gated(l.gate2_bias) ? W : 0);
        if (n_ff > 0 && !hyb_linear(s.h, l.w_ff_in, s.proj, T, n_ff, W, dt, stream)) return false;
        if (l.ff > 0) {   // the dense (or shared) expert
            const float limit = l.ff_kind == ATOMA_FF_MOE ? l.shared_limit : l.expert_limit;
            if (!hyb_glu_clamped(s.proj, n_ff, s.act, T, l.ff, limit, l.act_alpha, l.act_up_shift, dt, stream)) return false;
            if (!hyb_linear(s.act, l.w_down, s.y, T, W, l.ff, dt, stream)) return false;
            f.y = s.y;
            f.ld_y = W;
        }
        if (l.ff_kind == ATOMA_FF_MOE) {
            const bool row_gate = l.ff > 0 && l.w_shared_gate;
            if (!hyb_moe_route(s.h, l.w_router, row_gate ? l.w_shared_gate : nullptr, s.top_expert, s.top_weight, s.row_gate, T, W,
                               l.experts, l.top, l.renormalize, dt, stream))
                return false;
            atoma_moe_args e{};
            e.h = s.h;
            e.top_expert = s.top_expert;
            e.top_weight = s.top_weight;
            e.w_gate_up = l.w_expert_gate_up;
            e.w_down = l.w_expert_down;
            e.workspace = s.moe;
            e.workspace_bytes = s.moe_bytes;
            e.T = T;
            e.width = W;
            e.experts = l.experts;
            e.top = l.top;
            e.ff = l.expert_ff;
            e.limit = l.expert_limit;
            e.alpha = l.act_alpha;
            e.up_shift = l.act_up_shift;
            e.scale_input = 1;
            e.dtype = dt;
            const void *eo = nullptr;
            const int32_t *pr = nullptr;
            if (!hyb_moe_experts(e, &eo, &pr, stream)) return false;
            f.expert_out = eo;
            f.pair_row = pr;
            f.top = l.top;
            if (row_gate) f.row_scale = s.row_gate;
        }
        f.gate = gated(l.gate2_bias) ? s.proj + 2 * l.ff * es : nullptr;
        f.ld_gate = n_ff;
        f.gate_bias = l.gate2_bias;
        f.x = s.x;
        f.w_next = side ? nullptr : next_norm;
        f.h = s.h;
        f.x_cast = side ? s.xc : nullptr;
        f.T = T;
        f.width = W;
        f.groups = groups;
        f.eps = m.eps;
        f.weight_offset = off;
        f.dtype = dt;
        if (!hyb_gated_residual_norm(f, stream)) return false;
    }
    // ---- token side input ----
    if (side) {
        const int64_t D = m.side_dim;
        if (!m.side_table || D <= 0 || !l.side_proj || !l.side_norm) {
            set_status(kErrInvalidArg, "atoma_hybrid_step: a layer has a side input but the model has no side table");
            return false;
        }
        if (!hyb_linear(s.xc, l.side_gate, s.side_a, T, D, W, dt, stream)) return false;
        if (!hyb_side_gate(s.side_a, D, b.tokens, m.side_table, m.side_table_width, l.side_part, s.side_g, T, D, m.vocab, dt, stream))
            return false;
        if (!hyb_linear(s.side_g, l.side_proj, s.y, T, W, D, dt, stream)) return false;
        if (!hyb_unitnorm_add_norm(s.y, s.x, l.side_norm, next_norm, s.h, T, W, groups, m.eps, off, dt, stream)) return false;
    }
    return true;
}

// One layer of a design on residual lanes: the mixer reads sum_s in1[s] x_s and writes back through mix1 / out1, the
// feed-forward likewise with in2 / mix2 / out2.  s.h holds the mixer's normed input on entry and the next layer's (next_in /
// next_norm, may be NULL) on return; lane_sum (may be NULL) receives the sum of the lanes after the layer.
bool lanes_layer(const atoma_hybrid_model &m, const atoma_hybrid_batch &b, const atoma_hybrid_layer &l, const Scratch &s,
                 const float *next_in, const float *next_norm, float *lane_sum, cudaStream_t stream) {
    const uint32_t dt = m.dtype;
    const int64_t es = dt == ATOMA_DTYPE_F32 ? 4 : 2;
    const int64_t T = b.num_tokens, W = m.width;
    if (l.mixer != ATOMA_MIXER_SOFTMAX_ATTENTION) {
        set_status(kErrUnsupported, "atoma_hybrid_step: layers on residual lanes take the softmax-attention mixer, got %d", l.mixer);
        return false;
    }
    if (!l.lanes_in1 || !l.lanes_out1 || !l.lanes_mix1 || (l.has_mlp && (!l.lanes_in2 || !l.lanes_out2 || !l.lanes_mix2))) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: a layer on residual lanes has no lane weights");
        return false;
    }
    // ---- mixer: one product makes the queries, the keys (whose raw form is the values), and the output gate ----
    const int64_t n_in = softmax_proj_cols(l);
    const int64_t k_off = l.heads * l.dim;
    const int64_t v_off = l.values_are_keys ? k_off : k_off + l.kv_heads * l.dim;
    const int64_t g_off = v_off + (l.values_are_keys ? l.kv_heads * l.dim : l.kv_heads * l.vdim);
    if (l.values_are_keys && l.vdim != l.dim) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: values that are the key projections need vdim = dim");
        return false;
    }
    if (!hyb_linear(s.h, l.w_qkv, s.proj, T, n_in, W, dt, stream)) return false;
    if (!hyb_qk_headnorm_cache(s.proj, n_in, 0, k_off, v_off, l.q_norm, l.k_norm, m.norm_offset, b.slot_mapping, s.q, l.k_cache, l.v_cache, T,
                               l.heads, l.kv_heads, l.dim, l.vdim, m.eps, dt, stream))
        return false;
    atoma_softmax_attn_args a{};
    a.q = s.q;
    a.k_cache = l.k_cache;
    a.v_cache = l.v_cache;
    a.out = s.act;
    a.gate = l.out_gate ? s.proj + g_off * es : nullptr;
    a.ld_gate = n_in;
    a.dist_bias = l.dist_bias;
    a.dist_rows = l.dist_rows;
    a.positions = b.positions;
    a.token_seq = b.token_seq;
    a.query_start = b.query_start;
    a.block_tables = b.block_tables;
    a.T = T;
    a.B = b.num_seqs;
    a.max_blocks = b.max_blocks;
    a.H = l.heads;
    a.G = l.kv_heads;
    a.dim = l.dim;
    a.vdim = l.vdim;
    a.block_size = m.block_size;
    a.window = l.window;
    a.keep_first = l.keep_first;
    a.scale = l.scale;
    a.dtype = dt;
    a.max_query_len = b.max_query_len;
    a.max_seq_len = b.max_seq_len;
    a.long_min_q = b.long_min_q;
    a.long_seqs = b.long_seqs;
    a.long_tokens = b.long_tokens;
    a.long_ctx_sum = b.long_ctx_sum;
    if (!hyb_softmax_attention(a, stream)) return false;
    if (!hyb_linear(s.act, l.w_o, s.y, T, W, l.heads * l.vdim, dt, stream)) return false;
    atoma_lanes_update_args u{};
    u.y = s.y;
    u.x = s.x;
    u.w_mix = l.lanes_mix1;
    u.w_out = l.lanes_out1;
    u.w_in_next = l.has_mlp ? l.lanes_in2 : next_in;
    u.w_next = l.has_mlp ? l.norm2 : next_norm;
    u.h = s.h;
    u.lane_sum = l.has_mlp ? nullptr : lane_sum;
    u.T = T;
    u.lanes = m.lanes;
    u.width = W;
    u.eps = m.eps;
    u.weight_offset = m.norm_offset;
    u.dtype = dt;
    if (!hyb_lanes_update_norm(u, stream)) return false;
    if (!l.has_mlp) return true;
    // ---- feed-forward ----
    atoma_lanes_update_args f = u;
    f.y = nullptr;
    f.w_mix = l.lanes_mix2;
    f.w_out = l.lanes_out2;
    f.w_in_next = next_in;
    f.w_next = next_norm;
    f.lane_sum = lane_sum;
    if (l.ff > 0) {   // the dense feed-forward, or the shared expert of a mixture
        const bool moe = l.ff_kind == ATOMA_FF_MOE;
        if (!hyb_gate_up_clamped(s.h, moe ? l.w_ff_in : l.w_gate_up, moe ? nullptr : l.b_gate_up, s.proj, s.act, T, l.ff, W,
                                 moe ? l.shared_limit : l.expert_limit, l.act_alpha, l.act_up_shift, dt, stream))
            return false;
        if (!hyb_linear(s.act, l.w_down, s.y, T, W, l.ff, dt, stream)) return false;
        f.y = s.y;
        f.y_bias = moe ? nullptr : l.b_down;
    }
    if (l.ff_kind == ATOMA_FF_MOE) {
        const int64_t outputs = l.experts + l.identity_experts;
        if (!hyb_moe_route_grouped(s.h, l.w_router, l.router_correction, s.top_expert, s.top_weight, T, W, outputs, l.top, l.route_groups,
                                   l.route_keep, l.score_fn, l.renormalize, dt, stream))
            return false;
        atoma_moe_args e{};
        e.h = s.h;
        e.top_expert = s.top_expert;
        e.top_weight = s.top_weight;
        e.w_gate_up = l.w_expert_gate_up;
        e.w_down = l.w_expert_down;
        e.workspace = s.moe;
        e.workspace_bytes = s.moe_bytes;
        e.T = T;
        e.width = W;
        e.experts = l.experts;
        e.top = l.top;
        e.ff = l.expert_ff;
        e.limit = l.expert_limit;
        e.alpha = l.act_alpha;   // alpha 1, shift 0, no limit: silu(gate) * up
        e.up_shift = l.act_up_shift;
        e.scale_input = l.scale_input;
        e.dtype = dt;
        const void *eo = nullptr;
        const int32_t *pr = nullptr;
        if (!hyb_moe_experts(e, &eo, &pr, stream)) return false;
        f.expert_out = eo;
        f.pair_row = pr;
        f.top_expert = s.top_expert;
        f.top_weight = s.top_weight;
        f.h_in = s.h;
        f.top = l.top;
        f.experts = l.experts;
    }
    return hyb_lanes_update_norm(f, stream);
}

// One layer of a parallel design: h = norm1(x) (in s.h on entry); the mixer reads h + taps1(h), the feed-forward h + taps2(h);
// x += mixer + feed-forward, then whatever precedes the next layer (`next`, may be NULL), then its norm1 into s.h.
bool parallel_layer(const atoma_hybrid_model &m, const atoma_hybrid_batch &b, const atoma_hybrid_layer &l, const Scratch &s,
                    const atoma_hybrid_layer *next, float *trace, cudaStream_t stream) {
    const uint32_t dt = m.dtype;
    const int64_t es = dt == ATOMA_DTYPE_F32 ? 4 : 2;
    const int64_t T = b.num_tokens, W = m.width;
    if (!l.layer_state && (l.taps > 1 || l.mixer == ATOMA_MIXER_GLA || l.mixer == ATOMA_MIXER_PAIR)) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: a parallel layer with carried inputs or a recurrence has no state");
        return false;
    }
    // ---- the two sublayers' inputs ----
    const char *hm = s.h, *hf = s.h;
    const int64_t hist = l.taps > 1 ? (l.taps - 1) * W : 0;   // floats of the layer's state row that the input history takes
    if (l.taps > 0) {
        atoma_tap_filter_args f{};
        f.in = s.h;
        f.ld_in = W;
        f.w1 = l.tap_w1;
        f.w2 = l.has_mlp ? l.tap_w2 : nullptr;
        f.out1 = s.h1;
        f.out2 = l.has_mlp ? s.h2 : nullptr;
        f.ld_out = W;
        f.history = l.layer_state;
        f.history_stride = l.layer_state_stride;
        f.state_slots = b.state_slots;
        f.token_seq = b.token_seq;
        f.query_start = b.query_start;
        f.context_lens = b.context_lens;
        f.T = T;
        f.B = b.num_seqs;
        f.channels = W;
        f.taps = l.taps;
        f.residual = 1;
        f.act = 0;
        f.dtype = dt;
        if (!hyb_tap_filter(f, stream)) return false;
        hm = s.h1;
        hf = s.h2;
    }
    // ---- feed-forward ----
    if (l.has_mlp) {
        if (!hyb_gate_up_act(hf, l.w_gate_up, s.proj, s.act, T, l.ff, W, l.act, dt, stream)) return false;
        if (!hyb_linear(s.act, l.w_down, s.yf, T, W, l.ff, dt, stream)) return false;
    }
    // ---- mixer ----
    atoma_parallel_residual_args r{};
    r.mix_scale = 1.f;
    const int64_t P = l.proj_cols;
    if (!hyb_linear(hm, l.w_qkv, s.proj, T, P, W, dt, stream)) return false;
    if (l.mixer == ATOMA_MIXER_GLA) {
        const int64_t H = l.heads, D = l.dim, V = l.vdim;
        // decay pre-activation through its low-rank pair: the first product's columns are dense in s.cq
        if (!hyb_linear(hm, static_cast<const char *>(l.w_qkv) + l.a_off * W * es, s.cq, T, l.a_rank, W, dt, stream)) return false;
        if (!hyb_linear(s.cq, l.w_a2, s.q, T, H * D, l.a_rank, dt, stream)) return false;
        atoma_state_scan_args a{};
        a.kind = 0;
        a.q = s.proj + l.q_off * es;
        a.k = s.proj + l.k_off * es;
        a.v = s.proj + l.v_off * es;
        a.z = s.q;
        a.ld_q = a.ld_k = a.ld_v = P;
        a.ld_z = H * D;
        a.z_bias = l.a2_bias;
        a.tau = l.tau;
        a.q_scale = l.scale;
        a.state = l.layer_state + hist;
        a.state_stride = l.layer_state_stride;
        a.state_slots = b.state_slots;
        a.query_start = b.query_start;
        a.context_lens = b.context_lens;
        a.out = s.of32;
        a.T = T;
        a.B = b.num_seqs;
        a.H = H;
        a.G = H;
        a.dim = D;
        a.vdim = V;
        a.dtype = dt;
        if (!hyb_state_scan(a, stream)) return false;
        if (!hyb_headnorm_gate(s.of32, l.head_norm, s.proj + l.g_off * es, P, s.act, T, H, V, m.eps, dt, stream)) return false;
        if (!hyb_linear(s.act, l.w_o, s.y, T, W, H * V, dt, stream)) return false;
        r.y_a = s.y;
    } else if (l.mixer == ATOMA_MIXER_LATENT_ATTENTION) {
        const int64_t H = l.heads, row = l.kv_rank + l.rot_dim;
        if (!hyb_latent_norm_rope_cache(s.proj, P, l.dq_norm, l.dkv_norm, l.qk_freq, l.rot_pairs, l.rot_interleaved, b.positions, b.slot_mapping,
                                        s.cq, l.latent_cache, T, l.q_rank, l.kv_rank, l.rot_dim, m.eps, dt, stream))
            return false;
        if (!hyb_linear(s.cq, l.w_uq, s.q, T, H * (l.dim + l.rot_dim), l.q_rank, dt, stream)) return false;
        if (!hyb_latent_query_absorb_rope(s.q, l.w_uk, l.qk_freq, l.rot_pairs, l.rot_interleaved, b.positions, s.qlat, T, H, l.dim, l.rot_dim,
                                          l.kv_rank, dt, stream))
            return false;
        atoma_latent_attn_args a{};
        a.q_lat = s.qlat;
        a.latent_cache = l.latent_cache;
        a.out = s.olat;
        a.positions = b.positions;
        a.token_seq = b.token_seq;
        a.query_start = b.query_start;
        a.block_tables = b.block_tables;
        a.sink = l.sink;
        a.T = T;
        a.B = b.num_seqs;
        a.max_blocks = b.max_blocks;
        a.H = H;
        a.R = row;
        a.block_size = m.block_size;
        a.window = l.window;
        a.scale = l.scale;
        a.dtype = dt;
        a.max_query_len = b.max_query_len;
        a.max_seq_len = b.max_seq_len;
        a.out_cols = l.kv_rank;            // the rotated tail of a cached row takes part in the scores only
        if (!hyb_latent_attention(a, stream)) return false;
        if (!hyb_latent_expand_values(s.olat, l.w_uv, s.act, T, H, l.vdim, l.kv_rank, row, dt, stream)) return false;
        if (!hyb_linear(s.act, l.w_o, s.y, T, W, H * l.vdim, dt, stream)) return false;
        r.y_a = s.y;
    } else if (l.mixer == ATOMA_MIXER_PAIR) {
        // left: sigmoid attention with rotary positions on queries, keys and values
        atoma_qkv_rope_args q{};
        q.proj = s.proj;
        q.ld = P;
        q.q_off = l.q_off;
        q.k_off = l.k_off;
        q.v_off = l.v_off;
        q.q_weight = l.q_norm;
        q.k_weight = l.k_norm;
        q.qk_freq = l.qk_freq;
        q.v_freq = l.v_freq;
        q.rot_pairs = l.rot_pairs;
        q.v_pairs = l.v_pairs;
        q.interleaved = l.rot_interleaved;
        q.positions = b.positions;
        q.slot_mapping = b.slot_mapping;
        q.q_out = s.q;
        q.k_cache = l.k_cache;
        q.v_cache = l.v_cache;
        q.T = T;
        q.H = l.heads;
        q.G = l.kv_heads;
        q.dim = l.dim;
        q.vdim = l.vdim;
        q.eps = m.eps;
        q.dtype = dt;
        if (!hyb_qkv_headnorm_rope_cache(q, stream)) return false;
        atoma_sigmoid_attn_args a{};
        a.q = s.q;
        a.k_cache = l.k_cache;
        a.v_cache = l.v_cache;
        a.out = s.act;
        a.positions = b.positions;
        a.token_seq = b.token_seq;
        a.query_start = b.query_start;
        a.max_seq_len = b.max_seq_len;
        a.block_tables = b.block_tables;
        a.slopes = nullptr;               // no distance term, no talk between the heads: independent heads
        a.head_bias = l.head_bias;
        a.talk = nullptr;
        a.T = T;
        a.B = b.num_seqs;
        a.max_blocks = b.max_blocks;
        a.H = l.heads;
        a.G = l.kv_heads;
        a.dim = l.dim;
        a.vdim = l.vdim;
        a.block_size = m.block_size;
        a.scale = l.scale;
        a.softcap = 0.f;
        a.dtype = dt;
        a.max_query_len = b.max_query_len;
        if (!hyb_attention(a, stream)) return false;
        if (l.v_freq && !hyb_rotate_heads(s.act, b.positions, l.v_freq, T, l.heads, l.vdim, l.v_pairs, l.rot_interleaved, -1.f, dt, stream))
            return false;
        if (!hyb_linear(s.act, l.w_o, s.y, T, W, l.heads * l.vdim, dt, stream)) return false;
        // right: gated delta rule behind short filters
        const int64_t RH = l.r_heads, RG = l.r_kv_heads, RD = l.r_dim, RV = l.r_vdim;
        const int64_t C = 2 * RG * RD + RH * RV;
        atoma_tap_filter_args f{};
        f.in = s.proj + l.rq_off * es;     // q, k, v columns are neighbours in the stacked projection
        f.ld_in = P;
        f.w1 = l.r_tap_w;
        f.out1 = s.conv;
        f.ld_out = C;
        f.history = l.layer_state + hist;
        f.history_stride = l.layer_state_stride;
        f.state_slots = b.state_slots;
        f.token_seq = b.token_seq;
        f.query_start = b.query_start;
        f.context_lens = b.context_lens;
        f.T = T;
        f.B = b.num_seqs;
        f.channels = C;
        f.taps = l.r_taps;
        f.residual = 0;
        f.act = 1;
        f.dtype = dt;
        if (!hyb_tap_filter(f, stream)) return false;
        atoma_state_scan_args d{};
        d.kind = 1;
        d.q = s.conv;
        d.k = s.conv + RG * RD * es;
        d.v = s.conv + 2 * RG * RD * es;
        d.ld_q = d.ld_k = d.ld_v = C;
        d.b_pre = s.proj + l.rb_off * es;
        d.a_pre = s.proj + l.ra_off * es;
        d.ld_b = d.ld_a = P;
        d.a_log = l.r_a_log;
        d.dt_bias = l.r_dt_bias;
        d.q_scale = 1.0f / sqrtf(static_cast<float>(RD));
        d.unit_eps = 1e-6f;
        d.state = l.layer_state + hist + (l.r_taps > 1 ? (l.r_taps - 1) * C : 0);
        d.state_stride = l.layer_state_stride;
        d.state_slots = b.state_slots;
        d.query_start = b.query_start;
        d.context_lens = b.context_lens;
        d.out = s.of32;
        d.T = T;
        d.B = b.num_seqs;
        d.H = RH;
        d.G = RG;
        d.dim = RD;
        d.vdim = RV;
        d.dtype = dt;
        if (!hyb_state_scan(d, stream)) return false;
        if (!hyb_headnorm_gate(s.of32, l.r_head_norm, s.proj + l.rg_off * es, P, s.act, T, RH, RV, m.eps, dt, stream)) return false;
        if (!hyb_linear(s.act, l.r_w_o, s.y2, T, W, RH * RV, dt, stream)) return false;
        r.y_a = s.y;
        r.y_b = s.y2;
        r.norm_a = l.out_norm_a;
        r.norm_b = l.out_norm_b;
        r.mix_scale = 0.5f;
    } else {
        set_status(kErrUnsupported, "atoma_hybrid_step: parallel layers take gated linear attention, latent attention or the pair of mixers, got %d",
                   l.mixer);
        return false;
    }
    r.y_ff = l.has_mlp ? s.yf : nullptr;
    r.x = s.x;
    r.trace = trace;
    r.add_rows = next && next->add_embedding ? s.x0 : nullptr;
    r.add_vec = next ? next->add_vec : nullptr;
    r.w_next = next ? next->norm1 : nullptr;
    r.h = s.h;
    r.T = T;
    r.width = W;
    r.eps = m.eps;
    r.weight_offset = m.norm_offset;
    r.dtype = dt;
    return hyb_parallel_residual_norm(r, stream);
}

}  // namespace
}  // namespace atoma

using namespace atoma;

extern "C" int64_t atoma_hybrid_abi_sizeof(int which) {
    switch (which) {
        case 0: return sizeof(atoma_hybrid_layer);
        case 1: return sizeof(atoma_hybrid_model);
        case 2: return sizeof(atoma_hybrid_batch);
        case 3: return sizeof(atoma_sigmoid_attn_args);
        case 4: return sizeof(atoma_gated_residual_args);
        case 5: return sizeof(atoma_latent_attn_args);
        case 6: return sizeof(atoma_moe_args);
        case 7: return sizeof(atoma_latent_expanded_args);
        case 8: return sizeof(atoma_lanes_update_args);
        case 9: return sizeof(atoma_softmax_attn_args);
        case 10: return sizeof(atoma_parallel_residual_args);
        case 11: return sizeof(atoma_tap_filter_args);
        case 12: return sizeof(atoma_state_scan_args);
        case 13: return sizeof(atoma_qkv_rope_args);
        default: return -1;
    }
}

extern "C" int64_t atoma_hybrid_scratch_bytes(const atoma_hybrid_model *model, int64_t num_tokens, int64_t num_selected) {
    if (!model || !model->layers || num_tokens < 0 || num_selected < 0) return -1;
    return carve(*model, num_tokens, num_selected, nullptr).total;
}

extern "C" void atoma_hybrid_step(const atoma_hybrid_model *model, const atoma_hybrid_batch *batch, atoma_stream_t stream_) {
    clear_status();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!model || !batch || !model->layers) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: model / batch is NULL");
        return;
    }
    const atoma_hybrid_model &m = *model;
    const atoma_hybrid_batch &b = *batch;
    const int64_t T = b.num_tokens, B = b.num_seqs, S = b.num_selected;
    if (T <= 0 || B <= 0) return;
    if (!b.tokens || !b.positions || !b.slot_mapping || !b.token_seq || !b.query_start || !b.context_lens || !b.block_tables ||
        !b.state_slots || !b.scratch || (S > 0 && (!b.selected || !b.logits)) || !m.embed || (!m.inv_freq && !m.pos_table && m.block_style != ATOMA_BLOCK_LANES && m.block_style != ATOMA_BLOCK_PARALLEL) || !m.final_norm ||
        !m.head || m.width <= 0 || m.vocab <= 0 || m.num_layers <= 0) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: a required tensor is NULL");
        return;
    }
    const Scratch s = carve(m, T, S, b.scratch);
    if (s.total > b.scratch_bytes) {
        set_status(kErrInvalidArg, "atoma_hybrid_step: scratch of %lld bytes, %lld needed", static_cast<long long>(b.scratch_bytes),
                   static_cast<long long>(s.total));
        return;
    }
    nvtxRangePushA("atoma_hybrid_step");
    struct Pop {
        ~Pop() { nvtxRangePop(); }
    } pop;
    const uint32_t dt = m.dtype;
    const int64_t W = m.width;
    const float off = m.norm_offset;
    const int64_t groups = m.norm_groups > 0 ? m.norm_groups : 1;
    if (m.block_style == ATOMA_BLOCK_PARALLEL) {
        // the embedding rows (kept when a later pass adds them again), what precedes the first layer, its input norm
        const atoma_hybrid_layer &first = m.layers[0];
        if (!hyb_embed_scaled_lanes(b.tokens, m.embed, 1.f, s.x, T, 1, W, m.vocab, dt, stream)) return;
        if (s.x0) cudaMemcpyAsync(s.x0, s.x, static_cast<size_t>(T) * W * 4, cudaMemcpyDeviceToDevice, stream);
        atoma_parallel_residual_args r{};
        r.x = s.x;
        r.add_rows = first.add_embedding ? s.x0 : nullptr;
        r.add_vec = first.add_vec;
        r.w_next = first.norm1;
        r.h = s.h;
        r.T = T;
        r.width = W;
        r.eps = m.eps;
        r.weight_offset = off;
        r.dtype = dt;
        if (!hyb_parallel_residual_norm(r, stream)) return;
        for (int64_t i = 0; i < m.num_layers; ++i) {
            if (!parallel_layer(m, b, m.layers[i], s, i + 1 < m.num_layers ? &m.layers[i + 1] : nullptr,
                                b.residual_trace ? b.residual_trace + i * T * W : nullptr, stream))
                return;
        }
        if (S > 0) {
            if (!hyb_group_rmsnorm_rows(s.x, b.selected, m.final_norm, off, 1, s.hs, S, W, m.eps, dt, stream)) return;
            if (!hyb_linear(s.hs, m.head, s.lg, S, m.vocab, W, dt, stream)) return;
            if (!hyb_scale_greedy(s.lg, b.logits, b.next_tokens, S, m.vocab, m.logit_scale, m.logit_softcap, dt, stream)) return;
        }
        return;
    }
    if (m.block_style == ATOMA_BLOCK_LANES) {
        // scaled embedding into every lane; per layer the lanes are read, normed, run through the sublayer and written back
        const int64_t lanes = m.lanes;
        if (lanes < 1) {
            set_status(kErrInvalidArg, "atoma_hybrid_step: a design on residual lanes needs at least one lane");
            return;
        }
        if (!hyb_embed_scaled_lanes(b.tokens, m.embed, m.embed_scale, s.x, T, lanes, W, m.vocab, dt, stream)) return;
        if (!hyb_lanes_read_norm(s.x, m.layers[0].lanes_in1, nullptr, m.layers[0].norm1, off, s.h, nullptr, T, lanes, W, m.eps, dt, stream)) return;
        for (int64_t i = 0; i < m.num_layers; ++i) {
            const bool last = i + 1 == m.num_layers;
            if (!lanes_layer(m, b, m.layers[i], s, last ? nullptr : m.layers[i + 1].lanes_in1, last ? nullptr : m.layers[i + 1].norm1,
                             b.residual_trace ? b.residual_trace + i * T * W : nullptr, stream))
                return;
        }
        if (S > 0) {
            if (!hyb_lanes_read_norm(s.x, nullptr, b.selected, m.final_norm, off, s.hs, nullptr, S, lanes, W, m.eps, dt, stream)) return;
            if (!hyb_linear(s.hs, m.head, s.lg, S, m.vocab, W, dt, stream)) return;
            if (!hyb_scale_greedy(s.lg, b.logits, b.next_tokens, S, m.vocab, m.logit_scale, m.logit_softcap, dt, stream)) return;
        }
        return;
    }
    if (m.pos_table) {
        if (!hyb_embed_learned(b.tokens, b.positions, m.embed, m.pos_table, s.x, T, W, m.vocab, m.max_positions, dt, stream)) return;
    } else if (!hyb_embed_sinusoid(b.tokens, b.positions, m.embed, m.inv_freq, s.x, T, W, m.vocab, dt, stream)) {
        return;
    }
    if (!hyb_group_rmsnorm_rows(s.x, nullptr, m.layers[0].norm1, off, groups, s.h, T, W, m.eps, dt, stream)) return;
    for (int64_t i = 0; i < m.num_layers; ++i) {
        const atoma_hybrid_layer &l = m.layers[i];
        const float *next_norm = i + 1 < m.num_layers ? m.layers[i + 1].norm1 : nullptr;
        if (m.block_style == ATOMA_BLOCK_PRENORM) {
            if (!prenorm_layer(m, b, l, s, next_norm, stream)) return;
            if (b.residual_trace)
                cudaMemcpyAsync(b.residual_trace + i * T * W, s.x, static_cast<size_t>(T) * W * 4, cudaMemcpyDeviceToDevice, stream);
            continue;
        }
        if (l.mixer == ATOMA_MIXER_SIGMOID_ATTENTION) {
            const int64_t nqkv = (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim;
            if (!hyb_linear(s.h, l.w_qkv, s.proj, T, nqkv, W, dt, stream)) return;
            if (!hyb_qk_norm_cache(s.proj, l.b_qkv, l.q_norm, l.k_norm, b.positions, b.slot_mapping, s.q, l.k_cache, l.v_cache, T,
                                   l.heads, l.kv_heads, l.dim, l.vdim, m.eps, l.temp_coef, l.temp_every, dt, stream))
                return;
            atoma_sigmoid_attn_args a{};
            a.q = s.q;
            a.k_cache = l.k_cache;
            a.v_cache = l.v_cache;
            a.out = s.act;
            a.positions = b.positions;
            a.token_seq = b.token_seq;
            a.query_start = b.query_start;
            a.max_seq_len = b.max_seq_len;
            a.block_tables = b.block_tables;
            a.slopes = l.slopes;
            a.head_bias = l.head_bias;
            a.talk = l.talk;
            a.T = T;
            a.B = B;
            a.max_blocks = b.max_blocks;
            a.H = l.heads;
            a.G = l.kv_heads;
            a.dim = l.dim;
            a.vdim = l.vdim;
            a.block_size = m.block_size;
            a.scale = l.scale;
            a.softcap = l.softcap;
            a.dtype = dt;
            a.max_query_len = b.max_query_len;
            if (!hyb_attention(a, stream)) return;
            if (!hyb_linear(s.act, l.w_o, s.y, T, W, l.heads * l.vdim, dt, stream)) return;
        } else if (l.mixer == ATOMA_MIXER_MINGRU) {
            const int64_t Sw = l.state_width;
            if (!hyb_linear(s.h, l.w_zxg, s.proj, T, 3 * Sw, W, dt, stream)) return;
            if (!hyb_mingru_scan(s.proj, l.b_zxg, l.state, b.state_slots, b.query_start, b.context_lens, s.act, T, B, Sw,
                                 b.max_query_len, dt, stream))
                return;
            if (!hyb_linear(s.act, l.w_o, s.y, T, W, Sw, dt, stream)) return;
        } else {
            set_status(kErrInvalidArg, "atoma_hybrid_step: layer %lld has unknown mixer %d", static_cast<long long>(i), l.mixer);
            return;
        }
        if (!hyb_postnorm_add_prenorm(s.y, s.x, l.norm1b, l.has_mlp ? l.norm2 : next_norm, s.h, T, W, m.eps, off, dt, stream)) return;
        if (l.has_mlp) {
            if (!hyb_gate_up_act(s.h, l.w_gate_up, s.proj, s.act, T, l.ff, W, l.act, dt, stream)) return;
            if (!hyb_linear(s.act, l.w_down, s.y, T, W, l.ff, dt, stream)) return;
            if (!hyb_postnorm_add_prenorm(s.y, s.x, l.norm2b, next_norm, s.h, T, W, m.eps, off, dt, stream)) return;
        }
        if (b.residual_trace) {
            cudaMemcpyAsync(b.residual_trace + i * T * W, s.x, static_cast<size_t>(T) * W * 4, cudaMemcpyDeviceToDevice, stream);
        }
    }
    if (S > 0) {
        if (!hyb_group_rmsnorm_rows(s.x, b.selected, m.final_norm, off, groups, s.hs, S, W, m.eps, dt, stream)) return;
        if (!hyb_linear(s.hs, m.head, s.lg, S, m.vocab, W, dt, stream)) return;
        if (!hyb_scale_greedy(s.lg, b.logits, b.next_tokens, S, m.vocab, m.logit_scale, m.logit_softcap, dt, stream)) return;
    }
}
