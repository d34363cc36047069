"""Python face of the hybrid-model operators (include/atoma_hybrid.h): thin ctypes shims over torch tensors,
one function per operator, used by tests and by callers that compose the operators themselves.
`dtype` follows the activations: torch.bfloat16 or torch.float32.  No fallback path."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import SigmoidAttnArgs
from .ops import AtomaError

_CODES = {torch.bfloat16: 1, torch.float32: 2}


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _s():
    return torch.cuda.current_stream().cuda_stream


def _check():
    L = _lib.lib()
    if L.atoma_last_status() != 0:
        raise AtomaError(L.atoma_last_error().decode())


def debug_flags(flags: int) -> None:
    """bit 0: plain float32 GEMM everywhere; bit 1: general attention kernel only; bit 2: sequential minGRU scan;
    bit 3: the routed experts' tcgen05 products for steps of any size."""
    _lib.lib().atoma_debug_hybrid(int(flags))


def embed_sinusoid(tokens, positions, table, inv_freq):
    T, W = tokens.numel(), table.shape[1]
    out = torch.empty((T, W), dtype=torch.float32, device=table.device)
    _lib.lib().atoma_embed_sinusoid(_p(tokens), _p(positions), _p(table), _p(inv_freq), _p(out), T, W, table.shape[0],
                                    _CODES[table.dtype], _s())
    _check()
    return out


def rmsnorm_rows(x, weight, offset, eps, dtype, rows=None):
    R = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((R, x.shape[1]), dtype=dtype, device=x.device)
    _lib.lib().atoma_rmsnorm_rows(_p(x), _p(rows), _p(weight), offset, _p(out), R, x.shape[1], eps, _CODES[dtype], _s())
    _check()
    return out


def postnorm_add_prenorm(y, x, w_post, w_pre, eps, offset):
    """x is updated in place; returns the next sublayer's normed input (None without w_pre)."""
    h = torch.empty_like(y) if w_pre is not None else None
    _lib.lib().atoma_postnorm_add_prenorm(_p(y), _p(x), _p(w_post), _p(w_pre), _p(h), y.shape[0], y.shape[1], eps, offset,
                                          _CODES[y.dtype], _s())
    _check()
    return h


def qk_norm_cache(qkv, bias, q_w, k_w, positions, slots, k_cache, v_cache, H, G, dim, vdim, eps, temp_coef, temp_every):
    T = qkv.shape[0]
    q = torch.empty((T, H * dim), dtype=qkv.dtype, device=qkv.device)
    _lib.lib().atoma_qk_norm_cache(_p(qkv), _p(bias), _p(q_w), _p(k_w), _p(positions), _p(slots), _p(q), _p(k_cache), _p(v_cache),
                                   T, H, G, dim, vdim, eps, temp_coef, temp_every, _CODES[qkv.dtype], _s())
    _check()
    return q


def sigmoid_attention_paged(q, k_cache, v_cache, positions, token_seq, block_tables, slopes, head_bias, talk, H, G, dim, vdim,
                            block_size, scale, softcap, max_query_len, query_start=None, max_seq_len=None):
    T = q.shape[0]
    if query_start is None:
        counts = torch.bincount(token_seq.long(), minlength=block_tables.shape[0])
        query_start = torch.cat([counts.new_zeros(1), counts.cumsum(0)]).to(torch.int32)
    if max_seq_len is None:
        max_seq_len = int(positions.max()) + 1
    out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    a = SigmoidAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out = _p(q), _p(k_cache), _p(v_cache), _p(out)
    a.positions, a.token_seq, a.block_tables = _p(positions), _p(token_seq), _p(block_tables)
    a.query_start, a.max_seq_len = _p(query_start), int(max_seq_len)
    a.slopes, a.head_bias, a.talk = _p(slopes), _p(head_bias), _p(talk)
    a.T, a.B, a.max_blocks = T, block_tables.shape[0], block_tables.shape[1]
    a.H, a.G, a.dim, a.vdim, a.block_size = H, G, dim, vdim, block_size
    a.scale, a.softcap, a.dtype, a.max_query_len = scale, softcap, _CODES[q.dtype], max_query_len
    _lib.lib().atoma_sigmoid_attention_paged(C.byref(a), _s())
    _check()
    return out


def mingru_scan(zxg, bias, state, state_slots, query_start, context_lens, max_query_len):
    T, S = zxg.shape[0], zxg.shape[1] // 3
    out = torch.empty((T, S), dtype=zxg.dtype, device=zxg.device)
    _lib.lib().atoma_mingru_scan(_p(zxg), _p(bias), _p(state), _p(state_slots), _p(query_start), _p(context_lens), _p(out), T,
                                 state_slots.numel(), S, max_query_len, _CODES[zxg.dtype], _s())
    _check()
    return out


def glu(gu, act: int):
    T, ff = gu.shape[0], gu.shape[1] // 2
    out = torch.empty((T, ff), dtype=gu.dtype, device=gu.device)
    _lib.lib().atoma_glu(_p(gu), _p(out), T, ff, act, _CODES[gu.dtype], _s())
    _check()
    return out


def linear(x, w):
    y = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
    _lib.lib().atoma_linear(_p(x), _p(w), _p(y), x.shape[0], w.shape[0], x.shape[1], _CODES[x.dtype], _s())
    _check()
    return y


def scale_logits_greedy(logits, scale):
    R, V = logits.shape
    out = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    tok = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _lib.lib().atoma_scale_logits_greedy(_p(logits), _p(out), _p(tok), R, V, scale, _CODES[logits.dtype], _s())
    _check()
    return out, tok


def gate_up_act(x, w_gate_up, act: int):
    """act(x Wg^T) * (x Wu^T) with the activation in the projection's epilogue (bfloat16, T <= 128, K % 64 == 0)."""
    T, ff = x.shape[0], w_gate_up.shape[0] // 2
    out = torch.empty((T, ff), dtype=x.dtype, device=x.device)
    _lib.lib().atoma_gate_up_act(_p(x), _p(w_gate_up), _p(out), T, ff, x.shape[1], x.shape[1], x.shape[1], ff, act, 1, _s())
    _check()
    return out


# ---- pre-norm designs: learned positions, grouped norms, gated residuals, latent attention, mixtures of experts ----
def embed_learned(tokens, positions, table, pos_table):
    T, W = tokens.numel(), table.shape[1]
    out = torch.empty((T, W), dtype=torch.float32, device=table.device)
    _lib.lib().atoma_embed_learned(_p(tokens), _p(positions), _p(table), _p(pos_table), _p(out), T, W, table.shape[0], pos_table.shape[0],
                                   _CODES[table.dtype], _s())
    _check()
    return out


def group_rmsnorm_rows(x, weight, offset, groups, eps, dtype, rows=None):
    R = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((R, x.shape[1]), dtype=dtype, device=x.device)
    _lib.lib().atoma_group_rmsnorm_rows(_p(x), _p(rows), _p(weight), offset, groups, _p(out), R, x.shape[1], eps, _CODES[dtype], _s())
    _check()
    return out


def gated_residual_norm(x, y=None, gate=None, gate_bias=None, row_scale=None, expert_out=None, pair_row=None, top=0, w_next=None,
                        groups=1, eps=1e-5, offset=0.0, want_cast=False):
    """x (float32) is updated in place; returns (h, x_cast), each None when not asked for.  y / gate may be column slices of a
    wider row-major matrix (their row stride is passed on)."""
    from ._lib import GatedResidualArgs
    ref = y if y is not None else expert_out
    T, W = x.shape
    h = torch.empty((T, W), dtype=ref.dtype, device=x.device) if w_next is not None else None
    xc = torch.empty((T, W), dtype=ref.dtype, device=x.device) if want_cast else None
    a = GatedResidualArgs()
    a.y, a.ld_y = _p(y), (y.stride(0) if y is not None else 0)
    a.row_scale, a.expert_out, a.pair_row, a.top = _p(row_scale), _p(expert_out), _p(pair_row), top
    a.gate, a.ld_gate, a.gate_bias = _p(gate), (gate.stride(0) if gate is not None else 0), _p(gate_bias)
    a.x, a.w_next, a.h, a.x_cast = _p(x), _p(w_next), _p(h), _p(xc)
    a.T, a.width, a.groups, a.eps, a.weight_offset, a.dtype = T, W, groups, eps, offset, _CODES[ref.dtype]
    _lib.lib().atoma_gated_residual_norm(C.byref(a), _s())
    _check()
    return h, xc


def side_gate(a, tokens, side_table, part, dim):
    T = a.shape[0]
    out = torch.empty((T, dim), dtype=a.dtype, device=a.device)
    _lib.lib().atoma_side_gate(_p(a), a.stride(0), _p(tokens), _p(side_table), side_table.shape[1], part, _p(out), T, dim,
                               side_table.shape[0], _CODES[a.dtype], _s())
    _check()
    return out


def unitnorm_add_norm(y, x, w_unit, w_next, groups, eps, offset=0.0):
    h = torch.empty_like(y) if w_next is not None else None
    _lib.lib().atoma_unitnorm_add_norm(_p(y), _p(x), _p(w_unit), _p(w_next), _p(h), y.shape[0], y.shape[1], groups, eps, offset,
                                       _CODES[y.dtype], _s())
    _check()
    return h


def latent_norm_cache(proj, q_weight, kv_weight, slots, cache, q_rank, kv_rank, eps):
    T = proj.shape[0]
    cq = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device) if q_rank > 0 else None
    _lib.lib().atoma_latent_norm_cache(_p(proj), proj.stride(0), _p(q_weight), _p(kv_weight), _p(slots), _p(cq), _p(cache), T, q_rank,
                                       kv_rank, eps, _CODES[proj.dtype], _s())
    _check()
    return cq


def head_project(x, w, H, n, R, absorb: bool):
    """absorb: x [T, H n] -> float32 [T, H, R];  else x float32 [T, H, R] -> [T, H n] in w's format."""
    T = x.shape[0]
    out = (torch.empty((T, H, R), dtype=torch.float32, device=x.device) if absorb
           else torch.empty((T, H * n), dtype=w.dtype, device=x.device))
    _lib.lib().atoma_head_project(_p(x), _p(w), _p(out), T, H, n, R, 1 if absorb else 0, _CODES[w.dtype], _s())
    _check()
    return out


def latent_attention_paged(q_lat, cache, positions, token_seq, block_tables, sink, H, R, block_size, window, scale, max_query_len,
                           query_start=None, max_seq_len=None, out_cols=0):
    from ._lib import LatentAttnArgs
    T = q_lat.shape[0]
    if query_start is None:
        counts = torch.bincount(token_seq.long(), minlength=block_tables.shape[0])
        query_start = torch.cat([counts.new_zeros(1), counts.cumsum(0)]).to(torch.int32)
    if max_seq_len is None:
        max_seq_len = int(positions.max()) + 1
    out = torch.empty((T, H, R), dtype=torch.float32, device=q_lat.device)
    a = LatentAttnArgs()
    a.q_lat, a.latent_cache, a.out = _p(q_lat), _p(cache), _p(out)
    a.positions, a.token_seq, a.query_start, a.block_tables, a.sink = _p(positions), _p(token_seq), _p(query_start), _p(block_tables), _p(sink)
    a.T, a.B, a.max_blocks, a.H, a.R, a.block_size, a.window = T, block_tables.shape[0], block_tables.shape[1], H, R, block_size, window
    a.scale, a.dtype, a.max_query_len, a.max_seq_len, a.out_cols = scale, _CODES[cache.dtype], max_query_len, int(max_seq_len), out_cols
    _lib.lib().atoma_latent_attention_paged(C.byref(a), _s())
    _check()
    return out


def moe_route(h, w_router, w_row_gate, top, renormalize=False):
    T, E = h.shape[0], w_router.shape[0]
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    wgt = torch.empty((T, top), dtype=torch.float32, device=h.device)
    rg = torch.empty((T,), dtype=torch.float32, device=h.device) if w_row_gate is not None else None
    _lib.lib().atoma_moe_route(_p(h), _p(w_router), _p(w_row_gate), _p(idx), _p(wgt), _p(rg), T, h.shape[1], E, top,
                               1 if renormalize else 0, _CODES[h.dtype], _s())
    _check()
    return idx, wgt, rg


def glu_clamped(gu, ff, limit, alpha, up_shift):
    T = gu.shape[0]
    out = torch.empty((T, ff), dtype=gu.dtype, device=gu.device)
    _lib.lib().atoma_glu_clamped(_p(gu), gu.stride(0), _p(out), T, ff, limit, alpha, up_shift, _CODES[gu.dtype], _s())
    _check()
    return out


def moe_experts(h, top_expert, top_weight, w_gate_up, w_down, limit, alpha, up_shift, scale_input=True):
    """Returns the token's summed expert outputs as float32 [T, width] (the rows are summed here on the host side of the call
    for tests; the step executor sums them inside its residual kernel)."""
    from ._lib import MoeArgs
    T, W = h.shape
    E, ff2, _ = w_gate_up.shape
    top = top_expert.shape[1]
    code = _CODES[h.dtype]
    nbytes = int(_lib.lib().atoma_moe_workspace_bytes(T, top, E, W, ff2 // 2, code))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=h.device)
    a = MoeArgs()
    a.h, a.top_expert, a.top_weight, a.w_gate_up, a.w_down = _p(h), _p(top_expert), _p(top_weight), _p(w_gate_up), _p(w_down)
    a.workspace, a.workspace_bytes = _p(ws), nbytes
    a.T, a.width, a.experts, a.top, a.ff = T, W, E, top, ff2 // 2
    a.limit, a.alpha, a.up_shift, a.scale_input, a.dtype = limit, alpha, up_shift, 1 if scale_input else 0, code
    eo, pr = C.c_void_p(), C.c_void_p()
    _lib.lib().atoma_moe_experts(C.byref(a), C.byref(eo), C.byref(pr), _s())
    _check()
    x = torch.zeros((T, W), dtype=torch.float32, device=h.device)
    ga = _lib.GatedResidualArgs()
    ga.expert_out, ga.pair_row, ga.top, ga.x = eo.value, pr.value, top, _p(x)
    ga.T, ga.width, ga.groups, ga.eps, ga.dtype = T, W, 1, 1e-5, code
    _lib.lib().atoma_gated_residual_norm(C.byref(ga), _s())
    _check()
    x._workspace = ws             # the kernels may still be running: the workspace lives as long as the result
    return x


def finish_logits_greedy(logits, scale, softcap):
    R, V = logits.shape
    out = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    tok = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _lib.lib().atoma_finish_logits_greedy(_p(logits), _p(out), _p(tok), R, V, scale, softcap, _CODES[logits.dtype], _s())
    _check()
    return out, tok


def latent_attention_expanded(q, cache, w_uk, w_uv, query_start, context_lens, block_tables, sink, H, dim, R, block_size, window, scale,
                              min_q, max_query_len, max_seq_len, max_keys, out=None):
    """Rows of sequences with at least min_q tokens in the step are written; the others are left as they are in `out`."""
    from ._lib import LatentExpandedArgs
    T = q.shape[0]
    if out is None:
        out = torch.zeros((T, H * dim), dtype=q.dtype, device=q.device)
    a = LatentExpandedArgs()
    a.q, a.latent_cache, a.w_uk, a.w_uv, a.out = _p(q), _p(cache), _p(w_uk), _p(w_uv), _p(out)
    a.query_start, a.context_lens, a.block_tables, a.sink = _p(query_start), _p(context_lens), _p(block_tables), _p(sink)
    a.T, a.B, a.max_blocks, a.H, a.dim, a.R = T, block_tables.shape[0], block_tables.shape[1], H, dim, R
    a.block_size, a.window, a.max_keys, a.scale = block_size, window, max_keys, scale
    a.min_q, a.max_query_len, a.max_seq_len = min_q, max_query_len, max_seq_len
    _lib.lib().atoma_latent_attention_expanded(C.byref(a), _s())
    _check()
    return out


# ---- residual lanes, softmax attention with a distance table, restricted routing ----
def embed_scaled_lanes(tokens, table, scale, lanes):
    T, W = tokens.numel(), table.shape[1]
    x = torch.empty((T, lanes, W), dtype=torch.float32, device=table.device)
    _lib.lib().atoma_embed_scaled_lanes(_p(tokens), _p(table), scale, _p(x), T, lanes, W, table.shape[0], _CODES[table.dtype], _s())
    _check()
    return x


def lanes_read_norm(x, w_in, weight, offset, eps, dtype, rows=None, want_sum=False):
    """x float32 [T, lanes, width] -> (normed read in `dtype`, the un-normed read as float32 or None)."""
    T, S, W = x.shape
    R = T if rows is None else rows.numel()
    out = torch.empty((R, W), dtype=dtype, device=x.device)
    u = torch.empty((R, W), dtype=torch.float32, device=x.device) if want_sum else None
    _lib.lib().atoma_lanes_read_norm(_p(x), _p(w_in), _p(rows), _p(weight), offset, _p(out), _p(u), R, S, W, eps, _CODES[dtype], _s())
    _check()
    return out, u


def lanes_update_norm(x, y, w_mix, w_out, dtype, eps=1e-5, offset=0.0, y_bias=None, w_in_next=None, w_next=None, expert_out=None,
                      pair_row=None, top_expert=None, top_weight=None, h_in=None, experts=0, want_lane_sum=False):
    """x is updated in place; returns (next normed read or None, lane sum or None)."""
    from ._lib import LanesUpdateArgs
    T, S, W = x.shape
    h = torch.empty((T, W), dtype=dtype, device=x.device) if w_next is not None else None
    ls = torch.empty((T, W), dtype=torch.float32, device=x.device) if want_lane_sum else None
    a = LanesUpdateArgs()
    a.y, a.y_bias, a.expert_out, a.pair_row = _p(y), _p(y_bias), expert_out if isinstance(expert_out, int) else _p(expert_out), \
        pair_row if isinstance(pair_row, int) else _p(pair_row)
    a.top_expert, a.top_weight, a.h_in = _p(top_expert), _p(top_weight), _p(h_in)
    a.top, a.experts = (top_expert.shape[1] if top_expert is not None else 0), experts
    a.x, a.w_mix, a.w_out, a.w_in_next, a.w_next, a.h, a.lane_sum = _p(x), _p(w_mix), _p(w_out), _p(w_in_next), _p(w_next), _p(h), _p(ls)
    a.T, a.lanes, a.width, a.eps, a.weight_offset, a.dtype = T, S, W, eps, offset, _CODES[dtype]
    _lib.lib().atoma_lanes_update_norm(C.byref(a), _s())
    _check()
    return h, ls


def qk_headnorm_cache(proj, q_off, k_off, v_off, q_w, k_w, offset, slots, k_cache, v_cache, H, G, dim, vdim, eps):
    T = proj.shape[0]
    q = torch.empty((T, H * dim), dtype=proj.dtype, device=proj.device)
    _lib.lib().atoma_qk_headnorm_cache(_p(proj), proj.stride(0), q_off, k_off, v_off, _p(q_w), _p(k_w), offset, _p(slots), _p(q), _p(k_cache),
                                       _p(v_cache), T, H, G, dim, vdim, eps, _CODES[proj.dtype], _s())
    _check()
    return q


def softmax_attention_paged(q, k_cache, v_cache, positions, token_seq, block_tables, H, G, dim, vdim, block_size, scale, window=0,
                            keep_first=0, dist_bias=None, gate=None, max_query_len=None, query_start=None, max_seq_len=None, long_min_q=0, long_stats=None):
    """long_min_q > 0: sequences with at least that many tokens in the step take the long-portion path (where the shapes allow);
    long_stats = (how many such sequences, the sum of their tokens, the sum of their contexts) saves the host reads that find them."""
    from ._lib import SoftmaxAttnArgs
    T = q.shape[0]
    if query_start is None:
        counts = torch.bincount(token_seq.long(), minlength=block_tables.shape[0])
        query_start = torch.cat([counts.new_zeros(1), counts.cumsum(0)]).to(torch.int32)
    if max_query_len is None:
        max_query_len = int((query_start[1:] - query_start[:-1]).max())
    if max_seq_len is None:
        max_seq_len = int(positions.max()) + 1
    out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    a = SoftmaxAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out, a.gate = _p(q), _p(k_cache), _p(v_cache), _p(out), _p(gate)
    a.ld_gate = gate.stride(0) if gate is not None else 0
    a.dist_bias, a.dist_rows = _p(dist_bias), (dist_bias.shape[0] if dist_bias is not None else 0)
    a.positions, a.token_seq, a.query_start, a.block_tables = _p(positions), _p(token_seq), _p(query_start), _p(block_tables)
    a.T, a.B, a.max_blocks, a.H, a.G, a.dim, a.vdim = T, block_tables.shape[0], block_tables.shape[1], H, G, dim, vdim
    a.block_size, a.window, a.keep_first, a.scale, a.dtype = block_size, window, keep_first, scale, _CODES[q.dtype]
    a.max_query_len, a.max_seq_len = int(max_query_len), int(max_seq_len)
    if long_min_q > 0 and long_stats is not None:
        a.long_min_q, (a.long_seqs, a.long_tokens, a.long_ctx_sum) = long_min_q, long_stats
    elif long_min_q > 0:
        qs = query_start.cpu().tolist()
        ctx = [int(positions[qs[b]]) for b in range(len(qs) - 1)]
        long_ = [b for b in range(len(qs) - 1) if qs[b + 1] - qs[b] >= long_min_q]
        a.long_min_q, a.long_seqs = long_min_q, len(long_)
        a.long_tokens, a.long_ctx_sum = sum(qs[b + 1] - qs[b] for b in long_), sum(ctx[b] for b in long_)
    _lib.lib().atoma_softmax_attention_paged(C.byref(a), _s())
    _check()
    return out


def moe_route_grouped(h, w_router, correction, top, groups=1, keep=1, score="softmax", renormalize=True):
    T, E = h.shape[0], w_router.shape[0]
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    wgt = torch.empty((T, top), dtype=torch.float32, device=h.device)
    _lib.lib().atoma_moe_route_grouped(_p(h), _p(w_router), _p(correction), _p(idx), _p(wgt), T, h.shape[1], E, top, groups, keep,
                                       1 if score == "softmax" else 0, 1 if renormalize else 0, _CODES[h.dtype], _s())
    _check()
    return idx, wgt


def glu_clamped_bias(gu, bias, ff, limit, alpha, up_shift):
    T = gu.shape[0]
    out = torch.empty((T, ff), dtype=gu.dtype, device=gu.device)
    _lib.lib().atoma_glu_clamped_bias(_p(gu), gu.stride(0), _p(bias), _p(out), T, ff, limit, alpha, up_shift, _CODES[gu.dtype], _s())
    _check()
    return out


def linear_glu_clamped(x, w_gate_up, bias, limit, alpha, up_shift):
    """The clamped gated activation of the projection x w_gate_up^T: one kernel for decode-sized bfloat16 steps."""
    T, K = x.shape
    ff = w_gate_up.shape[0] // 2
    proj = torch.empty((T, 2 * ff), dtype=x.dtype, device=x.device)
    out = torch.empty((T, ff), dtype=x.dtype, device=x.device)
    _lib.lib().atoma_linear_glu_clamped(_p(x), _p(w_gate_up), _p(bias), _p(proj), _p(out), T, ff, K, limit, alpha, up_shift, _CODES[x.dtype], _s())
    _check()
    return out


def moe_expert_rows(h, top_expert, top_weight, w_gate_up, w_down, limit, alpha, up_shift, scale_input=False):
    """The routed experts' result rows as the step executor sees them: (expert_out address, pair_row address, workspace tensor
    that owns both).  For callers that hand them to lanes_update_norm."""
    from ._lib import MoeArgs
    T, W = h.shape
    E, ff2, _ = w_gate_up.shape
    top = top_expert.shape[1]
    code = _CODES[h.dtype]
    nbytes = int(_lib.lib().atoma_moe_workspace_bytes(T, top, E, W, ff2 // 2, code))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=h.device)
    a = MoeArgs()
    a.h, a.top_expert, a.top_weight, a.w_gate_up, a.w_down = _p(h), _p(top_expert), _p(top_weight), _p(w_gate_up), _p(w_down)
    a.workspace, a.workspace_bytes = _p(ws), nbytes
    a.T, a.width, a.experts, a.top, a.ff = T, W, E, top, ff2 // 2
    a.limit, a.alpha, a.up_shift, a.scale_input, a.dtype = limit, alpha, up_shift, 1 if scale_input else 0, code
    eo, pr = C.c_void_p(), C.c_void_p()
    _lib.lib().atoma_moe_experts(C.byref(a), C.byref(eo), C.byref(pr), _s())
    _check()
    return eo.value, pr.value, ws


# ---- parallel blocks: tap filters, matrix-state recurrences, rotary operators ----
def parallel_residual_norm(x, dtype, y_a=None, y_b=None, y_ff=None, norm_a=None, norm_b=None, mix_scale=1.0, add_rows=None, add_vec=None,
                           w_next=None, eps=1e-5, offset=0.0, want_trace=False):
    """x [T, width] float32 is updated in place; returns (h or None, trace or None)."""
    from ._lib import ParallelResidualArgs
    T, W = x.shape
    h = torch.empty((T, W), dtype=dtype, device=x.device) if w_next is not None else None
    trace = torch.empty_like(x) if want_trace else None
    a = ParallelResidualArgs()
    a.y_a, a.y_b, a.y_ff, a.norm_a, a.norm_b, a.mix_scale = _p(y_a), _p(y_b), _p(y_ff), _p(norm_a), _p(norm_b), mix_scale
    a.x, a.trace, a.add_rows, a.add_vec, a.w_next, a.h = _p(x), _p(trace), _p(add_rows), _p(add_vec), _p(w_next), _p(h)
    a.T, a.width, a.eps, a.weight_offset, a.dtype = T, W, eps, offset, _CODES[dtype]
    _lib.lib().atoma_parallel_residual_norm(C.byref(a), _s())
    _check()
    return h, trace


def tap_filter(x, w1, w2, history, state_slots, token_seq, query_start, context_lens, residual: bool, act: int = 0):
    """x [T, channels]; w1 / w2 [channels, taps] float32 (w2 may be None); history [slots, >= (taps - 1) channels] float32 is read
    and rewritten.  Returns (out1, out2 or None)."""
    from ._lib import TapFilterArgs
    T, Cn = x.shape
    out1 = torch.empty_like(x)
    out2 = torch.empty_like(x) if w2 is not None else None
    a = TapFilterArgs()
    a.in_, a.ld_in, a.w1, a.w2, a.out1, a.out2, a.ld_out = _p(x), x.stride(0), _p(w1), _p(w2), _p(out1), _p(out2), Cn
    a.history, a.history_stride = _p(history), 0 if history is None else history.stride(0)
    a.state_slots, a.token_seq, a.query_start, a.context_lens = _p(state_slots), _p(token_seq), _p(query_start), _p(context_lens)
    a.T, a.B, a.channels, a.taps, a.residual, a.act, a.dtype = T, context_lens.numel(), Cn, w1.shape[1], int(residual), act, _CODES[x.dtype]
    _lib.lib().atoma_tap_filter(C.byref(a), _s())
    _check()
    return out1, out2


def _scan_common(a, q, k, v, state, state_slots, query_start, context_lens, H, G, dim, vdim):
    T = q.shape[0]
    out = torch.empty((T, H * vdim), dtype=torch.float32, device=q.device)
    a.q, a.k, a.v, a.ld_q, a.ld_k, a.ld_v = _p(q), _p(k), _p(v), q.stride(0), k.stride(0), v.stride(0)
    a.state, a.state_stride = _p(state), state.stride(0)
    a.state_slots, a.query_start, a.context_lens, a.out = _p(state_slots), _p(query_start), _p(context_lens), _p(out)
    a.T, a.B, a.H, a.G, a.dim, a.vdim, a.dtype = T, context_lens.numel(), H, G, dim, vdim, _CODES[q.dtype]
    _lib.lib().atoma_state_scan(C.byref(a), _s())
    _check()
    return out


def gla_scan(q, k, v, z, z_bias, tau, q_scale, state, state_slots, query_start, context_lens, H, dim, vdim):
    """Gated linear attention over a mixed batch: q, k, z [T, H dim], v [T, H vdim] -> float32 [T, H vdim]; state [slots, H dim vdim]."""
    from ._lib import StateScanArgs
    a = StateScanArgs()
    a.kind, a.z, a.ld_z, a.z_bias, a.tau, a.q_scale = 0, _p(z), z.stride(0), _p(z_bias), tau, q_scale
    return _scan_common(a, q, k, v, state, state_slots, query_start, context_lens, H, H, dim, vdim)


def delta_rule_scan(q, k, v, b_pre, a_pre, a_log, dt_bias, q_scale, state, state_slots, query_start, context_lens, H, G, dim, vdim,
                    unit_eps=1e-6):
    """Gated delta rule over a mixed batch: q, k [T, G dim], v [T, H vdim], b_pre, a_pre [T, H] -> float32 [T, H vdim]."""
    from ._lib import StateScanArgs
    a = StateScanArgs()
    a.kind, a.b_pre, a.a_pre, a.ld_b, a.ld_a = 1, _p(b_pre), _p(a_pre), b_pre.stride(0), a_pre.stride(0)
    a.a_log, a.dt_bias, a.q_scale, a.unit_eps = _p(a_log), _p(dt_bias), q_scale, unit_eps
    return _scan_common(a, q, k, v, state, state_slots, query_start, context_lens, H, G, dim, vdim)


def headnorm_gate(o, weight, gate, H, vdim, eps, dtype):
    T = o.shape[0]
    out = torch.empty((T, H * vdim), dtype=dtype, device=o.device)
    _lib.lib().atoma_headnorm_gate(_p(o), _p(weight), _p(gate), 0 if gate is None else gate.stride(0), _p(out), T, H, vdim, eps,
                                   _CODES[dtype], _s())
    _check()
    return out


def qkv_headnorm_rope_cache(proj, q_off, k_off, v_off, q_w, k_w, qk_freq, v_freq, interleaved, positions, slots, k_cache, v_cache, H, G,
                            dim, vdim, eps):
    from ._lib import QkvRopeArgs
    T = proj.shape[0]
    q = torch.empty((T, H * dim), dtype=proj.dtype, device=proj.device)
    a = QkvRopeArgs()
    a.proj, a.ld, a.q_off, a.k_off, a.v_off = _p(proj), proj.stride(0), q_off, k_off, v_off
    a.q_weight, a.k_weight, a.qk_freq, a.v_freq = _p(q_w), _p(k_w), _p(qk_freq), _p(v_freq)
    a.rot_pairs, a.v_pairs, a.interleaved = 0 if qk_freq is None else qk_freq.numel(), 0 if v_freq is None else v_freq.numel(), int(interleaved)
    a.positions, a.slot_mapping, a.q_out, a.k_cache, a.v_cache = _p(positions), _p(slots), _p(q), _p(k_cache), _p(v_cache)
    a.T, a.H, a.G, a.dim, a.vdim, a.eps, a.dtype = T, H, G, dim, vdim, eps, _CODES[proj.dtype]
    _lib.lib().atoma_qkv_headnorm_rope_cache(C.byref(a), _s())
    _check()
    return q


def rotate_heads(x, positions, freq, H, n, interleaved, sign):
    """In place on x [T, H n]."""
    _lib.lib().atoma_rotate_heads(_p(x), _p(positions), _p(freq), x.shape[0], H, n, freq.numel(), int(interleaved), sign, _CODES[x.dtype], _s())
    _check()
    return x


def latent_norm_rope_cache(proj, q_weight, kv_weight, freq, interleaved, positions, slots, cache, q_rank, kv_rank, rot_dim, eps):
    T = proj.shape[0]
    cq = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device)
    _lib.lib().atoma_latent_norm_rope_cache(_p(proj), proj.stride(0), _p(q_weight), _p(kv_weight), _p(freq), 0 if freq is None else freq.numel(),
                                            int(interleaved), _p(positions), _p(slots), _p(cq), _p(cache), T, q_rank, kv_rank, rot_dim, eps,
                                            _CODES[proj.dtype], _s())
    _check()
    return cq


def latent_query_absorb_rope(q, w_uk, freq, interleaved, positions, H, dim, rot_dim, kv_rank):
    T = q.shape[0]
    out = torch.empty((T, H, kv_rank + rot_dim), dtype=torch.float32, device=q.device)
    _lib.lib().atoma_latent_query_absorb_rope(_p(q), _p(w_uk), _p(freq), 0 if freq is None else freq.numel(), int(interleaved), _p(positions),
                                              _p(out), T, H, dim, rot_dim, kv_rank, _CODES[q.dtype], _s())
    _check()
    return out


def latent_expand_values(o_lat, w_uv, H, vdim, kv_rank, dtype):
    T, row = o_lat.shape[0], o_lat.shape[-1]
    out = torch.empty((T, H * vdim), dtype=dtype, device=o_lat.device)
    _lib.lib().atoma_latent_expand_values(_p(o_lat), _p(w_uv), _p(out), T, H, vdim, kv_rank, row, _CODES[dtype], _s())
    _check()
    return out
