"""Nemasun: a decoder on several residual lanes, softmax attention whose values are its keys, clamped dense
feed-forwards and mixtures of experts with a corrected, group-restricted softmax router.

config.json gives every size and every constant that can differ between checkpoints:
  architecture "Nemasun", vocab, width, streams (the number of residual lanes), embedding {scale}, norm {eps}, and
  `layers`: per layer its `type` ("attention"), the mixer's sizes (`mixer`: heads, kv_heads, dim, vdim, scale,
  bias_max, mask {size, keep_first}) and its feed-forward (`mlp`: null, {kind "dense", ff, limit}, or {kind "moe",
  router {experts, identity, top, groups {count, keep}}, expert {ff}, shared {ff} or null}).
Fixed by the design (and therefore constants here): the embedding row times a scale, no position signal; every sublayer
reads sum_s in[s] lane_s through a plain-weight RMS norm and writes lane_t <- sum_s mix[s, t] lane_s + out[t] y;
the model's output is the final norm of the plain sum of the lanes.  Attention: grouped key/value heads, no value
projection (a value is the key projection before its norm), per-head q/k RMS norm with one weight of `dim` for all
heads, score * scale + table[bucket(distance), head], a window of mask.size positions that also keeps the first
mask.keep_first tokens, softmax, the heads' outputs times sigmoid(W_g h).  bucket(n) of a table with B rows: n below
B / 2, then floor(ln(n / (B / 2)) / ln(bias_max / (B / 2)) * (B - B / 2)) further rows, at most the last.  Dense
feed-forward: biases, g = min(gate, limit), u = clamp(up, +-limit), g sigmoid(1.702 g) (u + 1).  Experts: silu(gate) up,
no biases; softmax router over experts + identity outputs; the choice adds `correction` and is restricted to the best
groups; weights = chosen scores over (their sum + 1e-20); identity outputs hand the feed-forward's input through;
the shared expert is added ungated.

Checkpoint tensors: embed, head, final.norm and per layer i `l<i>.norm1 / norm2`, `l<i>.hc1 / hc2 .{in, out, mix}`,
`l<i>.mix.{q, k, g, o, rel}`, `l<i>.mix.{q, k}.norm`, `l<i>.mlp.{gate, up, down}` (+ `.b`) or
`l<i>.mlp.{router, correction}`, `l<i>.mlp.e<k>.{gate, up, down}`, `l<i>.mlp.shared.{gate, up, down}`.
This module turns that into the generic hybrid description (hybrid.py); it has no compute of its own.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from .hybrid import ClampedMlpSpec, HybridSpec, LayerSpec, MoeSpec, SoftmaxAttentionSpec
from .ops import AtomaError

ARCHITECTURE = "Nemasun"
DENSE_ALPHA = 1.702
DENSE_UP_SHIFT = 1.0


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a distance table with `rows` rows for the distance n >= 0 (`far` = the distance at which the last row begins)."""
    half = rows // 2
    if n < half or half == 0:
        return min(n, rows - 1)
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def expand_distance_table(table: torch.Tensor, far: float) -> torch.Tensor:
    """table [rows, heads] by bucket -> float32 [distances, heads] by distance; the last row stands for every larger distance."""
    rows = table.shape[0]
    half = rows // 2
    if rows > 1 and not far > half:
        raise AtomaError(f"a distance table of {rows} rows needs bias_max above {half}, got {far}")
    buckets: List[int] = []
    n = 0
    while True:
        buckets.append(distance_bucket(n, rows, far))
        if buckets[-1] == rows - 1:
            break
        n += 1
        if n > (1 << 22):
            raise AtomaError(f"distance table: bias_max {far} spreads {rows} rows over more than {1 << 22} distances")
    return table.to(torch.float32)[torch.tensor(buckets, dtype=torch.long)].contiguous()


def _layer_spec(i: int, l: dict) -> LayerSpec:
    if l.get("type") != "attention":
        raise AtomaError(f"layer {i}: mixer type {l.get('type')!r} is not part of the Nemasun design")
    m = l["mixer"]
    mask = m.get("mask") or {}
    att = SoftmaxAttentionSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                               scale=float(m["scale"]), window=int(mask.get("size") or 0), keep_first=int(mask.get("keep_first") or 0),
                               values_are_keys=True, out_gate=True, distance_bias=True)
    f = l.get("mlp")
    if f is None:
        return LayerSpec("softmax_attention", softmax=att, source=i)
    kind = f.get("kind")
    if kind == "dense":
        return LayerSpec("softmax_attention", softmax=att, source=i,
                         clamped_mlp=ClampedMlpSpec(ff=int(f["ff"]), limit=float(f.get("limit") or 0.0), alpha=DENSE_ALPHA,
                                                    up_shift=DENSE_UP_SHIFT, bias=True))
    if kind != "moe":
        raise AtomaError(f"layer {i}: feed-forward kind {kind!r} is not part of the Nemasun design")
    r = f["router"]
    gr = r.get("groups") or {}
    sh = f.get("shared") or None
    moe = MoeSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(f["expert"]["ff"]), limit=0.0, shared_ff=int(sh["ff"]) if sh else 0,
                  shared_limit=0.0, shared_gate=False, alpha=1.0, up_shift=0.0, renormalize=True, score="softmax", correction=True,
                  groups=int(gr.get("count") or 1), keep_groups=int(gr.get("keep") or gr.get("count") or 1),
                  identity=int(r.get("identity") or 0), scale_input=False)
    return LayerSpec("softmax_attention", softmax=att, moe=moe, source=i)


def spec_from_config(cfg: dict) -> HybridSpec:
    layers = tuple(_layer_spec(i, l) for i, l in enumerate(cfg["layers"]))
    norm = cfg.get("norm") or {}
    return HybridSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), eps=float(norm.get("eps", 1e-6)), logit_scale=1.0, layers=layers,
                      norm_offset=0.0, block_style="lanes", position="none", lanes=int(cfg.get("streams") or 1),
                      embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)))


def weights_from_checkpoint(spec: HybridSpec, cfg: dict, ckpt: Dict[str, torch.Tensor]) -> dict:
    """Checkpoint names -> the generic hybrid layout: the projections that read the same input stacked for one product, the
    experts stacked into [experts, ., .] tensors, the distance table expanded from buckets to distances."""
    W, S = spec.width, spec.lanes

    def get(name, shape):
        if name not in ckpt:
            raise AtomaError(f"tensor {name} is missing from the checkpoint")
        t = ckpt[name]
        if tuple(t.shape) != tuple(shape):
            raise AtomaError(f"tensor {name} has shape {tuple(t.shape)}, the configuration needs {tuple(shape)}")
        return t

    def lanes(prefix, q, w):
        if "streams" in cfg:
            w[f"lanes_in{q}"], w[f"lanes_out{q}"] = get(f"{prefix}hc{q}.in", (S,)), get(f"{prefix}hc{q}.out", (S,))
            w[f"lanes_mix{q}"] = get(f"{prefix}hc{q}.mix", (S, S))
        else:       # a single residual stream: x <- x + y
            w[f"lanes_in{q}"], w[f"lanes_out{q}"], w[f"lanes_mix{q}"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)

    out = {"embed": get("embed", (spec.vocab, W)), "head": get("head", (spec.vocab, W)), "final_norm": get("final.norm", (W,)), "layers": []}
    for i, (ls, lc) in enumerate(zip(spec.layers, cfg["layers"])):
        a, p = ls.softmax, f"l{i}."
        rel = ckpt.get(p + "mix.rel")
        if rel is None or rel.dim() != 2 or rel.shape[1] != a.heads:
            raise AtomaError(f"tensor {p}mix.rel is missing or not [rows, {a.heads}]")
        w = {"norm1": get(p + "norm1", (W,)),
             "w_qkv": torch.cat([get(p + "mix.q", (a.heads * a.dim, W)), get(p + "mix.k", (a.kv_heads * a.dim, W)),
                                 get(p + "mix.g", (a.heads * a.vdim, W))], 0),
             "q_norm": get(p + "mix.q.norm", (a.dim,)), "k_norm": get(p + "mix.k.norm", (a.dim,)),
             "dist_bias": expand_distance_table(rel, float(lc["mixer"]["bias_max"])),
             "w_o": get(p + "mix.o", (W, a.heads * a.vdim))}
        lanes(p, 1, w)
        q = p + "mlp."
        if ls.clamped_mlp is not None:
            f = ls.clamped_mlp
            w["norm2"] = get(p + "norm2", (W,))
            lanes(p, 2, w)
            w["w_gate_up"] = torch.cat([get(q + "gate", (f.ff, W)), get(q + "up", (f.ff, W))], 0)
            w["b_gate_up"] = torch.cat([get(q + "gate.b", (f.ff,)), get(q + "up.b", (f.ff,))], 0)
            w["w_down"], w["b_down"] = get(q + "down", (W, f.ff)), get(q + "down.b", (W,))
        elif ls.moe is not None:
            e = ls.moe
            w["norm2"] = get(p + "norm2", (W,))
            lanes(p, 2, w)
            w["w_router"] = get(q + "router", (e.experts + e.identity, W))
            w["router_correction"] = get(q + "correction", (e.experts + e.identity,))
            w["w_expert_gate_up"] = torch.stack([torch.cat([get(f"{q}e{k}.gate", (e.ff, W)), get(f"{q}e{k}.up", (e.ff, W))], 0)
                                                 for k in range(e.experts)], 0)
            w["w_expert_down"] = torch.stack([get(f"{q}e{k}.down", (W, e.ff)) for k in range(e.experts)], 0)
            if e.shared_ff > 0:
                w["w_ff_in"] = torch.cat([get(q + "shared.gate", (e.shared_ff, W)), get(q + "shared.up", (e.shared_ff, W))], 0)
                w["w_down"] = get(q + "shared.down", (W, e.shared_ff))
        out["layers"].append(w)
    return out
