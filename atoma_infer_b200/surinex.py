"""Surinex: a decoder of parallel blocks (one norm per layer; the mixer and the feed-forward read it through causal tap
filters) with three kinds of mixer and a span of layers that runs several times.

config.json gives every size and every constant that can differ between checkpoints:
  architecture "Surinex", vocab, width, norm {eps}, canon {taps} (the tap filters on the sublayers' inputs), loop {start, stop,
  times} (layers start .. stop - 1 run `times` times in a row with the same weights), and `layers`: per layer its `type`
  ("gla" | "latent_attention" | "parallel"), the mixer's sizes (`mixer`) and its feed-forward (`mlp`: null or {kind "dense", ff}).
    gla:               heads, dim, vdim, tau
    latent_attention:  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims, scaling?}
    parallel:          left  {heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling? {factor, low, high, original}}}
                       right {heads, kv_heads, dim, vdim, conv}
Fixed by the design (and therefore constants here): every pass over the looped span has a cache and state of its own; before every
pass but the first the embedding rows are added to the stream again, and before every pass a per-pass vector; x <- x + mixer(h +
taps1(h)) + ff(h + taps2(h)) with h = RMSnorm(x); plain-weight RMS norms.  Gated linear attention: q scaled by dim^(-1/2), per-channel
decay sigmoid(W_a2 W_a1 h + b)^(1 / tau), per-head RMS norm of the read-out, silu gate.  Latent attention: normed query and key/value
latents, heads laid out [dim plain | rot_dim rotated], one rotated key part for all heads, pairs (i, i + dims / 2), softmax.  The pair:
sigmoid attention with a per-head q/k norm, a per-head score bias and pairs (2i, 2i + 1) turned on queries, keys and — over all of
vdim, unscaled frequencies — values (a head's sum is turned back by the query's position), beside a gated delta rule with short
silu filters, unit-length q and k (1e-6 under the root) and q scaled by dim^(-1/2); each result RMS-normed over the width, then
averaged.  Feed-forward: W_down (silu(W_gate h) * W_up h).

Checkpoint tensors: embed, head, final.norm, loop.step [times, width], and per layer i `l<i>.norm1`, `l<i>.canon1 / canon2` [width, taps],
`l<i>.mlp.{gate, up, down}`, and under `l<i>.mix.`:
    gla:               q, k, v, g, o, norm, a1, a2, a2.b
    latent_attention:  dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o
    parallel:          left.{q, k, v, q.norm, k.norm, pb, o, out}, right.{q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o, out}
This module turns that into the generic hybrid description (hybrid.py); it has no compute of its own.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, List, Optional

import torch

from .hybrid import (DeltaRuleSpec, GatedLinearAttentionSpec, HybridSpec, LatentAttentionSpec, LayerSpec, MixerPairSpec, MlpSpec,
                     RotarySigmoidAttentionSpec, RotarySpec)
from .ops import AtomaError

ARCHITECTURE = "Surinex"
MIXERS = {"gla": "gla", "latent_attention": "latent_attention", "parallel": "pair"}


def _rotary(rot: Optional[dict], default_dims: int, interleaved: bool) -> Optional[RotarySpec]:
    if not rot:
        return None
    sc = rot.get("scaling")
    scaling = None if not sc else (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
    layout = rot.get("layout")
    if layout is not None:
        if layout not in ("interleaved", "halves"):
            raise AtomaError(f"unknown rotary layout {layout!r}")
        interleaved = layout == "interleaved"
    return RotarySpec(dims=int(rot.get("dims", default_dims)), base=float(rot.get("base", 10000.0)), interleaved=interleaved, scaling=scaling)


def _mlp(i: int, f: Optional[dict]) -> Optional[MlpSpec]:
    if f is None:
        return None
    if f.get("kind", "dense") != "dense":
        raise AtomaError(f"layer {i}: feed-forward kind {f.get('kind')!r} is not part of the Surinex design")
    return MlpSpec(ff=int(f["ff"]), act="silu")


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer index, number of the pass that starts with this run or None), one entry per layer run in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not (0 <= start < stop <= n) or times < 1:
        raise AtomaError(f"loop over layers {start} .. {stop - 1}, {times} times, in a model of {n} layers")
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def _layer_spec(i: int, l: dict, taps: int, start_of_pass: Optional[int]) -> LayerSpec:
    kind, m = l.get("type"), l["mixer"]
    if kind not in MIXERS:
        raise AtomaError(f"layer {i}: mixer type {kind!r} is not part of the Surinex design")
    common = dict(mlp=_mlp(i, l.get("mlp")), source=i, taps=taps, add_embedding=start_of_pass is not None and start_of_pass > 0,
                  pass_vector=start_of_pass)
    if kind == "gla":
        return LayerSpec("gla", gla=GatedLinearAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), decay_rank=0,
                                                             tau=float(m["tau"])), **common)
    if kind == "latent_attention":
        rot_dim = int(m.get("rot_dim", 0))
        return LayerSpec("latent_attention",
                         latent=LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), q_rank=int(m["q_rank"]),
                                                    kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot_dim=rot_dim,
                                                    rotary=_rotary(m.get("rot") or ({"dims": rot_dim} if rot_dim else None), rot_dim, False)),
                         **common)
    a, d = m["left"], m["right"]
    left = RotarySigmoidAttentionSpec(heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]), vdim=int(a["vdim"]),
                                      scale=float(a["scale"]), rotary=_rotary(a.get("rot"), int(a["dim"]), True), rotate_values=True)
    right = DeltaRuleSpec(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), taps=int(d["conv"]))
    return LayerSpec("pair", pair=MixerPairSpec(left, right), **common)


def spec_from_config(cfg: dict, ckpt_shapes: Optional[Dict[str, tuple]] = None) -> HybridSpec:
    """`ckpt_shapes` (tensor name -> shape) supplies what config.json leaves to the tensors: the rank of the decay's projections."""
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    layers = []
    for i, start_of_pass in layer_runs(cfg):
        ls = _layer_spec(i, cfg["layers"][i], taps, start_of_pass)
        if ls.gla is not None:
            shape = (ckpt_shapes or {}).get(f"l{i}.mix.a1")
            if shape is None or len(shape) != 2:
                raise AtomaError(f"layer {i}: the decay's first projection l{i}.mix.a1 gives its rank; it is missing")
            ls = replace(ls, gla=replace(ls.gla, decay_rank=int(shape[0])))
        layers.append(ls)
    norm = cfg.get("norm") or {}
    return HybridSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), eps=float(norm.get("eps", 1e-6)), logit_scale=1.0, layers=tuple(layers),
                      norm_offset=0.0, block_style="parallel", position="none")


def weights_from_checkpoint(spec: HybridSpec, cfg: dict, ckpt: Dict[str, torch.Tensor]) -> dict:
    """Checkpoint names -> the generic hybrid layout (one entry per LAYER; the runs of a looped layer share it)."""
    W = spec.width

    def get(name, shape):
        if name not in ckpt:
            raise AtomaError(f"tensor {name} is missing from the checkpoint")
        t = ckpt[name]
        if tuple(t.shape) != tuple(shape):
            raise AtomaError(f"tensor {name} has shape {tuple(t.shape)}, the configuration needs {tuple(shape)}")
        return t

    out = {"embed": get("embed", (spec.vocab, W)), "head": get("head", (spec.vocab, W)), "final_norm": get("final.norm", (W,)), "layers": []}
    loop = cfg.get("loop")
    if loop:
        out["pass_vectors"] = get("loop.step", (int(loop["times"]), W))
    by_layer = {}
    for ls in spec.layers:
        by_layer.setdefault(ls.source, ls)
    for i in range(len(cfg["layers"])):
        ls, p = by_layer[i], f"l{i}."
        w = {"norm1": get(p + "norm1", (W,))}
        if ls.taps >= 1:
            w["tap_w1"] = get(p + "canon1", (W, ls.taps))
        if ls.mlp is not None:
            F = ls.mlp.ff
            w["w_gate_up"] = torch.cat([get(p + "mlp.gate", (F, W)), get(p + "mlp.up", (F, W))], 0)
            w["w_down"] = get(p + "mlp.down", (W, F))
            if ls.taps >= 1:
                w["tap_w2"] = get(p + "canon2", (W, ls.taps))
        q = p + "mix."
        if ls.gla is not None:
            a = ls.gla
            w.update(w_q=get(q + "q", (a.heads * a.dim, W)), w_k=get(q + "k", (a.heads * a.dim, W)), w_v=get(q + "v", (a.heads * a.vdim, W)),
                     w_g=get(q + "g", (a.heads * a.vdim, W)), w_a1=get(q + "a1", (a.decay_rank, W)),
                     w_a2=get(q + "a2", (a.heads * a.dim, a.decay_rank)), a2_bias=get(q + "a2.b", (a.heads * a.dim,)),
                     head_norm=get(q + "norm", (a.vdim,)), w_o=get(q + "o", (W, a.heads * a.vdim)))
        elif ls.latent is not None:
            a = ls.latent
            w.update(w_dq=get(q + "dq", (a.q_rank, W)), dq_norm=get(q + "dq.norm", (a.q_rank,)),
                     w_uq=get(q + "uq", (a.heads * (a.dim + a.rot_dim), a.q_rank)), w_dkv=get(q + "dkv", (a.kv_rank + a.rot_dim, W)),
                     dkv_norm=get(q + "dkv.norm", (a.kv_rank,)), w_uk=get(q + "uk", (a.heads * a.dim, a.kv_rank)),
                     w_uv=get(q + "uv", (a.heads * a.vdim, a.kv_rank)), w_o=get(q + "o", (W, a.heads * a.vdim)))
        else:
            a, d = ls.pair.left, ls.pair.right
            l_, r_ = q + "left.", q + "right."
            nqk, nv = d.kv_heads * d.dim, d.heads * d.vdim
            w.update(w_q=get(l_ + "q", (a.heads * a.dim, W)), w_k=get(l_ + "k", (a.kv_heads * a.dim, W)), w_v=get(l_ + "v", (a.kv_heads * a.vdim, W)),
                     q_norm=get(l_ + "q.norm", (a.dim,)), k_norm=get(l_ + "k.norm", (a.dim,)), head_bias=get(l_ + "pb", (a.heads,)),
                     w_o=get(l_ + "o", (W, a.heads * a.vdim)), out_norm_a=get(l_ + "out", (W,)),
                     r_w_q=get(r_ + "q", (nqk, W)), r_w_k=get(r_ + "k", (nqk, W)), r_w_v=get(r_ + "v", (nv, W)), r_w_g=get(r_ + "g", (nv, W)),
                     r_w_b=get(r_ + "b", (d.heads, W)), r_w_a=get(r_ + "a", (d.heads, W)), r_tap_q=get(r_ + "q.conv", (nqk, d.taps)),
                     r_tap_k=get(r_ + "k.conv", (nqk, d.taps)), r_tap_v=get(r_ + "v.conv", (nv, d.taps)), r_a_log=get(r_ + "A_log", (d.heads,)),
                     r_dt_bias=get(r_ + "dt_bias", (d.heads,)), r_head_norm=get(r_ + "norm", (d.vdim,)), r_w_o=get(r_ + "o", (W, nv)),
                     out_norm_b=get(r_ + "out", (W,)))
        out["layers"].append(w)
    return out
