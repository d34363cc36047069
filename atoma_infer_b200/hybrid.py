"""Hybrid (attention + recurrent) decoder models: description, device layout and the step executor's host side.

A model family (atoma_infer_b200/lilovik.py is the first, patadra.py the second, nemasun.py the third) describes
itself as a `HybridSpec` — a list of layer RUNS, each a mixer (sigmoid attention, minGRU, latent attention or softmax
attention) with its sizes and constants and an optional feed-forward (gated dense, or a mixture of experts) — and hands over its
weights under the generic names below.  A design that runs a span of layers several times lists every run;
runs that name the same `source` share one copy of the weights and have caches of their own.  `HybridExecutor` lays them out
on the device, owns the paged key/value caches and the recurrent-state slots, and runs one step of a MIXED
batch (portions of prompts beside single decoded tokens) through ONE C call, `atoma_hybrid_step`
(csrc/hybrid_step.cu).  The step's integer inputs are built by the same `atoma_prepare_input` /
`InputStager` that the Llama decode step uses (worker.py), with chunked prefill on.

Weight layout (rows stacked so that one GEMM makes all projections of a sublayer):
  w_qkv     [H dim + G dim + G vdim, width]   b_qkv   [same] float32
  w_zxg     [3 S, width]                      b_zxg   [3 S] float32 (zero where the design has no bias)
  w_gate_up [2 ff, width]                     w_down  [width, ff]
  w_o       [width, H vdim] or [width, S]
  norms, q/k norm weights, talking-heads matrix, per-head bias and distance slopes: float32.
Pre-norm designs (block_style "prenorm"):
  w_down_in [q_rank + kv_rank (+ width), width]   query latent, key/value latent, residual gate rows
  w_uq [H dim, q_rank]   w_uk [H dim, kv_rank]   w_uv [H vdim, kv_rank]   dq_norm, dkv_norm, sink, gate biases: float32
  w_ff_in [2 shared_ff (+ width), width]   w_down [width, shared_ff]   w_router [experts, width] float32
  w_expert_gate_up [experts, 2 ff, width]   w_expert_down [experts, width, ff]   side_gate, side_proj, side_norm
Designs on residual lanes (block_style "lanes"):
  w_qkv [H dim + G dim (+ G vdim unless the values are the keys) (+ H vdim with an output gate), width]   w_o [width, H vdim]
  q_norm, k_norm [dim]   dist_bias [rows, H] float32 (bias by query-key distance, the last row for every larger distance)
  lanes_in1/out1 [lanes], lanes_mix1 [lanes, lanes] (and ..2 for the feed-forward), all float32
  dense: w_gate_up [2 ff, width], b_gate_up [2 ff], w_down [width, ff], b_down [width]
  experts: w_router [experts + identity, width] float32, router_correction [same], w_expert_gate_up, w_expert_down,
           shared expert w_ff_in [2 shared_ff, width], w_down [width, shared_ff]
Parallel blocks (block_style "parallel": one norm per layer, x += mixer(f1(h)) + ff(f2(h)) with causal tap filters f1, f2):
  norm1 [width]   tap_w1, tap_w2 [width, taps] float32   w_gate_up [2 ff, width]   w_down [width, ff]
  gated linear attention: w_q, w_k [H dim, width], w_v, w_g [H vdim, width], w_a1 [rank, width], w_a2 [H dim, rank], a2_bias [H dim],
                          head_norm [vdim], w_o [width, H vdim]
  latent attention with a rotated key part: w_dq [q_rank, width], w_dkv [kv_rank + rot_dim, width], dq_norm, dkv_norm, w_uq
                          [H (dim + rot_dim), q_rank], w_uk [H dim, kv_rank], w_uv [H vdim, kv_rank], w_o [width, H vdim]
  pair of mixers: left  w_q [H dim, width], w_k [G dim, width], w_v [G vdim, width], q_norm, k_norm [dim], head_bias [H], w_o
                  right r_w_q, r_w_k [G' dim', width], r_w_v, r_w_g [H' vdim', width], r_w_b, r_w_a [H', width], r_tap_q / r_tap_k / r_tap_v
                        [channels, taps'], r_a_log, r_dt_bias [H'], r_head_norm [vdim'], r_w_o [width, H' vdim']
                  out_norm_a, out_norm_b [width]
  the model: pass_vectors [passes, width] float32 (the vector added at the start of every pass over a looped span)
The executor stacks the projections that read the same input into one matrix (rows padded to a multiple of 8).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq_

import numpy as np
import torch

from . import _lib
from ._lib import HybridBatch, HybridLayer, HybridModel
from .ops import AtomaError
from .scheduler import StepPlan
from .worker import InputStager, SequenceInput

MIXER_ATTENTION, MIXER_MINGRU, MIXER_LATENT, MIXER_SOFTMAX, MIXER_GLA, MIXER_PAIR = 0, 1, 2, 3, 4, 5
LONG_PORTION = 128        # tokens of a sequence in one step from which attention runs on the tensor-memory prefill kernel
                          # (latent attention: on expanded keys and values; softmax attention: on gathered ones)
BLOCK_STYLES = {"sandwich": 0, "prenorm": 1, "lanes": 2, "parallel": 3}
SCORE_FNS = {"sigmoid": 0, "softmax": 1}
ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}
DTYPE_CODES = {torch.bfloat16: 1, torch.float32: 2}


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0
    temp_coef: float = 0.0
    temp_every: int = 0            # 0 = no query temperature
    slopes: Optional[Seq_[float]] = None   # per-head distance slopes; None = no distance bias


@dataclass(frozen=True)
class MinGruSpec:
    width: int


@dataclass(frozen=True)
class MlpSpec:
    ff: int
    act: str = "relu"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Queries, keys and values expanded from low-rank latents; the key/value latent alone is cached."""
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int = 0                # 0 = every earlier token is visible
    sink: bool = False             # a learned per-head term of the softmax denominator
    rot_dim: int = 0               # parallel blocks: rotated entries per query head and of the one key part all heads share
    rotary: Optional["RotarySpec"] = None


@dataclass(frozen=True)
class SoftmaxAttentionSpec:
    """Softmax attention with grouped key/value heads, a per-head q/k RMS norm, a window that also keeps the first tokens,
    a bias looked up by query-key distance, and an optional sigmoid gate on the heads' outputs."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                # 0 = every earlier token is visible
    keep_first: int = 0            # tokens at the start of the sequence that stay visible behind the window
    values_are_keys: bool = False  # no value projection: the values are the key projections before their norm
    out_gate: bool = False         # heads' outputs times sigmoid(W h) before the output projection
    distance_bias: bool = False    # weights carry dist_bias [rows, heads]


@dataclass(frozen=True)
class RotarySpec:
    """Rotary positions on the first `dims` entries of a head: pair i turns by position * base^(-2 i / dims).  `scaling`
    (factor, low, high, original) stretches long wavelengths: a wavelength below original / high keeps its frequency, one
    above original / low has it divided by factor, and in between the two are blended linearly in original / wavelength."""
    dims: int
    base: float = 10000.0
    interleaved: bool = False                 # pairs (2i, 2i + 1) instead of (i, i + dims / 2)
    scaling: Optional[Seq_[float]] = None     # (factor, low, high, original)

    def frequencies(self) -> List[float]:
        out = []
        for i in range(self.dims // 2):
            f = float(self.base) ** (-2.0 * i / self.dims)
            if self.scaling is not None:
                factor, low, high, original = (float(v) for v in self.scaling)
                wave = 2.0 * math.pi / f
                if wave > original / low:
                    f = f / factor
                elif wave >= original / high:
                    t = (original / wave - low) / (high - low)
                    f = (1.0 - t) * f / factor + t * f
            out.append(f)
        return out


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """A [dim, vdim] state per head whose rows decay by sigmoid(z)^(1 / tau) per key channel, z through a low-rank pair of
    projections; the read-out is RMS-normed per head and gated by silu(W_g h)."""
    heads: int
    dim: int
    vdim: int
    decay_rank: int
    tau: float = 16.0


@dataclass(frozen=True)
class RotarySigmoidAttentionSpec:
    """Sigmoid attention (weights sigmoid(score + per-head bias), not normalised) with a per-head q/k RMS norm, rotary
    positions on queries and keys, and values that are turned by their own position over all of vdim when cached; a head's
    sum is turned back by the query's position."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rotary: Optional[RotarySpec] = None
    rotate_values: bool = True


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule: short causal filters with silu on q / k / v, unit-length q and k, write strength sigmoid(W_b h) and decay
    exp(-exp(A_log) softplus(W_a h + dt_bias)) per head, read-out RMS-normed per head and gated by silu(W_g h)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int = 4


@dataclass(frozen=True)
class MixerPairSpec:
    """Two mixers on the same input; each result is RMS-normed over the model width and the two are averaged."""
    left: RotarySigmoidAttentionSpec
    right: DeltaRuleSpec


@dataclass(frozen=True)
class ClampedMlpSpec:
    """Dense feed-forward W_down (g sigmoid(alpha g) (u + up_shift)) on g = min(W_gate h + b, limit), u = clamp(W_up h + b)."""
    ff: int
    limit: float = 0.0
    alpha: float = 1.702
    up_shift: float = 1.0
    bias: bool = True


@dataclass(frozen=True)
class MoeSpec:
    """Routed experts with a clamped gated activation g sigmoid(alpha g) (u + up_shift), and an optional shared expert.
    The defaults are a sigmoid router that scales the experts' inputs; `score`, `correction`, `groups` / `keep_groups`,
    `identity` and `scale_input` describe routers whose choice is corrected and restricted and whose weights scale outputs."""
    experts: int
    top: int
    ff: int
    limit: float = 0.0             # clamp of gate (above) and up (both sides); 0 = none
    shared_ff: int = 0             # 0 = no shared expert
    shared_limit: float = 0.0
    shared_gate: bool = False      # the shared expert's output times sigmoid(w . h)
    alpha: float = 1.702
    up_shift: float = 1.0
    renormalize: bool = False      # chosen scores divided by their sum
    score: str = "sigmoid"         # "sigmoid" | "softmax" over all router outputs
    correction: bool = False       # a per-output term added to the scores for the choice only
    groups: int = 1                # router outputs form this many equal groups of neighbours ...
    keep_groups: int = 1           # ... of which only the best may be chosen from
    identity: int = 0              # router outputs after the experts that hand the token's input through
    scale_input: bool = True       # the router's weight multiplies the expert's input (False: its output)


@dataclass(frozen=True)
class LayerSpec:
    mixer: str                               # "attention" | "mingru" | "latent_attention" | "softmax_attention"
    attention: Optional[AttentionSpec] = None
    mingru: Optional[MinGruSpec] = None
    mlp: Optional[MlpSpec] = None
    latent: Optional[LatentAttentionSpec] = None
    moe: Optional[MoeSpec] = None
    softmax: Optional[SoftmaxAttentionSpec] = None
    clamped_mlp: Optional[ClampedMlpSpec] = None
    gated_residual: bool = False             # sublayer results times sigmoid(W h + b) before they join the stream
    side_part: Optional[int] = None          # which part of the token side table the layer reads; None = no side input
    source: Optional[int] = None             # entry of weights["layers"] the run uses; None = its own index
    gla: Optional["GatedLinearAttentionSpec"] = None
    pair: Optional["MixerPairSpec"] = None
    taps: int = 0                            # parallel blocks: taps of the filters on the sublayers' inputs (0: none)
    add_embedding: bool = False              # parallel blocks: the embedding rows are added to the stream before the layer
    pass_vector: Optional[int] = None        # ... and this row of weights["pass_vectors"]


@dataclass(frozen=True)
class HybridSpec:
    width: int
    vocab: int
    eps: float
    logit_scale: float
    layers: Seq_[LayerSpec] = ()
    norm_offset: float = 1.0                 # norm weights are stored as offsets from this value
    position_base: float = 10000.0
    block_style: str = "sandwich"            # "sandwich": x += norm(f(norm x));  "prenorm": x += gate * f(norm x)
    norm_groups: int = 1                     # RMS statistics over this many equal consecutive parts of the row
    position: str = "sinusoid"               # "sinusoid" | "learned" (a table of max_positions rows)
    max_positions: int = 0
    logit_softcap: float = 0.0               # logits <- cap * tanh(logits / cap); 0 = none
    side_dim: int = 0                        # width of one layer's part of the token side table
    lanes: int = 0                           # block_style "lanes": copies of the residual stream
    embed_scale: float = 1.0                 # block_style "lanes": the embedding row times this (no position signal)

    @property
    def has_state(self) -> bool:
        return any(l.mixer == "mingru" or l.taps > 1 or l.gla is not None or l.pair is not None for l in self.layers)

    def cache_bytes_per_token(self, dtype: torch.dtype) -> int:
        es = torch.empty((), dtype=dtype).element_size()
        return (sum(l.attention.kv_heads * (l.attention.dim + l.attention.vdim) * es for l in self.layers if l.mixer == "attention") +
                sum(l.softmax.kv_heads * (l.softmax.dim + l.softmax.vdim) * es for l in self.layers if l.mixer == "softmax_attention") +
                sum((l.latent.kv_rank + l.latent.rot_dim) * es for l in self.layers if l.mixer == "latent_attention") +
                sum(l.pair.left.kv_heads * (l.pair.left.dim + l.pair.left.vdim) * es for l in self.layers if l.pair is not None))


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor]           # float32 [num_selected, vocab] on the device (a view, valid until the next step)
    next_tokens: Optional[torch.Tensor]      # int32 [num_selected]: greedy choice
    rows: List[tuple] = field(default_factory=list)   # (seq_id, offset in its chunk) per selected row
    residual_trace: Optional[torch.Tensor] = None


class HybridExecutor:
    """Device state of one hybrid model + `execute(plan)`."""

    def __init__(self, spec: HybridSpec, weights: Dict[str, object], dtype: torch.dtype, device, num_blocks: int,
                 block_size: int = 16, num_state_slots: int = 4):
        if dtype not in DTYPE_CODES:
            raise AtomaError(f"hybrid models run in bfloat16 or float32, not {dtype}")
        if not torch.cuda.is_available():
            raise AtomaError("hybrid models need a CUDA device: there is no CPU path")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.block_size, self.num_blocks, self.num_state_slots = int(block_size), int(num_blocks), int(num_state_slots)
        self._keep: List[torch.Tensor] = []
        dev = self.device

        def big(t):          # matrices: the activation format
            t = t.to(dtype).contiguous().to(dev)
            self._keep.append(t)
            return t

        def small(t):        # per-channel parameters: float32
            t = torch.as_tensor(t).to(torch.float32).contiguous().to(dev)
            self._keep.append(t)
            return t

        if spec.block_style not in BLOCK_STYLES:
            raise AtomaError(f"unknown block style {spec.block_style!r}")
        self.embed, self.head = big(weights["embed"]), big(weights["head"])
        self.final_norm = small(weights["final_norm"])
        self.inv_freq = self.pos_table = self.side_table = None
        if spec.block_style == "lanes":
            if not 1 <= spec.lanes <= 16:
                raise AtomaError(f"{spec.lanes} residual lanes (1 to 16 are supported)")
        elif spec.block_style == "parallel":
            pass                  # positions enter through the mixers' rotations
        elif spec.position == "learned":
            self.pos_table = big(weights["pos"])
            if self.pos_table.shape[0] < spec.max_positions or spec.max_positions <= 0:
                raise AtomaError(f"position table of {self.pos_table.shape[0]} rows for {spec.max_positions} positions")
        else:
            half = (spec.width + 1) // 2
            inv = np.array([spec.position_base ** (-2.0 * i / spec.width) for i in range(half)], dtype=np.float64)
            self.inv_freq = torch.from_numpy(inv).to(dev)
        if spec.side_dim > 0:
            self.side_table = big(weights["side_table"])
        self.k_caches: List[Optional[torch.Tensor]] = []
        self.v_caches: List[Optional[torch.Tensor]] = []
        self.latent_caches: List[Optional[torch.Tensor]] = []
        self.states: List[Optional[torch.Tensor]] = []
        self._layers = (HybridLayer * len(spec.layers))()
        rows = self.num_blocks * self.block_size
        placed: Dict[int, HybridLayer] = {}      # weights already on the device, by their entry of weights["layers"]
        for i, ls in enumerate(spec.layers):
            L = self._layers[i]
            src = i if ls.source is None else ls.source
            w = weights["layers"][src]
            if spec.block_style == "lanes":
                if src in placed:
                    C.memmove(C.byref(L), C.byref(placed[src]), C.sizeof(HybridLayer))
                else:
                    self._place_lanes(L, i, ls, w, big, small)
                    placed[src] = L
                a = ls.softmax
                kc = torch.zeros((rows, a.kv_heads, a.dim), dtype=dtype, device=dev)
                vc = torch.zeros((rows, a.kv_heads, a.vdim), dtype=dtype, device=dev)
                L.k_cache, L.v_cache = kc.data_ptr(), vc.data_ptr()
                self.k_caches.append(kc)
                self.v_caches.append(vc)
                self.states.append(None)
                self.latent_caches.append(None)
                continue
            if spec.block_style == "parallel":
                if src in placed:
                    C.memmove(C.byref(L), C.byref(placed[src]), C.sizeof(HybridLayer))     # same weights; caches, state and pass start below
                else:
                    self._place_parallel(L, i, ls, w, big, small)
                    placed[src] = L
                self._parallel_run_state(L, i, ls, weights, small, rows)
                continue
            if spec.block_style == "prenorm":
                if src in placed:
                    C.memmove(C.byref(L), C.byref(placed[src]), C.sizeof(HybridLayer))     # same weights, a cache of its own below
                else:
                    self._place_prenorm(L, i, ls, w, big, small)
                    placed[src] = L
                lc = torch.zeros((rows, ls.latent.kv_rank), dtype=dtype, device=dev)
                L.latent_cache = lc.data_ptr()
                self.k_caches.append(None)
                self.v_caches.append(None)
                self.states.append(None)
                self.latent_caches.append(lc)
                continue
            self.latent_caches.append(None)
            L.norm1, L.norm1b = small(w["norm1"]).data_ptr(), small(w["norm1b"]).data_ptr()
            L.has_mlp = 1 if ls.mlp is not None else 0
            kc = vc = st = None
            if ls.mixer == "attention":
                a = ls.attention
                if a.heads % a.kv_heads:
                    raise AtomaError(f"layer {i}: {a.kv_heads} kv heads do not divide {a.heads} heads")
                L.mixer = MIXER_ATTENTION
                L.heads, L.kv_heads, L.dim, L.vdim, L.temp_every = a.heads, a.kv_heads, a.dim, a.vdim, a.temp_every
                L.scale, L.softcap, L.temp_coef = a.scale, a.softcap, a.temp_coef
                L.w_qkv, L.b_qkv = big(w["w_qkv"]).data_ptr(), small(w["b_qkv"]).data_ptr()
                L.q_norm, L.k_norm = small(w["q_norm"]).data_ptr(), small(w["k_norm"]).data_ptr()
                L.talk = small(w["talk"]).data_ptr() if w.get("talk") is not None else None
                L.head_bias = small(w["head_bias"] if w.get("head_bias") is not None else torch.zeros(a.heads)).data_ptr()
                L.slopes = small(torch.tensor(list(a.slopes) if a.slopes is not None else [0.0] * a.heads)).data_ptr()
                kc = torch.zeros((rows, a.kv_heads, a.dim), dtype=dtype, device=dev)
                vc = torch.zeros((rows, a.kv_heads, a.vdim), dtype=dtype, device=dev)
                L.k_cache, L.v_cache = kc.data_ptr(), vc.data_ptr()
            elif ls.mixer == "mingru":
                L.mixer = MIXER_MINGRU
                L.state_width = ls.mingru.width
                L.w_zxg, L.b_zxg = big(w["w_zxg"]).data_ptr(), small(w["b_zxg"]).data_ptr()
                st = torch.zeros((max(1, self.num_state_slots), ls.mingru.width), dtype=torch.float32, device=dev)
                L.state = st.data_ptr()
            else:
                raise AtomaError(f"layer {i}: unknown mixer {ls.mixer!r}")
            L.w_o = big(w["w_o"]).data_ptr()
            if ls.mlp is not None:
                if ls.mlp.act not in ACTIVATIONS:
                    raise AtomaError(f"layer {i}: unknown activation {ls.mlp.act!r}")
                L.norm2, L.norm2b = small(w["norm2"]).data_ptr(), small(w["norm2b"]).data_ptr()
                L.ff, L.act = ls.mlp.ff, ACTIVATIONS[ls.mlp.act]
                L.w_gate_up, L.w_down = big(w["w_gate_up"]).data_ptr(), big(w["w_down"]).data_ptr()
            self.k_caches.append(kc)
            self.v_caches.append(vc)
            self.states.append(st)
        m = HybridModel()
        m.width, m.vocab, m.num_layers, m.block_size = spec.width, spec.vocab, len(spec.layers), self.block_size
        m.eps, m.logit_scale, m.norm_offset, m.dtype = spec.eps, spec.logit_scale, spec.norm_offset, DTYPE_CODES[dtype]
        m.embed = self.embed.data_ptr()
        m.inv_freq = self.inv_freq.data_ptr() if self.inv_freq is not None else None
        m.final_norm, m.head = self.final_norm.data_ptr(), self.head.data_ptr()
        m.layers = C.cast(self._layers, C.POINTER(HybridLayer))
        m.block_style, m.norm_groups = BLOCK_STYLES[spec.block_style], spec.norm_groups
        m.pos_table = self.pos_table.data_ptr() if self.pos_table is not None else None
        m.max_positions, m.logit_softcap = spec.max_positions, spec.logit_softcap
        if self.side_table is not None:
            m.side_table, m.side_dim, m.side_table_width = self.side_table.data_ptr(), spec.side_dim, self.side_table.shape[1]
        m.lanes, m.embed_scale = spec.lanes, spec.embed_scale
        self._model = m
        self._stager = InputStager(device=dev, block_size=self.block_size, enable_chunked_prefill=True)
        self._extra_host = None
        self._extra_dev = None
        self._scratch = None
        self._logits = None
        self._next = None
        self.launches_last_step = 0

    def _place_prenorm(self, L, i: int, ls: LayerSpec, w: dict, big, small) -> None:
        """Device copies and sizes of one pre-norm layer (latent attention, optional experts, optional side input)."""
        if ls.mixer != "latent_attention" or ls.latent is None:
            raise AtomaError(f"layer {i}: pre-norm blocks take the latent-attention mixer, not {ls.mixer!r}")
        a = ls.latent
        L.mixer = MIXER_LATENT
        L.heads, L.kv_heads, L.dim, L.vdim = a.heads, 1, a.dim, a.vdim
        L.q_rank, L.kv_rank, L.window, L.scale = a.q_rank, a.kv_rank, a.window, a.scale
        L.norm1 = small(w["norm1"]).data_ptr()
        L.w_down_in = big(w["w_down_in"]).data_ptr()
        L.dq_norm, L.dkv_norm = small(w["dq_norm"]).data_ptr(), small(w["dkv_norm"]).data_ptr()
        L.sink = small(w["sink"]).data_ptr() if a.sink else None
        L.w_uq, L.w_uk, L.w_uv, L.w_o = (big(w[k]).data_ptr() for k in ("w_uq", "w_uk", "w_uv", "w_o"))
        L.gate1_bias = small(w["gate1_bias"]).data_ptr() if ls.gated_residual else None
        has_ff = ls.moe is not None or ls.mlp is not None
        L.has_mlp = 1 if has_ff else 0
        if has_ff:
            L.norm2 = small(w["norm2"]).data_ptr()
            L.gate2_bias = small(w["gate2_bias"]).data_ptr() if ls.gated_residual else None
        if ls.moe is not None:
            e = ls.moe
            if not 0 < e.top <= e.experts:
                raise AtomaError(f"layer {i}: top {e.top} of {e.experts} experts")
            L.ff_kind, L.renormalize = 1, 1 if e.renormalize else 0
            L.experts, L.top, L.expert_ff, L.ff = e.experts, e.top, e.ff, e.shared_ff
            L.expert_limit, L.shared_limit, L.act_alpha, L.act_up_shift = e.limit, e.shared_limit, e.alpha, e.up_shift
            L.w_router = small(w["w_router"]).data_ptr()
            L.w_expert_gate_up, L.w_expert_down = big(w["w_expert_gate_up"]).data_ptr(), big(w["w_expert_down"]).data_ptr()
            if e.shared_ff > 0:
                L.w_down = big(w["w_down"]).data_ptr()
                L.w_shared_gate = small(w["w_shared_gate"]).data_ptr() if e.shared_gate else None
            if e.shared_ff > 0 or ls.gated_residual:
                L.w_ff_in = big(w["w_ff_in"]).data_ptr()
        elif ls.mlp is not None:
            raise AtomaError(f"layer {i}: pre-norm blocks have a mixture-of-experts feed-forward or none")
        if ls.side_part is not None:
            L.side_part = ls.side_part
            L.side_gate, L.side_proj = big(w["side_gate"]).data_ptr(), big(w["side_proj"]).data_ptr()
            L.side_norm = small(w["side_norm"]).data_ptr()

    def _place_lanes(self, L, i: int, ls: LayerSpec, w: dict, big, small) -> None:
        """Device copies and sizes of one layer on residual lanes (softmax attention; dense or routed feed-forward or none)."""
        if ls.mixer != "softmax_attention" or ls.softmax is None:
            raise AtomaError(f"layer {i}: blocks on residual lanes take the softmax-attention mixer, not {ls.mixer!r}")
        a, S = ls.softmax, self.spec.lanes
        if a.heads % a.kv_heads:
            raise AtomaError(f"layer {i}: {a.kv_heads} kv heads do not divide {a.heads} heads")
        if a.values_are_keys and a.vdim != a.dim:
            raise AtomaError(f"layer {i}: values that are the key projections need vdim = dim, got {a.vdim} and {a.dim}")
        L.mixer = MIXER_SOFTMAX
        L.heads, L.kv_heads, L.dim, L.vdim = a.heads, a.kv_heads, a.dim, a.vdim
        L.scale, L.window, L.keep_first = a.scale, a.window, a.keep_first
        L.values_are_keys, L.out_gate = int(a.values_are_keys), int(a.out_gate)
        n_in = a.heads * a.dim + a.kv_heads * a.dim + (0 if a.values_are_keys else a.kv_heads * a.vdim) + (a.heads * a.vdim if a.out_gate else 0)
        if tuple(w["w_qkv"].shape) != (n_in, self.spec.width):
            raise AtomaError(f"layer {i}: stacked projection of shape {tuple(w['w_qkv'].shape)}, expected {(n_in, self.spec.width)}")
        L.norm1 = small(w["norm1"]).data_ptr()
        L.w_qkv, L.w_o = big(w["w_qkv"]).data_ptr(), big(w["w_o"]).data_ptr()
        L.q_norm, L.k_norm = small(w["q_norm"]).data_ptr(), small(w["k_norm"]).data_ptr()
        if a.distance_bias:
            db = small(w["dist_bias"])
            if db.dim() != 2 or db.shape[1] != a.heads or db.shape[0] < 1:
                raise AtomaError(f"layer {i}: distance table of shape {tuple(db.shape)} for {a.heads} heads")
            L.dist_bias, L.dist_rows = db.data_ptr(), db.shape[0]

        def lane_weights(q):
            t_in, t_out, t_mix = small(w[f"lanes_in{q}"]), small(w[f"lanes_out{q}"]), small(w[f"lanes_mix{q}"])
            if tuple(t_in.shape) != (S,) or tuple(t_out.shape) != (S,) or tuple(t_mix.shape) != (S, S):
                raise AtomaError(f"layer {i}: lane weights of shapes {tuple(t_in.shape)}, {tuple(t_out.shape)}, {tuple(t_mix.shape)} for {S} lanes")
            return t_in.data_ptr(), t_out.data_ptr(), t_mix.data_ptr()

        L.lanes_in1, L.lanes_out1, L.lanes_mix1 = lane_weights(1)
        if ls.clamped_mlp is None and ls.moe is None:
            L.has_mlp = 0
            return
        L.has_mlp = 1
        L.norm2 = small(w["norm2"]).data_ptr()
        L.lanes_in2, L.lanes_out2, L.lanes_mix2 = lane_weights(2)
        if ls.clamped_mlp is not None:
            f = ls.clamped_mlp
            L.ff_kind, L.ff = 0, f.ff
            L.expert_limit, L.act_alpha, L.act_up_shift = f.limit, f.alpha, f.up_shift
            L.w_gate_up, L.w_down = big(w["w_gate_up"]).data_ptr(), big(w["w_down"]).data_ptr()
            if f.bias:
                L.b_gate_up, L.b_down = small(w["b_gate_up"]).data_ptr(), small(w["b_down"]).data_ptr()
            return
        e = ls.moe
        outputs = e.experts + e.identity
        if e.score not in SCORE_FNS:
            raise AtomaError(f"layer {i}: unknown router score {e.score!r}")
        if not 0 < e.top <= outputs or e.experts < 1:
            raise AtomaError(f"layer {i}: top {e.top} of {outputs} router outputs ({e.experts} experts)")
        if e.groups < 1 or outputs % e.groups or not 1 <= e.keep_groups <= e.groups:
            raise AtomaError(f"layer {i}: {outputs} router outputs in {e.groups} groups, {e.keep_groups} kept")
        L.ff_kind, L.renormalize, L.score_fn, L.scale_input = 1, int(e.renormalize), SCORE_FNS[e.score], int(e.scale_input)
        L.experts, L.top, L.expert_ff, L.ff = e.experts, e.top, e.ff, e.shared_ff
        L.identity_experts, L.route_groups, L.route_keep = e.identity, e.groups, e.keep_groups
        L.expert_limit, L.shared_limit, L.act_alpha, L.act_up_shift = e.limit, e.shared_limit, e.alpha, e.up_shift
        L.w_router = small(w["w_router"]).data_ptr()
        if e.correction:
            L.router_correction = small(w["router_correction"]).data_ptr()
        L.w_expert_gate_up, L.w_expert_down = big(w["w_expert_gate_up"]).data_ptr(), big(w["w_expert_down"]).data_ptr()
        if e.shared_ff > 0:
            L.w_ff_in, L.w_down = big(w["w_ff_in"]).data_ptr(), big(w["w_down"]).data_ptr()

    def _place_parallel(self, L, i: int, ls: LayerSpec, w: dict, big, small) -> None:
        """Device copies and sizes of one parallel layer: the projections that read the mixer's input stacked into one matrix
        (every part starts at a multiple of 8 rows, so that each has 16-byte aligned columns in the product)."""
        W = self.spec.width

        def need(name, shape):
            t = w.get(name)
            if t is None or tuple(t.shape) != tuple(shape):
                raise AtomaError(f"layer {i}: tensor {name} is {None if t is None else tuple(t.shape)}, the description needs {tuple(shape)}")
            return t

        parts: List[torch.Tensor] = []
        offsets: Dict[str, int] = {}

        def stack(key, name, rows):
            t = need(name, (rows, W))
            offsets[key] = sum(p.shape[0] for p in parts)
            parts.append(t)
            pad = -rows % 8
            if pad:
                parts.append(torch.zeros((pad, W), dtype=t.dtype))

        L.norm1 = small(need("norm1", (W,))).data_ptr()
        L.taps = max(0, int(ls.taps))
        if ls.taps > 16:
            raise AtomaError(f"layer {i}: {ls.taps} taps (at most 16 are supported)")
        if ls.taps >= 1:
            L.tap_w1 = small(need("tap_w1", (W, ls.taps))).data_ptr()
        f = ls.mlp
        L.has_mlp = 1 if f is not None else 0
        if f is not None:
            if f.act not in ACTIVATIONS:
                raise AtomaError(f"layer {i}: unknown activation {f.act!r}")
            L.ff, L.act = f.ff, ACTIVATIONS[f.act]
            L.w_gate_up, L.w_down = big(need("w_gate_up", (2 * f.ff, W))).data_ptr(), big(need("w_down", (W, f.ff))).data_ptr()
            if ls.taps >= 1:
                L.tap_w2 = small(need("tap_w2", (W, ls.taps))).data_ptr()
        if ls.mixer == "gla":
            a = ls.gla
            L.mixer = MIXER_GLA
            L.heads, L.kv_heads, L.dim, L.vdim, L.tau, L.scale = a.heads, a.heads, a.dim, a.vdim, a.tau, a.dim ** -0.5
            if not a.tau > 0:
                raise AtomaError(f"layer {i}: tau must be positive, got {a.tau}")
            stack("q", "w_q", a.heads * a.dim)
            stack("k", "w_k", a.heads * a.dim)
            stack("v", "w_v", a.heads * a.vdim)
            stack("g", "w_g", a.heads * a.vdim)
            L.proj_cols = sum(p.shape[0] for p in parts)
            stack("a", "w_a1", a.decay_rank)              # behind the stacked product's rows: a product of its own
            L.q_off, L.k_off, L.v_off, L.g_off, L.a_off = (offsets[k] for k in "qkvga")
            L.a_rank = a.decay_rank
            L.w_a2 = big(need("w_a2", (a.heads * a.dim, a.decay_rank))).data_ptr()
            L.a2_bias = small(need("a2_bias", (a.heads * a.dim,))).data_ptr()
            L.head_norm = small(need("head_norm", (a.vdim,))).data_ptr()
            L.w_o = big(need("w_o", (W, a.heads * a.vdim))).data_ptr()
        elif ls.mixer == "latent_attention":
            a = ls.latent
            L.mixer = MIXER_LATENT
            L.heads, L.kv_heads, L.dim, L.vdim = a.heads, 1, a.dim, a.vdim
            L.q_rank, L.kv_rank, L.window, L.scale, L.rot_dim = a.q_rank, a.kv_rank, a.window, a.scale, a.rot_dim
            parts.extend([need("w_dq", (a.q_rank, W)), need("w_dkv", (a.kv_rank + a.rot_dim, W))])   # [c_q | c | rotated key part], no padding
            L.proj_cols = sum(p.shape[0] for p in parts)
            L.dq_norm, L.dkv_norm = small(need("dq_norm", (a.q_rank,))).data_ptr(), small(need("dkv_norm", (a.kv_rank,))).data_ptr()
            L.w_uq = big(need("w_uq", (a.heads * (a.dim + a.rot_dim), a.q_rank))).data_ptr()
            L.w_uk = big(need("w_uk", (a.heads * a.dim, a.kv_rank))).data_ptr()
            L.w_uv = big(need("w_uv", (a.heads * a.vdim, a.kv_rank))).data_ptr()
            L.w_o = big(need("w_o", (W, a.heads * a.vdim))).data_ptr()
            if a.rot_dim > 0:
                r = a.rotary or RotarySpec(dims=a.rot_dim)
                if r.dims > a.rot_dim or r.dims % 2:
                    raise AtomaError(f"layer {i}: {r.dims} rotated entries in a part of {a.rot_dim}")
                L.qk_freq, L.rot_pairs, L.rot_interleaved = small(torch.tensor(r.frequencies(), dtype=torch.float64)).data_ptr(), r.dims // 2, int(r.interleaved)
        elif ls.mixer == "pair":
            a, d = ls.pair.left, ls.pair.right
            L.mixer = MIXER_PAIR
            if a.heads % a.kv_heads or d.heads % d.kv_heads:
                raise AtomaError(f"layer {i}: key/value heads ({a.kv_heads}, {d.kv_heads}) must divide the heads ({a.heads}, {d.heads})")
            L.heads, L.kv_heads, L.dim, L.vdim, L.scale = a.heads, a.kv_heads, a.dim, a.vdim, a.scale
            stack("q", "w_q", a.heads * a.dim)
            stack("k", "w_k", a.kv_heads * a.dim)
            stack("v", "w_v", a.kv_heads * a.vdim)
            # the filtered columns q, k, v of the right mixer are neighbours: padding only after the three
            rq = need("r_w_q", (d.kv_heads * d.dim, W))
            rk = need("r_w_k", (d.kv_heads * d.dim, W))
            rv = need("r_w_v", (d.heads * d.vdim, W))
            offsets["rq"] = sum(p.shape[0] for p in parts)
            offsets["rk"], offsets["rv"] = offsets["rq"] + rq.shape[0], offsets["rq"] + rq.shape[0] + rk.shape[0]
            parts.extend([rq, rk, rv])
            pad = -(rq.shape[0] + rk.shape[0] + rv.shape[0]) % 8
            if pad:
                parts.append(torch.zeros((pad, W), dtype=rq.dtype))
            stack("rg", "r_w_g", d.heads * d.vdim)
            stack("rb", "r_w_b", d.heads)
            stack("ra", "r_w_a", d.heads)
            L.proj_cols = sum(p.shape[0] for p in parts)
            L.q_off, L.k_off, L.v_off = offsets["q"], offsets["k"], offsets["v"]
            L.rq_off, L.rk_off, L.rv_off, L.rg_off, L.rb_off, L.ra_off = (offsets[k] for k in ("rq", "rk", "rv", "rg", "rb", "ra"))
            L.q_norm, L.k_norm = small(need("q_norm", (a.dim,))).data_ptr(), small(need("k_norm", (a.dim,))).data_ptr()
            L.head_bias = small(need("head_bias", (a.heads,))).data_ptr()
            L.slopes = small(torch.zeros(a.heads)).data_ptr()
            L.w_o = big(need("w_o", (W, a.heads * a.vdim))).data_ptr()
            if a.rotary is not None:
                r = a.rotary
                if r.dims > a.dim or r.dims % 2:
                    raise AtomaError(f"layer {i}: {r.dims} rotated entries in a head of {a.dim}")
                L.qk_freq, L.rot_pairs, L.rot_interleaved = small(torch.tensor(r.frequencies(), dtype=torch.float64)).data_ptr(), r.dims // 2, int(r.interleaved)
                if a.rotate_values:
                    if a.vdim % 2:
                        raise AtomaError(f"layer {i}: rotated values need an even vdim, got {a.vdim}")
                    fv = RotarySpec(dims=a.vdim, base=r.base, interleaved=r.interleaved).frequencies()
                    L.v_freq, L.v_pairs = small(torch.tensor(fv, dtype=torch.float64)).data_ptr(), a.vdim // 2
            if not 1 <= d.taps <= 16:
                raise AtomaError(f"layer {i}: {d.taps} taps of the short filters (1 to 16 are supported)")
            L.r_heads, L.r_kv_heads, L.r_dim, L.r_vdim, L.r_taps = d.heads, d.kv_heads, d.dim, d.vdim, d.taps
            L.r_tap_w = small(torch.cat([need("r_tap_q", (d.kv_heads * d.dim, d.taps)), need("r_tap_k", (d.kv_heads * d.dim, d.taps)),
                                         need("r_tap_v", (d.heads * d.vdim, d.taps))], 0)).data_ptr()
            L.r_a_log, L.r_dt_bias = small(need("r_a_log", (d.heads,))).data_ptr(), small(need("r_dt_bias", (d.heads,))).data_ptr()
            L.r_head_norm = small(need("r_head_norm", (d.vdim,))).data_ptr()
            L.r_w_o = big(need("r_w_o", (W, d.heads * d.vdim))).data_ptr()
            L.out_norm_a, L.out_norm_b = small(need("out_norm_a", (W,))).data_ptr(), small(need("out_norm_b", (W,))).data_ptr()
        else:
            raise AtomaError(f"layer {i}: parallel blocks take the mixers gla, latent_attention and pair, not {ls.mixer!r}")
        L.w_qkv = big(torch.cat(parts, 0)).data_ptr()

    def state_floats(self, ls: LayerSpec) -> int:
        """float32 entries of one sequence's state in one run of a parallel layer: [input history | mixer state]."""
        n = max(0, ls.taps - 1) * self.spec.width
        if ls.gla is not None:
            n += ls.gla.heads * ls.gla.dim * ls.gla.vdim
        if ls.pair is not None:
            d = ls.pair.right
            n += max(0, d.taps - 1) * (2 * d.kv_heads * d.dim + d.heads * d.vdim) + d.heads * d.dim * d.vdim
        return n

    def _parallel_run_state(self, L, i: int, ls: LayerSpec, weights: dict, small, rows: int) -> None:
        """What one RUN of a parallel layer owns: its caches, its state rows, and what precedes it in the stream."""
        dev, dtype = self.device, self.dtype
        kc = vc = lc = st = None
        if ls.mixer == "latent_attention":
            lc = torch.zeros((rows, ls.latent.kv_rank + ls.latent.rot_dim), dtype=dtype, device=dev)
            L.latent_cache = lc.data_ptr()
        elif ls.mixer == "pair":
            a = ls.pair.left
            kc = torch.zeros((rows, a.kv_heads, a.dim), dtype=dtype, device=dev)
            vc = torch.zeros((rows, a.kv_heads, a.vdim), dtype=dtype, device=dev)
            L.k_cache, L.v_cache = kc.data_ptr(), vc.data_ptr()
        n = self.state_floats(ls)
        if n > 0:
            st = torch.zeros((max(1, self.num_state_slots), n), dtype=torch.float32, device=dev)
            L.layer_state, L.layer_state_stride = st.data_ptr(), n
        else:
            L.layer_state, L.layer_state_stride = None, 0
        L.add_embedding = int(ls.add_embedding)
        if ls.pass_vector is not None:
            pv = weights.get("pass_vectors")
            if pv is None or pv.dim() != 2 or pv.shape[1] != self.spec.width or not 0 <= ls.pass_vector < pv.shape[0]:
                raise AtomaError(f"layer run {i}: pass vector {ls.pass_vector} of a table {None if pv is None else tuple(pv.shape)}")
            L.add_vec = small(pv[ls.pass_vector]).data_ptr()
        else:
            L.add_vec = None
        self.k_caches.append(kc)
        self.v_caches.append(vc)
        self.latent_caches.append(lc)
        self.states.append(st)

    # ---- buffers (grow-only) ----
    def _reserve(self, T: int, S: int) -> None:
        L = _lib.lib()
        need = int(L.atoma_hybrid_scratch_bytes(C.byref(self._model), T, S))
        if need < 0:
            raise AtomaError("atoma_hybrid_scratch_bytes failed")
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=self.device)
        if self._logits is None or self._logits.shape[0] < S:
            cap = max(S, 8)
            self._logits = torch.empty((cap, self.spec.vocab), dtype=torch.float32, device=self.device)
            self._next = torch.zeros((cap,), dtype=torch.int32, device=self.device)

    def _extras(self, token_seq: np.ndarray, state_slots: np.ndarray, selected: np.ndarray):
        n = token_seq.size + state_slots.size + selected.size
        if self._extra_host is None or self._extra_host.numel() < n:
            cap = 1 << max(10, (n - 1).bit_length())
            torch.cuda.synchronize(self.device)
            self._extra_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._extra_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        else:
            torch.cuda.current_stream(self.device).synchronize()   # the previous copy has read the pinned buffer
        h = self._extra_host.numpy()
        a, b = token_seq.size, token_seq.size + state_slots.size
        h[:a], h[a:b], h[b:n] = token_seq, state_slots, selected
        self._extra_dev[:n].copy_(self._extra_host[:n], non_blocking=True)
        d = self._extra_dev
        return d[:a], d[a:b], d[b:n]

    # ---- one step ----
    def execute(self, plan: StepPlan, want_residual_trace: bool = False) -> StepOutput:
        chunks = plan.chunks
        if not chunks:
            return StepOutput(None, None)
        seqs, token_seq, slots, selected, rows = [], [], [], [], []
        t0 = 0
        for b, c in enumerate(chunks):
            end = c.start + c.count
            if self.spec.max_positions and end > self.spec.max_positions:
                raise AtomaError(f"sequence {c.seq.seq_id}: {end} tokens, the model has {self.spec.max_positions} positions")
            if -(-end // self.block_size) > len(c.block_table):
                raise AtomaError(f"sequence {c.seq.seq_id}: {end} tokens need more pages than its block table holds")
            ids = np.zeros(end, dtype=np.uint32)            # only the chunk's tokens are read (positions start .. end)
            ids[c.start:end] = c.seq.tokens[c.start:end]
            seqs.append(SequenceInput(ids, num_computed_tokens=c.start,
                                      token_chunk_size=c.count, block_table=np.asarray(c.block_table, dtype=np.uint32),
                                      is_prompt=True))
            token_seq.append(np.full(c.count, b, dtype=np.int32))
            slots.append(0 if c.state_slot is None else c.state_slot)
            for w in c.want:
                if not 0 <= w < c.count:
                    raise AtomaError(f"sequence {c.seq.seq_id}: wanted offset {w} outside a chunk of {c.count}")
                selected.append(t0 + w)
                rows.append((c.seq.seq_id, w))
            t0 += c.count
        T, B, S = t0, len(chunks), len(selected)
        lay, v = self._stager.prepare_raw(seqs)
        if lay.num_tokens != T or lay.num_slots != T:
            raise AtomaError(f"step inputs: {lay.num_tokens} tokens / {lay.num_slots} slots prepared for a plan of {T}")
        tseq, sslots, sel = self._extras(np.concatenate(token_seq), np.asarray(slots, dtype=np.int32),
                                         np.asarray(selected, dtype=np.int32))
        self._reserve(T, S)
        bt = v["block_tables"]
        trace = (torch.empty((len(self.spec.layers), T, self.spec.width), dtype=torch.float32, device=self.device)
                 if want_residual_trace else None)
        hb = HybridBatch()
        hb.num_tokens, hb.num_seqs, hb.num_selected, hb.max_blocks = T, B, S, bt.shape[1]
        hb.max_query_len = max(c.count for c in chunks)
        hb.max_seq_len = max(c.start + c.count for c in chunks)
        if self.spec.block_style in ("prenorm", "lanes"):
            long_ = [c for c in chunks if c.count >= LONG_PORTION]
            hb.long_seqs, hb.long_min_q = len(long_), LONG_PORTION
            hb.long_tokens, hb.long_ctx_sum = sum(c.count for c in long_), sum(c.start for c in long_)
        hb.tokens, hb.positions, hb.slot_mapping = v["tokens"].data_ptr(), v["positions"].data_ptr(), v["slot_mapping"].data_ptr()
        hb.token_seq, hb.query_start, hb.context_lens = tseq.data_ptr(), v["query_start"].data_ptr(), v["context_lengths"].data_ptr()
        hb.block_tables, hb.state_slots = bt.data_ptr(), sslots.data_ptr()
        hb.selected = sel.data_ptr() if S else None
        hb.scratch, hb.scratch_bytes = self._scratch.data_ptr(), self._scratch.numel()
        hb.logits = self._logits.data_ptr() if S else None
        hb.next_tokens = self._next.data_ptr() if S else None
        hb.residual_trace = trace.data_ptr() if trace is not None else None
        L = _lib.lib()
        L.atoma_reset_launch_count()
        L.atoma_hybrid_step(C.byref(self._model), C.byref(hb), torch.cuda.current_stream(self.device).cuda_stream)
        if L.atoma_last_status() != 0:
            raise AtomaError(L.atoma_last_error().decode())
        self.launches_last_step = int(L.atoma_launch_count())
        self._last = (hb, tseq, sslots, sel, trace)
        return StepOutput(self._logits[:S] if S else None, self._next[:S] if S else None, rows, trace)


def relaunch_last_step(ex: "HybridExecutor") -> None:
    """Enqueues the previous step's kernels again on the current stream with the inputs still on the device (timing and
    CUDA-graph capture of a step: `torch.cuda.graph` around this call).  Recurrent state advances again; everything else
    is rewritten with the same values."""
    L = _lib.lib()
    L.atoma_hybrid_step(C.byref(ex._model), C.byref(ex._last[0]), torch.cuda.current_stream(ex.device).cuda_stream)
    if L.atoma_last_status() != 0:
        raise AtomaError(L.atoma_last_error().decode())


def slopes_power_of_two(heads: int, exponent: float = 8.0) -> List[float]:
    """Distance slopes 2^(-exponent (h + 1) / heads), h = 0 .. heads - 1."""
    return [2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)]
