"""Surinex's configuration and checkpoint reading (host only): sizes and constants from the configuration, the order of layer
runs for looped spans, optional parts, the names and shapes wanted from a checkpoint, errors for what the design does not have."""
import pytest
import torch

import surinex_oracle as so
from atoma_infer_b200 import models, surinex
from atoma_infer_b200.ops import AtomaError


def shapes(w):
    return {k: tuple(v.shape) for k, v in w.items()}


def test_layer_runs_of_looped_spans():
    cfg = so.random_config(kinds=("gla", "latent_attention", "parallel", "gla", "gla"), loop=(1, 4, 3))
    runs = surinex.layer_runs(cfg)
    assert [i for i, _ in runs] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert [p for _, p in runs] == [None, 0, None, None, 1, None, None, 2, None, None, None]
    assert runs == so.layer_runs(cfg)
    once = so.random_config(kinds=("gla", "parallel"), loop=(0, 2, 1))
    assert surinex.layer_runs(once) == [(0, 0), (1, None)]               # a span that runs once still gets its pass vector
    assert surinex.layer_runs(so.random_config(kinds=("gla", "gla"), loop=None)) == [(0, None), (1, None)]
    for bad in [(2, 2, 2), (0, 5, 2), (0, 1, 0), (-1, 1, 2)]:
        with pytest.raises(AtomaError):
            surinex.layer_runs(so.random_config(kinds=("gla", "gla"), loop=bad))


def test_spec_reads_every_size_and_constant_from_the_configuration():
    cfg = so.random_config(width=56, vocab=83, taps=5, kinds=("parallel", "gla", "latent_attention"), loop=(1, 3, 2), ff=72,
                           mlps=[True, False, True], eps=3e-6, gla=dict(heads=3, dim=8, vdim=40, tau=5.0),
                           latent=dict(heads=5, dim=24, rot_dim=16, vdim=8, q_rank=20, kv_rank=48, scale=0.3, rot=dict(base=777.0, dims=16)),
                           left=dict(heads=6, kv_heads=3, dim=32, vdim=8, scale=0.11,
                                     rot=dict(base=12345.0, dims=12, scaling=dict(factor=5.0, low=2.0, high=6.0, original=96))),
                           right=dict(heads=6, kv_heads=2, dim=8, vdim=16, conv=2))
    w = so.random_weights(cfg, torch.Generator().manual_seed(0), decay_rank=7)
    spec = surinex.spec_from_config(cfg, shapes(w))
    assert (spec.width, spec.vocab, spec.eps, spec.block_style, spec.norm_offset, spec.logit_scale) == (56, 83, 3e-6, "parallel", 0.0, 1.0)
    assert [l.mixer for l in spec.layers] == ["pair", "gla", "latent_attention", "gla", "latent_attention"]
    assert [l.source for l in spec.layers] == [0, 1, 2, 1, 2]
    assert [(l.add_embedding, l.pass_vector) for l in spec.layers] == [(False, None), (False, 0), (False, None), (True, 1), (False, None)]
    assert all(l.taps == 5 for l in spec.layers)
    assert spec.layers[0].mlp.ff == 72 and spec.layers[1].mlp is None and spec.layers[2].mlp.act == "silu"
    a, d = spec.layers[0].pair.left, spec.layers[0].pair.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.rotate_values) == (6, 3, 32, 8, 0.11, True)
    assert (a.rotary.dims, a.rotary.base, a.rotary.interleaved, a.rotary.scaling) == (12, 12345.0, True, (5.0, 2.0, 6.0, 96.0))
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.taps) == (6, 2, 8, 16, 2)
    g = spec.layers[1].gla
    assert (g.heads, g.dim, g.vdim, g.decay_rank, g.tau) == (3, 8, 40, 7, 5.0)
    m = spec.layers[2].latent
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale) == (5, 24, 16, 8, 20, 48, 0.3)
    assert (m.rotary.dims, m.rotary.base, m.rotary.interleaved, m.rotary.scaling) == (16, 777.0, False, None)
    assert models.resolve(cfg).name == "Surinex" and models.resolve(cfg).needs_state(cfg)


def test_optional_parts():
    cfg = so.random_config(kinds=("gla", "parallel"), loop=None)
    del cfg["layers"][1]["mixer"]["left"]["rot"]["scaling"]
    w = so.random_weights(cfg, torch.Generator().manual_seed(1))
    spec = surinex.spec_from_config(cfg, shapes(w))
    assert spec.layers[1].pair.left.rotary.scaling is None
    assert all(l.pass_vector is None and not l.add_embedding for l in spec.layers)
    out = surinex.weights_from_checkpoint(spec, cfg, w)
    assert "pass_vectors" not in out and len(out["layers"]) == 2


def test_checkpoint_names_and_shapes():
    cfg = so.random_config(kinds=("gla", "latent_attention", "parallel"), loop=(0, 2, 2), mlps=[True, True, False])
    w = so.random_weights(cfg, torch.Generator().manual_seed(2))
    spec = surinex.spec_from_config(cfg, shapes(w))
    out = surinex.weights_from_checkpoint(spec, cfg, w)
    W, F = cfg["width"], cfg["layers"][0]["mlp"]["ff"]
    assert len(out["layers"]) == 3                                       # one entry per layer; the runs of a looped layer share it
    assert tuple(out["pass_vectors"].shape) == (2, W)
    l0, l1, l2 = out["layers"]
    assert tuple(l0["w_gate_up"].shape) == (2 * F, W) and torch.equal(l0["w_gate_up"][F:], w["l0.mlp.up"])
    assert torch.equal(l0["a2_bias"], w["l0.mix.a2.b"]) and torch.equal(l0["tap_w2"], w["l0.canon2"])
    assert torch.equal(l1["w_dkv"], w["l1.mix.dkv"]) and torch.equal(l1["dq_norm"], w["l1.mix.dq.norm"])
    assert "w_gate_up" not in l2 and "tap_w2" not in l2 and torch.equal(l2["tap_w1"], w["l2.canon1"])
    assert torch.equal(l2["head_bias"], w["l2.mix.left.pb"]) and torch.equal(l2["r_tap_v"], w["l2.mix.right.v.conv"])
    assert torch.equal(l2["out_norm_a"], w["l2.mix.left.out"]) and torch.equal(l2["out_norm_b"], w["l2.mix.right.out"])
    missing = dict(w)
    del missing["l2.mix.right.A_log"]
    with pytest.raises(AtomaError, match="A_log"):
        surinex.weights_from_checkpoint(spec, cfg, missing)
    wrong = dict(w)
    wrong["l0.mix.norm"] = torch.zeros(3)
    with pytest.raises(AtomaError, match="l0.mix.norm"):
        surinex.weights_from_checkpoint(spec, cfg, wrong)
    with pytest.raises(AtomaError, match="a1"):
        surinex.spec_from_config(cfg, {})


def test_what_the_design_does_not_have_is_refused():
    cfg = so.random_config(kinds=("gla",), loop=None)
    w = shapes(so.random_weights(cfg, torch.Generator().manual_seed(3)))
    other = so.json_copy(cfg)
    other["layers"][0]["type"] = "attention"
    with pytest.raises(AtomaError, match="attention"):
        surinex.spec_from_config(other, w)
    other = so.json_copy(cfg)
    other["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(AtomaError, match="moe"):
        surinex.spec_from_config(other, w)
