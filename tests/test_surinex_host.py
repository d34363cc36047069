"""Surinex's configuration and checkpoint reading (host only): sizes and constants from the configuration, the order of layer
runs of a looped span, rotary frequencies with stretched wavelengths, the per-run state size, errors for what the design lacks."""
import json

import pytest
import torch

import surinex_oracle as so
from atoma_infer_b200 import models, surinex
from atoma_infer_b200.hybrid import RotarySpec
from atoma_infer_b200.ops import AtomaError


def shapes(w):
    return {k: tuple(v.shape) for k, v in w.items()}


def test_spec_reads_every_size_and_constant_from_the_configuration():
    cfg = so.random_config(width=56, vocab=37, taps=4, kinds=("parallel", "gla", "latent_attention"), loop=(1, 3, 3), ff=24, mlps=[True, False, True],
                           eps=3e-6, gla=dict(heads=3, dim=10, vdim=14, tau=5.5),
                           latent=dict(heads=5, dim=12, rot_dim=6, vdim=10, q_rank=20, kv_rank=18, scale=0.3, rot=dict(base=777.0, dims=6)),
                           left=dict(heads=6, kv_heads=3, dim=12, vdim=10, scale=0.4, rot=dict(base=999.0, dims=4)),
                           right=dict(heads=6, kv_heads=2, dim=8, vdim=12, conv=2))
    w = so.random_weights(cfg, torch.Generator().manual_seed(0), decay_rank=7)
    spec = surinex.spec_from_config(cfg, shapes(w))
    assert (spec.block_style, spec.width, spec.vocab, spec.eps, spec.norm_offset) == ("parallel", 56, 37, 3e-6, 0.0)
    assert [(l.mixer, l.source, l.add_embedding, l.pass_vector) for l in spec.layers] == [
        ("pair", 0, False, None), ("gla", 1, False, 0), ("latent_attention", 2, False, None), ("gla", 1, True, 1),
        ("latent_attention", 2, False, None), ("gla", 1, True, 2), ("latent_attention", 2, False, None)]
    assert all(l.taps == 4 for l in spec.layers) and spec.has_state
    g = spec.layers[1].gla
    assert (g.heads, g.dim, g.vdim, g.tau, g.decay_rank) == (3, 10, 14, 5.5, 7) and spec.layers[1].mlp is None
    a = spec.layers[2].latent
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.q_rank, a.kv_rank, a.scale) == (5, 12, 6, 10, 20, 18, 0.3)
    assert (a.rotary.dims, a.rotary.base, a.rotary.interleaved, a.rotary.scaling) == (6, 777.0, False, None)
    p = spec.layers[0].pair
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.scale) == (6, 3, 12, 10, 0.4)
    assert (p.left.rotary.dims, p.left.rotary.base, p.left.rotary.interleaved) == (4, 999.0, True)
    assert (p.right.heads, p.right.kv_heads, p.right.dim, p.right.vdim, p.right.taps) == (6, 2, 8, 12, 2)
    assert spec.layers[0].mlp.ff == 24 and spec.layers[0].mlp.act == "silu"
    assert spec.cache_bytes_per_token(torch.bfloat16) == (3 * (12 + 10) + 3 * (18 + 6)) * 2
    assert models.resolve(cfg).name == "Surinex" and models.resolve(cfg).needs_state(cfg)


def test_layer_runs_of_looped_spans():
    def runs(n, loop):
        return surinex.layer_runs(dict(layers=[{}] * n, loop=None if loop is None else dict(start=loop[0], stop=loop[1], times=loop[2])))
    assert runs(3, None) == [(0, None), (1, None), (2, None)]
    assert runs(3, (0, 3, 1)) == [(0, 0), (1, None), (2, None)]
    assert runs(4, (1, 2, 3)) == [(0, None), (1, 0), (1, 1), (1, 2), (2, None), (3, None)]
    assert runs(4, (2, 4, 2)) == [(0, None), (1, None), (2, 0), (3, None), (2, 1), (3, None)]
    assert runs(4, (1, 2, 3)) == so.layer_runs(dict(layers=[{}] * 4, loop=dict(start=1, stop=2, times=3)))
    for bad in [(2, 2, 2), (0, 5, 2), (1, 3, 0)]:
        with pytest.raises(AtomaError):
            runs(4, bad)


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, None), (16, 1e6, (4.0, 1.0, 4.0, 512)), (32, 5e5, (8.0, 1.0, 4.0, 64)),
                                               (6, 50.0, (2.0, 0.5, 2.0, 10)), (64, 1e4, (3.0, 1.0, 2.0, 100))])
def test_rotary_frequencies(dims, base, scaling):
    got = RotarySpec(dims=dims, base=base, scaling=scaling).frequencies()
    sc = None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))
    want = so.rotary_frequencies(dims, base, sc)
    assert len(got) == dims // 2 and torch.allclose(torch.tensor(got, dtype=torch.float64), want, rtol=1e-12, atol=0)
    if scaling is not None:      # no frequency grows, the longest wavelengths are divided by the factor
        plain = RotarySpec(dims=dims, base=base).frequencies()
        assert all(p / scaling[0] * (1 - 1e-12) <= g <= p for g, p in zip(got, plain))


def test_weights_by_layer_and_errors():
    cfg = so.random_config(kinds=("gla", "parallel", "latent_attention"), loop=(0, 1, 2), mlps=[True, True, False])
    w = {k: v.to(torch.bfloat16) for k, v in so.random_weights(cfg, torch.Generator().manual_seed(1)).items()}
    spec = surinex.spec_from_config(cfg, shapes(w))
    out = surinex.weights_from_checkpoint(spec, cfg, w)
    assert len(out["layers"]) == 3 and tuple(out["pass_vectors"].shape) == (2, 48)
    assert torch.equal(out["layers"][0]["w_a1"], w["l0.mix.a1"]) and torch.equal(out["layers"][1]["r_tap_k"], w["l1.mix.right.k.conv"])
    assert torch.equal(out["layers"][0]["w_gate_up"][40:], w["l0.mlp.up"]) and "w_gate_up" not in out["layers"][2] and "tap_w2" not in out["layers"][2]
    assert torch.equal(out["layers"][1]["out_norm_b"], w["l1.mix.right.out"])
    missing = dict(w)
    del missing["l1.mix.left.pb"]
    with pytest.raises(AtomaError, match="left.pb"):
        surinex.weights_from_checkpoint(spec, cfg, missing)
    wrong = dict(w)
    wrong["l2.mix.uk"] = torch.zeros(5, 5)
    with pytest.raises(AtomaError, match="uk"):
        surinex.weights_from_checkpoint(spec, cfg, wrong)
    with pytest.raises(AtomaError, match="a1"):
        surinex.spec_from_config(cfg, {})
    other = json.loads(json.dumps(cfg))
    other["layers"][0]["type"] = "convolution"
    with pytest.raises(AtomaError, match="convolution"):
        surinex.spec_from_config(other, shapes(w))
    other = json.loads(json.dumps(cfg))
    other["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(AtomaError, match="moe"):
        surinex.spec_from_config(other, shapes(w))
