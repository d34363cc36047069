"""Nemasun's configuration and checkpoint reading (host only): sizes and constants from the configuration, optional parts,
the stacked weight layout, the distance table by distance, the C structures' sizes, errors for what the design does not have."""
import ctypes as C

import pytest
import torch

import nemasun_oracle as no
from atoma_infer_b200 import _lib, models, nemasun
from atoma_infer_b200.ops import AtomaError


def test_spec_reads_every_size_and_constant_from_the_configuration():
    cfg = no.checkpoint_config(no.random_config(width=50, vocab=37, lanes=3, heads=6, kv_heads=3, dim=6, window=33, keep=1, far=29, ff=11,
                                                limit=1.25, experts=7, identity=3, top=4, groups=5, keep_groups=3, expert_ff=9, shared_ff=13,
                                                layers=4, embed_scale=7.0, eps=3e-6, scale=0.21))
    spec = nemasun.spec_from_config(cfg)
    assert (spec.block_style, spec.lanes, spec.embed_scale, spec.eps, spec.norm_offset, spec.logit_scale) == ("lanes", 3, 7.0, 3e-6, 0.0, 1.0)
    assert [l.mixer for l in spec.layers] == ["softmax_attention"] * 4
    a = spec.layers[0].softmax
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first) == (6, 3, 6, 6, 0.21, 33, 1)
    assert a.values_are_keys and a.out_gate and a.distance_bias
    d, e = spec.layers[0].clamped_mlp, spec.layers[1].moe
    assert (d.ff, d.limit, d.alpha, d.up_shift, d.bias) == (11, 1.25, 1.702, 1.0, True)
    assert (e.experts, e.identity, e.top, e.groups, e.keep_groups, e.ff, e.shared_ff) == (7, 3, 4, 5, 3, 9, 13)
    assert (e.score, e.correction, e.renormalize, e.scale_input, e.alpha, e.up_shift, e.limit) == ("softmax", True, True, False, 1.0, 0.0, 0.0)
    assert spec.layers[2].clamped_mlp is None and spec.layers[2].moe is None
    assert spec.cache_bytes_per_token(torch.bfloat16) == 4 * 3 * (6 + 6) * 2
    assert models.resolve(cfg).name == "Nemasun" and not models.resolve(cfg).needs_state(cfg)
    bare = no.checkpoint_config(no.random_config(lanes=None, window=0, keep=0, identity=0, shared_ff=0, groups=1, keep_groups=1))
    s2 = nemasun.spec_from_config(bare)
    assert s2.lanes == 1 and s2.layers[0].softmax.window == 0 and s2.layers[0].softmax.keep_first == 0
    assert s2.layers[1].moe.identity == 0 and s2.layers[1].moe.shared_ff == 0 and s2.layers[1].moe.groups == 1


def test_weights_are_stacked_for_one_product_per_sublayer():
    full = no.random_config(lanes=3, layers=3)
    cfg = no.checkpoint_config(full)
    w = {k: v.to(torch.bfloat16) for k, v in no.random_weights(full, torch.Generator().manual_seed(0)).items()}
    spec = nemasun.spec_from_config(cfg)
    out = nemasun.weights_from_checkpoint(spec, cfg, w)
    l0, l1, l2 = out["layers"]
    H, G, D, W = 4, 2, 8, 48
    assert tuple(l0["w_qkv"].shape) == (H * D + G * D + H * D, W)
    assert torch.equal(l0["w_qkv"][H * D:H * D + G * D], w["l0.mix.k"]) and torch.equal(l0["w_qkv"][H * D + G * D:], w["l0.mix.g"])
    assert tuple(l0["w_gate_up"].shape) == (80, W) and tuple(l0["b_gate_up"].shape) == (80,) and torch.equal(l0["b_gate_up"][40:], w["l0.mlp.up.b"])
    assert tuple(l1["w_expert_gate_up"].shape) == (6, 40, W) and tuple(l1["w_expert_down"].shape) == (6, W, 20)
    assert tuple(l1["w_router"].shape) == (8, W) and tuple(l1["router_correction"].shape) == (8,) and tuple(l1["w_ff_in"].shape) == (24, W)
    assert torch.equal(l1["lanes_mix2"], w["l1.hc2.mix"]) and "norm2" not in l2 and "lanes_in2" not in l2
    # a configuration without residual lanes is a plain residual stream: unit lane weights, no such tensors wanted
    one = no.random_config(lanes=None, layers=2)
    w1 = {k: v.to(torch.bfloat16) for k, v in no.random_weights(one, torch.Generator().manual_seed(1)).items()}
    o1 = nemasun.weights_from_checkpoint(nemasun.spec_from_config(no.checkpoint_config(one)), no.checkpoint_config(one), w1)
    assert o1["layers"][0]["lanes_mix1"].tolist() == [[1.0]] and o1["layers"][0]["lanes_out2"].tolist() == [1.0]


def test_distance_table_by_distance():
    """The expanded table (one row per distance, the last for everything beyond) against the bucket formula."""
    for rows, far in [(10, 37), (16, 100), (2, 5), (32, 4000), (7, 50), (1, 9), (12, 6.5)]:
        g = torch.Generator().manual_seed(rows)
        table = torch.randn(rows, 3, generator=g)
        ex = nemasun.expand_distance_table(table, far)
        for n in list(range(0, int(3 * far))) + [int(10 * far)]:
            want = table[no.distance_bucket(n, rows, far)] if rows > 1 else table[0]
            assert torch.equal(ex[min(n, ex.shape[0] - 1)], want), (rows, far, n)
        assert ex.shape[0] <= int(far) + 2
    with pytest.raises(AtomaError):
        nemasun.expand_distance_table(torch.zeros(10, 2), 5)       # the logarithmic rows would begin beyond their end


def test_what_the_design_does_not_have_is_refused():
    full = no.random_config()
    cfg = no.checkpoint_config(full)
    w = {k: v.to(torch.bfloat16) for k, v in no.random_weights(full, torch.Generator().manual_seed(2)).items()}
    bad = {**cfg, "layers": [{**cfg["layers"][0], "type": "mingru"}]}
    with pytest.raises(AtomaError):
        nemasun.spec_from_config(bad)
    bad = {**cfg, "layers": [{**cfg["layers"][0], "mlp": {"kind": "conv"}}]}
    with pytest.raises(AtomaError):
        nemasun.spec_from_config(bad)
    spec = nemasun.spec_from_config(cfg)
    missing = {k: v for k, v in w.items() if k != "l1.mlp.correction"}
    with pytest.raises(AtomaError, match="correction"):
        nemasun.weights_from_checkpoint(spec, cfg, missing)
    wrong = dict(w)
    wrong["l0.hc1.mix"] = torch.zeros(3, 3)
    with pytest.raises(AtomaError, match="hc1.mix"):
        nemasun.weights_from_checkpoint(spec, cfg, wrong)


def test_c_structures_have_the_sizes_the_library_was_built_with():
    try:
        L = _lib.load()
    except Exception:
        pytest.skip("the shared library is not built here")
    mirrors = [_lib.HybridLayer, _lib.HybridModel, _lib.HybridBatch, _lib.SigmoidAttnArgs, _lib.GatedResidualArgs, _lib.LatentAttnArgs,
               _lib.MoeArgs, _lib.LatentExpandedArgs, _lib.LanesUpdateArgs, _lib.SoftmaxAttnArgs, _lib.ParallelResidualArgs,
               _lib.TapFilterArgs, _lib.StateScanArgs, _lib.QkvRopeArgs]
    for i, m in enumerate(mirrors):
        assert L.atoma_hybrid_abi_sizeof(i) == C.sizeof(m), m.__name__
    assert L.atoma_hybrid_abi_sizeof(len(mirrors)) == -1
