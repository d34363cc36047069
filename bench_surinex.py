"""bench.py --design surinex: prefill and decode throughput of the Surinex design (random weights) at sizes that resemble real
models' layers, beside the framework's closest existing model — Lilovik, the other design that mixes sigmoid attention with a
state-carrying mixer — at equal width, head counts, head size, feed-forward size and number of layer runs, and the design's own
kernels against the measured peaks beside Lilovik's like kernels.  Not the headline (config 2 is); ONE JSON line in the same format.

Per size: a model of three layers (gated linear attention, latent attention with a rotated key part, the pair of sigmoid attention and
gated delta rule; the first two run twice as a looped span) is served through the engine's executor: `prefill` = one 4096-token
prompt in one step; `decode` = one step of 32 sequences at context 4096 (built by prefilling them), timed with CUDA events around K
executor steps after W warm-up steps, inputs shipped from pinned memory every step, sampled tokens read back; the same step replayed
from a CUDA graph is the device-only figure.  Kernel rows: achieved bytes/s or FLOP/s over the measured peaks of MEASURED_PEAKS.json
(fallback figures when absent); L2 is flushed between their iterations."""
from __future__ import annotations

import json
import math
import os

import bench_hybrid
from bench_hybrid import BATCH, CTX, PROMPT, _peaks, _time
from bench_patadra import _row

SIZES = {
    "2k-wide": dict(width=2048, ff=8192, taps=4, vocab=32000,
                    gla=dict(heads=16, dim=64, vdim=128, rank=16, tau=16.0),
                    latent=dict(heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=512),
                    left=dict(heads=32, kv_heads=8, dim=64, vdim=64, rot=64), right=dict(heads=16, kv_heads=8, dim=128, vdim=128, taps=4)),
    "4k-wide": dict(width=4096, ff=14336, taps=4, vocab=32000,
                    gla=dict(heads=32, dim=64, vdim=128, rank=16, tau=16.0),
                    latent=dict(heads=32, dim=128, rot_dim=64, vdim=128, q_rank=1536, kv_rank=512),
                    left=dict(heads=32, kv_heads=8, dim=128, vdim=128, rot=64), right=dict(heads=32, kv_heads=16, dim=128, vdim=128, taps=4)),
}
RUNS = ((0, 0), (1, None), (0, 1), (1, None), (2, None))      # (layer, pass that starts here): layers 0 and 1 are a span that runs twice


def _spec(s):
    from atoma_infer_b200.hybrid import (DeltaRuleSpec, GatedLinearAttentionSpec, HybridSpec, LatentAttentionSpec, LayerSpec, MixerPairSpec, MlpSpec,
                                         RotarySigmoidAttentionSpec, RotarySpec)
    g, l, a, d = s["gla"], s["latent"], s["left"], s["right"]
    mixers = [
        dict(mixer="gla", gla=GatedLinearAttentionSpec(g["heads"], g["dim"], g["vdim"], g["rank"], g["tau"])),
        dict(mixer="latent_attention", latent=LatentAttentionSpec(l["heads"], l["dim"], l["vdim"], l["q_rank"], l["kv_rank"],
                                                                  1.0 / math.sqrt(l["dim"] + l["rot_dim"]), rot_dim=l["rot_dim"],
                                                                  rotary=RotarySpec(l["rot_dim"], 5e5))),
        dict(mixer="pair", pair=MixerPairSpec(RotarySigmoidAttentionSpec(a["heads"], a["kv_heads"], a["dim"], a["vdim"], 1.0 / math.sqrt(a["dim"]),
                                                                         RotarySpec(a["rot"], 1e6, True, (8.0, 1.0, 4.0, 8192))),
                                              DeltaRuleSpec(d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["taps"]))),
    ]
    layers = tuple(LayerSpec(mlp=MlpSpec(s["ff"], "silu"), source=i, taps=s["taps"], add_embedding=bool(p), pass_vector=p, **mixers[i]) for i, p in RUNS)
    return HybridSpec(s["width"], s["vocab"], 1e-5, 1.0, layers, norm_offset=0.0, block_style="parallel", position="none")


def _weights(torch, spec, s, dev):
    gen = torch.Generator(device=dev).manual_seed(17)

    def r(*shape, scale=1.0, mean=0.0):
        return (mean + torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)

    W, F, K = spec.width, s["ff"], s["taps"]
    lin = lambda o, i: r(o, i, scale=i ** -0.5)
    out = {"embed": r(spec.vocab, W), "head": lin(spec.vocab, W), "final_norm": r(W, scale=0.1, mean=1.0), "pass_vectors": r(2, W, scale=0.1),
           "layers": []}
    by_layer = {}
    for ls in spec.layers:
        by_layer.setdefault(ls.source, ls)
    for i in sorted(by_layer):
        ls = by_layer[i]
        w = {"norm1": r(W, scale=0.1, mean=1.0), "tap_w1": r(W, K, scale=0.3), "tap_w2": r(W, K, scale=0.3),
             "w_gate_up": lin(2 * F, W), "w_down": lin(W, F)}
        if ls.gla is not None:
            a = ls.gla
            w.update(w_q=lin(a.heads * a.dim, W), w_k=lin(a.heads * a.dim, W), w_v=lin(a.heads * a.vdim, W), w_g=lin(a.heads * a.vdim, W),
                     w_a1=lin(a.decay_rank, W), w_a2=lin(a.heads * a.dim, a.decay_rank), a2_bias=r(a.heads * a.dim, mean=3.0),
                     head_norm=r(a.vdim, scale=0.1, mean=1.0), w_o=lin(W, a.heads * a.vdim))
        elif ls.latent is not None:
            a = ls.latent
            w.update(w_dq=lin(a.q_rank, W), dq_norm=r(a.q_rank, scale=0.1, mean=1.0), w_uq=lin(a.heads * (a.dim + a.rot_dim), a.q_rank),
                     w_dkv=lin(a.kv_rank + a.rot_dim, W), dkv_norm=r(a.kv_rank, scale=0.1, mean=1.0), w_uk=lin(a.heads * a.dim, a.kv_rank),
                     w_uv=lin(a.heads * a.vdim, a.kv_rank), w_o=lin(W, a.heads * a.vdim))
        else:
            a, d = ls.pair.left, ls.pair.right
            nqk, nv = d.kv_heads * d.dim, d.heads * d.vdim
            w.update(w_q=lin(a.heads * a.dim, W), w_k=lin(a.kv_heads * a.dim, W), w_v=lin(a.kv_heads * a.vdim, W), q_norm=r(a.dim, scale=0.1, mean=1.0),
                     k_norm=r(a.dim, scale=0.1, mean=1.0), head_bias=r(a.heads, scale=0.5, mean=-6.0), w_o=lin(W, a.heads * a.vdim),
                     out_norm_a=r(W, scale=0.1, mean=1.0), out_norm_b=r(W, scale=0.1, mean=1.0), r_w_q=lin(nqk, W), r_w_k=lin(nqk, W),
                     r_w_v=lin(nv, W), r_w_g=lin(nv, W), r_w_b=lin(d.heads, W), r_w_a=lin(d.heads, W), r_tap_q=r(nqk, d.taps, scale=0.5),
                     r_tap_k=r(nqk, d.taps, scale=0.5), r_tap_v=r(nv, d.taps, scale=0.5), r_a_log=r(d.heads, scale=0.5, mean=-1.0),
                     r_dt_bias=r(d.heads, scale=0.5), r_head_norm=r(d.vdim, scale=0.1, mean=1.0), r_w_o=lin(W, nv))
        out["layers"].append(w)
    return out


def _lilovik_model(torch, s, dev, steps, warmup, n_runs):
    """Prefill and decode of a Lilovik model (sigmoid attention layers, one minGRU layer) of equal width, heads, head size, feed-forward
    size and number of layer runs, through the same executor."""
    import numpy as np
    from atoma_infer_b200.cache import CacheManager
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.hybrid import HybridExecutor, relaunch_last_step
    a = s["left"]
    ls = dict(width=s["width"], heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], ff=s["ff"], state=s["width"], vocab=s["vocab"], layers=n_runs)
    spec = bench_hybrid._spec(torch, ls)
    page = 16
    nblocks = BATCH * ((CTX + 64) // page + 1) + PROMPT // page + 8
    ex = HybridExecutor(spec, bench_hybrid._weights(torch, spec, dev), torch.bfloat16, dev, nblocks, page, BATCH + 1)
    eng = Engine(ex, CacheManager(nblocks, page, BATCH + 1), max_num_batched_tokens=PROMPT, max_num_seqs=BATCH + 1)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, s["vocab"], size=PROMPT).tolist()

    def prefill():
        eng.step_forced([("p", prompt, [PROMPT - 1])], end=["p"]).next_tokens.cpu()
    ms_prefill = _time(torch, prefill, min(steps, 10), warmup)
    for b in range(BATCH):
        eng.step_forced([(f"d{b}", rng.integers(0, s["vocab"], size=CTX).tolist(), [])])
    tok = [int(t) for t in rng.integers(0, s["vocab"], size=BATCH)]
    eng.step_forced([(f"d{b}", [tok[b]], [0]) for b in range(BATCH)]).next_tokens.cpu()
    launches = ex.launches_last_step
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        relaunch_last_step(ex)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        relaunch_last_step(ex)
    ms_graph = _time(torch, graph.replay, steps, warmup)
    del graph, eng, ex
    torch.cuda.empty_cache()
    return dict(sizes=ls, prefill_ms=round(ms_prefill, 3), prefill_tokens_per_s=round(PROMPT / ms_prefill * 1e3, 1),
                decode_graph_ms_per_step=round(ms_graph, 4), decode_graph_tokens_per_s=round(BATCH / ms_graph * 1e3, 1), decode_launches_per_step=launches)


def _kernel_rows(torch, s, dev, steps, warmup, hbm, tf):
    """The design's kernels beside Lilovik's like kernels at the same shapes."""
    from atoma_infer_b200 import hybrid_ops as ho
    bf, W = torch.bfloat16, s["width"]
    rows = {}
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    rn = lambda *shape: torch.randn(shape, device=dev, dtype=bf)
    # ---- recurrences: one 4096-token prompt, and a decode step of BATCH sequences ----
    g, d = s["gla"], s["right"]
    for name, T, B in (("prefill", PROMPT, 1), ("decode", BATCH, BATCH)):
        qs = i32([i * (T // B) for i in range(B + 1)])
        ctx, slots = i32([0 if name == "prefill" else CTX] * B), i32(list(range(B)))
        H, D, V = g["heads"], g["dim"], g["vdim"]
        q, k, v, z = rn(T, H * D), rn(T, H * D), rn(T, H * V), rn(T, H * D)
        zb, state = torch.full((H * D,), 3.0, device=dev), torch.zeros((B, H * D * V), device=dev)
        f = lambda: ho.gla_scan(q, k, v, z, zb, g["tau"], D ** -0.5, state, slots, qs, ctx, H, D, V)
        nbytes = T * (3 * H * D * 2 + H * V * 2 + H * V * 4) + B * H * D * V * 4 * 2
        rows[f"gla_scan_{name}"] = _row(_time(torch, f, steps, warmup, flush), nbytes=nbytes, hbm=hbm, flops=4.0 * T * H * D * V, tf=tf)
        H, G, D, V = d["heads"], d["kv_heads"], d["dim"], d["vdim"]
        q, k, v, bp, ap = rn(T, G * D), rn(T, G * D), rn(T, H * V), rn(T, H), rn(T, H)
        al, dtb, state = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.zeros((B, H * D * V), device=dev)
        f = lambda: ho.delta_rule_scan(q, k, v, bp, ap, al, dtb, D ** -0.5, state, slots, qs, ctx, H, G, D, V)
        nbytes = T * (2 * G * D * 2 + H * V * 2 + 2 * H * 2 + H * V * 4) + B * H * D * V * 4 * 2
        rows[f"delta_rule_scan_{name}"] = _row(_time(torch, f, steps, warmup, flush), nbytes=nbytes, hbm=hbm, flops=6.0 * T * H * D * V, tf=tf)
        S = W                                                   # Lilovik's recurrence: one state per channel
        zxg, bias, st = rn(T, 3 * S), torch.zeros(3 * S, device=dev), torch.zeros((B, S), device=dev)
        f = lambda: ho.mingru_scan(zxg, bias, st, slots, qs, ctx, T // B)
        rows[f"lilovik_mingru_scan_{name}"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * S * (3 * 2 + 2) + B * S * 8, hbm=hbm)
    # ---- row operators at 8192 tokens ----
    T = 8192
    qs, ctx, slots, tseq = i32([0, T]), i32([0]), i32([0]), torch.zeros(T, dtype=torch.int32, device=dev)
    h, w1, w2 = rn(T, W), torch.randn((W, s["taps"]), device=dev), torch.randn((W, s["taps"]), device=dev)
    hist = torch.zeros((1, (s["taps"] - 1) * W), device=dev)
    f = lambda: ho.tap_filter(h, w1, w2, hist, slots, tseq, qs, ctx, True, 0)
    rows["tap_filter_two_outputs"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * 2 * 3, hbm=hbm)
    x, ya, yb, yf = torch.randn((T, W), device=dev), rn(T, W), rn(T, W), rn(T, W)
    na, wn = torch.ones(W, device=dev), torch.ones(W, device=dev)
    f = lambda: ho.parallel_residual_norm(x, bf, y_a=ya, y_ff=yf, w_next=wn)
    rows["parallel_residual_norm"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * (2 * 2 + 8 + 2), hbm=hbm)
    f = lambda: ho.parallel_residual_norm(x, bf, y_a=ya, y_b=yb, y_ff=yf, norm_a=na, norm_b=na, mix_scale=0.5, w_next=wn)
    rows["parallel_residual_norm_pair"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * (3 * 2 + 8 + 2), hbm=hbm)
    f = lambda: ho.postnorm_add_prenorm(ya, x, na, wn, 1e-5, 0.0)
    rows["lilovik_postnorm_add_prenorm"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * (2 + 8 + 2), hbm=hbm)
    del x, ya, yb, yf, h
    a = s["left"]
    H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    N = H * D + G * D + G * V
    proj, pos, slot = rn(T, N), torch.arange(T, device=dev), torch.randperm(T, device=dev)
    kc, vc = torch.empty((T, G, D), device=dev, dtype=bf), torch.empty((T, G, V), device=dev, dtype=bf)
    qw, fq, fv = torch.ones(D, device=dev), torch.rand(a["rot"] // 2, device=dev), torch.rand(V // 2, device=dev)
    f = lambda: ho.qkv_headnorm_rope_cache(proj, 0, H * D, H * D + G * D, qw, qw, fq, fv, True, pos, slot, kc, vc, H, G, D, V, 1e-5)
    rows["qkv_headnorm_rope_cache"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * (N * 2 + H * D * 2 + G * (D + V) * 2), hbm=hbm)
    qn, kn, bias = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev), torch.zeros(N, device=dev)
    f = lambda: ho.qk_norm_cache(proj, bias, qn, kn, pos, slot, kc, vc, H, G, D, V, 1e-5, 0.25, 64)
    rows["lilovik_qk_norm_cache"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * (N * 2 + H * D * 2 + G * (D + V) * 2), hbm=hbm)
    o = rn(T, H * V)
    f = lambda: ho.rotate_heads(o, pos, fv, H, V, True, -1.0)
    rows["rotate_heads_back"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * H * V * 2 * 2, hbm=hbm)
    of, gate, hw = torch.randn((T, H * V), device=dev), rn(T, H * V), torch.ones(V, device=dev)
    f = lambda: ho.headnorm_gate(of, hw, gate, H, V, 1e-5, bf)
    rows["headnorm_gate"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * H * V * (4 + 2 + 2), hbm=hbm)
    del proj, kc, vc, o, of, gate
    torch.cuda.empty_cache()
    # ---- attention: one 4096-token prompt, and a decode step of BATCH sequences at context CTX ----
    page = 16
    pb, talk = torch.zeros(H, device=dev) - 3, torch.eye(H, device=dev) + 0.05
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
    l = s["latent"]
    LH, R, Rk = l["heads"], l["kv_rank"] + l["rot_dim"], l["kv_rank"]
    for name, T, B, ctx in (("prefill", PROMPT, 1, 0), ("decode", BATCH, BATCH, CTX)):
        n = T // B
        mb = (ctx + n + page - 1) // page
        bt = torch.randperm(B * mb, device=dev).to(torch.int32).reshape(B, mb)
        pos = (torch.arange(n, device=dev) + ctx).repeat(B)
        tseq, qs = torch.arange(B, device=dev, dtype=torch.int32).repeat_interleave(n), i32([i * n for i in range(B + 1)])
        kc, vc, q = rn(B * mb * page, G, D), rn(B * mb * page, G, V), rn(T, H * D)
        pairs = B * (n * ctx + n * (n + 1) / 2)
        mine = lambda: ho.sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, None, pb, None, H, G, D, V, page, D ** -0.5, 0.0, n, query_start=qs,
                                                  max_seq_len=ctx + n)
        like = lambda: ho.sigmoid_attention_paged(q, kc, vc, pos, tseq, bt, slopes, pb, talk, H, G, D, V, page, D ** -0.5, 30.0, n, query_start=qs,
                                                  max_seq_len=ctx + n)
        for key, f in ((f"sigmoid_attention_{name}", mine), (f"lilovik_sigmoid_attention_{name}", like)):
            rows[key] = _row(_time(torch, f, steps, warmup, flush), nbytes=B * (ctx + n) * G * (D + V) * 2, hbm=hbm, flops=2.0 * pairs * H * (D + V), tf=tf)
        del kc, vc, q
        cache, ql = rn(B * mb * page, R), torch.randn((T, LH * R), device=dev) * 0.1
        f = lambda: ho.latent_attention_paged(ql, cache, pos, tseq, bt, None, LH, R, page, 0, R ** -0.5, n, query_start=qs, max_seq_len=ctx + n, out_cols=Rk)
        rows[f"latent_attention_{name}"] = _row(_time(torch, f, steps, warmup, flush), nbytes=B * (ctx + n) * R * 2, hbm=hbm, flops=2.0 * pairs * LH * (R + Rk), tf=tf)
        if name == "decode":                                 # the like kernel: the same operator on rows without a score-only tail
            qk, ck = ql[:, :LH * Rk].contiguous(), cache[:, :Rk].contiguous()
            f = lambda: ho.latent_attention_paged(qk, ck, pos, tseq, bt, None, LH, Rk, page, 0, R ** -0.5, n, query_start=qs, max_seq_len=ctx + n)
            rows["patadra_latent_attention_decode"] = _row(_time(torch, f, steps, warmup, flush), nbytes=B * (ctx + n) * Rk * 2, hbm=hbm,
                                                           flops=4.0 * pairs * LH * Rk, tf=tf)
            del qk, ck
        del cache, ql
    return rows


def run(args, torch, dev, json_fd):
    import numpy as np
    from atoma_infer_b200 import _lib
    from atoma_infer_b200.cache import CacheManager
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.hybrid import HybridExecutor, relaunch_last_step
    if args.impl != "ours":
        os.write(json_fd, (json.dumps({"impl": "reference", "unavailable": "the reference has no model of this design"}) + "\n").encode())
        return
    _lib.lib()
    hbm, tf, src = _peaks()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    page = 16
    out_sizes, headline = {}, None
    import time
    from bench import ClockSampler
    sampler, t_clock0 = ClockSampler(torch.cuda.current_device()), time.time()
    for name, s in SIZES.items():
        spec = _spec(s)
        weights = _weights(torch, spec, s, dev)
        nblocks = BATCH * ((CTX + 64) // page + 1) + PROMPT // page + 8
        ex = HybridExecutor(spec, weights, torch.bfloat16, dev, nblocks, page, BATCH + 1)
        del weights
        eng = Engine(ex, CacheManager(nblocks, page, BATCH + 1), max_num_batched_tokens=PROMPT, max_num_seqs=BATCH + 1)
        rng = np.random.default_rng(0)
        prompt = rng.integers(0, s["vocab"], size=PROMPT).tolist()

        def prefill():
            eng.step_forced([("p", prompt, [PROMPT - 1])], end=["p"]).next_tokens.cpu()
        ms_prefill = _time(torch, prefill, min(steps, 10), warmup)
        prefill_launches = ex.launches_last_step
        for b in range(BATCH):
            eng.step_forced([(f"d{b}", rng.integers(0, s["vocab"], size=CTX).tolist(), [])])
        tok = [int(t) for t in rng.integers(0, s["vocab"], size=BATCH)]

        def decode():
            eng.step_forced([(f"d{b}", [tok[b]], [0]) for b in range(BATCH)]).next_tokens.cpu()
        ms_decode = _time(torch, decode, min(steps, 40), warmup)
        launches = ex.launches_last_step
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            relaunch_last_step(ex)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            relaunch_last_step(ex)
        ms_decode_graph = _time(torch, graph.replay, steps, warmup)
        del graph
        h2d = BATCH * (4 + 8 + 8 + 4 + 4 + 4 + 4) + BATCH * ((CTX + 64) // page + 1) * 4
        for b in range(BATCH):
            eng.finish_request(f"d{b}")
        del eng, ex
        torch.cuda.empty_cache()
        lilovik = _lilovik_model(torch, s, dev, steps, warmup, len(RUNS))
        rows = _kernel_rows(torch, s, dev, max(3, steps // 2), 3, hbm, tf)
        torch.cuda.empty_cache()
        out_sizes[name] = {
            "sizes": s, "layer_runs": len(RUNS),
            "prefill_tokens_per_s": round(PROMPT / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3), "prefill_launches": prefill_launches,
            "decode_tokens_per_s": round(BATCH / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
            "decode_graph_tokens_per_s": round(BATCH / ms_decode_graph * 1e3, 1), "decode_graph_ms_per_step": round(ms_decode_graph, 4),
            "lilovik_equal_size": lilovik, "decode_launches_per_step": launches, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": BATCH * 4,
            "kernels": rows,
        }
        headline = out_sizes[name]
    clocks = sampler.stop(t_clock0, time.time())             # all of the run: every size's model steps and kernel rows are timed regions
    line = {
        "metric": "Surinex decode tokens/s, batch 32, context 4096, 4k-wide layer sizes (5 layer runs), through the engine's executor",
        "value": headline["decode_graph_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": headline["decode_graph_ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, random tokens)", "impl": "ours",
        "gpu_launches": headline["decode_launches_per_step"], "clocks": clocks,
        "e2e": {"value": headline["decode_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": headline["h2d_bytes_per_step"],
                "d2h_bytes_per_step": headline["d2h_bytes_per_step"]},
        "config": {"design": "Surinex", "batch": BATCH, "ctx": CTX, "prompt": PROMPT, "peaks": src, "hbm_gbs": hbm, "bf16_tflops": tf,
                   "l2": "kernel rows flush L2 between iterations; model steps stream more than L2", "sizes": out_sizes},
    }
    os.write(json_fd, (json.dumps(line) + "\n").encode())
