"""bench.py --design nemasun: prefill and decode throughput of the Nemasun design (random weights) at sizes that
resemble real models' layers, beside the framework's closest existing model — Llama — at equal width, head counts,
head size, layer count and (mean) ACTIVATED feed-forward size, and the design's hot kernels against the measured
peaks beside their Llama counterparts.  Not the headline (config 2 is); ONE JSON line in the same format.

Per size: a model of a few layers (dense and routed feed-forwards alternating) is served through the engine's
executor: `prefill` = one 4096-token prompt in one step; `decode` = one step of 32 sequences at context 4096 (built
by prefilling them), timed with CUDA events around K executor steps after W warm-up steps, inputs shipped from pinned
memory every step, sampled tokens read back; the same step replayed from a CUDA graph is the device-only figure.
Kernel rows: achieved FLOP/s or bytes/s over the measured peaks of MEASURED_PEAKS.json (fallback figures when absent);
L2 is flushed between their iterations."""
from __future__ import annotations

import json
import math
import os

from bench_hybrid import BATCH, CTX, PROMPT, _llama_decode, _peaks, _time
from bench_patadra import _row

SIZES = {
    "2k-wide": dict(width=2048, lanes=4, heads=32, kv_heads=8, dim=64, window=1024, keep=4, table_rows=512, ff=8192, limit=7.0,
                    experts=32, identity=4, top=4, groups=4, keep_groups=2, expert_ff=1024, shared_ff=2048, vocab=32000,
                    kinds=("dense", "moe", "dense", "moe")),
    "4k-wide": dict(width=4096, lanes=4, heads=32, kv_heads=8, dim=128, window=4096, keep=4, table_rows=1024, ff=14336, limit=7.0,
                    experts=64, identity=8, top=6, groups=8, keep_groups=4, expert_ff=1408, shared_ff=2816, vocab=32000,
                    kinds=("dense", "moe")),
}


def _spec(s):
    from atoma_infer_b200.hybrid import ClampedMlpSpec, HybridSpec, LayerSpec, MoeSpec, SoftmaxAttentionSpec
    att = SoftmaxAttentionSpec(s["heads"], s["kv_heads"], s["dim"], s["dim"], 1.0 / math.sqrt(s["dim"]), s["window"], s["keep"], True, True, True)
    dense = ClampedMlpSpec(s["ff"], s["limit"], 1.702, 1.0, True)
    moe = MoeSpec(experts=s["experts"], top=s["top"], ff=s["expert_ff"], shared_ff=s["shared_ff"], alpha=1.0, up_shift=0.0, renormalize=True,
                  score="softmax", correction=True, groups=s["groups"], keep_groups=s["keep_groups"], identity=s["identity"], scale_input=False)
    layers = tuple(LayerSpec("softmax_attention", softmax=att, clamped_mlp=dense if k == "dense" else None, moe=moe if k == "moe" else None, source=i)
                   for i, k in enumerate(s["kinds"]))
    return HybridSpec(s["width"], s["vocab"], 1e-6, 1.0, layers, norm_offset=0.0, block_style="lanes", position="none", lanes=s["lanes"],
                      embed_scale=1.0)


def _weights(torch, spec, s, dev):
    g = torch.Generator(device=dev).manual_seed(13)

    def r(*shape, scale=1.0, mean=0.0):
        return (mean + torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)

    W, S = spec.width, spec.lanes
    out = {"embed": r(spec.vocab, W), "head": r(spec.vocab, W, scale=W ** -0.5), "final_norm": r(W, scale=0.1, mean=1.0), "layers": []}
    for ls in spec.layers:
        a = ls.softmax
        w = {"norm1": r(W, scale=0.1, mean=1.0), "w_qkv": r(a.heads * a.dim + a.kv_heads * a.dim + a.heads * a.vdim, W, scale=W ** -0.5),
             "q_norm": r(a.dim, scale=0.1, mean=1.0), "k_norm": r(a.dim, scale=0.1, mean=1.0),
             "dist_bias": torch.randn((s["table_rows"], a.heads), generator=g, device=dev) * 0.5,
             "w_o": r(W, a.heads * a.vdim, scale=(a.heads * a.vdim) ** -0.5)}
        for q in (1, 2):
            w[f"lanes_in{q}"], w[f"lanes_out{q}"] = torch.full((S,), 1.0 / S), torch.ones(S)
            w[f"lanes_mix{q}"] = torch.eye(S) * 0.9 + 0.1 / S
        if ls.clamped_mlp is not None:
            f = ls.clamped_mlp
            w.update(norm2=r(W, scale=0.1, mean=1.0), w_gate_up=r(2 * f.ff, W, scale=W ** -0.5), b_gate_up=r(2 * f.ff, scale=0.1),
                     w_down=r(W, f.ff, scale=f.ff ** -0.5), b_down=r(W, scale=0.1))
        if ls.moe is not None:
            e = ls.moe
            w.update(norm2=r(W, scale=0.1, mean=1.0), w_router=r(e.experts + e.identity, W, scale=W ** -0.5),
                     router_correction=r(e.experts + e.identity, scale=0.01), w_expert_gate_up=r(e.experts, 2 * e.ff, W, scale=W ** -0.5),
                     w_expert_down=r(e.experts, W, e.ff, scale=e.ff ** -0.5), w_ff_in=r(2 * e.shared_ff, W, scale=W ** -0.5),
                     w_down=r(W, e.shared_ff, scale=e.shared_ff ** -0.5))
        out["layers"].append(w)
    return out


def _kernel_rows(torch, s, dev, steps, warmup, hbm, tf):
    """The design's kernels beside Llama's like kernels at the same shapes."""
    from atoma_infer_b200 import hybrid_ops as ho, ops
    H, G, D, W, S = s["heads"], s["kv_heads"], s["dim"], s["width"], PROMPT
    bf, page = torch.bfloat16, 16
    rows = {}
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    win, keep = s["window"], s["keep"]
    table = torch.randn((s["table_rows"], H), device=dev) * 0.5
    scale = 1 / math.sqrt(D)
    # ---- prompt attention: one prompt of S tokens under the window ----
    nb = S // page
    kc, vc = torch.randn((nb * page, G, D), device=dev, dtype=bf), torch.randn((nb * page, G, D), device=dev, dtype=bf)
    q = torch.randn((S, H * D), device=dev, dtype=bf)
    gate = torch.randn((S, H * D), device=dev, dtype=bf)
    pos = torch.arange(S, device=dev, dtype=torch.int64)
    tseq = torch.zeros(S, device=dev, dtype=torch.int32)
    bt = torch.arange(nb, device=dev, dtype=torch.int32).reshape(1, nb)
    qs = torch.tensor([0, S], device=dev, dtype=torch.int32)
    f = lambda: ho.softmax_attention_paged(q, kc, vc, pos, tseq, bt, H, G, D, D, page, scale, window=win, keep_first=keep, dist_bias=table,
                                           gate=gate, max_query_len=S, query_start=qs, max_seq_len=S)
    pairs = sum(min(i + 1, win) + min(keep, max(0, i + 1 - win)) for i in range(S))
    rows["softmax_attention_prefill_short_portions"] = _row(_time(torch, f, steps, warmup, flush), flops=4.0 * H * D * pairs, tf=tf)
    # the same prompt as a long portion (what portions of 128 tokens and more run): gather + tensor-memory kernel + kept-token merge and gate
    f = lambda: ho.softmax_attention_paged(q, kc, vc, pos, tseq, bt, H, G, D, D, page, scale, window=win, keep_first=keep, dist_bias=table,
                                           gate=gate, max_query_len=S, query_start=qs, max_seq_len=S, long_min_q=128, long_stats=(1, S, 0))
    rows["softmax_attention_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=4.0 * H * D * pairs, tf=tf)
    q3 = torch.randn((S, H, D), device=dev, dtype=bf)
    k3, v3 = torch.randn((S, G, D), device=dev, dtype=bf), torch.randn((S, G, D), device=dev, dtype=bf)
    cu = torch.tensor([0, S], device=dev, dtype=torch.int32)
    f = lambda: ops.flash_attn_varlen(q3, k3, v3, cu, cu, S, S, scale, True)
    rows["llama_attention_prefill"] = _row(_time(torch, f, steps, warmup, flush), flops=4.0 * H * D * S * (S + 1) / 2, tf=tf)
    del kc, vc
    # ---- decode attention: BATCH sequences at context CTX ----
    mb = (CTX + page) // page
    nb = BATCH * mb
    kc, vc = torch.randn((nb * page, G, D), device=dev, dtype=bf), torch.randn((nb * page, G, D), device=dev, dtype=bf)
    qd = torch.randn((BATCH, H * D), device=dev, dtype=bf)
    gd = torch.randn((BATCH, H * D), device=dev, dtype=bf)
    pos = torch.full((BATCH,), CTX, device=dev, dtype=torch.int64)
    tseq = torch.arange(BATCH, device=dev, dtype=torch.int32)
    bt = torch.randperm(nb, device=dev).to(torch.int32).reshape(BATCH, mb)
    qs = torch.arange(BATCH + 1, device=dev, dtype=torch.int32)
    f = lambda: ho.softmax_attention_paged(qd, kc, vc, pos, tseq, bt, H, G, D, D, page, scale, window=win, keep_first=keep, dist_bias=table,
                                           gate=gd, max_query_len=1, query_start=qs, max_seq_len=CTX + 1)
    seen = min(CTX + 1, win) + min(keep, max(0, CTX + 1 - win))
    rows["softmax_attention_decode"] = _row(_time(torch, f, steps, warmup, flush), nbytes=BATCH * seen * G * 2 * D * 2, hbm=hbm)
    rows["softmax_attention_decode"]["keys_per_sequence"] = seen
    k4, v4 = kc.view(nb, page, G, D), vc.view(nb, page, G, D)
    q4 = torch.randn((BATCH, 1, H, D), device=dev, dtype=bf)
    sl = torch.full((BATCH,), CTX + 1, device=dev, dtype=torch.int32)
    f = lambda: ops.flash_attn_kv_cache_full(q4, k4, v4, None, scale, bt, sl, True)
    rows["llama_attention_decode"] = _row(_time(torch, f, steps, warmup, flush), nbytes=BATCH * (CTX + 1) * G * 2 * D * 2, hbm=hbm)
    del kc, vc, k4, v4
    # ---- per-head norms + cache write ----
    T = 8192
    ncol = H * D + G * D + H * D
    proj = torch.randn((T, ncol), device=dev, dtype=bf)
    kc, vc = torch.empty((T, G, D), device=dev, dtype=bf), torch.empty((T, G, D), device=dev, dtype=bf)
    slots = torch.randperm(T, device=dev).to(torch.int64)
    qw = torch.ones(D, device=dev)
    f = lambda: ho.qk_headnorm_cache(proj, 0, H * D, H * D, qw, qw, 0.0, slots, kc, vc, H, G, D, D, 1e-6)
    rows["qk_headnorm_cache"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * ((H + G) * D * 2 + H * D * 2 + 2 * G * D * 2), hbm=hbm)
    del proj, kc, vc
    # ---- lanes: write back + next read + norm, beside Llama's add + RMS norm ----
    L = s["lanes"]
    y = torch.randn((T, W), device=dev, dtype=bf)
    x = torch.randn((T, L, W), device=dev)
    mix, wo, wi, w1 = torch.eye(L, device=dev), torch.ones(L, device=dev), torch.ones(L, device=dev) / L, torch.ones(W, device=dev)
    f = lambda: ho.lanes_update_norm(x, y, mix, wo, bf, eps=1e-6, w_in_next=wi, w_next=w1)
    rows["lanes_update_norm"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * (2 + 2 * 4 * L + 2), hbm=hbm)
    if hasattr(ops, "add_rmsnorm"):
        res, wbf = torch.randn((T, W), device=dev, dtype=bf), torch.ones(W, device=dev, dtype=bf)
        f = lambda: ops.add_rmsnorm(y, res, wbf, 1e-5)
        rows["llama_add_rmsnorm"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * 2 * 4, hbm=hbm)
    del x, y
    # ---- router and routed experts: prompt (compute bound) and decode step (weight stream) beside a dense feed-forward of the activated size ----
    E, ident, top, ff = s["experts"], s["identity"], s["top"], s["expert_ff"]
    wgu = torch.randn((E, 2 * ff, W), device=dev, dtype=bf) * W ** -0.5
    wd = torch.randn((E, W, ff), device=dev, dtype=bf) * ff ** -0.5
    wr = torch.randn((E + ident, W), device=dev) * W ** -0.5
    corr = torch.randn(E + ident, device=dev) * 0.01
    for name, T in (("prefill", S), ("decode", BATCH)):
        h = torch.randn((T, W), device=dev, dtype=bf)
        idx, wgt = ho.moe_route_grouped(h, wr, corr, top, s["groups"], s["keep_groups"])
        real = idx[(idx >= 0) & (idx < E)]
        used, pairs = int(torch.unique(real).numel()), int(real.numel())
        f = lambda: ho.moe_expert_rows(h, idx, wgt, wgu, wd, 0.0, 1.0, 0.0, scale_input=False)
        ms = _time(torch, f, steps, warmup, flush)
        rows[f"experts_{name}"] = _row(ms, flops=6.0 * pairs * ff * W, nbytes=used * 3 * ff * W * 2, hbm=hbm, tf=tf)
        rows[f"experts_{name}"].update(experts_used=used, pairs_on_experts=pairs, pairs_on_identity=int((idx >= E).sum()))
        f = lambda: ho.moe_route_grouped(h, wr, corr, top, s["groups"], s["keep_groups"])
        rows[f"router_{name}"] = _row(_time(torch, f, steps, warmup, flush), nbytes=T * W * 2 + (E + ident) * W * 4, hbm=hbm)
        F = top * ff
        wgu_d, wd_d = torch.randn((2 * F, W), device=dev, dtype=bf), torch.randn((W, F), device=dev, dtype=bf)
        f = lambda: ho.linear(ho.glu(ho.linear(h, wgu_d), 0), wd_d)
        rows[f"llama_mlp_{name}"] = _row(_time(torch, f, steps, warmup, flush), flops=6.0 * T * F * W, nbytes=3 * F * W * 2, hbm=hbm, tf=tf)
        del wgu_d, wd_d
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
    for name, s in SIZES.items():
        spec = _spec(s)
        weights = _weights(torch, spec, s, dev)
        nblocks = BATCH * ((CTX + 64) // page + 1) + PROMPT // page + 8
        ex = HybridExecutor(spec, weights, torch.bfloat16, dev, nblocks, page, 0)
        del weights
        eng = Engine(ex, CacheManager(nblocks, page, 0), max_num_batched_tokens=PROMPT, max_num_seqs=BATCH + 1)
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
        n = len(spec.layers)
        act_ff = sum(s["ff"] if k == "dense" else s["top"] * s["expert_ff"] + s["shared_ff"] for k in s["kinds"]) // n
        llama = dict(width=s["width"], heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], ff=act_ff // 64 * 64, vocab=s["vocab"], layers=n)
        ms_llama = _llama_decode(torch, llama, dev, steps, warmup)
        rows = _kernel_rows(torch, s, dev, max(3, steps // 2), 3, hbm, tf)
        torch.cuda.empty_cache()
        out_sizes[name] = {
            "sizes": {k: (list(v) if isinstance(v, tuple) else v) for k, v in s.items()}, "layers": n,
            "prefill_tokens_per_s": round(PROMPT / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3), "prefill_launches": prefill_launches,
            "decode_tokens_per_s": round(BATCH / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
            "decode_graph_tokens_per_s": round(BATCH / ms_decode_graph * 1e3, 1), "decode_graph_ms_per_step": round(ms_decode_graph, 4),
            "llama_equal_size": llama, "llama_decode_tokens_per_s": round(BATCH / ms_llama * 1e3, 1) if ms_llama else None,
            "llama_decode_ms_per_step": round(ms_llama, 4) if ms_llama else None,
            "decode_launches_per_step": launches, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": BATCH * 4, "kernels": rows,
        }
        headline = out_sizes[name]
    line = {
        "metric": "Nemasun decode tokens/s, batch 32, context 4096, 4k-wide layer sizes (2 layers), through the engine's executor",
        "value": headline["decode_graph_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": headline["decode_graph_ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, random tokens)", "impl": "ours",
        "gpu_launches": headline["decode_launches_per_step"],
        "e2e": {"value": headline["decode_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": headline["h2d_bytes_per_step"],
                "d2h_bytes_per_step": headline["d2h_bytes_per_step"]},
        "config": {"design": "Nemasun", "batch": BATCH, "ctx": CTX, "prompt": PROMPT, "peaks": src, "hbm_gbs": hbm, "bf16_tflops": tf,
                   "l2": "kernel rows flush L2 between iterations; model steps stream more than L2", "sizes": out_sizes},
    }
    os.write(json_fd, (json.dumps(line) + "\n").encode())
