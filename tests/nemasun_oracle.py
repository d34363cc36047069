"""Plain float64 restatement of the Nemasun design: one function per mechanism, Python loops, whole sequences,
no paging, no batching.  It shares no code with the package; the GPU tests compare the framework against it.

Notation: matrices are stored [out, in] and applied as `h @ W.T`; sigma is the logistic function; `lanes` is the
list of residual lanes (the design keeps several copies of the residual stream and mixes them around every sublayer).
"""
import math

import torch

F64 = torch.float64


def sigma(z):
    return 1.0 / (1.0 + torch.exp(-z))


def unit_rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(v, weight, eps):
    return unit_rms(v, eps) * weight


# ---- embedding ----
def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens)] * scale


# ---- residual lanes ----
def lanes_read(lanes, w_in):
    """The sublayer's input before its norm: a weighted sum of the lanes."""
    return sum(w_in[s] * lanes[s] for s in range(len(lanes)))


def lanes_write(lanes, w_mix, w_out, y):
    """All lanes at once from the old ones: lane t <- sum_s w_mix[s, t] lane_s + w_out[t] y."""
    n = len(lanes)
    return [sum(w_mix[s, t] * lanes[s] for s in range(n)) + w_out[t] * y for t in range(n)]


# ---- attention ----
def distance_bucket(n, rows, far):
    """Row of the distance table for a distance n >= 0: one row per distance below rows // 2, logarithmic steps up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def visible(i, j, window, keep):
    return j <= i and (i - j < window or j < keep)


def attention(h, w_q, w_k, w_g, w_o, q_norm, k_norm, table, heads, kv_heads, dim, scale, far, window, keep, eps):
    """h [T, W] -> [T, W].  Values are the key projections as they leave w_k; scores use the normed ones."""
    T = h.shape[0]
    q = rms_norm((h @ w_q.T).reshape(T, heads, dim), q_norm, eps)
    v = (h @ w_k.T).reshape(T, kv_heads, dim)
    k = rms_norm(v, k_norm, eps)
    rep = heads // kv_heads
    rows = table.shape[0]
    out = torch.zeros(T, heads, dim, dtype=F64)
    for i in range(T):
        js = torch.tensor([j for j in range(i + 1) if visible(i, j, window, keep)])
        rows_of = torch.tensor([distance_bucket(i - int(j), rows, far) for j in js])
        for hd in range(heads):
            g = hd // rep
            s = (k[js, g] @ q[i, hd]) * scale + table[rows_of, hd]
            out[i, hd] = torch.softmax(s, 0) @ v[js, g]
    gate = sigma(h @ w_g.T)
    return (out.reshape(T, heads * dim) * gate) @ w_o.T


# ---- feed-forwards ----
def clamped_ff(h, w_gate, b_gate, w_up, b_up, w_down, b_down, limit):
    g = torch.clamp(h @ w_gate.T + b_gate, max=limit)
    u = torch.clamp(h @ w_up.T + b_up, -limit, limit)
    return (g * sigma(1.702 * g) * (u + 1.0)) @ w_down.T + b_down


def silu_ff(h, w_gate, w_up, w_down):
    g = h @ w_gate.T
    return (g * sigma(g) * (h @ w_up.T)) @ w_down.T


def route(h_row, w_router, correction, top, groups, keep_groups):
    """One token -> (chosen router outputs, their weights).  Softmax scores; the choice adds `correction` and is restricted
    to the `keep_groups` groups of neighbours whose best corrected score is largest; the weights are the plain scores of
    the chosen outputs over their sum."""
    s = torch.softmax(w_router @ h_row, 0)
    c = s + correction
    n = s.shape[0]
    per = n // groups
    best = [max(float(c[g * per + e]) for e in range(per)) for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-best[g], g))[:keep_groups]
    allowed = [e for e in range(n) if e // per in kept]
    chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    w = torch.stack([s[e] for e in chosen])
    return chosen, w / (w.sum() + 1e-20)


def moe_ff(h, w_router, correction, experts, identity, top, groups, keep_groups, shared):
    """experts: list of (w_gate, w_up, w_down); router outputs len(experts) .. + identity - 1 hand the input through."""
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, w = route(h[t], w_router, correction, top, groups, keep_groups)
        for e, we in zip(chosen, w):
            out[t] += we * (silu_ff(h[t:t + 1], *experts[e])[0] if e < len(experts) else h[t])
    if shared is not None:
        out = out + silu_ff(h, *shared)
    return out


# ---- the model ----
def forward(cfg, w, tokens):
    """cfg: the configuration as config.json has it; w: tensors by checkpoint name (float64).  Returns (logits [T, vocab],
    the sum of the lanes after every layer [layers, T, W])."""
    eps = cfg["norm"]["eps"]
    n_lanes = int(cfg.get("streams") or 1)
    if "streams" not in cfg:        # one residual stream, x <- x + y
        w = dict(w)
        for i in range(len(cfg["layers"])):
            for q in (1, 2):
                w[f"l{i}.hc{q}.in"], w[f"l{i}.hc{q}.out"], w[f"l{i}.hc{q}.mix"] = torch.ones(1, dtype=F64), torch.ones(1, dtype=F64), torch.ones(1, 1, dtype=F64)
    x0 = embed(tokens, w["embed"], cfg["embedding"]["scale"])
    lanes = [x0.clone() for _ in range(n_lanes)]
    trace = []
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = l["mixer"]
        mask = m.get("mask") or {}
        h = rms_norm(lanes_read(lanes, w[p + "hc1.in"]), w[p + "norm1"], eps)
        y = attention(h, w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.g"], w[p + "mix.o"], w[p + "mix.q.norm"], w[p + "mix.k.norm"],
                      w[p + "mix.rel"], m["heads"], m["kv_heads"], m["dim"], m["scale"], m["bias_max"],
                      mask.get("size") or (1 << 60), mask.get("keep_first") or 0, eps)
        lanes = lanes_write(lanes, w[p + "hc1.mix"], w[p + "hc1.out"], y)
        f = l.get("mlp")
        if f is not None:
            h = rms_norm(lanes_read(lanes, w[p + "hc2.in"]), w[p + "norm2"], eps)
            q = p + "mlp."
            if f["kind"] == "dense":
                y = clamped_ff(h, w[q + "gate"], w[q + "gate.b"], w[q + "up"], w[q + "up.b"], w[q + "down"], w[q + "down.b"], f["limit"])
            else:
                r = f["router"]
                ex = [(w[f"{q}e{k}.gate"], w[f"{q}e{k}.up"], w[f"{q}e{k}.down"]) for k in range(r["experts"])]
                sh = (w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"]) if f.get("shared") else None
                gr = r.get("groups") or {"count": 1, "keep": 1}
                y = moe_ff(h, w[q + "router"], w[q + "correction"], ex, r.get("identity") or 0, r["top"], gr["count"], gr["keep"], sh)
            lanes = lanes_write(lanes, w[p + "hc2.mix"], w[p + "hc2.out"], y)
        trace.append(sum(lanes))
    x = rms_norm(sum(lanes), w["final.norm"], eps)
    return x @ w["head"].T, torch.stack(trace)


# ---- test inputs ----
def random_config(width=48, vocab=61, lanes=2, layers=3, heads=4, kv_heads=2, dim=8, scale=0.3, table_rows=10, far=37, window=13, keep=3,
                  ff=40, limit=0.8, experts=6, identity=2, top=3, groups=4, keep_groups=2, expert_ff=20, shared_ff=12, embed_scale=3.0,
                  eps=1e-5, kinds=None):
    """A small configuration in the checkpoint's own format.  kinds: per layer "dense" | "moe" | None (default: alternating)."""
    kinds = kinds or [("dense", "moe", None)[i % 3] if layers > 2 else ("moe", "dense")[i % 2] for i in range(layers)]
    out = []
    for kind in kinds:
        mask = {}
        if window:
            mask["size"] = window
        if keep:
            mask["keep_first"] = keep
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "bias_max": far, "mask": mask, "_rows": table_rows}
        if kind == "dense":
            mlp = {"kind": "dense", "ff": ff, "limit": limit}
        elif kind == "moe":
            mlp = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep_groups}},
                   "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff} if shared_ff else None}
        else:
            mlp = None
        out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Nemasun", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "layers": out}
    if lanes:
        cfg["streams"] = lanes
    return cfg


def random_weights(cfg, g):
    """Random tensors under the checkpoint's names, rounded to what bfloat16 holds (float64)."""
    W, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")

    def r(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(F64)

    def mat(o, i):
        return r(o, i, s=1.0 / math.sqrt(i))

    w = {"embed": r(V, W, s=0.5), "head": mat(V, W), "final.norm": 1 + r(W, s=0.2)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, G, D = m["heads"], m["kv_heads"], m["dim"]
        w[p + "norm1"] = 1 + r(W, s=0.2)
        w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.g"], w[p + "mix.o"] = mat(H * D, W), mat(G * D, W), mat(H * D, W), mat(W, H * D)
        w[p + "mix.q.norm"], w[p + "mix.k.norm"] = 1 + r(D, s=0.3), 1 + r(D, s=0.3)
        w[p + "mix.rel"] = r(m["_rows"], H, s=1.5)
        for q in (1, 2):
            if S and (q == 1 or l["mlp"] is not None):
                w[f"{p}hc{q}.in"] = 1.0 / S + r(S, s=0.3)
                w[f"{p}hc{q}.out"] = 1 + r(S, s=0.3)
                w[f"{p}hc{q}.mix"] = (torch.eye(S) + torch.randn(S, S, generator=g) * 0.25).to(torch.bfloat16).to(F64)
        f = l["mlp"]
        if f is None:
            continue
        w[p + "norm2"] = 1 + r(W, s=0.2)
        q = p + "mlp."
        if f["kind"] == "dense":
            n = f["ff"]
            w[q + "gate"], w[q + "up"], w[q + "down"] = mat(n, W), mat(n, W), mat(W, n)
            w[q + "gate.b"], w[q + "up.b"], w[q + "down.b"] = r(n, s=0.5), r(n, s=0.5), r(W, s=0.5)
        else:
            ro, n = f["router"], f["expert"]["ff"]
            outs = ro["experts"] + ro.get("identity", 0)
            w[q + "router"] = r(outs, W, s=2.0 / math.sqrt(W))
            w[q + "correction"] = r(outs, s=0.15)          # the size of the scores themselves: it changes the choice, and some are negative
            for k in range(ro["experts"]):
                w[f"{q}e{k}.gate"], w[f"{q}e{k}.up"], w[f"{q}e{k}.down"] = mat(n, W), mat(n, W), mat(W, n)
            if f.get("shared"):
                n = f["shared"]["ff"]
                w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = mat(n, W), mat(n, W), mat(W, n)
    return {k: v.to(torch.bfloat16).to(F64) for k, v in w.items()}      # sums like 1 + r are rounded once more


def checkpoint_config(cfg):
    """The configuration without the generator's private keys (the table's row count is the tensor's shape)."""
    out = {k: v for k, v in cfg.items() if k != "layers"}
    out["layers"] = [{**l, "mixer": {k: v for k, v in l["mixer"].items() if not k.startswith("_")}} for l in cfg["layers"]]
    return out
