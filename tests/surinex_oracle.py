"""Plain float64 restatement of the Surinex design: one function per mechanism, Python loops, whole sequences,
no paging, no batching, no carried state.  It shares no code with the package; the GPU tests compare the framework
against it.

Notation: matrices are stored [out, in] and applied as `h @ W.T`; sigma is the logistic function; P are the weights
by their checkpoint names; a layer's sublayers both read ONE normed input, each through its own causal tap filter.
"""
import math

import torch

F64 = torch.float64


def sigma(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigma(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def unit_rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(v, weight, eps):
    return unit_rms(v, eps) * weight


# ---- causal tap filters ----
def causal_taps(x, w):
    """x [T, C], w [C, taps]; the last column weighs the current token, the one before it the previous token, ...;
    what lies before the sequence is zero."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * x[s]
    return out


def tap_residual(h, w):
    """What a sublayer reads: its input plus the tap filter of its input."""
    return h + causal_taps(h, w)


# ---- rotations ----
def rotary_frequencies(dims, base, scaling=None):
    """dims / 2 frequencies base^(-2i / dims); `scaling` = {factor, low, high, original} stretches long wavelengths:
    untouched below original / high, divided by factor above original / low, blended in between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > orig / lo:
                f = f / fac
            elif wave >= orig / hi:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate(x, positions, freqs, layout, sign=1.0):
    """x [T, ..., n]: the first 2 len(freqs) entries of the last axis are turned pairwise by sign * position * freq;
    layout "interleaved" pairs (2i, 2i + 1), "halves" pairs (i, i + len(freqs))."""
    nf = len(freqs)
    if nf == 0:
        return x.clone()
    ang = sign * torch.as_tensor(positions, dtype=F64)[:, None] * freqs[None, :]        # [T, nf]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    if layout == "interleaved":
        a, b = x[..., 0:2 * nf:2], x[..., 1:2 * nf:2]
        out[..., 0:2 * nf:2] = a * c - b * s
        out[..., 1:2 * nf:2] = b * c + a * s
    else:
        a, b = x[..., :nf], x[..., nf:2 * nf]
        out[..., :nf] = a * c - b * s
        out[..., nf:2 * nf] = b * c + a * s
    return out


# ---- mixers ----
def gla_recurrence(q, k, v, alpha):
    """q, k, alpha [T, H, D], v [T, H, V] -> [T, H, V]:  S <- diag(alpha) S + k v^T;  o = S^T q."""
    T, H, D = q.shape
    V = v.shape[-1]
    o = torch.zeros(T, H, V, dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def gated_linear_attention(h, P, pre, m, eps):
    """Per head a [dim, vdim] state whose rows decay by a data-dependent factor per key channel."""
    T = h.shape[0]
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ P[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ P[pre + "k"].T).reshape(T, H, D)
    v = (h @ P[pre + "v"].T).reshape(T, H, V)
    z = (h @ P[pre + "a1"].T) @ P[pre + "a2"].T + P[pre + "a2.b"]
    alpha = (sigma(z) ** (1.0 / tau)).reshape(T, H, D)
    o = rms_norm(gla_recurrence(q, k, v, alpha), P[pre + "norm"], eps).reshape(T, H * V)
    return (o * silu(h @ P[pre + "g"].T)) @ P[pre + "o"].T


def latent_attention(h, P, pre, m, eps, positions):
    """Queries through a normed low-rank latent; keys and values expanded from a normed shared latent; one rotated key
    part shared by all heads."""
    T = h.shape[0]
    H, D, Rd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    freqs = rotary_frequencies(int(rot.get("dims", Rd)), rot.get("base", 10000.0), rot.get("scaling"))
    cq = rms_norm(h @ P[pre + "dq"].T, P[pre + "dq.norm"], eps)
    q = (cq @ P[pre + "uq"].T).reshape(T, H, D + Rd)
    layout = rot.get("layout", "halves")
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], positions, freqs, layout)
    dkv = h @ P[pre + "dkv"].T
    c = rms_norm(dkv[:, :R], P[pre + "dkv.norm"], eps)
    k_rot = rotate(dkv[:, R:], positions, freqs, layout)
    k_plain = (c @ P[pre + "uk"].T).reshape(T, H, D)
    v = (c @ P[pre + "uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        for hd in range(H):
            s = (k_plain[: i + 1, hd] @ q_plain[i, hd] + k_rot[: i + 1] @ q_rot[i, hd]) * float(m["scale"])
            out[i, hd] = torch.softmax(s, 0) @ v[: i + 1, hd]
    return out.reshape(T, H * V) @ P[pre + "o"].T


def sigmoid_attention_rotated_values(h, P, pre, m, eps, positions, layout="interleaved"):
    """Unnormalised attention: a visible key weighs sigma(score + per-head bias).  Values are turned by their own position
    when stored and a head's sum is turned back by the query's position."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    f_qk = rotary_frequencies(int(rot["dims"]), rot["base"], rot.get("scaling")) if rot else torch.zeros(0, dtype=F64)
    f_v = rotary_frequencies(V, rot["base"], None) if rot else torch.zeros(0, dtype=F64)
    q = rms_norm((h @ P[pre + "q"].T).reshape(T, H, D), P[pre + "q.norm"], eps)
    k = rms_norm((h @ P[pre + "k"].T).reshape(T, G, D), P[pre + "k.norm"], eps)
    q, k = rotate(q, positions, f_qk, layout), rotate(k, positions, f_qk, layout)
    v = rotate((h @ P[pre + "v"].T).reshape(T, G, V), positions, f_v, layout)
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            w = sigma((k[: i + 1, g] @ q[i, hd]) * float(m["scale"]) + P[pre + "pb"][hd])
            out[i, hd] = w @ v[: i + 1, g]
    out = rotate(out, positions, f_v, layout, sign=-1.0)
    return out.reshape(T, H * V) @ P[pre + "o"].T


def unit_length(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def delta_recurrence(q, k, v, beta, decay):
    """q, k [T, G, D] (head h reads group h // (H / G)), v [T, H, V], beta, decay [T, H] -> [T, H, V]:
    S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q (the read-out sees the token's own write)."""
    T, G, D = q.shape
    H, V = v.shape[1], v.shape[2]
    o = torch.zeros(T, H, V, dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            o[t, hd] = S[hd].T @ q[t, g]
    return o


def gated_delta_rule(h, P, pre, m, eps):
    """Per head a [dim, vdim] state: decay, then replace what the key reads by a blend with the new value, then read."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def short(name, n):
        return silu(causal_taps(h @ P[pre + name].T, P[pre + name + ".conv"])).reshape(T, n, -1)

    q, k, v = unit_length(short("q", G)) * D ** -0.5, unit_length(short("k", G)), short("v", H)
    beta = sigma(h @ P[pre + "b"].T)
    decay = torch.exp(-torch.exp(P[pre + "A_log"]) * softplus(h @ P[pre + "a"].T + P[pre + "dt_bias"]))
    o = rms_norm(delta_recurrence(q, k, v, beta, decay), P[pre + "norm"], eps).reshape(T, H * V)
    return (o * silu(h @ P[pre + "g"].T)) @ P[pre + "o"].T


def paired_mixer(h, P, pre, m, eps, positions, layout="interleaved"):
    """Two mixers on the same input; each result is normed over the model width before the two are averaged."""
    left = sigmoid_attention_rotated_values(h, P, pre + "left.", m["left"], eps, positions, layout)
    right = gated_delta_rule(h, P, pre + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, P[pre + "left.out"], eps) + rms_norm(right, P[pre + "right.out"], eps))


# ---- feed-forward ----
def gated_ff(h, P, pre):
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


# ---- the model ----
def layer(x, P, i, lc, eps, positions):
    p = f"l{i}."
    h = rms_norm(x, P[p + "norm1"], eps)
    hm = tap_residual(h, P[p + "canon1"])
    m, kind = lc["mixer"], lc["type"]
    if kind == "gla":
        y = gated_linear_attention(hm, P, p + "mix.", m, eps)
    elif kind == "latent_attention":
        y = latent_attention(hm, P, p + "mix.", m, eps, positions)
    elif kind == "parallel":
        y = paired_mixer(hm, P, p + "mix.", m, eps, positions, (m["left"].get("rot") or {}).get("layout", "interleaved"))
    else:
        raise ValueError(kind)
    if lc.get("mlp") is not None:
        y = y + gated_ff(tap_residual(h, P[p + "canon2"]), P, p + "mlp.")
    return x + y


def layer_runs(cfg):
    """(layer index, number of the pass that starts at this run or None) for every run, in order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, P, tokens):
    """tokens -> (logits [T, vocab], residual stream after every layer run [runs, T, width]), float64."""
    P = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in P.items()}
    eps = float(cfg["norm"]["eps"])
    positions = list(range(len(tokens)))
    x0 = P["embed"][torch.as_tensor(tokens)]
    x = x0.clone()
    trace = []
    for i, start_of_pass in layer_runs(cfg):
        if start_of_pass is not None:
            if start_of_pass > 0:
                x = x + x0
            x = x + P["loop.step"][start_of_pass]
        x = layer(x, P, i, cfg["layers"][i], eps, positions)
        trace.append(x)
    logits = rms_norm(x, P["final.norm"], eps) @ P["head"].T
    return logits, torch.stack(trace)


# ---- random small models for the tests ----
def random_config(width=48, vocab=61, taps=3, kinds=("gla", "latent_attention", "parallel", "gla"), loop=(0, 2, 2), ff=40, mlps=None, eps=1e-5,
                  gla=None, latent=None, left=None, right=None):
    """A configuration in the checkpoint's format.  `mlps`: per layer True / False (no feed-forward); mixer sizes by keyword."""
    g_ = dict(heads=2, dim=16, vdim=24, tau=8.0)
    g_.update(gla or {})
    l_ = dict(heads=3, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=32, scale=0.2, rot=dict(base=5000.0, dims=8))
    l_.update(latent or {})
    a_ = dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, rot=dict(base=20000.0, dims=8, scaling=dict(factor=3.0, low=1.0, high=3.0, original=64)))
    a_.update(left or {})
    r_ = dict(heads=4, kv_heads=2, dim=16, vdim=24, conv=3)
    r_.update(right or {})
    layers = []
    for i, kind in enumerate(kinds):
        mixer = {"gla": g_, "latent_attention": l_, "parallel": dict(left=a_, right=r_)}[kind]
        has = True if mlps is None else mlps[i]
        layers.append(dict(type=kind, mixer=json_copy(mixer), mlp=dict(kind="dense", ff=ff) if has else None))
    cfg = dict(architecture="Surinex", vocab=vocab, width=width, norm=dict(eps=eps), canon=dict(taps=taps), layers=layers)
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


def json_copy(x):
    import json
    return json.loads(json.dumps(x))


def random_weights(cfg, g, decay_rank=5):
    """float32 tensors under the checkpoint's names, already rounded to bfloat16 values (so that a bfloat16 file holds them exactly)."""
    W, P = cfg["width"], {}

    def rnd(*shape, scale=1.0, shift=0.0):
        return ((torch.randn(*shape, generator=g) * scale + shift).to(torch.bfloat16)).float()

    def lin(out, inp, gain=1.0):
        return rnd(out, inp, scale=gain * inp ** -0.5)

    P["embed"], P["head"], P["final.norm"] = rnd(cfg["vocab"], W), lin(cfg["vocab"], W), rnd(W, scale=0.1, shift=1.0)
    if cfg.get("loop"):
        P["loop.step"] = rnd(cfg["loop"]["times"], W, scale=0.3)
    taps = cfg["canon"]["taps"]
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        P[p + "norm1"] = rnd(W, scale=0.1, shift=1.0)
        P[p + "canon1"] = rnd(W, taps, scale=0.3)
        if l["mlp"] is not None:
            F = l["mlp"]["ff"]
            P[p + "canon2"] = rnd(W, taps, scale=0.3)
            P[p + "mlp.gate"], P[p + "mlp.up"], P[p + "mlp.down"] = lin(F, W), lin(F, W), lin(W, F)
        q = p + "mix."
        if l["type"] == "gla":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            P[q + "q"], P[q + "k"], P[q + "v"], P[q + "g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            P[q + "a1"], P[q + "a2"], P[q + "a2.b"] = lin(decay_rank, W), lin(H * D, decay_rank, 2.0), rnd(H * D, scale=1.0, shift=2.0)
            P[q + "norm"], P[q + "o"] = rnd(V, scale=0.1, shift=1.0), lin(W, H * V)
        elif l["type"] == "latent_attention":
            H, D, Rd, V, Rq, Rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            P[q + "dq"], P[q + "dq.norm"], P[q + "uq"] = lin(Rq, W), rnd(Rq, scale=0.1, shift=1.0), lin(H * (D + Rd), Rq, 2.0)
            P[q + "dkv"], P[q + "dkv.norm"] = lin(Rk + Rd, W, 2.0), rnd(Rk, scale=0.1, shift=1.0)
            P[q + "uk"], P[q + "uv"], P[q + "o"] = lin(H * D, Rk, 2.0), lin(H * V, Rk), lin(W, H * V)
        else:
            a, d = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            x = q + "left."
            P[x + "q"], P[x + "k"], P[x + "v"] = lin(H * D, W), lin(G * D, W), lin(G * V, W)
            P[x + "q.norm"], P[x + "k.norm"] = rnd(D, scale=0.2, shift=1.5), rnd(D, scale=0.2, shift=1.5)
            P[x + "pb"], P[x + "o"], P[x + "out"] = rnd(H, scale=0.5, shift=-2.0), lin(W, H * V), rnd(W, scale=0.1, shift=1.0)
            H, G, D, V, K = d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["conv"]
            x = q + "right."
            P[x + "q"], P[x + "k"], P[x + "v"], P[x + "g"] = lin(G * D, W), lin(G * D, W), lin(H * V, W), lin(H * V, W)
            P[x + "q.conv"], P[x + "k.conv"], P[x + "v.conv"] = rnd(G * D, K, scale=0.5), rnd(G * D, K, scale=0.5), rnd(H * V, K, scale=0.5)
            P[x + "b"], P[x + "a"] = lin(H, W), lin(H, W)
            P[x + "A_log"], P[x + "dt_bias"] = rnd(H, scale=0.5, shift=-1.0), rnd(H, scale=0.5)
            P[x + "norm"], P[x + "o"], P[x + "out"] = rnd(V, scale=0.1, shift=1.0), lin(W, H * V), rnd(W, scale=0.1, shift=1.0)
    return P
