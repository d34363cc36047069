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
def gated_linear_attention(h, P, pre, m, eps):
    """Per head a [dim, vdim] state whose rows decay by a data-dependent factor per key channel."""
    T = h.shape[0]
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ P[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ P[pre + "k"].T).reshape(T, H, D)
    v = (h @ P[pre + "v"].T).reshape(T, H, V)
    z = (h @ P[pre + "a1"].T) @ P[pre + "a2"].T + P[pre + "a2.b"]
    alpha = (sigma(z) ** (1.0 / tau)).reshape(T, H, D)
    o = torch.zeros(T, H, V, dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, P[pre + "norm"], eps).reshape(T, H * V)
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
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], positions, freqs, "halves")
    dkv = h @ P[pre + "dkv"].T
    c = rms_norm(dkv[:, :R], P[pre + "dkv.norm"], eps)
    k_rot = rotate(dkv[:, R:], positions, freqs, "halves")
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
    rot = m["rot"]
    f_qk = rotary_frequencies(int(rot["dims"]), rot["base"], rot.get("scaling"))
    f_v = rotary_frequencies(V, rot["base"], None)
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


def gated_delta_rule(h, P, pre, m, eps):
    """Per head a [dim, vdim] state: decay, then replace what the key reads by a blend with the new value, then read."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def short(name, n):
        return silu(causal_taps(h @ P[pre + name].T, P[pre + name + ".conv"])).reshape(T, n, -1)

    q, k, v = short("q", G), short("k", G), short("v", H)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigma(h @ P[pre + "b"].T)
    decay = torch.exp(-torch.exp(P[pre + "A_log"]) * softplus(h @ P[pre + "a"].T + P[pre + "dt_bias"]))
    o = torch.zeros(T, H, V, dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            o[t, hd] = S[hd].T @ q[t, g]
    o = rms_norm(o, P[pre + "norm"], eps).reshape(T, H * V)
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
        y = paired_mixer(hm, P, p + "mix.", m, eps, positions)
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
