"""Surinex on the GPU against the plain implementation of tests/surinex_oracle.py (float64): every mechanism alone, then the
model through the engine — whole prompts, token-by-token decoding, portions down to two tokens, mixed batches against each
request alone, reused pages and state slots, keys far away and at page borders, the first tokens of a sequence, long decoding,
other sizes and layer orders, greedy generation through the scheduler and the command line."""
import json

import numpy as np
import pytest
import torch

import surinex_oracle as so

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
BOTH = [torch.float32, torch.bfloat16]


def _ops():
    from atoma_infer_b200 import hybrid_ops
    return hybrid_ops


@pytest.fixture(autouse=True)
def _reset_flags():
    yield
    if torch.cuda.is_available():
        _ops().debug_flags(0)


def nerr(got, want):
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    return float(((got - want) ** 2).mean().sqrt() / (want ** 2).mean().sqrt().clamp_min(1e-30))


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def bf(t):
    return t.to(torch.bfloat16).float()


def rnd(g, *shape, scale=1.0, shift=0.0):
    return bf(torch.randn(*shape, generator=g) * scale + shift)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def batch_layout(counts):
    """token_seq, query_start for sequences with `counts` tokens each in the step."""
    seq = [b for b, n in enumerate(counts) for _ in range(n)]
    return i32(seq), i32([0] + list(np.cumsum(counts)))


# ------------------------------------------------------------------------------------------------
# residual update of a parallel block
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("W,pair,ff,start", [(40, False, True, False), (64, True, True, True), (33, True, False, False), (50, False, False, True)])
def test_residual_update_with_what_precedes_the_next_layer(dtype, W, pair, ff, start):
    g = torch.Generator().manual_seed(W)
    T, eps = 7, 1e-5
    x, ya, yb, yf, e = rnd(g, T, W), rnd(g, T, W), rnd(g, T, W), rnd(g, T, W), rnd(g, T, W)
    na, nb, vec, wn = rnd(g, W, shift=1.0), rnd(g, W, shift=1.0), rnd(g, W), rnd(g, W, shift=1.0)
    mix = (0.5 * (so.rms_norm(ya.double(), na.double(), eps) + so.rms_norm(yb.double(), nb.double(), eps))) if pair else ya.double()
    after = x.double() + mix + (yf.double() if ff else 0)
    nxt = after + (e.double() + vec.double() if start else 0)
    xd = x.to(DEV).clone()
    h, trace = _ops().parallel_residual_norm(xd, dtype, y_a=ya.to(dtype).to(DEV), y_b=yb.to(dtype).to(DEV) if pair else None,
                                             y_ff=yf.to(dtype).to(DEV) if ff else None, norm_a=na.to(DEV) if pair else None,
                                             norm_b=nb.to(DEV) if pair else None, mix_scale=0.5 if pair else 1.0,
                                             add_rows=e.to(DEV) if start else None, add_vec=vec.to(DEV) if start else None, w_next=wn.to(DEV),
                                             eps=eps, want_trace=True)
    assert nerr(trace, after) < 1e-6 and nerr(xd, nxt) < 1e-6
    assert nerr(h, so.rms_norm(nxt, wn.double(), eps)) < tol(dtype, 1e-6, 5e-3)


# ------------------------------------------------------------------------------------------------
# tap filters with carried inputs
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("taps,C,residual,act", [(1, 40, True, 0), (2, 33, True, 0), (3, 64, True, 0), (4, 50, False, 1), (7, 24, False, 1)])
def test_tap_filters_over_portions_of_any_size(dtype, taps, C, residual, act):
    """Three sequences cut into steps of unequal portions (down to one token, shorter than the filter), on state slots whose old
    content is garbage: every step's output equals the filter over the whole sequence."""
    g = torch.Generator().manual_seed(taps * 100 + C)
    lens = [23, 9, 14]
    xs = [rnd(g, n, C) for n in lens]
    w1, w2 = rnd(g, C, taps, scale=0.5), rnd(g, C, taps, scale=0.5)

    def whole(x, w):
        y = so.causal_taps(x.double(), w.double())
        y = x.double() + y if residual else y
        return so.silu(y) if act else y

    want1, want2 = [whole(x, w1) for x in xs], [whole(x, w2) for x in xs]
    hist = torch.full((5, max(1, taps - 1) * C + 3), 77.0, device=DEV)
    slots = [4, 0, 2]
    done = [0, 0, 0]
    cuts = [[1, 1, 5, 2, 14], [9], [3, 1, 1, 1, 8]]
    step = 0
    while any(d < n for d, n in zip(done, lens)):
        members = [b for b in range(3) if step < len(cuts[b])]
        counts = [cuts[b][step] for b in members]
        x = torch.cat([xs[b][done[b]:done[b] + c] for b, c in zip(members, counts)]).to(dtype).to(DEV)
        tseq, qs = batch_layout(counts)
        o1, o2 = _ops().tap_filter(x, w1.to(DEV), w2.to(DEV), hist, i32([slots[b] for b in members]), tseq, qs,
                                   i32([done[b] for b in members]), residual, act)
        at = 0
        for b, c in zip(members, counts):
            assert nerr(o1[at:at + c], want1[b][done[b]:done[b] + c]) < tol(dtype, 1e-6, 8e-3), (step, b)
            assert nerr(o2[at:at + c], want2[b][done[b]:done[b] + c]) < tol(dtype, 1e-6, 8e-3), (step, b)
            at += c
            done[b] += c
        step += 1


@pytest.mark.parametrize("taps,act", [(2, 0), (3, 1), (4, 0)])
@pytest.mark.parametrize("counts", [[700, 3, 1, 520, 77], [2500, 1, 1700, 13]])
def test_tap_filters_on_long_steps(taps, act, counts):
    """Long steps, where a thread walks several tokens with the last inputs in registers: portions that start in the middle of a
    thread's run, sequences that continue from carried inputs beside fresh ones, against the plain filter over the whole sequences,
    and bit for bit against the kernel that reads every input anew."""
    C = 72
    g = torch.Generator().manual_seed(taps + len(counts))
    before = [5, 0, 1, 0, 2][:len(counts)]                   # tokens of each sequence that an earlier step brought
    xs = [bf(rnd(g, b + n, C)) for b, n in zip(before, counts)]
    w1, w2 = rnd(g, C, taps, scale=0.5), rnd(g, C, taps, scale=0.5)
    residual = not act

    def whole(x, w):
        y = so.causal_taps(x.double(), w.double())
        y = x.double() + y if residual else y
        return so.silu(y) if act else y

    outs = []
    for flags in (0, 2):
        _ops().debug_flags(flags)
        hist = torch.full((len(counts), (taps - 1) * C), 55.0, device=DEV)
        slots = i32(list(range(len(counts)))[::-1])
        first = [b for b in range(len(counts)) if before[b]]
        tseq, qs = batch_layout([before[b] for b in first])
        x0 = torch.cat([xs[b][:before[b]] for b in first]).to(torch.bfloat16).to(DEV)
        _ops().tap_filter(x0, w1.to(DEV), w2.to(DEV), hist, slots[first], tseq, qs, i32([0] * len(first)), residual, act)
        tseq, qs = batch_layout(counts)
        x = torch.cat([xs[b][before[b]:] for b in range(len(counts))]).to(torch.bfloat16).to(DEV)
        outs.append(_ops().tap_filter(x, w1.to(DEV), w2.to(DEV), hist, slots, tseq, qs, i32(before), residual, act))
    (a1, a2), (b1, b2) = outs
    assert torch.equal(a1, b1) and torch.equal(a2, b2)
    at = 0
    for b, n in enumerate(counts):
        assert nerr(a1[at:at + n], whole(xs[b], w1)[before[b]:]) < 8e-3, b
        assert nerr(a2[at:at + n], whole(xs[b], w2)[before[b]:]) < 8e-3, b
        at += n


# ------------------------------------------------------------------------------------------------
# matrix-state recurrences
# ------------------------------------------------------------------------------------------------
def scan_steps(cuts, lens, run):
    """Runs `run(members, counts, starts)` step by step over sequences cut as `cuts`; returns per sequence the concatenated rows."""
    done, got, step = [0] * len(lens), [[] for _ in lens], 0
    while any(d < n for d, n in zip(done, lens)):
        members = [b for b in range(len(lens)) if step < len(cuts[b])]
        counts = [cuts[b][step] for b in members]
        out = run(members, counts, [done[b] for b in members])
        at = 0
        for b, c in zip(members, counts):
            got[b].append(out[at:at + c].clone())
            at += c
            done[b] += c
        step += 1
    return [torch.cat(x) for x in got]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows", [0, 16])                  # 8 rows of the state per lane (steps of few CTAs) / many
@pytest.mark.parametrize("H,D,V,tau", [(2, 16, 24, 8.0), (3, 48, 40, 16.0), (1, 80, 72, 4.0), (2, 130, 32, 2.0), (4, 8, 5, 1.0), (1, 300, 9, 3.0)])
def test_gated_linear_attention_recurrence(dtype, rows, H, D, V, tau):
    _ops().debug_flags(rows)
    g = torch.Generator().manual_seed(H * 1000 + D)
    lens, cuts, slots = [37, 12], [[1, 20, 2, 14], [12]], [3, 1]
    qs_, ks_, vs_, zs_ = ([rnd(g, n, H * d_, scale=s) for n in lens] for d_, s in ((D, 1.0), (D, 0.5), (V, 1.0), (D, 2.0)))
    zb = rnd(g, H * D, shift=2.0)
    want = []
    for q, k, v, z in zip(qs_, ks_, vs_, zs_):
        n = q.shape[0]
        alpha = so.sigma(z.double() + zb.double()) ** (1.0 / tau)
        want.append(so.gla_recurrence((q.double() * D ** -0.5).reshape(n, H, D), k.double().reshape(n, H, D), v.double().reshape(n, H, V),
                                      alpha.reshape(n, H, D)).reshape(n, H * V))
    state = torch.full((4, H * D * V + 5), 9.0, device=DEV)

    def run(members, counts, starts):
        cat = lambda xs: torch.cat([xs[b][s:s + c] for b, c, s in zip(members, counts, starts)]).to(dtype).to(DEV)
        _, qs = batch_layout(counts)
        return _ops().gla_scan(cat(qs_), cat(ks_), cat(vs_), cat(zs_), zb.to(DEV), tau, D ** -0.5, state, i32([slots[b] for b in members]), qs,
                               i32(starts), H, D, V)

    for got, w in zip(scan_steps(cuts, lens, run), want):
        assert nerr(got, w) < 1e-5        # the inputs are bfloat16 values in both formats; the recurrence itself is float32


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows", [0, 16])
@pytest.mark.parametrize("H,G,D,V", [(4, 2, 16, 24), (2, 1, 32, 32), (3, 3, 80, 40), (6, 2, 48, 72), (2, 2, 130, 8), (1, 1, 260, 6)])
def test_gated_delta_rule_recurrence(dtype, rows, H, G, D, V):
    _ops().debug_flags(rows)
    g = torch.Generator().manual_seed(H * 1000 + D + 7)
    lens, cuts, slots = [41, 10], [[2, 1, 30, 8], [10]], [0, 2]
    qs_, ks_, vs_ = ([rnd(g, n, c) for n in lens] for c in (G * D, G * D, H * V))
    bs_, as_ = ([rnd(g, n, H) for n in lens] for _ in range(2))
    a_log, dt = rnd(g, H, scale=0.5, shift=-1.0), rnd(g, H, scale=0.5)
    want = []
    for q, k, v, b, a in zip(qs_, ks_, vs_, bs_, as_):
        n = q.shape[0]
        decay = torch.exp(-torch.exp(a_log.double()) * so.softplus(a.double() + dt.double()))
        want.append(so.delta_recurrence(so.unit_length(q.double().reshape(n, G, D)) * D ** -0.5, so.unit_length(k.double().reshape(n, G, D)),
                                        v.double().reshape(n, H, V), so.sigma(b.double()), decay).reshape(n, H * V))
    state = torch.full((3, H * D * V), -3.0, device=DEV)

    def run(members, counts, starts):
        cat = lambda xs: torch.cat([xs[b][s:s + c] for b, c, s in zip(members, counts, starts)]).to(dtype).to(DEV)
        _, qs = batch_layout(counts)
        return _ops().delta_rule_scan(cat(qs_), cat(ks_), cat(vs_), cat(bs_), cat(as_), a_log.to(DEV), dt.to(DEV), D ** -0.5, state,
                                      i32([slots[b] for b in members]), qs, i32(starts), H, G, D, V)

    for got, w in zip(scan_steps(cuts, lens, run), want):
        assert nerr(got, w) < 2e-5


@pytest.mark.parametrize("kind,D", [("gla", 48), ("gla", 128), ("gla", 200), ("delta", 64), ("delta", 128), ("delta", 256)])
def test_both_splits_of_the_state_over_lanes_give_the_same_bits(kind, D):
    """A step of few CTAs spreads the rows of a column over more lanes than a step of many; a request's numbers must not depend on
    which one served it.  One 70-token portion after a 3-token one, outputs and carried state compared bit for bit."""
    H, G, V, n = 2, 1, 24, 73
    g = torch.Generator().manual_seed(D)
    outs = []
    q, k = (rnd(g, n, (H if kind == "gla" else G) * D).to(torch.bfloat16).to(DEV) for _ in range(2))
    v, z = rnd(g, n, H * V).to(torch.bfloat16).to(DEV), rnd(g, n, H * D, scale=2.0).to(torch.bfloat16).to(DEV)
    bp, ap = rnd(g, n, H).to(torch.bfloat16).to(DEV), rnd(g, n, H).to(torch.bfloat16).to(DEV)
    zb, al, dt = rnd(g, H * D, shift=2.0).to(DEV), rnd(g, H, scale=0.5, shift=-1.0).to(DEV), rnd(g, H, scale=0.5).to(DEV)
    for flags in (0, 16):
        _ops().debug_flags(flags)
        state = torch.full((1, H * D * V), 4.0, device=DEV)
        got = []
        for lo, hi in ((0, 3), (3, n)):
            sl = slice(lo, hi)
            if kind == "gla":
                got.append(_ops().gla_scan(q[sl], k[sl], v[sl], z[sl], zb, 6.0, D ** -0.5, state, i32([0]), i32([0, hi - lo]), i32([lo]), H, D, V))
            else:
                got.append(_ops().delta_rule_scan(q[sl], k[sl], v[sl], bp[sl], ap[sl], al, dt, D ** -0.5, state, i32([0]), i32([0, hi - lo]),
                                                  i32([lo]), H, G, D, V))
        outs.append((torch.cat(got), state.clone()))
    assert torch.isfinite(outs[0][0]).all()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_a_write_far_back_is_still_read():
    """One key direction is written once at the start with a large value and never touched again (all later keys are orthogonal
    to it, no decay): a query along it 300 tokens later reads exactly that value — in one portion and token by token."""
    H, G, D, V, n = 1, 1, 16, 8, 300
    q, k, v = torch.zeros(n, D), torch.zeros(n, D), torch.zeros(n, V)
    k[0, 0], v[0] = 1.0, torch.arange(1, V + 1).float()
    g = torch.Generator().manual_seed(5)
    k[1:, 1:] = rnd(g, n - 1, D - 1)
    v[1:] = rnd(g, n - 1, V)
    q[:, 1:] = rnd(g, n, D - 1) * 1e-3
    q[n - 1] = 0
    q[n - 1, 0] = 1.0
    b, a = torch.full((n, H), 30.0), torch.full((n, H), -30.0)       # write strength 1, decay exp(-exp(a_log) softplus(-30)) = 1
    a_log, dt = torch.zeros(H), torch.zeros(H)
    for cuts in ([n], [1] * n, [7, 2] + [1] * 50 + [n - 59]):
        state = torch.zeros((1, H * D * V), device=DEV)
        done, last = 0, None
        for c in cuts:
            sl = slice(done, done + c)
            last = _ops().delta_rule_scan(q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), b[sl].to(DEV), a[sl].to(DEV), a_log.to(DEV), dt.to(DEV),
                                          1.0, state, i32([0]), i32([0, c]), i32([done]), H, G, D, V, unit_eps=0.0)
            done += c
        assert torch.allclose(last[-1].cpu(), v[0], atol=1e-4), cuts


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,V", [(2, 24), (5, 64), (1, 7), (12, 130)])
def test_head_norm_and_gate(dtype, H, V):
    g = torch.Generator().manual_seed(H + V)
    o, w, gate = rnd(g, 9, H * V, scale=3.0), rnd(g, V, shift=1.0), rnd(g, 9, H * V)
    want = (so.rms_norm(o.double().reshape(9, H, V), w.double(), 1e-5).reshape(9, H * V)) * so.silu(gate.double())
    got = _ops().headnorm_gate(o.to(DEV), w.to(DEV), gate.to(dtype).to(DEV), H, V, 1e-5, dtype)
    assert nerr(got, want) < tol(dtype, 1e-6, 5e-3)


# ------------------------------------------------------------------------------------------------
# rotary sigmoid attention with rotated values
# ------------------------------------------------------------------------------------------------
def paged(n_tokens, bs, n_seqs, g, extra=3):
    """Shuffled pages for sequences of n_tokens[b] tokens: block tables [B, max] and per-token cache rows."""
    need = [-(-n // bs) for n in n_tokens]
    perm = torch.randperm(sum(need) + extra, generator=g).tolist()
    tables, at = [], 0
    for k in need:
        tables.append(perm[at:at + k])
        at += k
    mb = max(need)
    bt = torch.tensor([t + [0] * (mb - len(t)) for t in tables], dtype=torch.int32)
    rows = [[tables[b][p // bs] * bs + p % bs for p in range(n_tokens[b])] for b in range(n_seqs)]
    return bt, rows, (sum(need) + extra) * bs


def plain_rotary_sigmoid(q, k, v, qn, kn, pb, f_qk, f_v, layout, scale, H, G, D, V, eps):
    n = q.shape[0]
    pos = list(range(n))
    qh = so.rotate(so.rms_norm(q.double().reshape(n, H, D), qn.double(), eps), pos, f_qk, layout)
    kh = so.rotate(so.rms_norm(k.double().reshape(n, G, D), kn.double(), eps), pos, f_qk, layout)
    vh = so.rotate(v.double().reshape(n, G, V), pos, f_v, layout)
    out = torch.zeros(n, H, V, dtype=F64)
    for i in range(n):
        for h in range(H):
            w = so.sigma((kh[:i + 1, h // (H // G)] @ qh[i, h]) * scale + pb[h].double())
            out[i, h] = w @ vh[:i + 1, h // (H // G)]
    return so.rotate(out, pos, f_v, layout, sign=-1.0).reshape(n, H * V)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("H,G,D,V,dims,layout,scaling", [(4, 2, 16, 24, 8, "interleaved", True), (8, 2, 64, 64, 24, "interleaved", True),
                                                          (3, 3, 10, 6, 10, "halves", False), (2, 1, 32, 16, 12, "halves", True),
                                                          (2, 2, 64, 64, 64, "interleaved", False)])
def test_rotary_sigmoid_attention_on_a_mixed_batch(dtype, general, H, G, D, V, dims, layout, scaling):
    """A prompt portion that continues a cached context, a whole prompt and a single decoded token in one step, on shuffled pages."""
    ops = _ops()
    ops.debug_flags(2 if general else 0)
    g = torch.Generator().manual_seed(H * 100 + D + dims)
    bs, eps, scale, base = 8, 1e-5, 0.3, 3000.0
    sc = dict(factor=4.0, low=1.0, high=4.0, original=32) if scaling else None
    f_qk, f_v = so.rotary_frequencies(dims, base, sc), so.rotary_frequencies(V, base, None)
    lens, starts = [53, 21, 40], [30, 0, 39]          # tokens in total, tokens already cached
    N = H * D + G * D + G * V
    proj = [rnd(g, n, N) for n in lens]
    qn, kn, pb = rnd(g, D, shift=1.0, scale=0.2), rnd(g, D, shift=1.0, scale=0.2), rnd(g, H, shift=-1.0)
    bt, rows, n_rows = paged(lens, bs, 3, g)
    kc = torch.full((n_rows, G, D), 50.0, dtype=dtype, device=DEV)
    vc = torch.full((n_rows, G, V), 50.0, dtype=dtype, device=DEV)
    il = layout == "interleaved"
    fq, fv = f_qk.float().to(DEV), f_v.float().to(DEV)

    def step(members, spans):
        x = torch.cat([proj[b][lo:hi] for b, (lo, hi) in zip(members, spans)]).to(dtype).to(DEV)
        pos = torch.tensor([p for lo, hi in spans for p in range(lo, hi)], dtype=torch.int64, device=DEV)
        slot = torch.tensor([rows[b][p] for b, (lo, hi) in zip(members, spans) for p in range(lo, hi)], dtype=torch.int64, device=DEV)
        q = ops.qkv_headnorm_rope_cache(x, 0, H * D, H * D + G * D, qn.to(DEV), kn.to(DEV), fq, fv, il, pos, slot, kc, vc, H, G, D, V, eps)
        tseq, qs = batch_layout([hi - lo for lo, hi in spans])
        out = ops.sigmoid_attention_paged(q, kc, vc, pos, tseq, bt[members].contiguous().to(DEV), None, pb.to(DEV), None,
                                          H, G, D, V, bs, scale, 0.0, max(hi - lo for lo, hi in spans), query_start=qs,
                                          max_seq_len=max(hi for _, hi in spans))
        return ops.rotate_heads(out, pos, fv, H, V, il, -1.0)

    step([0, 2], [(0, starts[0]), (0, starts[2])])                       # contexts
    got = step([0, 1, 2], [(starts[0], lens[0]), (0, lens[1]), (starts[2], lens[2])])
    at = 0
    for b in range(3):
        want = plain_rotary_sigmoid(proj[b][:, :H * D], proj[b][:, H * D:H * D + G * D], proj[b][:, H * D + G * D:], qn, kn, pb, f_qk, f_v, layout,
                                    scale, H, G, D, V, eps)[starts[b]:]
        assert nerr(got[at:at + want.shape[0]], want) < tol(dtype, 2e-5, 2e-2), b
        at += want.shape[0]


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 32, 32), (6, 3, 64, 32), (2, 1, 128, 128), (20, 1, 16, 48)])
def test_sigmoid_attention_of_independent_heads_over_long_contexts(H, G, D, V):
    """bfloat16 heads that do not talk to each other run on key tiles: a 700-token portion that continues a 300-token context (many
    query tiles, the diagonal inside a tile), a whole 130-token prompt, and single tokens after 1500 and 70 cached ones (keys split
    over several CTAs and merged; more heads per key/value head than a tile has rows), on shuffled pages, against plain sums."""
    ops = _ops()
    g = torch.Generator().manual_seed(H * 10 + D)
    bs, scale = 16, D ** -0.5
    spans = [(300, 1000), (0, 130), (1500, 1501), (70, 71)]                 # tokens of the step: positions lo .. hi - 1
    lens = [hi for _, hi in spans]
    bt, rows, n_rows = paged(lens, bs, len(lens), g)
    ks = [bf(rnd(g, n, G, D)) for n in lens]
    vs = [bf(rnd(g, n, G, V)) for n in lens]
    qs_ = [bf(rnd(g, hi - lo, H, D, scale=2.0)) for lo, hi in spans]
    pb = rnd(g, H, shift=-3.0)
    kc = torch.zeros((n_rows, G, D), dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros((n_rows, G, V), dtype=torch.bfloat16, device=DEV)
    for b in range(len(lens)):
        idx = torch.tensor(rows[b], device=DEV)
        kc[idx], vc[idx] = ks[b].to(torch.bfloat16).to(DEV), vs[b].to(torch.bfloat16).to(DEV)
    q = torch.cat(qs_).reshape(-1, H * D).to(torch.bfloat16).to(DEV)
    pos = torch.cat([torch.arange(lo, hi) for lo, hi in spans]).to(DEV)
    tseq, qs = batch_layout([hi - lo for lo, hi in spans])
    outs = []
    for flags in (0, 2):
        ops.debug_flags(flags)
        outs.append(ops.sigmoid_attention_paged(q, kc, vc, pos, tseq, bt.to(DEV), None, pb.to(DEV), None, H, G, D, V, bs, scale, 0.0,
                                                max(hi - lo for lo, hi in spans), query_start=qs, max_seq_len=max(lens)))
    at = 0
    for b, (lo, hi) in enumerate(spans):
        k, v, qq = ks[b].double(), vs[b].double(), qs_[b].double()
        kh, vh = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)          # [n, H, .]
        sc = torch.einsum("ihd,jhd->hij", qq, kh) * scale + pb.double()[:, None, None]
        vis = torch.arange(hi)[None, :] <= torch.arange(lo, hi)[:, None]
        w = so.sigma(sc) * vis[None]
        want = torch.einsum("hij,jhv->ihv", w, vh).reshape(hi - lo, H * V)
        for got in outs:
            assert nerr(got[at:at + hi - lo], want) < 1e-2, (b, nerr(got[at:at + hi - lo], want))
        at += hi - lo


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("far", [15, 16, 17, 400, 1023])
def test_one_loud_key_far_back_carries_its_value_home(far, decode):
    """Every key but one is muted by the per-head bias; the loud one lies `far` tokens back (inside a page, on its border, far away).
    The head's sum, turned back by the query's position, is that key's value turned by the distance alone."""
    ops = _ops()
    H = G = 1
    D, V, bs, n = 16, 8, 16, far + 1
    g = torch.Generator().manual_seed(far)
    base = 100.0
    f = so.rotary_frequencies(V, base, None)
    k, v, q = rnd(g, n, D, scale=0.01), rnd(g, n, V), torch.zeros(n, D)
    k[0] = 0
    k[0, 0] = 8.0
    q[n - 1, 0] = 8.0
    proj = torch.cat([q, k, v], 1)
    bt, rows, n_rows = paged([n], bs, 1, g)
    kc, vc = torch.zeros((n_rows, G, D), device=DEV), torch.zeros((n_rows, G, V), device=DEV)
    pb = torch.tensor([-40.0])          # sigmoid(64 - 40) = 1 for the loud pair, sigmoid(-40) = 0 for the rest
    fv = f.float().to(DEV)
    pos = torch.arange(n, dtype=torch.int64, device=DEV)
    slot = torch.tensor(rows[0], dtype=torch.int64, device=DEV)
    spans = [(0, n)] if not decode else [(0, n - 1), (n - 1, n)]
    for lo, hi in spans:
        qd = ops.qkv_headnorm_rope_cache(proj[lo:hi].to(DEV), 0, D, 2 * D, None, None, None, fv, True, pos[lo:hi], slot[lo:hi], kc, vc, H, G, D, V, 1e-5)
        out = ops.sigmoid_attention_paged(qd, kc, vc, pos[lo:hi], i32([0] * (hi - lo)), bt.to(DEV), None, pb.to(DEV), None,
                                          H, G, D, V, bs, 1.0, 0.0, hi - lo, query_start=i32([0, hi - lo]), max_seq_len=hi)
        out = ops.rotate_heads(out, pos[lo:hi], fv, H, V, True, -1.0)
    want = so.rotate(v[0:1].double().reshape(1, 1, V), [-(n - 1)], f, "interleaved").reshape(V)
    assert nerr(out[-1], want) < 2e-4


# ------------------------------------------------------------------------------------------------
# latent attention with a rotated key part
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,D,Rd,V,Rq,Rk,dims,layout", [(3, 16, 8, 16, 24, 32, 8, "halves"), (6, 64, 32, 64, 72, 128, 32, "halves"),
                                                       (2, 10, 6, 12, 9, 14, 4, "interleaved"), (4, 32, 64, 48, 40, 128, 64, "halves")])
def test_latent_attention_with_a_rotated_key_part(dtype, H, D, Rd, V, Rq, Rk, dims, layout):
    ops = _ops()
    g = torch.Generator().manual_seed(H * 10 + Rd)
    bs, eps, scale = 8, 1e-5, 0.17
    lens, starts = [45, 20, 33], [20, 0, 32]
    m = dict(heads=H, dim=D, rot_dim=Rd, vdim=V, q_rank=Rq, kv_rank=Rk, scale=scale, rot=dict(base=700.0, dims=dims, layout=layout))
    W = 24
    P = {"dq": rnd(g, Rq, W, scale=0.3), "dq.norm": rnd(g, Rq, shift=1.0, scale=0.1), "uq": rnd(g, H * (D + Rd), Rq, scale=0.4),
         "dkv": rnd(g, Rk + Rd, W, scale=0.4), "dkv.norm": rnd(g, Rk, shift=1.0, scale=0.1), "uk": rnd(g, H * D, Rk, scale=0.3),
         "uv": rnd(g, H * V, Rk, scale=0.2), "o": torch.eye(H * V)}
    hs = [rnd(g, n, W) for n in lens]
    freq = so.rotary_frequencies(dims, 700.0, None).float().to(DEV)
    bt, rows, n_rows = paged(lens, bs, 3, g)
    cache = torch.full((n_rows, Rk + Rd), 30.0, dtype=dtype, device=DEV)
    w_in = torch.cat([P["dq"], P["dkv"]]).to(dtype).to(DEV)
    il = layout == "interleaved"

    def step(members, spans):
        h = torch.cat([hs[b][lo:hi] for b, (lo, hi) in zip(members, spans)]).to(dtype).to(DEV)
        pos = torch.tensor([p for lo, hi in spans for p in range(lo, hi)], dtype=torch.int64, device=DEV)
        slot = torch.tensor([rows[b][p] for b, (lo, hi) in zip(members, spans) for p in range(lo, hi)], dtype=torch.int64, device=DEV)
        proj = ops.linear(h, w_in)
        cq = ops.latent_norm_rope_cache(proj, P["dq.norm"].to(DEV), P["dkv.norm"].to(DEV), freq, il, pos, slot, cache, Rq, Rk, Rd, eps)
        q = ops.linear(cq, P["uq"].to(dtype).to(DEV))
        qlat = ops.latent_query_absorb_rope(q, P["uk"].to(dtype).to(DEV), freq, il, pos, H, D, Rd, Rk)
        tseq, qs = batch_layout([hi - lo for lo, hi in spans])
        olat = ops.latent_attention_paged(qlat.reshape(qlat.shape[0], -1), cache, pos, tseq, bt[members].contiguous().to(DEV), None, H, Rk + Rd, bs,
                                          0, scale, max(hi - lo for lo, hi in spans), query_start=qs, max_seq_len=max(hi for _, hi in spans))
        return ops.latent_expand_values(olat.reshape(-1, H, Rk + Rd), P["uv"].to(dtype).to(DEV), H, V, Rk, dtype)

    step([0, 2], [(0, starts[0]), (0, starts[2])])
    got = step([0, 1, 2], [(starts[0], lens[0]), (0, lens[1]), (starts[2], lens[2])])
    at = 0
    for b in range(3):
        want = so.latent_attention(hs[b].double(), {k: v.double() for k, v in P.items()}, "", m, eps, list(range(lens[b])))[starts[b]:]
        assert nerr(got[at:at + want.shape[0]], want) < tol(dtype, 2e-5, 3e-2), b
        at += want.shape[0]


# ------------------------------------------------------------------------------------------------
# the model through the engine
# ------------------------------------------------------------------------------------------------
def make_engine(tmp_path, cfg, weights, dtype, max_tokens=512, block_size=16, live=4, budget=2048):
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.engine import Engine
    tmp_path.mkdir(exist_ok=True)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return Engine.from_model_dir(tmp_path, dtype=dtype, device=DEV, max_tokens=max_tokens, block_size=block_size,
                                 max_live_requests=live, max_num_batched_tokens=budget)


VARIANTS = {
    "base": dict(),
    "no_loop_other_order": dict(kinds=("parallel", "latent_attention", "gla"), loop=None, mlps=[True, False, True]),
    "loop_at_the_end": dict(kinds=("latent_attention", "gla", "parallel"), loop=(1, 3, 3), taps=2),
    "one_tap_whole_loop": dict(kinds=("gla", "parallel"), loop=(0, 2, 2), taps=1, right=dict(conv=1)),
    "odd_sizes": dict(width=50, vocab=37, taps=4, ff=22, kinds=("gla", "parallel", "latent_attention"), loop=(2, 3, 2),
                      gla=dict(heads=3, dim=10, vdim=14, tau=3.0),
                      latent=dict(heads=5, dim=12, rot_dim=6, vdim=10, q_rank=20, kv_rank=18, scale=0.3, rot=dict(base=777.0, dims=6)),
                      left=dict(heads=6, kv_heads=3, dim=12, vdim=10, scale=0.4, rot=dict(base=999.0, dims=4)),
                      right=dict(heads=6, kv_heads=2, dim=8, vdim=12, conv=2)),
    "wide_heads": dict(width=64, kinds=("parallel", "gla", "latent_attention"), loop=(0, 1, 2), gla=dict(heads=2, dim=80, vdim=64, tau=16.0),
                       latent=dict(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=48, kv_rank=96, scale=0.1, rot=dict(base=1e5, dims=32)),
                       left=dict(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.125,
                                 rot=dict(base=1e6, dims=32, scaling=dict(factor=8.0, low=1.0, high=4.0, original=128))),
                       right=dict(heads=4, kv_heads=4, dim=64, vdim=32, conv=4)),
    "halves_layout_whole_head": dict(kinds=("parallel", "gla"), loop=(1, 2, 2), left=dict(heads=2, kv_heads=2, dim=16, vdim=16, scale=0.25,
                                                                                         rot=dict(base=500.0, dims=16, layout="halves"))),
}


def build(name, seed=0):
    g = torch.Generator().manual_seed(500 + seed)
    cfg = so.random_config(**VARIANTS[name])
    return cfg, so.random_weights(cfg, g), g


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_matches_the_plain_model(tmp_path, dtype, name):
    cfg, w, g = build(name)
    toks = torch.randint(0, cfg["vocab"], (83,), generator=g).tolist()
    want, layers = so.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, dtype)
    out = eng.step_forced([("a", toks, list(range(len(toks))))], want_residual_trace=True)
    assert out.residual_trace.shape[0] == len(layers)
    for i in range(len(layers)):
        assert nerr(out.residual_trace[i], layers[i]) < tol(dtype, 5e-6, 3e-2), i
    assert nerr(out.logits, want) < tol(dtype, 1e-5, 5e-2)


@pytest.mark.parametrize("name", ["base", "odd_sizes", "one_tap_whole_loop", "wide_heads"])
def test_decoding_token_by_token_equals_the_whole_prompt(tmp_path, name):
    """70 single-token steps on pages of four tokens: every page border and the first tokens of the sequence, where the tap filters
    and the short filters still look before its start."""
    cfg, w, g = build(name, 1)
    toks = torch.randint(0, cfg["vocab"], (70,), generator=g).tolist()
    want, _ = so.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=128, block_size=4)
    got = [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks]
    assert nerr(torch.cat(got), want) < 1e-5


def test_long_decoding(tmp_path):
    """A short prompt and 400 decoded tokens: the states are carried for hundreds of steps, the caches grow over many pages."""
    cfg, w, g = build("base", 2)
    toks = torch.randint(0, cfg["vocab"], (420,), generator=g).tolist()
    want, _ = so.forward(cfg, w, toks)
    for dtype in BOTH:
        eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=512, block_size=16)
        eng.step_forced([("a", toks[:20], [])])
        got = [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks[20:]]
        assert nerr(torch.cat(got), want[20:]) < tol(dtype, 2e-5, 6e-2)
        eng.finish_request("a")


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", ["base", "wide_heads", "odd_sizes"])
@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [40, 2, 17, 1, 1, 2, 64, 5], [1, 130, 1, 1], [19, 20, 21]])
def test_portions_of_any_size_equal_the_whole_prompt(tmp_path, dtype, name, sizes):
    cfg, w, g = build(name, 3)
    toks = torch.randint(0, cfg["vocab"], (sum(sizes),), generator=g).tolist()
    want, _ = so.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=256, block_size=8)
    got, at = [], 0
    for n in sizes:
        got.append(eng.step_forced([("a", toks[at:at + n], list(range(n)))]).logits.clone())
        at += n
    assert nerr(torch.cat(got), want) < tol(dtype, 1e-5, 5e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", ["base", "wide_heads"])
def test_mixed_batches_with_reused_pages_and_slots_equal_each_request_alone(tmp_path, dtype, name):
    """Six requests through an engine with three state slots and a small page pool: portions beside single tokens, requests that end
    and hand their pages and slot to the next one.  Every wanted row equals the request run alone by the plain model."""
    cfg, w, g = build(name, 4)
    lens = [37, 5, 61, 18, 2, 44]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    want = [so.forward(cfg, w, t)[0] for t in reqs]
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=160, block_size=8, live=3)
    plan = [[(0, 20), (1, 2)], [(0, 1), (1, 3), (2, 16)], [(0, 16), (2, 1)], [(2, 30), (3, 2)], [(2, 14), (3, 1), (4, 2)], [(3, 15), (5, 40)],
            [(5, 1)], [(5, 3)]]
    done = [0] * 6
    for step in plan:
        entries, end = [], []
        for r, n in step:
            entries.append((f"r{r}", reqs[r][done[r]:done[r] + n], list(range(n))))
            done[r] += n
            if done[r] == lens[r]:
                end.append(f"r{r}")
        out = eng.step_forced(entries, end)
        at = 0
        for r, n in step:
            assert nerr(out.logits[at:at + n], want[r][done[r] - n:done[r]]) < tol(dtype, 1e-5, 6e-2), (step, r)
            at += n
    assert done == lens and eng.cache.live == 0 and eng.cache.state_slots.num_free == 3


def test_batch_members_do_not_change_each_other(tmp_path):
    cfg, w, g = build("base", 5)
    a, b = (torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (33, 50))
    eng = make_engine(tmp_path, cfg, w, torch.float32)
    alone = eng.step_forced([("a", a, [32])], ["a"]).logits.clone()
    both = eng.step_forced([("b", b, [49]), ("a", a, [32])], ["a", "b"]).logits.clone()
    assert nerr(both[1], alone[0]) < 1e-6


def test_the_first_token_is_felt_far_away_through_every_mixer(tmp_path):
    """Changing token 0 changes the logits 200 tokens later (states and caches reach back) exactly as the plain model says, whether
    the 200 tokens came as one prompt or were decoded one by one."""
    for kinds in (("gla",), ("latent_attention",), ("parallel",)):
        cfg = so.random_config(kinds=kinds, loop=(0, 1, 2))
        g = torch.Generator().manual_seed(11)
        w = so.random_weights(cfg, g)
        t1 = torch.randint(0, cfg["vocab"], (201,), generator=g).tolist()
        t2 = [(t1[0] + 1) % cfg["vocab"]] + t1[1:]
        eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=512)
        res = {}
        for name, t in (("one", t1), ("two", t2)):
            res[name] = eng.step_forced([("a", t, [200])], ["a"]).logits[0].clone()
            assert nerr(res[name], so.forward(cfg, w, t)[0][200]) < 1e-5, kinds
            eng.step_forced([("b", t[:3], [])])
            for tok in t[3:]:
                last = eng.step_forced([("b", [tok], [0])]).logits[0].clone()
            eng.finish_request("b")
            assert nerr(last, res[name]) < 1e-5, kinds
        assert nerr(res["one"], res["two"]) > 1e-4, kinds


def test_greedy_generation_through_the_scheduler(tmp_path):
    cfg, w, g = build("base", 6)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (19, 3, 41, 1)]
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=256, block_size=8, live=2, budget=16)
    got = eng.generate(prompts, max_new_tokens=6)
    assert eng.cache.live == 0 and eng.cache.blocks.num_free == eng.cache.blocks.capacity
    for p, out in zip(prompts, got):
        assert len(out) == 6
        t = list(p)
        for tok in out:
            lg = so.forward(cfg, w, t)[0][-1]
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) < 1e-3:
                break
            assert int(lg.argmax()) == tok
            t.append(tok)


def test_command_line_and_trace_replay(tmp_path, capsys, monkeypatch):
    import io
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.__main__ import main
    cfg, w, g = build("no_loop_other_order", 7)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    assert main(["generate", "--model", str(tmp_path), "--prompt-ids", "3,4,5,6", "--max-new-tokens", "2", "--dtype", "float32",
                 "--max-tokens", "128", "--max-live", "2"]) == 0
    line = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.startswith("{")][0]
    lg = so.forward(cfg, w, [3, 4, 5, 6])[0][-1]
    if float(torch.topk(lg, 2).values[0] - torch.topk(lg, 2).values[1]) > 1e-3:
        assert line["generated"][0] == int(lg.argmax())
    toks = [5, 9, 2, 30, 11, 7]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:4], "want": [1, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[4:5], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[5:], "want": [0]}, {"id": "b", "tokens": toks[:2], "want": [1]}], "end": ["a", "b"]}]
    monkeypatch.setattr("sys.stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out = tmp_path / "out"
    assert main(["trace", "--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert [x for x in capsys.readouterr().out.split("\n") if x.startswith("done")] == ["done 0", "done 1", "done 2"]
    want, _ = so.forward(cfg, w, toks)
    assert not (out / "1.f32").exists()
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1)
    assert nerr(a, want[[1, 3]]) < 1e-5 and nerr(b, torch.stack([want[5], want[1]])) < 1e-5
