"""Nemasun on the GPU against the plain implementation of tests/nemasun_oracle.py (float64): every mechanism alone,
then the model through the engine — whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches against each request alone, reused pages, keys far away, at page borders, just inside / outside the window
and the kept first tokens, decoding far past the window, other sizes, greedy generation through the scheduler."""
import json

import numpy as np
import pytest
import torch

import nemasun_oracle as no

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


def model_close(got, want, dtype, f32=1e-5):
    """float32: the sharp comparison over all rows.  bfloat16: rounding the router's input can flip the choice between two
    outputs whose corrected scores nearly tie, which changes that token's row by far more than rounding does elsewhere, so
    the bound is on the typical row (median of the per-row errors) with a loose one on the whole."""
    if dtype == torch.float32:
        return nerr(got, want) < f32
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    rows = ((got - want) ** 2).mean(-1).sqrt() / (want ** 2).mean(-1).sqrt().clamp_min(1e-30)
    return float(rows.median()) < 8e-2 and nerr(got, want) < 0.5


def bf(t):
    return t.to(torch.bfloat16).float()


# ------------------------------------------------------------------------------------------------
# residual lanes
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("lanes", [1, 3, 4])
def test_scaled_embedding_fills_every_lane(dtype, lanes):
    g = torch.Generator().manual_seed(0)
    table = bf(torch.randn(20, 34, generator=g))
    toks = torch.tensor([3, 19, 0, 7, 7], dtype=torch.int32)
    x = _ops().embed_scaled_lanes(toks.to(DEV), table.to(dtype).to(DEV), 2.5, lanes)
    want = no.embed(toks.long(), table.double(), 2.5)
    assert x.shape == (5, lanes, 34)
    for s in range(lanes):
        assert torch.equal(x[:, s].cpu().double(), want)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("lanes,width", [(1, 40), (2, 50), (3, 64), (5, 33)])
def test_lanes_read_then_norm(dtype, lanes, width):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, lanes, width, generator=g) * 3
    w_in, w = torch.randn(lanes, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
    lanes_list = [x[:, s].double() for s in range(lanes)]
    h, u = _ops().lanes_read_norm(x.to(DEV), w_in.to(DEV), w.to(DEV), 0.0, 1e-5, dtype, want_sum=True)
    want_u = no.lanes_read(lanes_list, w_in.double())
    assert nerr(u, want_u) < 1e-6 and nerr(h, no.rms_norm(want_u, w.double(), 1e-5)) < tol(dtype, 2e-6, 4e-3)
    # the model's last read: a plain sum of the lanes, of the wanted rows only
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    h, _ = _ops().lanes_read_norm(x.to(DEV), None, w.to(DEV), 0.0, 1e-5, dtype, rows=rows.to(DEV))
    assert nerr(h, no.rms_norm(sum(lanes_list)[rows.long()], w.double(), 1e-5)) < tol(dtype, 2e-6, 4e-3)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("lanes,width", [(1, 40), (2, 50), (3, 64), (4, 33)])
def test_lanes_write_with_the_next_read(dtype, lanes, width):
    """The mix matrix is indexed [from, to]: a matrix that is far from symmetric tells the two readings apart."""
    g = torch.Generator().manual_seed(2)
    T = 7
    x0 = torch.randn(T, lanes, width, generator=g) * 2
    y = torch.randn(T, width, generator=g).to(dtype)
    mix = torch.triu(torch.randn(lanes, lanes, generator=g)) + torch.eye(lanes)
    w_out, w_in, wn, bias = torch.randn(lanes, generator=g), torch.randn(lanes, generator=g), 1 + 0.2 * torch.randn(width, generator=g), \
        torch.randn(width, generator=g)
    x = x0.clone().to(DEV)
    h, ls = _ops().lanes_update_norm(x, y.to(DEV), mix.to(DEV), w_out.to(DEV), dtype, y_bias=bias.to(DEV), w_in_next=w_in.to(DEV),
                                     w_next=wn.to(DEV), want_lane_sum=True)
    old = [x0[:, s].double() for s in range(lanes)]
    new = no.lanes_write(old, mix.double(), w_out.double(), y.double() + bias.double())
    for s in range(lanes):
        assert nerr(x[:, s], new[s]) < 1e-6, s
    assert nerr(ls, sum(new)) < 1e-6
    assert nerr(h, no.rms_norm(no.lanes_read(new, w_in.double()), wn.double(), 1e-5)) < tol(dtype, 2e-6, 4e-3)
    if lanes > 1:
        wrong = no.lanes_write(old, mix.double().T, w_out.double(), y.double() + bias.double())
        assert nerr(x[:, 0], wrong[0]) > 1e-2
    # no following read, no bias
    x = x0.clone().to(DEV)
    h, ls = _ops().lanes_update_norm(x, y.to(DEV), mix.to(DEV), w_out.to(DEV), dtype)
    assert h is None and ls is None and nerr(x[:, lanes - 1], no.lanes_write(old, mix.double(), w_out.double(), y.double())[lanes - 1]) < 1e-6


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,dim,vdim,same", [(4, 2, 8, 8, True), (6, 1, 16, 16, True), (3, 3, 10, 6, False), (2, 1, 64, 64, True)])
def test_per_head_norms_and_cache_write(dtype, H, G, dim, vdim, same):
    g = torch.Generator().manual_seed(3)
    T, bs, eps = 9, 4, 1e-5
    extra = 5
    ncol = H * dim + G * dim + (0 if same else G * vdim) + extra
    proj = bf(torch.randn(T, ncol, generator=g) * 2).to(dtype)
    qw, kw = 1 + 0.3 * torch.randn(dim, generator=g), 1 + 0.3 * torch.randn(dim, generator=g)
    slots = torch.tensor([5, 0, 31, -1, 7, 8, 9, 30, 2], dtype=torch.int64)
    kc = torch.full((32, G, dim), 7.0).to(dtype).to(DEV)
    vc = torch.full((32, G, vdim), 7.0).to(dtype).to(DEV)
    k_off = H * dim
    v_off = k_off if same else k_off + G * dim
    q = _ops().qk_headnorm_cache(proj.to(DEV), 0, k_off, v_off, qw.to(DEV), kw.to(DEV), 0.0, slots.to(DEV), kc, vc, H, G, dim, vdim, eps)
    p = proj.double()
    want_q = no.rms_norm(p[:, :k_off].reshape(T, H, dim), qw.double(), eps).reshape(T, H * dim)
    raw_k = p[:, k_off:k_off + G * dim].reshape(T, G, dim)
    want_k = no.rms_norm(raw_k, kw.double(), eps)
    want_v = raw_k if same else p[:, v_off:v_off + G * vdim].reshape(T, G, vdim)
    assert nerr(q, want_q) < tol(dtype, 2e-6, 4e-3)
    for t in range(T):
        if slots[t] < 0:
            continue
        assert nerr(kc[slots[t]], want_k[t]) < tol(dtype, 2e-6, 4e-3)
        assert torch.equal(vc[slots[t]].cpu().double(), want_v[t])          # values are copied, not normed
    untouched = [s for s in range(32) if s not in slots.tolist()]
    assert bool((kc[untouched] == 7).all()) and bool((vc[untouched] == 7).all())


def attention_plain(q, k, v, table, scale, window, keep, i, rep):
    """q [H, dim] of position i; k, v [L, G, .] of positions 0 .. L - 1; table [distances, H] or None -> [H, vdim]"""
    H = q.shape[0]
    js = torch.tensor([j for j in range(i + 1) if no.visible(i, j, window or (1 << 60), keep)])
    out = []
    for h in range(H):
        s = (k[js, h // rep] @ q[h]) * scale
        if table is not None:
            s = s + table[torch.clamp(i - js, max=table.shape[0] - 1), h]
        out.append(torch.softmax(s, 0) @ v[js, h // rep])
    return torch.stack(out)


def paged_kv(g, seqs, G, dim, vdim, bs, dtype, extra_pages=3):
    """seqs: (context, portion) per sequence -> device tensors of a mixed batch over a shuffled page pool full of garbage."""
    pages = sum(-(-(c + n) // bs) for c, n in seqs) + extra_pages
    order = torch.randperm(pages, generator=g).tolist()
    kc = bf(torch.randn(pages * bs, G, dim, generator=g) * 50)          # what other requests left behind
    vc = bf(torch.randn(pages * bs, G, vdim, generator=g) * 50)
    maxb = max(-(-(c + n) // bs) for c, n in seqs)
    bt = torch.zeros(len(seqs), maxb, dtype=torch.int32)
    ks, vs, pos, tseq = [], [], [], []
    for b, (ctx, n) in enumerate(seqs):
        L = ctx + n
        k, v = bf(torch.randn(L, G, dim, generator=g)), bf(torch.randn(L, G, vdim, generator=g))
        for i in range(-(-L // bs)):
            bt[b, i] = order.pop()
        for j in range(L):
            kc[int(bt[b, j // bs]) * bs + j % bs], vc[int(bt[b, j // bs]) * bs + j % bs] = k[j], v[j]
        ks.append(k)
        vs.append(v)
        pos += list(range(ctx, L))
        tseq += [b] * n
    return (kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), bt.to(DEV), torch.tensor(pos, dtype=torch.int64, device=DEV),
            torch.tensor(tseq, dtype=torch.int32, device=DEV), ks, vs)


def attention_case(g, dtype, seqs, H, G, dim, vdim, window, keep, rows, gate, general, bs=8, scale=0.35, long_min_q=0):
    kc, vc, bt, pos, tseq, ks, vs = paged_kv(g, seqs, G, dim, vdim, bs, dtype)
    T = pos.numel()
    q = bf(torch.randn(T, H * dim, generator=g))
    table = torch.randn(rows, H, generator=g) * 1.5 if rows else None
    gt = bf(torch.randn(T, H * vdim + 8, generator=g)) if gate else None
    if general:
        _ops().debug_flags(2)
    got = _ops().softmax_attention_paged(q.to(dtype).to(DEV), kc, vc, pos, tseq, bt, H, G, dim, vdim, bs, scale, window=window, keep_first=keep,
                                         dist_bias=table.to(DEV) if rows else None,
                                         gate=gt.to(dtype).to(DEV)[:, 8:] if gate else None, long_min_q=long_min_q)
    want, t = [], 0
    for b, (ctx, n) in enumerate(seqs):
        for i in range(ctx, ctx + n):
            o = attention_plain(q[t].double().reshape(H, dim), ks[b].double(), vs[b].double(), table.double() if rows else None, scale, window, keep,
                                i, H // G).reshape(-1)
            if gate:
                o = o * no.sigma(gt[t, 8:].double())
            want.append(o)
            t += 1
    return got, torch.stack(want)


SHAPES = [  # H, G, dim, vdim, window, keep, table rows, gate
    (4, 2, 8, 8, 13, 3, 10, True),
    (6, 1, 16, 16, 20, 0, 25, True),
    (3, 3, 10, 6, 0, 0, 0, False),
    (2, 1, 64, 64, 33, 5, 40, True),
    (8, 2, 32, 32, 70, 70, 90, False),        # more kept tokens than a key tile holds
    (5, 5, 16, 16, 1, 2, 4, True),            # a window of one: the token itself and the kept ones
    (32, 1, 16, 16, 9, 1, 7, True),           # more heads per key/value head than a tile has rows
    (2, 2, 128, 128, 100, 4, 12, True),
    (3, 1, 48, 48, 50, 2, 20, True),          # a head size between the tile sizes
    (4, 2, 96, 96, 0, 0, 3000, False),        # a table longer than the kernel keeps in shared memory
]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("H,G,dim,vdim,window,keep,rows,gate", SHAPES)
def test_attention_on_a_mixed_batch(dtype, general, H, G, dim, vdim, window, keep, rows, gate):
    """Portions with and without context, single tokens at several depths, one sequence that starts at 0."""
    g = torch.Generator().manual_seed(4)
    seqs = [(0, 37), (90, 1), (21, 70), (0, 1), (140, 3), (7, 1), (200, 1)]
    got, want = attention_case(g, dtype, seqs, H, G, dim, vdim, window, keep, rows, gate, general)
    assert nerr(got, want) < tol(dtype, 3e-6, 1.5e-2)


@pytest.mark.parametrize("H,G,dim,window,keep,rows,gate", [(4, 2, 64, 0, 0, 40, True), (2, 1, 128, 100, 5, 30, True), (4, 2, 64, 150, 70, 3000, False),
                                                        (3, 1, 128, 129, 200, 12, True), (2, 2, 64, 1, 3, 5, True)])
def test_long_portions_on_the_tensor_memory_kernel(H, G, dim, window, keep, rows, gate):
    """Portions of 128 tokens and more (bfloat16 heads of 64 / 128) run on gathered keys and values with the kept first tokens
    merged afterwards; shorter portions and single tokens of the same step run on the other kernels."""
    g = torch.Generator().manual_seed(12)
    seqs = [(0, 140), (90, 1), (77, 130), (0, 40), (200, 129), (5, 127)]
    got, want = attention_case(g, torch.bfloat16, seqs, H, G, dim, dim, window, keep, rows, gate, False, bs=16, scale=dim ** -0.5, long_min_q=128)
    t = 0
    for ctx, n in seqs:       # per sequence, so that a long one's error cannot hide among the others
        assert nerr(got[t:t + n], want[t:t + n]) < 1.5e-2, (ctx, n)
        t += n
    # only long sequences in the step
    got, want = attention_case(g, torch.bfloat16, [(0, 130), (64, 128)], H, G, dim, dim, window, keep, rows, gate, False, bs=16, scale=dim ** -0.5,
                               long_min_q=128)
    assert nerr(got, want) < 1.5e-2


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("window,keep", [(0, 0), (150, 7), (700, 100)])
@pytest.mark.parametrize("dim", [16, 64])
def test_attention_decoding_over_long_contexts(dtype, window, keep, dim):
    """Single tokens only (the key/value head's query heads are the tile's rows; few sequences: the keys are split over CTAs)."""
    g = torch.Generator().manual_seed(5)
    seqs = [(1500, 1), (3, 1), (777, 1)]
    got, want = attention_case(g, dtype, seqs, 4, 2, dim, dim, window, keep, 30, True, False, bs=16)
    assert nerr(got, want) < tol(dtype, 3e-6, 1.5e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("dim", [8, 64])
@pytest.mark.parametrize("decode", [False, True])
def test_one_loud_key_is_seen_just_inside_and_not_just_outside(dtype, dim, decode):
    """One key that the query matches far better than all others, placed at the window's last position, one before it,
    at the last kept token, just after the kept ones, at page borders, hundreds of tokens back, and at position 0: the
    output is that key's value when it is visible and has no trace of it when it is not."""
    g = torch.Generator().manual_seed(6)
    H, G, bs, window, keep, L = 2, 1, 8, 41, 5, 300
    p = L - 1
    places = {p - 40: True, p - 41: False, keep - 1: True, keep: False, 0: True, 256: False, 263: True, 264: True, p: True, p - 17: True, 100: False}
    for j, seen in places.items():
        seqs = [(p, 1)] if decode else [(p - 20, 21)]
        kc, vc, bt, pos, tseq, ks, vs = paged_kv(g, seqs, G, dim, dim, bs, dtype)
        q = bf(torch.randn(pos.numel(), H * dim, generator=g))
        k = ks[0]
        loud = bf(torch.randn(dim, generator=g))
        loud = loud / loud.norm() * 6
        slot = int(bt[0, j // bs]) * bs + j % bs
        kc[slot, 0] = loud.to(dtype)
        vc[slot, 0] = torch.full((dim,), 100.0).to(dtype)
        q[-1] = torch.cat([loud, loud]) * 6                     # both heads of the last token shout for it
        got = _ops().softmax_attention_paged(q.to(dtype).to(DEV), kc, vc, pos, tseq, bt, H, G, dim, dim, bs, 1.0, window=window, keep_first=keep)
        last = got[-1].float().cpu()
        if seen:
            assert float((last - 100.0).abs().max()) < 2.0, j
        else:
            assert float(last.abs().max()) < 20.0, j


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("decode", [False, True])
def test_the_bias_row_of_a_distance_decides(dtype, decode):
    """Equal keys everywhere, a table that is zero but for one distance: the weights pile on the key at that distance; beyond
    the table's last row every distance reads the last row."""
    H, G, dim, bs, L = 2, 1, 16, 8, 120
    p = L - 1
    for dist, rows in [(0, 50), (17, 50), (49, 50), (90, 50)]:
        g = torch.Generator().manual_seed(7)
        seqs = [(p, 1)] if decode else [(p - 9, 10)]
        kc, vc, bt, pos, tseq, ks, vs = paged_kv(g, seqs, G, dim, dim, bs, dtype)
        for j in range(L):
            slot = int(bt[0, j // bs]) * bs + j % bs
            kc[slot, 0] = 0
            vc[slot, 0] = float(j)
        table = torch.zeros(rows, H)
        table[min(dist, rows - 1), 1] = 30.0          # head 1 only
        q = bf(torch.randn(pos.numel(), H * dim, generator=g))
        got = _ops().softmax_attention_paged(q.to(dtype).to(DEV), kc, vc, pos, tseq, bt, H, G, dim, dim, bs, 1.0, dist_bias=table.to(DEV))
        last = got[-1].float().cpu().reshape(H, dim)
        assert abs(float(last[0, 0]) - p / 2) < 1.0                       # head 0: the plain mean of all positions
        if dist < rows - 1:
            assert abs(float(last[1, 0]) - (p - dist)) < 0.6, dist
        else:                                                                # the last row holds for every distance from rows - 1 on
            far = [p - d for d in range(rows - 1, L)]
            assert abs(float(last[1, 0]) - sum(far) / len(far)) < 1.0, dist


# ------------------------------------------------------------------------------------------------
# feed-forwards
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
def test_clamped_activation_with_biases(dtype):
    g = torch.Generator().manual_seed(8)
    ff = 24
    gu = bf(torch.randn(5, 2 * ff + 7, generator=g) * 3)
    bias = torch.randn(2 * ff, generator=g)
    for limit in (0.7, 0.0):
        got = _ops().glu_clamped_bias(gu.to(dtype).to(DEV), bias.to(DEV), ff, limit, 1.702, 1.0)
        a, b = gu.double()[:, :ff] + bias.double()[:ff], gu.double()[:, ff:2 * ff] + bias.double()[ff:]
        if limit > 0:
            a, b = torch.clamp(a, max=limit), torch.clamp(b, -limit, limit)
        assert nerr(got, a * no.sigma(1.702 * a) * (b + 1.0)) < tol(dtype, 2e-6, 5e-3)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,W,ff,limit", [(6, 64, 24, 0.9), (200, 64, 40, 0.5), (33, 128, 72, 0.0), (5, 40, 24, 1.5)])
def test_dense_feed_forward_from_its_operators(dtype, T, W, ff, limit):
    """Decode-sized bfloat16 steps run the activation in the projection's epilogue, everything else projection + activation
    kernel; both against the plain feed-forward, with and without biases."""
    g = torch.Generator().manual_seed(9)
    h = bf(torch.randn(T, W, generator=g))
    wg, wu, wd = bf(torch.randn(ff, W, generator=g) / 6), bf(torch.randn(ff, W, generator=g) / 6), bf(torch.randn(W, ff, generator=g) / 5)
    bg, bu, bd = torch.randn(ff, generator=g), torch.randn(ff, generator=g), torch.randn(W, generator=g)
    hd, wgu = h.to(dtype).to(DEV), torch.cat([wg, wu]).to(dtype).to(DEV)
    a = _ops().linear_glu_clamped(hd, wgu, torch.cat([bg, bu]).to(DEV), limit, 1.702, 1.0)
    y = _ops().linear(a, wd.to(dtype).to(DEV))
    x = torch.zeros(T, 1, W, device=DEV)
    _ops().lanes_update_norm(x, y, torch.ones(1, 1, device=DEV), torch.ones(1, device=DEV), dtype, y_bias=bd.to(DEV))
    lim = limit if limit > 0 else 1e30
    want = no.clamped_ff(h.double(), wg.double(), bg.double(), wu.double(), bu.double(), wd.double(), bd.double(), lim)
    assert nerr(x[:, 0], want) < tol(dtype, 3e-6, 1e-2)
    # no biases, another activation constant: the shared expert's form silu(g) u
    a = _ops().linear_glu_clamped(hd, wgu, None, 0.0, 1.0, 0.0)
    gq, uq = h.double() @ wg.double().T, h.double() @ wu.double().T
    assert nerr(a, gq * no.sigma(gq) * uq) < tol(dtype, 3e-6, 1e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("outputs,top,groups,keep", [(8, 3, 4, 2), (12, 4, 1, 1), (20, 4, 4, 3), (6, 6, 3, 3), (9, 2, 9, 2), (40, 5, 5, 1), (8, 4, 4, 1)])
def test_router_choice_and_weights(dtype, outputs, top, groups, keep):
    """Corrections of the scores' own size, many of them negative: an excluded group must count as minus infinity, not zero."""
    g = torch.Generator().manual_seed(10)
    T, W = 50, 48
    h = bf(torch.randn(T, W, generator=g))
    wr = bf(torch.randn(outputs, W, generator=g) * 0.3)
    corr = bf(torch.randn(outputs, generator=g) * 0.1 - 0.1)
    idx, wgt = _ops().moe_route_grouped(h.to(dtype).to(DEV), wr.to(DEV), corr.to(DEV), top, groups, keep)
    n_top = min(top, keep * (outputs // groups))
    flips = 0
    for t in range(T):
        chosen, w = no.route(h[t].double(), wr.double(), corr.double(), top, groups, keep)
        got = idx[t].tolist()
        if got[:n_top] != chosen:
            flips += 1            # a near tie, decided the other way by float32 rounding
            continue
        assert got[n_top:] == [-1] * (top - n_top)
        assert nerr(wgt[t, :n_top], w) < 1e-5
        assert abs(float(wgt[t].sum()) - 1.0) < 1e-5
    assert flips <= 1


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T", [9, 300])
def test_experts_identity_outputs_and_the_shared_expert(dtype, T):
    """The feed-forward from its operators: router, routed experts (the weight on the output), identity outputs that hand the
    input through, the shared expert, all summed into one lane; a crowded expert and an unused one."""
    g = torch.Generator().manual_seed(11)
    W, E, ident, top, ff, sff = 48, 5, 3, 3, 24, 16
    h = bf(torch.randn(T, W, generator=g))
    wr = bf(torch.randn(E + ident, W, generator=g) * 0.3)
    corr = torch.zeros(E + ident)
    corr[1], corr[3], corr[E] = 0.5, -5.0, 0.3            # expert 1 crowded, expert 3 never chosen, identity output E popular
    wgu = bf(torch.randn(E, 2 * ff, W, generator=g) / 6)
    wd = bf(torch.randn(E, W, ff, generator=g) / 5)
    sgu, sd = bf(torch.randn(2 * sff, W, generator=g) / 6), bf(torch.randn(W, sff, generator=g) / 4)
    hd = h.to(dtype).to(DEV)
    idx, wgt = _ops().moe_route_grouped(hd, wr.to(DEV), corr.to(DEV), top, 4, 3)
    assert int((idx == 1).sum()) > T // 2 and int((idx == 3).sum()) == 0 and int((idx >= E).sum()) > 0
    eo, pr, ws = _ops().moe_expert_rows(hd, idx, wgt, wgu.to(dtype).to(DEV), wd.to(dtype).to(DEV), 0.0, 1.0, 0.0, scale_input=False)
    y = _ops().linear(_ops().glu_clamped_bias(_ops().linear(hd, sgu.to(dtype).to(DEV)), None, sff, 0.0, 1.0, 0.0), sd.to(dtype).to(DEV))
    x = torch.zeros(T, 1, W, device=DEV)
    _ops().lanes_update_norm(x, y, torch.ones(1, 1, device=DEV), torch.ones(1, device=DEV), dtype, expert_out=eo, pair_row=pr, top_expert=idx,
                             top_weight=wgt, h_in=hd, experts=E)
    want = torch.zeros(T, W, dtype=F64)
    hq = hd.double().cpu()
    for t in range(T):
        for k in range(top):
            e, we = int(idx[t, k]), float(wgt[t, k])
            want[t] += we * (no.silu_ff(hq[t:t + 1], wgu[e, :ff].double(), wgu[e, ff:].double(), wd[e].double())[0] if e < E else hq[t])
    want += no.silu_ff(hq, sgu[:sff].double(), sgu[sff:].double(), sd.double())
    assert nerr(x[:, 0], want) < tol(dtype, 3e-6, 1.2e-2)
    del ws


# ------------------------------------------------------------------------------------------------
# the model through the engine
# ------------------------------------------------------------------------------------------------
def make_engine(tmp_path, cfg, weights, dtype, max_tokens=512, block_size=16, live=4, budget=2048):
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.engine import Engine
    tmp_path.mkdir(exist_ok=True)
    (tmp_path / "config.json").write_text(json.dumps(no.checkpoint_config(cfg)))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return Engine.from_model_dir(tmp_path, dtype=dtype, device=DEV, max_tokens=max_tokens, block_size=block_size,
                                 max_live_requests=live, max_num_batched_tokens=budget)


VARIANTS = {
    "base": dict(),
    "one_stream": dict(lanes=None, layers=2),
    "one_lane": dict(lanes=1, layers=2, identity=0, groups=1, keep_groups=1, shared_ff=0, window=0, keep=0),
    "four_lanes_all_groups": dict(lanes=4, layers=2, heads=3, kv_heads=3, dim=10, groups=2, keep_groups=2, identity=0, experts=4, top=2, keep=0),
    "window_of_one": dict(window=1, keep=2, layers=2, top=1, kinds=["moe", None]),
    "kept_beyond_the_window": dict(window=6, keep=20, layers=2, table_rows=6, far=11),
    "heads_of_64": dict(width=64, heads=4, kv_heads=1, dim=64, window=150, keep=9, layers=2, table_rows=24, far=300, expert_ff=32, shared_ff=32,
                        scale=0.125),
    "odd_sizes": dict(width=50, vocab=37, lanes=3, heads=6, kv_heads=3, dim=6, window=33, keep=1, table_rows=7, far=29, ff=11, experts=7,
                      identity=3, top=4, groups=5, keep_groups=3, expert_ff=9, shared_ff=13, layers=4),
}


def build(name, seed=0):
    g = torch.Generator().manual_seed(300 + seed)
    cfg = no.random_config(**VARIANTS[name])
    return cfg, no.random_weights(cfg, g), g


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_matches_the_plain_model(tmp_path, dtype, name):
    cfg, w, g = build(name)
    toks = torch.randint(0, cfg["vocab"], (83,), generator=g).tolist()
    want, layers = no.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, dtype)
    out = eng.step_forced([("a", toks, list(range(len(toks))))], want_residual_trace=True)
    assert out.residual_trace.shape[0] == len(layers)
    for i in range(len(layers)):
        assert model_close(out.residual_trace[i], layers[i], dtype, 5e-6), i
    assert model_close(out.logits, want, dtype)


@pytest.mark.parametrize("name", ["base", "odd_sizes", "window_of_one", "kept_beyond_the_window"])
def test_decoding_token_by_token_equals_the_whole_prompt(tmp_path, name):
    """70 single-token steps on pages of four tokens: every page border, the first tokens, the kept tokens falling out of the
    window, and the window passing over decoded tokens."""
    cfg, w, g = build(name, 1)
    toks = torch.randint(0, cfg["vocab"], (70,), generator=g).tolist()
    want, _ = no.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, torch.float32, max_tokens=128, block_size=4)
    got = [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks]
    assert nerr(torch.cat(got), want) < 1e-5


@pytest.mark.parametrize("dtype", BOTH)
def test_long_portions_beside_decoded_tokens(tmp_path, dtype):
    """Portions of 128 tokens and more (bfloat16: the tensor-memory kernel) in one step with short portions and single tokens,
    over a window that the long portions cross and kept tokens that fall behind it."""
    cfg, w, g = build("heads_of_64", 8)
    toks = {k: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for k, n in (("a", 400), ("b", 40), ("c", 330))}
    want = {k: no.forward(cfg, w, t)[0] for k, t in toks.items()}
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=1024)
    steps = [[("a", 200), ("b", 3)], [("a", 130), ("b", 1), ("c", 129)], [("c", 200), ("a", 69), ("b", 36)], [("a", 1), ("c", 1)]]
    at, got = {k: 0 for k in toks}, {k: [] for k in toks}
    for step in steps:
        entries = []
        for k, n in step:
            entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
        out = eng.step_forced(entries)
        r = 0
        for k, n in step:
            got[k].append(out.logits[r:r + n].clone())
            r += n
    for k in toks:
        assert at[k] == len(toks[k]) and model_close(torch.cat(got[k]), want[k], dtype), k


def test_long_decoding_far_past_the_window(tmp_path):
    cfg, w, g = build("heads_of_64", 2)
    toks = torch.randint(0, cfg["vocab"], (260,), generator=g).tolist()
    want, _ = no.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, torch.bfloat16, max_tokens=320, block_size=16)
    got = [eng.step_forced([("a", toks[:30], list(range(30)))]).logits.clone()]
    got += [eng.step_forced([("a", [t], [0])]).logits.clone() for t in toks[30:]]
    assert model_close(torch.cat(got), want, torch.bfloat16)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", ["base", "heads_of_64"])
@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [40, 2, 17, 1, 1, 2, 64, 5], [1, 130, 1, 1], [19, 20, 21]])
def test_portions_of_any_size_equal_the_whole_prompt(tmp_path, dtype, name, sizes):
    cfg, w, g = build(name, 3)
    n = sum(sizes)
    toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
    want, _ = no.forward(cfg, w, toks)
    eng = make_engine(tmp_path, cfg, w, dtype, block_size=16)
    got, at = [], 0
    for s in sizes:
        got.append(eng.step_forced([("a", toks[at:at + s], list(range(s)))]).logits.clone())
        at += s
    assert model_close(torch.cat(got), want, dtype)
    if dtype == torch.bfloat16:      # how the prompt was cut changes the result by rounding only
        whole = make_engine(tmp_path / "w", cfg, w, dtype).step_forced([("a", toks, list(range(n)))]).logits
        assert model_close(torch.cat(got), whole, dtype)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", ["base", "heads_of_64"])
def test_mixed_batches_with_reused_pages_equal_each_request_alone(tmp_path, dtype, name):
    """Five requests through a pool of 12 pages of 16, at most two live: later requests inherit the pages of ended ones (full of
    their keys and values, in every layer's cache) and must not see them."""
    cfg, w, g = build(name, 4)
    lens = {"a": 70, "b": 9, "c": 55, "d": 33, "e": 60}
    toks = {k: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for k, n in lens.items()}
    want = {k: no.forward(cfg, w, t)[0] for k, t in toks.items()}
    eng = make_engine(tmp_path, cfg, w, dtype, max_tokens=12 * 16 - 2 * 16, block_size=16, live=2)
    assert eng.cache.blocks.capacity == 12
    steps = [[("a", 40), ("b", 3)], [("a", 2), ("b", 1)], [("b", 5), ("a", 27)], [("a", 1), ("c", 30)], [("c", 1), ("d", 2)],
             [("d", 31), ("c", 24)], [("e", 59)], [("e", 1)]]
    at, got = {k: 0 for k in lens}, {k: [] for k in lens}
    for step in steps:
        entries, end = [], []
        for k, n in step:
            entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == lens[k]:
                end.append(k)
        out = eng.step_forced(entries, end)
        r = 0
        for k, n in step:
            got[k].append(out.logits[r:r + n].clone())
            r += n
    assert at == lens and eng.cache.live == 0
    for k in lens:
        assert model_close(torch.cat(got[k]), want[k], dtype), k


def test_batch_members_do_not_change_each_other(tmp_path):
    """bfloat16: a request's logits are bit-identical alone and beside others (same cut of its own prompt)."""
    cfg, w, g = build("heads_of_64", 5)
    ta, tb = (torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (50, 33))
    alone = make_engine(tmp_path / "x", cfg, w, torch.bfloat16)
    a1 = alone.step_forced([("a", ta[:49], list(range(49)))]).logits.clone()
    a2 = alone.step_forced([("a", ta[49:], [0])]).logits.clone()
    both = make_engine(tmp_path / "y", cfg, w, torch.bfloat16)
    both.step_forced([("b", tb[:32], [])])
    b1 = both.step_forced([("b", tb[32:], [0]), ("a", ta[:49], list(range(49)))]).logits[1:].clone()
    both.step_forced([("c", tb, [])])
    b2 = both.step_forced([("c", tb[:1], []), ("a", ta[49:], [0])]).logits.clone()
    assert torch.equal(a1, b1) and torch.equal(a2, b2)


def test_a_changed_token_matters_where_it_is_visible_only(tmp_path):
    """One layer, window 12, 3 kept tokens: the logits at position p feel the token at p - 11 and at 2, not the one at p - 12
    or at 3 — in a prompt's portion and when decoded alone."""
    cfg = no.random_config(layers=1, window=12, keep=3, kinds=["dense"])
    g = torch.Generator().manual_seed(77)
    w = no.random_weights(cfg, g)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    p = 39
    for decoded in (False, True):
        res = {}
        for name, j in (("same", None), ("inside", p - 11), ("outside", p - 12), ("kept", 2), ("not_kept", 3)):
            t = list(toks)
            if j is not None:
                t[j] = (t[j] + 1) % cfg["vocab"]
            eng = make_engine(tmp_path / f"{name}{decoded}", cfg, w, torch.float32)
            if decoded:
                eng.step_forced([("a", t[:p], [])])
                res[name] = eng.step_forced([("a", t[p:], [0])]).logits[0].clone()
            else:
                res[name] = eng.step_forced([("a", t, [p])]).logits[0].clone()
            assert nerr(res[name], no.forward(cfg, w, t)[0][p]) < 1e-5
        assert nerr(res["outside"], res["same"]) < 1e-6 and nerr(res["not_kept"], res["same"]) < 1e-6
        assert nerr(res["inside"], res["same"]) > 1e-3 and nerr(res["kept"], res["same"]) > 1e-3


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
            lg = no.forward(cfg, w, t)[0][-1]
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) < 1e-3:
                break
            assert int(lg.argmax()) == tok
            t.append(tok)


def test_command_line_and_trace_replay(tmp_path, capsys, monkeypatch):
    import io
    from atoma_infer_b200 import checkpoint
    from atoma_infer_b200.__main__ import main
    cfg, w, g = build("one_stream", 7)
    (tmp_path / "config.json").write_text(json.dumps(no.checkpoint_config(cfg)))
    checkpoint.write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    assert main(["generate", "--model", str(tmp_path), "--prompt-ids", "3,4,5,6", "--max-new-tokens", "2", "--dtype", "float32",
                 "--max-tokens", "128", "--max-live", "2"]) == 0
    line = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.startswith("{")][0]
    lg = no.forward(cfg, w, [3, 4, 5, 6])[0][-1]
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
    want, _ = no.forward(cfg, w, toks)
    assert not (out / "1.f32").exists()
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1)
    assert nerr(a, want[[1, 3]]) < 1e-5 and nerr(b, torch.stack([want[5], want[1]])) < 1e-5
