"""The CUDA kernels and kernel options that the Mamusun family brought, each alone against its plain restatement in
tests/torch_kernels.py: the step between a grouped attention's projection and its scores (bias, norms per head or over the whole
projection, before or after a rotation of halves or of neighbours, keys as values, a layer without keys), the sink of the
softmax on both attention kernels, norms behind a scaled sum with the average over depth, the mean of normed branches, the normed
polynomial, the gated linear recurrence with its convolution (portions, segments, slots used again), and routing by a softmax over
the chosen outputs.  Planted scores show a sink that is left out, scaled or counted per split, and a window that is one off."""
import math

import pytest
import torch

import torch_kernels as R
from test_fomerax_kernels_gpu import fill_pages
from test_rodapel_kernels_gpu import close, flat_plan, meta_for, paged, rnd

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def K():
    from iitj_llm_coopt_b200 import kernels
    return kernels.load()


def tables_for(pos, rot, amp=1.0):
    if not rot:
        return None
    inv = 1.0 / (300.0 ** (torch.arange(0, rot, 2).float() / rot))
    ang = torch.tensor(pos).float().unsqueeze(1) * inv.unsqueeze(0)
    return (ang.cos() * amp).cuda().contiguous(), (ang.sin() * amp).cuda().contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,norm,gains,norm_first,rot,inter,bias,own,vfk,page", [
    (4, 2, 16, 24, "head", True, True, 0, False, False, True, False, 8),        # head norms with gains, no rotation
    (4, 2, 16, 24, "head", True, True, 0, False, False, False, False, 8),       # queries alone
    (6, 3, 32, 16, "head", False, False, 8, True, False, True, False, 16),      # neighbours rotate, then unit norms
    (8, 8, 12, 12, "row", True, True, 12, False, True, True, True, 4),          # biases, whole-projection norms, halves, keys as values
    (3, 1, 40, 40, "row", True, True, 6, False, True, True, True, 16),
    (2, 2, 8, 6, "none", False, True, 4, True, True, True, False, 8),           # a bias on the values too
    (1, 1, 130, 70, "head", False, True, 130, False, False, True, False, 32),   # a whole wide head rotates
    (64, 8, 128, 128, "row", True, True, 64, False, True, True, True, 16),      # a row beyond 48 KB of shared memory
])
def test_qk_prepare(K, dtype, heads, kv_heads, dim, vdim, norm, gains, norm_first, rot, inter, bias, own, vfk, page):
    lens = [37, 5]
    per = kv_heads * (dim + vdim)
    cache, table = paged(dtype, 2, lens, page, per, seed=dim)
    ref_cache = cache.clone()
    cols = heads * dim + (kv_heads * dim if own else 0) + (kv_heads * vdim if own and not vfk else 0)
    gq = gk = b = None
    if gains:
        n = dim if norm == "head" else heads * dim
        gq, gk = rnd(n, seed=1) * 0.2 + 1.0, rnd(dim if norm == "head" else kv_heads * dim, seed=2) * 0.2 + 1.0
    if bias:
        b = rnd(cols, seed=3, s=0.5)
    RK = R.TorchKernels()
    done = [0, 0]
    for portion in ([30, 5], [2, 0], [5, 0]):
        req, pos = [], []
        for r, n in enumerate(portion):
            req += [r] * n
            pos += list(range(done[r], done[r] + n))
            done[r] += n
        T = len(req)
        slots = torch.tensor([int(table[r, p // page]) * page + p % page for r, p in zip(req, pos)], dtype=torch.int32).cuda() if own else None
        a = rnd(T, cols, dtype=dtype, seed=T, s=1.5)
        want = a.clone()
        tabs = tables_for(pos, rot, 1.2)
        kw = dict(bias=b, norm=norm, q_gain=gq, k_gain=gk if own else None, norm_first=norm_first, tables=tabs, rotary_dim=rot, interleaved=inter,
                  own_kv=own, value_from_key=vfk)
        K.qk_prepare(a, heads, kv_heads, dim, vdim, 1e-5, cache_layer=cache, slots=slots, **kw)
        RK.qk_prepare(want, heads, kv_heads, dim, vdim, 1e-5, cache_layer=ref_cache, slots=slots, **kw)
        close(a[:, :heads * dim], want[:, :heads * dim], dtype)
        assert torch.equal(a[:, heads * dim:], want[:, heads * dim:])          # the rest of the row stays as it was
    written = ~torch.isnan(ref_cache.float())
    assert torch.equal(written, ~torch.isnan(cache.float()))
    if own:
        close(cache.float()[written], ref_cache.float()[written], dtype)
    else:
        assert not written.any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,window", [(4, 2, 32, 32, 16, 0), (6, 6, 16, 16, 8, 0), (3, 1, 24, 8, 4, 13), (8, 2, 64, 64, 16, 0),
                                                                  (1, 1, 8, 8, 8, 0), (2, 1, 96, 96, 16, 40)])
def test_sinks_on_both_attention_kernels(K, dtype, heads, kv_heads, dim, vdim, page, window):
    lens = [300, 11]
    per = kv_heads * (dim + vdim)
    cache, table = paged(dtype, 2, lens, page, per, seed=dim)
    g = torch.Generator().manual_seed(dim)
    kplane, vplane, _ = R.flat_planes(cache, kv_heads, dim, vdim, False)
    for b, n in enumerate(lens):
        for j in range(n):
            pg, o = int(table[b, j // page]), j % page
            kplane[pg, :, o] = torch.randn(kv_heads, dim, generator=g).to(dtype)
            vplane[pg, :, o] = torch.randn(kv_heads, vdim, generator=g).to(dtype)
    sinks = rnd(heads, seed=5, s=2.0).abs() + 3.0
    RK = R.TorchKernels()
    for req, pos in (([0] * 40 + [1] * 11, list(range(0, 40)) + list(range(11))), ([0] * 2 + [1], [40, 41, 10]), ([0], [299]), ([0], [0]),
                     ([0] * 30, list(range(270, 300)))):
        T = len(req)
        q = rnd(T, heads * dim, dtype=dtype, seed=T, s=1.0)
        meta = meta_for(table, req, pos)
        want = torch.empty(T, heads * vdim, dtype=torch.float32, device="cuda")
        RK.attention_flat(q, cache, meta, want, heads, kv_heads, dim, vdim, scale=0.3, window=window, sinks=sinks)
        plain = torch.empty_like(want)
        RK.attention_flat(q, cache, meta, plain, heads, kv_heads, dim, vdim, scale=0.3, window=window)
        assert (plain - want).abs().max() > 1e-3                     # the sink matters at these sizes
        out = torch.empty(T, heads * vdim, dtype=dtype, device="cuda")
        plans = [None, flat_plan(K, req, pos, heads, kv_heads, dim, vdim, window)]
        if T == 1:
            plans.append(flat_plan(K, req, pos, heads, kv_heads, dim, vdim, window, splits=3))
        for plan in plans:
            out.fill_(float("nan"))
            K.attention_flat(q, cache, meta, out, heads, kv_heads, dim, vdim, scale=0.3, window=window, plan=plan, sinks=sinks)
            close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page,window,total", [(4, 0, 40), (16, 9, 300), (8, 16, 64)])
def test_planted_scores_show_the_sink_and_the_window_s_edge(K, dtype, page, window, total):
    """One head whose keys all score 0 except key `far`, which scores a; every value is 0 except key far's and key (p - window + 1)'s.
    The output's first number is then the weight of key far, e^a / (e^a + n - 1 + e^sink) with n the visible keys, straight from the
    definition: a sink that is scaled, masked or counted once per split gives another number, and so does a window that is one
    token wider or narrower (its edge key carries the second value)."""
    dim, vdim, a, sink, scale = 16, 8, 3.0, 1.25, 0.5
    far = 1
    cache, table = paged(dtype, 1, [total], page, dim + vdim, seed=page)
    keys, vals = torch.zeros(total, 1, dim), torch.zeros(total, 1, vdim)
    keys[far, 0, 0] = a / scale
    vals[far, 0, 0] = 1.0
    fill_pages(cache, table, page, 1, dim, vdim, False, keys, vals)
    kplane, vplane, _ = R.flat_planes(cache, 1, dim, vdim, False)
    sinks = torch.tensor([sink]).cuda()
    for p in sorted({far, far + 1, total - 1, min(total - 1, far + max(window, 2) - 1), min(total - 1, far + max(window, 2))}):
        lo = max(0, p - window + 1) if window else 0
        n = p - lo + 1
        sees_far = lo <= far <= p
        want0 = math.exp(a) / (math.exp(a) + n - 1 + math.exp(sink)) if sees_far else 0.0
        edge = 1.0 / ((math.exp(a) if sees_far else 0.0) + n - (1 if sees_far else 0) + math.exp(sink))      # weight of a key that scores 0
        pg, o = int(table[0, lo // page]), lo % page
        before = vplane[pg, 0, o].clone()
        if lo != far:
            vplane[pg, 0, o, 1] = 1.0                       # the first key inside the window carries the second value
        if lo > 0:
            pg2, o2 = int(table[0, (lo - 1) // page]), (lo - 1) % page
            keep2 = vplane[pg2, 0, o2].clone()
            if lo - 1 != far:
                vplane[pg2, 0, o2, 2] = 1.0                 # the key just outside carries a third that must not show
        q = torch.zeros(1, dim, dtype=dtype, device="cuda")
        q[:, 0] = 1.0
        meta = meta_for(table, [0], [p])
        out = torch.empty(1, vdim, dtype=dtype, device="cuda")
        for plan in (None, flat_plan(K, [0], [p], 1, 1, dim, vdim, window), flat_plan(K, [0], [p], 1, 1, dim, vdim, window, splits=4)):
            out.fill_(float("nan"))
            K.attention_flat(q, cache, meta, out, 1, 1, dim, vdim, scale=scale, window=window, plan=plan, sinks=sinks)
            tol = 1e-5 if dtype == torch.float32 else 6e-3
            assert abs(out[0, 0].item() - want0) < tol, (p, out[0], want0)
            if lo != far:
                assert abs(out[0, 1].item() - edge) < tol, (p, out[0], edge)
            assert out[0, 2].item() == 0.0
        vplane[pg, 0, o] = before
        if lo > 0:
            vplane[pg2, 0, o2] = keep2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width,inputs", [(1, 8, 2), (5, 200, 3), (3, 2050, 7), (2, 13000, 2)])
def test_post_norm_and_the_average_over_depth(K, dtype, tokens, width, inputs):
    x, branch, gain = rnd(tokens, width, seed=1), rnd(tokens, width, dtype=dtype, seed=2, s=3.0), rnd(width, seed=3) * 0.1 + 1.0
    for alpha in (1.0, 3.5):
        out, cast = torch.empty_like(x), torch.empty(tokens, width, dtype=dtype, device="cuda")
        K.post_norm(x, branch, alpha, gain, 1e-5, out, cast_out=cast)
        want = R.ref_post_norm(x, branch, alpha, gain, 1e-5)
        close(out, want, torch.float32)
        assert torch.equal(cast, out.to(dtype))
        # through a history: the row becomes its last entry, the weighted sum over it what goes on; in place
        hist = rnd(inputs + 1, tokens, width, seed=4)
        keep = hist.clone()
        mix = rnd(inputs, seed=5)
        xs = x.clone()
        K.post_norm(xs, branch, alpha, gain, 1e-5, xs, cast_out=cast, history=hist[:inputs], mix=mix)
        close(hist[inputs - 1], want, torch.float32)
        assert torch.equal(hist[:inputs - 1], keep[:inputs - 1]) and torch.equal(hist[inputs], keep[inputs])
        mixed = (mix.view(-1, 1, 1) * torch.cat([keep[:inputs - 1], want.unsqueeze(0)])).sum(0)
        close(xs, mixed, torch.float32, scale=max(mixed.abs().max().item(), 1.0))
        assert torch.equal(cast, xs.to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width,n", [(1, 8, 2), (7, 200, 2), (3, 2050, 3), (2, 40, 1)])
def test_branch_mean(K, dtype, tokens, width, n):
    branches = [rnd(tokens, width, dtype=dtype, seed=i, s=1.0 + i) for i in range(n)]
    gains = [rnd(width, seed=10 + i) * 0.2 + 1.0 for i in range(n)]
    out = torch.empty(tokens, width, device="cuda")
    K.branch_mean(branches, gains, 0.5, 1e-5, out)
    close(out, R.ref_branch_mean(branches, gains, 0.5, 1e-5), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,inner", [(1, 8), (7, 37), (3, 3000)])
def test_poly_norm(K, dtype, tokens, inner):
    z = rnd(tokens, inner, dtype=dtype, s=2.0)
    coef = torch.tensor([0.9, -0.4, 0.25, 0.1]).cuda()
    act = torch.empty_like(z)
    K.poly_norm(z, coef, 1e-5, act)
    close(act, R.ref_poly_norm(z, coef, 1e-5), dtype)


@pytest.mark.parametrize("outputs,top", [(12, 1), (5, 2), (3, 3), (1, 1), (64, 6)])
def test_route_by_softmax_over_the_chosen(K, outputs, top):
    scores, bias = rnd(9, outputs, s=2.0), rnd(outputs, seed=4, s=2.0)
    for b in (bias, None):
        chosen = torch.empty(9, top, dtype=torch.int32, device="cuda")
        weights = torch.empty(9, top, dtype=torch.float32, device="cuda")
        K.route_topk(scores, b, chosen, weights, chosen_softmax=True)
        c, w = R.ref_route_topk(scores, b, top, chosen_softmax=True)
        assert torch.equal(chosen, c)
        close(weights, w, torch.float32)
        assert (weights.sum(1) - 1.0).abs().max() < 1e-5
    if outputs > top:            # the bias decides the choice
        c0, _ = R.ref_route_topk(scores, None, top, chosen_softmax=True)
        c1, _ = R.ref_route_topk(scores, bias, top, chosen_softmax=True)
        assert not torch.equal(c0, c1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,blocks,taps", [(16, 2, 4), (48, 3, 2), (200, 1, 5), (256, 4, 3), (96, 96, 1), (64, 2, 12)])
def test_gated_recurrence_in_portions_segments_and_reused_slots(K, dtype, width, blocks, taps):
    """Three requests over four state slots: whole prompts of 150 tokens and more in one step (segments), the same in portions down to
    one token (the walk), two requests side by side, against the plain restatement run over each request whole; a slot that is
    cleared and used again starts from zero."""
    side = width // blocks
    ld = 2 * width + 5
    lens = [150, 70, 9]
    proj = [rnd(n, ld, dtype=dtype, seed=20 + i, s=1.0) for i, n in enumerate(lens)]
    by, bx, cb = rnd(width, seed=1, s=0.3), rnd(width, seed=2, s=0.3), rnd(width, seed=3, s=0.2)
    tw = rnd(width, taps, seed=4, s=0.5)
    ra, ri = rnd(blocks, side, side, dtype=dtype, seed=5, s=side ** -0.5), rnd(blocks, side, side, dtype=dtype, seed=6, s=side ** -0.5)
    rab, rib, lam = rnd(width, seed=7, s=0.5), rnd(width, seed=8, s=0.5), rnd(width, seed=9) - 1.0
    y_col, x_col = 3, width + 5

    def run(kern, state, steps):
        """steps: list of [(request, slot, first, count)]; returns {request: rows}"""
        got = {r: [] for r in range(len(lens))}
        for entries in steps:
            rows = torch.cat([proj[r][a:a + n] for r, _, a, n in entries])
            cu = torch.tensor([0] + list(torch.tensor([n for *_, n in entries]).cumsum(0)), dtype=torch.int32).cuda()
            slots = torch.tensor([s for _, s, _, _ in entries], dtype=torch.int32).cuda()
            tr = torch.tensor([i for i, (*_, n) in enumerate(entries) for _ in range(n)], dtype=torch.int32).cuda()
            out = torch.empty(rows.shape[0], width, dtype=dtype, device="cuda")
            kern.lru(rows, y_col, x_col, width, by, bx, tw, cb, ra, ri, rab, rib, lam, 8.0, state, slots, tr, cu, out,
                     longest=max(n for *_, n in entries))
            at = 0
            for r, _, _, n in entries:
                got[r].append(out[at:at + n].float())
                at += n
        return {r: torch.cat(v) for r, v in got.items() if v}

    RK = R.TorchKernels()
    whole = [[(0, 2, 0, 150)], [(1, 0, 0, 70), (2, 3, 0, 9)]]
    want = run(RK, torch.zeros(4, taps, width, device="cuda"), whole)
    state = torch.zeros(4, taps, width, device="cuda")
    got = run(K, state, whole)
    for r in want:
        close(got[r], want[r], dtype)
    ref_state = torch.zeros(4, taps, width, device="cuda")
    run(RK, ref_state, whole)
    close(state, ref_state, torch.float32, scale=max(ref_state.abs().max().item(), 1e-3) * (1 if dtype == torch.float32 else 4))
    # the same requests cut up, in other slots, beside one another; slots 2 and 0 are cleared and used again
    state[2].zero_()
    state[0].zero_()
    cut = [[(0, 0, 0, 1)], [(0, 0, 1, 2), (1, 2, 0, 65)], [(0, 0, 3, 100), (1, 2, 65, 1)], [(1, 2, 66, 4), (0, 0, 103, 47)]]
    again = run(K, state, cut)
    for r in (0, 1):
        close(again[r], want[r], dtype)
    if dtype == torch.float32:
        assert max((again[r] - got[r]).abs().max().item() for r in (0, 1)) < 1e-5
    # two requests side by side, one token a step (the one-launch form), one of them ending early
    state.zero_()
    single = [[(1, 1, i, 1), (2, 3, i, 1)] if i < 9 else [(1, 1, i, 1)] for i in range(25)]
    one = run(K, state, single)
    close(one[2], want[2], dtype)
    close(one[1], want[1][:25], dtype)
