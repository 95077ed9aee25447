"""The CUDA kernels and kernel options that the Fomerax family brought, each alone against its plain restatement in
tests/torch_kernels.py: scaled rotation tables, a branch norm that also norms the new row, norms of column ranges, gated
activations, the token input's gate, grouped products with a sigmoid gate in the epilogue, sigmoid routing, experts that
take their weight on the input, a latent row beside queries of another product, and the score options of the attention
over flat pages (a tanh cap, a distance bias per head, a query temperature, a gate on every output number, a window over
shared key/value rows), on both of its kernels.  Planted keys show a window, a distance or a period that is one off."""
import math

import pytest
import torch

import torch_kernels as R
from test_rodapel_kernels_gpu import close, flat_plan, meta_for, paged, rnd

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def K():
    from iitj_llm_coopt_b200 import kernels
    return kernels.load()


def test_rope_tables_with_amplitude(K):
    pos = torch.tensor([0, 1, 7, 4095, 100000], dtype=torch.int32).cuda()
    inv = (1.0 / 300.0 ** (torch.arange(0, 10, 2).float() / 10)).cuda()
    got = [torch.empty(5, 5, device="cuda") for _ in range(2)]
    want = [torch.empty(5, 5, device="cuda") for _ in range(2)]
    for amp in (1.0, 1.2079):
        K.rope_tables(pos, inv, got[0], got[1], amplitude=amp)
        R.TorchKernels().rope_tables(pos, inv, want[0], want[1], amplitude=amp)
        assert (got[0] - want[0]).abs().max() < 2e-3 and (got[1] - want[1]).abs().max() < 2e-3     # float32 angles of 1e5
        assert (got[0][:3] - want[0][:3]).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width", [(1, 8), (5, 200), (3, 2050), (2, 4099)])
def test_norm_add_with_the_next_norm(K, dtype, tokens, width):
    res, branch = rnd(tokens, width, seed=1), rnd(tokens, width, dtype=dtype, seed=2, s=3.0)
    w, w2 = rnd(width, seed=3) + 1.0, rnd(width, seed=4) + 1.0
    r = res.clone()
    nxt = torch.empty(tokens, width, dtype=dtype, device="cuda")
    K.norm_add(r, branch, w, 1e-5, next_weight=w2, next_out=nxt)
    want = R.ref_norm_add(res, branch, w, 1e-5)
    close(r, want, torch.float32)
    close(nxt, R.ref_rmsnorm_rows(want, w2, 1e-5), dtype)
    # with a copy of the new rows as well
    r2, cast = res.clone(), torch.empty(tokens, width, dtype=dtype, device="cuda")
    K.norm_add(r2, branch, w, 1e-5, cast_out=cast, next_weight=w2, next_out=nxt)
    assert torch.equal(r2, r) and torch.equal(cast, r.to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,cols,lead,wide", [(1, 3, 0, 3), (7, 80, 0, 176), (5, 24, 20, 60), (3, 1030, 2, 1040)])
def test_rmsnorm_rows_of_a_column_range(K, dtype, rows, cols, lead, wide):
    a = rnd(rows, wide, dtype=dtype, seed=5, s=2.0)
    gain = rnd(cols, seed=6) * 0.2 + 1.0
    out = torch.full((rows, cols + 3), 9.0, dtype=dtype, device="cuda")
    K.rmsnorm_rows(a[:, lead:lead + cols], gain, 1e-6, out[:, 1:1 + cols])
    close(out[:, 1:1 + cols], R.ref_rmsnorm_rows(a[:, lead:lead + cols], gain, 1e-6), dtype)
    assert (out[:, 0] == 9.0).all() and (out[:, 1 + cols:] == 9.0).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_glu_act(K, dtype, activation):
    gu = rnd(7, 2 * 37, dtype=dtype, s=3.0)
    act = torch.empty(7, 37, dtype=dtype, device="cuda")
    K.glu_act(gu, act, activation)
    close(act, R.ref_glu_act(gu, activation), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,dim,table_width,offset", [(1, 1, 1, 0), (9, 8, 32, 16), (5, 3, 9, 6), (4, 130, 400, 137)])
def test_token_side_gate(K, dtype, tokens, dim, table_width, offset):
    gate, table = rnd(tokens, dim, dtype=dtype, s=2.0), rnd(50, table_width, dtype=dtype, seed=7)
    ids = torch.randint(0, 50, (tokens,), dtype=torch.int32).cuda()
    out = torch.empty(tokens, dim, dtype=dtype, device="cuda")
    K.token_side_gate(gate, table, ids, offset, out)
    close(out, R.ref_token_side_gate(gate, table, ids, offset), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,groups,n,k", [(5, 3, 24, 16), (70, 8, 32, 64), (1, 1, 7, 13), (33, 5, 20, 40)])
def test_linear_by_group_with_a_gate(K, dtype, rows, groups, n, k):
    a = rnd(rows, groups * k, dtype=dtype, seed=4)
    w = rnd(groups, n, k, dtype=dtype, seed=5, s=k ** -0.5)
    gate = rnd(rows, groups * n, seed=6, s=2.0)
    out = torch.zeros(rows, groups * n, dtype=dtype, device="cuda")
    K.linear_by_group(a, w, out, a_stride=k, out_stride=n, out_gate=gate)
    want = torch.zeros_like(out, dtype=torch.float32)
    R.TorchKernels().linear_by_group(a, w, want, a_stride=k, out_stride=n, out_gate=gate)
    close(out, want, dtype)


@pytest.mark.parametrize("outputs,top", [(12, 1), (5, 2), (3, 3), (1, 1), (64, 6)])
def test_route_topk_by_sigmoid(K, outputs, top):
    scores = rnd(9, outputs, s=2.0)
    chosen = torch.empty(9, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(9, top, dtype=torch.float32, device="cuda")
    K.route_topk(scores, None, chosen, weights, sigmoid=True)
    c, w = R.ref_route_topk(scores, None, top, sigmoid=True)
    assert torch.equal(chosen, c)
    close(weights, w, torch.float32)
    assert (weights.sum(1) > 1.0).any() or top == 1           # the scores stand as they are: nothing is renormalised


def weighted_moe_case(K, dtype, tokens, top, experts, width, ff, chosen=None, seed=0):
    """sum_j expert_{c_j}(w_j x) through plan, grouped products and combine, and through the gathered, weighted rows."""
    g = torch.Generator().manual_seed(seed)
    if chosen is None:
        chosen = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)])
    chosen = chosen.to(torch.int32).cuda()
    weights = (torch.rand(tokens, top, generator=g) * 0.9 + 0.05).cuda()
    x = rnd(tokens, width, dtype=dtype, seed=seed + 1)
    w1 = rnd(experts, 2 * ff, width, dtype=dtype, seed=seed + 2, s=width ** -0.5)
    w2 = rnd(experts, width, ff, dtype=dtype, seed=seed + 3, s=ff ** -0.5)
    rows = tokens * top
    outs = []
    for kern in (K, R.TorchKernels()):
        def ints(n):
            return torch.zeros(n, dtype=torch.int32, device="cuda")
        plan = kern.moe_plan(chosen, experts, ints(rows), ints(rows), torch.zeros(kern.moe_tile_bound(rows, experts) + 1, 4, dtype=torch.int32, device="cuda"),
                             weights=weights, row_weight=torch.zeros(rows, device="cuda"))
        act = torch.zeros(rows, ff, dtype=dtype, device="cuda")
        kern.moe_linear(x, w1, act, plan, gather=True, glu="silu_weighted")
        y = torch.zeros(rows, width, dtype=dtype, device="cuda")
        kern.moe_linear(act, w2, y, plan)
        out = torch.zeros(tokens, width, dtype=dtype, device="cuda")
        kern.moe_combine(y, plan, chosen, None, x, experts, out)
        side = torch.zeros(rows, width, dtype=dtype, device="cuda")
        kern.gather_rows(x, plan, side, weighted=True)
        outs.append((plan, out, side))
    (pk, ok, sk), (pr, orf, sr) = outs
    assert torch.equal(pk["place"], pr["place"]) and torch.equal(pk["row_weight"], pr["row_weight"])
    close(ok, orf, dtype)
    close(sk, sr, dtype)
    # straight from the definition, token by token
    want = torch.zeros(tokens, width, device="cuda")
    for t in range(tokens):
        for j in range(top):
            e, z = int(chosen[t, j]), x[t].float() * weights[t, j]
            h = z @ w1[e].float().t()
            want[t] += (torch.nn.functional.silu(h[:ff]) * h[ff:]) @ w2[e].float().t()
    close(ok, want, dtype, scale=max(want.abs().max().item(), 1e-6) * (1 if dtype == torch.float32 else 2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_weighted_on_their_input(K, dtype):
    weighted_moe_case(K, dtype, tokens=11, top=1, experts=12, width=40, ff=24)
    weighted_moe_case(K, dtype, tokens=150, top=2, experts=3, width=64, ff=100, seed=3)            # several tiles per expert
    weighted_moe_case(K, dtype, tokens=70, top=1, experts=5, width=33, ff=17, chosen=torch.full((70, 1), 4), seed=5)
    weighted_moe_case(K, dtype, tokens=9, top=1, experts=1, width=16, ff=8, seed=7)                # one expert
    weighted_moe_case(K, dtype, tokens=6, top=3, experts=3, width=16, ff=8, seed=9)                # every expert chosen


def fill_pages(cache, table, page, kv_heads, key_dim, value_dim, shared, keys, vals):
    """keys [n, G, Dk] and vals [n, G, Dv] (None with shared rows) of request 0 into its pages."""
    kplane, vplane, _ = R.flat_planes(cache, kv_heads, key_dim, value_dim, shared)
    for j in range(keys.shape[0]):
        pg, o = int(table[0, j // page]), j % page
        kplane[pg, :, o] = keys[j].to(cache.dtype)
        if vals is not None:
            vplane[pg, :, o] = vals[j].to(cache.dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot,rank,q_rank,window,page", [(4, 24, 8, 40, 12, 9, 8), (2, 16, 16, 32, 20, 17, 16), (1, 8, 4, 8, 5, 1, 4),
                                                                   (6, 32, 16, 64, 48, 0, 16)])
def test_latent_rows_beside_queries_of_another_product(K, dtype, heads, dim, rot, rank, q_rank, window, page):
    """The latent row and the shared key part are columns [q_rank, q_rank + rank + rot) of one product, the queries come from
    another; then the windowed attention over the shared rows, in portions of 2, 30 and 1 tokens."""
    row, total = rank + rot, 45
    cache, table = paged(dtype, 1, [total], page, row, seed=rank)
    ref_cache = cache.clone()
    gain = rnd(rank, seed=9) * 0.1 + 1.0
    RK = R.TorchKernels()
    done = 0
    for n in (2, 30, 1, 12):
        pos = list(range(done, done + n))
        done += n
        slots = torch.tensor([int(table[0, p // page]) * page + p % page for p in pos], dtype=torch.int32).cuda()
        down = rnd(n, q_rank + row + 3, dtype=dtype, seed=done)
        qd = rnd(n, heads * (dim + rot), dtype=dtype, seed=done + 1)
        inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))
        ang = torch.tensor(pos).float().unsqueeze(1) * inv.unsqueeze(0)
        tables = ((ang.cos() * 1.3).cuda().contiguous(), (ang.sin() * 1.3).cuda().contiguous())
        qa = rnd(n, heads * row, dtype=dtype, seed=done + 5)
        qb = qa.clone()
        kv = down[:, q_rank:q_rank + row]
        K.latent_prepare(qd, tables, rot, True, gain, 1e-5, qa, cache, slots, heads, dim, rot, rank, kv=kv)
        RK.latent_prepare(qd, tables, rot, True, gain, 1e-5, qb, ref_cache, slots, heads, dim, rot, rank, kv=kv)
        close(qa, qb, dtype)
        meta = meta_for(table, [0] * n, pos)
        out = torch.empty(n, heads * rank, dtype=dtype, device="cuda")
        want = torch.empty(n, heads * rank, dtype=torch.float32, device="cuda")
        RK.attention_flat(qb, ref_cache, meta, want, heads, 1, row, rank, shared_value=True, scale=0.2, window=window)
        for plan in (None, flat_plan(K, [0] * n, pos, heads, 1, row, rank, window), flat_plan(K, [0] * n, pos, heads, 1, row, rank, window, splits=2)):
            out.fill_(float("nan"))
            K.attention_flat(qa, cache, meta, out, heads, 1, row, rank, shared_value=True, scale=0.2, window=window, plan=plan)
            close(out, want, dtype)
    written = ~torch.isnan(ref_cache.float())
    assert torch.equal(written, ~torch.isnan(cache.float()))
    close(cache.float()[written], ref_cache.float()[written], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,softcap,temp,bias", [
    (4, 2, 32, 48, 16, 6.0, (0.3, 5), True), (6, 6, 16, 16, 8, 0.0, (0.5, 1), True), (3, 1, 24, 8, 4, 2.5, None, False),
    (8, 2, 64, 64, 16, 0.0, None, True), (2, 1, 40, 24, 32, 30.0, (0.1, 64), False), (1, 1, 8, 8, 8, 1.0, (1.0, 3), True)])
def test_score_options(K, dtype, heads, kv_heads, dim, vdim, page, softcap, temp, bias):
    """A tanh cap, a distance bias per head, a query temperature and a gate per output number, in every combination the
    parameters give, on both attention kernels: two requests, portions beside single tokens."""
    lens = [90, 11]
    per = kv_heads * (dim + vdim)
    cache, table = paged(dtype, 2, lens, page, per, seed=dim)
    g = torch.Generator().manual_seed(dim)
    for b, n in enumerate(lens):
        kplane, vplane, _ = R.flat_planes(cache, kv_heads, dim, vdim, False)
        for j in range(n):
            pg, o = int(table[b, j // page]), j % page
            kplane[pg, :, o] = torch.randn(kv_heads, dim, generator=g).to(dtype)
            vplane[pg, :, o] = torch.randn(kv_heads, vdim, generator=g).to(dtype)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]).cuda() if bias else None
    RK = R.TorchKernels()
    for req, pos in (([0] * 40 + [1] * 11, list(range(0, 40)) + list(range(11))), ([0] * 2 + [1], [40, 41, 10]), ([0], [89]),
                     ([0] * 30, list(range(60, 90)))):
        T = len(req)
        q = rnd(T, heads * dim + 8, dtype=dtype, seed=T, s=1.5)
        gate = rnd(T, heads * vdim, seed=T + 1, s=2.0)
        meta = meta_for(table, req, pos)
        want = torch.empty(T, heads * vdim, dtype=torch.float32, device="cuda")
        RK.attention_flat(q, cache, meta, want, heads, kv_heads, dim, vdim, scale=0.4, gate=gate, softcap=softcap, slopes=slopes, q_temp=temp)
        out = torch.empty(T, heads * vdim, dtype=dtype, device="cuda")
        for plan in (None, flat_plan(K, req, pos, heads, kv_heads, dim, vdim, 0), flat_plan(K, req, pos, heads, kv_heads, dim, vdim, 0, splits=3)):
            out.fill_(float("nan"))
            K.attention_flat(q, cache, meta, out, heads, kv_heads, dim, vdim, scale=0.4, gate=gate, plan=plan, softcap=softcap,
                             slopes=slopes, q_temp=temp)
            close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("every,page", [(7, 4), (1, 8), (16, 16)])
def test_planted_scores_show_the_temperature_s_period_the_cap_and_the_distance(K, dtype, every, page):
    """One head, two kinds of keys: key 0 scores a against the query, all others 0, so that the weight of key 0 is
    1 / (1 + sum_j exp(-c(a m_p) + slope * p - slope * (p - j))) straight from the definition (m_p the temperature at position
    p, c the cap).  Asked at the positions around every multiple of `every`, where m_p steps, in a portion and one by one."""
    heads, dim, vdim, total, coef, cap, a = 1, 16, 8, 3 * every + 3, 0.75, 3.0, 2.0
    slope = 2.0 ** -8.0
    cache, table = paged(dtype, 1, [total], page, dim + vdim, seed=every)
    keys, vals = torch.zeros(total, 1, dim), torch.zeros(total, 1, vdim)
    keys[0, 0, 0], vals[0, 0, :] = a, 1.0
    fill_pages(cache, table, page, 1, dim, vdim, False, keys, vals)
    asked = sorted({p for m in (1, 2, 3) for p in (m * every - 2, m * every - 1, m * every) if 0 < p < total})
    want = []
    for p in asked:
        m = 1.0 + coef * math.log((p + 1) // every + 1.0)
        s0 = cap * math.tanh(a * m / cap) - slope * p
        rest = sum(math.exp(-slope * (p - j)) for j in range(1, p + 1))
        want.append(math.exp(s0) / (math.exp(s0) + rest))
    want = torch.tensor(want).cuda()
    slopes = torch.tensor([slope]).cuda()
    for rows in ([asked] if len(asked) < 2 else [asked, asked[:1], asked[-1:]]):
        q = torch.zeros(len(rows), dim, dtype=dtype, device="cuda")
        q[:, 0] = 1.0
        meta = meta_for(table, [0] * len(rows), rows)
        out = torch.empty(len(rows), vdim, dtype=dtype, device="cuda")
        w = want[[asked.index(p) for p in rows]]
        for plan in (None, flat_plan(K, [0] * len(rows), rows, heads, 1, dim, vdim, 0)):
            out.fill_(float("nan"))
            K.attention_flat(q, cache, meta, out, heads, 1, dim, vdim, scale=1.0, plan=plan, softcap=cap, slopes=slopes, q_temp=(coef, every))
            assert (out[:, 0].float() - w).abs().max() < (1e-5 if dtype == torch.float32 else 6e-3), (rows, out[:, 0], w)
    for p in (every - 1, 2 * every - 1):              # a period that is one position off would give another weight here
        if p in asked:
            m = 1.0 + coef * math.log(p // every + 1.0)
            s0 = cap * math.tanh(a * m / cap) - slope * p
            off = math.exp(s0) / (math.exp(s0) + sum(math.exp(-slope * (p - j)) for j in range(1, p + 1)))
            assert abs(off - want[asked.index(p)].item()) > 0.01
