"""A model family beside the Llama of the same layer sizes (`bench.py --family NAME --shape SIZE`).

Both models get the same width, inner width, head counts, head size, vocabulary and depth (eight layers), random
weights, and run through the same engine: one prompt of `prefill_tokens` tokens in one step, and decode steps of
`batch` requests with `context` tokens each in the cache, timed on the device with CUDA events (three or more
warm-up runs, a write of 256 MB between prefill runs so that nothing of the run before is left in L2; a decode step
reads more weights than L2 holds).  Then the family's own kernels alone, at the shapes they have in those steps,
each with the bytes it must move and the fraction of the copy bandwidth that is, beside the Llama kernels that do
the like work (rotation and cache store for the convolution kernel, prefill and decode attention).
"""
from __future__ import annotations

import statistics
import time
from types import SimpleNamespace


def _timed(fn, reps, warmup, flush=None):
    import torch
    times = []
    for it in range(warmup + reps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if flush is not None:
            flush.add_(1.0)          # runs just before the timed work, so the launch's way to the GPU is not in the time
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def _engine(config_dict, page, pool_tokens, max_seqs, step_tokens, graphs):
    from . import LLM
    from .config.registry import architecture_for
    typed = architecture_for(config_dict).config_class.from_dict(config_dict)
    return LLM(config=typed, random_seed=3, dtype="bfloat16", page_size=page, num_pages=-(-pool_tokens // page),
               max_num_seqs=max_seqs, max_num_batched_tokens=step_tokens, max_model_len=1 << 20, cuda_graphs=graphs)


def _model_runs(name, config_dict, vocab, batch, context, steps, warmup, prefill_tokens, flush):
    """Prefill ms, decode ms per step and kernel launches per decode step of one model."""
    import torch

    from . import StepEntry
    page = 16
    pool = batch * (context + steps + warmup + 16 + 2 * page) + prefill_tokens + 4 * page
    llm = _engine(config_dict, page, pool, max(batch, 8), max(prefill_tokens, batch), True)
    eng = llm.engine
    runner, cache, sampler, kernels = eng.runner, eng.cache, eng.sampler, eng.sampler.k
    for g in cache.groups:
        if g.storage is not None and g.storage.dtype == torch.bfloat16:
            g.storage.normal_(0.0, 0.5)
    gen = torch.Generator().manual_seed(0)

    def prefill():
        cache.admit("p")
        runner.step([StepEntry("p", toks, [prefill_tokens - 1])])
        cache.release("p")
    toks = torch.randint(0, vocab, (prefill_tokens,), generator=gen).tolist()
    prefill_ms = _timed(prefill, 5, warmup, flush)

    ids = [f"d{i}" for i in range(batch)]
    for r in ids:
        cache.admit(r)
        for upto in list(range(prefill_tokens, context, prefill_tokens)) + [context]:     # as portions would fill it: a windowed
            cache.ensure(r, upto)                                                        # group's pool holds windows, not contexts
            cache.advance(r, upto)
    first = torch.randint(0, vocab, (batch,), generator=gen).tolist()
    prev, launches = None, 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prime = 5                                   # a step's shape is captured into a graph at its fourth sighting
    for it in range(-prime, warmup + steps):
        if it == warmup:
            torch.cuda.synchronize()
            launches = kernels.launches
            start.record()
        entries = [StepEntry(r, [t], [0]) for r, t in zip(ids, first)] if prev is None else \
            [StepEntry(r, [0], [0], source_rows=[i]) for i, r in enumerate(ids)]
        logits = runner.step(entries, prev_ids=prev)
        out, _ = sampler._buffers(batch)
        kernels.sample(logits, None, None, out)
        prev = out
    end.record()
    torch.cuda.synchronize()
    decode_ms = start.elapsed_time(end) / steps
    launches = (kernels.launches - launches) / steps
    kernels.check_health()
    params = eng.runner.model.parameter_bytes()
    del llm, eng, runner, cache
    torch.cuda.empty_cache()
    return {"model": name, "prefill_tokens": prefill_tokens, "prefill_ms": prefill_ms,
            "prefill_tok_s": prefill_tokens / (prefill_ms / 1e3), "decode_batch": batch, "decode_context": context,
            "decode_ms_per_step": decode_ms, "decode_tok_s": batch / (decode_ms / 1e3), "launches_per_decode_step": launches,
            "parameter_bytes": params}


def _kernels_alone_lifusun(lif, llama, tokens, batch, context, hbm_gbs, flush):
    """The family's kernels (and Llama's like ones) alone at the shapes of a `tokens`-token prompt and of a decode
    step of `batch` requests: microseconds, bytes that must move, fraction of the copy bandwidth."""
    import torch

    from . import kernels as _k
    K = _k.load()
    dev, bf = "cuda", torch.bfloat16
    att = next(l["mixer"] for l in lif["layers"] if l["type"] == "attention" and l["mixer"].get("kv_from") is None)
    ret = next(l["mixer"] for l in lif["layers"] if l["type"] == "retention")
    H, G, D, V, taps, chunk = att["heads"], att["kv_heads"], att["dim"], att["vdim"], att["conv"], att["mask"]["size"]
    page = 16
    out = []

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    def record(name, us, nbytes, like=None):
        out.append({"kernel": name, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                    "frac_of_copy_bandwidth": round(nbytes / (us * 1e-6) / (hbm_gbs * 1e9), 3), **({"like": like} if like else {})})

    for label, T, B, per in (("prefill", tokens, 1, tokens), ("decode", batch, batch, 1)):
        ctx_len = per if label == "prefill" else context
        pages_per = -(-ctx_len // page)
        cu, treq = [i * per for i in range(B + 1)], [b for b in range(B) for _ in range(per)]
        pos = [ctx_len - per + i for _ in range(B) for i in range(per)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        slots = [int(table[b, p // page]) * page + p % page for b, p in zip(treq, pos)]
        meta = SimpleNamespace(block_table=table, token_request=i32(treq), positions=i32(pos), query_lens=[per] * B,
                               seq_lens_host=[ctx_len] * B, attention_plan=None)
        # --- Lifusun: convolution + norms + cache store
        C = H * D + G * (D + V)
        u = torch.randn(T, C, device=dev).to(bf)
        cache = torch.randn(B * pages_per + 1, G * page * (D + V), device=dev).to(bf)
        q = torch.empty(T, H * D, device=dev, dtype=bf)
        state = torch.zeros(B + 1, taps - 1, C, device=dev)
        bias, tw = torch.randn(C, device=dev), torch.randn(C, taps, device=dev)
        qg, kg = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
        sl, tr, cs, ss = i32(slots), i32(treq), i32(cu), i32(list(range(B)))
        us = 1e3 * _timed(lambda: K.conv_norm_store(u, bias, tw, qg, kg, state, ss, tr, cs, q, cache, sl, H, G, D, V, 1e-6), 10, 3, flush)
        record(f"conv_norm_store ({label})", us, 2 * T * C * 2 + (B * (taps - 1) * C * 8 if label == "decode" else 0),
               like="llm_rope_store")
        # --- Llama: rotation + cache store on the same projection widths
        if D == V:
            qkv = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
            lcache = torch.zeros(B * pages_per + 1, 2, G, page, D, device=dev, dtype=bf)
            inv = (1.0 / 500000.0 ** (torch.arange(0, D, 2, device=dev).float() / D)).contiguous()
            posd = i32(pos)
            us = 1e3 * _timed(lambda: K.rope_store(qkv, posd, inv, sl, lcache, H, G, D, D), 10, 3, flush)
            record(f"llm_rope_store ({label})", us, T * (H + 2 * G) * D * 2 + T * (H + 2 * G) * D * 2)
        # --- Lifusun: talking attention
        talk = (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, device=dev)).contiguous()
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
        ao = torch.empty(T, H * V, device=dev, dtype=bf)
        keys = min(chunk, ctx_len)
        kv_read = (T if label == "decode" else -(-T // chunk)) * keys * G * (D + V) * 2
        us = 1e3 * _timed(lambda: K.talking_attention(q, cache, meta, talk, slopes, ao, H, G, D, V, chunk, D ** -0.5), 10, 3, flush)
        record(f"talking_attention, a token a block ({label})", us, T * H * (D + V) * 2 + kv_read, like="llama attention")
        if label == "prefill":
            tiles = i32([[r, min(16, T - r), pos[r], treq[r]] for r in range(0, T, 16)])
            us = 1e3 * _timed(lambda: K.talking_attention(q, cache, meta, talk, slopes, ao, H, G, D, V, chunk, D ** -0.5, tiles=tiles), 10, 3, flush)
            record(f"talking_attention, 16 tokens a block on the tensor core ({label})", us, T * H * (D + V) * 2 + kv_read, like="llama attention")
        # --- Llama: attention over the whole context
        if D == V:
            lq = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
            lo = torch.empty(T, H * D, device=dev, dtype=bf)
            lcache.normal_(0, 0.5)
            meta.attention_plan = None
            us = 1e3 * _timed(lambda: K.attention(lq, lcache, meta, lo, H, G, D), 10, 3, flush)
            rec = {"kernel": f"llama attention ({label})", "us": round(us, 2)}
            if label == "decode":
                nb = B * ctx_len * G * 2 * D * 2
                rec.update(mbytes=round(nb / 1e6, 2), frac_of_copy_bandwidth=round(nb / (us * 1e-6) / (hbm_gbs * 1e9), 3))
            else:
                rec.update(tflops=round(4 * (T * (T + 1) // 2) * H * D / (us * 1e-6) / 1e12, 1))
            out.append(rec)
        # --- Lifusun: retention scan and head norm with gate
        RH, RD, RV = ret["heads"], ret["dim"], ret["vdim"]
        cols = 2 * RH * (RD + RV)
        proj = torch.randn(T, cols, device=dev).to(bf)
        half = ret["rot"]["dims"] // 2
        ang = torch.tensor(pos, device=dev).float().unsqueeze(1) * (1.0 / 1e6 ** (torch.arange(half, device=dev).float() / half))
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        decay = torch.tensor(ret["decay"], device=dev)
        rstate = torch.zeros(B + 1, RH, RV, RD, device=dev)
        o = torch.empty(T, RH * RV, device=dev)
        us = 1e3 * _timed(lambda: K.retention(proj, (cos, sin), 2 * half, decay, rstate, ss, cs, o, RH, RD, RV, RD ** -0.5, longest=per), 10, 3, flush)
        record(f"retention_scan ({label})", us, T * RH * (2 * RD + RV) * 2 + T * RH * RV * 4 + 2 * B * RH * RD * RV * 4)
        gated = torch.empty(T, RH * RV, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.headnorm_gate(o, proj, 2 * RH * RD + RH * RV, gated, RH, RV, 1e-6), 10, 3, flush)
        record(f"headnorm_gate ({label})", us, T * RH * RV * (4 + 2 + 2))
    return out

def _kernels_alone_rodapel(cfg, llama, tokens, batch, context, hbm_gbs, flush):
    """Rodapel's kernels (and Llama's like ones) alone at the shapes of a `tokens`-token prompt and of a decode step of
    `batch` requests: microseconds, the bytes that must move and the fraction of the copy bandwidth that is, or for the
    arithmetic-bound prompt attention the TFLOP/s of the causal scores and sums."""
    import torch

    from . import kernels as _k
    K = _k.load()
    dev, bf = "cuda", torch.bfloat16
    att = next(l["mixer"] for l in cfg["layers"] if l["type"] == "attention")
    lat = next(l["mixer"] for l in cfg["layers"] if l["type"] == "latent_attention")
    rec = next(l["mixer"] for l in cfg["layers"] if l["type"] == "wkv")
    moe = next(l["mlp"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    width = cfg["width"]
    H, G, D, V, window = att["heads"], att["kv_heads"], att["dim"], att["vdim"], att["mask"]["size"]
    LH, LD, LR, LC = lat["heads"], lat["dim"], lat["rot_dim"], lat["kv_rank"]
    page = 16
    out = []

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    def record(name, us, nbytes=None, flops=None, like=None):
        r = {"kernel": name, "us": round(us, 2)}
        if nbytes is not None:
            r.update(mbytes=round(nbytes / 1e6, 2), frac_of_copy_bandwidth=round(nbytes / (us * 1e-6) / (hbm_gbs * 1e9), 3))
        if flops is not None:
            r.update(tflops=round(flops / (us * 1e-6) / 1e12, 1))
        if like:
            r["like"] = like
        out.append(r)

    for label, T, B, per in (("prefill", tokens, 1, tokens), ("decode", batch, batch, 1)):
        ctx_len = per if label == "prefill" else context
        pages_per = -(-ctx_len // page)
        cu, treq = [i * per for i in range(B + 1)], [b for b in range(B) for _ in range(per)]
        pos = [ctx_len - per + i for _ in range(B) for i in range(per)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        slots = i32([int(table[b, p // page]) * page + p % page for b, p in zip(treq, pos)])
        meta = SimpleNamespace(block_table=table, token_request=i32(treq), positions=i32(pos), query_lens=[per] * B,
                               seq_lens_host=[ctx_len] * B, attention_plan=None)
        from .parts.base import StepShape
        from .parts.flat_tiles import plan_flat_tiles

        def plan_for(heads, kv_heads, key_dim, value_dim, win, shared=False):
            plan = plan_flat_tiles(K, StepShape([per] * B, [ctx_len] * B, T, label == "decode", False, dev), heads, kv_heads,
                                   key_dim, value_dim, win, shared_value=shared)
            plan.bind({"tiles": i32(plan.arrays["tiles"])})
            return plan
        seen = sum(min(p + 1, window) for p in pos)                     # keys the windowed queries see, in all
        causal = sum(p + 1 for p in pos)
        # --- windowed attention: head norms + store, attention with the gate
        qkv = torch.randn(T, H * D + G * (D + V), device=dev).to(bf)
        cache = (torch.randn(B * pages_per + 1, G * page * (D + V), device=dev) * 0.5).to(bf)
        gain = torch.ones(D, device=dev)
        us = 1e3 * _timed(lambda: K.headnorm_store(qkv, gain, gain, 1e-6, cache, slots, H, G, D, V), 10, 3, flush)
        record(f"headnorm_store ({label})", us, nbytes=T * (2 * H * D + 2 * G * (D + V)) * 2, like="llm_rope_store")
        gate = torch.randn(T, H, device=dev)
        ao = torch.empty(T, H * V, device=dev, dtype=bf)
        wplan = plan_for(H, G, D, V, window)
        us = 1e3 * _timed(lambda: K.attention_flat(qkv, cache, meta, ao, H, G, D, V, window=window, scale=D ** -0.5, gate=gate, plan=wplan), 5, 3, flush)
        if label == "decode":
            record(f"attention_flat, window {window} ({label})", us, nbytes=B * min(ctx_len, window) * G * (D + V) * 2, like="llama attention")
        else:
            record(f"attention_flat, window {window} ({label})", us, flops=2 * seen * H * (D + V), like="llama attention")
        # --- Llama: rotation + store, attention over the whole context, the pre-norm
        if D == V:
            lqkv = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
            lcache = (torch.randn(B * pages_per + 1, 2, G, page, D, device=dev) * 0.5).to(bf)
            inv = (1.0 / 500000.0 ** (torch.arange(0, D, 2, device=dev).float() / D)).contiguous()
            posd = i32(pos)
            us = 1e3 * _timed(lambda: K.rope_store(lqkv, posd, inv, slots, lcache, H, G, D, D), 10, 3, flush)
            record(f"llm_rope_store ({label})", us, nbytes=T * (H + 2 * G) * D * 2 * 2)
            lo = torch.empty(T, H * D, device=dev, dtype=bf)
            meta.attention_plan = None
            us = 1e3 * _timed(lambda: K.attention(lqkv, lcache, meta, lo, H, G, D), 10, 3, flush)
            if label == "decode":
                record(f"llama attention ({label})", us, nbytes=B * ctx_len * G * 2 * D * 2)
            else:
                record(f"llama attention ({label})", us, flops=4 * causal * H * D)
        # --- latent attention: prepare + store, the absorbed queries, attention over the latent rows, the values' product
        row = LC + LR
        qd = torch.randn(T, LH * (LD + LR) + row, device=dev).to(bf)
        lat_cache = (torch.randn(B * pages_per + 1, page * row, device=dev) * 0.5).to(bf)
        ang = torch.tensor(pos, device=dev).float().unsqueeze(1) * (1.0 / 1e6 ** (torch.arange(LR // 2, device=dev).float() / (LR // 2)))
        tabs = (ang.cos().contiguous(), ang.sin().contiguous())
        lgain = torch.ones(LC, device=dev)
        qa = torch.empty(T, LH * row, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.latent_prepare(qd, tabs, LR, True, lgain, 1e-6, qa, lat_cache, slots, LH, LD, LR, LC), 10, 3, flush)
        record(f"latent_prepare ({label})", us, nbytes=T * (LH * (LD + 2 * LR) + 2 * row) * 2, like="llm_rope_store")
        uk = (torch.randn(LH, LC, LD, device=dev) * LD ** -0.5).to(bf)
        us = 1e3 * _timed(lambda: K.linear_by_group(qd, uk, qa, a_stride=LD + LR, out_stride=row), 10, 3, flush)
        record(f"absorbed queries, a product per head ({label})", us, nbytes=(T * LH * (LD + LC) + LH * LC * LD) * 2,
               flops=2 * T * LH * LD * LC)
        lo2 = torch.empty(T, LH * LC, device=dev, dtype=bf)
        lplan = plan_for(LH, 1, row, LC, 0, shared=True)
        us = 1e3 * _timed(lambda: K.attention_flat(qa, lat_cache, meta, lo2, LH, 1, row, LC, shared_value=True, scale=0.07, plan=lplan), 3, 3, flush)
        if label == "decode":
            record(f"attention_flat, latent rows ({label})", us, nbytes=B * ctx_len * row * 2, like="llama attention")
        else:
            record(f"attention_flat, latent rows ({label})", us, flops=2 * causal * LH * (row + LC), like="llama attention")
        # --- wkv: shift, decay, walk
        RH, RD = rec["heads"], rec["dim"]
        n = RH * RD
        x = torch.randn(T, width, device=dev).to(bf)
        mu = torch.rand(5 * width, device=dev)
        before = torch.zeros(B + 1, width, device=dev)
        ss, cs, tr = i32(list(range(B))), i32(cu), i32(treq)
        mixes = torch.empty(5 * T, width, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.token_shift(x, mu, before, ss, tr, cs, mixes), 10, 3, flush)
        record(f"token_shift ({label})", us, nbytes=T * width * 2 * 6)
        rkvg = torch.randn(4 * T, n, device=dev).to(bf)
        decay = torch.rand(T, n, device=dev) * 0.5 + 0.5
        u, g1 = torch.randn(RH, RD, device=dev) * 0.3, torch.ones(n, device=dev)
        state = torch.zeros(B + 1, RH, RD, RD, device=dev)
        wo = torch.empty(T, n, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.wkv_scan(rkvg, decay, u, g1, 1e-6, state, ss, cs, wo, RH, RD), 5, 3, flush)
        record(f"wkv_scan ({label})", us, nbytes=T * n * (4 * 2 + 4 + 2) + 2 * B * n * RD * 4, flops=4 * T * n * RD, like="retention_scan")
        # --- routed experts: choice, sort, the two grouped products, the weighted sum
        E, I, top, ff = moe["router"]["experts"], moe["router"]["identity"], moe["router"]["top"], moe["expert"]["ff"]
        scores = torch.randn(T, E + I, device=dev)
        corr = torch.zeros(E + I, device=dev)
        chosen = torch.empty(T, top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, top, device=dev)
        us = 1e3 * _timed(lambda: K.route_topk(scores, corr, chosen, wts), 10, 3, flush)
        record(f"route_topk ({label})", us)
        rows = T * top
        bufs = (torch.zeros(rows, dtype=torch.int32, device=dev), torch.zeros(rows, dtype=torch.int32, device=dev),
                torch.zeros(K.moe_tile_bound(rows, E) + 1, 4, dtype=torch.int32, device=dev))
        us = 1e3 * _timed(lambda: K.moe_plan(chosen, E, *bufs), 10, 3, flush)
        record(f"moe_plan ({label})", us)
        plan = K.moe_plan(chosen, E, *bufs)
        w1 = (torch.randn(E, 2 * ff, width, device=dev) * width ** -0.5).to(bf)
        w2 = (torch.randn(E, width, ff, device=dev) * ff ** -0.5).to(bf)
        act = torch.empty(rows, ff, device=dev, dtype=bf)
        y = torch.empty(rows, width, device=dev, dtype=bf)
        live = int(plan["tiles"][0, 1])
        us = 1e3 * _timed(lambda: K.moe_linear(x, w1, act, plan, gather=True, glu=True, limit=7.0, slope=1.702), 5, 3, flush)
        record(f"experts' gate/up product with the gate ({label})", us, nbytes=w1.numel() * 2 + live * (width + ff) * 2,
               flops=4 * live * ff * width, like="gate/up product (SwiGLU)")
        us = 1e3 * _timed(lambda: K.moe_linear(act, w2, y, plan), 5, 3, flush)
        record(f"experts' down product ({label})", us, nbytes=w2.numel() * 2 + live * (width + ff) * 2, flops=2 * live * ff * width,
               like="down product")
        mo = torch.empty(T, width, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.moe_combine(y, plan, chosen, wts, x, E, mo), 10, 3, flush)
        record(f"moe_combine ({label})", us, nbytes=(rows + 2 * T) * width * 2)
        # --- the dense products of Llama's feed-forward at the same width, for the experts' products to stand beside
        inner = llama["intermediate_size"]
        wg = (torch.randn(2 * inner, width, device=dev) * width ** -0.5).to(bf)
        a2 = torch.empty(T, inner, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.linear(x, wg, a2, swiglu=True), 5, 3, flush)
        record(f"gate/up product (SwiGLU) ({label})", us, nbytes=wg.numel() * 2 + T * (width + inner) * 2, flops=4 * T * inner * width)
        # --- the branch norm beside the pre-norm
        res = torch.randn(T, width, device=dev)
        branch = torch.randn(T, width, device=dev).to(bf)
        nw = torch.ones(width, device=dev)
        cast = torch.empty(T, width, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.norm_add(res, branch, nw, 1e-6, cast_out=cast), 10, 3, flush)
        record(f"norm_add ({label})", us, nbytes=T * width * (2 + 4 + 4 + 2), like="llm_add_rmsnorm")
        us = 1e3 * _timed(lambda: K.add_rmsnorm(res, branch, nw, 1e-6, cast), 10, 3, flush)
        record(f"llm_add_rmsnorm ({label})", us, nbytes=T * width * (2 + 4 + 4 + 2))
    return out


def _kernels_alone_fomerax(cfg, rod, tokens, batch, context, hbm_gbs, flush):
    """The kernels and kernel options that Fomerax brought, alone at the shapes of a `tokens`-token prompt and of a decode
    step of `batch` requests, each beside the like kernel as Rodapel runs it at the same shape (the same kernel without
    the option, mostly): microseconds, the bytes that must move and the fraction of the copy bandwidth that is, or for the
    arithmetic-bound prompt attention the TFLOP/s of the scores and sums."""
    import torch

    from . import kernels as _k
    from .parts.base import StepShape
    from .parts.flat_tiles import plan_flat_tiles
    K = _k.load()
    dev, bf = "cuda", torch.bfloat16
    att = next(l["mixer"] for l in cfg["layers"] if l["type"] == "attention")
    lat = next(l["mixer"] for l in cfg["layers"] if l["type"] == "latent_attention")
    moe = next(l["mlp"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    dense = next(l["mlp"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "dense")
    width, side = cfg["width"], cfg["token_side"]["dim"]
    H, G, D, V = att["heads"], att["kv_heads"], att["dim"], att["vdim"]
    LH, LD, LR, LC, LQ, LV, window = lat["heads"], lat["dim"], lat["rot_dim"], lat["kv_rank"], lat["q_rank"], lat["vdim"], lat["mask"]["size"]
    page = 16
    out = []

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    def record(name, us, nbytes=None, flops=None, like=None):
        r = {"kernel": name, "us": round(us, 2)}
        if nbytes is not None:
            r.update(mbytes=round(nbytes / 1e6, 2), frac_of_copy_bandwidth=round(nbytes / (us * 1e-6) / (hbm_gbs * 1e9), 3))
        if flops is not None:
            r.update(tflops=round(flops / (us * 1e-6) / 1e12, 1))
        if like:
            r["like"] = like
        out.append(r)

    for label, T, B, per in (("prefill", tokens, 1, tokens), ("decode", batch, batch, 1)):
        ctx_len = per if label == "prefill" else context
        pages_per = -(-ctx_len // page)
        treq = [b for b in range(B) for _ in range(per)]
        pos = [ctx_len - per + i for _ in range(B) for i in range(per)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        slots = i32([int(table[b, p // page]) * page + p % page for b, p in zip(treq, pos)])
        meta = SimpleNamespace(block_table=table, token_request=i32(treq), positions=i32(pos), query_lens=[per] * B,
                               seq_lens_host=[ctx_len] * B, attention_plan=None)

        def plan_for(heads, kv_heads, key_dim, value_dim, win, shared=False):
            plan = plan_flat_tiles(K, StepShape([per] * B, [ctx_len] * B, T, label == "decode", False, dev), heads, kv_heads,
                                   key_dim, value_dim, win, shared_value=shared)
            plan.bind({"tiles": i32(plan.arrays["tiles"])})
            return plan
        causal = sum(p + 1 for p in pos)
        seen = sum(min(p + 1, window) for p in pos)
        # --- biased attention over all earlier keys: cap, distance bias, temperature, a gate per output number; beside the plain
        #     scores with a gate per head
        qkv = torch.randn(T, H * D + G * (D + V), device=dev).to(bf)
        cache = (torch.randn(B * pages_per + 1, G * page * (D + V), device=dev) * 0.5).to(bf)
        ao = torch.empty(T, H * V, device=dev, dtype=bf)
        egate, hgate = torch.randn(T, H * V, device=dev), torch.randn(T, H, device=dev)
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
        plan = plan_for(H, G, D, V, 0)
        extras = dict(softcap=float(att.get("softcap") or 0.0), slopes=slopes,
                      q_temp=(att["q_temp"]["coef"], att["q_temp"]["every"]) if att.get("q_temp") else None)
        for name, kw, like in ((f"attention_flat, cap + bias + temperature + gate per number ({label})", dict(gate=egate, **extras), f"attention_flat, plain scores ({label})"),
                               (f"attention_flat, plain scores ({label})", dict(gate=hgate), None)):
            us = 1e3 * _timed(lambda: K.attention_flat(qkv, cache, meta, ao, H, G, D, V, scale=D ** -0.5, plan=plan, **kw), 5, 3, flush)
            if label == "decode":
                record(name, us, nbytes=B * ctx_len * G * (D + V) * 2, like=like)
            else:
                record(name, us, flops=2 * causal * H * (D + V), like=like)
        # --- latent attention: the queries' latent normed, the latent rows beside queries of another product, the window
        row = LC + LR
        down = torch.randn(T, LQ + row, device=dev).to(bf)
        cq = torch.empty(T, LQ, device=dev, dtype=bf)
        qgain = torch.ones(LQ, device=dev)
        us = 1e3 * _timed(lambda: K.rmsnorm_rows(down[:, :LQ], qgain, 1e-6, cq), 10, 3, flush)
        record(f"rmsnorm_rows, the queries' latent ({label})", us, nbytes=T * LQ * 2 * 2, like="norm_add")
        qd = torch.randn(T, LH * (LD + LR), device=dev).to(bf)
        qd_all = torch.randn(T, LH * (LD + LR) + row, device=dev).to(bf)
        lat_cache = (torch.randn(B * pages_per + 1, page * row, device=dev) * 0.5).to(bf)
        ang = torch.tensor(pos, device=dev).float().unsqueeze(1) * (1.0 / 1e4 ** (torch.arange(LR // 2, device=dev).float() / (LR // 2)))
        tabs = (ang.cos().contiguous(), ang.sin().contiguous())
        lgain = torch.ones(LC, device=dev)
        qa = torch.empty(T, LH * row, device=dev, dtype=bf)
        moved = T * (LH * (LD + 2 * LR) + 2 * row) * 2
        us = 1e3 * _timed(lambda: K.latent_prepare(qd, tabs, LR, True, lgain, 1e-6, qa, lat_cache, slots, LH, LD, LR, LC, kv=down[:, LQ:]), 10, 3, flush)
        record(f"latent_prepare, rows of another product ({label})", us, nbytes=moved, like=f"latent_prepare ({label})")
        us = 1e3 * _timed(lambda: K.latent_prepare(qd_all, tabs, LR, True, lgain, 1e-6, qa, lat_cache, slots, LH, LD, LR, LC), 10, 3, flush)
        record(f"latent_prepare ({label})", us, nbytes=moved)
        lo2 = torch.empty(T, LH * LC, device=dev, dtype=bf)
        for win, name, like in ((window, f"attention_flat, latent rows, window {window} ({label})", f"attention_flat, latent rows ({label})"),
                                (0, f"attention_flat, latent rows ({label})", None)):
            lplan = plan_for(LH, 1, row, LC, win, shared=True)
            us = 1e3 * _timed(lambda: K.attention_flat(qa, lat_cache, meta, lo2, LH, 1, row, LC, shared_value=True, scale=0.07, window=win, plan=lplan), 3, 3, flush)
            keys = seen if win else causal
            if label == "decode":
                record(name, us, nbytes=B * (min(ctx_len, win) if win else ctx_len) * row * 2, like=like)
            else:
                record(name, us, flops=2 * keys * LH * (row + LC), like=like)
        uv = (torch.randn(LH, LV, LC, device=dev) * LC ** -0.5).to(bf)
        vo = torch.empty(T, LH * LV, device=dev, dtype=bf)
        lgate = torch.randn(T, LH * LV, device=dev)
        nb = (T * LH * (LC + LV) + LH * LC * LV) * 2
        us = 1e3 * _timed(lambda: K.linear_by_group(lo2, uv, vo, a_stride=LC, out_stride=LV, out_gate=lgate), 10, 3, flush)
        record(f"values' product per head with the gate ({label})", us, nbytes=nb + T * LH * LV * 4, flops=2 * T * LH * LV * LC,
               like=f"values' product per head ({label})")
        us = 1e3 * _timed(lambda: K.linear_by_group(lo2, uv, vo, a_stride=LC, out_stride=LV), 10, 3, flush)
        record(f"values' product per head ({label})", us, nbytes=nb, flops=2 * T * LH * LV * LC)
        # --- norms on both sides: the branch norm that also norms the new row, beside the branch norm alone
        res = torch.randn(T, width, device=dev)
        branch = torch.randn(T, width, device=dev).to(bf)
        nw = torch.ones(width, device=dev)
        cast, nxt = torch.empty(T, width, device=dev, dtype=bf), torch.empty(T, width, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.norm_add(res, branch, nw, 1e-6, next_weight=nw, next_out=nxt), 10, 3, flush)
        record(f"norm_add with the next norm ({label})", us, nbytes=T * width * (2 + 4 + 4 + 2), like=f"norm_add ({label})")
        us = 1e3 * _timed(lambda: K.norm_add(res, branch, nw, 1e-6, cast_out=cast), 10, 3, flush)
        record(f"norm_add ({label})", us, nbytes=T * width * (2 + 4 + 4 + 2))
        # --- the token input's gate
        z = torch.randn(T, side, device=dev).to(bf)
        n_layers = len(cfg["layers"])
        stable = torch.randn(4096, n_layers * side, device=dev).to(bf)
        ids = torch.randint(0, 4096, (T,), dtype=torch.int32, device=dev)
        g = torch.empty(T, side, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.token_side_gate(z, stable, ids, side, g), 10, 3, flush)
        record(f"token_side_gate ({label})", us, nbytes=T * side * 2 * 3, like=f"glu_clamped ({label})")
        # --- the dense feed-forward's activation, beside the clamped one
        inner = dense["ff"]
        gu = torch.randn(T, 2 * inner, device=dev).to(bf)
        act = torch.empty(T, inner, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.glu_act(gu, act, "gelu_tanh"), 10, 3, flush)
        record(f"glu_act gelu_tanh ({label})", us, nbytes=T * inner * 2 * 3, like=f"glu_clamped ({label})")
        us = 1e3 * _timed(lambda: K.glu_clamped(gu, act, 7.0, 1.702), 10, 3, flush)
        record(f"glu_clamped ({label})", us, nbytes=T * inner * 2 * 3)
        x = torch.randn(T, width, device=dev).to(bf)
        wg = (torch.randn(2 * inner, width, device=dev) * width ** -0.5).to(bf)
        us = 1e3 * _timed(lambda: K.linear(x, wg, gu), 5, 3, flush)
        record(f"gate/up product ({label})", us, nbytes=wg.numel() * 2 + T * (width + 2 * inner) * 2, flops=4 * T * inner * width)
        # --- routed experts: choice by sigmoid, the plan with row weights, the first product with weighted silu, the plain sum
        E, top, ff = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]
        scores = torch.randn(T, E, device=dev)
        corr = torch.zeros(E, device=dev)
        chosen = torch.empty(T, top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, top, device=dev)
        us = 1e3 * _timed(lambda: K.route_topk(scores, None, chosen, wts, sigmoid=True), 10, 3, flush)
        record(f"route_topk, sigmoid ({label})", us, like=f"route_topk, softmax ({label})")
        us = 1e3 * _timed(lambda: K.route_topk(scores, corr, chosen, wts), 10, 3, flush)
        record(f"route_topk, softmax ({label})", us)
        K.route_topk(scores, None, chosen, wts, sigmoid=True)
        rows = T * top
        bufs = (torch.zeros(rows, dtype=torch.int32, device=dev), torch.zeros(rows, dtype=torch.int32, device=dev),
                torch.zeros(K.moe_tile_bound(rows, E) + 1, 4, dtype=torch.int32, device=dev))
        rw = torch.zeros(rows, device=dev)
        us = 1e3 * _timed(lambda: K.moe_plan(chosen, E, *bufs, weights=wts, row_weight=rw), 10, 3, flush)
        record(f"moe_plan with row weights ({label})", us, like=f"moe_plan ({label})")
        us = 1e3 * _timed(lambda: K.moe_plan(chosen, E, *bufs), 10, 3, flush)
        record(f"moe_plan ({label})", us)
        plan_w = K.moe_plan(chosen, E, *bufs, weights=wts, row_weight=rw)
        w1 = (torch.randn(E, 2 * ff, width, device=dev) * width ** -0.5).to(bf)
        w2 = (torch.randn(E, width, ff, device=dev) * ff ** -0.5).to(bf)
        eact = torch.empty(rows, ff, device=dev, dtype=bf)
        y = torch.empty(rows, width, device=dev, dtype=bf)
        live = int(plan_w["tiles"][0, 1])
        nb = w1.numel() * 2 + live * (width + ff) * 2
        us = 1e3 * _timed(lambda: K.moe_linear(x, w1, eact, plan_w, gather=True, glu="silu_weighted"), 5, 3, flush)
        record(f"experts' gate/up product, weighted silu ({label})", us, nbytes=nb, flops=4 * live * ff * width,
               like=f"experts' gate/up product, clamped gate ({label})")
        us = 1e3 * _timed(lambda: K.moe_linear(x, w1, eact, plan_w, gather=True, glu=True, limit=7.0, slope=1.702), 5, 3, flush)
        record(f"experts' gate/up product, clamped gate ({label})", us, nbytes=nb, flops=4 * live * ff * width)
        us = 1e3 * _timed(lambda: K.moe_linear(eact, w2, y, plan_w), 5, 3, flush)
        record(f"experts' down product ({label})", us, nbytes=w2.numel() * 2 + live * (width + ff) * 2, flops=2 * live * ff * width)
        mo = torch.empty(T, width, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.moe_combine(y, plan_w, chosen, None, x, E, mo), 10, 3, flush)
        record(f"moe_combine, plain sum ({label})", us, nbytes=(rows + T) * width * 2, like=f"moe_combine, weighted ({label})")
        us = 1e3 * _timed(lambda: K.moe_combine(y, plan_w, chosen, wts, x, E, mo), 10, 3, flush)
        record(f"moe_combine, weighted ({label})", us, nbytes=(rows + T) * width * 2)
    return out


def _kernels_alone_mamusun(cfg, rod, tokens, batch, context, hbm_gbs, flush):
    """The kernels and kernel options that Mamusun brought, alone at the shapes of a `tokens`-token prompt and of a decode step of
    `batch` requests, each beside the like kernel as Rodapel runs it at the same shape: microseconds, the bytes that must move and
    the fraction of the copy bandwidth that is, or for arithmetic-bound kernels the TFLOP/s."""
    import torch

    from . import kernels as _k
    from .parts.base import StepShape
    from .parts.flat_tiles import plan_flat_tiles
    K = _k.load()
    dev, bf = "cuda", torch.bfloat16
    sink = next(l["mixer"] for l in cfg["layers"] if l["type"] == "attention_2")
    att = next(l["mixer"] for l in cfg["layers"] if l["type"] == "attention")
    par = next(l["mixer"] for l in cfg["layers"] if l["type"] == "parallel")
    moe = next(l["mlp"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    dense = next(l["mlp"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "dense")
    width, n_layers = cfg["width"], len(cfg["layers"])
    H, G, D, window = att["heads"], att["kv_heads"], att["dim"], att["mask"]["size"]
    rot = par["left"]["rot"]["dims"]
    inner, blocks, taps = par["right"]["width"], par["right"]["blocks"], par["right"]["conv"]
    page = 16
    out = []

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    def record(name, us, nbytes=None, flops=None, like=None):
        r = {"kernel": name, "us": round(us, 2)}
        if nbytes is not None:
            r.update(mbytes=round(nbytes / 1e6, 2), frac_of_copy_bandwidth=round(nbytes / (us * 1e-6) / (hbm_gbs * 1e9), 3))
        if flops is not None:
            r.update(tflops=round(flops / (us * 1e-6) / 1e12, 1))
        if like:
            r["like"] = like
        out.append(r)

    for label, T, B, per in (("prefill", tokens, 1, tokens), ("decode", batch, batch, 1)):
        ctx_len = per if label == "prefill" else context
        pages_per = -(-ctx_len // page)
        treq = [b for b in range(B) for _ in range(per)]
        pos = [ctx_len - per + i for _ in range(B) for i in range(per)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        slots = i32([int(table[b, p // page]) * page + p % page for b, p in zip(treq, pos)])
        meta = SimpleNamespace(block_table=table, token_request=i32(treq), positions=i32(pos), query_lens=[per] * B,
                               seq_lens_host=[ctx_len] * B, attention_plan=None)

        def plan_for(win):
            plan = plan_flat_tiles(K, StepShape([per] * B, [ctx_len] * B, T, label == "decode", False, dev), H, G, D, D, win)
            plan.bind({"tiles": i32(plan.arrays["tiles"])})
            return plan
        causal = sum(p + 1 for p in pos)
        seen = sum(min(p + 1, window) for p in pos)
        # --- between the projection and the scores: the three forms beside the head norms with store
        cache = (torch.randn(B * pages_per + 1, G * page * 2 * D, device=dev) * 0.5).to(bf)
        qkv = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
        qk = torch.randn(T, (H + G) * D, device=dev).to(bf)
        gains_h = torch.ones(D, device=dev)
        gq, gk, bias = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev), torch.zeros((H + G) * D, device=dev)
        ang = torch.tensor(pos, device=dev).float().unsqueeze(1) * (1.0 / 1e4 ** (torch.arange(D // 2, device=dev).float() / (D // 2)))
        full = (ang.cos().contiguous(), ang.sin().contiguous())
        part = (full[0][:, :rot // 2].contiguous(), full[1][:, :rot // 2].contiguous())
        moved = T * ((2 * H + 2 * G) * D + G * D) * 2
        like = f"headnorm_store ({label})"
        us = 1e3 * _timed(lambda: K.qk_prepare(qk, H, G, D, D, 1e-6, cache_layer=cache, slots=slots, bias=bias, norm="row", q_gain=gq, k_gain=gk,
                                               tables=full, rotary_dim=D, value_from_key=True), 10, 3, flush)
        record(f"qk_prepare: bias, norm of the whole projection, halves rotate, keys as values ({label})", us, nbytes=moved, like=like)
        us = 1e3 * _timed(lambda: K.qk_prepare(qkv, H, G, D, D, 1e-6, cache_layer=cache, slots=slots, norm="head", norm_first=False, tables=part,
                                               rotary_dim=rot, interleaved=True), 10, 3, flush)
        record(f"qk_prepare: neighbours rotate, then unit head norms ({label})", us, nbytes=moved, like=like)
        us = 1e3 * _timed(lambda: K.qk_prepare(qkv[:, :H * D].contiguous(), H, G, D, D, 1e-6, norm="head", q_gain=gains_h, own_kv=False), 10, 3, flush)
        record(f"qk_prepare: head norms of queries alone ({label})", us, nbytes=T * 2 * H * D * 2, like=like)
        us = 1e3 * _timed(lambda: K.headnorm_store(qkv, gains_h, gains_h, 1e-6, cache, slots, H, G, D, D), 10, 3, flush)
        record(like, us, nbytes=moved)
        # --- the sink in the softmax, causal; the window beside it
        ao = torch.empty(T, H * D, device=dev, dtype=bf)
        sinks = torch.zeros(H, device=dev)
        for name, win, kw, lk in ((f"attention_flat with sinks ({label})", 0, dict(sinks=sinks), f"attention_flat, plain scores ({label})"),
                                  (f"attention_flat, plain scores ({label})", 0, {}, None),
                                  (f"attention_flat, window {window} ({label})", window, {}, None)):
            plan = plan_for(win)
            us = 1e3 * _timed(lambda: K.attention_flat(qkv, cache, meta, ao, H, G, D, D, scale=D ** -0.5, window=win, plan=plan, **kw), 5, 3, flush)
            if label == "decode":
                record(name, us, nbytes=B * (min(ctx_len, win) if win else ctx_len) * G * 2 * D * 2, like=lk)
            else:
                record(name, us, flops=2 * (seen if win else causal) * H * 2 * D, like=lk)
        # --- norms behind the sums, the average over depth, the mean of normed branches; beside the branch norm
        x = torch.randn(T, width, device=dev)
        branch = torch.randn(T, width, device=dev).to(bf)
        nw = torch.ones(width, device=dev)
        mid, cast = torch.empty(T, width, device=dev), torch.empty(T, width, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.post_norm(x, branch, 3.0, nw, 1e-6, mid, cast_out=cast), 10, 3, flush)
        record(f"post_norm ({label})", us, nbytes=T * width * (4 + 2 + 4 + 2), like=f"norm_add ({label})")
        hist = torch.randn(n_layers + 1, T, width, device=dev)
        mix = torch.ones(n_layers + 1, device=dev) / (n_layers + 1)
        us = 1e3 * _timed(lambda: K.post_norm(mid, branch, 3.0, nw, 1e-6, x, cast_out=cast, history=hist, mix=mix), 10, 3, flush)
        record(f"post_norm with the average over {n_layers + 1} entries ({label})", us, nbytes=T * width * (4 + 2 + 4 + 2 + 4 * (n_layers + 1)),
               like=f"norm_add ({label})")
        b2 = torch.randn(T, width, device=dev).to(bf)
        fo = torch.empty(T, width, device=dev)
        us = 1e3 * _timed(lambda: K.branch_mean([branch, b2], [nw, nw], 0.5, 1e-6, fo), 10, 3, flush)
        record(f"branch_mean of two ({label})", us, nbytes=T * width * (2 + 2 + 4), like=f"norm_add ({label})")
        us = 1e3 * _timed(lambda: K.norm_add(x, branch, nw, 1e-6, cast_out=cast), 10, 3, flush)
        record(f"norm_add ({label})", us, nbytes=T * width * (2 + 4 + 4 + 2))
        # --- the normed polynomial beside the clamped gate
        ff = dense["ff"]
        z = torch.randn(T, ff, device=dev).to(bf)
        act = torch.empty(T, ff, device=dev, dtype=bf)
        coef = torch.tensor([0.8, 0.5, 0.3, 0.1], device=dev)
        us = 1e3 * _timed(lambda: K.poly_norm(z, coef, 1e-6, act), 10, 3, flush)
        record(f"poly_norm ({label})", us, nbytes=T * ff * 2 * 2, like=f"glu_clamped ({label})")
        gu = torch.randn(T, 2 * ff, device=dev).to(bf)
        us = 1e3 * _timed(lambda: K.glu_clamped(gu, act, 7.0, 1.702), 10, 3, flush)
        record(f"glu_clamped ({label})", us, nbytes=T * ff * 2 * 3)
        # --- the gated recurrence with its convolution and gates, beside Rodapel's wkv walk
        side = inner // blocks
        proj = torch.randn(T, 2 * inner, device=dev).to(bf)
        vec = [torch.zeros(inner, device=dev) for _ in range(6)]
        tw = torch.randn(inner, taps, device=dev) * 0.5
        ra = (torch.randn(blocks, side, side, device=dev) * side ** -0.5).to(bf)
        ri = (torch.randn(blocks, side, side, device=dev) * side ** -0.5).to(bf)
        state = torch.zeros(B, taps, inner, device=dev)
        sl, cu = i32(list(range(B))), i32([per * b for b in range(B + 1)])
        lo = torch.empty(T, inner, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.lru(proj, 0, inner, inner, vec[0], vec[1], tw, vec[2], ra, ri, vec[3], vec[4], vec[5], 8.0, state, sl,
                                        i32(treq), cu, lo, longest=per), 5, 3, flush)
        record(f"lru: convolution, gates and recurrence ({label})", us, nbytes=T * inner * 6 + 2 * ra.numel() * 2 + B * taps * inner * 8,
               flops=4 * T * inner * side, like=f"wkv_scan ({label})")
        rmix = next(l["mixer"] for l in rod["layers"] if l["type"] == "wkv")
        rheads, rdim = rmix["heads"], rmix["dim"]
        rn = rheads * rdim
        rkvg = torch.randn(4 * T, rn, device=dev).to(bf)
        decay = torch.rand(T, rn, device=dev)
        wstate = torch.zeros(B, rheads, rdim, rdim, device=dev)
        wo = torch.empty(T, rn, device=dev, dtype=bf)
        us = 1e3 * _timed(lambda: K.wkv_scan(rkvg, decay, torch.zeros(rheads, rdim, device=dev), torch.ones(rn, device=dev), 1e-6, wstate, sl, cu, wo,
                                             rheads, rdim), 5, 3, flush)
        record(f"wkv_scan ({label})", us, nbytes=T * rn * (8 + 4 + 2) + B * rn * rdim * 8)
        # --- routing by a softmax over the chosen
        E, top = moe["router"]["experts"], moe["router"]["top"]
        scores, rb = torch.randn(T, E, device=dev), torch.zeros(E, device=dev)
        chosen, wts = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
        us = 1e3 * _timed(lambda: K.route_topk(scores, rb, chosen, wts, chosen_softmax=True), 10, 3, flush)
        record(f"route_topk, softmax over the chosen ({label})", us, like=f"route_topk, softmax ({label})")
        us = 1e3 * _timed(lambda: K.route_topk(scores, rb, chosen, wts), 10, 3, flush)
        record(f"route_topk, softmax ({label})", us)
    return out


def run(family, shape, steps, warmup, batch, context, prefill_tokens, peaks_and_source) -> dict:
    import torch

    from .presets import SHAPES
    peaks, source = peaks_and_source
    if shape not in ("8b", "3b", "1b", "toy"):
        raise SystemExit(f"--family {family}: --shape must be one of 8b, 3b, 1b, toy")
    _, lif = SHAPES[f"{family}-{shape}"]
    llama_name, llama = SHAPES[shape]
    llama = dict(llama, num_hidden_layers=len(lif["layers"]))
    flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")       # 256 MB: larger than L2
    t0 = time.time()
    rows = [_model_runs(f"{family}-{shape}", lif, lif["vocab"], batch, context, steps, warmup, prefill_tokens, flush)]
    beside = None
    if family in ("fomerax", "mamusun"):          # the closest family stands beside it too: windowed attention, a recurrence, routed experts
        _, beside = SHAPES[f"rodapel-{shape}"]
        rows.append(_model_runs(f"rodapel-{shape}", beside, beside["vocab"], batch, context, steps, warmup, prefill_tokens, flush))
    rows.append(_model_runs(f"{llama_name} cut to {len(lif['layers'])} layers", llama, llama["vocab_size"], batch, context, steps, warmup,
                            prefill_tokens, flush))
    alone = {"lifusun": _kernels_alone_lifusun, "rodapel": _kernels_alone_rodapel, "fomerax": _kernels_alone_fomerax,
             "mamusun": _kernels_alone_mamusun}[family](
        lif, beside if beside is not None else llama, prefill_tokens, batch, context, peaks["hbm_gbs"], flush)
    return {"family": family, "shape": shape, "dtype": "bf16", "data": "synthetic (random weights, random tokens)",
            "models": rows, "kernels_alone": alone, "copy_bandwidth_gbs": peaks["hbm_gbs"], "peaks": f"of {source}",
            "l2": "256 MB written between timed runs", "steps": steps, "warmup": warmup, "seconds": round(time.time() - t0, 1)}
