"""Tiny Mamusun configurations for the tests and a writer of random model folders for them.

The writer names the checkpoint's tensors itself (from the configuration alone), so the engine's mapping from its parameters
to tensor names is tested against it.  The configurations differ in everything a model of this family can vary: widths and
vocabularies that are no multiples of 8, the order of layers, head counts (grouped, ungrouped, one key/value head), key and
value sizes that differ, rotated parts that are all of a head or a few numbers of it, frequency laws with and without
scaling, windows (one token, shorter than a page, exactly a page, across pages, longer than the prompts, none), a borrowing
layer whose window is wider than the lender's, recurrences with one block or several and two to five taps, experts (one,
several chosen, all chosen), layers without a feed-forward, residual factors of 1 and other values.  The attention scales
are large on purpose: with a peaked softmax one key too many or too few moves the logits far beyond any tolerance.
"""
import json
import os

import torch
from safetensors.torch import save_file


def attention(heads, kv_heads, dim, vdim, scale, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def sink_attention(heads, kv_heads, dim, scale, rot_dims, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if scaling is not None:
        factor, original, fast, slow = scaling
        m["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return m


def parallel(heads, kv_heads, dim, vdim, scale, window, rot_dims, inner, blocks, taps, base=10000.0, scaling=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if window is not None:
        left["mask"] = {"size": window}
    if scaling is not None:
        factor, low, high, original = scaling
        left["rot"]["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return {"left": left, "right": {"width": inner, "blocks": blocks, "conv": taps}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, eps, alpha, layers):
    return {"architecture": "Mamusun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "postln_alpha": alpha, "layers": layers}


# every mixer once and a borrowing layer with the lender's window; a window shorter than a page and one across pages; two of
# five experts; a recurrence of three blocks and three taps
MAM_A = config(48, 150, 1e-5, 2.0, [
    layer("attention_2", sink_attention(4, 2, 16, 0.6, 8, base=500.0, scaling=(4.0, 32, 8.0, 1.0)), dense(40)),
    layer("attention", attention(4, 2, 8, 12, 0.8, window=10), moe(5, 2, 16, 1.5)),
    layer("parallel", parallel(2, 1, 16, 8, 0.7, 21, 6, 24, 3, 3, base=100.0, scaling=(4.0, 1.0, 4.0, 32)), dense(36)),
    layer("attention", attention(4, 2, 8, 12, 0.5, window=10, kv_from=1), None),
])
# a borrowing layer whose window is wider than the lender's (the cache keeps the wider one) and one that sees everything while
# the lender has a window; unscaled rotations; every expert chosen; one expert; one block, two taps; alpha 1
MAM_B = config(40, 77, 1e-6, 1.0, [
    layer("attention", attention(3, 3, 12, 20, 0.7, window=5), moe(3, 3, 24, 0.7)),
    layer("parallel", parallel(6, 1, 8, 8, 0.9, 16, 8, 40, 1, 2), moe(1, 1, 12, 2.0)),
    layer("attention", attention(6, 3, 12, 20, 0.6, window=23, kv_from=0), dense(33)),
    layer("attention_2", sink_attention(3, 3, 8, 0.9, 2), None),
    layer("attention", attention(3, 3, 12, 20, 0.5, kv_from=0), dense(24)),
])
# odd sizes, parallel layers only and first: a window of one token, then none at all; five taps; rotations of a whole head
MAM_C = config(36, 131, 2e-5, 3.5, [
    layer("parallel", parallel(3, 3, 4, 6, 1.1, 1, 4, 30, 5, 5, base=50.0), dense(20)),
    layer("parallel", parallel(4, 2, 8, 4, 0.8, None, 2, 12, 2, 4, scaling=(8.0, 1.0, 2.0, 16)), moe(4, 1, 8, 1.0)),
])
# sink attention first and last, a rotation of the whole head with a steep ramp; an attention without a window; a window of a page
MAM_D = config(64, 90, 1e-5, 0.5, [
    layer("attention_2", sink_attention(2, 1, 32, 0.4, 32, base=10000.0, scaling=(16.0, 64, 4.0, 2.0)), moe(2, 2, 8, 3.0)),
    layer("attention", attention(8, 4, 8, 8, 0.9), dense(48)),
    layer("attention", attention(2, 2, 16, 8, 0.6, window=4), None),
    layer("attention_2", sink_attention(5, 5, 8, 0.7, 4, base=20.0), dense(16)),
])

CONFIGS = {"A": (MAM_A, 41, 16), "B": (MAM_B, 42, 8), "C": (MAM_C, 43, 16), "D": (MAM_D, 44, 4)}      # config, seed, page size


def make_tensors(cfg, seed, std=0.08):
    """{checkpoint name: bfloat16 tensor}."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, s=std):
        return torch.randn(*shape, generator=g) * s

    w, t = cfg["width"], {}
    t["embed"], t["head"] = normal(cfg["vocab"], w, s=1.0), normal(cfg["vocab"], w, s=0.3)
    t["final.norm"] = normal(w, s=0.1)

    def heads_of(p, m, own=True, values=True):
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
        t[p + "q"] = normal(H * D, w, s=0.3)
        if own:
            t[p + "k"] = normal(G * D, w, s=0.3)
            if values:
                t[p + "v"] = normal(G * V, w, s=0.2)
        t[p + "o"] = normal(w, H * V, s=0.2)

    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}.mix."
        t[f"l{i}.norm1"] = normal(w, s=0.1)
        t[f"l{i}.dwa"] = torch.softmax(normal(i + 2, s=1.0), 0) * (1.0 + normal(i + 2, s=0.2))
        if lay["type"] == "attention":
            own = m.get("kv_from") is None
            heads_of(p, m, own=own)
            t[p + "q.norm"] = 1.0 + normal(m["dim"], s=0.2)
            if own:
                t[p + "k.norm"] = 1.0 + normal(m["dim"], s=0.2)
        elif lay["type"] == "attention_2":
            heads_of(p, m, values=False)
            H, G, D = m["heads"], m["kv_heads"], m["dim"]
            t[p + "q.b"], t[p + "k.b"] = normal(H * D, s=0.3), normal(G * D, s=0.3)
            t[p + "q.norm"], t[p + "k.norm"] = 1.0 + normal(H * D, s=0.2), 1.0 + normal(G * D, s=0.2)
            t[p + "sink"] = normal(H, s=1.5)
        else:
            heads_of(p + "left.", m["left"])
            r = m["right"]
            n, b, taps = r["width"], r["blocks"], r["conv"]
            q = p + "right."
            t[q + "y"], t[q + "y.b"], t[q + "x"], t[q + "x.b"] = normal(n, w, s=0.3), normal(n, s=0.3), normal(n, w, s=0.3), normal(n, s=0.3)
            t[q + "conv"], t[q + "conv.b"] = normal(n, taps, s=0.5), normal(n, s=0.2)
            t[q + "ra"], t[q + "ra.b"] = normal(b, n // b, n // b, s=0.5), normal(b, n // b, s=0.5)
            t[q + "ri"], t[q + "ri.b"] = normal(b, n // b, n // b, s=0.5), normal(b, n // b, s=0.5)
            t[q + "lam"] = normal(n, s=1.0) - 1.0
            t[q + "o"] = normal(w, n, s=0.3)
            t[p + "left.out"], t[p + "right.out"] = 1.0 + normal(w, s=0.2), 0.7 + normal(w, s=0.2)
        mlp = lay["mlp"]
        if mlp is None:
            continue
        t[f"l{i}.norm2"] = normal(w, s=0.1)
        q = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            t[q + "up"], t[q + "down"] = normal(ff, w, s=0.4), normal(w, ff, s=0.3)
            t[q + "act"] = torch.tensor([0.8, 0.5, 0.3, 0.1]) + normal(4, s=0.1)
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            t[q + "router"], t[q + "router.b"] = normal(r["experts"], w, s=0.5), normal(r["experts"], s=0.5)
            for e in range(r["experts"]):
                t[f"{q}e{e}.gate"], t[f"{q}e{e}.up"], t[f"{q}e{e}.down"] = normal(ff, w, s=0.4), normal(ff, w, s=0.4), normal(w, ff, s=0.3)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg, out_dir, seed, std=0.08, tensors=None):
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors or make_tensors(cfg, seed, std), os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir
