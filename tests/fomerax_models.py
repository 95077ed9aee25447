"""Tiny Fomerax configurations for the tests and a writer of random model folders for them.

The writer names the checkpoint's tensors itself (from the configuration alone), so the engine's mapping from its
parameters to tensor names is tested against it.  The configurations differ in everything a model of this family can
vary: widths and vocabularies that are no multiples of 8, the order of layers, head counts (grouped, ungrouped, one),
unrotated, rotated and value sizes of a latent head that all differ, latent rows narrower and wider than a head, windows
(one token, shorter than a page, exactly a page, across pages, longer than the prompts, none), frequency scaling or none,
query temperatures whose period is 1, a few tokens or longer than every prompt, tanh caps or none, experts (one, several
chosen, all chosen), layers without a feed-forward, models with and without the per-layer token input.  The attention
scales are large on purpose: with a peaked softmax one key too many or too few moves the logits far beyond any tolerance.
"""
import json
import os

import torch
from safetensors.torch import save_file


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, window=None, base=10000.0, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if scaling is not None:
        factor, original, fast, slow = scaling
        m["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, eps, layers, side=None):
    c = {"architecture": "Fomerax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    return c


# a window shorter than a page with scaled frequencies; two of five experts; a temperature period of a few tokens under a
# cap; a latent layer without feed-forward whose window is one token; ungrouped heads without cap or temperature
FOM_A = config(64, 150, 1e-5, [
    layer("latent_attention", latent(3, 12, 8, 20, 24, 20, 0.5, window=10, base=1000.0, scaling=(4.0, 16, 8.0, 1.0)), moe(5, 2, 20)),
    layer("attention", attention(4, 2, 16, 24, 0.6, softcap=6.0, q_temp=(0.3, 7)), dense(48)),
    layer("latent_attention", latent(2, 8, 16, 8, 40, 12, 0.4, window=1), None),
    layer("attention", attention(2, 2, 8, 8, 0.4), moe(3, 1, 16)),
], side=8)
# no token input; a latent layer that sees everything (no window, no scaling) with one head; six query heads on one
# key/value head, a period of one token; every expert chosen; one expert; a window across pages
FOM_B = config(96, 131, 1e-6, [
    layer("latent_attention", latent(1, 20, 12, 10, 16, 48, 0.45, base=50.0), moe(3, 3, 33)),
    layer("attention", attention(6, 1, 24, 16, 0.5, softcap=30.0, q_temp=(0.8, 1)), moe(1, 1, 24)),
    layer("latent_attention", latent(4, 8, 4, 12, 12, 8, 0.5, window=33, scaling=(16.0, 64, 4.0, 2.0)), dense(64)),
], side=None)
# odd sizes throughout, a token input of three columns, a window of exactly one page, a period longer than every prompt
FOM_C = config(40, 77, 2e-5, [
    layer("attention", attention(3, 3, 12, 20, 0.7, q_temp=(0.5, 1000)), dense(36)),
    layer("latent_attention", latent(5, 6, 6, 7, 10, 9, 0.6, window=16, base=300.0, scaling=(2.0, 8, 2.0, 0.5)), moe(4, 2, 12)),
    layer("attention", attention(8, 2, 8, 8, 0.9, softcap=2.0), None),
], side=3)
# latent layers only: a window longer than most prompts, then one of two tokens; the token input of one column
FOM_D = config(48, 90, 1e-5, [
    layer("latent_attention", latent(2, 16, 8, 24, 32, 16, 0.35, window=70), dense(40)),
    layer("latent_attention", latent(6, 8, 2, 4, 8, 24, 0.8, window=2, base=20.0), moe(2, 2, 8)),
], side=1)

CONFIGS = {"A": (FOM_A, 31, 16), "B": (FOM_B, 32, 8), "C": (FOM_C, 33, 16), "D": (FOM_D, 34, 4)}      # config, seed, page size


def make_tensors(cfg, seed, std=0.08):
    """{checkpoint name: bfloat16 tensor}."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, s=std):
        return torch.randn(*shape, generator=g) * s

    def gains(n):
        return 1.0 + normal(n, s=0.1)

    w, t = cfg["width"], {}
    n_layers = len(cfg["layers"])
    side = (cfg.get("token_side") or {}).get("dim", 0)
    t["embed"] = normal(cfg["vocab"], w, s=1.0)
    t["final.norm"] = gains(w)
    if side:
        t["side.embed"] = normal(cfg["vocab"], n_layers * side, s=1.0)
    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}.mix."
        t[f"l{i}.norm1"], t[f"l{i}.norm1b"] = gains(w), gains(w) * (0.5 + 0.1 * i)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if lay["type"] == "latent_attention":
            R, C, Q = m["rot_dim"], m["kv_rank"], m["q_rank"]
            t[p + "dq"], t[p + "dq.norm"] = normal(Q, w, s=0.25), gains(Q)
            t[p + "uq"] = normal(H * (D + R), Q, s=0.5)
            t[p + "dkv"], t[p + "dkv.norm"] = normal(C + R, w, s=0.25), gains(C)
            t[p + "uk"], t[p + "uv"] = normal(H * D, C, s=0.3), normal(H * V, C, s=0.2)
        else:
            G = m["kv_heads"]
            t[p + "q"], t[p + "k"], t[p + "v"] = normal(H * D, w, s=0.2), normal(G * D, w, s=0.2), normal(G * V, w)
        t[p + "g"] = normal(H * V, w, s=0.3)
        t[p + "o"] = normal(w, H * V)
        if side:
            q = f"l{i}.side."
            t[q + "gate"], t[q + "proj"], t[q + "norm"] = normal(side, w, s=0.3), normal(w, side, s=0.5), gains(w) * 0.4
        mlp = lay["mlp"]
        if mlp is None:
            continue
        t[f"l{i}.norm2"], t[f"l{i}.norm2b"] = gains(w) * 0.8, gains(w) * 0.6
        q = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            t[q + "gate"], t[q + "up"], t[q + "down"] = normal(ff, w, s=0.4), normal(ff, w, s=0.4), normal(w, ff)
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            t[q + "router"] = normal(r["experts"], w, s=0.5)
            for e in range(r["experts"]):
                t[f"{q}e{e}.gate"], t[f"{q}e{e}.up"], t[f"{q}e{e}.down"] = normal(ff, w, s=0.4), normal(ff, w, s=0.4), normal(w, ff)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg, out_dir, seed, std=0.08, tensors=None):
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors or make_tensors(cfg, seed, std), os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir
