"""A plain, slow restatement of the Fomerax family in float64 torch: one function per mechanism, whole sequences at
once, no cache, nothing carried between calls.  It shares no code with the engine: it reads config.json and the
checkpoint's tensors by their names.  The tests compare the engine with it.

Notation: x [T, w] is the residual stream of one sequence (positions 0 .. T-1), h a sub-layer's input.  A layer is

    x += norm1b(mixer(norm1(x)));   x += norm2b(ff(norm2(x)));   x += side_norm(side(x, token))      (the last if the
    model has a per-layer token input, the feed-forward if the layer has one)
"""
import json
import math
import os

import torch
from safetensors import safe_open


def read_model_dir(path):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(path, "model.safetensors"), "pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    return cfg, w


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def visible(T, size=0):
    """[T, T]: which keys j each query i sees: j <= i, and i - j < size when a window is given."""
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    ok = j <= i
    return ok & (i - j < size) if size else ok


def softmax_over_visible(s, ok):
    return torch.softmax(s.masked_fill(~ok, float("-inf")), dim=-1)


# ---- rotation -----------------------------------------------------------------------------------------------------
def yarn_frequencies(dims, base, scaling):
    """(frequencies [dims/2], amplitude): plain base^(-2i/dims), blended with their `factor`-th part along a ramp over
    the pair index, and the factor by which both sine and cosine grow."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(f, dtype=torch.float64), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_index(scaling["fast"])), 0)
    hi = min(math.ceil(turn_index(scaling["slow"])), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v, rot):
    """v [T, H, D]: the leading rot["dims"] numbers of each head rotate, neighbours (2i, 2i + 1) as a pair."""
    T, dims = v.shape[0], int(rot["dims"])
    freq, amp = yarn_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    a = torch.arange(T, dtype=torch.float64).view(T, 1, 1) * freq.view(1, 1, -1)
    c, s = torch.cos(a) * amp, torch.sin(a) * amp
    out = v.clone()
    even, odd = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = even * c - odd * s
    out[..., 1:dims:2] = odd * c + even * s
    return out


# ---- mixers -------------------------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps):
    """Queries through a normed low-rank row; keys and values of all heads from another; one rotated key part shared by
    the heads; a sliding window; the heads' outputs times a sigmoid gate, number by number."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], m["rot"])
    down = h @ w[p + "dkv"].T
    latent = rms_norm(down[:, :C], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, C:].reshape(T, 1, R), m["rot"])[:, 0]
    k_plain = (latent @ w[p + "uk"].T).view(T, H, D)
    v = (latent @ w[p + "uv"].T).view(T, H, V)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    size = int((m.get("mask") or {}).get("size", 0))
    pr = softmax_over_visible(s, visible(T, size))
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(T, H * V)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def biased_attention(h, w, p, m, eps):
    """Grouped heads, no rotation; the query grows with the logarithm of its position, the scores are squashed by a
    tanh and lose slope_h * distance; the heads' outputs times a sigmoid gate, number by number."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D).repeat_interleave(H // G, dim=1)
    v = (h @ w[p + "v"].T).view(T, G, V).repeat_interleave(H // G, dim=1)
    qt = m.get("q_temp")
    if qt:
        pos = torch.arange(T, dtype=torch.float64)
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((pos + 1) / qt["every"]) + 1.0)).view(T, 1, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    dist = (torch.arange(T).view(T, 1) - torch.arange(T).view(1, T)).double()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=torch.float64)
    s = s - slopes.view(H, 1, 1) * dist
    pr = softmax_over_visible(s, visible(T))
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(T, H * V)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h, w, p, mlp, chosen_out=None):
    """Every token goes to the `top` experts with the largest sigmoid of the router's outputs; an expert is fed the
    token's row times that sigmoid, and the experts' outputs are summed as they are."""
    r = mlp["router"]
    score = torch.sigmoid(h @ w[p + "router"].T)
    top = torch.topk(score, int(r["top"]), dim=-1)
    if chosen_out is not None:
        chosen_out.append(top.indices)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(top.indices[t].tolist(), top.values[t]):
            z = h[t] * s
            pe = f"{p}e{e}."
            out[t] += (silu(z @ w[pe + "gate"].T) * (z @ w[pe + "up"].T)) @ w[pe + "down"].T
    return out


def token_side(x, tokens, w, p, i, dim, eps):
    """The layer's own slice of a second embedding row of the token, gated by the stream, projected back and normed."""
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[p + "side.gate"].T) * e) @ w[p + "side.proj"].T
    return rms_norm(y, w[p + "side.norm"], eps)


# ---- the model -----------------------------------------------------------------------------------------------------
MIXERS = {"latent_attention": latent_attention, "attention": biased_attention}


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] (float64) of one sequence of token ids; `layers_out` (a list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens]
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(a, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            f = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp)
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        if side:
            x = x + token_side(x, tokens, w, p, i, int(side["dim"]), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T


def greedy(cfg, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]
