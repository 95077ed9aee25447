"""A plain, slow restatement of the Mamusun family in float64 torch: one function per mechanism, whole sequences at
once, no cache, nothing carried between calls.  It shares no code with the engine: it reads config.json and the
checkpoint's tensors by their names.  The tests compare the engine with it.

Notation: x [T, w] is what a layer reads of one sequence (positions 0 .. T-1).  A layer is

    x1 = norm1(alpha x + mixer(x));   X = norm2(alpha x1 + ff(x1))      (norms with gain 1 + w, no ff: X = x1)

and what the next layer reads is a weighted sum of the embedding and of every layer's X so far.
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


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def visible(T, size=0):
    """[T, T]: which keys j each query i sees: j <= i, and i - j < size when a window is given."""
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    ok = j <= i
    return ok & (i - j < size) if size else ok


# ---- rotations ----------------------------------------------------------------------------------------------------
def plain_frequencies(dims, base):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)


def stretched_frequencies(dims, base, sc):
    """Frequencies whose long wavelengths are stretched by `factor`, with a linear blend between the two bounds
    original/high and original/low of the wavelength; amplitude 1."""
    out = []
    for f in plain_frequencies(dims, base).tolist():
        lam = 2.0 * math.pi / f
        if lam < sc["original"] / sc["high"]:
            out.append(f)
        elif lam > sc["original"] / sc["low"]:
            out.append(f / sc["factor"])
        else:
            s = (sc["original"] / lam - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * f / sc["factor"] + s * f)
    return torch.tensor(out, dtype=torch.float64), 1.0


def ramped_frequencies(dims, base, sc):
    """Frequencies blended with their `factor`-th part along a ramp over the pair index, and the amplitude that sine and
    cosine both get."""
    def turns(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns(sc["fast"])), 0)
    hi = min(math.ceil(turns(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base).tolist()):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, freqs, amplitude, dims, neighbours):
    """x [T, heads, d]: the first `dims` numbers of every head turned by position * freqs; `neighbours` pairs (2i, 2i+1),
    else (i, i + dims/2)."""
    T = x.shape[0]
    ang = torch.arange(T, dtype=torch.float64).view(T, 1, 1) * freqs.view(1, 1, -1)
    c, s = torch.cos(ang) * amplitude, torch.sin(ang) * amplitude
    out = x.clone()
    if neighbours:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = u * c - v * s, v * c + u * s
    return out


# ---- attention ----------------------------------------------------------------------------------------------------
def attend(q, k, v, scale, ok, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv].  `sink` [H]: one more term exp(sink_h) in every row's
    denominator, with no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    outs = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        if sink is None:
            p = torch.softmax(s, dim=-1)
        else:
            full = torch.cat([s, sink[h].expand(T, 1)], dim=1)
            p = torch.softmax(full, dim=-1)[:, :T]
        outs.append(p @ v[:, g])
    return torch.cat(outs, dim=1)


def window_attention(h, w, pre, m, eps, borrowed=None):
    """The mixer "attention": head norms with one gain per head number, no rotation, a window.  Returns (output, (k, v)):
    a later layer that borrows reads the keys (normed) and values of this one."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w[pre + "q"].T).view(T, H, d), eps) * w[pre + "q.norm"]
    if borrowed is None:
        k = unit_rms((h @ w[pre + "k"].T).view(T, G, d), eps) * w[pre + "k.norm"]
        v = (h @ w[pre + "v"].T).view(T, G, dv)
    else:
        k, v = borrowed
    size = (m.get("mask") or {}).get("size", 0)
    return attend(q, k, v, m["scale"], visible(T, size)) @ w[pre + "o"].T, (k, v)


def rotated_window_attention(h, w, pre, m, eps):
    """The left half of "parallel": neighbours rotate, stretched frequencies, then a unit norm per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    f, amp = stretched_frequencies(rot["dims"], rot["base"], rot["scaling"]) if rot.get("scaling") else (plain_frequencies(rot["dims"], rot["base"]), 1.0)
    q = unit_rms(rotate((h @ w[pre + "q"].T).view(T, H, d), f, amp, rot["dims"], True), eps)
    k = unit_rms(rotate((h @ w[pre + "k"].T).view(T, G, d), f, amp, rot["dims"], True), eps)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    size = (m.get("mask") or {}).get("size", 0)
    return attend(q, k, v, m["scale"], visible(T, size)) @ w[pre + "o"].T


def sink_attention(h, w, pre, m, eps):
    """The mixer "attention_2": biases, a norm over the whole projection, halves rotate with ramped frequencies, values
    are the keys as projected, a sink in the softmax."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    rot = m["rot"]
    f, amp = ramped_frequencies(rot["dims"], rot["base"], rot["scaling"]) if rot.get("scaling") else (plain_frequencies(rot["dims"], rot["base"]), 1.0)
    q0 = h @ w[pre + "q"].T + w[pre + "q.b"]
    k0 = h @ w[pre + "k"].T + w[pre + "k.b"]
    q = rotate((unit_rms(q0, eps) * w[pre + "q.norm"]).view(T, H, d), f, amp, rot["dims"], False)
    k = rotate((unit_rms(k0, eps) * w[pre + "k.norm"]).view(T, G, d), f, amp, rot["dims"], False)
    size = (m.get("mask") or {}).get("size", 0)
    return attend(q, k, k0.view(T, G, d), m["scale"], visible(T, size), sink=w[pre + "sink"]) @ w[pre + "o"].T


# ---- the gated linear recurrence ---------------------------------------------------------------------------------
def causal_conv(z, taps, bias):
    """z [T, C], taps [C, n] (last column: the current token): c_t = bias + sum_j taps[:, j] z_(t - n + 1 + j)."""
    T, C = z.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=z.dtype), z], dim=0)
    out = bias.expand(T, C).clone()
    for j in range(n):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def gated_recurrence(h, w, pre, m):
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    u = causal_conv(h @ w[pre + "x"].T + w[pre + "x.b"], w[pre + "conv"], w[pre + "conv.b"])
    ub = u.view(T, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[pre + "ra"]) + w[pre + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[pre + "ri"]) + w[pre + "ri.b"]).reshape(T, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[pre + "lam"])
    a = torch.exp(log_a)
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(width, dtype=torch.float64)
    out = []
    for t in range(T):
        S = a[t] * S + b[t]
        out.append(S * y[t])
    return torch.stack(out) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    left = rotated_window_attention(h, w, pre + "left.", m["left"], eps)
    right = gated_recurrence(h, w, pre + "right.", m["right"])
    return 0.5 * (unit_rms(left, eps) * w[pre + "left.out"] + unit_rms(right, eps) * w[pre + "right.out"])


# ---- feed-forwards ------------------------------------------------------------------------------------------------
def poly_norm(z, coef, eps):
    a, b, c, e = coef.tolist()
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, w, pre, eps):
    return poly_norm(h @ w[pre + "up"].T, w[pre + "act"], eps) @ w[pre + "down"].T


def expert_ff(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def routed_ff(h, w, pre, mlp):
    top = mlp["router"]["top"]
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    p = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += p[t, j] * expert_ff(h[t:t + 1], w, f"{pre}e{int(idx[t, j])}.", mlp["expert"]["limit"])[0]
    return out


# ---- the model ----------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence (and, asked for, what every layer hands on: [layers, T, w])."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    history, kept, handed = [x], {}, []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            a, kept[i] = window_attention(x, w, pre + "mix.", m, eps, kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "attention_2":
            a = sink_attention(x, w, pre + "mix.", m, eps)
        elif layer["type"] == "parallel":
            a = parallel_mixer(x, w, pre + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = unit_rms(alpha * x + a, eps) * (1.0 + w[pre + "norm1"])
        mlp = layer.get("mlp")
        if mlp is not None:
            f = dense_ff(x, w, pre + "mlp.", eps) if mlp["kind"] == "dense" else routed_ff(x, w, pre + "mlp.", mlp)
            x = unit_rms(alpha * x + f, eps) * (1.0 + w[pre + "norm2"])
        history.append(x)
        x = sum(w[pre + "dwa"][j] * history[j] for j in range(i + 2))
        handed.append(x)
    logits = (unit_rms(x, eps) * (1.0 + w["final.norm"])) @ w["head"].T
    return (logits, torch.stack(handed)) if want_layers else logits


def greedy(cfg, w, prompt, n):
    """n tokens chosen by the largest logit, each fed back."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
