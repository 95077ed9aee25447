"""Position encodings applied to queries and keys inside a mixer.

`RotaryEmbedding`: half-split rotation (engine/model.py:92-94, 199-200) with inverse
frequencies 1 / theta^(2i/d) and the optional llama3 scaling law (engine/model.py:68-82).
The frequencies are computed once in float32 on the host with the reference's formula; the
angle position * inv_freq and its sine and cosine are evaluated in float32 inside the
kernel for every token, so no table of max_position rows exists and none is rounded to
the model's type.

A scaling law of type "yarn" (factor, original, fast, slow) blends every pair's frequency f_i with f_i / factor along
a ramp over the pair index i: with turns(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turns(fast)), 0),
hi = min(ceil(turns(slow)), rotary_dim - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency becomes
f_i / factor * r_i + f_i * (1 - r_i), and sine and cosine are both multiplied by 0.1 ln(factor) + 1 (`rope_amplitude`).

`NoPosition` leaves queries and keys as they are and only stores keys and values.
"""
from __future__ import annotations

import math

import torch

from .base import Part


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """float32 [rotary_dim/2]; llama3 scaling as engine/model.py:71-82.  A scaling dict with a true "float64" entry has the
    frequencies (and the law, if it names one) worked out in double precision and rounded to float32 once, at the end."""
    dt = torch.float64 if scaling and scaling.get("float64") else torch.float32
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.int64).to(dt) / rotary_dim))
    if not scaling or scaling.get("rope_type", scaling.get("type")) != "llama3":
        return inv_freq.float()
    factor, lo, hi = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    old = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = old / lo, old / hi
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old / wavelen - lo) / (hi - lo)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled).float()


def yarn_frequencies(rotary_dim: int, theta: float, scaling: dict) -> torch.Tensor:
    """float32 [rotary_dim/2]: the blended frequencies of the "yarn" law (module text), computed in double precision."""
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns(t: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))

    lo = max(math.floor(turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns(float(scaling["slow"]))), rotary_dim - 1)
    out = []
    for i in range(rotary_dim // 2):
        f = theta ** (-2.0 * i / rotary_dim)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64).float()


def rope_amplitude(scaling: dict | None) -> float:
    """The factor on sine and cosine alike that a scaling law asks for (1 for none and for llama3)."""
    if scaling and scaling.get("type") == "yarn":
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


class RotaryEmbedding(Part):
    graph_safe = True
    takes_partial_sums = True     # encode_and_store adds the k-split parts of the qkv product as it reads them

    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k = spec, kernels
        self.head_dim, self.rotary_dim = spec.head_dim, spec.rotary_dim
        scaling = spec.scaling_dict()
        if scaling.get("type") == "yarn":
            self.inv_freq = yarn_frequencies(spec.rotary_dim, spec.theta, scaling).to(device)
        else:
            self.inv_freq = rope_inverse_frequencies(spec.rotary_dim, spec.theta, scaling).to(device)
        self.amplitude = rope_amplitude(scaling)

    def tables(self, ctx):
        """cos and sin of this step's positions, computed by the first layer that asks and shared by
        every layer with the same position spec."""
        key = ("rope", self.spec)
        tabs = ctx.shared.get(key)
        if tabs is None:
            half = self.rotary_dim // 2
            name = f"rope.{hash(self.spec) & 0xffffffff:x}"
            cos = ctx.buffer(name + ".cos", (ctx.num_tokens, half), torch.float32)
            sin = ctx.buffer(name + ".sin", (ctx.num_tokens, half), torch.float32)
            if self.amplitude != 1.0:
                tabs = ctx.shared[key] = self.k.rope_tables(ctx.positions, self.inv_freq, cos, sin, amplitude=self.amplitude)
            else:
                tabs = ctx.shared[key] = self.k.rope_tables(ctx.positions, self.inv_freq, cos, sin)
        return tabs

    def encode_and_store(self, ctx, qkv, cache_view, slots, heads, kv_heads):
        return self.k.rope_store(qkv, ctx.positions, self.inv_freq, slots, cache_view, heads, kv_heads,
                                 self.head_dim, self.rotary_dim, tables=self.tables(ctx) if self.rotary_dim else None)

    def decode_tables(self, ctx):
        """(cos, sin) for a mixer whose decode kernel rotates and stores by itself, or None if this encoding
        cannot be handed over like that (only part of the head is rotated)."""
        return self.tables(ctx) if self.rotary_dim == self.head_dim and self.amplitude == 1.0 else None


class NoPosition(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k, self.head_dim = spec, kernels, spec.head_dim

    def encode_and_store(self, ctx, qkv, cache_view, slots, heads, kv_heads):
        if slots is not None:
            self.k.rope_store(qkv, ctx.positions, None, slots, cache_view, heads, kv_heads, self.head_dim, 0)
