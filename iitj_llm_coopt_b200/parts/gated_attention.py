"""`GatedAttention`: grouped-query attention without a rotation, over a sliding window (or all earlier keys), with
optional norms on every query and key head and an optional gate on every head's output.

    [q, k, v] = x W^T                    (one product; no biases)
    q_h = rmsnorm(q_h) * q_gain,  k_g = rmsnorm(k_g) * k_gain        per head, one gain vector of head_dim for all heads (`qk_norm`)
    s   = scale * q_h . k_kv(h),   softmax over the keys j with 0 <= i - j < window (window 0: all j <= i)
    o_h = (P_h v_kv(h)) * sigmoid(x Wg^T)_h                          one gate number per head (`head_gate`)
    out = concat_h(o_h) Wo^T

Further options of the spec: `element_gate` puts a gate on every output number instead of one per head
(o = (P v) * sigmoid(x Wg^T), Wg [heads * value_dim, width]); `softcap` c > 0 squashes the scaled score to c tanh(s / c);
`bias_slope_exponent` b > 0 then takes slope_h * (i - j) off the score of query i and key j, slope_h = 2^(-b (h + 1) / heads);
`q_temp` = (coef, every) multiplies the query at position p by 1 + coef ln(floor((p + 1) / every) + 1) (folded into the
score's scale in float32).

Options that change what happens between the projection and the scores (any of them routes the layer through
`Kernels.qk_prepare`, one kernel per token row with every step in float32):
  `qk_norm`               True or "head": the gains above; "unit": every head divided by its root mean square, no gain; "row": all of q
                          at once (and all of k) divided by its root mean square, with gains of heads * head_dim (kv_heads * head_dim)
  `norm_after_rotation`   the norm follows the rotation instead of preceding it
  `bias`                  a bias on q and k (and v, where the layer has a v), added as the projection leaves the product
  `value_from_key`        no v projection: the values are the keys as projected (with their bias), before norm and rotation
  `sinks`                 one learned number per head whose exponential joins the softmax's denominator (no key, no value, no scale)
  `own_kv` False          the layer has no keys and values: the run order points its call at the entry of the layer it reads
                          (`call.write` false), whose window is `cache_window` (the widest of all readers; what the cache keeps)
  the spec's `position`   a rotation of the leading rotary_dim numbers of every head (the position part's tables of the step)

Value heads may be wider or narrower than key heads: a page of the cache is the key plane followed by the value plane
(`CacheNeed.value_dim`).  What the cache holds are the normed keys.  Norm statistics, scores, softmax and the gate are float32.
"""
from __future__ import annotations

import torch

from ..config.specs import CacheNeed
from .base import ParamSpec, Part
from .flat_tiles import flat_prepare_key, plan_flat_tiles


class GatedAttention(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.heads, self.kv_heads = spec.width, spec.heads, spec.kv_heads
        self.head_dim, self.value_dim = spec.head_dim, spec.value_dim or spec.head_dim
        if self.heads % self.kv_heads:
            raise ValueError(f"gated attention: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.window = int(spec.window)
        self.scale = spec.softmax_scale or self.head_dim ** -0.5
        norm = spec.option("qk_norm", False)
        self.norm_form = "head" if norm is True else (norm or "none")
        if self.norm_form not in ("none", "head", "unit", "row"):
            raise ValueError(f"gated attention: qk_norm {norm!r} is not known (head, unit, row)")
        self.qk_norm, self.head_gate = self.norm_form in ("head", "row"), bool(spec.option("head_gate", False))
        self.position = position
        self.rotary_dim = getattr(position, "rotary_dim", 0) if position is not None else 0
        self.interleaved = getattr(getattr(position, "spec", None), "pairing", "half") == "interleaved"
        self.norm_first = not bool(spec.option("norm_after_rotation", False))
        self.has_bias, self.value_from_key = bool(spec.option("bias", False)), bool(spec.option("value_from_key", False))
        self.has_sinks, self.own_kv = bool(spec.option("sinks", False)), bool(spec.option("own_kv", True))
        if self.value_from_key and (spec.value_dim or spec.head_dim) != spec.head_dim:
            raise ValueError("gated attention: values that are the keys have the keys' size")
        # the plain route (head norms with gains or none, then the store) stays on the kernel it always ran on
        self.prepared = (self.norm_form in ("unit", "row") or not self.norm_first or self.has_bias or self.value_from_key
                         or not self.own_kv or self.rotary_dim > 0)
        self.element_gate = bool(spec.option("element_gate", False))
        if self.head_gate and self.element_gate:
            raise ValueError("gated attention: one gate per head or one per output number, not both")
        self.softcap = float(spec.option("softcap", 0.0) or 0.0)
        self.q_temp = spec.option("q_temp", None)
        b = float(spec.option("bias_slope_exponent", 0.0) or 0.0)
        self.slope_values = [2.0 ** (-b * (h + 1) / self.heads) for h in range(self.heads)] if b > 0 else None
        self.slopes = None
        self.extras = {}        # score options handed to the attention kernel (none: a kernel set without them still serves)
        if self.softcap > 0:
            self.extras["softcap"] = self.softcap
        if self.q_temp:
            self.extras["q_temp"] = (float(self.q_temp[0]), int(self.q_temp[1]))
        self.eps = float(spec.option("eps", 1e-6))
        self.cols = sum(n for _, n in self._rows(spec))
        self.qkv = self.o = self.q_norm = self.k_norm = self.gate = self.qkv_bias = self.sink = None
        self.prepare_key = flat_prepare_key(self.heads, self.kv_heads, self.head_dim, self.value_dim, self.window)

    @staticmethod
    def _rows(spec) -> tuple:
        """The pieces of the fused projection: q, then k and v where the layer has them."""
        rows = (("q", spec.heads * spec.head_dim),)
        if spec.option("own_kv", True):
            rows += (("k", spec.kv_heads * spec.head_dim),)
            if not spec.option("value_from_key", False):
                rows += (("v", spec.kv_heads * (spec.value_dim or spec.head_dim)),)
        return rows

    @classmethod
    def parameters(cls, spec) -> dict:
        v = spec.value_dim or spec.head_dim
        rows = cls._rows(spec)
        out = {"qkv": ParamSpec((sum(n for _, n in rows), spec.width), pieces=rows),
               "o": ParamSpec((spec.width, spec.heads * v))}
        norm, own = spec.option("qk_norm", False), spec.option("own_kv", True)
        if norm is True or norm in ("head", "row"):
            out["q_norm"] = ParamSpec((spec.heads * spec.head_dim if norm == "row" else spec.head_dim,), kind="vector")
            if own:
                out["k_norm"] = ParamSpec((spec.kv_heads * spec.head_dim if norm == "row" else spec.head_dim,), kind="vector")
        if spec.option("bias", False):
            out["qkv_bias"] = ParamSpec((sum(n for _, n in rows),), kind="vector", pieces=rows)
        if spec.option("sinks", False):
            out["sink"] = ParamSpec((spec.heads,), kind="vector")
        if spec.option("head_gate", False):
            out["gate"] = ParamSpec((spec.heads, spec.width))
        if spec.option("element_gate", False):
            out["gate"] = ParamSpec((spec.heads * v, spec.width))
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        window = spec.option("cache_window", None)
        return CacheNeed(kind="paged_kv", kv_heads=spec.kv_heads, head_dim=spec.head_dim,
                         window=int(spec.window if window is None else window), value_dim=spec.value_dim or spec.head_dim)

    def subparts(self) -> tuple:
        return (self.position,) if self.position is not None else ()

    def prepare_step(self, shape):
        return plan_flat_tiles(self.k, shape, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.window)

    def load(self, tensors: dict) -> None:
        super().load(tensors)
        for name in ("q_norm", "k_norm", "qkv_bias", "sink"):     # they enter float32 arithmetic: kept in float32
            if getattr(self, name) is not None:
                setattr(self, name, getattr(self, name).float().contiguous())
        if self.has_sinks:
            self.extras["sinks"] = self.sink
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float32, device=self.qkv.device)
            self.extras["slopes"] = self.slopes

    def forward(self, ctx, x, call):
        t = x.shape[0]
        group, view = ctx.cache.view(call.cache)
        meta = ctx.group(group)
        qkv = ctx.buffer("gattn.qkv", (t, self.cols), self.dtype)
        self.k.linear(x, self.qkv, qkv)
        gate = None
        if self.head_gate or self.element_gate:
            gate = ctx.buffer("gattn.gate", (t, self.gate.shape[0]), torch.float32)
            self.k.linear(x, self.gate, gate)
        if call.write and not self.own_kv:
            raise ValueError("gated attention: a layer without keys and values of its own cannot write a cache entry")
        if self.prepared:
            self.k.qk_prepare(qkv, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.eps, cache_layer=view,
                              slots=meta.slots if call.write else None, bias=self.qkv_bias,
                              norm="head" if self.norm_form == "unit" else self.norm_form, q_gain=self.q_norm, k_gain=self.k_norm,
                              norm_first=self.norm_first, tables=self.position.tables(ctx) if self.rotary_dim else None,
                              rotary_dim=self.rotary_dim, interleaved=self.interleaved, own_kv=self.own_kv,
                              value_from_key=self.value_from_key)
        else:
            self.k.headnorm_store(qkv, self.q_norm, self.k_norm, self.eps, view, meta.slots if call.write else None,
                                  self.heads, self.kv_heads, self.head_dim, self.value_dim)
        attn = ctx.buffer("gattn.ctx", (t, self.heads * self.value_dim), self.dtype)
        self.k.attention_flat(qkv, view, meta, attn, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                              window=self.window, scale=self.scale, gate=gate, plan=ctx.prepared.get(self.prepare_key), **self.extras)
        out = ctx.buffer("attn.out", (t, self.width), self.dtype)
        return self.k.linear(attn, self.o, out)
