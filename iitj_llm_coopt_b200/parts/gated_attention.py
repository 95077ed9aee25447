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
        self.qk_norm, self.head_gate = bool(spec.option("qk_norm", False)), bool(spec.option("head_gate", False))
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
        self.cols = self.heads * self.head_dim + self.kv_heads * (self.head_dim + self.value_dim)
        self.qkv = self.o = self.q_norm = self.k_norm = self.gate = None
        self.prepare_key = flat_prepare_key(self.heads, self.kv_heads, self.head_dim, self.value_dim, self.window)

    @classmethod
    def parameters(cls, spec) -> dict:
        v = spec.value_dim or spec.head_dim
        q, k = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        out = {"qkv": ParamSpec((q + k + spec.kv_heads * v, spec.width), pieces=(("q", q), ("k", k), ("v", spec.kv_heads * v))),
               "o": ParamSpec((spec.width, spec.heads * v))}
        if spec.option("qk_norm", False):
            out["q_norm"] = ParamSpec((spec.head_dim,), kind="vector")
            out["k_norm"] = ParamSpec((spec.head_dim,), kind="vector")
        if spec.option("head_gate", False):
            out["gate"] = ParamSpec((spec.heads, spec.width))
        if spec.option("element_gate", False):
            out["gate"] = ParamSpec((spec.heads * v, spec.width))
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="paged_kv", kv_heads=spec.kv_heads, head_dim=spec.head_dim, window=int(spec.window),
                         value_dim=spec.value_dim or spec.head_dim)

    def prepare_step(self, shape):
        return plan_flat_tiles(self.k, shape, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.window)

    def load(self, tensors: dict) -> None:
        super().load(tensors)
        if self.qk_norm:
            self.q_norm, self.k_norm = self.q_norm.float().contiguous(), self.k_norm.float().contiguous()
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
        self.k.headnorm_store(qkv, self.q_norm, self.k_norm, self.eps, view, meta.slots if call.write else None,
                              self.heads, self.kv_heads, self.head_dim, self.value_dim)
        attn = ctx.buffer("gattn.ctx", (t, self.heads * self.value_dim), self.dtype)
        self.k.attention_flat(qkv, view, meta, attn, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                              window=self.window, scale=self.scale, gate=gate, plan=ctx.prepared.get(self.prepare_key), **self.extras)
        out = ctx.buffer("attn.out", (t, self.width), self.dtype)
        return self.k.linear(attn, self.o, out)
