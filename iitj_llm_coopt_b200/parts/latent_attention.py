"""`LatentAttention`: causal attention whose keys and values of all heads are rebuilt from one low-rank row per token.

    [q, d] = x [Wq; Wdkv]^T          q: heads x (head_dim unrotated + rot_dim rotated) numbers; d: kv_rank + rot_dim numbers
    c      = rmsnorm(d[:kv_rank]) * gain               the latent row (float32 statistics)
    kr     = rotate(d[kv_rank:])                       one rotated key part that every head shares
    k_h    = Wuk_h c,   v_h = Wuv_h c                  per head
    s      = scale * (q_h[:head_dim] . k_h + rotate(q_h[head_dim:]) . kr),   causal softmax,   out = concat_h(P_h v_h) Wo^T

Only [c, kr] is cached, one row of kv_rank + rot_dim numbers per token (`CacheNeed.shared_value`: the value is the row's
leading kv_rank numbers).  The products with Wuk and Wuv are moved to the query side: since q_h . (Wuk_h c) =
(Wuk_h^T q_h) . c, each head's query becomes a row of kv_rank + rot_dim numbers that is scored against the cached rows as
they lie, the weighted sum of the latent rows comes back per head, and Wuv_h is applied to that sum.  So nothing is rebuilt
per key, in prompts or in decoding, and the attention kernel sees `heads` query heads over one shared key/value head.

Options of the spec beyond those sizes: `q_rank` > 0 sends the queries through a latent row of their own,
q = Wuq (rmsnorm(Wdq x) * gain), with Wdq and Wdkv as one product; the spec's `window` > 0 lets position i see the keys j
with 0 <= i - j < window only (the cache then gives back the pages a window has passed); `gate` = "element" multiplies
the concatenated heads, before Wo, number by number with sigmoid(Wg x).

The rotation is the mixer's position part (its float32 cos/sin tables of the step); which numbers pair up is the position
spec's `pairing`.  Every size and constant comes from the spec (options kv_rank, rot_dim, eps).
"""
from __future__ import annotations

import torch

from ..config.specs import CacheNeed
from .base import ParamSpec, Part
from .flat_tiles import flat_prepare_key, plan_flat_tiles


class LatentAttention(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.heads, self.head_dim = spec.width, spec.heads, spec.head_dim
        self.value_dim = spec.value_dim or spec.head_dim
        self.rank, self.rot_dim = int(spec.option("kv_rank")), int(spec.option("rot_dim", 0))
        self.eps = float(spec.option("eps", 1e-6))
        self.scale = spec.softmax_scale or (self.head_dim + self.rot_dim) ** -0.5
        self.position = position                       # None: nothing is rotated
        self.rotary_dim = getattr(position, "rotary_dim", 0) if position is not None else 0
        self.interleaved = getattr(getattr(position, "spec", None), "pairing", "half") == "interleaved"
        self.q_width = self.heads * (self.head_dim + self.rot_dim)
        self.row = self.rank + self.rot_dim            # what the cache holds per token, and a head's absorbed query
        self.q_rank, self.window = int(spec.option("q_rank", 0)), int(spec.window)
        self.element_gate = spec.option("gate", "none") == "element"
        self.q_dkv = self.dkv_norm = self.uk = self.uv = self.o = self.uk_t = self.uv_g = None
        self.dq_dkv = self.dq_norm = self.uq = self.gate = None
        self.prepare_key = flat_prepare_key(self.heads, 1, self.row, self.rank, self.window)

    @classmethod
    def parameters(cls, spec) -> dict:
        rank, rot = int(spec.option("kv_rank")), int(spec.option("rot_dim", 0))
        q = spec.heads * (spec.head_dim + rot)
        v = spec.heads * (spec.value_dim or spec.head_dim)
        out = {"dkv_norm": ParamSpec((rank,), kind="vector"),
               "uk": ParamSpec((spec.heads * spec.head_dim, rank)),
               "uv": ParamSpec((v, rank)),
               "o": ParamSpec((spec.width, v))}
        q_rank = int(spec.option("q_rank", 0))
        if q_rank:
            out["dq_dkv"] = ParamSpec((q_rank + rank + rot, spec.width), pieces=(("dq", q_rank), ("dkv", rank + rot)))
            out["dq_norm"] = ParamSpec((q_rank,), kind="vector")
            out["uq"] = ParamSpec((q, q_rank))
        else:
            out["q_dkv"] = ParamSpec((q + rank + rot, spec.width), pieces=(("q", q), ("dkv", rank + rot)))
        if spec.option("gate", "none") == "element":
            out["gate"] = ParamSpec((v, spec.width))
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        rank, rot = int(spec.option("kv_rank")), int(spec.option("rot_dim", 0))
        return CacheNeed(kind="paged_kv", kv_heads=1, head_dim=rank + rot, value_dim=rank, shared_value=True,
                         window=int(spec.window))

    def subparts(self) -> tuple:
        return (self.position,) if self.position is not None else ()

    def prepare_step(self, shape):
        return plan_flat_tiles(self.k, shape, self.heads, 1, self.row, self.rank, self.window, shared_value=True)

    def load(self, tensors: dict) -> None:
        super().load(tensors)
        self.dkv_norm = self.dkv_norm.float().contiguous()
        if self.q_rank:
            self.dq_norm = self.dq_norm.float().contiguous()
        # per head, as the [n, k] operand of a product: Wuk_h^T [kv_rank, head_dim] and Wuv_h [value_dim, kv_rank]
        self.uk_t = self.uk.view(self.heads, self.head_dim, self.rank).transpose(1, 2).contiguous()
        self.uv_g = self.uv.view(self.heads, self.value_dim, self.rank)
        self.uk = None

    def forward(self, ctx, x, call):
        t = x.shape[0]
        group, view = ctx.cache.view(call.cache)
        meta = ctx.group(group)
        tables = self.position.tables(ctx) if self.rotary_dim else None
        q = ctx.buffer("lat.q", (t, self.heads * self.row), self.dtype)
        slots = meta.slots if call.write else None
        if self.q_rank:
            # both down-projections as one product; the queries' latent row normed, then projected up
            down = ctx.buffer("lat.down", (t, self.q_rank + self.row), self.dtype)
            self.k.linear(x, self.dq_dkv, down)
            cq = ctx.buffer("lat.cq", (t, self.q_rank), self.dtype)
            self.k.rmsnorm_rows(down[:, :self.q_rank], self.dq_norm, self.eps, cq)
            qd = ctx.buffer("lat.qd", (t, self.q_width), self.dtype)
            self.k.linear(cq, self.uq, qd)
            self.k.latent_prepare(qd, tables, self.rotary_dim, self.interleaved, self.dkv_norm, self.eps, q, view, slots,
                                  self.heads, self.head_dim, self.rot_dim, self.rank, kv=down[:, self.q_rank:])
        else:
            qd = ctx.buffer("lat.qd", (t, self.q_width + self.row), self.dtype)
            self.k.linear(x, self.q_dkv, qd)
            # latent norm, rotation of the shared key part, store; the queries' rotated parts land behind their absorbed parts
            self.k.latent_prepare(qd, tables, self.rotary_dim, self.interleaved, self.dkv_norm, self.eps, q, view, slots,
                                  self.heads, self.head_dim, self.rot_dim, self.rank)
        gate = None
        if self.element_gate:
            gate = ctx.buffer("lat.gate", (t, self.heads * self.value_dim), torch.float32)
            self.k.linear(x, self.gate, gate)
        self.k.linear_by_group(qd, self.uk_t, q, a_stride=self.head_dim + self.rot_dim, out_stride=self.row)
        lat = ctx.buffer("lat.ctx", (t, self.heads * self.rank), self.dtype)
        if self.window:
            self.k.attention_flat(q, view, meta, lat, self.heads, 1, self.row, self.rank, shared_value=True, scale=self.scale,
                                  window=self.window, plan=ctx.prepared.get(self.prepare_key))
        else:
            self.k.attention_flat(q, view, meta, lat, self.heads, 1, self.row, self.rank, shared_value=True, scale=self.scale,
                                  plan=ctx.prepared.get(self.prepare_key))
        attn = ctx.buffer("lat.v", (t, self.heads * self.value_dim), self.dtype)
        if gate is not None:       # the gate rides in the epilogue of the values' product
            self.k.linear_by_group(lat, self.uv_g, attn, a_stride=self.rank, out_stride=self.value_dim, out_gate=gate)
        else:
            self.k.linear_by_group(lat, self.uv_g, attn, a_stride=self.rank, out_stride=self.value_dim)
        out = ctx.buffer("attn.out", (t, self.width), self.dtype)
        return self.k.linear(attn, self.o, out)
