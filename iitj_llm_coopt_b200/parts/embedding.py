"""Token embedding and the output head.

`Embedding`: x = table[token_ids] (engine/model.py:191), written as the float32 residual stream.
`OutputHead`: logits = x . W^T in float32 (engine/model.py:215-218); W is the embedding table
when the model ties them (engine/model.py:106).
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part


class Embedding(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype=None):
        self.spec, self.vocab, self.width, self.k, self.scale = spec, spec.vocab, spec.width, kernels, spec.scale
        self.weight = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab, spec.width), kind="table")}

    def forward(self, ctx):
        out = ctx.buffer("residual", (ctx.num_tokens, self.width), torch.float32)
        return self.k.embed(ctx.token_ids, self.weight, out, self.scale)


class NormedEmbedding(Embedding):
    """x = rmsnorm(table[token_ids]) * norm: a norm with a gain per channel on the looked-up rows, statistics in
    float32 (`eps` among the spec's options).  In a bfloat16 engine the rounded copy of the stream that the first layer
    reads is written on the way (shared as BranchNormBlock.CAST)."""

    def __init__(self, spec, kernels, dtype=None):
        super().__init__(spec, kernels, dtype)
        self.eps = float(dict(spec.options).get("eps", 1e-6))
        self.dtype = dtype
        self.norm = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab, spec.width), kind="table"), "norm": ParamSpec((spec.width,), kind="vector")}

    def forward(self, ctx):
        raw = ctx.buffer("embedding.raw", (ctx.num_tokens, self.width), torch.float32)
        self.k.embed(ctx.token_ids, self.weight, raw, self.scale)
        out = ctx.buffer("residual", (ctx.num_tokens, self.width), torch.float32)
        cast = None
        if self.dtype is not None and self.dtype != torch.float32:
            cast = ctx.buffer("residual.cast", (ctx.num_tokens, self.width), self.dtype)
            ctx.shared["residual.cast"] = cast
        self.k.norm_add(out, raw, self.norm, self.eps, cast_out=cast, accumulate=False)
        return out


class SideTableEmbedding(Embedding):
    """x = table[token_ids], and a second table [vocab, side_width] (option `side_width`) whose rows the layers' token
    inputs read by the same ids: it is left in `ctx.shared` for them every step (parts/token_input.py)."""

    def __init__(self, spec, kernels, dtype=None):
        super().__init__(spec, kernels, dtype)
        self.side = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab, spec.width), kind="table"),
                "side": ParamSpec((spec.vocab, int(dict(spec.options)["side_width"])), kind="table")}

    def forward(self, ctx):
        from .token_input import SIDE_TABLE
        ctx.shared[SIDE_TABLE] = self.side
        return super().forward(ctx)


class OutputHead(Part):
    graph_safe = True

    tied_parameter = "weight"     # the parameter that is the embedding's table when the model ties them

    def __init__(self, spec, kernels, dtype=None):
        self.spec, self.vocab, self.width, self.k, self.scale = spec, spec.vocab, spec.width, kernels, spec.scale
        self.weight = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab, spec.width), kind="matrix")}

    def forward(self, ctx, x):
        logits = ctx.buffer("logits", (x.shape[0], self.vocab), torch.float32)
        self.k.linear(x, self.weight, logits)
        if self.scale != 1.0:
            self.k.scale_(logits, self.scale)
        return logits
