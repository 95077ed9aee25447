"""What a layer reads of the token itself, beside the stream.

`GatedTableInput` ("gated_table"): every token has a second embedding row, `table_width` wide, of which the layer owns the
columns [offset, offset + dim).  With e that slice of the token's row and x the stream after the layer's sub-layers:

    g = gelu_tanh(x Wgate^T) * e          Wgate [dim, width]
    y = g Wproj^T                         Wproj [width, dim]
    x += y * rsqrt(mean(y^2) + eps) * gain          (float32 statistics and sum)

The table belongs to the embedding part (kind "table_side"), which leaves it in `ctx.shared[SIDE_TABLE]` every step.
"""
from __future__ import annotations

from .base import ParamSpec, Part

SIDE_TABLE = "embedding.side_table"


class GatedTableInput(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.dim, self.offset, self.table_width, self.eps = spec.width, spec.dim, spec.offset, spec.table_width, spec.eps
        self.gate = self.proj = self.norm = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"gate": ParamSpec((spec.dim, spec.width)), "proj": ParamSpec((spec.width, spec.dim)),
                "norm": ParamSpec((spec.width,), kind="vector")}

    def forward(self, ctx, residual, x):
        """`x`: the stream as the engine's type (the residual itself in a float32 engine).  Adds into `residual`."""
        table = ctx.shared.get(SIDE_TABLE)
        if table is None or table.shape[1] != self.table_width:
            raise RuntimeError("token input: the model's embedding part holds no second table of the width this layer reads")
        t = x.shape[0]
        z = ctx.buffer("side.z", (t, self.dim), self.dtype)
        self.k.linear(x, self.gate, z)
        g = ctx.buffer("side.g", (t, self.dim), self.dtype)
        self.k.token_side_gate(z, table, ctx.token_ids, self.offset, g)
        y = ctx.buffer("side.y", (t, self.width), self.dtype)
        self.k.linear(g, self.proj, y)
        self.k.norm_add(residual, y, self.norm, self.eps)
        return residual
