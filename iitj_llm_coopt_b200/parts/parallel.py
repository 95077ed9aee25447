"""`ParallelMixer`: two mixers side by side that read the same input; the result is the scaled sum of their outputs, each first
divided by its root mean square over the model width and multiplied by a gain vector of its own:

    out = scale * (rmsnorm(left(x)) * left_gain + rmsnorm(right(x)) * right_gain)            (float32 statistics and sum)

The two sides are mixers of any registered kind: their spec records are the options `left` and `right` of this part's spec.
The left side owns the layer's cache entry (`LayerCall.cache`), the right side the call's second entry (`LayerCall.state`), so a
paged attention and a recurrent mixer fit together.  The spec's `position` (if any) is the left side's.
"""
from __future__ import annotations

import dataclasses

import torch

from .base import ParamSpec, Part

SIDES = ("left", "right")


def _side_class(spec):
    from . import MIXERS
    if spec.kind not in MIXERS:
        raise KeyError(f"parallel mixer: mixer kind {spec.kind!r} is not registered; known: {', '.join(sorted(MIXERS))}")
    return MIXERS[spec.kind]


class ParallelMixer(Part):

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.eps, self.scale = spec.width, float(spec.option("eps", 1e-6)), float(spec.option("scale", 0.5))
        left, right = spec.option("left"), spec.option("right")
        self.left = _side_class(left)(left, kernels, dtype, position=position)
        self.right = _side_class(right)(right, kernels, dtype, position=None)
        self.left_gain = self.right_gain = None

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    @classmethod
    def parameters(cls, spec) -> dict:
        out = {"left_gain": ParamSpec((spec.width,), kind="vector"), "right_gain": ParamSpec((spec.width,), kind="vector")}
        for side in SIDES:
            sub = spec.option(side)
            for name, ps in _side_class(sub).parameters(sub).items():
                out[f"{side}_{name}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        left = spec.option("left")
        return _side_class(left).cache_need(left)

    @classmethod
    def state_need(cls, spec):
        right = spec.option("right")
        return _side_class(right).cache_need(right)

    def subparts(self) -> tuple:
        return (self.left, self.right) + tuple(self.left.subparts()) + tuple(self.right.subparts())

    def load(self, tensors: dict) -> None:
        per = {side: {} for side in SIDES}
        for name, t in tensors.items():
            if name in ("left_gain", "right_gain"):
                setattr(self, name, t.float().contiguous())
                continue
            side, _, rest = name.partition("_")
            per[side][rest] = t
        self.left.load(per["left"])
        self.right.load(per["right"])

    def forward(self, ctx, x, call):
        if call.state is None:
            raise ValueError("parallel mixer: the right side needs a cache entry of its own (LayerCall.state)")
        self.left.part_name, self.right.part_name = self.part_name + ".left", self.part_name + ".right"
        a = self.left.forward(ctx, x, call)
        b = self.right.forward(ctx, x, dataclasses.replace(call, cache=call.state, state=None))
        out = ctx.buffer("parallel.out", (x.shape[0], self.width), torch.float32)
        return self.k.branch_mean([a, b], [self.left_gain, self.right_gain], self.scale, self.eps, out)
