"""Parts that decide what a layer hands on to the next one, beside its own result.

`DepthAverage`: what goes on after layer i is a weighted sum over depth,  x = sum_j weight[j] * X_j,  j = 0 .. i + 1,  with X_0 the
embedding's output and X_(j+1) the result of layer j (`inputs` = i + 2 weights, a parameter of the layer).  The step keeps every X_j
of its tokens in one float32 buffer [total, T, w] (`history`); the sum itself rides in the kernel that makes the layer's last norm
(`Kernels.post_norm`), so the part only owns the weights and the buffer.
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part

HISTORY = "depth.history"


class DepthAverage(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inputs, self.total = spec.width, int(spec.inputs), int(spec.total)
        if not 2 <= self.inputs <= self.total:
            raise ValueError(f"depth average: {self.inputs} inputs of a history of {self.total}")
        self.weight = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((int(spec.inputs),), kind="vector")}

    def load(self, tensors: dict) -> None:
        self.weight = tensors["weight"].float().contiguous()

    def history(self, ctx, stream):
        """The step's history buffer.  The layer with two inputs is the first: what it reads is the embedding's output, X_0."""
        hist = ctx.buffer(HISTORY, (self.total, stream.shape[0], self.width), torch.float32)
        if self.inputs == 2:
            hist[0].copy_(stream)
        return hist
