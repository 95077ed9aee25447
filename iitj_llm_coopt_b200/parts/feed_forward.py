"""Feed-forward parts.

`SwiGLU`: x -> (silu(x Wgate^T) * (x Wup^T)) Wdown^T, no bias (engine/model.py:210-211), with
gate and up stored as one [2*inner, width] matrix, gate rows first (engine/model.py:116).
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part, StepPlan


class SwiGLU(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        if spec.activation != "silu":
            raise ValueError(f"SwiGLU: activation {spec.activation!r} is not supported")
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner = spec.width, spec.inner
        self.gate_up = self.down = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {
            "gate_up": ParamSpec((2 * spec.inner, spec.width), pieces=(("gate", spec.inner), ("up", spec.inner))),
            "down": ParamSpec((spec.width, spec.inner)),
        }

    def forward(self, ctx, x):
        t = x.shape[0]
        act = ctx.buffer("ffn.act", (t, self.inner), self.dtype)
        self.k.linear(x, self.gate_up, act, swiglu=True)
        out = ctx.buffer("ffn.out", (t, self.width), self.dtype)
        return self.k.linear(act, self.down, out, defer=True)


class GLU(Part):
    """x -> (f(x Wgate^T) * (x Wup^T)) Wdown^T with f the spec's `activation`: "silu", or "gelu_tanh", the tanh form of
    gelu, f(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  The silu form runs as `SwiGLU` does (the activation in the
    product's epilogue); any other as one product and one activation kernel."""
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        if spec.activation not in kernels.GLU_ACTIVATIONS:
            raise ValueError(f"GLU: activation {spec.activation!r} is not known ({', '.join(kernels.GLU_ACTIVATIONS)})")
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner, self.activation = spec.width, spec.inner, spec.activation
        self.gate_up = self.down = None

    parameters = SwiGLU.parameters

    def forward(self, ctx, x):
        t = x.shape[0]
        act = ctx.buffer("ffn.act", (t, self.inner), self.dtype)
        if self.activation == "silu":
            self.k.linear(x, self.gate_up, act, swiglu=True)
        else:
            gu = ctx.buffer("ffn.gate_up", (t, 2 * self.inner), self.dtype)
            self.k.linear(x, self.gate_up, gu)
            self.k.glu_act(gu, act, self.activation)
        out = ctx.buffer("ffn.out", (t, self.width), self.dtype)
        return self.k.linear(act, self.down, out)


class ClampedGLU(Part):
    """A gated feed-forward with clamped branches and a sigmoid gate of a given slope:

        g = min(x Wgate^T, limit),  u = clamp(x Wup^T, -limit, limit),  y = g * sigmoid(slope * g) * (u + 1),  out = y Wdown^T

    `limit` and `slope` are options of the spec; gate and up are stored as one [2*inner, width] matrix, gate rows first."""
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner = spec.width, spec.inner
        self.limit, self.slope = float(spec.option("limit", 0.0)), float(spec.option("slope", 1.0))
        self.gate_up = self.down = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {
            "gate_up": ParamSpec((2 * spec.inner, spec.width), pieces=(("gate", spec.inner), ("up", spec.inner))),
            "down": ParamSpec((spec.width, spec.inner)),
        }

    def forward(self, ctx, x):
        t = x.shape[0]
        gu = ctx.buffer("ffn.gate_up", (t, 2 * self.inner), self.dtype)
        self.k.linear(x, self.gate_up, gu)
        act = ctx.buffer("ffn.act", (t, self.inner), self.dtype)
        self.k.glu_clamped(gu, act, self.limit, self.slope)
        out = ctx.buffer("ffn.out", (t, self.width), self.dtype)
        return self.k.linear(act, self.down, out)


class PolyNormMLP(Part):
    """x -> act(x Wup^T) Wdown^T with a normed polynomial as activation: with N dividing a token's row of inner values by its root
    mean square (float32 statistics, the spec's option `eps`) and powers taken element by element,

        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,        (a, b, c, e) the four numbers of the parameter `act`."""
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner, self.eps = spec.width, spec.inner, float(spec.option("eps", 1e-6))
        self.up = self.down = self.act = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"up": ParamSpec((spec.inner, spec.width)), "down": ParamSpec((spec.width, spec.inner)),
                "act": ParamSpec((4,), kind="vector")}

    def load(self, tensors: dict) -> None:
        super().load(tensors)
        self.act = self.act.float().contiguous()

    def forward(self, ctx, x):
        t = x.shape[0]
        z = ctx.buffer("ffn.up", (t, self.inner), self.dtype)
        self.k.linear(x, self.up, z)
        act = ctx.buffer("ffn.act", (t, self.inner), self.dtype)
        self.k.poly_norm(z, self.act, self.eps, act)
        out = ctx.buffer("ffn.out", (t, self.width), self.dtype)
        return self.k.linear(act, self.down, out)


class RoutedGLU(Part):
    """A mixture of `experts` small ClampedGLU feed-forwards of which each token uses `experts_per_token`.

        z = x Wrouter^T  (float32),  s = softmax(z) over all router outputs,  chosen = the top entries of s + correction,
        out = sum over the chosen e of s[e] * expert_e(x)            (the weights are not renormalised)

    Options of the spec: `router` = "sigmoid" takes s = sigmoid(z) of every output by itself instead of the softmax;
    `router` = "chosen_softmax" compares the router outputs themselves and takes the softmax over the chosen ones alone as weights
    (they sum to one); `router_bias` = True adds a stored bias to the router outputs before anything else;
    `correction` = False: there is no stored correction and the choice is by s alone; `expert` = "silu" makes the
    experts plain silu-gated ones, silu(g) * u, instead of the clamped form; `weight_on` = "input" feeds expert e the row
    s[e] * x and sums the experts' outputs as they are, out = sum expert_e(s[e] * x) (the first product being linear in
    its row, the weight is applied to gate and up in that product's epilogue, or to the gathered rows).

    The last `identity` router outputs stand for experts without tensors that hand their input back (s[e] * x).
    Rows are sorted by expert on the device (`Kernels.moe_plan`), the experts' products run as one grouped product each
    (the first reads its rows through the sorted index, applies the gate in its epilogue), and the chosen experts'
    outputs of a token are added in the order of its choices, so a token's result does not depend on the batch.
    Nothing of that comes back to the host, so decode steps replay from CUDA graphs.  A step with many rows (a prompt
    portion; `Kernels.moe_dense_rows`) that is not being captured reads the experts' row counts once and runs each
    expert's rows, gathered side by side, through the dense product kernels, which are several times faster at that size."""
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner = spec.width, spec.inner
        self.experts, self.top = int(spec.experts), int(spec.experts_per_token)
        self.identity = int(spec.option("identity", 0))
        self.limit, self.slope = float(spec.option("limit", 0.0)), float(spec.option("slope", 1.0))
        self.sigmoid = spec.option("router", "softmax") == "sigmoid"
        self.chosen_softmax = spec.option("router", "softmax") == "chosen_softmax"
        self.has_router_bias = bool(spec.option("router_bias", False))
        if self.has_router_bias and not self.chosen_softmax:
            raise ValueError("routed feed-forward: a router bias goes with router = chosen_softmax")
        if self.chosen_softmax and spec.option("correction", True):
            raise ValueError("routed feed-forward: router = chosen_softmax has no correction (correction = False)")
        self.has_correction = bool(spec.option("correction", True))
        self.on_input = spec.option("weight_on", "output") == "input"
        self.silu = spec.option("expert", "clamped") == "silu"
        if spec.option("router", "softmax") not in ("softmax", "sigmoid", "chosen_softmax") or spec.option("weight_on", "output") not in ("input", "output"):
            raise ValueError("routed feed-forward: router is softmax or sigmoid, weight_on is input or output")
        if self.on_input and (self.identity or not self.silu):
            raise ValueError("routed feed-forward: weights on the experts' inputs go with plain silu experts and no identity experts")
        if self.silu and not self.on_input:
            raise ValueError("routed feed-forward: plain silu experts are served with the weight on their input")
        self.router = self.correction = self.router_bias = self.expert_gate_up = self.expert_down = None
        self.prepare_key = f"routed_glu.{self.top}"          # layers with as many choices a token share the step's plan

    def _by_expert(self, tokens: int) -> bool:
        """Whether a step of `tokens` tokens runs its experts one by one on the dense product kernels."""
        dense_rows = getattr(self.k, "moe_dense_rows", 0)
        return bool(self.experts) and bool(dense_rows) and tokens * self.top >= dense_rows

    def prepare_step(self, shape):
        """A step that reads the experts' row counts on the host stays out of CUDA graphs."""
        if not self._by_expert(shape.num_tokens):
            return None
        plan = StepPlan()
        plan.capture = False
        return plan

    @classmethod
    def parameters(cls, spec) -> dict:
        e, ff, w = int(spec.experts), spec.inner, spec.width
        outputs = e + int(spec.option("identity", 0))
        out = {"router": ParamSpec((outputs, w))}
        if spec.option("correction", True):
            out["correction"] = ParamSpec((outputs,), kind="vector")
        if spec.option("router_bias", False):
            out["router_bias"] = ParamSpec((outputs,), kind="vector")
        if e:
            out["expert_gate_up"] = ParamSpec((e * 2 * ff, w), pieces=tuple(
                (f"e{j}.{name}", ff) for j in range(e) for name in ("gate", "up")))
            out["expert_down"] = ParamSpec((e * w, ff), pieces=tuple((f"e{j}.down", w) for j in range(e)))
        return out

    def load(self, tensors: dict) -> None:
        super().load(tensors)
        if self.has_correction:
            self.correction = self.correction.float().contiguous()
        if self.has_router_bias:
            self.router_bias = self.router_bias.float().contiguous()

    def forward(self, ctx, x):
        t = x.shape[0]
        scores = ctx.buffer("moe.scores", (t, self.experts + self.identity), torch.float32)
        self.k.linear(x, self.router, scores)
        chosen = ctx.buffer("moe.chosen", (t, self.top), torch.int32)
        weights = ctx.buffer("moe.weights", (t, self.top), torch.float32)
        if self.chosen_softmax:
            self.k.route_topk(scores, self.router_bias, chosen, weights, chosen_softmax=True)
        else:
            self.k.route_topk(scores, self.correction, chosen, weights, sigmoid=self.sigmoid)
        out = ctx.buffer("ffn.out", (t, self.width), self.dtype)
        plan = y = None
        if self.experts:
            rows = t * self.top
            w1 = self.expert_gate_up.view(self.experts, 2 * self.inner, self.width)
            w2 = self.expert_down.view(self.experts, self.width, self.inner)
            by_expert = self._by_expert(t) and not (x.is_cuda and torch.cuda.is_current_stream_capturing())
            counts = ctx.buffer("moe.counts", (self.experts,), torch.int32) if by_expert else None
            plan = self.k.moe_plan(chosen, self.experts, ctx.buffer("moe.source", (rows,), torch.int32),
                                   ctx.buffer("moe.place", (rows,), torch.int32),
                                   ctx.buffer("moe.tiles", (self.k.moe_tile_bound(rows, self.experts) + 1, 4), torch.int32),
                                   **({"counts": counts} if by_expert else {}),
                                   **({"weights": weights, "row_weight": ctx.buffer("moe.row_weight", (rows,), torch.float32)}
                                      if self.on_input else {}))
            act = ctx.buffer("moe.act", (rows, self.inner), self.dtype)
            y = ctx.buffer("moe.y", (rows, self.width), self.dtype)
            if by_expert:
                sizes = counts.tolist()                      # the one read of the host in this layer
                xs = self.k.gather_rows(x, plan, ctx.buffer("moe.rows", (rows, self.width), self.dtype), weighted=self.on_input)
                gu = ctx.buffer("moe.gate_up", (rows, 2 * self.inner), self.dtype)
                live, spans = 0, []
                for n in sizes:
                    spans.append((live, live + n))
                    live += n
                for e, (lo, hi) in enumerate(spans):
                    if hi > lo:
                        self.k.linear(xs[lo:hi], w1[e], gu[lo:hi])
                if live and self.silu:
                    self.k.glu_act(gu[:live], act[:live], "silu")
                elif live:
                    self.k.glu_clamped(gu[:live], act[:live], self.limit, self.slope)
                for e, (lo, hi) in enumerate(spans):
                    if hi > lo:
                        self.k.linear(act[lo:hi], w2[e], y[lo:hi])
            else:
                self.k.moe_linear(x, w1, act, plan, gather=True, glu="silu_weighted" if self.silu else True, limit=self.limit,
                                  slope=self.slope)
                self.k.moe_linear(act, w2, y, plan)
        return self.k.moe_combine(y, plan, chosen, None if self.on_input else weights, x, self.experts, out)
