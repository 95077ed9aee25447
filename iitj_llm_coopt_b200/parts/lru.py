"""`GatedLRU`: a recurrent block with a gated linear recurrence per channel (the real-gated linear recurrent unit of Griffin).

    y = gelu_tanh(x Wy^T + by),      z = x Wx^T + bx                      two branches of `inner` channels, as one product
    u_t = conv_bias + sum_j taps[:, j] z_(t - n + 1 + j)                  a causal convolution per channel over n = `conv_taps` tokens
                                                                          (the last tap is the current token's; zeros before the first)
    r = sigmoid(Ra u + ra_bias),   i = sigmoid(Ri u + ri_bias)            Ra, Ri block-diagonal: `blocks` square matrices [out, in]
    a = exp(-decay_scale * r * softplus(lam)),   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) (i_t u_t)     S = 0 for a new request
    out = (S * y) Wo^T

The state is the layer's cache entry (kind "state", [conv_taps, inner] float32): row 0 is S, the other rows are the last
conv_taps - 1 rows of z.  The cache manager clears it when it admits a request, so a portion of a prompt simply continues from
what the slot holds.  The convolution, the gates, the decay and the recurrence are float32 in both engine types.
"""
from __future__ import annotations

from ..config.specs import CacheNeed
from .base import ParamSpec, Part

_FLOAT32 = ("yx_bias", "conv", "conv_bias", "ra_bias", "ri_bias", "lam")


class GatedLRU(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner = spec.width, int(spec.option("inner"))
        self.blocks, self.taps = int(spec.option("blocks")), int(spec.option("conv_taps"))
        self.decay_scale = float(spec.option("decay_scale", 8.0))
        if self.inner % self.blocks:
            raise ValueError(f"gated lru: {self.inner} channels are not a multiple of {self.blocks} blocks")
        self.yx = self.yx_bias = self.conv = self.conv_bias = self.ra = self.ri = self.ra_bias = self.ri_bias = self.lam = self.o = None

    @classmethod
    def parameters(cls, spec) -> dict:
        n, w, blocks, taps = int(spec.option("inner")), spec.width, int(spec.option("blocks")), int(spec.option("conv_taps"))
        side = n // blocks
        return {"yx": ParamSpec((2 * n, w), pieces=(("y", n), ("x", n))),
                "yx_bias": ParamSpec((2 * n,), kind="vector", pieces=(("y", n), ("x", n))),
                "conv": ParamSpec((n, taps), kind="vector"),
                "conv_bias": ParamSpec((n,), kind="vector"),
                "ra": ParamSpec((blocks, side, side)),
                "ri": ParamSpec((blocks, side, side)),
                "ra_bias": ParamSpec((blocks, side), kind="vector"),
                "ri_bias": ParamSpec((blocks, side), kind="vector"),
                "lam": ParamSpec((n,), kind="vector"),
                "o": ParamSpec((w, n))}

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(int(spec.option("conv_taps")), int(spec.option("inner"))), state_dtype="float32")

    def load(self, tensors: dict) -> None:
        for name, t in tensors.items():        # the small tensors enter float32 arithmetic: kept in float32
            setattr(self, name, t.float().contiguous() if name in _FLOAT32 else t)
        self.ra_bias, self.ri_bias = self.ra_bias.reshape(-1), self.ri_bias.reshape(-1)

    def forward(self, ctx, x, call):
        t = x.shape[0]
        _, state = ctx.cache.view(call.cache)
        proj = ctx.buffer("lru.proj", (t, 2 * self.inner), self.dtype)
        self.k.linear(x, self.yx, proj)
        gated = ctx.buffer("lru.gated", (t, self.inner), self.dtype)
        self.k.lru(proj, 0, self.inner, self.inner, self.yx_bias[:self.inner], self.yx_bias[self.inner:], self.conv, self.conv_bias,
                   self.ra, self.ri, self.ra_bias, self.ri_bias, self.lam, self.decay_scale, state, ctx.state_slots, ctx.token_request,
                   ctx.cu_seqlens, gated, longest=max(ctx.query_lens) if ctx.query_lens else 0, write=call.write)
        out = ctx.buffer("lru.out", (t, self.width), self.dtype)
        return self.k.linear(gated, self.o, out)
