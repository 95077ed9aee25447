"""How the parts of one layer are wired.

An arrangement declares, in `PARTS`, the names of its parts and the family each is looked up in ("norm", "mixer",
"feed_forward": parts.FAMILIES); a `LayerSpec` holds one spec record per name, the model builder builds the parts and
hands them over as keywords.  At most one part of an arrangement is of family "mixer": it owns the layer's cache
entry.  `forward(ctx, residual, delta, call)` returns the new (residual, delta): the residual stream stays apart in
float32, and a sub-layer's output travels as a `delta` that the next norm adds into the residual before it normalises.

`BranchNormBlock` puts the norms on the sub-layers' outputs: the sub-layers read the residual stream itself (as the
engine's type), and  residual += mixer_norm(mixer(residual));  residual += feed_forward_norm(feed_forward(residual)).
Nothing is left over for the next layer, so its delta is None.

`PreNormBlock` (the reference's decoder layer, engine/model.py:192-211 and its fused form 230-253):

    x = mixer_norm(residual += delta_in);        a = mixer(x)
    x = feed_forward_norm(residual += a);        delta_out = feed_forward(x)
"""
from __future__ import annotations

from ..kernels import materialize
from .base import delta_for


class Arrangement:
    PARTS: dict = {}             # part name -> family
    options: dict = {}           # the layer spec's constants of the arrangement itself (set by the model builder)

    def __init__(self, **parts):
        missing = [n for n in self.PARTS if n not in parts]
        extra = [n for n in parts if n not in self.PARTS]
        if missing or extra:
            raise TypeError(f"{type(self).__name__} is wired from {sorted(self.PARTS)}; missing {missing}, unexpected {extra}")
        self._parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)

    def parts(self) -> dict:
        return self._parts

    def all_parts(self) -> list:
        """The parts and the parts they own (a mixer's position encoding)."""
        out = []
        for p in self._parts.values():
            out.append(p)
            out.extend(getattr(p, "subparts", lambda: ())())
        return out

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.all_parts())

    def forward(self, ctx, residual, delta, call):
        raise NotImplementedError


class PreNormBlock(Arrangement):
    PARTS = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, residual, delta, call):
        x = self.mixer_norm.forward(ctx, residual, delta_for(self.mixer_norm, delta))
        a = self.mixer.forward(ctx, x, call)
        x = self.feed_forward_norm.forward(ctx, residual, delta_for(self.feed_forward_norm, a))
        return residual, self.feed_forward.forward(ctx, x)


class PreNormMixerBlock(Arrangement):
    """A layer without a feed-forward:  x = mixer_norm(residual += delta_in);  delta_out = mixer(x)."""
    PARTS = {"mixer_norm": "norm", "mixer": "mixer"}

    def forward(self, ctx, residual, delta, call):
        x = self.mixer_norm.forward(ctx, residual, delta_for(self.mixer_norm, delta))
        return residual, self.mixer.forward(ctx, x, call)


class BranchNormBlock(Arrangement):
    """Norms on the branches:  residual += mixer_norm(mixer(residual));  residual += feed_forward_norm(feed_forward(residual)).
    The sub-layers read the stream as the engine's type: in float32 that is the stream itself, in bfloat16 a rounded copy
    that the kernel which adds a normed branch writes on the way (`Kernels.norm_add`)."""
    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}
    CAST = "residual.cast"          # name of the rounded copy in the step's workspace and in `ctx.shared`

    def _stream(self, ctx, residual, delta):
        """(the stream with a pending delta of an earlier layer added, its copy of the engine's type)"""
        dtype = self.mixer.dtype
        if delta is not None:
            residual.add_(delta_for(None, delta))
            ctx.shared.pop(self.CAST, None)
        if dtype == residual.dtype:
            return residual
        x = ctx.shared.get(self.CAST)
        if x is None:
            x = ctx.buffer(self.CAST, tuple(residual.shape), dtype)
            x.copy_(residual)
            ctx.shared[self.CAST] = x
        return x

    def _add_branch(self, ctx, residual, branch, norm):
        dtype = self.mixer.dtype
        cast = None if dtype == residual.dtype else ctx.buffer(self.CAST, tuple(residual.shape), dtype)
        norm.k.norm_add(residual, materialize(branch), norm.weight, norm.eps, cast_out=cast)
        if cast is not None:
            ctx.shared[self.CAST] = cast
        return residual if cast is None else cast

    def forward(self, ctx, residual, delta, call):
        x = self._stream(ctx, residual, delta)
        x = self._add_branch(ctx, residual, self.mixer.forward(ctx, x, call), self.mixer_norm)
        self._add_branch(ctx, residual, self.feed_forward.forward(ctx, x), self.feed_forward_norm)
        return residual, None


class BranchNormMixerBlock(BranchNormBlock):
    """The same without a feed-forward."""
    PARTS = {"mixer": "mixer", "mixer_norm": "norm"}

    def forward(self, ctx, residual, delta, call):
        x = self._stream(ctx, residual, delta)
        self._add_branch(ctx, residual, self.mixer.forward(ctx, x, call), self.mixer_norm)
        return residual, None


class SandwichBlock(Arrangement):
    """Norms in front of and behind every sub-layer:

        residual += mixer_post_norm(mixer(mixer_norm(residual)))
        residual += feed_forward_post_norm(feed_forward(feed_forward_norm(residual)))
        residual += token_input(residual, token)            (arrangements with a "token_input" part)

    The kernel that adds a normed branch also norms the new row for the sub-layer that follows in the same layer
    (`Kernels.norm_add` with a second gain), and writes the copy of the engine's type that a token input's gate product
    reads.  A pending delta of an earlier layer is added first; nothing is left over for the next layer."""
    PARTS = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    CAST = BranchNormBlock.CAST

    def _last_add(self, ctx, residual, branch, norm):
        """residual += norm(branch), then the layer's token input (if it has one) on the new stream."""
        side = getattr(self, "token_input", None)
        cast = None
        if side is not None and self.mixer.dtype != residual.dtype:
            cast = ctx.buffer(self.CAST, tuple(residual.shape), self.mixer.dtype)
        norm.k.norm_add(residual, materialize(branch), norm.weight, norm.eps, cast_out=cast)
        ctx.shared.pop(self.CAST, None)
        if side is not None:
            side.forward(ctx, residual, residual if cast is None else cast)

    def _enter(self, ctx, residual, delta):
        if delta is not None:
            residual.add_(delta_for(None, delta))
            ctx.shared.pop(self.CAST, None)
        return self.mixer_norm.forward(ctx, residual, None)

    def forward(self, ctx, residual, delta, call):
        a = self.mixer.forward(ctx, self._enter(ctx, residual, delta), call)
        post, front = self.mixer_post_norm, self.feed_forward_norm
        x = ctx.buffer(f"norm.{front.part_name}.out", tuple(residual.shape), self.mixer.dtype)
        post.k.norm_add(residual, materialize(a), post.weight, post.eps, next_weight=front.weight, next_out=x)
        self._last_add(ctx, residual, self.feed_forward.forward(ctx, x), self.feed_forward_post_norm)
        return residual, None


class SandwichMixerBlock(SandwichBlock):
    """The same without a feed-forward."""
    PARTS = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm"}

    def forward(self, ctx, residual, delta, call):
        a = self.mixer.forward(ctx, self._enter(ctx, residual, delta), call)
        self._last_add(ctx, residual, a, self.mixer_post_norm)
        return residual, None


class SandwichSideBlock(SandwichBlock):
    PARTS = dict(SandwichBlock.PARTS, token_input="token_input")


class SandwichMixerSideBlock(SandwichMixerBlock):
    PARTS = dict(SandwichMixerBlock.PARTS, token_input="token_input")


class PostNormDepthBlock(Arrangement):
    """Norms behind the sums, a scaled residual, and a mix over depth at the layer's end:

        x1 = mixer_norm(alpha * x + mixer(x))
        X  = feed_forward_norm(alpha * x1 + feed_forward(x1))
        what the next layer reads = stream_mix over the embedding's output and every layer's X so far

    `alpha` is the arrangement's option.  The sub-layers read the stream as the engine's type (a rounded copy that the norm
    kernels write on the way); the stream, the sums and the norms are float32.  The last norm of the layer, the store of X in
    the step's history and the weighted sum over it are one kernel (`Kernels.post_norm`)."""
    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm",
             "stream_mix": "stream_mix"}
    CAST = BranchNormBlock.CAST

    def _enter(self, ctx, residual, delta):
        """(the float32 stream, its copy of the engine's type)"""
        if delta is not None:
            residual.add_(delta_for(None, delta))
            ctx.shared.pop(self.CAST, None)
        if self.mixer.dtype == residual.dtype:
            return residual, residual
        x = ctx.shared.get(self.CAST)
        if x is None:
            x = ctx.buffer(self.CAST, tuple(residual.shape), self.mixer.dtype)
            x.copy_(residual)
            ctx.shared[self.CAST] = x
        return residual, x

    def _mid_norm(self, ctx, x, branch, norm):
        """rmsnorm(alpha * x + branch) * gain as float32 and, beside it, as the engine's type."""
        typed = self.mixer.dtype != x.dtype
        out = ctx.buffer("postnorm.mid", tuple(x.shape), x.dtype)
        cast = ctx.buffer("postnorm.mid.cast", tuple(x.shape), self.mixer.dtype) if typed else None
        norm.k.post_norm(x, materialize(branch), float(self.options.get("alpha", 1.0)), norm.weight, norm.eps, out, cast_out=cast)
        return out, cast if typed else out

    def forward(self, ctx, residual, delta, call):
        stream, x = self._enter(ctx, residual, delta)
        hist = self.stream_mix.history(ctx, stream)             # X_0 is kept before the stream changes
        mid, mid_x = self._mid_norm(ctx, stream, self.mixer.forward(ctx, x, call), self.mixer_norm)
        ff = self.feed_forward.forward(ctx, mid_x)
        alpha = float(self.options.get("alpha", 1.0))
        typed = self.mixer.dtype != stream.dtype
        cast = ctx.buffer(self.CAST, tuple(stream.shape), self.mixer.dtype) if typed else None
        mix, norm = self.stream_mix, self.feed_forward_norm
        norm.k.post_norm(mid, materialize(ff), alpha, norm.weight, norm.eps, stream, cast_out=cast, history=hist[:mix.inputs], mix=mix.weight)
        if typed:
            ctx.shared[self.CAST] = cast
        return stream, None


class PostNormDepthMixerBlock(PostNormDepthBlock):
    """The same without a feed-forward: X = mixer_norm(alpha * x + mixer(x))."""
    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "stream_mix": "stream_mix"}

    def forward(self, ctx, residual, delta, call):
        stream, x = self._enter(ctx, residual, delta)
        hist = self.stream_mix.history(ctx, stream)
        branch = self.mixer.forward(ctx, x, call)
        typed = self.mixer.dtype != stream.dtype
        cast = ctx.buffer(self.CAST, tuple(stream.shape), self.mixer.dtype) if typed else None
        mix, norm = self.stream_mix, self.mixer_norm
        norm.k.post_norm(stream, materialize(branch), float(self.options.get("alpha", 1.0)), norm.weight, norm.eps, stream, cast_out=cast,
                         history=hist[:mix.inputs], mix=mix.weight)
        if typed:
            ctx.shared[self.CAST] = cast
        return stream, None
