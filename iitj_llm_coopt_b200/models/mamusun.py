"""Mamusun: layers whose norms sit behind the sums (x <- norm(alpha x + sub-layer(x)), gains stored around zero) and whose results
are mixed over depth (every layer hands on a weighted sum of the embedding and of all layers' results so far).  Three mixers:
grouped window attention with head norms and no rotation, which may read an earlier layer's keys and values; grouped causal
attention with biased projections, norms over the whole projection, a rotation of halves with ramped frequencies, the keys as
values and a sink in the softmax; and a window attention (neighbours rotate, unit head norms) side by side with a gated linear
recurrence behind a short convolution, their normed outputs averaged.  Feed-forwards: one matrix up and one down around a normed
polynomial, or routed clamped experts whose weights are the softmax over the chosen router outputs.

Checkpoint tensor names: embed, head, final.norm, and for layer i: l<i>.norm1, l<i>.norm2, l<i>.dwa, l<i>.mix.<name>,
l<i>.mlp.<name>.  Mixer tensors: q, k, v, o, q.b, k.b, q.norm, k.norm, sink; in a parallel layer left.{q,k,v,o,out} and
right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o,out}.  Feed-forward tensors: up, down, act; routed: router, router.b and
e<j>.{gate,up,down} for every expert j.
"""
from __future__ import annotations

import re

from ..config.mamusun import NAME, MamusunConfig
from ..config.registry import register_architecture
from .base import Architecture

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")

_ATTENTION = {            # (parameter, piece) -> what follows the mixer's prefix
    ("qkv", "q"): "q", ("qkv", "k"): "k", ("qkv", "v"): "v", ("qkv_bias", "q"): "q.b", ("qkv_bias", "k"): "k.b", ("qkv_bias", "v"): "v.b",
    ("q_norm", None): "q.norm", ("k_norm", None): "k.norm", ("sink", None): "sink", ("o", None): "o",
}
_RECURRENT = {
    ("yx", "y"): "y", ("yx", "x"): "x", ("yx_bias", "y"): "y.b", ("yx_bias", "x"): "x.b", ("conv", None): "conv",
    ("conv_bias", None): "conv.b", ("ra", None): "ra", ("ri", None): "ri", ("ra_bias", None): "ra.b", ("ri_bias", None): "ri.b",
    ("lam", None): "lam", ("o", None): "o",
}
_MIXER = dict(_ATTENTION)
_MIXER.update({("left_gain", None): "left.out", ("right_gain", None): "right.out"})
_MIXER.update({("left_" + p, piece): "left." + name for (p, piece), name in _ATTENTION.items()})
_MIXER.update({("right_" + p, piece): "right." + name for (p, piece), name in _RECURRENT.items()})
_IN_LAYER = {
    ("mixer_norm.weight", None): "norm1", ("feed_forward_norm.weight", None): "norm2", ("stream_mix.weight", None): "dwa",
    ("feed_forward.up", None): "mlp.up", ("feed_forward.down", None): "mlp.down", ("feed_forward.act", None): "mlp.act",
    ("feed_forward.router", None): "mlp.router", ("feed_forward.router_bias", None): "mlp.router.b",
}
_TOP = {"embedding.weight": "embed", "final_norm.weight": "final.norm", "lm_head.weight": "head"}
_EXPERT_PIECE = re.compile(r"^e(\d+)\.(gate|up|down)$")


class Mamusun(Architecture):
    name = NAME
    config_class = MamusunConfig

    def checkpoint_name(self, path: str, piece: str | None) -> str:
        if path in _TOP and piece is None:
            return _TOP[path]
        m = _LAYER.match(path)
        if m:
            rest = m.group(2)
            if (rest, piece) in _IN_LAYER:
                return f"l{m.group(1)}." + _IN_LAYER[(rest, piece)]
            if rest in ("feed_forward.expert_gate_up", "feed_forward.expert_down") and piece and _EXPERT_PIECE.match(piece):
                return f"l{m.group(1)}.mlp.{piece}"
            if rest.startswith("mixer.") and (rest[6:], piece) in _MIXER:
                return f"l{m.group(1)}.mix." + _MIXER[(rest[6:], piece)]
        raise KeyError(f"{NAME} has no checkpoint tensor for parameter {path!r} piece {piece!r}")


register_architecture(Mamusun())
