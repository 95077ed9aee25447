"""Fomerax: layers of latent attention (queries through a normed low-rank row; one normed low-rank row and one rotated key
part per token serve every head as key and as value; a sliding window) and of grouped attention without rotation (a query
temperature that grows with the logarithm of the position, tanh-squashed scores, a distance bias per head), both with a
sigmoid gate on every output number; dense gelu-gated or routed silu-gated feed-forwards; norms before and after every
sub-layer; a slice of a second embedding row of the token entering each layer through a gate.

Checkpoint tensor names: embed (also the output projection), side.embed, final.norm, and for layer i: l<i>.norm1,
l<i>.norm1b, l<i>.norm2, l<i>.norm2b, l<i>.mix.<name>, l<i>.mlp.<name>, l<i>.side.{gate,proj,norm}.  Mixer tensors: latent
attention dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o; attention q, k, v, g, o.  Feed-forward tensors: gate, up, down;
routed: router and e<j>.{gate,up,down} for every expert j.
"""
from __future__ import annotations

import re

from ..config.fomerax import NAME, FomeraxConfig
from ..config.registry import register_architecture
from .base import Architecture

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")

_MIXER = {            # (parameter, piece) -> what follows "l<i>.mix."
    ("dq_dkv", "dq"): "dq", ("dq_dkv", "dkv"): "dkv", ("dq_norm", None): "dq.norm", ("uq", None): "uq",
    ("dkv_norm", None): "dkv.norm", ("uk", None): "uk", ("uv", None): "uv",
    ("qkv", "q"): "q", ("qkv", "k"): "k", ("qkv", "v"): "v",
    ("gate", None): "g", ("o", None): "o",
}
_IN_LAYER = {
    ("mixer_norm.weight", None): "norm1", ("mixer_post_norm.weight", None): "norm1b",
    ("feed_forward_norm.weight", None): "norm2", ("feed_forward_post_norm.weight", None): "norm2b",
    ("feed_forward.gate_up", "gate"): "mlp.gate", ("feed_forward.gate_up", "up"): "mlp.up",
    ("feed_forward.down", None): "mlp.down", ("feed_forward.router", None): "mlp.router",
    ("token_input.gate", None): "side.gate", ("token_input.proj", None): "side.proj", ("token_input.norm", None): "side.norm",
}
_TOP = {"embedding.weight": "embed", "embedding.side": "side.embed", "final_norm.weight": "final.norm"}
_EXPERT_PIECE = re.compile(r"^e(\d+)\.(gate|up|down)$")


class Fomerax(Architecture):
    name = NAME
    config_class = FomeraxConfig

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


register_architecture(Fomerax())
