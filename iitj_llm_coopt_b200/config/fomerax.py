"""Typed configuration of the Fomerax family, read from its config.json.

Keys: "architecture" ("Fomerax"), "width", "vocab", "norm" {"eps"}, "token_side" {"dim"} (absent: the layers read nothing
of the token beside the stream) and "layers", a list whose entries give "type" (which mixer the layer has), the mixer's
sizes under "mixer" and the feed-forward under "mlp" (null: none).

Mixers:
  "latent_attention"  "heads", "dim" (unrotated query/key numbers of a head), "rot_dim" (rotated ones), "vdim",
                      "kv_rank" (width of the latent row that is cached), "q_rank" (width of the queries' latent row),
                      "scale", "rot" {"dims", "base", "scaling" {"factor", "original", "fast", "slow"} (absent: none)},
                      "mask" {"size"} (sliding window; absent: causal).
  "attention"         "heads", "kv_heads", "dim", "vdim", "scale", "softcap" (absent or 0: none), "q_temp" {"coef",
                      "every"} (absent: none), "mask" {"size"} (absent: causal).
Feed-forwards:
  {"kind": "dense", "ff"}
  {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}

Every size is read from the file; a missing key is an error at once.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field

from .errors import ConfigError
from .specs import (EmbeddingSpec, FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                    TokenInputSpec)

NAME = "Fomerax"
_MAX_POSITION = 1 << 30          # the design has no position table: int32 positions are the only bound
BIAS_SLOPE_EXPONENT = 8.0        # the design fixes the distance bias of head h of H at 2^(-8 (h + 1) / H) per position


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json lacks required key {key!r} in {where}")
    return d[key]


@dataclass
class FomeraxConfig:
    width: int
    vocab: int
    eps: float
    side_dim: int = 0                                # columns of the second embedding table that each layer reads (0: none)
    layers: list = field(default_factory=list)       # the file's "layers" entries, as read

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, c: dict) -> "FomeraxConfig":
        side = c.get("token_side")
        cfg = cls(width=int(_get(c, "width", "the file")), vocab=int(_get(c, "vocab", "the file")),
                  eps=float(_get(_get(c, "norm", "the file"), "eps", "norm")),
                  side_dim=int(_get(side, "dim", "token_side")) if side is not None else 0,
                  layers=copy.deepcopy(list(_get(c, "layers", "the file"))))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "FomeraxConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        out = {"architecture": NAME, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
               "layers": copy.deepcopy(self.layers)}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out

    # ---- checks --------------------------------------------------------------------------
    def validate(self) -> None:
        if self.width <= 0 or self.vocab <= 0:
            raise ConfigError("width and vocab must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if self.side_dim < 0:
            raise ConfigError("token_side.dim must be positive")
        if not self.layers:
            raise ConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind, m = _get(layer, "type", where), _get(layer, "mixer", where)
            if kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"):
                    _get(m, k, where + ".mixer")
                rot = _get(m, "rot", where + ".mixer")
                dims = int(_get(rot, "dims", where + ".mixer.rot"))
                if float(_get(rot, "base", where + ".mixer.rot")) <= 0:
                    raise ConfigError(f"{where}: rot.base must be positive")
                if dims % 2 or dims < 0 or dims > int(m["rot_dim"]):
                    raise ConfigError(f"{where}: rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
                sc = rot.get("scaling")
                if sc is not None:
                    for k in ("factor", "original", "fast", "slow"):
                        if float(_get(sc, k, where + ".mixer.rot.scaling")) <= 0:
                            raise ConfigError(f"{where}: rot.scaling.{k} must be positive")
            elif kind == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim", "scale"):
                    _get(m, k, where + ".mixer")
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
                if m.get("softcap") is not None and float(m["softcap"]) < 0:
                    raise ConfigError(f"{where}: softcap must not be negative")
                qt = m.get("q_temp")
                if qt is not None:
                    _get(qt, "coef", where + ".mixer.q_temp")
                    if int(_get(qt, "every", where + ".mixer.q_temp")) <= 0:
                        raise ConfigError(f"{where}: q_temp.every must be positive")
            else:
                raise ConfigError(f"{where}: type {kind!r} is not known (latent_attention, attention)")
            if m.get("mask") is not None and int(_get(m["mask"], "size", where + ".mixer.mask")) <= 0:
                raise ConfigError(f"{where}: mask.size must be positive")
            if any(int(v) <= 0 for k, v in m.items() if k in ("heads", "kv_heads", "dim", "vdim", "kv_rank", "q_rank", "rot_dim")):
                raise ConfigError(f"{where}: sizes must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            ff_kind = _get(mlp, "kind", where + ".mlp")
            if ff_kind == "dense":
                if int(_get(mlp, "ff", where + ".mlp")) <= 0:
                    raise ConfigError(f"{where}: mlp.ff must be positive")
            elif ff_kind == "moe":
                e, r = _get(mlp, "expert", where + ".mlp"), _get(mlp, "router", where + ".mlp")
                if int(_get(e, "ff", where + ".mlp.expert")) <= 0:
                    raise ConfigError(f"{where}: mlp.expert.ff must be positive")
                experts, top = int(_get(r, "experts", where + ".mlp.router")), int(_get(r, "top", where + ".mlp.router"))
                if experts <= 0 or not 1 <= top <= experts:
                    raise ConfigError(f"{where}: router takes {top} of {experts} experts")
            else:
                raise ConfigError(f"{where}: mlp.kind {ff_kind!r} is not known (dense, moe)")

    # ---- derived -------------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        """The layers as data.  Cache entry i belongs to layer i: pages of latent rows, or pages of keys and values."""
        norm = NormSpec(kind="rmsnorm", width=self.width, eps=self.eps)
        n = len(self.layers)
        layers, order = [], []
        for i, layer in enumerate(self.layers):
            m, kind = layer["mixer"], layer["type"]
            window = int((m.get("mask") or {}).get("size", 0))
            if kind == "latent_attention":
                rot = m["rot"]
                sc = rot.get("scaling")
                scaling = () if sc is None else tuple(sorted({"type": "yarn", "factor": float(sc["factor"]),
                                                              "original": float(sc["original"]), "fast": float(sc["fast"]),
                                                              "slow": float(sc["slow"])}.items()))
                pos = PositionSpec(kind="rope", head_dim=int(m["rot_dim"]), rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   scaling=scaling, max_position=_MAX_POSITION, pairing="interleaved")
                mixer = MixerSpec(kind="latent_attention", width=self.width, heads=int(m["heads"]), kv_heads=1,
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=window, softmax_scale=float(m["scale"]),
                                  position=pos if pos.rotary_dim else None,
                                  options=(("eps", self.eps), ("gate", "element"), ("kv_rank", int(m["kv_rank"])),
                                           ("q_rank", int(m["q_rank"])), ("rot_dim", int(m["rot_dim"]))))
            else:
                qt = m.get("q_temp")
                mixer = MixerSpec(kind="gated_attention", width=self.width, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=window, softmax_scale=float(m["scale"]),
                                  options=(("bias_slope_exponent", BIAS_SLOPE_EXPONENT), ("element_gate", True), ("eps", self.eps),
                                           ("q_temp", (float(qt["coef"]), int(qt["every"])) if qt else None),
                                           ("softcap", float(m.get("softcap") or 0.0))))
            order.append(LayerCall(layer=i, cache=i, write=True))
            parts = {"mixer_norm": norm, "mixer": mixer, "mixer_post_norm": norm}
            name = "sandwich"
            mlp = layer.get("mlp")
            if mlp is None:
                name += "_mixer"
            else:
                if mlp["kind"] == "dense":
                    ff = FeedForwardSpec(kind="glu", width=self.width, inner=int(mlp["ff"]), activation="gelu_tanh")
                else:
                    r = mlp["router"]
                    ff = FeedForwardSpec(kind="routed_glu", width=self.width, inner=int(mlp["expert"]["ff"]), activation="silu",
                                         experts=int(r["experts"]), experts_per_token=int(r["top"]),
                                         options=(("correction", False), ("expert", "silu"), ("router", "sigmoid"), ("weight_on", "input")))
                parts.update(feed_forward_norm=norm, feed_forward=ff, feed_forward_post_norm=norm)
            if self.side_dim:
                name += "_side"
                parts["token_input"] = TokenInputSpec(kind="gated_table", width=self.width, dim=self.side_dim, offset=i * self.side_dim,
                                                      table_width=n * self.side_dim, eps=self.eps)
            layers.append(LayerSpec.of(name, **parts))
        emb = EmbeddingSpec(kind="table_side" if self.side_dim else "table", vocab=self.vocab, width=self.width,
                            options=(("side_width", n * self.side_dim),) if self.side_dim else ())
        return ModelSpec(width=self.width, vocab=self.vocab, layers=tuple(layers), order=tuple(order), final_norm=norm,
                         tie_embeddings=True, max_position=_MAX_POSITION, embedding=emb)
