"""Typed configuration of the Mamusun family, read from its config.json.

Keys: "architecture" ("Mamusun"), "width", "vocab", "norm" {"eps"}, "postln_alpha" and "layers", a list whose entries give
"type" (which mixer the layer has), the mixer's sizes under "mixer" and the feed-forward under "mlp" (null: none).

Mixers:
  "attention"    "heads", "kv_heads", "dim", "vdim", "scale", "mask" {"size"} (absent: causal), "kv_from" (absent: keys and
                 values of its own; else the index of the layer whose cache it reads).
  "attention_2"  "heads", "kv_heads", "dim", "scale", "rot" {"dims", "base", "scaling" {"factor", "original", "fast", "slow"}
                 (absent: none)}, "mask" {"size"} (absent: causal); its values are its keys, so "vdim" equals "dim" if given.
  "parallel"     "left": "heads", "kv_heads", "dim", "vdim", "scale", "rot" {"dims", "base", "scaling" {"factor", "low", "high",
                 "original"} (absent: none)}, "mask" {"size"} (absent: causal);  "right": "width", "blocks", "conv".
Feed-forwards:
  {"kind": "dense", "ff"}
  {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}

Every size is read from the file; a missing key is an error at once.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field

from .errors import ConfigError
from .specs import (EmbeddingSpec, FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                    StreamMixSpec)

NAME = "Mamusun"
_MAX_POSITION = 1 << 30          # the design has no position table: int32 positions are the only bound
DECAY_SCALE = 8.0                # the design fixes the recurrence's decay at exp(-8 r softplus(lam))
EXPERT_SLOPE = 1.702             # and the slope of its experts' sigmoid gate


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json lacks required key {key!r} in {where}")
    return d[key]


def _window(m: dict) -> int:
    return int((m.get("mask") or {}).get("size", 0))


@dataclass
class MamusunConfig:
    width: int
    vocab: int
    eps: float
    alpha: float
    layers: list = field(default_factory=list)       # the file's "layers" entries, as read

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, c: dict) -> "MamusunConfig":
        cfg = cls(width=int(_get(c, "width", "the file")), vocab=int(_get(c, "vocab", "the file")),
                  eps=float(_get(_get(c, "norm", "the file"), "eps", "norm")), alpha=float(_get(c, "postln_alpha", "the file")),
                  layers=copy.deepcopy(list(_get(c, "layers", "the file"))))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "MamusunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": NAME, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
                "postln_alpha": self.alpha, "layers": copy.deepcopy(self.layers)}

    # ---- checks --------------------------------------------------------------------------
    @staticmethod
    def _check_heads(m: dict, where: str, value_key: bool = True) -> None:
        for k in ("heads", "kv_heads", "dim", "scale") + (("vdim",) if value_key else ()):
            _get(m, k, where)
        if any(int(m[k]) <= 0 for k in ("heads", "kv_heads", "dim") + (("vdim",) if value_key else ())):
            raise ConfigError(f"{where}: sizes must be positive")
        if int(m["heads"]) % int(m["kv_heads"]):
            raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
        if m.get("mask") is not None and int(_get(m["mask"], "size", where + ".mask")) <= 0:
            raise ConfigError(f"{where}: mask.size must be positive")

    @staticmethod
    def _check_rot(m: dict, where: str, law: tuple) -> None:
        rot = _get(m, "rot", where)
        dims = int(_get(rot, "dims", where + ".rot"))
        if float(_get(rot, "base", where + ".rot")) <= 0:
            raise ConfigError(f"{where}: rot.base must be positive")
        if dims % 2 or dims < 0 or dims > int(m["dim"]):
            raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {m['dim']}")
        sc = rot.get("scaling")
        if sc is not None:
            for k in law:
                if float(_get(sc, k, where + ".rot.scaling")) <= 0:
                    raise ConfigError(f"{where}: rot.scaling.{k} must be positive")
            if "high" in law and float(sc["high"]) == float(sc["low"]):
                raise ConfigError(f"{where}: rot.scaling.high and low must differ")

    def validate(self) -> None:
        if self.width <= 0 or self.vocab <= 0:
            raise ConfigError("width and vocab must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if not self.layers:
            raise ConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind, m = _get(layer, "type", where), _get(layer, "mixer", where)
            if kind == "attention":
                self._check_heads(m, where + ".mixer")
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or self.layers[src].get("type") != "attention" or self.layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from {src} must name an earlier attention layer with keys and values of its own")
                    o = self.layers[src]["mixer"]
                    if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"{where}: kv_from {src} has other key/value sizes")
            elif kind == "attention_2":
                self._check_heads(m, where + ".mixer", value_key=False)
                if m.get("vdim") is not None and int(m["vdim"]) != int(m["dim"]):
                    raise ConfigError(f"{where}: the values are the keys, vdim {m['vdim']} must equal dim {m['dim']}")
                self._check_rot(m, where + ".mixer", ("factor", "original", "fast", "slow"))
            elif kind == "parallel":
                left, right = _get(m, "left", where + ".mixer"), _get(m, "right", where + ".mixer")
                self._check_heads(left, where + ".mixer.left")
                self._check_rot(left, where + ".mixer.left", ("factor", "low", "high", "original"))
                for k in ("width", "blocks", "conv"):
                    if int(_get(right, k, where + ".mixer.right")) <= 0:
                        raise ConfigError(f"{where}: right.{k} must be positive")
                if int(right["width"]) % int(right["blocks"]):
                    raise ConfigError(f"{where}: right.width {right['width']} is not a multiple of blocks {right['blocks']}")
            else:
                raise ConfigError(f"{where}: type {kind!r} is not known (attention, attention_2, parallel)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            ff_kind = _get(mlp, "kind", where + ".mlp")
            if ff_kind == "dense":
                if int(_get(mlp, "ff", where + ".mlp")) <= 0:
                    raise ConfigError(f"{where}: mlp.ff must be positive")
            elif ff_kind == "moe":
                e, r = _get(mlp, "expert", where + ".mlp"), _get(mlp, "router", where + ".mlp")
                if int(_get(e, "ff", where + ".mlp.expert")) <= 0 or float(_get(e, "limit", where + ".mlp.expert")) < 0:
                    raise ConfigError(f"{where}: mlp.expert.ff must be positive and limit not negative")
                experts, top = int(_get(r, "experts", where + ".mlp.router")), int(_get(r, "top", where + ".mlp.router"))
                if experts <= 0 or not 1 <= top <= experts:
                    raise ConfigError(f"{where}: router takes {top} of {experts} experts")
            else:
                raise ConfigError(f"{where}: mlp.kind {ff_kind!r} is not known (dense, moe)")

    # ---- derived -------------------------------------------------------------------------
    def _rope(self, m: dict, law: str, pairing: str) -> PositionSpec | None:
        rot = m["rot"]
        if not int(rot["dims"]):
            return None
        sc = rot.get("scaling")
        scaling = ()
        if sc is not None and law == "yarn":
            scaling = tuple(sorted({"type": "yarn", "factor": float(sc["factor"]), "original": float(sc["original"]),
                                    "fast": float(sc["fast"]), "slow": float(sc["slow"])}.items()))
        elif sc is not None:
            scaling = tuple(sorted({"type": "llama3", "float64": True, "factor": float(sc["factor"]), "low_freq_factor": float(sc["low"]),
                                    "high_freq_factor": float(sc["high"]),
                                    "original_max_position_embeddings": float(sc["original"])}.items()))
        else:
            scaling = (("float64", True), ("type", "none"))
        return PositionSpec(kind="rope", head_dim=int(m["dim"]), rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                            scaling=scaling, max_position=_MAX_POSITION, pairing=pairing)

    def model_spec(self) -> ModelSpec:
        """The layers as data.  A layer with keys and values of its own owns one cache entry (pages), a parallel layer a second
        one (the recurrence's record); a layer that borrows reads the lender's entry, whose window covers both."""
        norm = NormSpec(kind="rmsnorm_one_plus", width=self.width, eps=self.eps)
        n = len(self.layers)
        # a lender's pages must outlive the widest window that reads them (0: all tokens)
        reach = {i: _window(l["mixer"]) for i, l in enumerate(self.layers) if l["type"] == "attention"}
        for i, l in enumerate(self.layers):
            src = l["mixer"].get("kv_from") if l["type"] == "attention" else None
            if src is not None:
                mine = _window(l["mixer"])
                reach[int(src)] = 0 if (mine == 0 or reach[int(src)] == 0) else max(reach[int(src)], mine)
        layers, order, entry_of, entries = [], [], {}, 0
        for i, layer in enumerate(self.layers):
            m, kind = layer["mixer"], layer["type"]
            state = None
            if kind == "attention":
                own = m.get("kv_from") is None
                mixer = MixerSpec(kind="gated_attention", width=self.width, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=_window(m), softmax_scale=float(m["scale"]),
                                  options=(("cache_window", reach[i] if own else reach[int(m["kv_from"])]), ("eps", self.eps),
                                           ("own_kv", own), ("qk_norm", True)))
                if own:
                    entry_of[i], cache = entries, entries
                    entries += 1
                else:
                    cache = entry_of[int(m["kv_from"])]
                call = LayerCall(layer=i, cache=cache, write=own)
            elif kind == "attention_2":
                mixer = MixerSpec(kind="gated_attention", width=self.width, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["dim"]), window=_window(m), softmax_scale=float(m["scale"]),
                                  position=self._rope(m, "yarn", "half"),
                                  options=(("bias", True), ("eps", self.eps), ("qk_norm", "row"), ("sinks", True), ("value_from_key", True)))
                call = LayerCall(layer=i, cache=entries, write=True)
                entries += 1
            else:
                lm, rm = m["left"], m["right"]
                left = MixerSpec(kind="gated_attention", width=self.width, heads=int(lm["heads"]), kv_heads=int(lm["kv_heads"]),
                                 head_dim=int(lm["dim"]), value_dim=int(lm["vdim"]), window=_window(lm), softmax_scale=float(lm["scale"]),
                                 position=self._rope(lm, "llama3", "interleaved"),
                                 options=(("eps", self.eps), ("norm_after_rotation", True), ("qk_norm", "unit")))
                right = MixerSpec(kind="gated_lru", width=self.width,
                                  options=(("blocks", int(rm["blocks"])), ("conv_taps", int(rm["conv"])), ("decay_scale", DECAY_SCALE),
                                           ("inner", int(rm["width"]))))
                mixer = MixerSpec(kind="parallel", width=self.width, position=left.position,
                                  options=(("eps", self.eps), ("left", left), ("right", right), ("scale", 0.5)))
                call = LayerCall(layer=i, cache=entries, write=True, state=entries + 1)
                entries += 2
            order.append(call)
            mix = StreamMixSpec(kind="depth_average", width=self.width, inputs=i + 2, total=n + 1)
            parts = {"mixer": mixer, "mixer_norm": norm, "stream_mix": mix}
            name = "postnorm_depth_mixer"
            mlp = layer.get("mlp")
            if mlp is not None:
                name = "postnorm_depth"
                if mlp["kind"] == "dense":
                    ff = FeedForwardSpec(kind="poly_norm_mlp", width=self.width, inner=int(mlp["ff"]), activation="poly_norm",
                                         options=(("eps", self.eps),))
                else:
                    r = mlp["router"]
                    ff = FeedForwardSpec(kind="routed_glu", width=self.width, inner=int(mlp["expert"]["ff"]), activation="clamped",
                                         experts=int(r["experts"]), experts_per_token=int(r["top"]),
                                         options=(("correction", False), ("limit", float(mlp["expert"]["limit"])),
                                                  ("router", "chosen_softmax"), ("router_bias", True), ("slope", EXPERT_SLOPE)))
                parts.update(feed_forward=ff, feed_forward_norm=norm)
            layers.append(LayerSpec(name, tuple(parts.items()), options=(("alpha", self.alpha),)))
        return ModelSpec(width=self.width, vocab=self.vocab, layers=tuple(layers), order=tuple(order), final_norm=norm,
                         tie_embeddings=False, max_position=_MAX_POSITION,
                         embedding=EmbeddingSpec(kind="table", vocab=self.vocab, width=self.width))
