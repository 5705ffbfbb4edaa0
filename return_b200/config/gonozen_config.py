"""Configuration of the Gonozen decoder, read from its own config.json keys.

``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (optional) and ``layers``: a list of entries with ``type`` (which
mixer the layer has: ``latent_attention`` or ``latent_attention_2``), ``mixer`` (its sizes and constants) and ``mlp``
(``{"kind": "moe", "router": {...}, "expert": {...}, "shared": {...}}`` or null).

``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale`` and ``rot`` (``base``, ``dims`` = rot_dim, optionally
``scaling`` with ``factor, original, fast, slow``).  ``latent_attention_2``: ``heads, dim, vdim, kv_rank, q_rank, scale``
and ``mask.size`` (the window).  Router: ``experts, top`` and optionally ``groups`` (``count, keep``).  Expert and shared
expert: ``ff, limit``.
"""
from __future__ import annotations

import copy

from .model_config import ConfigError

MIXER_TYPES = ("latent_attention", "latent_attention_2")


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {missing}")


class GonozenConfig:
    def __init__(self, raw: dict):
        self.raw = copy.deepcopy(raw)
        self.validate()

    @classmethod
    def from_dict(cls, raw: dict) -> "GonozenConfig":
        return cls(raw)

    # ------------------------------------------------------------------ what it holds
    @property
    def vocab(self) -> int:
        return int(self.raw["vocab"])

    vocab_size = vocab

    @property
    def width(self) -> int:
        return int(self.raw["width"])

    @property
    def eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @property
    def logit_softcap(self):
        cap = self.raw.get("logit_softcap")
        return float(cap) if cap else None

    @property
    def layers(self):
        return self.raw["layers"]

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        raw = self.raw
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        if self.vocab <= 0 or self.width <= 0 or not (self.eps > 0):
            raise ConfigError("vocab, width and norm.eps must be positive")
        if raw.get("logit_softcap") is not None and not (float(raw["logit_softcap"]) > 0):
            raise ConfigError("logit_softcap must be positive")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one entry")
        for i, layer in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            if layer["type"] not in MIXER_TYPES:
                raise ConfigError(f"{where}.type={layer['type']!r}; known: {list(MIXER_TYPES)}")
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"), where + ".mixer")
                rd = int(m["rot_dim"])
                if rd < 0 or rd % 2:
                    raise ConfigError(f"{where}.mixer.rot_dim={rd} must be even")
                if rd:
                    _need(m, ("rot",), where + ".mixer")
                    _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                    if int(m["rot"]["dims"]) != rd:
                        raise ConfigError(f"{where}.mixer.rot.dims must equal rot_dim={rd}: the rotated part is turned whole")
                    if m["rot"].get("scaling"):
                        _need(m["rot"]["scaling"], ("factor", "original", "fast", "slow"), where + ".mixer.rot.scaling")
                        if not float(m["rot"]["scaling"]["factor"]) > 0:
                            raise ConfigError(f"{where}.mixer.rot.scaling.factor must be positive")
            else:
                _need(m, ("heads", "dim", "vdim", "kv_rank", "q_rank", "scale"), where + ".mixer")
                if m.get("mask") is not None:
                    _need(m["mask"], ("size",), where + ".mixer.mask")
                    if int(m["mask"]["size"]) <= 0:
                        raise ConfigError(f"{where}.mixer.mask.size must be positive")
            if min(int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"])) <= 0:
                raise ConfigError(f"{where}.mixer: heads, dim, vdim and kv_rank must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "router", "expert"), where + ".mlp")
                if mlp["kind"] != "moe":
                    raise ConfigError(f"{where}.mlp.kind={mlp['kind']!r}: only 'moe' exists")
                _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                _need(mlp["expert"], ("ff", "limit"), where + ".mlp.expert")
                E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                g = mlp["router"].get("groups")
                count, keep = (int(g["count"]), int(g["keep"])) if g else (1, 1)
                if g:
                    _need(g, ("count", "keep"), where + ".mlp.router.groups")
                if count < 1 or E % count or not (1 <= keep <= count) or not (1 <= top <= keep * (E // count)):
                    raise ConfigError(f"{where}.mlp.router: {top} of {E} experts in {count} groups of which {keep} are kept")
                if mlp.get("shared") is not None:
                    _need(mlp["shared"], ("ff", "limit"), where + ".mlp.shared")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", "Gonozen")
        return d
