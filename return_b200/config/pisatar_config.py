"""Configuration of the Pisatar decoder, read from its own config.json keys.

``vocab``, ``width``, ``norm.eps`` and ``layers``: a list of entries with ``type`` (which mixer the layer has:
``retention``, ``channel_delta`` or ``parallel``), ``mixer`` (the mixer's sizes and constants), ``mlp``
(``{"kind": "dense", "ff": n}`` or null) and optionally ``weights_of`` (the layer whose tensors this layer uses,
with a cache or state of its own).  Two sizes of a ``channel_delta`` mixer are not config keys but shapes of its
tensors: the ranks of its two low-rank projections.  ``from_model_dir`` reads them from the safetensors header
and keeps them in the mixer's entry as ``decay_rank`` and ``gate_rank``, so that the configuration alone says
every size from then on (``to_dict`` writes them, ``from_dict`` takes them back).
"""
from __future__ import annotations

import copy
import json
import os
from typing import Optional

from .model_config import ConfigError

MIXER_TYPES = ("retention", "channel_delta", "parallel")


def _need(d: dict, keys, where: str) -> None:
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {missing}")


def _check_rot(rot, dim: int, where: str, scaling_allowed: bool = True) -> None:
    _need(rot, ("base", "dims"), where + ".rot")
    dims = int(rot["dims"])
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{where}.rot.dims={dims} must be even and at most dim={dim}")
    sc = rot.get("scaling")
    if sc is not None:
        _need(sc, ("factor", "low", "high", "original"), where + ".rot.scaling")
        if float(sc["high"]) == float(sc["low"]):
            raise ConfigError(f"{where}.rot.scaling: high and low must differ")


class PisatarConfig:
    def __init__(self, raw: dict):
        self.raw = copy.deepcopy(raw)
        self.validate()

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "PisatarConfig":
        return cls(raw)

    @classmethod
    def from_model_dir(cls, model_dir: str, raw: Optional[dict] = None) -> "PisatarConfig":
        """config.json plus the sizes that only tensor shapes give."""
        if raw is None:
            with open(os.path.join(model_dir, "config.json")) as f:
                raw = json.load(f)
        raw = copy.deepcopy(raw)
        layers = raw.get("layers") or []
        wanted = [i for i, layer in enumerate(layers)
                  if isinstance(layer, dict) and layer.get("type") == "channel_delta" and layer.get("weights_of") is None
                  and isinstance(layer.get("mixer"), dict)
                  and not ("decay_rank" in layer["mixer"] and "gate_rank" in layer["mixer"])]
        if wanted:
            from ..weights.safetensors_io import ModelFiles
            files = ModelFiles(model_dir)
            try:
                for i in wanted:
                    for key, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                        if name not in files:
                            raise ConfigError(f"{model_dir}: tensor {name} is missing; its rows give {key}")
                        layers[i]["mixer"][key] = int(files.shape(name)[0])
            finally:
                files.close()
        for i, layer in enumerate(layers):               # a layer that borrows weights has the lender's sizes
            j = layer.get("weights_of") if isinstance(layer, dict) else None
            if j is not None and layer.get("type") == "channel_delta" and 0 <= int(j) < len(layers):
                src = layers[cls._owner(layers, i)].get("mixer", {})
                for key in ("decay_rank", "gate_rank"):
                    if key in src:
                        layer["mixer"].setdefault(key, src[key])
        return cls(raw)

    # ------------------------------------------------------------------ what it holds
    @property
    def vocab(self) -> int:
        return int(self.raw["vocab"])

    @property
    def width(self) -> int:
        return int(self.raw["width"])

    @property
    def eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @property
    def layers(self):
        return self.raw["layers"]

    @staticmethod
    def _owner(layers, i: int) -> int:
        seen = set()
        while layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError("weights_of goes round in a circle")
            seen.add(i)
            i = int(layers[i]["weights_of"])
            if not (0 <= i < len(layers)):
                raise ConfigError(f"weights_of names layer {i}, there are {len(layers)}")
        return i

    def weight_layer(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless it has ``weights_of``)."""
        return self._owner(self.layers, i)

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        raw = self.raw
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        if self.vocab <= 0 or self.width <= 0 or not (self.eps > 0):
            raise ConfigError("vocab, width and norm.eps must be positive")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one entry")
        for i, layer in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            if layer["type"] not in MIXER_TYPES:
                raise ConfigError(f"{where}.type={layer['type']!r}; known: {list(MIXER_TYPES)}")
            m = layer["mixer"]
            if layer["type"] == "retention":
                _need(m, ("heads", "dim", "vdim", "decay", "rot"), where + ".mixer")
                if len(m["decay"]) != int(m["heads"]):
                    raise ConfigError(f"{where}.mixer.decay has {len(m['decay'])} entries for {m['heads']} heads")
                _check_rot(m["rot"], int(m["dim"]), where + ".mixer")
            elif layer["type"] == "channel_delta":
                _need(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".mixer")
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}.mixer: heads must be a multiple of kv_heads")
                if int(m["conv"]) < 1:
                    raise ConfigError(f"{where}.mixer.conv must be at least 1")
            else:
                _need(m, ("left", "right", "left_scale", "right_scale"), where + ".mixer")
                left, right = m["left"], m["right"]
                _need(left, ("heads", "kv_heads", "dim", "vdim", "rot", "scale"), where + ".mixer.left")
                _need(right, ("heads", "dim", "vdim", "gate_cap"), where + ".mixer.right")
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ConfigError(f"{where}.mixer.left: heads must be a multiple of kv_heads")
                _check_rot(left["rot"], int(left["dim"]), where + ".mixer.left")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "ff"), where + ".mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"{where}.mlp.kind={mlp['kind']!r}: only 'dense' exists")
            if layer.get("weights_of") is not None:
                j = self.weight_layer(i)
                other = raw["layers"][j]
                same = lambda a, b: {k: v for k, v in a.items() if k not in ("decay_rank", "gate_rank")} == \
                                    {k: v for k, v in b.items() if k not in ("decay_rank", "gate_rank")}
                if other["type"] != layer["type"] or not same(other["mixer"], m) or other.get("mlp") != mlp:
                    raise ConfigError(f"{where} uses the weights of layer {j} but is not shaped like it")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", "Pisatar")
        return d
