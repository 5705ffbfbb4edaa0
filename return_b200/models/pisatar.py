"""The Pisatar decoder as a ``DecoderSpec`` plus the map from its checkpoint tensor names to the parts' parameters.

Embedding, then a norm; layers of the parallel form x += mixer(norm1(x)) + mlp(norm2(x)), whose mixer is a
retention, a channel-wise gated delta rule, or the sum of a softmax attention and a matrix memory; a final norm and
an untied head.  Every norm of the stream stores its weight around zero (offset 1).  A layer with ``weights_of``
runs another layer's parts with a state of its own: the specification holds each set of weights once and the
schedule names it as often as it runs.

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``head``; ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.<name>`` (under ``.left`` / ``.right`` for the sum of two), ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.pisatar_config import PisatarConfig
from ..config.model_config import ConfigError
from ..parts.spec import (AttentionSpec, ChannelDeltaSpec, DecoderSpec, MatrixMemorySpec, MixerSumSpec, NormSpec,
                          ParallelBlockSpec, RetentionSpec, ScaledRopeSpec, ScheduleEntry, SwiGLUSpec)
from ..weights.loader import Source


def _rope(rot: dict, max_positions: int) -> Optional[ScaledRopeSpec]:
    if int(rot["dims"]) == 0:
        return None
    sc = rot.get("scaling")
    scaling = (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])) if sc else None
    return ScaledRopeSpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_positions=max_positions,
                          scaling=scaling)


def _padded_head(m: dict) -> int:
    """The head size the attention kernels run: key and value sizes padded to one multiple of 16."""
    return (max(int(m["dim"]), int(m["vdim"])) + 15) // 16 * 16


def _interleave(ff: int) -> int:
    return 8 if ff % 8 == 0 else 0


def _mixer_spec(kind: str, m: dict, width: int, eps: float, max_positions: int):
    if kind == "retention":
        return RetentionSpec(hidden_size=width, num_heads=int(m["heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]),
                             decay=tuple(float(x) for x in m["decay"]), eps=eps, position=_rope(m["rot"], max_positions))
    if kind == "channel_delta":
        if "decay_rank" not in m or "gate_rank" not in m:
            raise ConfigError("a channel_delta mixer's low ranks are shapes of its tensors: read the configuration with "
                              "PisatarConfig.from_model_dir, or give decay_rank and gate_rank in the mixer's entry")
        return ChannelDeltaSpec(hidden_size=width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                                key_dim=int(m["dim"]), value_dim=int(m["vdim"]), conv_taps=int(m["conv"]),
                                decay_rank=int(m["decay_rank"]), gate_rank=int(m["gate_rank"]), eps=eps)
    left, right = m["left"], m["right"]
    attention = AttentionSpec(hidden_size=width, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]),
                              head_dim=_padded_head(left), scale=float(left["scale"]), window=None, qk_norm=None,
                              position=_rope(left["rot"], max_positions), key_dim=int(left["dim"]),
                              value_dim=int(left["vdim"]))
    memory = MatrixMemorySpec(hidden_size=width, num_heads=int(right["heads"]), key_dim=int(right["dim"]),
                              value_dim=int(right["vdim"]), gate_cap=float(right["gate_cap"]), eps=eps)
    return MixerSumSpec(names=("left", "right"), mixers=(attention, memory),
                        scales=(float(m["left_scale"]), float(m["right_scale"])))


def _owners(cfg: PisatarConfig):
    """Config layers that have tensors of their own, in order, and config layer -> index among them."""
    owners = [i for i in range(len(cfg.layers)) if cfg.layers[i].get("weights_of") is None]
    place = {i: k for k, i in enumerate(owners)}
    return owners, place


def decoder_spec(cfg: PisatarConfig, max_positions: Optional[int] = None) -> DecoderSpec:
    max_positions = max_positions or 4096
    W, eps = cfg.width, cfg.eps
    norm = NormSpec(size=W, eps=eps, offset=1.0)
    owners, place = _owners(cfg)
    blocks = []
    for i in owners:
        layer = cfg.layers[i]
        mlp = layer.get("mlp")
        ff = SwiGLUSpec(hidden_size=W, intermediate_size=int(mlp["ff"]), interleave=_interleave(int(mlp["ff"]))) if mlp else None
        blocks.append(ParallelBlockSpec(mixer=_mixer_spec(layer["type"], layer["mixer"], W, eps, max_positions),
                                        feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm if mlp else None))
    schedule = tuple(ScheduleEntry(place[cfg.weight_layer(i)]) for i in range(len(cfg.layers)))
    return DecoderSpec(vocab_size=cfg.vocab, hidden_size=W, layers=tuple(blocks), schedule=schedule, final_norm=norm,
                       tie_embeddings=False, embedding_norm=norm)


def weight_sources(cfg: PisatarConfig) -> Dict[str, Source]:
    m: Dict[str, Source] = {"embed": Source(("embed",)), "embedding_norm.weight": Source(("embed.norm",)),
                            "final_norm.weight": Source(("final.norm",)), "lm_head": Source(("head",))}
    owners, _ = _owners(cfg)
    for k, i in enumerate(owners):
        layer = cfg.layers[i]
        src, dst = f"l{i}.", f"layers.{k}."
        mix, kind, mm = src + "mix.", layer["type"], layer["mixer"]
        m[dst + "mixer_norm.weight"] = Source((src + "norm1",))
        if layer.get("mlp"):
            m[dst + "feed_forward_norm.weight"] = Source((src + "norm2",))
            m[dst + "feed_forward.gate_up"] = Source((src + "mlp.gate", src + "mlp.up"),
                                                     interleave=_interleave(int(layer["mlp"]["ff"])))
            m[dst + "feed_forward.down"] = Source((src + "mlp.down",))
        if kind == "retention":
            m[dst + "mixer.in"] = Source((mix + "q", mix + "k", mix + "v", mix + "g"))
            m[dst + "mixer.o"] = Source((mix + "o",))
        elif kind == "channel_delta":
            m[dst + "mixer.in"] = Source((mix + "q", mix + "k", mix + "v", mix + "a1", mix + "g1"))
            m[dst + "mixer.conv"] = Source((mix + "q.conv", mix + "k.conv", mix + "v.conv"))
            m[dst + "mixer.beta"] = Source((mix + "b",))
            m[dst + "mixer.decay_up"] = Source((mix + "a2",))
            m[dst + "mixer.gate_up"] = Source((mix + "g2",))
            for name in ("A_log", "dt_bias", "norm", "o"):
                m[dst + "mixer." + name] = Source((mix + name,))
        else:
            left, right = mm["left"], mm["right"]
            D = _padded_head(left)
            kpad, vpad = (int(left["dim"]), D), (int(left["vdim"]), D)
            m[dst + "mixer.left.qkv"] = Source((mix + "left.q", mix + "left.k", mix + "left.v"),
                                               pad_rows=(kpad, kpad, vpad))
            m[dst + "mixer.left.o"] = Source((mix + "left.o",), pad_cols=vpad)
            r = mix + "right."
            m[dst + "mixer.right.in"] = Source((r + "q", r + "k", r + "v", r + "g"))
            m[dst + "mixer.right.gates"] = Source((r + "i", r + "f"))
            m[dst + "mixer.right.gate_bias"] = Source((r + "i.b", r + "f.b"))
            m[dst + "mixer.right.norm"] = Source((r + "norm",))
            m[dst + "mixer.right.o"] = Source((r + "o",))
    return m


def checkpoint_shapes(cfg: PisatarConfig) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every tensor of a checkpoint: name -> (shape, law of its random values).  Matrices are drawn with a deviation of
    fan_in^-1/2, norm weights of the stream around zero, the others so that gates and decays are neither shut nor open."""
    W, V = cfg.width, cfg.vocab
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {
        "embed": ((V, W), "normal:1.0"), "embed.norm": ((W,), "zeros_normal"),
        "final.norm": ((W,), "zeros_normal"), "head": ((V, W), "fan_in")}
    owners, _ = _owners(cfg)
    for i in owners:
        layer = cfg.layers[i]
        p, kind, m = f"l{i}.", layer["type"], layer["mixer"]
        out[p + "norm1"] = ((W,), "zeros_normal")
        if layer.get("mlp"):
            ff = int(layer["mlp"]["ff"])
            out[p + "norm2"] = ((W,), "zeros_normal")
            out[p + "mlp.gate"] = ((ff, W), "fan_in")
            out[p + "mlp.up"] = ((ff, W), "fan_in")
            out[p + "mlp.down"] = ((W, ff), "fan_in")
        x = p + "mix."
        if kind == "retention":
            H, D, Vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            for name, rows in (("q", H * D), ("k", H * D), ("v", H * Vd), ("g", H * Vd)):
                out[x + name] = ((rows, W), "fan_in")
            out[x + "o"] = ((W, H * Vd), "fan_in")
        elif kind == "channel_delta":
            if "decay_rank" not in m or "gate_rank" not in m:
                raise ConfigError("a channel_delta mixer needs decay_rank and gate_rank to size its tensors")
            H, G, D, Vd, K = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"])
            ra, rg = int(m["decay_rank"]), int(m["gate_rank"])
            for name, rows in (("q", G * D), ("k", G * D), ("v", H * Vd)):
                out[x + name] = ((rows, W), "fan_in")
                out[x + name + ".conv"] = ((rows, K), "normal:0.5")
            out[x + "b"] = ((H, W), "fan_in")
            out[x + "A_log"] = ((H,), "normal:0.5")
            out[x + "norm"] = ((Vd,), "ones_normal")
            out[x + "a1"] = ((ra, W), "fan_in")
            out[x + "a2"] = ((H * D, ra), "fan_in")
            out[x + "dt_bias"] = ((H * D,), "normal:0.5")
            out[x + "g1"] = ((rg, W), "fan_in")
            out[x + "g2"] = ((H * Vd, rg), "fan_in")
            out[x + "o"] = ((W, H * Vd), "fan_in")
        else:
            left, right = m["left"], m["right"]
            H, G, D, Vd = int(left["heads"]), int(left["kv_heads"]), int(left["dim"]), int(left["vdim"])
            out[x + "left.q"] = ((H * D, W), "fan_in")
            out[x + "left.k"] = ((G * D, W), "fan_in")
            out[x + "left.v"] = ((G * Vd, W), "fan_in")
            out[x + "left.o"] = ((W, H * Vd), "fan_in")
            H, D, Vd = int(right["heads"]), int(right["dim"]), int(right["vdim"])
            for name, rows in (("q", H * D), ("k", H * D), ("v", H * Vd), ("g", H * Vd)):
                out[x + "right." + name] = ((rows, W), "fan_in")
            out[x + "right.o"] = ((W, H * Vd), "fan_in")
            out[x + "right.norm"] = ((H * Vd,), "ones_normal")
            for gate in ("i", "f"):
                out[x + "right." + gate] = ((H, W), "fan_in")
                out[x + "right." + gate + ".b"] = ((H,), "normal:0.5")
    return out


def ignorable_tensors(cfg: PisatarConfig):
    """A layer without a feed-forward never reads its second norm; a file may hold one all the same."""
    owners, _ = _owners(cfg)
    return {f"l{i}.norm2" for i in owners if not cfg.layers[i].get("mlp")}
