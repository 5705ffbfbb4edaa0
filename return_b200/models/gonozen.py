"""The Gonozen decoder as a ``DecoderSpec`` plus the map from its checkpoint tensor names to the parts' parameters.

Embedding; layers of the sandwich form (a norm before and after each sublayer) whose mixer is an attention over cached
latents, in one of two forms, and whose feed-forward is a mixture of experts with a shared expert; a final norm, the
embedding table as the output head, and a soft cap on the logits.

The two mixer types are one part (``LatentAttentionSpec``) with different options: ``latent_attention`` has a rotated
key part shared by the heads (frequencies stretched along a ramp) and a gate per head on the output;
``latent_attention_2`` has no positions, queries through a latent of their own, a sliding window and a sink per head.

Tensor names: ``embed``, ``final.norm``; ``l<i>.norm1 / norm1b / norm2 / norm2b``; ``l<i>.mix.{q, dkv, dkv.norm, uk,
uv, g, o}`` or ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, o}``; ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.{gate, up, down}``, ``l<i>.mlp.shared.{gate, up, down}``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.gonozen_config import GonozenConfig
from ..parts.spec import (ClampedGLUSpec, DecoderSpec, LatentAttentionSpec, MoESpec, NormSpec, RampedRopeSpec,
                          SandwichBlockSpec)
from ..weights.loader import Source


def _rope(m: dict, max_positions: int) -> Optional[RampedRopeSpec]:
    if not int(m.get("rot_dim", 0)):
        return None
    rot = m["rot"]
    sc = rot.get("scaling") or None
    return RampedRopeSpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_positions=max_positions,
                          factor=float(sc["factor"]) if sc else None, original=float(sc["original"]) if sc else 0.0,
                          fast=float(sc["fast"]) if sc else 0.0, slow=float(sc["slow"]) if sc else 0.0)


def _mixer_spec(kind: str, m: dict, width: int, eps: float, max_positions: int) -> LatentAttentionSpec:
    common = dict(hidden_size=width, num_heads=int(m["heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]),
                  kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), eps=eps)
    if kind == "latent_attention":
        return LatentAttentionSpec(rot_dim=int(m["rot_dim"]), gate=True, position=_rope(m, max_positions), **common)
    mask = m.get("mask")
    return LatentAttentionSpec(rot_dim=0, q_rank=int(m["q_rank"]), window=int(mask["size"]) if mask else None, sink=True,
                               **common)


def _mlp_spec(mlp: Optional[dict], width: int) -> Optional[MoESpec]:
    if not mlp:
        return None
    r, e, sh = mlp["router"], mlp["expert"], mlp.get("shared")
    g = r.get("groups")
    return MoESpec(hidden_size=width, num_experts=int(r["experts"]), top=int(r["top"]),
                   expert=ClampedGLUSpec(hidden_size=width, intermediate_size=int(e["ff"]), limit=float(e["limit"])),
                   groups=int(g["count"]) if g else 1, keep_groups=int(g["keep"]) if g else 1,
                   shared=ClampedGLUSpec(hidden_size=width, intermediate_size=int(sh["ff"]), limit=float(sh["limit"])) if sh else None)


def decoder_spec(cfg: GonozenConfig, max_positions: Optional[int] = None) -> DecoderSpec:
    max_positions = max_positions or 4096
    W, eps = cfg.width, cfg.eps
    norm = NormSpec(size=W, eps=eps)
    blocks = []
    for layer in cfg.layers:
        ff = _mlp_spec(layer.get("mlp"), W)
        blocks.append(SandwichBlockSpec(mixer=_mixer_spec(layer["type"], layer["mixer"], W, eps, max_positions),
                                        feed_forward=ff, mixer_norm=norm, mixer_post_norm=norm,
                                        feed_forward_norm=norm if ff else None, feed_forward_post_norm=norm if ff else None))
    return DecoderSpec(vocab_size=cfg.vocab, hidden_size=W, layers=tuple(blocks), schedule=DecoderSpec.in_order(len(blocks)),
                       final_norm=norm, tie_embeddings=True, logit_softcap=cfg.logit_softcap)


def weight_sources(cfg: GonozenConfig) -> Dict[str, Source]:
    m: Dict[str, Source] = {"embed": Source(("embed",)), "final_norm.weight": Source(("final.norm",))}
    for i, layer in enumerate(cfg.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        mix = src + "mix."
        m[dst + "mixer_norm.weight"] = Source((src + "norm1",))
        m[dst + "mixer_post_norm.weight"] = Source((src + "norm1b",))
        if layer["type"] == "latent_attention":
            m[dst + "mixer.in"] = Source((mix + "q", mix + "dkv", mix + "g"))
        else:
            m[dst + "mixer.in"] = Source((mix + "dq", mix + "dkv"))
            m[dst + "mixer.q_norm.weight"] = Source((mix + "dq.norm",))
            m[dst + "mixer.uq"] = Source((mix + "uq",))
            m[dst + "mixer.sink"] = Source((mix + "sink",))
        m[dst + "mixer.kv_norm.weight"] = Source((mix + "dkv.norm",))
        for name in ("uk", "uv", "o"):
            m[dst + "mixer." + name] = Source((mix + name,))
        mlp = layer.get("mlp")
        if mlp:
            E = int(mlp["router"]["experts"])
            p = src + "mlp."
            m[dst + "feed_forward_norm.weight"] = Source((src + "norm2",))
            m[dst + "feed_forward_post_norm.weight"] = Source((src + "norm2b",))
            m[dst + "feed_forward.router"] = Source((p + "router",))
            m[dst + "feed_forward.experts.gate_up"] = Source(tuple(f"{p}e{j}.{n}" for j in range(E) for n in ("gate", "up")))
            m[dst + "feed_forward.experts.down"] = Source(tuple(f"{p}e{j}.down" for j in range(E)))
            if mlp.get("shared"):
                m[dst + "feed_forward.shared.gate_up"] = Source((p + "shared.gate", p + "shared.up"))
                m[dst + "feed_forward.shared.down"] = Source((p + "shared.down",))
    return m


def checkpoint_shapes(cfg: GonozenConfig) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every tensor of a checkpoint: name -> (shape, law of its random values).  Matrices are drawn with a deviation of
    fan_in^-1/2, norm weights around one, sinks and the embedding around zero."""
    W, V = cfg.width, cfg.vocab
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {"embed": ((V, W), "normal:1.0"), "final.norm": ((W,), "ones_normal")}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        x = p + "mix."
        H, D, Vd, C = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"])
        for n in ("norm1", "norm1b"):
            out[p + n] = ((W,), "ones_normal")
        if layer["type"] == "latent_attention":
            R = int(m["rot_dim"])
            out[x + "q"] = ((H * (D + R), W), "fan_in")
            out[x + "dkv"] = ((C + R, W), "fan_in")
            out[x + "g"] = ((H, W), "fan_in")
        else:
            Q = int(m["q_rank"])
            out[x + "dq"] = ((Q, W), "fan_in")
            out[x + "dq.norm"] = ((Q,), "ones_normal")
            out[x + "uq"] = ((H * D, Q), "fan_in")
            out[x + "dkv"] = ((C, W), "fan_in")
            out[x + "sink"] = ((H,), "normal:1.0")
        out[x + "dkv.norm"] = ((C,), "ones_normal")
        out[x + "uk"] = ((H * D, C), "fan_in")
        out[x + "uv"] = ((H * Vd, C), "fan_in")
        out[x + "o"] = ((W, H * Vd), "fan_in")
        mlp = layer.get("mlp")
        if mlp:
            for n in ("norm2", "norm2b"):
                out[p + n] = ((W,), "ones_normal")
            E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            y = p + "mlp."
            out[y + "router"] = ((E, W), "fan_in")
            units = [(f"{y}e{j}.", F) for j in range(E)]
            if mlp.get("shared"):
                units.append((y + "shared.", int(mlp["shared"]["ff"])))
            for u, ff in units:
                out[u + "gate"] = ((ff, W), "fan_in")
                out[u + "up"] = ((ff, W), "fan_in")
                out[u + "down"] = ((W, ff), "fan_in")
    return out


def ignorable_tensors(cfg: GonozenConfig):
    """A layer without a feed-forward never reads the norms around one; a file may hold them all the same."""
    return {f"l{i}.{n}" for i, layer in enumerate(cfg.layers) if not layer.get("mlp") for n in ("norm2", "norm2b")}
