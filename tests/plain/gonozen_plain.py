"""Plain, slow, whole-sequence implementation of the Gonozen decoder: the oracle of its tests.

One function per mechanism, in the precision it is given (float64 by default).  No cache, no batching, no
kernels; nothing is shared with the ``return_b200`` package.  The configuration is config.json as a plain dict,
the weights a dict name -> tensor.

Notation.  h: a sublayer's input [T, width].  Linear maps are stored [out, in] and applied as ``h @ W.T``.
Keys and values of the attentions are never cached here: every head's keys and values are expanded from the
latent of every token, and the scores are a dense [T, T] matrix with a mask.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


# --------------------------------------------------------------------------- files

def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=_DT[m["dtype"]]).reshape(m["shape"]).clone()
    return out


def read_model(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    w = {k: (v.to(dtype) if v.is_floating_point() else v)
         for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return c, w


# --------------------------------------------------------------------------- small pieces

def rms_norm(x, w, eps):
    """x over the root of (its mean square plus eps), times a plain weight."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# --------------------------------------------------------------------------- rotary positions

def rotary_frequencies(rot, dtype=torch.float64):
    """(frequency of every pair [dims / 2], factor on cos and sin).  With ``scaling`` the frequencies whose index
    lies above a ramp are divided by ``factor``; the ramp's ends are the indices at which a wave turns ``fast``
    and ``slow`` times within ``original`` positions."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, ..., D]: the first rot.dims elements of the last axis turned by the position, element i with
    i + dims / 2; the rest is left as it is."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot, x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]                      # [T, dims / 2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (ang.cos() * mag).reshape(shape), (ang.sin() * mag).reshape(shape)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- attention

def masked_softmax(scores, visible, sink=None):
    """Softmax over the visible keys of every query.  scores [H, T, T], visible [T, T] bool, sink [H] or None: a
    term exp(sink) in the denominator that has no key."""
    s = scores.masked_fill(~visible[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def visible_keys(T, window=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    return ok


def latent_attention(h, w, p, m, eps, positions):
    """Attention whose keys and values are expanded from a latent of ``kv_rank`` numbers a token, with a rotated
    key part of ``rot_dim`` numbers shared by the heads and a gate per head on the output."""
    T = h.shape[0]
    H, D, R, Vd, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (h @ w[p + "q"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :C], w[p + "dkv.norm"], eps)
    k_rot = dkv[:, C:]
    if R:
        q_rot = rotate(q_rot, positions, m["rot"])
        k_rot = rotate(k_rot, positions, m["rot"])
    k = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, Vd)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k)
    if R:
        scores = scores + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    a = masked_softmax(scores * float(m["scale"]), visible_keys(T))
    o = torch.einsum("hij,jhd->ihd", a, v)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * Vd) @ w[p + "o"].T


def latent_attention_2(h, w, p, m, eps, positions):
    """Attention without positions: queries through a normed latent of ``q_rank`` numbers, keys and values from a
    normed latent of ``kv_rank``, a sliding window, and a sink per head in the softmax."""
    T = h.shape[0]
    H, D, Vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, D)
    c = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, Vd)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    window = int(m["mask"]["size"]) if m.get("mask") else None
    a = masked_softmax(scores, visible_keys(T, window), w[p + "sink"] if (p + "sink") in w else None)
    o = torch.einsum("hij,jhd->ihd", a, v)
    return o.reshape(T, H * Vd) @ w[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "latent_attention_2": latent_attention_2}


# --------------------------------------------------------------------------- feed-forward

def expert(h, w, p, limit):
    """A gated unit whose gate is capped above and whose other branch is clamped on both sides."""
    g = (h @ w[p + "gate"].T).clamp(max=limit)
    u = (h @ w[p + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(z, router):
    """(chosen experts [T, top], their weights [T, top]) from router logits z [T, experts]."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.softmax(z, dim=-1)
    allowed = s
    g = router.get("groups")
    if g and int(g["count"]) > 1:
        count, keep = int(g["count"]), int(g["keep"])
        best = s.reshape(-1, count, E // count).max(-1).values                    # [T, count]
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        mask = kept[:, :, None].expand(-1, -1, E // count).reshape(-1, E)
        allowed = s.masked_fill(~mask, -1.0)
    idx = allowed.topk(top, dim=-1).indices
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20)


def mixture_of_experts(h, w, p, mlp):
    z = h @ w[p + "router"].T
    idx, weight = route(z, mlp["router"])
    out = torch.zeros_like(h)
    limit = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), weight[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", limit)[0]
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.", float(mlp["shared"]["limit"]))
    return out


# --------------------------------------------------------------------------- the model

def forward(config, w, tokens, keep_layers=False):
    """Logits [T, vocab] of a whole sequence; with ``keep_layers`` also the stream after every layer."""
    dtype = w["embed"].dtype
    eps = float(config["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["embed"][ids]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mixed = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps, positions)
        x = x + rms_norm(mixed, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            y = mixture_of_experts(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    logits = logits.to(dtype)
    return (logits, torch.stack(after)) if keep_layers else logits
