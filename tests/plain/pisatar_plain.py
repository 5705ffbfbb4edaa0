"""Plain, slow, whole-sequence implementation of the Pisatar decoder: the oracle of its tests.

Every mechanism is one function that walks a sequence token by token in the precision it is given
(float64 by default).  No cache, no batching, no kernels; nothing is shared with the ``return_b200``
package.  The configuration is config.json as a plain dict, the weights a dict name -> tensor.

Notation.  h: the mixer's input [T, width].  Linear maps are stored [out, in] and applied as
``h @ W.T``.  A recurrent state S of a head is a [key dim, value dim] matrix read out as ``S.T @ q``.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- files

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


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

def rms(x, eps):
    """x over the root of (its mean square plus eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def stream_norm(x, w, eps):
    """The norm of the residual stream: its weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def rotary_frequencies(rot, dtype):
    """f_i = base^(-2 i / dims), i < dims/2; with ``scaling`` the long wavelengths are slowed down:
    wavelength below original/high: kept; above original/low: f / factor; between: a blend."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f.tolist():
            lam = 2.0 * math.pi / fi
            if lam < sc["original"] / sc["high"]:
                out.append(fi)
            elif lam > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / lam - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(dtype)


def rotate(x, rot, positions):
    """x [T, heads, dim]: the first ``dims`` elements of every head turned by position * f_i, element i
    paired with element i + dims/2; the rest untouched."""
    dims = rot["dims"]
    half = dims // 2
    f = rotary_frequencies(rot, x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]                # [T, half]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def causal_conv(x, taps):
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, K-1-j] * x_(t-j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y


# --------------------------------------------------------------------------- mixers

def retention(h, m, w, p, eps, positions):
    """Linear attention with one fixed decay a head: S <- decay S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    q = rotate(q, m["rot"], positions)
    k = rotate(k, m["rot"], positions) * D ** -0.5
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps).reshape(T, H * V)
    return (o * F.silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def channel_delta(h, m, w, p, eps, positions):
    """Gated delta rule with a decay per key channel: S <- g * S (rows); u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = F.silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = F.silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                         # [T, H]
    step = F.softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, D)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)                # [T, H, D]
    S = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    rep = H // G
    for t in range(T):
        kt = k[t].repeat_interleave(rep, 0)                                        # head -> its q/k head
        qt = q[t].repeat_interleave(rep, 0)
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, qt)
    o = rms(o, eps) * w[p + "norm"]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, V)
    return (o * gate).reshape(T, H * V) @ w[p + "o"].T


def softmax_attention(h, m, w, p, eps, positions):
    """Causal grouped-query softmax attention with separate key and value sizes."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[p + "q"].T).view(T, H, D), m["rot"], positions)
    k = rotate((h @ w[p + "k"].T).view(T, G, D), m["rot"], positions)
    v = (h @ w[p + "v"].T).view(T, G, V)
    rep = H // G
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            g = hh // rep
            s = (k[:t + 1, g] @ q[t, hh]) * m["scale"]
            out[t, hh] = torch.softmax(s, 0) @ v[:t + 1, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


def matrix_memory(h, m, w, p, eps, positions):
    """Matrix memory with exponential gates kept stable by a running maximum that starts at zero."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                  # [T, H], logarithms
    fg = F.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    S = torch.zeros(H, D, V, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(fg[t] + mx, ig[t])
        a = torch.exp(fg[t] + mx - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = rms(o, eps).reshape(T, H * V) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel(h, m, w, p, eps, positions):
    """Two mixers on the same input, their outputs added with fixed weights."""
    left = softmax_attention(h, m["left"], w, p + "left.", eps, positions)
    right = matrix_memory(h, m["right"], w, p + "right.", eps, positions)
    return m["left_scale"] * left + m["right_scale"] * right


MIXERS = {"retention": retention, "channel_delta": channel_delta, "parallel": parallel}


def dense_mlp(h, w, p):
    return (F.silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# --------------------------------------------------------------------------- the model

def weight_layer(c, i):
    """The layer whose tensors layer i uses."""
    seen = set()
    while "weights_of" in c["layers"][i] and c["layers"][i]["weights_of"] is not None:
        if i in seen:
            raise ValueError("weights_of goes round in a circle")
        seen.add(i)
        i = c["layers"][i]["weights_of"]
    return i


def forward(c, w, ids, dtype=torch.float64):
    """(logits [T, vocab], residual stream after every layer [layers, T, width])."""
    eps = c["norm"]["eps"]
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.shape[0]
    positions = torch.arange(T)
    x = stream_norm(w["embed"][ids].to(dtype), w["embed.norm"], eps)
    after = []
    for i, layer in enumerate(c["layers"]):
        p = f"l{weight_layer(c, i)}."
        y = MIXERS[layer["type"]](stream_norm(x, w[p + "norm1"], eps), layer["mixer"], w, p + "mix.", eps, positions)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward {layer['mlp']['kind']!r}")
            y = y + dense_mlp(stream_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        x = x + y
        after.append(x)
    logits = stream_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(after)
