"""Attention over a paged cache of latents.

Every token leaves one vector in the cache: a normed latent c of ``kv_rank`` numbers and, behind it, a rotated key
part of ``rot_dim`` numbers that all heads share.  A head's key is ``[U_h c | rotated part]`` and its value ``V_h c``.
The engine never expands them: since ``q_h . (U_h c) = (U_h^T q_h) . c`` and ``sum_j a_j V_h c_j = V_h sum_j a_j c_j``,
a head's query is carried into the latent's space once per token (a product per head with U_h^T), the attention
runs over the cached vectors themselves, one kv head for all query heads, and the weighted mean of the latents is carried
to the head's value space afterwards (a product per head with V_h).  The same path serves prompts, portions and
decoded tokens, so the cache is all a request keeps.

Parameters: ``in`` (all projections of the mixer's input, fused: the queries or their latent, the key/value latent
with the rotated part, the gates), ``q_norm.weight`` / ``uq`` (queries through a latent), ``kv_norm.weight``,
``uk`` [heads * key_dim, kv_rank], ``uv`` [heads * value_dim, kv_rank], ``sink`` [heads], ``o``.
"""
from __future__ import annotations

import torch

from ..ext import ops
from .base import MIXERS, POSITION_ENCODINGS, LatentCacheNeed, Mixer, ParamSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.rot_dim % 2 or s.rot_dim < 0:
            raise ValueError(f"rot_dim={s.rot_dim} must be even")
        if s.rot_dim and (s.position is None or s.position.rotary_dim != s.rot_dim):
            raise ValueError("a rotated part needs a position encoding of its width")
        if s.window is not None and s.window <= 0:
            raise ValueError("window must be positive")
        if not (0 < s.kv_rank <= ops.LATENT_MAX_RANK):
            raise ValueError(f"kv_rank={s.kv_rank}: the kernels take latents of up to {ops.LATENT_MAX_RANK} numbers")
        self.position = POSITION_ENCODINGS.build(s.position, env) if s.rot_dim else None
        self.q_head = s.key_dim + s.rot_dim
        self.q_size = s.num_heads * self.q_head
        self.first = s.q_rank if s.q_rank is not None else self.q_size          # queries, or their latent
        self.c_off = self.first
        self.g_off = self.first + s.kv_rank + s.rot_dim
        self.in_size = self.g_off + (s.num_heads if s.gate else 0)

    # ------------------------------------------------------------------ parameters and cache
    def params(self):
        s = self.spec
        p = {"in": ParamSpec((self.in_size, s.hidden_size)),
             "kv_norm.weight": ParamSpec((s.kv_rank,), role="vector", init="ones_normal"),
             "uk": ParamSpec((s.num_heads * s.key_dim, s.kv_rank)),
             "uv": ParamSpec((s.num_heads * s.value_dim, s.kv_rank)),
             "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim))}
        if s.q_rank is not None:
            p["q_norm.weight"] = ParamSpec((s.q_rank,), role="vector", init="ones_normal")
            p["uq"] = ParamSpec((self.q_size, s.q_rank))
        if s.sink:
            p["sink"] = ParamSpec((s.num_heads,), role="vector", init="normal")
        return p

    def bind(self, tensors):
        s = self.spec
        super().bind(tensors)
        # U_h^T per head, [heads, kv_rank, key_dim]: the map that carries a head's query into the latent's space
        self.uk_t = self.p_uk.view(s.num_heads, s.key_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.uv_h = self.p_uv.view(s.num_heads, s.value_dim, s.kv_rank)
        self.sink_f32 = self.p_sink.float().contiguous() if s.sink else None

    def cache_need(self):
        return LatentCacheNeed(self.spec.kv_rank + self.spec.rot_dim, self.spec.window)

    # ------------------------------------------------------------------ one step
    def forward(self, x, ctx):
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T, dt, dev = x.shape[0], x.dtype, x.device
        H, D, R, C = s.num_heads, s.key_dim, s.rot_dim, s.kv_rank
        proj = ctx.buffer("latent.in", (T, self.in_size), dt, dev)
        ops.linear(x, self.p_in, proj)
        if s.q_rank is not None:
            cq = ctx.buffer("latent.cq", (T, s.q_rank), dt, dev)
            ops.rmsnorm_columns(proj[:, :s.q_rank], self.p_q_norm_weight, s.eps, cq)
            q = ctx.buffer("latent.q", (T, self.q_size), dt, dev)
            ops.linear(cq, self.p_uq, q)
            q_off = 0
        else:
            q, q_off = proj, 0
        cos, sin, _ = self.position.rotary_tables() if self.position is not None else (None, None, 0)
        q_rot = ctx.buffer("latent.q_rot", (H, T, R), dt, dev) if R else None
        ops.latent_write(proj, self.c_off, self.p_kv_norm_weight, s.eps, C, R, cos, sin, b, kv.block_table, kv.page_size,
                         kv.k, ctx.write_cache, xq=q, q_off=q_off, heads=H, dim=D, q_rot=q_rot)
        # the unrotated parts of the queries, head by head, into the latent's space
        q_heads = q[:, q_off:q_off + self.q_size].view(T, H, self.q_head)[:, :, :D].transpose(0, 1)      # [H, T, D]
        q_lat = ctx.buffer("latent.q_lat", (H, T, C), dt, dev)
        ops.linear_heads(q_heads, self.uk_t, q_lat)
        o_lat = ctx.buffer("latent.o_lat", (H, T, C), dt, dev)
        ops.latent_attention(q_lat, q_rot, kv.k, b, kv.block_table, kv.page_size, self.sink_f32, o_lat, s.scale, s.window)
        v = ctx.buffer("latent.v", (H, T, s.value_dim), dt, dev)
        ops.linear_heads(o_lat, self.uv_h, v)
        packed = ctx.buffer("latent.packed", (T, H * s.value_dim), dt, dev)
        ops.head_pack_gate(v, proj[:, self.g_off:self.g_off + H] if s.gate else None, packed)
        y = ctx.buffer("latent.y", (T, s.hidden_size), dt, dev)
        ops.linear(packed, self.p_o, y)
        return y
