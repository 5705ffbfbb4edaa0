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
from .base import MIXERS, POSITION_ENCODINGS, LatentCacheNeed, Mixer, ParamSpec, Tiling


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
        # a cached vector's width: latent and rotated part, padded to whole 16s (the tensor-core kernels' head sizes)
        self.width = (s.kv_rank + s.rot_dim + 15) // 16 * 16

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
        return LatentCacheNeed(self.width, self.spec.window)

    def _on_tensor_cores(self):
        return ops.latent_on_tensor_cores(self.env.act_dtype, self.width)

    def batch_tilings(self):
        """The row blocks of the tensor-core attention kernel for prompt portions that this width runs on."""
        if not self._on_tensor_cores():
            return {}
        if self.width in ops.TC5_ATTENTION_HEAD_DIMS:
            return {ops.TILES_TC5: Tiling(ops.TC5_TILE_ROWS, heaviest_first=True)}
        return {ops.TILES_MMA: Tiling(ops.MMA_TILE_ROWS)}

    def graph_variant(self, n_tokens, longest_context):
        """A captured step cannot change the grid of the split-KV decode kernel: the number of key splits is fixed per
        captured graph (all query heads share the one key/value head)."""
        if not self._on_tensor_cores():
            return {}
        s = self.spec
        return {ops.decode_splits_key(s.num_heads, 1, s.window): ops.decode_splits_for(n_tokens, longest_context, s.num_heads, 1, s.window)}

    # ------------------------------------------------------------------ one step
    def forward(self, x, ctx):
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T, dt, dev = x.shape[0], x.dtype, x.device
        H, D, R, C, W = s.num_heads, s.key_dim, s.rot_dim, s.kv_rank, self.width
        proj = ctx.buffer("latent.in", (T, self.in_size), dt, dev)
        ops.linear(x, self.p_in, proj)
        if s.q_rank is not None:
            cq = ctx.buffer("latent.cq", (T, s.q_rank), dt, dev)
            ops.rmsnorm_columns(proj[:, :s.q_rank], self.p_q_norm_weight, s.eps, cq)
            q = ctx.buffer("latent.q", (T, self.q_size), dt, dev)
            ops.linear(cq, self.p_uq, q)
        else:
            q = proj                                             # the queries are the first columns of the projection
        cos, sin, _ = self.position.rotary_tables() if self.position is not None else (None, None, 0)
        # a head's query as the attention reads it: [its unrotated part carried into the latent's space | its rotated part]
        q_abs = ctx.buffer("latent.q_abs", (T, H * W), dt, dev)
        ops.latent_write(proj, self.c_off, self.p_kv_norm_weight, s.eps, C, R, cos, sin, b, kv.block_table, kv.page_size,
                         kv.k, ctx.write_cache, q, 0, H, D, q_abs)
        q_heads = q[:, :self.q_size].view(T, H, self.q_head)[:, :, :D].transpose(0, 1)                   # [H, T, D]
        ops.linear_heads(q_heads, self.uk_t, q_abs.view(T, H, W)[:, :, :C].transpose(0, 1))
        o_abs = ctx.buffer("latent.o_abs", (T, H * W), dt, dev)
        ops.latent_attention(q_abs, kv.k, b, kv.block_table, kv.page_size, self.sink_f32, o_abs, H, C, R, s.scale, s.window)
        # the weighted means of the latents, head by head, into the heads' value spaces
        packed = ctx.buffer("latent.packed", (T, H * s.value_dim), dt, dev)
        ops.linear_heads(o_abs.view(T, H, W)[:, :, :C].transpose(0, 1), self.uv_h, packed.view(T, H, s.value_dim).transpose(0, 1))
        if s.gate:
            ops.head_gate(packed, proj[:, self.g_off:self.g_off + H], H)
        y = ctx.buffer("latent.y", (T, s.hidden_size), dt, dev)
        ops.linear(packed, self.p_o, y)
        return y
