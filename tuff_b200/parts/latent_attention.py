"""Attention over a latent cache.

Per token the mixer keeps one small vector c (RMS-normed, `kv_rank` wide) and one rotated key part kr
(`rot_dim` wide) that all heads share; a head's plain key part and its value are linear images of c:
k_h = [U_h c | kr], v_h = V_h c.  A query head is [plain (`dim`) | rotated (`rot_dim`)], the score is
(q_plain . U_h c + q_rot . kr) * scale, causal, with a learned sink per head in the softmax's denominator.

Only [c | kr] is cached, one row per token in pages of a single key/value head.  The query is carried
into the latent space instead of the cache being expanded: q~_h = [U_h^T q_plain | q_rot], so that the score
is q~_h . [c | kr]; attention runs over the cached rows with the values being the rows' first `kv_rank`
elements, and V_h is applied to the weighted sum of latents afterwards.  This is the same sum in another
order; scores, softmax, the norm of c and the rotation are fp32.

Weights: `q` [H (dim + rot_dim), d], `dkv` [kv_rank + rot_dim, d], `dkv_norm` [kv_rank], `uk` [H dim, kv_rank],
`uv` [H vdim, kv_rank], `sink` [H], `o` [d, H vdim].  The rotation pairs neighbouring elements (2i, 2i+1) of the
first `rot_dims` elements of the rotated part, at the angle pos * rot_base^(-2i / rot_dims).
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import Mixer, PagedKVNeed, WeightDecl, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, d_model: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int,
                 rot_base: float, rot_dims: int | None = None, scale: float | None = None, norm_eps: float = 1e-6,
                 sink: str | None = "learned"):
        self.d, self.H, self.dim, self.rd = int(d_model), int(num_heads), int(head_dim), int(rot_dim)
        self.vd, self.rank = int(v_head_dim), int(kv_rank)
        self.rot_dims = self.rd if rot_dims is None else int(rot_dims)
        if self.rd % 2 or self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rd:
            raise ValueError(f"latent_attention: rot_dim {self.rd} / rotated span {self.rot_dims} must be even, the span within rot_dim")
        self.rot_base = float(rot_base)
        self.scale = float(scale) if scale is not None else (self.dim + self.rd) ** -0.5
        self.eps = float(norm_eps)
        if sink not in (None, "learned"):
            raise ValueError(f"latent_attention: sink {sink!r}; choose learned or None")
        self.learned_sink = sink == "learned"
        self._inv_freq = None

    def weight_decls(self):
        H, d = self.H, self.d
        decls = {"q": WeightDecl((H * (self.dim + self.rd), d)), "dkv": WeightDecl((self.rank + self.rd, d)),
                 "dkv_norm": WeightDecl((self.rank,), role="vector", init="norm"),
                 "uk": WeightDecl((H * self.dim, self.rank)), "uv": WeightDecl((H * self.vd, self.rank)),
                 "o": WeightDecl((d, H * self.vd))}
        if self.learned_sink:
            decls["sink"] = WeightDecl((H,), role="vector")
        return decls

    def cache_need(self):
        return PagedKVNeed(kv_heads=1, head_dim=self.rank + self.rd, v_head_dim=self.rank, values_in_keys=True)

    def bind(self, weights, act_dtype):
        super().bind(weights, act_dtype)
        H = self.H
        self.w_in = torch.cat([weights["q"], weights["dkv"]], dim=0).contiguous()          # one product for q, c and kr
        # U_h^T as the matrix of a product: [H, kv_rank, dim]; V_h: [H, vdim, kv_rank]
        self.ukt = weights["uk"].view(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = weights["uv"].view(H, self.vd, self.rank).contiguous()
        self.wo = weights["o"]
        self.c_norm = weights["dkv_norm"]
        self.sinks = weights["sink"].contiguous() if self.learned_sink else None
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        inv = (self.rot_base ** (-2.0 * i / max(self.rot_dims, 1))).astype(np.float32)
        self._inv_freq = torch.from_numpy(inv).to(self.wo.device)
        self.w = {"o": self.wo}

    def forward(self, ctx, cache, h, residual, reads_only=False):
        T = h.shape[0]
        H, dim, rd, rank, vd = self.H, self.dim, self.rd, self.rank, self.vd
        hl = rank + rd
        dev = h.device
        qd = torch.empty((T, H * (dim + rd) + hl), dtype=self.act_dtype, device=dev)
        ops.linear(h, self.w_in, qd)
        ql = torch.empty((T, H, hl), dtype=self.act_dtype, device=dev)          # the query in the latent space
        table = ctx.block_tables[cache.group]
        ops.latent_prepare(qd, ql, self.c_norm, self._inv_freq, ctx.positions, ctx.row_of_token, table, cache.k_pages,
                           H, dim, rd, rank, self.rot_dims, self.eps, write_kv=not reads_only)
        ops.head_linear(qd[:, : H * (dim + rd)].unflatten(1, (H, dim + rd))[:, :, :dim], self.ukt, ql[:, :, :rank])
        lat = torch.empty((T, H * rank), dtype=self.act_dtype, device=dev)
        ops.paged_attention(ql.view(T, H * hl), cache.k_pages, None, table, ctx.positions, ctx.row_of_token, lat,
                            H, 1, hl, self.scale, 0, ctx=ctx, sink=self.sinks, v_head_dim=rank, values_in_keys=True)
        att = torch.empty((T, H, vd), dtype=self.act_dtype, device=dev)
        ops.head_linear(lat.view(T, H, rank), self.uv, att)
        ops.linear(att.view(T, H * vd), self.wo, residual, accumulate=True)
