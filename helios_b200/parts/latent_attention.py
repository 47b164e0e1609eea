"""Attention over a low-rank latent cache.

Per token the mixer keeps ONE row: the latent c (``rank`` values, RMS-normed) and a rotated
key part r (``rot`` values) that all heads share.  Head h's key is [W_uk[h] c | r] and its
value W_uv[h] c; a query is [q_nope (``nope`` values) | q_rot (``rot`` values, rotated)] and

    score = (q_nope . W_uk[h] c + q_rot . r) * scale,     softmax over the positions <= own.

The up-projections are folded into the query and the output, so that the cache is never
expanded: q_lat = W_uk[h]^T q_nope attends the latents themselves, and the head's output is
W_uv[h] (sum_j p_j c_j).  Rotary pairs dimension 2i with 2i + 1 over the first
``position.rotary_dim`` of the ``rot`` values.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import LayerCache, Mixer, PagedCacheSpec, WeightSpec, register_part


class LatentAttention(Mixer):
    def __init__(self, width: int, heads: int, nope: int, rot: int, vdim: int, rank: int,
                 scale: float, eps: float, position,
                 names=("q", "dkv", "dkv.norm", "uk", "uv", "o")) -> None:
        """``position``: the rotary encoding whose tables rotate the ``rot`` parts
        (``position.rotary_dim`` <= rot, even).  ``scale`` multiplies the scores as given.
        ``eps``: of the latent's RMS norm."""
        if position.rotary_dim > rot:
            raise ValueError(f"{position.rotary_dim} rotated dimensions exceed the rotated part of {rot}")
        self.width, self.heads, self.nope, self.rot = width, heads, nope, rot
        self.vdim, self.rank = vdim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.position = position
        self.names = tuple(names)
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.norm_weight = None

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(1, self.rank + self.rot, None, planes=1)

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ("latent_attention",)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, dkv, norm, uk, uv, o = self.names
        H = self.heads
        return {
            q: WeightSpec((H * (self.nope + self.rot), self.width)),
            dkv: WeightSpec((self.rank + self.rot, self.width)),
            norm: WeightSpec((self.rank,), kind="vector", init="ones_jitter"),
            uk: WeightSpec((H * self.nope, self.rank)),
            uv: WeightSpec((H * self.vdim, self.rank)),
            o: WeightSpec((self.width, H * self.vdim)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, dkv, norm, uk, uv, o = self.names
        H = self.heads
        self.w_in = torch.cat([tensors[q], tensors[dkv]], dim=0).contiguous()
        self.norm_weight = tensors[norm].contiguous()
        # [heads, rank, nope]: the matrix that takes a head's q_nope to the latent space
        self.w_uk_t = tensors[uk].view(H, self.nope, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[uv].view(H, self.vdim, self.rank).contiguous()
        self.w_o = tensors[o].contiguous()

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        H, T = self.heads, x.shape[0]
        proj = ops.linear(x, self.w_in)
        cos, sin = self.position.tables(ctx)
        table = ctx.block_tables[cache.group]
        ops.latent_prepare(proj, cache.k_pages, self.norm_weight, cos, sin, ctx.positions,
                           ctx.seq_of_token, table, H, self.nope, self.rot, self.rank,
                           cache.page_size, self.eps, write_cache=cache.write)
        q = proj[:, :H * (self.nope + self.rot)].view(T, H, self.nope + self.rot)
        q_lat = ops.head_gemm(q[:, :, :self.nope], self.w_uk_t)
        o_lat = ops.latent_attention(ctx, q_lat, q[:, :, self.nope:], cache.k_pages, table,
                                     self.rank, self.rot, cache.page_size, self.scale)
        o = ops.head_gemm(o_lat, self.w_uv)
        return ops.linear(o.reshape(T, H * self.vdim), self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
