"""Grouped-query attention over the paged cache
(python/helios/exec/model.py:156-251; math of python/helios/exec/paged_attn.py:264-408).

One fused projection gives q, k and v (+ bias where the configuration has one);
one kernel rotates q and k and writes k and v into the request's pages before
attending, so a portion of a prompt sees itself (model.py:203-206); attention
runs over the cache for every token of the batch, whatever mix of prompt
portions and single decoded tokens it is; then the output projection.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import DeferredNorm, LayerCache, Mixer, PagedCacheSpec, WeightSpec, register_part
from .norm import RMSNorm


class GQAAttention(Mixer):
    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, qkv_bias: bool, window: Optional[int] = None,
                 rotary: bool = True, position=None) -> None:
        """``position``: the encoding whose cos/sin tables rotate q and k (its
        ``tables(ctx)``); None takes the tables the plan's own encoding left on the step
        context.  ``rotary=False``: no rotation at all."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported (even, at most 256)")
        self.width = width
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qkv_bias = qkv_bias
        self.window = window
        self.rotary = rotary
        self.position = position
        self.w_qkv = self.b_qkv = self.w_o = None

    # ---------------------------------------------------------------- what it keeps
    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def kernel_libraries(self, dtype):
        return (ops.linear_libraries(dtype, self.width)
                + ops.attention_libraries(dtype, self.num_heads, self.num_kv_heads, self.head_dim))

    # ---------------------------------------------------------------- tensors
    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, kv = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {
            "q_proj.weight": WeightSpec((q, self.width)),
            "k_proj.weight": WeightSpec((kv, self.width)),
            "v_proj.weight": WeightSpec((kv, self.width)),
            "o_proj.weight": WeightSpec((self.width, q)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = WeightSpec((q,), kind="vector", init="normal")
            specs["k_proj.bias"] = WeightSpec((kv,), kind="vector", init="normal")
            specs["v_proj.bias"] = WeightSpec((kv,), kind="vector", init="normal")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]], dim=0).contiguous()

    # ---------------------------------------------------------------- forward
    def _rotary_tables(self, ctx):
        if not self.rotary:
            return None, None
        if self.position is not None:
            return self.position.tables(ctx)
        return ctx.rotary_cos, ctx.rotary_sin

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm, cache: LayerCache, state=None,
                              pre=None, then=None):
        """Steps of few tokens run without norm launches: q|k|v takes the 1 / rms of ``pre``
        as a factor on its accumulators (the norm kernel runs where nothing was handed over),
        and the output projection adds into the residual and leaves ``then`` all but done."""
        if ctx.act_dtype != torch.bfloat16 or type(norm) is not RMSNorm or cache is None \
                or not ops.deferred_norm_fits(ctx.num_tokens, self.w_qkv, self.w_o):
            return False
        if pre is not None:
            qkv = ops.linear_bf16(pre.scaled, self.w_qkv, self.b_qkv, sumsq=pre.sumsq, eps=norm.eps)
        else:
            qkv = ops.linear_bf16(norm.add_forward(residual, None, ctx.act_dtype), self.w_qkv, self.b_qkv)
        attn = self._attend(ctx, qkv, cache)
        if type(then) is RMSNorm:
            scaled, sumsq = ops.linear_bf16(attn, self.w_o, residual=residual, norm_weight=then.weight)
            return DeferredNorm(then, scaled, sumsq)
        ops.linear_bf16(attn, self.w_o, residual=residual)
        return True

    def _attend(self, ctx, qkv: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        table = ctx.block_tables[cache.group]
        cos, sin = self._rotary_tables(ctx)
        return ops.attention(ctx, qkv, cache.k_pages, cache.v_pages, table, self.num_heads,
                             self.num_kv_heads, self.head_dim, cache.page_size, self.window,
                             self.scale, fresh=(cos, sin, cache.write))

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        return ops.linear(self._attend(ctx, ops.linear(x, self.w_qkv, self.b_qkv), cache), self.w_o)


register_part("mixer", "gqa_attention", GQAAttention)


def distance_slopes(num_heads: int, exponent: float = 8.0):
    """Slope of head h = 2 ^ (-exponent * (h + 1) / heads): the geometric sequence a linear
    distance bias on the scores usually takes."""
    return [2.0 ** (-exponent * (h + 1) / num_heads) for h in range(num_heads)]


class SinkGQAAttention(Mixer):
    """Grouped-query attention without rotation whose score carries the position:

        q = norm_q(W_q h) * temp(p),   k = norm_k(W_k h),   v = W_v h
        s_ij = q_i . k_j * scale - slope_h * (i - j)              (j <= i)
        p_ij = exp(s_ij) / (1 + sum_j exp(s_ij))                  (``sink``: a key of score 0 without a value)
        out  = W_o concat_h(sigmoid(W_g h)_h * sum_j p_ij v_j)    (``head_gate``: one number a head)

    norm_q / norm_k: RMS norm over a head's ``head_dim`` values with one weight shared by all
    heads (``qk_norm``); temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
    (``q_temperature`` = (coef, every) or None); slope_h from ``slopes`` (a list, one a head, or
    None).  Values may have another size than keys (``value_dim``).  Every option can be left
    out; the constants are the caller's.  One fused projection gives q | k | v | gate; q and
    k are normed and k and v written into the request's pages by one launch before attention,
    or, in steps of single tokens, inside the decode kernel; the gate is applied where
    attention writes its output."""

    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 value_dim: Optional[int] = None, qk_norm: bool = True, eps: float = 1e-6,
                 q_temperature=None, slopes=None, sink: bool = True, head_gate: bool = True,
                 window: Optional[int] = None,
                 names=("q", "k", "v", "o", "g", "q.norm", "k.norm")) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        value_dim = value_dim or head_dim
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"heads of {head_dim} / {value_dim} values are not supported (at most 256)")
        if slopes is not None and len(slopes) != num_heads:
            raise ValueError(f"{len(slopes)} slopes for {num_heads} heads")
        self.width, self.num_heads, self.num_kv_heads = width, num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale, self.eps = float(scale), float(eps)
        self.qk_norm, self.sink, self.head_gate = bool(qk_norm), bool(sink), bool(head_gate)
        self.q_temperature = None if not q_temperature else (float(q_temperature[0]), int(q_temperature[1]))
        self.slope_values = None if slopes is None else [float(x) for x in slopes]
        self.window = window
        self.names = tuple(names)
        self.w_in = self.w_o = self.q_weight = self.k_weight = self.slopes = None
        q, kv = num_heads * head_dim, num_kv_heads * head_dim
        self._gate_col = q + kv + num_kv_heads * value_dim

    # ---------------------------------------------------------------- what it keeps
    def cache_spec(self) -> PagedCacheSpec:
        vd = None if self.value_dim == self.head_dim else self.value_dim
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window, value_dim=vd)

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ops.option_attention_libraries(
            dtype, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim)

    # ---------------------------------------------------------------- tensors
    def weight_specs(self) -> Dict[str, WeightSpec]:
        nq, nk, nv, no, ng, nqn, nkn = self.names
        q, kv = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {nq: WeightSpec((q, self.width)), nk: WeightSpec((kv, self.width)),
                 nv: WeightSpec((self.num_kv_heads * self.value_dim, self.width)),
                 no: WeightSpec((self.width, self.num_heads * self.value_dim))}
        if self.head_gate:
            specs[ng] = WeightSpec((self.num_heads, self.width))
        if self.qk_norm:
            specs[nqn] = WeightSpec((self.head_dim,), kind="vector", init="ones_jitter")
            specs[nkn] = WeightSpec((self.head_dim,), kind="vector", init="ones_jitter")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        nq, nk, nv, no, ng, nqn, nkn = self.names
        mats = [tensors[nq], tensors[nk], tensors[nv]]
        if self.head_gate:
            mats.append(tensors[ng])
        rows = sum(m.shape[0] for m in mats)
        pad = -rows % 8            # rows of the fused projection's output stay 16-byte aligned
        if pad:
            mats.append(torch.zeros((pad, self.width), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[no].contiguous()
        if self.qk_norm:
            self.q_weight, self.k_weight = tensors[nqn].contiguous(), tensors[nkn].contiguous()
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float32, device=self.w_o.device)

    # ---------------------------------------------------------------- forward
    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        rows = ops.linear(x, self.w_in)
        table = ctx.block_tables[cache.group]
        coef, every = self.q_temperature or (0.0, 0)
        gate = rows[:, self._gate_col:self._gate_col + self.num_heads] if self.head_gate else None
        options = ops.AttentionOptions(slopes=self.slopes, sink=self.sink, gate=gate,
                                       value_dim=None if self.value_dim == self.head_dim else self.value_dim)
        attn = ops.attention(ctx, rows, cache.k_pages, cache.v_pages, table, self.num_heads,
                             self.num_kv_heads, self.head_dim, cache.page_size, self.window, self.scale,
                             options=options,
                             prepare=(self.q_weight, self.k_weight, self.eps, coef, every, cache.write))
        return ops.linear(attn, self.w_o)


register_part("mixer", "sink_gqa_attention", SinkGQAAttention)
