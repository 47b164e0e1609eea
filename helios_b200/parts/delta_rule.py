"""A recurrent mixer: the gated delta rule with one decay per head and key channel.

q, k (``kv_heads`` x ``dk``; head h reads q/k head h // (heads / kv_heads)) and v (``heads``
x ``dv``) each pass a short causal convolution over time per channel and silu; q and k are
made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dk^-1/2.  Per token and
head, with beta = sigmoid(W_b h) and g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))
(one value per key channel):

    S <- g (.) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

o is RMS-normed per head over dv, times a weight shared by the heads, times
sigmoid(W_g2 W_g1 h); then the output projection.  A request's slot holds S (float32) and
the last taps - 1 inputs of the convolutions; nothing is kept per token.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Mixer, StateSpec, WeightSpec, register_part


class GatedDeltaMixer(Mixer):
    def __init__(self, width: int, heads: int, kv_heads: int, dk: int, dv: int, taps: int,
                 decay_rank: int, gate_rank: int, eps: float) -> None:
        """``decay_rank`` / ``gate_rank``: inner sizes of the two-step projections of the decay
        (a1, a2) and of the output gate (g1, g2).  ``eps``: of the output norm."""
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} q/k heads")
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.width, self.heads, self.kv_heads = width, heads, kv_heads
        self.dk, self.dv, self.taps, self.eps = dk, dv, taps, float(eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.conv_channels = 2 * kv_heads * dk + heads * dv
        self.state_floats = heads * dk * dv
        self.w_in = self.w_a2 = self.w_g2 = self.w_o = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_weight = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.state_floats + self.conv_channels * (self.taps - 1),), torch.float32)

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ("delta_rule",)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        qk, v = self.kv_heads * self.dk, self.heads * self.dv
        a = self.heads * self.dk
        return {
            "q": WeightSpec((qk, self.width)), "q.conv": WeightSpec((qk, self.taps), kind="vector", std=0.3),
            "k": WeightSpec((qk, self.width)), "k.conv": WeightSpec((qk, self.taps), kind="vector", std=0.3),
            "v": WeightSpec((v, self.width)), "v.conv": WeightSpec((v, self.taps), kind="vector", std=0.3),
            "b": WeightSpec((self.heads, self.width)),
            "A_log": WeightSpec((self.heads,), kind="vector", std=0.5),
            "norm": WeightSpec((self.dv,), kind="vector", init="ones_jitter"),
            "a1": WeightSpec((self.decay_rank, self.width)), "a2": WeightSpec((a, self.decay_rank)),
            "dt_bias": WeightSpec((a,), kind="vector", std=0.5),
            "g1": WeightSpec((self.gate_rank, self.width)), "g2": WeightSpec((v, self.gate_rank)),
            "o": WeightSpec((self.width, v)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = tensors
        # one projection for everything that reads the mixer's input
        self.w_in = torch.cat([t["q"], t["k"], t["v"], t["a1"], t["g1"], t["b"]], dim=0).contiguous()
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).contiguous()
        self.w_a2, self.w_g2, self.w_o = t["a2"].contiguous(), t["g2"].contiguous(), t["o"].contiguous()
        self.a_log, self.dt_bias = t["A_log"].contiguous(), t["dt_bias"].contiguous()
        self.norm_weight = t["norm"].contiguous()

    def forward(self, ctx, x: torch.Tensor, cache, state: torch.Tensor) -> torch.Tensor:
        C, Ra, Rg = self.conv_channels, self.decay_rank, self.gate_rank
        proj = ops.linear(x, self.w_in)
        qkv = ops.causal_conv_silu(ctx, proj, C, self.conv_w, state[:, self.state_floats:])
        a_raw = ops.linear_rows(proj[:, C:C + Ra], self.w_a2)
        gate = ops.linear_rows(proj[:, C + Ra:C + Ra + Rg], self.w_g2)
        qk = self.kv_heads * self.dk
        o = ops.delta_rule(ctx, qkv, (0, qk, 2 * qk), proj[:, C + Ra + Rg:], a_raw, self.a_log,
                           self.dt_bias, state[:, :self.state_floats], self.heads, self.kv_heads,
                           self.dk, self.dv)
        return ops.linear(ops.gated_rmsnorm(o, gate, self.norm_weight, self.heads, self.dv, self.eps),
                          self.w_o)


register_part("mixer", "gated_delta", GatedDeltaMixer)
