"""Routed feed-forward: a router picks ``top`` of ``experts`` small gated feed-forward
layers for every token.

    z = W_router h  (float32 sums; h in the activation dtype)
    s = sigmoid(z); the ``top`` experts with the largest s are chosen
    out = sum over the chosen e of expert_e(s_e * h)

The weight is the expert's score itself, not renormalised over the chosen ones, and it
multiplies the expert's INPUT (the experts are not linear, so this is not the same as
weighting their outputs).  An expert is down(act(gate x) * up x) without biases, with the
activation and its constants as parameters (the clamped form of ``ops.glu_act`` here).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, WeightSpec, register_part


class RoutedExperts(FeedForward):
    def __init__(self, width: int, inner: int, experts: int, top: int, limit: float,
                 router_name: str = "router", expert_prefix: str = "e",
                 names=("gate", "up", "down")) -> None:
        if not 0 < top <= experts:
            raise ValueError(f"top {top} of {experts} experts")
        self.width, self.inner, self.experts, self.top = width, inner, experts, top
        self.limit = float(limit)
        self.router_name, self.expert_prefix, self.names = router_name, expert_prefix, tuple(names)
        self.w_router = self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        g, u, d = self.names
        specs = {}
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            specs[p + g] = WeightSpec((self.inner, self.width))
            specs[p + u] = WeightSpec((self.inner, self.width))
            specs[p + d] = WeightSpec((self.width, self.inner))
        specs[self.router_name] = WeightSpec((self.experts, self.width))
        return specs

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ("moe",)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u, d = self.names
        p = self.expert_prefix
        self.w_router = tensors[self.router_name].contiguous()
        self.w_gate_up = torch.stack([torch.cat([tensors[f"{p}{e}.{g}"], tensors[f"{p}{e}.{u}"]], dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[f"{p}{e}.{d}"] for e in range(self.experts)]).contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear_logits(x, self.w_router)          # float32 [T, experts]
        ids, weights = ops.moe_topk(logits, self.top)
        return ops.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, self.limit)


register_part("feed_forward", "routed_experts", RoutedExperts)
