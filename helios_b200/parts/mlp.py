"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(python/helios/exec/model.py:321-337).  gate and up are one fused projection."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import DeferredNorm, FeedForward, WeightSpec, register_part
from .norm import RMSNorm


class SwiGLU(FeedForward):
    def __init__(self, width: int, inner: int) -> None:
        self.width = width
        self.inner = inner
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "gate_proj.weight": WeightSpec((self.inner, self.width)),
            "up_proj.weight": WeightSpec((self.inner, self.width)),
            "down_proj.weight": WeightSpec((self.width, self.inner)),
        }

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.linear_swiglu(x, self.w_gate_up), self.w_down)

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm, pre=None, then=None):
        """Steps of few tokens run without norm launches: gate|up takes the 1 / rms of ``pre``
        as a factor on its accumulators, and the down projection adds into the residual and
        leaves ``then`` all but done."""
        if ctx.act_dtype != torch.bfloat16 or type(norm) is not RMSNorm \
                or not ops.deferred_norm_fits(ctx.num_tokens, self.w_gate_up, self.w_down):
            return False
        if pre is not None:
            h = ops.linear_bf16(pre.scaled, self.w_gate_up, glu=True, sumsq=pre.sumsq, eps=norm.eps)
        else:
            h = ops.linear_bf16(norm.add_forward(residual, None, ctx.act_dtype), self.w_gate_up, glu=True)
        if type(then) is RMSNorm:
            scaled, sumsq = ops.linear_bf16(h, self.w_down, residual=residual, norm_weight=then.weight)
            return DeferredNorm(then, scaled, sumsq)
        ops.linear_bf16(h, self.w_down, residual=residual)
        return True


register_part("feed_forward", "swiglu", SwiGLU)


class GatedMLP(FeedForward):
    """Dense gated feed-forward down(act(gate(x)) * up(x)) with the activation as a parameter
    (``ops.GLU_KINDS``: "silu", "gelu_tanh", "clamped_swish" with its ``limit``) and optional
    biases on all three projections.  gate and up are one fused projection; the tensors are
    named ``names`` = (gate, up, down) below the part's prefix, a bias ``<name><bias_suffix>``."""

    def __init__(self, width: int, inner: int, activation: str = "silu", bias: bool = False,
                 limit: float = 0.0, names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"),
                 bias_suffix: str = ".b") -> None:
        if activation not in ops.GLU_KINDS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.GLU_KINDS)}")
        self.width = width
        self.inner = inner
        self.activation = activation
        self.bias = bool(bias)
        self.limit = float(limit)
        self.names = tuple(names)
        self.bias_suffix = bias_suffix
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        g, u, d = self.names
        specs = {g: WeightSpec((self.inner, self.width)), u: WeightSpec((self.inner, self.width)),
                 d: WeightSpec((self.width, self.inner))}
        if self.bias:
            s = self.bias_suffix
            specs[g + s] = WeightSpec((self.inner,), kind="vector")
            specs[u + s] = WeightSpec((self.inner,), kind="vector")
            specs[d + s] = WeightSpec((self.width,), kind="vector")
        return specs

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u, d = self.names
        self.w_gate_up = torch.cat([tensors[g], tensors[u]], dim=0).contiguous()
        self.w_down = tensors[d].contiguous()
        if self.bias:
            s = self.bias_suffix
            self.b_gate_up = torch.cat([tensors[g + s], tensors[u + s]], dim=0).contiguous()
            self.b_down = tensors[d + s].contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        if self.activation == "silu" and not self.bias:
            return ops.linear(ops.linear_swiglu(x, self.w_gate_up), self.w_down)
        gate_up = ops.linear(x, self.w_gate_up, self.b_gate_up)
        return ops.linear(ops.glu_act(gate_up, self.activation, self.limit), self.w_down, self.b_down)


register_part("feed_forward", "gated_mlp", GatedMLP)
