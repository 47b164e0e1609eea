"""RMSNorm (python/helios/exec/model.py:95-114): statistics in float32, no mean
subtraction, no bias.  The weight is kept in float32 in both modes."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Norm, WeightSpec, register_part


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, tensor_name: str = "weight") -> None:
        """``tensor_name``: the weight's name below the part's prefix ("" where the
        checkpoint names the norm itself)."""
        self.width = width
        self.eps = float(eps)
        self.tensor_name = tensor_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.tensor_name: WeightSpec((self.width,), kind="vector", init="ones_jitter")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, residual, delta, out_dtype, rows=None):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype, rows)

    def add_normed(self, residual, y, out_dtype):
        """``y`` None: only the residual in ``out_dtype``."""
        return ops.rmsnorm_add(residual, y, self.weight, self.eps, out_dtype)


register_part("norm", "rmsnorm", RMSNorm)
