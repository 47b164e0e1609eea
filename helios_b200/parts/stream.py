"""Parts that stand between blocks and rewrite the whole residual stream."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import StreamStage, WeightSpec


class StreamInputMix(StreamStage):
    """x <- W [x ; x0]: the stream beside the model's embedded input x0 (the stream as the
    input stage left it), through one matrix [width, 2 width] whose first ``width`` columns
    meet x.  A model that runs a stretch of its layers several times over places it before
    the first layer of every pass.  The two halves are rounded to the activation dtype for
    the product; the sums and the new stream are float32."""

    needs_input = True
    _ROWS = "stream_input_mix.rows"

    def __init__(self, width: int, tensor_name: str = "in") -> None:
        self.width = width
        self.tensor_name = tensor_name
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.tensor_name: WeightSpec((self.width, 2 * self.width))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name].contiguous()

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width)

    def forward(self, ctx, residual: torch.Tensor) -> torch.Tensor:
        # the x0 half is written once a step, the x half before every product
        rows = ctx.step_tables.get((self._ROWS, id(self)))
        if rows is None:
            rows = torch.empty((residual.shape[0], 2 * self.width), dtype=ctx.act_dtype, device=residual.device)
            ops.cast_rows(rows, self.width, ctx.stream_input)
            ctx.step_tables[(self._ROWS, id(self))] = rows
        ops.cast_rows(rows, 0, residual)
        return ops.linear_logits(rows, self.weight)
