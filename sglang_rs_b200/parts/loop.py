"""What runs at the head of a pass over a stretch of layers that a model walks several times.

x <- W_in [x ; x0] + step[t]: the stream x is joined with the embedding output x0 (x first), mixed by one
matrix [width, 2 width], and the pass's own vector step[t] (t = 0, 1, ...: the number of the pass) is added.
The product's result and the sum are 32-bit: they become the residual stream.

:class:`PassSum` is the head of a pass without tensors: x <- x + x0, the embedding output added to the stream, in 32-bit.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import Part, TensorSpec, matrix_to, scale_to
from .norm import add_pending


class PassEntry(Part):
    graph_safe = True

    def __init__(self, width: int, passes: int, matrix_name: str, step_name: str):
        self.width, self.passes, self.matrix_name, self.step_name = int(width), int(passes), matrix_name, step_name
        self.matrix = self.steps = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.matrix_name: TensorSpec((self.width, 2 * self.width)),
                self.step_name: TensorSpec((self.passes, self.width))}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.matrix = matrix_to(tensors[self.matrix_name], device, dtype)
        self.steps = scale_to(tensors[self.step_name], device)

    def forward(self, ctx, residual: torch.Tensor, delta, origin: torch.Tensor, pass_index: int) -> torch.Tensor:
        """The new residual stream (a tensor of its own; ``residual`` and ``origin`` are left as they are, apart
        from the pending term, which is added to ``residual``)."""
        joined = torch.empty((residual.shape[0], 2 * self.width), dtype=ctx.dtype, device=residual.device)
        add_pending(residual, delta, None, joined, extra=origin)
        return ops.linear(joined, self.matrix, self.steps[pass_index], out_dtype=torch.float32, error_word=ctx.error_word)


class PassSum(Part):
    """x <- x + x0 at the head of a pass: the embedding output is added to the stream, once, right before the pass's
    first layer.  The pending term of the layer before (with its norm, if it has one), this sum and the write of the
    stream are one kernel; all 32-bit.  The stream is changed in place, so the model keeps the embedding output apart."""
    graph_safe = True
    #: the stream that ``forward`` returns is the one it was given
    in_place = True

    def forward(self, ctx, residual: torch.Tensor, delta, origin: torch.Tensor, pass_index: int) -> torch.Tensor:
        add_pending(residual, delta, None, None, addend=origin)
        return residual
