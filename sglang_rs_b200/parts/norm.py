"""RMSNorm, fused with the residual sum that precedes it.

y = x / sqrt(mean(x^2) + eps) * w with eps inside the root and the weight multiplying
directly (reference: crates/sglang-kernel/src/cpu.rs:26-34).  The sum x = residual + delta,
the mean of squares and the scaling are 32-bit; only the result is rounded to the
compute dtype.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Norm, NormedDelta, TensorSpec, scale_to


class RmsNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,), "scale")}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.weight = scale_to(tensors[self.weight_name], device)

    def spec(self):
        return ("rms", self.weight, None, self.eps)

    def native_record(self):
        """This norm for the step executor: its scale, eps and width."""
        from ..ops.records import SxNorm
        return None if self.weight is None else SxNorm(self.weight.data_ptr(), self.eps, self.width)

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                 row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (in place, unless rows are picked); returns norm(residual).
        ``delta`` may be float32 [parts, rows, width]: partial sums, added in order."""
        rows = residual.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.width), dtype=out_dtype, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, row_index=row_index,
                        write_residual=row_index is None)
        return out


class GroupedRmsNorm(Norm):
    """An RMS norm taken in ``groups`` equal consecutive parts of the row: each part is divided by its own
    sqrt(mean(part^2) + eps), then the whole row is multiplied by the weight and by ``scale`` (a constant, 1 unless a
    design weighs the normed term in a residual sum).  With one group and scale 1 it is the plain RMS norm.
    ``weight_offset``: the checkpoint stores the weight minus this number (1 for weights kept around zero: the row is
    multiplied by 1 + w); the sum is taken once, at load, in 32-bit.  Like
    :class:`LayerNorm` it takes the pending term as a tensor or as a :class:`NormedDelta`, so a norm behind a sublayer,
    the residual sum and this norm run in one kernel; means, roots and the sum are 32-bit."""
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str, groups: int = 1, scale: float = 1.0,
                 weight_offset: float = 0.0):
        if groups < 1 or width % groups:
            raise ValueError(f"a row of {width} entries does not split into {groups} equal parts")
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.groups, self.scale, self.weight_offset = int(groups), float(scale), float(weight_offset)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        # a weight stored minus an offset lies around zero
        return {self.weight_name: TensorSpec((self.width,), "normal" if self.weight_offset else "scale")}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.weight = scale_to(tensors[self.weight_name], device)
        if self.weight_offset:
            self.weight = self.weight + self.weight_offset

    def spec(self):
        return ("rms", self.weight, None, self.eps, self.groups, self.scale)

    def add_norm(self, residual: torch.Tensor, delta, out_dtype: torch.dtype,
                 row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = residual.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.width), dtype=out_dtype, device=residual.device)
        add_pending(residual, delta, self.spec(), out, row_index)
        return out


class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b, eps inside the root, all in 32-bit.

    ``add_norm`` takes the pending term as a tensor (added as it is) or as a :class:`NormedDelta` (its own
    norm is applied first, of either kind), adds it to the residual stream and returns this norm of the sum:
    one kernel for "norm behind a sublayer, residual sum, norm ahead of the next sublayer"."""
    graph_safe = True
    kind = "layer"

    def __init__(self, width: int, eps: float, weight_name: str, bias_name: Optional[str]):
        self.width, self.eps, self.weight_name, self.bias_name = int(width), float(eps), weight_name, bias_name
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.weight_name: TensorSpec((self.width,), "scale")}
        if self.bias_name:
            specs[self.bias_name] = TensorSpec((self.width,))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.weight = scale_to(tensors[self.weight_name], device)
        self.bias = scale_to(tensors[self.bias_name], device) if self.bias_name else None

    def spec(self):
        return ("layer", self.weight, self.bias, self.eps)

    def add_norm(self, residual: torch.Tensor, delta, out_dtype: torch.dtype,
                 row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = residual.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.width), dtype=out_dtype, device=residual.device)
        add_pending(residual, delta, self.spec(), out, row_index)
        return out


def add_pending(residual: torch.Tensor, delta, outer, out: Optional[torch.Tensor],
                row_index: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
                addend: Optional[torch.Tensor] = None) -> None:
    """residual += delta (a tensor, a :class:`NormedDelta` or None) (+ ``addend``), then ``out`` = ``outer`` of the sum."""
    inner = None
    if isinstance(delta, NormedDelta):
        inner, delta = delta.norm.spec(), delta.values
    ops.norm_add_norm(residual, delta, inner, outer, out, row_index=row_index, write_residual=row_index is None,
                      extra=extra, addend=addend)
