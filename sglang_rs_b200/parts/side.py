"""A token's own input to a layer, read from a table that the token indexes.

For the residual stream x of a row whose token is t:  g = act(W_gate x) * e  with e the layer's slice
[offset, offset + dim) of row t of a table [vocab, >= offset + dim];  y = W_proj g.  The block that holds the part
adds the RMS norm of y (a plain weight, the part's ``norm``) to the stream.  The table belongs to the embedding (one
table for all layers, loaded once: ``TokenEmbedding(side_tables=...)``); each layer holds its own two matrices and its
norm's weight.  W_gate reads the stream rounded to the compute dtype; the norm and the sum are 32-bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping

import torch

from .. import ops
from .base import Norm, Part, TensorSpec, matrix_to
from .embedding import TokenEmbedding


@dataclass(frozen=True)
class TokenSideNames:
    gate: str
    proj: str


class TokenSideInput(Part):
    graph_safe = True

    def __init__(self, hidden: int, dim: int, offset: int, embedding: TokenEmbedding, table_name: str, norm: Norm,
                 names: TokenSideNames, activation: str = "gelu_tanh"):
        """``norm``: the norm of y as the residual sum takes it (its ``spec()`` rides in the next norm kernel)."""
        if dim <= 0 or offset < 0 or offset + dim > embedding.side_tables.get(table_name, 0):
            raise ValueError(f"entries {offset} .. {offset + dim} do not lie inside the rows of table {table_name!r}")
        if activation not in ops.ACTIVATIONS or activation in ops.PARAMETRIC_ACTIVATIONS:
            raise ValueError(f"unsupported activation {activation}")
        self.hidden, self.dim, self.offset = int(hidden), int(dim), int(offset)
        self.embedding, self.table_name, self.norm, self.names, self.activation = embedding, table_name, norm, names, activation
        self.w_gate = self.w_proj = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.names.gate: TensorSpec((self.dim, self.hidden)), self.names.proj: TensorSpec((self.hidden, self.dim))}
        specs.update(self.norm.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.w_gate = matrix_to(tensors[self.names.gate], device, dtype)
        self.w_proj = matrix_to(tensors[self.names.proj], device, dtype)
        self.norm.load(tensors, device, dtype)

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        """``x``: the stream rounded to the compute dtype [rows, hidden]; returns y [rows, hidden], not yet normed."""
        gate = ops.linear(x, self.w_gate, error_word=ctx.error_word)
        gated = torch.empty_like(gate)
        ops.token_gate(gate, ctx.token_ids, self.embedding.side[self.table_name], self.offset, gated, ctx.error_word,
                       self.activation)
        return ops.linear(gated, self.w_proj, error_word=ctx.error_word)
