"""Token embedding and output head.

h0 = embed[token] * scale (scale 1 unless the architecture says otherwise; the product is 32-bit); logits = norm(h) . W_out^T with W_out the head's own
matrix or, if tied, the embedding table (reference:
crates/sglang-srt/src/cpu_reference.rs:741-752, :176-185).  Logits are 32-bit in every mode.

:class:`PairTokenEmbedding` adds a row of a second table that the token and the token before it choose
together, and writes the result once per copy of the residual stream.  The head may squash its logits:
z <- cap * tanh(z / cap).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Part, RequestState, TensorSpec, matrix_to


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, width: int, weight_name: str, scale: float = 1.0,
                 side_tables: Optional[Mapping[str, int]] = None):
        """``side_tables``: further tables indexed by the token (checkpoint name -> row width) that other parts read
        (``parts/side.py``); they are loaded once, here, and found in ``self.side[name]``."""
        self.vocab, self.width, self.weight_name, self.scale = int(vocab), int(width), weight_name, float(scale)
        self.table: Optional[torch.Tensor] = None
        self.side_tables = dict(side_tables or {})
        self.side: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.weight_name: TensorSpec((self.vocab, self.width))}
        for name, width in self.side_tables.items():
            specs[name] = TensorSpec((self.vocab, width))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.table = matrix_to(tensors[self.weight_name], device, dtype)
        self.side = {name: matrix_to(tensors[name], device, dtype) for name in self.side_tables}

    def native_record(self):
        """The step executor reads the table itself; the record says only that there is one (it knows no scale)."""
        return None if self.table is None or self.scale != 1.0 else True

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        residual = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embedding(token_ids, self.table, residual, ctx.error_word, self.scale)
        return residual


class PairTokenEmbedding(Part):
    """h0 = embed[token] * scale + pairs[(previous * mul_prev + token * mul_cur) mod buckets]; a sequence's first
    token takes the table's last row (number ``buckets``).  The previous token of a request's first row in a step
    is remembered on the device, one int32 per request (``cache_need``), so that portions of a prompt and decoded
    tokens, also tokens that never reach the host, continue where the step before ended.  ``pair_name`` None: no
    second table.  The result is written ``copies`` times per row: float32 [rows, copies * width]."""
    graph_safe = True

    def __init__(self, vocab: int, width: int, weight_name: str, scale: float = 1.0, *, copies: int = 1,
                 pair_name: Optional[str] = None, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0):
        if pair_name is not None and buckets <= 0:
            raise ValueError("a pair table needs a positive number of buckets")
        self.vocab, self.width, self.weight_name, self.scale = int(vocab), int(width), weight_name, float(scale)
        self.copies, self.pair_name = int(copies), pair_name
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.table: Optional[torch.Tensor] = None
        self.pairs: Optional[torch.Tensor] = None

    def cache_need(self):
        return RequestState((1,), torch.int32) if self.pair_name is not None else None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.weight_name: TensorSpec((self.vocab, self.width))}
        if self.pair_name is not None:
            specs[self.pair_name] = TensorSpec((self.buckets + 1, self.width))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.table = matrix_to(tensors[self.weight_name], device, dtype)
        self.pairs = matrix_to(tensors[self.pair_name], device, dtype) if self.pair_name is not None else None

    def forward(self, ctx, token_ids: torch.Tensor, cache=None) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.copies * self.width), dtype=torch.float32, device=token_ids.device)
        if self.pairs is None:
            ops.embedding_pairs(token_ids, self.table, out, ctx.error_word, scale=self.scale, copies=self.copies)
            return out
        if cache is None or cache.state is None:
            raise RuntimeError("an embedding with a pair table needs its per-request state")
        last = cache.state.view(-1)
        ops.embedding_pairs(token_ids, self.table, out, ctx.error_word, scale=self.scale, copies=self.copies,
                            pairs=self.pairs, buckets=self.buckets, mul_prev=self.mul_prev, mul_cur=self.mul_cur,
                            positions=ctx.positions, row_request=ctx.row_request, cu_rows=ctx.cu_rows,
                            state_slots=ctx.state_slots, last_token=last)
        if cache.writable:
            ops.remember_tokens(token_ids, ctx.cu_rows, ctx.state_slots, last, ctx.num_requests)
        return out


class OutputHead(Part):
    """``weight_name`` None ties the head to ``embedding``'s table."""
    graph_safe = True


    def __init__(self, vocab: int, width: int, weight_name: Optional[str], embedding: Optional[TokenEmbedding] = None,
                 softcap: Optional[float] = None, scale: float = 1.0):
        """``scale`` multiplies the 32-bit logits (1: as they are)."""
        if weight_name is None and embedding is None:
            raise ValueError("a tied head needs the embedding it shares")
        if softcap is not None and not softcap > 0:
            raise ValueError("the cap of the logits must be positive")
        self.vocab, self.width, self.weight_name, self.embedding = int(vocab), int(width), weight_name, embedding
        self.softcap, self.scale = softcap, float(scale)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.vocab, self.width))} if self.weight_name else {}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        if self.weight_name:
            self.weight = matrix_to(tensors[self.weight_name], device, dtype)

    def native_record(self):
        weight = self.weight if self.weight_name else self.embedding.table
        return None if weight is None or self.softcap is not None or self.scale != 1.0 else True

    def forward(self, ctx, normed: torch.Tensor) -> torch.Tensor:
        weight = self.weight if self.weight_name else self.embedding.table
        logits = ops.linear(normed, weight, out_dtype=torch.float32, error_word=ctx.error_word)
        if self.scale != 1.0:
            ops.scale_values(logits, self.scale)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits
