"""Arrangement of the parts of one layer.

Pre-norm residual form (reference: crates/sglang-srt/src/cpu_reference.rs:257-317):
h' = h + mixer(norm_1(h)); h'' = h' + feed_forward(norm_2(h')).  The hidden state travels
as (residual, delta) with h = residual + delta; each norm takes the pending sum first, in
32-bit, so no separate add kernel runs.  :class:`SandwichBlock` norms each sublayer on both sides;
:class:`ParallelBlock` runs mixer and feed-forward side by side from one norm.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

import torch

from .. import ops
from .base import FeedForward, Mixer, Norm, NormedDelta, Part, TensorSpec


class PreNormBlock(Part):
    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, feed_forward: FeedForward):
        self.input_norm, self.mixer, self.post_norm, self.feed_forward = input_norm, mixer, post_norm, feed_forward

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def parts(self):
        return (self.input_norm, self.mixer, self.post_norm, self.feed_forward)

    def cache_need(self):
        return self.mixer.cache_need()

    def split_scratch(self):
        return self.mixer.split_scratch()

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for part in self.parts():
            specs.update(part.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        for part in self.parts():
            part.load(tensors, device, dtype)

    def native_record(self):
        """This block for the step executor, if each of its parts has a record of the kind the executor's
        pre-norm block is made of; else None, and the block runs part by part."""
        from ..ops.records import SxAttention, SxBlock, SxGatedMlp, SxNorm
        found = [part.native_record() if hasattr(part, "native_record") else None for part in self.parts()]
        kinds = (SxNorm, SxAttention, SxNorm, SxGatedMlp)
        if not all(isinstance(record, kind) for record, kind in zip(found, kinds)):
            return None
        return SxBlock(*found)

    def forward(self, ctx, cache, residual: torch.Tensor,
                delta: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        normed = self.input_norm.add_norm(residual, delta, ctx.dtype)
        delta = self.mixer.forward(ctx, cache, normed)
        normed = self.post_norm.add_norm(residual, delta, ctx.dtype)
        delta = self.feed_forward.forward(ctx, normed)
        return residual, delta


class SandwichBlock(Part):
    """A norm ahead of and behind each sublayer: h' = h + norm_1b(mixer(norm_1(h))),
    h'' = h' + norm_2b(feed_forward(norm_2(h'))); without a feed-forward the block ends after the mixer.

    The hidden state travels as (residual, pending) with the pending term a :class:`NormedDelta`: the norm
    behind a sublayer, the residual sum and the norm ahead of the next sublayer are one kernel
    (``Norm.add_norm``), also across the border between two blocks."""

    def __init__(self, norm_1: Norm, mixer: Mixer, norm_1b: Norm, norm_2: Optional[Norm] = None,
                 feed_forward: Optional[FeedForward] = None, norm_2b: Optional[Norm] = None):
        if (feed_forward is None) != (norm_2 is None) or (feed_forward is None) != (norm_2b is None):
            raise ValueError("a feed-forward comes with the norms ahead of and behind it, or not at all")
        self.norm_1, self.mixer, self.norm_1b = norm_1, mixer, norm_1b
        self.norm_2, self.feed_forward, self.norm_2b = norm_2, feed_forward, norm_2b

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def parts(self):
        return tuple(part for part in (self.norm_1, self.mixer, self.norm_1b, self.norm_2, self.feed_forward,
                                       self.norm_2b) if part is not None)

    def cache_need(self):
        return self.mixer.cache_need()

    def split_scratch(self):
        return self.mixer.split_scratch()

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for part in self.parts():
            specs.update(part.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        for part in self.parts():
            part.load(tensors, device, dtype)

    def forward(self, ctx, cache, residual: torch.Tensor, delta):
        normed = self.norm_1.add_norm(residual, delta, ctx.dtype)
        delta = NormedDelta(self.mixer.forward(ctx, cache, normed), self.norm_1b)
        if self.feed_forward is None:
            return residual, delta
        normed = self.norm_2.add_norm(residual, delta, ctx.dtype)
        return residual, NormedDelta(self.feed_forward.forward(ctx, normed), self.norm_2b)


class ParallelBlock(Part):
    """Both sublayers read ONE norm of the stream and their results are added together:
    h = norm(x); x <- x + mult * (mixer(h) + feed_forward(h)); without a feed-forward only the mixer's term.  Then,
    with ``side`` (``parts/side.py``), x <- x + norm_side(side(x)), the side norm carrying its own factor.

    The sum is one kernel (``ops.scaled_sum``: 32-bit, the mixer's result rounded, 32-bit or in partial sums along K, the
    feed-forward's 32-bit) that also writes the rounded stream the side part's product reads.  The side's result travels
    on as a :class:`NormedDelta`, so its norm, the residual sum and the next block's norm (or the final norm) are one
    kernel."""

    def __init__(self, norm: Norm, mixer: Mixer, feed_forward: Optional[FeedForward], mult: float = 1.0, side=None):
        self.norm, self.mixer, self.feed_forward, self.mult, self.side = norm, mixer, feed_forward, float(mult), side

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def parts(self):
        return tuple(part for part in (self.norm, self.mixer, self.feed_forward, self.side) if part is not None)

    def cache_need(self):
        return self.mixer.cache_need()

    def split_scratch(self):
        return self.mixer.split_scratch()

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for part in self.parts():
            specs.update(part.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        for part in self.parts():
            part.load(tensors, device, dtype)

    def forward(self, ctx, cache, residual: torch.Tensor, delta):
        normed = self.norm.add_norm(residual, delta, ctx.dtype)
        mixed = self.mixer.forward(ctx, cache, normed)
        fed = self.feed_forward.forward(ctx, normed) if self.feed_forward is not None else None
        if self.side is None:
            ops.scaled_sum(residual, mixed, fed, self.mult)
            return residual, None
        rounded = torch.empty(residual.shape, dtype=ctx.dtype, device=residual.device)
        ops.scaled_sum(residual, mixed, fed, self.mult, rounded)
        return residual, NormedDelta(self.side.forward(ctx, rounded), self.side.norm)
