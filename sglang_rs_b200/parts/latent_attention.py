"""Attention through latents, with a sink per head and an output gate.

For the mixer's input h (one row per token):

* queries: c_q = RMSnorm(W_dq h) * w_dq, q = W_uq c_q, head by head [dim plain | rot_dim rotated];
* keys and values: W_dkv h = [kv_rank | rot_dim]; c = RMSnorm(first part) * w_dkv is the latent, the
  second part (not normed) is one rotated key part that all heads share; per head k_plain = W_uk c and
  v = W_uv c;
* score(i, j) = (q_plain_i . k_plain_j + q_rot_i . k_rot_j) * scale for j <= i; softmax whose denominator
  also holds exp(sink_h); head h's result is multiplied by sigmoid(W_g h)_h; W_o on the joined heads.

Only c and the rotated key part are kept per token: one pool row [kv_rank + rot_dim], one "kv head".
The up-projections never touch the cache: since q_plain . (W_uk c) = (W_uk^T q_plain) . c, each query
head is carried into the latent space (``head_linear`` with W_uk^T per head), attention then runs over
the cached rows themselves with ``heads`` query heads on one shared key row whose first kv_rank
entries are also the value, and W_uv is applied per head to the attention's result (with the gate in
the same kernel).  Scores, softmax, norms and angles are 32-bit in both dtypes.

W_dq, W_dkv and W_g read the same input and are one product (rows stacked at load).

Variations, each off unless asked for: queries straight from the input, q = W_q h, without a query latent
(``q_rank`` 0: ``names.q_up`` is W_q and reads h; ``names.q_down`` and ``names.q_norm`` are None); no rotated part
(``rot_dim`` 0); a sliding window (``window``: a row sees itself and the ``window`` - 1 rows before it); a layer without
a down-projection of its own (``names.kv_down`` None) that reads the latents another layer's cache holds, with its own
W_uk, W_uv, queries and window: the model's program gives it that layer's cache, read-only (``LayerCall.cache_from``).
``cache_window`` is what the cache must keep (the widest window of all layers that read it; None: every row).
The rotation may pair entry 2i with 2i + 1 (``rotary.interleaved``) and may stretch its long wavelengths and scale its
cosines and sines (``rotary.scaling``); the gate may be one logit per entry of the joined heads instead of one per head
(``gate_per_entry``: ``names.gate`` is then [heads * vdim, hidden]).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Mixer, PagedKV, TensorSpec, matrix_to, scale_to
from .rope import RotaryEncoding


@dataclass(frozen=True)
class LatentAttentionNames:
    q_down: Optional[str]
    q_norm: Optional[str]
    q_up: str
    kv_down: Optional[str]
    kv_norm: Optional[str]
    k_up: str
    v_up: str
    o: str
    sink: Optional[str] = None
    gate: Optional[str] = None


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, dim: int, rot_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float, rotary: Optional[RotaryEncoding], names: LatentAttentionNames, *,
                 window: Optional[int] = None, cache_window: Optional[int] = -1, gate_per_entry: bool = False,
                 partial_sums: bool = False):
        """``rotary``: the rotation of the rot_dim part (its ``rotary_dim`` leading entries are rotated, the rest
        pass unchanged); None leaves it alone.  ``names.sink`` / ``names.gate`` None: no sink / no gate.
        ``cache_window`` -1: the layer's own window."""
        for name, value in (("heads", num_heads), ("dim", dim), ("vdim", value_dim), ("kv_rank", kv_rank)):
            if value <= 0:
                raise ValueError(f"latent attention: {name} must be positive, found {value}")
        q_rank = int(q_rank or 0)
        if q_rank < 0 or (q_rank == 0) != (names.q_down is None) or (names.q_down is None) != (names.q_norm is None):
            raise ValueError("latent attention: a query latent comes with its rank, its down-projection and its norm, or not at all")
        if (names.kv_down is None) != (names.kv_norm is None):
            raise ValueError("latent attention: a down-projection comes with its norm, or not at all")
        if names.kv_down is None and rot_dim:
            raise ValueError("latent attention: a layer that reads another layer's latents has no rotated key part of its own")
        if window is not None and window <= 0:
            raise ValueError(f"latent attention: a window of {window} rows")
        if cache_window == -1:
            cache_window = window
        if window is None and cache_window is not None or (window and cache_window and cache_window < window):
            raise ValueError("latent attention: the cache keeps fewer rows than the layer sees")
        if rot_dim < 0 or (rotary is not None and rotary.rotary_dim > rot_dim):
            raise ValueError(f"latent attention: the rotation covers more than the {rot_dim} rotated entries")
        self.gate_per_entry = bool(gate_per_entry)
        #: whether the output product may hand on partial sums along K (for a consumer that adds them in order)
        self.partial_sums = bool(partial_sums)
        if kv_rank > 1024:
            raise ValueError(f"latent attention: a latent of {kv_rank} entries exceeds the 1024 the attention kernel takes")
        self.hidden, self.heads, self.dim, self.rot_dim, self.vdim = int(hidden), int(num_heads), int(dim), int(rot_dim), int(value_dim)
        self.q_rank, self.kv_rank, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        self.rotary, self.names = rotary, names
        self.window, self.cache_window = window, cache_window
        self.w_in = self.w_uq = self.w_qk = self.w_uv = self.w_o = self.q_norm = self.kv_norm = self.sink = None

    @property
    def row_width(self) -> int:
        return self.kv_rank + self.rot_dim

    def cache_need(self) -> PagedKV:
        return PagedKV(1, self.row_width, self.cache_window, values=False)

    def split_scratch(self):
        return (self.heads * self.kv_rank, self.heads * 2)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, h = self.names, self.heads
        specs = {
            n.q_up: TensorSpec((h * (self.dim + self.rot_dim), self.q_rank or self.hidden)),
            n.k_up: TensorSpec((h * self.dim, self.kv_rank)), n.v_up: TensorSpec((h * self.vdim, self.kv_rank)),
            n.o: TensorSpec((self.hidden, h * self.vdim)),
        }
        if self.q_rank:
            specs.update({n.q_down: TensorSpec((self.q_rank, self.hidden)), n.q_norm: TensorSpec((self.q_rank,), "scale")})
        if n.kv_down:
            specs.update({n.kv_down: TensorSpec((self.kv_rank + self.rot_dim, self.hidden)),
                          n.kv_norm: TensorSpec((self.kv_rank,), "scale")})
        if n.sink:
            specs[n.sink] = TensorSpec((h,))
        if n.gate:
            specs[n.gate] = TensorSpec((h * self.vdim if self.gate_per_entry else h, self.hidden))
        if self.rotary is not None:
            specs.update(self.rotary.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        n, h = self.names, self.heads
        # one product for all that reads the input: [query latent, or the queries themselves | latent and shared key part | gate]
        stacked = ([tensors[n.q_down if self.q_rank else n.q_up]] + ([tensors[n.kv_down]] if n.kv_down else [])
                   + ([tensors[n.gate]] if n.gate else []))
        self.w_in = matrix_to(torch.cat(stacked, dim=0), device, dtype)
        self.w_uq = matrix_to(tensors[n.q_up], device, dtype) if self.q_rank else None
        # per head W_uk^T [kv_rank, dim]: carries a query head into the latent space
        self.w_qk = matrix_to(tensors[n.k_up].view(h, self.dim, self.kv_rank).transpose(1, 2), device, dtype)
        self.w_uv = matrix_to(tensors[n.v_up].view(h, self.vdim, self.kv_rank), device, dtype)
        self.w_o = matrix_to(tensors[n.o], device, dtype)
        self.q_norm = scale_to(tensors[n.q_norm], device) if self.q_rank else None
        self.kv_norm = scale_to(tensors[n.kv_norm], device) if n.kv_norm else None
        self.sink = scale_to(tensors[n.sink], device) if n.sink else None
        if self.rotary is not None:
            self.rotary.load(tensors, device, dtype)

    def forward(self, ctx, cache, x: torch.Tensor) -> torch.Tensor:
        batch = ctx.paged[cache.group]
        rows, h = x.shape[0], self.heads
        rotary = self.rotary.fused_rotary() if self.rotary is not None else None
        inv_freq, rotary_dim = (rotary.inv_freq, rotary.rotary_dim) if rotary is not None else (None, 0)
        turn = dict(interleaved=rotary.interleaved, magnitude=rotary.magnitude) if rotary is not None else {}
        proj = ops.linear(x, self.w_in, error_word=ctx.error_word)
        q_cols = self.q_rank or h * (self.dim + self.rot_dim)
        kv_cols = self.row_width if self.names.kv_down else 0
        stores = cache.writable and kv_cols > 0
        q_latent = torch.empty((rows, self.q_rank), dtype=x.dtype, device=x.device) if self.q_rank else None
        if self.q_rank:
            ops.latent_prepare(proj, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm, self.eps,
                               ctx.positions, inv_freq, rotary_dim, q_latent, cache.k_pool if stores else None,
                               batch.slots if stores else None, ctx.error_word, **turn)
            q = ops.linear(q_latent, self.w_uq, error_word=ctx.error_word).view(rows, h, self.dim + self.rot_dim)
        else:
            if stores:
                ops.latent_prepare(proj[:, q_cols:], 0, self.kv_rank, self.rot_dim, None, self.kv_norm, self.eps,
                                   ctx.positions, inv_freq, rotary_dim, None, cache.k_pool, batch.slots, ctx.error_word,
                                   **turn)
            q = proj[:, :q_cols].unflatten(1, (h, self.dim + self.rot_dim))
        # queries in the cache's own space: [W_uk^T q_plain | rotated part]
        q_row = torch.empty((rows, h, self.row_width), dtype=x.dtype, device=x.device)
        ops.head_linear(q, self.w_qk, q_row)
        if self.rot_dim:
            ops.rope_slice(q, self.dim, q_row, self.kv_rank, self.rot_dim, rotary_dim, ctx.positions, inv_freq, **turn)
        mixed = torch.empty((rows, h, self.kv_rank), dtype=x.dtype, device=x.device)
        tensor_cores = ops.latent_attention_takes(x.dtype, self.row_width, self.kv_rank)
        window = self.window or 0
        for launch in batch.launches:
            b, e = launch.begin, launch.end
            if tensor_cores and launch.tiles is not None:
                # prompt portions: the tiles name their rows of the whole step
                ops.latent_attention(q_row, cache.k_pool, mixed, ctx.positions, ctx.row_request, batch.block_table,
                                     scale=self.scale, sinks=self.sink, error_word=ctx.error_word, tiles=launch.tiles,
                                     window=window)
                continue
            if tensor_cores and launch.split_size and launch.split_size % 64 == 0:
                ops.latent_attention(q_row[b:e], cache.k_pool, mixed[b:e], ctx.positions[b:e], ctx.row_request[b:e],
                                     batch.block_table, scale=self.scale, sinks=self.sink, error_word=ctx.error_word,
                                     split_size=launch.split_size, max_splits=launch.max_splits,
                                     scratch_acc=batch.scratch_acc, scratch_ml=batch.scratch_ml, window=window)
                continue
            ops.paged_attention(q_row[b:e], cache.k_pool, None, mixed[b:e], ctx.positions[b:e], ctx.row_request[b:e],
                                batch.block_table, scale=self.scale, window=window, split_size=launch.split_size,
                                max_splits=launch.max_splits, scratch_acc=batch.scratch_acc,
                                scratch_ml=batch.scratch_ml, error_word=ctx.error_word, sinks=self.sink)
        out = torch.empty((rows, h, self.vdim), dtype=x.dtype, device=x.device)
        gate = proj[:, q_cols + kv_cols:] if self.names.gate else None
        ops.head_linear(mixed, self.w_uv, out, gate=gate, gate_per_entry=self.gate_per_entry)
        return ops.linear(out.view(rows, h * self.vdim), self.w_o, error_word=ctx.error_word, partial_ok=self.partial_sums)
