"""Grouped-query attention over the paged cache.

Order as in the reference (crates/sglang-srt/src/cpu_reference.rs:442-546): q, k, v
projections (+ bias if the checkpoint has them); RMSNorm of each q and k head with a
shared [head_dim] weight, before the rotation; rotation of q and k; k and v stored at the
row's slot; scores (q . k) * scale over the keys the row may see, kv head = q head /
(n_q / n_kv) (crates/sglang-kernel/src/cpu.rs:475-479); softmax; weighted sum of v; output
projection.  q, k and v come from one product with the row-wise concatenation of the
three matrices, made at load time.

Two variations that other designs use, both off by default: ``names.v`` None means there is no value
projection and the value of a key is the key itself as projected, before the rotation (the product then
holds q and k only, and the fused kernel stores the unrotated key in the value pool); ``chunk`` makes a row
see, of the keys up to its own, only those of its own chunk of ``chunk`` positions (chunks counted from
position 0 of the sequence, whatever portion of a prompt brought the row).

Four more, also off by default.  ``whole_norm``: q and k are each normed over the WHOLE projection (all heads of the row
together, before they are split into heads) with a weight per entry of the projection, ``names.q_norm`` [n_q * head_dim]
and ``names.k_norm`` [n_kv * head_dim], instead of head by head with a shared weight.  ``value_dim``: values of another
width than queries and keys (W_v is [n_kv * value_dim, hidden], W_o [hidden, n_q * value_dim], the value pool has rows of
that width).  ``sink``: a number that joins the softmax's denominator as exp(sink) beside the keys' terms, the same for
every head (0 adds one to the denominator); it has no key and no value.  ``names.gate``: a matrix [n_q, hidden] whose
product with the mixer's input gives a logit per head; head h's result is multiplied by its sigmoid before the output
projection (the matrix rides in the q/k/v product, the factor in the attention kernel's last step).  A mixer with any of
these runs ``ops.proj_norm_rope_kv`` between the product and attention; every attention kernel takes the sink and the
gates, and the tensor-core ones serve where values are as wide as the keys.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Mixer, PagedKV, PositionEncoding, TensorSpec, matrix_to, scale_to


@dataclass(frozen=True)
class AttentionNames:
    q: str
    k: str
    v: Optional[str]
    o: str
    q_norm: Optional[str] = None
    k_norm: Optional[str] = None
    q_bias: Optional[str] = None
    k_bias: Optional[str] = None
    v_bias: Optional[str] = None
    o_bias: Optional[str] = None
    gate: Optional[str] = None


class GroupedQueryAttention(Mixer):
    graph_safe = True
    #: what the attention kernels take: the generic one gives a warp to each query head of a kv head (at most
    #: 32 warps a block) and keeps up to 16 values of a head per lane
    MAX_HEAD_DIM = 512
    MAX_HEADS_PER_KV_HEAD = 32

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 position: PositionEncoding, names: AttentionNames, *, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, chunk: Optional[int] = None, whole_norm: bool = False,
                 value_dim: Optional[int] = None, sink: Optional[float] = None, partial_sums: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        if not 0 < head_dim <= self.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {head_dim} is outside what the attention kernels take (1 to {self.MAX_HEAD_DIM})")
        self.hidden, self.n_q, self.n_kv, self.d = int(hidden), int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.position, self.names = float(scale), position, names
        self.qk_norm_eps, self.window = qk_norm_eps, window
        if chunk is not None and chunk <= 0:
            raise ValueError(f"a chunk of {chunk} positions")
        self.chunk = chunk
        self.values_from_keys = names.v is None
        if self.values_from_keys and names.v_bias:
            raise ValueError("values that are the keys have no bias of their own")
        self.whole_norm, self.sink = bool(whole_norm), None if sink is None else float(sink)
        self.vd = int(value_dim) if value_dim is not None else self.d
        if not 0 < self.vd <= 1024:
            raise ValueError(f"values of {self.vd} entries are outside what the attention kernels take (1 to 1024)")
        #: whether the output product may hand on partial sums along K (a consumer that cannot add them says no)
        self.partial_sums = bool(partial_sums)
        #: the arrangement that ``ops.proj_norm_rope_kv`` prepares
        self.wide = self.whole_norm or self.vd != self.d or self.sink is not None or names.gate is not None
        if not self.wide and num_heads // num_kv_heads > self.MAX_HEADS_PER_KV_HEAD:
            # (the fused per-head kernel's limit; the other arrangement goes through kernels that take the heads of a kv
            # head in chunks)
            raise ValueError(f"{num_heads // num_kv_heads} query heads per kv head exceed the "
                             f"{self.MAX_HEADS_PER_KV_HEAD} that the attention kernels take")
        if self.wide and (self.values_from_keys or names.q_bias or names.k_bias or names.v_bias):
            raise ValueError("norms over whole projections, values of their own width, a sink and a gate are not built "
                             "together with biases or with values that are the keys")
        if self.whole_norm and (names.q_norm is None or names.k_norm is None):
            raise ValueError("norms over whole projections need both weights")
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.q_norm = self.k_norm = self.sinks = None

    def cache_need(self) -> PagedKV:
        return PagedKV(self.n_kv, self.d, self.window, value_dim=None if self.vd == self.d else self.vd)

    def split_scratch(self):
        return (self.n_q * self.vd, self.n_q * 2)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n = self.names
        specs = {
            n.q: TensorSpec((self.n_q * self.d, self.hidden)),
            n.k: TensorSpec((self.n_kv * self.d, self.hidden)),
            n.o: TensorSpec((self.hidden, self.n_q * self.vd)),
        }
        if n.v:
            specs[n.v] = TensorSpec((self.n_kv * self.vd, self.hidden))
        if n.q_norm:
            specs[n.q_norm] = TensorSpec((self.n_q * self.d if self.whole_norm else self.d,), "scale")
        if n.k_norm:
            specs[n.k_norm] = TensorSpec((self.n_kv * self.d if self.whole_norm else self.d,), "scale")
        if n.gate:
            specs[n.gate] = TensorSpec((self.n_q, self.hidden))
        for name, width in ((n.q_bias, self.n_q * self.d), (n.k_bias, self.n_kv * self.d),
                            (n.v_bias, self.n_kv * self.d), (n.o_bias, self.hidden)):
            if name:
                specs[name] = TensorSpec((width,))
        specs.update(self.position.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        n = self.names
        stacked = [tensors[n.q], tensors[n.k]] + ([tensors[n.v]] if n.v else []) + ([tensors[n.gate]] if n.gate else [])
        self.sinks = torch.full((self.n_q,), self.sink, dtype=torch.float32, device=device) if self.sink is not None else None
        self.w_qkv = matrix_to(torch.cat(stacked, dim=0), device, dtype)
        self.w_o = matrix_to(tensors[n.o], device, dtype)
        self.q_norm = scale_to(tensors[n.q_norm], device) if n.q_norm else None
        self.k_norm = scale_to(tensors[n.k_norm], device) if n.k_norm else None
        if n.q_bias or n.k_bias or n.v_bias:
            parts = []
            for name, width in ((n.q_bias, self.n_q * self.d), (n.k_bias, self.n_kv * self.d),
                                (n.v_bias, self.n_kv * self.d))[:2 if self.values_from_keys else 3]:
                parts.append(tensors[name].to(torch.float32) if name else torch.zeros(width))
            self.b_qkv = scale_to(torch.cat(parts), device)
        self.b_o = scale_to(tensors[n.o_bias], device) if n.o_bias else None
        self.position.load(tensors, device, dtype)

    def native_record(self):
        """This mixer for the step executor, or None if its position encoding is not of the kind the fused
        kernel applies from a frequency table (an encoding that computes its angles in Python keeps the
        part-by-part path)."""
        from ..ops.records import SxAttention, linear_record
        if self.w_qkv is None or not self.position.fused or self.values_from_keys or self.chunk or self.wide:
            return None
        rotary = self.position.fused_rotary()
        if rotary is not None and (rotary.angles is not None or rotary.inv_freq is None or rotary.magnitude != 1.0):
            return None
        return SxAttention(
            linear_record(self.w_qkv, self.b_qkv), linear_record(self.w_o, self.b_o),
            None if self.q_norm is None else self.q_norm.data_ptr(), None if self.k_norm is None else self.k_norm.data_ptr(),
            None if rotary is None else rotary.inv_freq.data_ptr(),
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, self.scale,
            rotary.rotary_dim if rotary is not None else 0, int(rotary.interleaved) if rotary is not None else 0,
            self.n_q, self.n_kv, self.d, self.window or 0)

    def forward(self, ctx, cache, x: torch.Tensor) -> torch.Tensor:
        batch = ctx.paged[cache.group]
        rows = x.shape[0]
        qkv = ops.linear(x, self.w_qkv, self.b_qkv, error_word=ctx.error_word, partial_ok=True)
        q = torch.empty((rows, self.n_q, self.d), dtype=x.dtype, device=x.device)
        rotary = self.position.fused_rotary() if self.position.fused else None
        if not self.position.fused:
            raise NotImplementedError("a position encoding with kernels of its own is applied by its mixer")
        if self.wide:
            return self._forward_wide(ctx, cache, batch, qkv, q, rotary)
        ops.qk_norm_rope_kv(
            qkv, q, cache.k_pool if cache.writable else None, cache.v_pool if cache.writable else None,
            ctx.positions, batch.slots if cache.writable else None, self.q_norm, self.k_norm,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
            rotary.inv_freq if rotary else None, rotary.rotary_dim if rotary else 0,
            rotary.interleaved if rotary else False, self.n_q, self.n_kv, self.d, ctx.error_word,
            angles=rotary.angles(ctx.positions) if rotary is not None and rotary.angles is not None else None,
            magnitude=rotary.magnitude if rotary is not None else 1.0, values_from_keys=self.values_from_keys)
        out = torch.empty_like(q)
        self._attend(ctx, cache, batch, q, out, None)
        return ops.linear(out.view(rows, self.n_q * self.d), self.w_o, self.b_o, error_word=ctx.error_word,
                          partial_ok=self.partial_sums)

    def _attend(self, ctx, cache, batch, q, out, gates) -> None:
        """The step's attention launches: the tensor-core kernels where they take the sizes (values as wide as the keys,
        heads of 64 or 128), the generic kernel elsewhere; the sink and the gates go to whichever runs."""
        chunk, sinks = self.chunk or 0, self.sinks
        same_width = self.vd == self.d
        for launch in batch.launches:
            b, e = launch.begin, launch.end
            if same_width and launch.wide_tiles is not None and ops.tiled_attention_tc_takes(
                    q.dtype, self.n_q, self.n_kv, self.d, cache.k_pool.shape[2]):
                ops.tiled_attention_tc(q, cache.k_pool, cache.v_pool, out, launch.wide_tiles, batch.block_table,
                                       scale=self.scale, window=self.window or 0, error_word=ctx.error_word, chunk=chunk,
                                       sinks=sinks, gates=gates)
                continue
            if same_width and launch.tiles is not None and ops.tiled_attention_takes(q.dtype, self.n_q, self.n_kv, self.d):
                ops.tiled_attention(q, cache.k_pool, cache.v_pool, out, launch.tiles, batch.block_table,
                                    scale=self.scale, window=self.window or 0, error_word=ctx.error_word, chunk=chunk,
                                    sinks=sinks, gates=gates)
                continue
            row_gates = None if gates is None else gates[b:e]
            if (same_width and launch.tiles is None and launch.split_size and batch.counters is not None
                    and batch.counters.numel() >= (e - b) * self.n_kv
                    and ops.decode_attention_takes(q.dtype, self.n_q, self.n_kv, self.d)):
                ops.decode_attention(q[b:e], cache.k_pool, cache.v_pool, out[b:e], ctx.positions[b:e],
                                     ctx.row_request[b:e], batch.block_table, scale=self.scale,
                                     window=self.window or 0, scratch_acc=batch.scratch_acc,
                                     scratch_ml=batch.scratch_ml, counters=batch.counters,
                                     error_word=ctx.error_word, max_keys=launch.max_keys, chunk=chunk, sinks=sinks,
                                     gates=row_gates)
                continue
            ops.paged_attention(q[b:e], cache.k_pool, cache.v_pool, out[b:e], ctx.positions[b:e],
                                ctx.row_request[b:e], batch.block_table, scale=self.scale,
                                window=self.window or 0, split_size=launch.split_size,
                                max_splits=launch.max_splits, scratch_acc=batch.scratch_acc,
                                scratch_ml=batch.scratch_ml, error_word=ctx.error_word, chunk=chunk, sinks=sinks,
                                gates=row_gates)

    def _forward_wide(self, ctx, cache, batch, qkv, q, rotary) -> torch.Tensor:
        """Norms over the whole projections, values of their own width, a sink and a gate per head: one kernel between
        the product and attention, the attention kernels with the sink in the denominator and the gate in their last
        step, the output product."""
        if rotary is not None and rotary.angles is not None:
            raise NotImplementedError("angles computed per step are not built for this arrangement")
        rows = q.shape[0]
        gates = torch.empty((rows, self.n_q), dtype=torch.float32, device=q.device) if self.names.gate else None
        ops.proj_norm_rope_kv(
            qkv, q, cache.k_pool, cache.v_pool, ctx.positions, batch.slots if cache.writable else None,
            self.q_norm if self.whole_norm else None, self.k_norm if self.whole_norm else None,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, rotary.inv_freq if rotary else None,
            rotary.rotary_dim if rotary else 0, rotary.interleaved if rotary else False, self.n_q, self.n_kv, self.d,
            self.vd, ctx.error_word, magnitude=rotary.magnitude if rotary is not None else 1.0, gate_out=gates)
        out = torch.empty((rows, self.n_q, self.vd), dtype=q.dtype, device=q.device)
        self._attend(ctx, cache, batch, q, out, gates)
        return ops.linear(out.view(rows, self.n_q * self.vd), self.w_o, self.b_o, error_word=ctx.error_word,
                          partial_ok=self.partial_sums)
