"""A state-space mixer with a scalar decay per head and token ("Mamba-2") over a state of fixed size per request.

With inner = heads * vdim, N = state and G = groups, W_in h = [z: inner | x: inner | B: G N | C: G N | dt: heads].
x, B and C pass a causal convolution per channel over the last ``taps`` tokens (a bias per channel, the filter's last
column is the current token's, zeros before the sequence starts) and SiLU.  Per head (whose B and C are those of group
head // (heads / G)):

    dt_t = softplus(dt_t + dt_bias)        S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T        y_t = S_t^T C_t + D x_t

y (heads joined) is multiplied by silu(z), RMS-normed in ``norm_groups`` equal parts, multiplied by the norm's weight
and projected by W_o.  Per request the part keeps, in 32-bit floats whatever the compute dtype, the convolution's last
``taps`` - 1 inputs and S [heads, vdim, N] (``RequestState``; a request that starts at position 0 starts from zeros).
Step sizes, decays, the state, its sums, the gate and the norm are 32-bit; the two projections run in the compute dtype.
The recurrence walks a request's rows in order from its state, prompt portions and decoded tokens alike, so a row's
result does not depend on how the sequence was cut.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping

import torch

from .. import ops
from .base import Mixer, RequestState, TensorSpec, matrix_to, scale_to


@dataclass(frozen=True)
class MambaNames:
    w_in: str
    conv: str
    conv_bias: str
    dt_bias: str
    a_log: str
    d: str
    norm: str
    o: str


class MambaMixer(Mixer):
    graph_safe = True
    #: a step in which some request brings more rows than this runs the chunk-parallel kernels (bfloat16, a state of 64
    #: or 128 entries a side per head); other steps walk each request's rows token by token from its state
    CHUNKED_FROM = 8

    def __init__(self, hidden: int, heads: int, vdim: int, state: int, groups: int, taps: int, norm_groups: int, eps: float,
                 names: MambaNames):
        for name, value in (("heads", heads), ("vdim", vdim), ("state", state), ("groups", groups), ("conv", taps),
                            ("norm_groups", norm_groups)):
            if value <= 0:
                raise ValueError(f"state-space mixer: {name} must be positive, found {value}")
        if heads % groups:
            raise ValueError(f"state-space mixer: {heads} heads do not split into {groups} groups")
        if (heads * vdim) % norm_groups:
            raise ValueError(f"state-space mixer: {heads * vdim} entries do not split into {norm_groups} equal parts")
        if taps > 16 or state > 256:
            raise ValueError(f"state-space mixer: the kernels take at most 16 taps and a state of 256 entries per column, "
                             f"not {taps} and {state}")
        self.hidden, self.heads, self.vdim, self.state, self.groups = int(hidden), int(heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps, self.names = int(taps), int(norm_groups), float(eps), names
        self.w_in = self.w_o = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.d = self.norm = None

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:
        return self.inner + 2 * self.groups * self.state

    @property
    def sizes(self) -> Dict[str, int]:
        return dict(heads=self.heads, vdim=self.vdim, nstate=self.state, groups=self.groups, taps=self.taps)

    def cache_need(self) -> RequestState:
        return RequestState((ops.mamba_slot_floats(**self.sizes),), torch.float32)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n = self.names
        return {n.w_in: TensorSpec((self.inner + self.channels + self.heads, self.hidden)),
                n.conv: TensorSpec((self.channels, self.taps)), n.conv_bias: TensorSpec((self.channels,)),
                n.dt_bias: TensorSpec((self.heads,)), n.a_log: TensorSpec((self.heads,)), n.d: TensorSpec((self.heads,), "scale"),
                n.norm: TensorSpec((self.inner,), "scale"), n.o: TensorSpec((self.hidden, self.inner))}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        n = self.names
        self.w_in, self.w_o = matrix_to(tensors[n.w_in], device, dtype), matrix_to(tensors[n.o], device, dtype)
        self.conv, self.conv_bias = scale_to(tensors[n.conv], device), scale_to(tensors[n.conv_bias], device)
        self.dt_bias, self.a_log, self.d = (scale_to(tensors[name], device) for name in (n.dt_bias, n.a_log, n.d))
        self.norm = scale_to(tensors[n.norm], device)

    def forward(self, ctx, cache, x: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
        proj = ops.linear(x, self.w_in, error_word=ctx.error_word)
        counts = [b - a for a, b in zip(ctx.host_cu_rows, ctx.host_cu_rows[1:])]
        chunked = (len(counts) == ctx.num_requests and max(counts, default=0) > self.CHUNKED_FROM
                   and ops.mamba_chunks_takes(proj.dtype, self.vdim, self.state))
        xbc = torch.empty((rows, self.channels), dtype=proj.dtype if chunked else torch.float32, device=x.device)
        ops.mamba_conv(proj, self.conv, self.conv_bias, ctx.positions, ctx.row_request, ctx.cu_rows, ctx.state_slots,
                       cache.state, xbc, ctx.num_requests, read_only=not cache.writable, **self.sizes)
        y = torch.empty((rows, self.inner), dtype=torch.float32, device=x.device)
        if chunked:
            # prompt portions: chunks in parallel on the tensor cores
            chunks = sum(-(-count // ops.MAMBA_CHUNK_TOKENS) for count in counts)
            ops.mamba_chunks(proj, xbc, self.a_log, self.d, self.dt_bias, ctx.positions, ctx.cu_rows, ctx.state_slots,
                             cache.state, y, ctx.num_requests, chunks, read_only=not cache.writable, **self.sizes)
        else:
            ops.mamba_scan(proj, xbc, self.a_log, self.d, self.dt_bias, ctx.positions, ctx.cu_rows, ctx.state_slots, cache.state,
                           y, ctx.num_requests, read_only=not cache.writable, **self.sizes)
        gated = torch.empty((rows, self.inner), dtype=x.dtype, device=x.device)
        ops.mamba_gate_norm(y, proj, self.norm, self.eps, self.norm_groups, gated)
        return ops.linear(gated, self.w_o, error_word=ctx.error_word, partial_ok=True)
