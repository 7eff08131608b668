"""Python face of the CUDA kernels.

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity), launches on torch's current stream and raises :class:`KernelError` with the
library's message if the kernel refuses the sizes.  Nothing here computes on the host
and nothing falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_library
from . import records, trace
from .trace import traced

F32, BF16 = 0, 1

# Products of more than a few rows go to cuBLAS (``library_product``), on a handle whose math mode forbids
# partial sums of a split along K in bfloat16: every product of this engine accumulates in 32 bits to the
# end.  The same is asked of torch's own handle, for callers that mix torch's products with this package.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(tensor: Optional[torch.Tensor]):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


_scoped_stream = None


def _stream():
    if _scoped_stream is not None:
        return _scoped_stream
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks up torch's current stream once for all kernel launches inside the ``with`` block
    (the look-up costs as much as a small launch).  The current stream must not change inside."""

    def __enter__(self):
        global _scoped_stream
        self._previous = _scoped_stream
        _scoped_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._previous
        return False


def _need(tensor: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no host path")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {tensor.dtype}")


#: kernels of this package launched so far (the bench reports the count of a timed region)
launch_count = 0


def _check(library, status: int, launches: int = 1) -> None:
    global launch_count
    launch_count += launches
    if status != 0:
        raise KernelError(library.srb_last_error().decode("utf-8", "replace") or f"kernel status {status}")


#: the compute capability the kernels are compiled for (sm_100a: tcgen05, tensor memory, TMA)
REQUIRED_CAPABILITY = (10, 0)
_sm_counts: dict = {}


def require_supported_device(device) -> None:
    """Fails at start-up, with the device's name, on a GPU that the kernels are not built for (the
    reference decides the same from the SM version, crates/sglang-srt/src/backend.rs:355-366); without
    this check the first tcgen05 launch would fail with a bare CUDA error."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is visible; this engine has no host path")
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    capability = torch.cuda.get_device_capability(index)
    if tuple(capability) != REQUIRED_CAPABILITY:
        raise KernelError(
            f"device cuda:{index} ({torch.cuda.get_device_name(index)}) has compute capability "
            f"{capability[0]}.{capability[1]}; the kernels of this engine are built for sm_100a "
            f"({REQUIRED_CAPABILITY[0]}.{REQUIRED_CAPABILITY[1]}, B200) only")


def sm_count(device=None) -> int:
    """SMs of ``device`` (default: the current one), asked once."""
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None \
        else torch.device(device).index
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return count


def new_error_word(device) -> torch.Tensor:
    """Device-side word that kernels OR fault bits into (bad token, slot or page)."""
    return torch.zeros(1, dtype=torch.int32, device=device)


ERROR_BITS = {1: "token id outside the vocabulary", 2: "cache slot outside the pool",
              4: "page id outside the pool", 8: "a device-side wait ran out",
              16: "a row of a split attention run has more key splits than the launch was given"}


def raise_on_error_word(word: torch.Tensor) -> None:
    raise_on_error_value(int(word.item()), word)


def raise_on_error_value(value: int, word: torch.Tensor) -> None:
    """``value``: what ``word`` held when it was last copied to the host."""
    if value:
        word.zero_()
        what = [text for bit, text in ERROR_BITS.items() if value & bit]
        raise KernelError("device-side check failed: " + "; ".join(what))


# --------------------------------------------------------------------------- rows

@traced("embedding")
def embedding(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, error_word: torch.Tensor,
              scale: float = 1.0) -> None:
    """residual[r, :] = float(table[ids[r], :]) * scale"""
    _need(ids, "ids", torch.int32); _need(table, "table"); _need(residual, "residual", torch.float32)
    rows, width = residual.shape
    if ids.numel() != rows or table.shape[1] != width:
        raise KernelError("embedding: shapes of ids, table and residual do not agree")
    lib = load_library("elementwise")
    _check(lib, lib.srb_embedding_scaled(_ptr(ids), _ptr(table), _ptr(residual), rows, width, table.shape[0],
                                         _ptr(error_word), dtype_code(table.dtype), ctypes.c_float(scale), _stream()))


@traced("embedding")
def take_tokens(tokens: torch.Tensor, source: torch.Tensor, index: torch.Tensor, error_word: torch.Tensor) -> None:
    """tokens[i] = source[index[i]] where index[i] >= 0 (int32, on the device): the token ids that the
    step before chose and that have not been to the host yet."""
    _need(tokens, "tokens", torch.int32); _need(source, "source", torch.int32); _need(index, "index", torch.int32)
    if index.numel() < tokens.numel():
        raise KernelError("take_tokens: one index per token is needed")
    lib = load_library("elementwise")
    _check(lib, lib.srb_take_tokens(_ptr(tokens), _ptr(source), _ptr(index), tokens.numel(), source.numel(),
                                    _ptr(error_word), _stream()))


@traced("norm")
def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, row_index: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """x = residual (+ delta); residual = x if asked; out = x / sqrt(mean(x^2) + eps) * weight.

    ``delta`` is [rows, width] of ``out``'s dtype, or float32 [parts, rows, width]: partial sums
    of a product cut along K, added in order.  With ``row_index`` the rows ``row_index[i]`` are
    read and ``out[i]`` is written."""
    _need(residual, "residual", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    width = residual.shape[1]
    rows = out.shape[0]
    whole = parts = None
    num_parts = part_stride = 0
    if delta is not None and delta.dim() == 3:
        _need(delta, "delta", torch.float32)
        if delta.shape[1:] != residual.shape:
            raise KernelError("add_rmsnorm: partial sums and residual differ in shape")
        parts, num_parts, part_stride = delta, delta.shape[0], delta.stride(0)
    elif delta is not None:
        _need(delta, "delta", out.dtype)
        if delta.shape != residual.shape:
            raise KernelError("add_rmsnorm: delta and residual differ in shape")
        whole = delta
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
        if row_index.numel() != rows:
            raise KernelError("add_rmsnorm: one output row per index is needed")
    elif rows != residual.shape[0]:
        raise KernelError("add_rmsnorm: out and residual differ in rows")
    if weight.numel() != width or out.shape[1] != width:
        raise KernelError("add_rmsnorm: widths do not agree")
    lib = load_library("elementwise")
    _check(lib, lib.srb_add_rmsnorm(_ptr(residual), _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(part_stride),
                                    _ptr(weight), _ptr(out), _ptr(row_index), rows, width, ctypes.c_float(eps),
                                    int(write_residual), dtype_code(out.dtype), _stream()))


#: kinds of norm that :func:`norm_add_norm` applies, by the numbers of csrc/elementwise.cu
NORM_KINDS = {"none": 0, "rms": 1, "layer": 2}


@traced("norm")
def norm_add_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], inner, outer, out: Optional[torch.Tensor],
                  row_index: Optional[torch.Tensor] = None, write_residual: bool = True,
                  extra: Optional[torch.Tensor] = None, addend: Optional[torch.Tensor] = None) -> None:
    """x = residual + inner(delta) (+ addend); residual = x if asked; out = outer(x), all sums and means in 32-bit.
    ``addend`` (float32, shaped like the residual) is a second term of the sum, added after the pending one.
    ``delta`` may also be float32 [parts, rows, width]: partial sums of a product cut along K, added in part order
    before the inner norm.

    ``inner`` and ``outer`` are ``(kind, weight, bias, eps)`` with kind one of ``NORM_KINDS`` (``none``: the
    identity; ``rms``: v / sqrt(mean(v^2) + eps) * w; ``layer``: (v - mean) / sqrt(var + eps) * w + b) or None
    for the identity.  A spec may go on with ``(..., groups, scale)``: an RMS norm taken in ``groups`` equal
    consecutive parts of the row, each with its own mean, and a factor on the normalised values.  ``delta`` is [rows, width] of ``out``'s dtype or float32, or None (x is the residual).
    ``out`` may be None (only the sum is wanted) and may have rows longer than ``width``; with ``extra``
    (float32, shaped like the residual) its rows are written, rounded, into columns width .. 2 width - 1 of out."""
    _need(residual, "residual", torch.float32)
    width = residual.shape[1]
    def spec(norm):
        if norm is None:
            return 0, None, None, 0.0, 1, 1.0
        kind, weight, bias, eps = norm[:4]
        groups, scale = (norm[4], norm[5]) if len(norm) > 4 else (1, 1.0)
        if groups < 1 or width % groups or (groups > 1 and kind != "rms"):
            raise KernelError(f"norm_add_norm: {width} entries in {groups} parts of a {kind} norm are not taken")
        for name, tensor in (("weight", weight), ("bias", bias)):
            if tensor is not None:
                _need(tensor, name, torch.float32)
                if tensor.numel() != width:
                    raise KernelError(f"norm_add_norm: a norm's {name} must have {width} entries")
        return NORM_KINDS[kind], weight, bias, float(eps), int(groups), float(scale)
    inner_kind, inner_w, inner_b, inner_eps, inner_groups, inner_scale = spec(inner)
    outer_kind, outer_w, outer_b, outer_eps, outer_groups, outer_scale = spec(outer)
    whole = as_float = None
    num_parts = part_stride = 0
    if delta is not None:
        _need(delta, "delta")
        if delta.dim() == 3:
            _need(delta, "delta", torch.float32)
            if delta.shape[1:] != residual.shape:
                raise KernelError("norm_add_norm: partial sums and residual differ in shape")
            as_float, num_parts, part_stride = delta, delta.shape[0], delta.stride(0)
        elif delta.shape != residual.shape:
            raise KernelError("norm_add_norm: delta and residual differ in shape")
        elif delta.dtype == torch.float32 and (out is None or out.dtype != torch.float32):
            as_float = delta
        else:
            whole = delta
    rows = residual.shape[0] if row_index is None else row_index.numel()
    pitch = 0
    dtype = residual.dtype if out is None else out.dtype
    if out is not None:
        if out.dim() != 2 or out.stride(1) != 1 or out.shape[0] != rows or not out.is_cuda:
            raise KernelError("norm_add_norm: out must be a CUDA matrix with dense rows, one per row")
        pitch = out.stride(0)
        if out.shape[1] < width * (2 if extra is not None else 1):
            raise KernelError("norm_add_norm: rows of out are too short")
    elif whole is not None:
        dtype = whole.dtype
    if whole is not None and whole.dtype != dtype:
        raise KernelError("norm_add_norm: delta must be float32 or of out's dtype")
    if extra is not None:
        _need(extra, "extra", torch.float32)
        if extra.shape != residual.shape:
            raise KernelError("norm_add_norm: extra and residual differ in shape")
    if addend is not None:
        _need(addend, "addend", torch.float32)
        if addend.shape != residual.shape:
            raise KernelError("norm_add_norm: addend and residual differ in shape")
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
    lib = load_library("elementwise")
    _check(lib, lib.srb_norm_add_norm_parts(
        _ptr(residual), _ptr(whole), _ptr(as_float), inner_kind, _ptr(inner_w), _ptr(inner_b), ctypes.c_float(inner_eps),
        inner_groups, ctypes.c_float(inner_scale), outer_kind, _ptr(outer_w), _ptr(outer_b), ctypes.c_float(outer_eps),
        outer_groups, ctypes.c_float(outer_scale), _ptr(out), ctypes.c_longlong(pitch),
        _ptr(extra), _ptr(row_index), rows, width, int(write_residual), dtype_code(dtype), _ptr(addend), num_parts,
        ctypes.c_longlong(part_stride), _stream()))


#: activations of a gated feed-forward, act(gate) * up, by the numbers of csrc/activations.cuh
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2, "swiglu_clamp": 3}
#: activations with a parameter (``swiglu_clamp``: min(g, limit) sigmoid(1.702 min(g, limit)) (clamp(u, -limit, limit) + 1),
#: the parameter being the limit); only the experts' products carry one (``routed_experts(activation_param=)``)
PARAMETRIC_ACTIVATIONS = frozenset({"swiglu_clamp"})


def activation_code(name: str, parametric: bool = False) -> int:
    try:
        code = ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"unknown activation {name!r}; the kernels have {sorted(ACTIVATIONS)}") from None
    if name in PARAMETRIC_ACTIVATIONS and not parametric:
        raise KernelError(f"activation {name!r} has a parameter, which this kernel does not take")
    return code


@traced("activation")
def gated_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[r, j] = act(gate_up[r, j]) * gate_up[r, inner + j]"""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    rows, inner = out.shape
    if gate_up.shape != (rows, 2 * inner):
        raise KernelError("gated_mul: gate_up must be [rows, 2 * inner]")
    lib = load_library("elementwise")
    _check(lib, lib.srb_gated_mul(_ptr(gate_up), _ptr(out), rows, inner, activation_code(activation),
                                  dtype_code(out.dtype), _stream()))


@traced("bias")
def add_bias(values: torch.Tensor, bias: torch.Tensor) -> None:
    _need(values, "values"); _need(bias, "bias", torch.float32)
    rows, width = values.shape
    if bias.numel() != width:
        raise KernelError("add_bias: bias width differs")
    lib = load_library("elementwise")
    _check(lib, lib.srb_add_bias(_ptr(values), _ptr(bias), rows, width, dtype_code(values.dtype), _stream()))


# --------------------------------------------------------------------------- attention

@traced("rope_kv")
def qk_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                    v_pool: Optional[torch.Tensor], positions: torch.Tensor, slots: Optional[torch.Tensor],
                    q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                    inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, n_q: int, n_kv: int,
                    head_dim: int, error_word: torch.Tensor, angles: Optional[torch.Tensor] = None,
                    cos_sin: Optional[torch.Tensor] = None, magnitude: float = 1.0,
                    values_from_keys: bool = False) -> None:
    """Per-head norm of q and k, rotation of q and k, q to ``q_out``, k and v into the pages.

    ``qkv`` is [rows, >= (n_q + 2 n_kv) head_dim] with q heads, k heads, v heads in that order,
    of ``q_out``'s dtype, or float32 [parts, rows, width] partial sums that are added in order;
    pools are [pages, n_kv, page_size, head_dim]; ``slots[r]`` = page * page_size + offset.
    With ``slots`` None nothing is written to the pages.  The rotation takes its angles as
    ``positions[r] * inv_freq[i]`` or, if ``angles`` (float32 [rows, rotary_dim / 2]) is given,
    from there.  ``cos_sin``: the table of :func:`rope_table` for these rows; the kernel for many rows
    then reads the cosines and sines instead of computing them (the same values).  ``magnitude`` multiplies the
    cosines and sines (a ``cos_sin`` table must hold them multiplied already).  With ``values_from_keys`` the rows
    of ``qkv`` hold q and k heads only, and the value stored for a key is the key as projected, unrotated."""
    _need(qkv, "qkv"); _need(q_out, "q_out"); _need(positions, "positions", torch.int32)
    if angles is not None:
        _need(angles, "angles", torch.float32)
        if angles.shape != (qkv.shape[-2], rotary_dim // 2):
            raise KernelError("qk_norm_rope_kv: angles must be [rows, rotary_dim / 2]")
    whole = parts = None
    num_parts = part_stride = 0
    if qkv.dim() == 3:
        _need(qkv, "qkv", torch.float32)
        parts, num_parts, part_stride = qkv, qkv.shape[0], qkv.stride(0)
    else:
        _need(qkv, "qkv", q_out.dtype)
        whole = qkv
    rows = qkv.shape[-2]
    page_size = num_pages = 1
    if slots is not None:
        _need(slots, "slots", torch.int32); _need(k_pool, "k_pool", q_out.dtype); _need(v_pool, "v_pool", q_out.dtype)
        num_pages, pool_heads, page_size, pool_dim = k_pool.shape
        if (pool_heads, pool_dim) != (n_kv, head_dim) or v_pool.shape != k_pool.shape:
            raise KernelError("qk_norm_rope_kv: pools must be [pages, n_kv, page_size, head_dim]")
        if qkv.shape[-1] < (n_q + (1 if values_from_keys else 2) * n_kv) * head_dim:
            raise KernelError("qk_norm_rope_kv: qkv is narrower than its heads together")
    for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None:
            _need(w, name, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"qk_norm_rope_kv: {name} must have head_dim elements")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("qk_norm_rope_kv: inv_freq must have rotary_dim / 2 elements")
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        if cos_sin.shape != (rows, rotary_dim):
            raise KernelError("qk_norm_rope_kv: cos_sin must be [rows, rotary_dim]")
    lib = load_library("rope_kv")
    _check(lib, lib.srb_qk_norm_rope_kv_ex(
        _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(part_stride), qkv.stride(-2), _ptr(q_out), _ptr(k_pool),
        _ptr(v_pool), _ptr(positions), _ptr(slots), _ptr(q_norm), _ptr(k_norm), ctypes.c_float(eps), _ptr(inv_freq),
        _ptr(angles), _ptr(cos_sin), rotary_dim, int(interleaved), rows, n_q, n_kv, head_dim, page_size, num_pages,
        _ptr(error_word), dtype_code(q_out.dtype), ctypes.c_float(magnitude), int(values_from_keys), _stream()))


@traced("rope_kv")
def proj_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                      positions: torch.Tensor, slots: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
                      k_weight: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                      interleaved: bool, n_q: int, n_kv: int, head_dim: int, value_dim: int, error_word: torch.Tensor, *,
                      magnitude: float = 1.0, gate_out: Optional[torch.Tensor] = None) -> None:
    """The step between the q/k/v product and attention for a mixer that norms q and k over the WHOLE projection (all
    heads of a row together, a weight per entry: ``q_weight`` [n_q * head_dim], ``k_weight`` [n_kv * head_dim]; None: no
    norm), then rotates the leading ``rotary_dim`` entries of every head, writes q to ``q_out`` [rows, n_q, head_dim], k
    into ``k_pool`` [pages, n_kv, page_size, head_dim] and the values, as projected, into ``v_pool`` [pages, n_kv,
    page_size, value_dim].  Rows of ``qkv`` are [q | k | v | gate logits]; ``gate_out`` (float32 [rows, gates]) receives
    the sigmoids of the logits behind the values.  ``qkv`` is of ``q_out``'s dtype or float32 [parts, rows, width]
    partial sums.  ``slots`` None: nothing is stored."""
    _need(qkv, "qkv"); _need(q_out, "q_out"); _need(positions, "positions", torch.int32)
    whole = parts = None
    num_parts = part_stride = 0
    if qkv.dim() == 3:
        _need(qkv, "qkv", torch.float32)
        parts, num_parts, part_stride = qkv, qkv.shape[0], qkv.stride(0)
    else:
        _need(qkv, "qkv", q_out.dtype)
        whole = qkv
    rows = qkv.shape[-2]
    gate_cols = 0
    if gate_out is not None:
        _need(gate_out, "gate_out", torch.float32)
        if gate_out.dim() != 2 or gate_out.shape[0] != rows:
            raise KernelError("proj_norm_rope_kv: gate_out must be [rows, gates]")
        gate_cols = gate_out.shape[1]
    if qkv.shape[-1] < (n_q + n_kv) * head_dim + n_kv * value_dim + gate_cols:
        raise KernelError("proj_norm_rope_kv: qkv is narrower than its parts together")
    if q_out.shape != (rows, n_q, head_dim):
        raise KernelError("proj_norm_rope_kv: q_out must be [rows, n_q, head_dim]")
    page_size = num_pages = 1
    if slots is not None:
        _need(slots, "slots", torch.int32); _need(k_pool, "k_pool", q_out.dtype); _need(v_pool, "v_pool", q_out.dtype)
        num_pages, pool_heads, page_size, pool_dim = k_pool.shape
        if (pool_heads, pool_dim) != (n_kv, head_dim) or v_pool.shape != (num_pages, n_kv, page_size, value_dim):
            raise KernelError("proj_norm_rope_kv: pools must be [pages, n_kv, page_size, head_dim] and [..., value_dim]")
    for name, w, count in (("q_weight", q_weight, n_q * head_dim), ("k_weight", k_weight, n_kv * head_dim)):
        if w is not None:
            _need(w, name, torch.float32)
            if w.numel() != count:
                raise KernelError(f"proj_norm_rope_kv: {name} must have {count} entries")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("proj_norm_rope_kv: inv_freq must have rotary_dim / 2 entries")
    lib = load_library("rope_kv")
    _check(lib, lib.srb_proj_norm_rope_kv(
        _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(part_stride), qkv.stride(-2), _ptr(q_out),
        _ptr(k_pool) if slots is not None else None, _ptr(v_pool) if slots is not None else None, _ptr(gate_out),
        _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps), _ptr(inv_freq), rotary_dim,
        int(interleaved), ctypes.c_float(magnitude), rows, n_q, n_kv, head_dim, value_dim, gate_cols, page_size, num_pages,
        _ptr(error_word), dtype_code(q_out.dtype), _stream()))


@traced("rope_kv")
def rope_table(positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
               angles: Optional[torch.Tensor] = None, magnitude: float = 1.0) -> torch.Tensor:
    """float32 [rows, rotary_dim]: per row the cosines, then the sines, of ``positions[r] * inv_freq[i]`` (or of
    ``angles[r, i]``), computed once for a step; the step executor hands it to the rope kernel of every layer."""
    _need(positions, "positions", torch.int32)
    rows = positions.numel()
    out = torch.empty((rows, rotary_dim), dtype=torch.float32, device=positions.device)
    lib = load_library("rope_kv")
    _check(lib, lib.srb_rope_table_scaled(_ptr(positions), _ptr(inv_freq), _ptr(angles), rows, rotary_dim, _ptr(out),
                                          ctypes.c_float(magnitude), _stream()))
    return out


def attention_scratch_sizes(rows: int, n_q: int, head_dim: int, max_splits: int) -> tuple[int, int]:
    """Floats of scratch that a split run needs: (partial accumulators, partial max and sum)."""
    return rows * n_q * max_splits * head_dim, rows * n_q * max_splits * 2


@traced("attention_generic")
def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                    positions: torch.Tensor, row_request: torch.Tensor, block_table: torch.Tensor, *,
                    scale: float, window: int, split_size: int, max_splits: int,
                    scratch_acc: Optional[torch.Tensor], scratch_ml: Optional[torch.Tensor],
                    error_word: torch.Tensor, sinks: Optional[torch.Tensor] = None, chunk: int = 0,
                    gates: Optional[torch.Tensor] = None) -> None:
    """out[r, h, :] = softmax over the keys row r may see of (q . k) * scale, times v.

    A row at position p sees the keys max(0, p - window + 1) .. p (``window`` 0: from 0) and, with ``chunk`` > 0,
    of those only the keys of its own chunk of positions, floor(p / chunk) * chunk .. p.

    ``sinks`` (float32, one per query head): the softmax's denominator also holds exp(sink_h), a term without
    key or value.  ``v_pool`` may hold rows of another width than the keys (``out`` is as wide as they are), and may be
    None: the value of a key is then the first ``out.shape[2]`` entries of its key row.  ``gates`` (float32
    [rows, n_q]): a factor on the result of every (row, query head).

    q, out: [rows, n_q, head_dim]; pools [pages, n_kv, page_size, head_dim]; block_table
    [requests, stride].  ``split_size`` 0 walks all keys in one block per (row, kv head);
    otherwise partials go through the scratch tensors and are merged in split order.
    This is the generic kernel (any head_dim that is a multiple of 16, float32 or bfloat16)."""
    _need(q, "q"); _need(out, "out", q.dtype); _need(k_pool, "k_pool", q.dtype)
    _need(positions, "positions", torch.int32); _need(row_request, "row_request", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    value_dim = out.shape[2]
    if pool_dim != head_dim or out.shape[:2] != q.shape[:2] or (v_pool is None and value_dim > head_dim):
        raise KernelError("paged_attention: shapes of q, out and the pools do not agree")
    if gates is not None:
        _need(gates, "gates", torch.float32)
        if gates.shape != (rows, n_q):
            raise KernelError("paged_attention: one gate per row and query head is needed")
    if v_pool is not None:
        _need(v_pool, "v_pool", q.dtype)
        if v_pool.shape != (*k_pool.shape[:3], value_dim):
            raise KernelError("paged_attention: the value pool must be [pages, n_kv, page_size, width of out]")
    if sinks is not None:
        _need(sinks, "sinks", torch.float32)
        if sinks.numel() != n_q:
            raise KernelError("paged_attention: one sink per query head is needed")
    if split_size:
        need_acc, need_ml = attention_scratch_sizes(rows, n_q, value_dim, max_splits)
        if scratch_acc is None or scratch_ml is None or scratch_acc.numel() < need_acc or scratch_ml.numel() < need_ml:
            raise KernelError("paged_attention: scratch tensors are too small for this split run")
        _need(scratch_acc, "scratch_acc", torch.float32); _need(scratch_ml, "scratch_ml", torch.float32)
    lib = load_library("attention")
    _check(lib, lib.srb_paged_attention_gated(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(scratch_acc), _ptr(scratch_ml), _ptr(positions),
        _ptr(row_request), _ptr(block_table), block_table.stride(0), rows, n_q, n_kv, head_dim, page_size,
        num_pages, int(window), int(chunk), int(split_size), int(max_splits), ctypes.c_float(scale), _ptr(error_word),
        dtype_code(q.dtype), _ptr(sinks), value_dim, _ptr(gates), _stream()), launches=2 if split_size else 1)





def latent_attention_takes(dtype: torch.dtype, row_dim: int, value_dim: int) -> bool:
    """True if the tensor-core kernel for attention over rows that are key and value takes these sizes (the rule of
    srb_latent_attention_supports, asked here so that other models never compile it)."""
    return (dtype == torch.bfloat16 and row_dim % 16 == 0 and value_dim % 32 == 0 and 0 < value_dim <= min(row_dim, 512))


@traced("attention_latent")
def latent_attention(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                     row_request: torch.Tensor, block_table: torch.Tensor, *, scale: float, sinks: Optional[torch.Tensor],
                     error_word: torch.Tensor, tiles: Optional[torch.Tensor] = None, split_size: int = 0, max_splits: int = 1,
                     scratch_acc: Optional[torch.Tensor] = None, scratch_ml: Optional[torch.Tensor] = None,
                     window: int = 0) -> None:
    """Attention of ``n_q`` query heads over cache rows that are key (the whole row) and value (its first
    ``out.shape[2]`` entries), bfloat16 on the tensor cores, with an optional sink per head.

    With ``tiles`` (int32 [n, 4]: first row, rows <= 64, request, first position) the rows of the tiles are prompt
    portions: every row sees the keys up to its own position, and rows outside the tiles are left untouched.  Without,
    every row of ``q`` is one decoded token whose keys are cut every ``split_size`` positions (a multiple of 64); partial
    results go through the scratch tensors (rows * n_q * max_splits * value_dim and rows * n_q * max_splits * 2 floats).
    ``window`` > 0: a row sees itself and the ``window`` - 1 keys before it; splits are then counted from the split of a
    row's first visible key, as the planner of a window group counts them."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pool, "pool", torch.bfloat16)
    _need(positions, "positions", torch.int32); _need(row_request, "row_request", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, row_dim = q.shape
    num_pages, kv_heads, page_size, pool_dim = pool.shape
    value_dim = out.shape[2]
    if kv_heads != 1 or pool_dim != row_dim or out.shape[:2] != q.shape[:2] or not latent_attention_takes(q.dtype, row_dim, value_dim):
        raise KernelError("latent_attention: shapes of q, out and the pool do not agree or are not taken")
    if sinks is not None:
        _need(sinks, "sinks", torch.float32)
        if sinks.numel() != n_q:
            raise KernelError("latent_attention: one sink per query head is needed")
    num_tiles = 0
    if tiles is not None:
        _need(tiles, "tiles", torch.int32)
        if tiles.shape[-1] != 4:
            raise KernelError("latent_attention: tiles must be [n, 4]")
        num_tiles, split_size, max_splits = tiles.shape[0], 0, 1
    else:
        need_acc, need_ml = attention_scratch_sizes(rows, n_q, value_dim, max_splits)
        if scratch_acc is None or scratch_ml is None or scratch_acc.numel() < need_acc or scratch_ml.numel() < need_ml:
            raise KernelError("latent_attention: scratch tensors are too small for this split run")
        _need(scratch_acc, "scratch_acc", torch.float32); _need(scratch_ml, "scratch_ml", torch.float32)
    lib = load_library("attention_latent")
    _check(lib, lib.srb_latent_attention_masked(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(scratch_acc), _ptr(scratch_ml), _ptr(positions), _ptr(row_request),
        _ptr(block_table), block_table.stride(0), rows, n_q, row_dim, value_dim, page_size, num_pages, int(split_size),
        int(max_splits), _ptr(tiles), num_tiles, ctypes.c_float(scale), _ptr(sinks), int(window), _ptr(error_word), _stream()),
        launches=1 if tiles is not None else 2)


#: the most blocks per (row, kv head) that :func:`decode_splits` ever returns
DECODE_MAX_SPLITS = 64


def decode_attention_takes(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int) -> bool:
    """True if the tensor-core kernel for decoded tokens takes these sizes (the rule of
    srb_decode_attention_supports, asked here so that other models never compile it)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_q % n_kv == 0 and n_q // n_kv <= 16




def decode_splits(rows: int, n_kv: int, max_keys: Optional[int] = None, sms: Optional[int] = None) -> int:
    """Blocks per (row, kv head).  A function of the shape and of the device's SM count (``sms``;
    default: the current device's) only; defined in csrc/step_exec.cu, where the step executor uses it too.

    Without ``max_keys`` (the most keys any row sees): as many as make about three blocks per SM.
    With it, the count that makes the step shortest under a simple model: the blocks run in waves
    of three per SM, and a wave lasts as long as one block's share of the keys plus a fixed cost.
    Many rows then still get their keys cut (512 blocks are 1.15 waves: nearly half the second
    wave's time is lost), and no block walks fewer than two 64-key units."""
    return records.library().sx_decode_splits(int(rows), int(n_kv), -1 if max_keys is None else int(max_keys),
                                              int(sms if sms is not None else sm_count()))


def decode_splits_bound(max_keys: int) -> int:
    """No call of :func:`decode_splits` with this ``max_keys`` returns more, whatever the rows and heads."""
    return records.library().sx_decode_splits_bound(int(max_keys))


@traced("attention_decode")
def decode_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                     positions: torch.Tensor, row_request: torch.Tensor, block_table: torch.Tensor, *,
                     scale: float, window: int, scratch_acc: torch.Tensor, scratch_ml: torch.Tensor,
                     counters: torch.Tensor, error_word: torch.Tensor, max_keys: Optional[int] = None,
                     chunk: int = 0, sinks: Optional[torch.Tensor] = None, gates: Optional[torch.Tensor] = None) -> None:
    """Attention of decoded tokens (one row each), bfloat16, head_dim 64 or 128; ``window``, ``chunk``, ``sinks`` and
    ``gates`` as in :func:`paged_attention` (the sink joins where a row's splits are merged, once).

    The keys of a (row, kv head) are shared by ``decode_splits(rows, n_kv, max_keys)`` blocks
    (``max_keys``: the most keys any row sees, if known); the block that finishes last merges them.  ``counters``: int32, zero, at least rows * n_kv entries; they
    are zero again afterwards.  Scratch: rows * n_q * splits * head_dim and rows * n_q * splits * 2
    floats."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(positions, "positions", torch.int32)
    _need(row_request, "row_request", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(scratch_acc, "scratch_acc", torch.float32); _need(scratch_ml, "scratch_ml", torch.float32)
    _need(counters, "counters", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape:
        raise KernelError("decode_attention: shapes of q, out and the pools do not agree")
    # never more blocks than the scratch memory holds partial results for
    splits = max(1, min(decode_splits(rows, n_kv, max_keys), scratch_acc.numel() // (rows * n_q * head_dim),
                        scratch_ml.numel() // (rows * n_q * 2)))
    if scratch_acc.numel() < rows * n_q * splits * head_dim or scratch_ml.numel() < rows * n_q * splits * 2:
        raise KernelError("decode_attention: scratch tensors are too small")
    if counters.numel() < rows * n_kv:
        raise KernelError("decode_attention: too few counters")
    rows_, heads_ = q.shape[0], q.shape[1]
    if sinks is not None:
        _need(sinks, "sinks", torch.float32)
        if sinks.numel() != heads_:
            raise KernelError("decode_attention: one sink per query head is needed")
    if gates is not None:
        _need(gates, "gates", torch.float32)
        if gates.shape != (rows_, heads_):
            raise KernelError("decode_attention: one gate per row and query head is needed")
    lib = load_library("attention_decode")
    _check(lib, lib.srb_decode_attention_gated(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(scratch_acc), _ptr(scratch_ml), _ptr(counters),
        _ptr(positions), _ptr(row_request), _ptr(block_table), block_table.stride(0), rows, n_q, n_kv, head_dim,
        page_size, num_pages, int(window), int(chunk), splits, ctypes.c_float(scale), _ptr(error_word), _ptr(sinks),
        _ptr(gates), _stream()))


def tiled_attention_takes(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int) -> bool:
    """True if the tensor-core kernel for prompt portions takes these sizes."""
    # the same rule as srb_prefill_attention_supports, asked here so that a model the kernel
    # does not take never compiles it
    return dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_q % n_kv == 0


@traced("attention_prefill")
def tiled_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                    tiles: torch.Tensor, block_table: torch.Tensor, *, scale: float, window: int,
                    error_word: torch.Tensor, chunk: int = 0, sinks: Optional[torch.Tensor] = None,
                    gates: Optional[torch.Tensor] = None) -> None:
    """Attention of prompt portions, bfloat16 (``sinks``, ``gates``: as in :func:`paged_attention`).  ``tiles`` is int32 [n, 4]: first row of the
    step, rows (at most 64, consecutive rows of one request), request index, first position.
    Rows outside the tiles are left untouched."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(tiles, "tiles", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape or tiles.shape[-1] != 4:
        raise KernelError("tiled_attention: shapes of q, out, the pools and the tiles do not agree")
    rows_, heads_ = q.shape[0], q.shape[1]
    if sinks is not None:
        _need(sinks, "sinks", torch.float32)
        if sinks.numel() != heads_:
            raise KernelError("tiled_attention: one sink per query head is needed")
    if gates is not None:
        _need(gates, "gates", torch.float32)
        if gates.shape != (rows_, heads_):
            raise KernelError("tiled_attention: one gate per row and query head is needed")
    lib = load_library("attention_prefill")
    _check(lib, lib.srb_prefill_attention_gated(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(tiles), tiles.shape[0], _ptr(block_table),
        block_table.stride(0), n_q, n_kv, head_dim, page_size, num_pages, int(window), int(chunk), ctypes.c_float(scale),
        _ptr(error_word), _ptr(sinks), _ptr(gates), _stream()))


TC_TILE_ROWS = 128


def tiled_attention_tc_takes(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """True if the tcgen05 kernel for prompt portions takes these sizes (the rule of
    srb_prefill_tc_supports)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_q % n_kv == 0
            and page_size >= 8 and page_size % 8 == 0 and 64 % page_size == 0)


@traced("attention_prefill")
def tiled_attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                       tiles: torch.Tensor, block_table: torch.Tensor, *, scale: float, window: int,
                       error_word: torch.Tensor, chunk: int = 0, sinks: Optional[torch.Tensor] = None,
                       gates: Optional[torch.Tensor] = None) -> None:
    """Attention of prompt portions on tcgen05 tensor cores (S, P and O in tensor memory, operands
    by TMA; ``sinks``, ``gates``: as in :func:`paged_attention`).  ``tiles`` as for :func:`tiled_attention`, with at most 128 rows per tile."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(tiles, "tiles", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape or tiles.shape[-1] != 4:
        raise KernelError("tiled_attention_tc: shapes of q, out, the pools and the tiles do not agree")
    rows_, heads_ = q.shape[0], q.shape[1]
    if sinks is not None:
        _need(sinks, "sinks", torch.float32)
        if sinks.numel() != heads_:
            raise KernelError("tiled_attention_tc: one sink per query head is needed")
    if gates is not None:
        _need(gates, "gates", torch.float32)
        if gates.shape != (rows_, heads_):
            raise KernelError("tiled_attention_tc: one gate per row and query head is needed")
    lib = load_library("attention_prefill_tc")
    _check(lib, lib.srb_prefill_attention_tc_gated(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(tiles), tiles.shape[0], rows, _ptr(block_table),
        block_table.stride(0), n_q, n_kv, head_dim, page_size, num_pages, int(window), int(chunk), ctypes.c_float(scale),
        _ptr(error_word), _ptr(sinks), _ptr(gates), _stream()))


# --------------------------------------------------------------------------- latents and per-head products

@traced("latent_prepare")
def latent_prepare(proj: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, q_weight: Optional[torch.Tensor],
                   kv_weight: torch.Tensor, eps: float, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                   rotary_dim: int, q_latent: Optional[torch.Tensor], pool: Optional[torch.Tensor],
                   slots: Optional[torch.Tensor], error_word: torch.Tensor, interleaved: bool = False,
                   magnitude: float = 1.0) -> None:
    """Rows of ``proj`` hold [query latent (q_rank) | key/value latent (kv_rank) | shared key part (rot_dim) | ...].
    ``q_latent[r]`` = RMS norm of the first; the row's slot of ``pool`` ([pages, 1, page_size, kv_rank + rot_dim])
    receives the RMS norm of the second and the rotated third.  ``slots`` None: nothing is stored.  The rotation pairs
    entry i with entry i + rotary_dim / 2, or, with ``interleaved``, entry 2i with 2i + 1; ``magnitude`` multiplies the
    cosines and sines."""
    _need(positions, "positions", torch.int32); _need(kv_weight, "kv_weight", torch.float32)
    if proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("latent_prepare: proj must be a CUDA matrix with dense rows")
    rows = proj.shape[0]
    if proj.shape[1] < q_rank + kv_rank + rot_dim:
        raise KernelError("latent_prepare: rows of proj are too short")
    if q_rank:
        _need(q_latent, "q_latent", proj.dtype); _need(q_weight, "q_weight", torch.float32)
        if q_latent.shape != (rows, q_rank) or q_weight.numel() != q_rank:
            raise KernelError("latent_prepare: the query latent must be [rows, q_rank]")
    pool_rows = 0
    if slots is not None:
        _need(slots, "slots", torch.int32); _need(pool, "pool", proj.dtype)
        if pool.shape[-1] != kv_rank + rot_dim or pool.shape[1] != 1:
            raise KernelError("latent_prepare: the pool must be [pages, 1, page_size, kv_rank + rot_dim]")
        pool_rows = pool.shape[0] * pool.shape[2]
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("latent_prepare: inv_freq must have rotary_dim / 2 entries")
    lib = load_library("latent")
    _check(lib, lib.srb_latent_prepare_ex(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), rows, q_rank, kv_rank, rot_dim, _ptr(q_weight), _ptr(kv_weight),
        ctypes.c_float(eps), _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(q_latent), _ptr(pool), _ptr(slots),
        ctypes.c_longlong(pool_rows), _ptr(error_word), dtype_code(proj.dtype), int(interleaved), ctypes.c_float(magnitude),
        _stream()))


@traced("rope_slice")
def rope_slice(x: torch.Tensor, in_offset: int, out: torch.Tensor, out_offset: int, width: int, rotary_dim: int,
               positions: torch.Tensor, inv_freq: Optional[torch.Tensor], interleaved: bool = False,
               magnitude: float = 1.0) -> None:
    """out[r, h, out_offset + i] = rotated(x[r, h, in_offset + i]), i < width, pairs (i, i + rotary_dim / 2) or, with
    ``interleaved``, (2i, 2i + 1); ``magnitude`` multiplies the cosines and sines; entries from ``rotary_dim`` on are
    copied.  x, out: [rows, heads, *] with dense last axis."""
    _need(x, "x"); _need(out, "out", x.dtype); _need(positions, "positions", torch.int32)
    if x.dim() != 3 or out.dim() != 3 or x.shape[:2] != out.shape[:2]:
        raise KernelError("rope_slice: x and out must be [rows, heads, *]")
    if in_offset + width > x.shape[2] or out_offset + width > out.shape[2]:
        raise KernelError("rope_slice: the slice does not fit")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rope_slice: inv_freq must have rotary_dim / 2 entries")
    lib = load_library("latent")
    _check(lib, lib.srb_rope_slice_ex(
        _ptr(x), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(x.stride(1)), in_offset, _ptr(out),
        ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out.stride(1)), out_offset, x.shape[0], x.shape[1], width,
        rotary_dim, _ptr(positions), _ptr(inv_freq), dtype_code(x.dtype), int(interleaved), ctypes.c_float(magnitude),
        _stream()))


@traced("head_linear")
def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                gate_per_entry: bool = False) -> None:
    """out[r, h, :n_out] = weight[h] @ x[r, h, :n_in] with ``weight`` [heads, n_out, n_in]; x and out are views
    [rows, heads, >= n] with a dense last axis.  ``gate`` ([rows, >= heads] view of logits): head h's result is
    multiplied by sigmoid(gate[r, h]); with ``gate_per_entry`` the gate is [rows, >= heads * n_out] and entry o of head
    h is multiplied by sigmoid(gate[r, h * n_out + o])."""
    heads, n_out, n_in = weight.shape
    _need(weight, "weight", x.dtype)
    if (x.dim() != 3 or out.dim() != 3 or x.shape[1] != heads or out.shape[1] != heads or x.shape[0] != out.shape[0]
            or x.shape[2] < n_in or out.shape[2] < n_out or x.stride(2) != 1 or out.stride(2) != 1 or out.dtype != x.dtype):
        raise KernelError("head_linear: x, weight and out do not fit")
    gate_row = 0
    if gate is not None:
        gates = heads * (n_out if gate_per_entry else 1)
        if gate.dim() != 2 or gate.shape[0] != x.shape[0] or gate.shape[1] < gates or gate.stride(1) != 1 or gate.dtype != x.dtype:
            raise KernelError("head_linear: gate must be [rows, heads (times entries)] of x's dtype with a dense last axis")
        gate_row = gate.stride(0)
    lib = load_library("latent")
    _check(lib, lib.srb_head_linear_ex(
        _ptr(x), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(x.stride(1)), _ptr(weight), _ptr(out),
        ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out.stride(1)), x.shape[0], heads, n_in, n_out, _ptr(gate),
        ctypes.c_longlong(gate_row), n_out if gate_per_entry else 1, 1 if gate_per_entry else 0, dtype_code(x.dtype),
        _stream()))


# --------------------------------------------------------------------------- routed experts

#: bfloat16 steps with many choices per expert run the experts' two products on the grouped mode of the tcgen05
#: kernel (csrc/gemm_bf16.cu) over rows gathered into slot order; SRB_GROUPED_EXPERTS=0 keeps the mma.sync tiles
GROUPED_EXPERTS = os.environ.get("SRB_GROUPED_EXPERTS", "1") not in ("0", "off", "false")
#: from this many rows on the router's logits come from the product kernels (every block of the fused router kernel reads
#: the whole router matrix: 94 us at 2,048 rows and 64 experts of width 2,048 against the product's few)
ROUTER_PRODUCT_MIN_ROWS = 128
#: slots of a tile of the grouped products (128 or 256): 256 reads an expert's weight tile once for twice as many rows
GROUPED_TILE_SLOTS = int(os.environ.get("SRB_GROUPED_TILE_SLOTS", "256"))
#: how a router's logits become scores, by the numbers of csrc/moe.cu
ROUTER_SCORING = {"softmax": 0, "sigmoid": 1}


@traced("routed_experts")
def routed_experts(h: torch.Tensor, router: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, top: int,
                   activation: str, renormalize: bool, error_word: torch.Tensor, *, gated: bool = True,
                   router_bias: Optional[torch.Tensor] = None, base: Optional[torch.Tensor] = None,
                   scoring: str = "softmax", choice_bias: Optional[torch.Tensor] = None, weight_scale: float = 1.0,
                   norm_eps: float = 0.0, activation_param: float = 0.0, identity: int = 0) -> torch.Tensor:
    """sum over the ``top`` experts with the largest router scores of score * expert(h), float32 [rows, width].

    ``identity``: the router has this many outputs more than there are expert matrices; they stand for experts that return
    their input, so a row that chooses one gets weight * h[row] as that expert's term (the scores and the choice run over
    all outputs alike; ``router``, ``router_bias`` and ``choice_bias`` have experts + identity rows).

    ``gated`` False: an expert is W_down act(W_up h) and ``w_gate_up`` holds the up matrices alone
    [experts, inner, width].  ``router_bias`` (float32 [experts]) is added to the router's logits before the choice.
    ``base`` (float32 [rows, width]): a term that every row gets beside its experts' (an expert that all rows
    share); the sum starts from it.  ``scoring`` ``sigmoid``: an expert's score is the sigmoid of its logit instead of
    the softmax over all; ``choice_bias`` (float32 [experts]) is added to the scores for the choice only; the weights
    are the chosen scores, with ``renormalize`` divided by (their sum + ``norm_eps``), then times ``weight_scale``.
    ``activation_param``: the parameter of an activation that has one.

    ``router`` [experts, width]; ``w_gate_up`` [experts, 2 * inner, width] (an expert's gate rows over its up rows);
    ``w_down`` [experts, width, inner], all of h's dtype.  Scores are a softmax over all experts, in 32-bit; with
    ``renormalize`` the chosen ones are divided by their sum.  Five launches (six with the gather of the grouped
    products), nothing decided on the host.

    The two products: float32 and odd sizes on FFMA or 64 x 64 mma tiles; bfloat16 on mma.sync tiles with asynchronous
    copies, or, where a step has many choices per expert (tiles of 128 slots), on tcgen05 tensor cores through the
    grouped mode of :func:`gemm_bf16`'s kernel: the rows are gathered into slot order first, so that a tile's operand is
    128 consecutive rows that TMA can fetch."""
    _need(h, "h"); _need(router, "router", h.dtype); _need(w_gate_up, "w_gate_up", h.dtype); _need(w_down, "w_down", h.dtype)
    rows, width = h.shape
    experts, inner = w_gate_up.shape[0], w_gate_up.shape[1] // (2 if gated else 1)
    routes = experts + int(identity)
    if identity < 0 or routes > 1024:
        raise KernelError(f"routed_experts: {routes} router outputs are outside what the router kernels take (1024)")
    if (router.shape != (routes, width) or w_gate_up.shape != (experts, (2 if gated else 1) * inner, width)
            or w_down.shape != (experts, width, inner)):
        raise KernelError("routed_experts: shapes of the router and the experts do not agree")
    if router_bias is not None:
        _need(router_bias, "router_bias", torch.float32)
        if router_bias.numel() != routes:
            raise KernelError("routed_experts: one router bias per router output is needed")
    if base is not None:
        _need(base, "base", torch.float32)
        if base.shape != (rows, width):
            raise KernelError("routed_experts: the shared term must be float32 [rows, width]")
    if choice_bias is not None:
        _need(choice_bias, "choice_bias", torch.float32)
        if choice_bias.numel() != routes:
            raise KernelError("routed_experts: one choice bias per router output is needed")
    rule = (int(renormalize), ROUTER_SCORING[scoring], _ptr(choice_bias), ctypes.c_float(weight_scale), ctypes.c_float(norm_eps))
    act_code, act_param = activation_code(activation, parametric=True), ctypes.c_float(activation_param)
    lib = load_library("moe")
    device = h.device
    entries = rows * top
    chosen = torch.empty(entries, dtype=torch.int32, device=device)
    weights = torch.empty(entries, dtype=torch.float32, device=device)
    grouped = (GROUPED_EXPERTS and h.dtype == torch.bfloat16 and width % 8 == 0 and inner % 8 == 0
               and lib.srb_moe_tile_rows(rows, top, experts) == 128)
    tile_slots = GROUPED_TILE_SLOTS if grouped else lib.srb_moe_tile_rows(rows, top, experts)
    plan = torch.empty(lib.srb_moe_plan_ints_of(rows, top, experts, tile_slots), dtype=torch.int32, device=device)
    slot_row = torch.empty(entries, dtype=torch.int32, device=device)
    entry_slot = torch.empty(entries, dtype=torch.int32, device=device)
    act = torch.empty((entries, inner), dtype=h.dtype, device=device)
    y = torch.empty((entries, width), dtype=torch.float32, device=device)
    out = torch.empty((rows, width), dtype=torch.float32, device=device)
    code, stream = dtype_code(h.dtype), _stream()
    if rows >= ROUTER_PRODUCT_MIN_ROWS or router_bias is not None:
        # many rows: the logits are a product like any other (32-bit accumulation, 32-bit result), the choice a kernel of its own
        logits = linear(h, router, router_bias, out_dtype=torch.float32, error_word=error_word)
        _check(lib, lib.srb_moe_select_ex(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, routes, top, *rule,
                                          _ptr(chosen), _ptr(weights), stream))
    else:
        _check(lib, lib.srb_moe_route_ex(_ptr(h), _ptr(router), rows, width, routes, top, *rule, _ptr(chosen),
                                         _ptr(weights), code, stream))
    _check(lib, lib.srb_moe_plan_of(_ptr(chosen), rows, top, experts, tile_slots, _ptr(plan), _ptr(slot_row),
                                    _ptr(entry_slot), _ptr(error_word), stream))
    if grouped:
        product = load_library("gemm_bf16")
        max_tiles = lib.srb_moe_max_tiles_of(rows, top, experts, tile_slots)
        gathered = torch.empty((entries, width), dtype=h.dtype, device=device)
        # the plan's last offset is the number of slots handed out (choices of experts without tensors get none)
        used = ctypes.c_void_p(plan.data_ptr() + 4 * (1 + experts))
        _check(lib, lib.srb_moe_gather_used(_ptr(h), _ptr(slot_row), entries, width, _ptr(gathered), used, code, stream))
        _check(product, product.srb_gemm_bf16_grouped(
            _ptr(gathered), _ptr(w_gate_up), _ptr(act), _ptr(plan), max_tiles, tile_slots, entries, experts,
            (2 if gated else 1) * inner, inner, width, inner, inner if gated else 0, GEMM_MODES["gated" if gated else "act"],
            act_code, act_param, _ptr(error_word), stream))
        _check(product, product.srb_gemm_bf16_grouped(
            _ptr(act), _ptr(w_down), _ptr(y), _ptr(plan), max_tiles, tile_slots, entries, experts, width, width, inner, width, 0,
            GEMM_MODES["f32"], 0, ctypes.c_float(0.0), _ptr(error_word), stream))
    else:
        element = h.element_size()
        if gated:
            w_up = ctypes.c_void_p(w_gate_up.data_ptr() + inner * width * element)
            _check(lib, lib.srb_moe_gated_up(_ptr(h), _ptr(w_gate_up), w_up, ctypes.c_longlong(2 * inner * width), _ptr(plan),
                                             _ptr(slot_row), rows, top, experts, width, inner, act_code, act_param,
                                             _ptr(act), code, stream))
        else:
            _check(lib, lib.srb_moe_act_up(_ptr(h), _ptr(w_gate_up), _ptr(plan), _ptr(slot_row), rows, top, experts, width,
                                           inner, act_code, act_param, _ptr(act), code, stream))
        _check(lib, lib.srb_moe_down(_ptr(act), _ptr(w_down), _ptr(plan), rows, top, experts, width, inner, _ptr(y), code,
                                     stream))
    # choices of `experts` and above have no slot in the plan: they are the experts that return their input
    _check(lib, lib.srb_moe_combine_identity(_ptr(y), _ptr(entry_slot), _ptr(weights), rows, top, width, _ptr(out), _ptr(base),
                                             _ptr(chosen) if identity else None, experts, _ptr(h) if identity else None, code,
                                             stream))
    return out


def route(h: torch.Tensor, router: torch.Tensor, top: int, renormalize: bool = False, *, scoring: str = "softmax",
          choice_bias: Optional[torch.Tensor] = None, weight_scale: float = 1.0, norm_eps: float = 0.0):
    """The router alone: (chosen experts int32 [rows, top], their weights float32 [rows, top]); the options are
    those of :func:`routed_experts`."""
    _need(h, "h"); _need(router, "router", h.dtype)
    if choice_bias is not None:
        _need(choice_bias, "choice_bias", torch.float32)
    rows, width = h.shape
    chosen = torch.empty((rows, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((rows, top), dtype=torch.float32, device=h.device)
    lib = load_library("moe")
    _check(lib, lib.srb_moe_route_ex(_ptr(h), _ptr(router), rows, width, router.shape[0], top, int(renormalize),
                                     ROUTER_SCORING[scoring], _ptr(choice_bias), ctypes.c_float(weight_scale),
                                     ctypes.c_float(norm_eps), _ptr(chosen), _ptr(weights), dtype_code(h.dtype), _stream()))
    return chosen, weights


# --------------------------------------------------------------------------- matrix products

#: The two thresholds below were measured at Qwen3-8B sizes on a B200; they are tunables (the environment
#: variables SRB_OWN_GEMM_MAX_TOKENS and SRB_PAIR_GEMM_MIN_TOKENS set them), read at every step.
#: up to this many rows a bfloat16 product runs on this package's tcgen05 kernel for few tokens.  With 65 to
#: 128 rows the kernel has one block per SM and no cut along K, and the library is twice as fast
#: (Qwen3-8B sizes on B200, chained in a graph: QKV 12 against 20 us, down 23 against 52 us; a 12-layer
#: decode step at batch 128 takes 3.80 ms instead of 4.48 ms)
OWN_GEMM_MAX_TOKENS = int(os.environ.get("SRB_OWN_GEMM_MAX_TOKENS", "64"))
#: from this many rows on the gate/up product runs on the persistent CTA-pair kernel, which takes SiLU(gate) * up
#: into its epilogue.  Measured at Qwen3-8B sizes on B200, chained in a graph, against the library's product
#: followed by the SiLU kernel: 64.8 against 53.7 us at 256 rows (96 tiles of 256 tokens leave the second
#: round of the 74 pairs mostly empty), 155 against 155 us at 1,024, 214 against 219 us at 1,536, 280 against
#: 301 us at 2,048.  The plain products stay with the library at every size: the pair kernel reaches 0.92 to
#: 1.0 of it alone, and whole prefill steps measured no gain from switching them.
PAIR_GEMM_MIN_TOKENS = int(os.environ.get("SRB_PAIR_GEMM_MIN_TOKENS", "1280"))


def gemm_splits(tokens: int, features: int, k: int, sms: Optional[int] = None) -> int:
    """Into how many partial sums a small-batch product is cut along K.  A function of the
    shape and of the device's SM count only: blocks of 128 weight rows alone cannot occupy the SMs when
    there are few of them, so K is cut until about two blocks per SM exist (two fit), each with at least
    8 K blocks.  Defined in csrc/step_exec.cu, where the step executor uses it too."""
    return records.library().sx_gemm_splits(int(tokens), int(features), int(k), int(sms if sms is not None else sm_count()),
                                            OWN_GEMM_MAX_TOKENS)


@traced("gemm")
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, error_word: Optional[torch.Tensor] = None,
           partial_ok: bool = False) -> torch.Tensor:
    """y = x @ weight^T (+ bias); weight is [out, in], row-major.

    float32: the FFMA kernel of this package, true 32-bit.  bfloat16: up to
    ``OWN_GEMM_MAX_TOKENS`` rows the tcgen05 kernel of this package, above that cuBLAS
    (:func:`library_product`: what the reference's engine calls for every projection,
    crates/sglang-kernel/src/cublas.rs:383-410); both accumulate in 32-bit.  ``out_dtype``
    float32 keeps the accumulator's precision (used for the logits).  With ``partial_ok`` the
    result may be float32 [parts, rows, out]: partial sums over K that the consumer adds in
    order (``add_rmsnorm`` and ``qk_norm_rope_kv`` do)."""
    _need(x, "x"); _need(weight, "weight", x.dtype)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} and weight {tuple(weight.shape)} do not fit")
    m, k = x.shape
    n = weight.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        if bias is not None:
            _need(bias, "bias", torch.float32)
        lib = load_library("gemm_f32")
        _check(lib, lib.srb_gemm_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k, x.stride(0),
                                     weight.stride(0), out.stride(0), _stream()))
        return out
    if m <= OWN_GEMM_MAX_TOKENS and error_word is not None and gemm_bf16_takes(k):
        splits = gemm_splits(m, n, k) if partial_ok else 1
        if splits > 1:
            out = gemm_bf16(x, weight, error_word, mode="partial", splits=splits)
            if bias is not None:
                add_bias(out[0], bias)
            return out
        out = gemm_bf16(x, weight, error_word, mode="f32" if out_dtype == torch.float32 else "bf16")
    else:
        out = library_product(x, weight, torch.float32 if out_dtype == torch.float32 else torch.bfloat16)
    if bias is not None:
        add_bias(out, bias)
    return out


def library_product(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y = x @ weight^T by cuBLAS (``cublasGemmEx``, bfloat16 operands, 32-bit accumulation to the end), the
    call the reference's engine makes for every projection (crates/sglang-kernel/src/cublas.rs:383-410).  The
    same call, through the same handle and scratch memory, takes the products of many rows inside the step
    executor."""
    records.ensure_cublas(x.device)
    m, k = x.shape
    n = weight.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    lib = records.library()
    _check(lib, lib.sx_cublas_product(_ptr(x), _ptr(weight), _ptr(out), m, n, k, x.stride(0), weight.stride(0), out.stride(0),
                                      int(out_dtype == torch.float32), _stream()))
    return out


@traced("gemm")
def gated_product(x: torch.Tensor, weight: torch.Tensor, inner: int, error_word: Optional[torch.Tensor] = None,
                  activation: str = "silu") -> torch.Tensor:
    """act(x gate^T) * (x up^T) for ``weight`` = gate rows stacked over up rows [2 inner, in].

    bfloat16 with few rows: one tcgen05 kernel whose epilogue takes the product of its two
    accumulators, so the [rows, 2 inner] intermediate never exists; with many rows the CTA-pair
    kernel does the same.  Otherwise the product (``linear``) followed by the activation kernel."""
    if (x.dtype == torch.bfloat16 and x.shape[0] <= OWN_GEMM_MAX_TOKENS and error_word is not None
            and gemm_bf16_takes(x.shape[1])):
        return gemm_bf16(x, weight, error_word, mode="gated", features=inner, up_row_offset=inner, activation=activation)
    if (x.dtype == torch.bfloat16 and error_word is not None and weight.shape[0] == 2 * inner
            and pair_gemm_takes(x.shape[0], inner, x.shape[1])):
        return gemm_bf16_pair(x, weight, error_word, mode="gated", features=inner, up_row_offset=inner,
                              activation=activation)
    gate_up = linear(x, weight, error_word=error_word)
    act = torch.empty((x.shape[0], inner), dtype=x.dtype, device=x.device)
    gated_mul(gate_up, act, activation)
    return act


GEMM_MODES = {"bf16": 0, "f32": 1, "gated": 2, "partial": 3, "add": 4, "act": 5}
#: the blocks of a thread-block cluster: at most this many K splits add their sums inside the kernel
GEMM_CLUSTER_SPLITS = 8


@traced("gemm")
def gemm_bf16(x: torch.Tensor, w: torch.Tensor, error_word: torch.Tensor, *, mode: str = "bf16",
              features: Optional[int] = None, up_row_offset: int = 0, splits: int = 1,
              out: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """y = x @ w^T on tcgen05 tensor cores (bfloat16 in, 32-bit accumulation).

    x [tokens, k], w [rows, k], k a multiple of 8.  ``mode``: ``bf16`` / ``f32`` store
    [tokens, features]; ``gated`` treats w as gate rows [0, features) stacked over up rows
    [up_row_offset, up_row_offset + features) and stores act(gate) * up (``activation``: a name of
    ``ACTIVATIONS``); ``act`` stores act(x w^T) in bfloat16; ``partial`` stores
    ``splits`` float partial sums [splits, tokens, features] that the consumer adds in order;
    ``add`` adds the product to ``out`` (float32 [tokens, features], e.g. the residual stream) in
    place, K cut into at most ``GEMM_CLUSTER_SPLITS`` blocks that sum inside the kernel in block order.
    (The engine's decode steps do not use ``add``: measured at Qwen3-8B sizes, partial sums that the
    next norm kernel adds are quicker, 3.22 / 3.48 / 7.21 ms per step at batch 1 / 8 / 64 against
    3.37 / 3.52 / 7.69 ms, because clusters of 8 blocks start later and end with two cluster barriers.)"""
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
    tokens, k = x.shape
    rows = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm_bf16: x {tuple(x.shape)} and w {tuple(w.shape)} do not fit")
    if features is None:
        features = rows
    code = GEMM_MODES[mode]
    pitch = features
    if mode == "partial":
        out = torch.empty((splits, tokens, features), dtype=torch.float32, device=x.device)
    elif mode == "add":
        if out is None or not out.is_cuda or out.dtype != torch.float32 or out.dim() != 2 or out.stride(1) != 1:
            raise KernelError("gemm_bf16: the tensor added to must be a float32 CUDA matrix with dense rows")
        if out.shape[0] != tokens or out.shape[1] != features or not 1 <= splits <= GEMM_CLUSTER_SPLITS:
            raise KernelError("gemm_bf16: the tensor added to must be [tokens, features], the splits at most "
                              f"{GEMM_CLUSTER_SPLITS}")
        pitch = out.stride(0)
    else:
        splits = 1
        out = torch.empty((tokens, features), dtype=torch.float32 if mode == "f32" else torch.bfloat16, device=x.device)
    lib = load_library("gemm_bf16")
    _check(lib, lib.srb_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), tokens, features, k, x.stride(0), w.stride(0), pitch,
                                  rows, int(up_row_offset), code, int(splits), activation_code(activation),
                                  _ptr(error_word), _stream()))
    return out


@traced("gemm")
def gemm_bf16_pair(x: torch.Tensor, w: torch.Tensor, error_word: torch.Tensor, *, mode: str = "bf16",
                   features: Optional[int] = None, up_row_offset: int = 0, activation: str = "silu") -> torch.Tensor:
    """y = x @ w^T for many tokens: 256 x 256 tiles on pairs of CTAs (``tcgen05.mma.cta_group::2``) in a
    persistent kernel.  ``mode`` ``bf16``, ``gated`` or ``act`` as in :func:`gemm_bf16`; the result is bfloat16."""
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
    tokens, k = x.shape
    rows = w.shape[0]
    if w.shape[1] != k or mode not in ("bf16", "gated", "act"):
        raise KernelError(f"gemm_bf16_pair: x {tuple(x.shape)}, w {tuple(w.shape)} or mode {mode!r} do not fit")
    if features is None:
        features = rows
    pitch = -(-features // 8) * 8
    out = torch.empty((tokens, pitch), dtype=torch.bfloat16, device=x.device)
    lib = load_library("gemm_bf16_pair")
    _check(lib, lib.srb_gemm_bf16_pair(_ptr(x), _ptr(w), _ptr(out), tokens, features, k, x.stride(0), w.stride(0), pitch,
                                       rows, int(up_row_offset), GEMM_MODES[mode], activation_code(activation),
                                       _ptr(error_word), _stream()))
    return out if pitch == features else out[:, :features]


def pair_gemm_takes(tokens: int, features: int, k: int) -> bool:
    """True if a bfloat16 gate/up product of this shape goes to the CTA-pair kernel."""
    return tokens >= PAIR_GEMM_MIN_TOKENS and features % 8 == 0 and k % 8 == 0


def gemm_bf16_takes(k: int) -> bool:
    """TMA needs 16-byte rows: the inner size must be a multiple of 8 bfloat16 values."""
    return k % 8 == 0


@traced("gemm")
def activated_product(x: torch.Tensor, weight: torch.Tensor, activation: str,
                      error_word: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x weight^T): the first product of a feed-forward without a gate.  bfloat16 with few rows: the tcgen05
    kernel applies the activation in its epilogue, and with many rows the CTA-pair kernel does; otherwise the product
    followed by the activation kernel."""
    if (x.dtype == torch.bfloat16 and x.shape[0] <= OWN_GEMM_MAX_TOKENS and error_word is not None
            and gemm_bf16_takes(x.shape[1])):
        return gemm_bf16(x, weight, error_word, mode="act", activation=activation)
    if (x.dtype == torch.bfloat16 and error_word is not None and pair_gemm_takes(x.shape[0], weight.shape[0], x.shape[1])):
        return gemm_bf16_pair(x, weight, error_word, mode="act", activation=activation)
    up = linear(x, weight, error_word=error_word)
    activate(up, up, activation)
    return up


@traced("activation")
def activate(x: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(x), element by element (``out`` may be ``x``)."""
    _need(x, "x"); _need(out, "out", x.dtype)
    if out.shape != x.shape:
        raise KernelError("activate: x and out differ in shape")
    lib = load_library("streams")
    _check(lib, lib.srb_activate(_ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), activation_code(activation),
                                 dtype_code(x.dtype), _stream()))


@traced("activation")
def softcap(values: torch.Tensor, cap: float) -> None:
    """values <- cap * tanh(values / cap), in place (float32)."""
    _need(values, "values", torch.float32)
    lib = load_library("streams")
    _check(lib, lib.srb_softcap(_ptr(values), ctypes.c_longlong(values.numel()), ctypes.c_float(cap), _stream()))


# --------------------------------------------------------------------------- copies of the residual stream

@traced("embedding")
def embedding_pairs(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor, *,
                    scale: float = 1.0, copies: int = 1, pairs: Optional[torch.Tensor] = None, buckets: int = 0,
                    mul_prev: int = 0, mul_cur: int = 0, positions: Optional[torch.Tensor] = None,
                    row_request: Optional[torch.Tensor] = None, cu_rows: Optional[torch.Tensor] = None,
                    state_slots: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None) -> None:
    """out[r, c, :] = table[ids[r]] * scale + pairs[row(r)] for every copy c; float32 [rows, copies, width].

    ``pairs`` [buckets + 1, width]: row(r) = (previous token * mul_prev + ids[r] * mul_cur) mod buckets, and row
    ``buckets`` where ``positions[r]`` is 0.  The previous token of a request's first row in this step is
    ``last_token[state_slots[request]]``; :func:`remember_tokens` stores it after the step's embedding."""
    _need(ids, "ids", torch.int32); _need(table, "table"); _need(out, "out", torch.float32)
    rows, width = ids.numel(), table.shape[1]
    if out.numel() != rows * copies * width:
        raise KernelError("embedding_pairs: out must hold rows * copies * width floats")
    if pairs is not None:
        _need(pairs, "pairs", table.dtype)
        if pairs.shape != (buckets + 1, width):
            raise KernelError("embedding_pairs: the pair table must be [buckets + 1, width]")
        for name, tensor in (("positions", positions), ("row_request", row_request), ("cu_rows", cu_rows),
                             ("state_slots", state_slots), ("last_token", last_token)):
            if tensor is None:
                raise KernelError(f"embedding_pairs: {name} is needed with a pair table")
            _need(tensor, name, torch.int32)
    lib = load_library("streams")
    _check(lib, lib.srb_embedding_pairs(
        _ptr(ids), _ptr(positions), _ptr(row_request), _ptr(cu_rows), _ptr(state_slots), _ptr(last_token), _ptr(table),
        _ptr(pairs), _ptr(out), rows, width, table.shape[0], int(copies), ctypes.c_longlong(buckets),
        ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur), ctypes.c_float(scale), _ptr(error_word),
        dtype_code(table.dtype), _stream()))


@traced("embedding")
def remember_tokens(ids: torch.Tensor, cu_rows: torch.Tensor, state_slots: torch.Tensor, last_token: torch.Tensor,
                    requests: int) -> None:
    """last_token[state_slots[q]] = the last id that request q brought in this step."""
    _need(ids, "ids", torch.int32); _need(cu_rows, "cu_rows", torch.int32); _need(state_slots, "state_slots", torch.int32)
    _need(last_token, "last_token", torch.int32)
    lib = load_library("streams")
    _check(lib, lib.srb_remember_tokens(_ptr(ids), _ptr(cu_rows), _ptr(state_slots), _ptr(last_token), int(requests),
                                        _stream()))


@traced("norm")
def stream_step(x: torch.Tensor, y: Optional[torch.Tensor], mix: Optional[torch.Tensor], spread: Optional[torch.Tensor],
                gather: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor],
                row_index: Optional[torch.Tensor] = None, norm: bool = True) -> None:
    """One pass over the copies of the residual stream ``x`` (float32 [rows, streams, width]).

    With ``mix`` ([streams, streams], indexed [from, to]) and ``spread`` ([streams]): every copy is replaced, all at
    once from the old ones, x_t <- sum_s mix[s, t] x_s + spread[t] * y, where ``y`` is the result of the sublayer
    before ([rows, width] of ``out``'s dtype or float32, or float32 [parts, rows, width] partial sums added in order).
    With ``gather`` ([streams]): u = sum_t gather[t] x_t and ``out`` = u / sqrt(mean(u^2) + eps) * weight (``norm``
    False: u * weight; ``weight`` None: no scaling).  With ``row_index`` only those rows are read, ``out[i]`` is
    written, and the copies in memory stay as they are."""
    _need(x, "x", torch.float32)
    if x.dim() != 3:
        raise KernelError("stream_step: x must be [rows, streams, width]")
    total_rows, streams, width = x.shape
    rows = total_rows if row_index is None else row_index.numel()
    whole = parts = None
    num_parts = part_stride = 0
    if mix is not None:
        _need(mix, "mix", torch.float32); _need(spread, "spread", torch.float32)
        if mix.numel() != streams * streams or spread.numel() != streams or y is None:
            raise KernelError("stream_step: the update needs [streams, streams] weights, [streams] weights and a result")
        _need(y, "y")
        if y.dim() == 3 or y.dtype == torch.float32 and (out is None or out.dtype != torch.float32):
            _need(y, "y", torch.float32)
            parts = y if y.dim() == 3 else y.unsqueeze(0)
            if parts.shape[1:] != (total_rows, width):
                raise KernelError("stream_step: the partial sums must be [parts, rows, width]")
            num_parts, part_stride = parts.shape[0], parts.stride(0)
        else:
            if y.shape != (total_rows, width):
                raise KernelError("stream_step: the result must be [rows, width]")
            whole = y
    dtype = x.dtype
    pitch = 0
    if gather is not None:
        _need(gather, "gather", torch.float32)
        if out is None or out.dim() != 2 or out.shape != (rows, width) or out.stride(1) != 1 or not out.is_cuda:
            raise KernelError("stream_step: out must be a CUDA matrix [rows, width] with dense rows")
        dtype, pitch = out.dtype, out.stride(0)
        if weight is not None:
            _need(weight, "weight", torch.float32)
    if whole is not None:
        if gather is not None and whole.dtype != dtype:
            raise KernelError("stream_step: the result must be float32 or of out's dtype")
        dtype = whole.dtype
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
    lib = load_library("streams")
    _check(lib, lib.srb_stream_step(
        _ptr(x), _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(part_stride), _ptr(mix), _ptr(spread), _ptr(gather),
        _ptr(weight), ctypes.c_float(eps), int(norm), _ptr(out), ctypes.c_longlong(pitch), _ptr(row_index), rows, streams,
        width, 1, dtype_code(dtype), _stream()))


# --------------------------------------------------------------------------- linear attention over a state

@traced("lightning")
def lightning_scan(proj: torch.Tensor, q_offset: int, k_offset: int, v_offset: int, cu_rows: torch.Tensor,
                   positions: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, decay: torch.Tensor,
                   out: torch.Tensor, requests: int, read_only: bool = False, single_rows: bool = False) -> None:
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v the SiLU of the row's projections.
    ``single_rows``: every request of the step brings exactly one row (decoded tokens); a kernel that makes one pass
    over the states then takes the step.

    ``proj`` [rows, *]: q heads (dim entries each) from column ``q_offset``, k heads from ``k_offset``, v heads
    (vdim each) from ``v_offset``; ``state`` float32 [slots, heads, dim, vdim], updated in place for the slots
    ``state_slots[request]`` (a request whose first row is at position 0 starts from zero); ``out`` float32
    [rows, heads * vdim].  The rows of request r are ``cu_rows[r] .. cu_rows[r + 1]``."""
    _need(positions, "positions", torch.int32); _need(cu_rows, "cu_rows", torch.int32)
    _need(state_slots, "state_slots", torch.int32); _need(state, "state", torch.float32); _need(decay, "decay", torch.float32)
    _need(out, "out", torch.float32)
    if proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("lightning_scan: proj must be a CUDA matrix with dense rows")
    _, heads, dim, vdim = state.shape
    if decay.numel() != heads or out.shape != (proj.shape[0], heads * vdim):
        raise KernelError("lightning_scan: shapes of the state, the decays and out do not agree")
    if max(q_offset, k_offset) + heads * dim > proj.shape[1] or v_offset + heads * vdim > proj.shape[1]:
        raise KernelError("lightning_scan: rows of proj are too short")
    lib = load_library("lightning")
    entry = lib.srb_lightning_scan_single if single_rows else lib.srb_lightning_scan
    _check(lib, entry(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), q_offset, k_offset, v_offset, _ptr(cu_rows), _ptr(positions),
        _ptr(state_slots), _ptr(state), _ptr(decay), _ptr(out), int(requests), heads, dim, vdim, int(read_only),
        dtype_code(proj.dtype), _stream()))


def lightning_chunks_takes(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """True if the tensor-core kernels for prompt portions take these sizes (the rule of srb_lightning_chunks_supports)."""
    return dtype == torch.bfloat16 and dim in (64, 128) and vdim in (64, 128)


#: tokens per chunk of :func:`lightning_chunks` (LC_TOKENS of csrc/lightning.cu)
LIGHTNING_CHUNK_TOKENS = 128


@traced("lightning")
def lightning_chunks(proj: torch.Tensor, q_offset: int, k_offset: int, v_offset: int, cu_rows: torch.Tensor,
                     positions: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, decay: torch.Tensor,
                     out: torch.Tensor, requests: int, chunks: int, read_only: bool = False) -> None:
    """What :func:`lightning_scan` computes, for prompt portions in bfloat16: the rows of every request are cut into
    chunks of ``LIGHTNING_CHUNK_TOKENS`` tokens that run in parallel on the tensor cores (each chunk's own contribution
    to the state, then the states before every chunk in order, then the results).  ``chunks``: the number of chunks of
    the step, sum over the requests of ceil(rows / LIGHTNING_CHUNK_TOKENS), or more.  The q, k and v columns of ``proj``
    are replaced by their SiLU on the way; rows and the three column offsets must lie on 16-byte borders."""
    _need(proj, "proj", torch.bfloat16); _need(positions, "positions", torch.int32); _need(cu_rows, "cu_rows", torch.int32)
    _need(state_slots, "state_slots", torch.int32); _need(state, "state", torch.float32); _need(decay, "decay", torch.float32)
    _need(out, "out", torch.float32)
    _, heads, dim, vdim = state.shape
    if proj.dim() != 2 or decay.numel() != heads or out.shape != (proj.shape[0], heads * vdim):
        raise KernelError("lightning_chunks: shapes of proj, the state, the decays and out do not agree")
    if max(q_offset, k_offset) + heads * dim > proj.shape[1] or v_offset + heads * vdim > proj.shape[1]:
        raise KernelError("lightning_chunks: rows of proj are too short")
    scratch = torch.empty((max(int(chunks), 1), heads, dim, vdim), dtype=torch.float32, device=proj.device)
    lib = load_library("lightning")
    _check(lib, lib.srb_lightning_chunks(
        _ptr(proj), proj.shape[0], ctypes.c_longlong(proj.stride(0)), q_offset, k_offset, v_offset, _ptr(cu_rows), _ptr(positions),
        _ptr(state_slots), _ptr(state), _ptr(decay), _ptr(scratch), _ptr(out), int(requests), int(chunks), heads, dim, vdim,
        int(read_only), _stream()), launches=4)


@traced("lightning")
def lightning_gate_norm(o: torch.Tensor, proj: torch.Tensor, g_offset: int, weight: torch.Tensor, eps: float,
                        out: torch.Tensor) -> None:
    """out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g): the heads' results of a row normed together; the gate's
    logits are the columns ``g_offset`` .. of ``proj``."""
    _need(o, "o", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out", proj.dtype)
    rows, width = o.shape
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[0] != rows or g_offset + width > proj.shape[1]:
        raise KernelError("lightning_gate_norm: proj does not hold the gate's logits")
    if out.shape != o.shape or weight.numel() != width:
        raise KernelError("lightning_gate_norm: shapes do not agree")
    lib = load_library("lightning")
    _check(lib, lib.srb_lightning_gate_norm(_ptr(o), _ptr(proj), ctypes.c_longlong(proj.stride(0)), g_offset, _ptr(weight),
                                            ctypes.c_float(eps), rows, width, _ptr(out), dtype_code(proj.dtype), _stream()))


# --------------------------------------------------------------------------- sampling

# --------------------------------------------------------------------------- a state-space mixer over a state per request

def mamba_slot_floats(heads: int, vdim: int, nstate: int, groups: int, taps: int) -> int:
    """Floats of state per request: the convolution's last ``taps`` - 1 inputs [taps - 1, channels], then S [heads, vdim, nstate]."""
    return (taps - 1) * (heads * vdim + 2 * groups * nstate) + heads * nstate * vdim


def _mamba_args(proj, state, heads, vdim, nstate, groups, taps):
    if proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("mamba: the in-projection must be a CUDA matrix with dense rows")
    _need(state, "state", torch.float32)
    if state.dim() != 2 or state.shape[1] != mamba_slot_floats(heads, vdim, nstate, groups, taps):
        raise KernelError("mamba: the state must be float32 [slots, floats per slot]")
    if proj.shape[1] < 2 * heads * vdim + 2 * groups * nstate + heads:
        raise KernelError("mamba: rows of the in-projection are too short")


@traced("mamba_conv")
def mamba_conv(proj: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, positions: torch.Tensor, row_request: torch.Tensor,
               cu_rows: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, out: torch.Tensor, num_requests: int, *,
               heads: int, vdim: int, nstate: int, groups: int, taps: int, read_only: bool = False) -> None:
    """The causal convolution per channel and SiLU of the x, B and C entries of ``proj``'s rows
    ([z | x | B | C | dt]); ``out`` [rows, channels], float32 or (beside a bfloat16 ``proj``, for :func:`mamba_chunks`)
    bfloat16.  Inputs before a request's first row of the step come from
    its slot of ``state`` (zeros before position 0); unless ``read_only`` the slot then keeps the sequence's last
    ``taps`` - 1 inputs.  ``weight`` float32 [channels, taps] (the last column is the current token's), ``bias`` [channels]."""
    _mamba_args(proj, state, heads, vdim, nstate, groups, taps)
    channels = heads * vdim + 2 * groups * nstate
    _need(weight, "weight", torch.float32); _need(bias, "bias", torch.float32)
    _need(out, "out", torch.float32 if out.dtype != proj.dtype else proj.dtype)
    for name, t in (("positions", positions), ("row_request", row_request), ("cu_rows", cu_rows), ("state_slots", state_slots)):
        _need(t, name, torch.int32)
    rows = proj.shape[0]
    if weight.shape != (channels, taps) or bias.numel() != channels or out.shape != (rows, channels):
        raise KernelError("mamba_conv: shapes of the filter, its bias and the output do not agree")
    lib = load_library("mamba")
    _check(lib, lib.srb_mamba_conv(_ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(weight), _ptr(bias), _ptr(positions),
                                   _ptr(row_request), _ptr(cu_rows), _ptr(state_slots), _ptr(state),
                                   ctypes.c_longlong(state.stride(0)), _ptr(out), rows, int(num_requests), heads, vdim, nstate,
                                   groups, taps, int(not read_only), dtype_code(proj.dtype), dtype_code(out.dtype), _stream()),
           launches=1 if read_only or taps == 1 else 2)


@traced("mamba_scan")
def mamba_scan(proj: torch.Tensor, xbc: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor, dt_bias: torch.Tensor,
               positions: torch.Tensor, cu_rows: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, y: torch.Tensor,
               num_requests: int, *, heads: int, vdim: int, nstate: int, groups: int, taps: int, read_only: bool = False) -> None:
    """The recurrence per head, token by token from each request's state: dt = softplus(dt + dt_bias), S <- exp(-exp(A_log) dt) S
    + dt B x^T, y = S^T C + D x, all in 32-bit.  ``xbc``: what :func:`mamba_conv` wrote; ``y`` float32 [rows, heads * vdim]."""
    _mamba_args(proj, state, heads, vdim, nstate, groups, taps)
    rows, inner = proj.shape[0], heads * vdim
    _need(xbc, "xbc", torch.float32); _need(y, "y", torch.float32)
    for name, t in (("a_log", a_log), ("d_skip", d_skip), ("dt_bias", dt_bias)):
        _need(t, name, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"mamba_scan: {name} needs one entry per head")
    for name, t in (("positions", positions), ("cu_rows", cu_rows), ("state_slots", state_slots)):
        _need(t, name, torch.int32)
    if xbc.shape != (rows, inner + 2 * groups * nstate) or y.shape != (rows, inner):
        raise KernelError("mamba_scan: shapes of the convolved inputs and the output do not agree")
    lib = load_library("mamba")
    _check(lib, lib.srb_mamba_scan(_ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(xbc), _ptr(a_log), _ptr(d_skip),
                                   _ptr(dt_bias), _ptr(positions), _ptr(cu_rows), _ptr(state_slots), _ptr(state),
                                   ctypes.c_longlong(state.stride(0)), _ptr(y), rows, int(num_requests), heads, vdim, nstate, groups,
                                   taps, int(not read_only), dtype_code(proj.dtype), _stream()))


def mamba_chunks_takes(dtype: torch.dtype, vdim: int, nstate: int) -> bool:
    """True if the tensor-core kernels for prompt portions take these sizes (the rule of srb_mamba_chunks_supports)."""
    return dtype == torch.bfloat16 and vdim in (64, 128) and nstate in (64, 128)


#: tokens per chunk of :func:`mamba_chunks` (LC_TOKENS of csrc/chunk_helpers.cuh)
MAMBA_CHUNK_TOKENS = 128


@traced("mamba_scan")
def mamba_chunks(proj: torch.Tensor, xbc: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor, dt_bias: torch.Tensor,
                 positions: torch.Tensor, cu_rows: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, y: torch.Tensor,
                 num_requests: int, chunks: int, *, heads: int, vdim: int, nstate: int, groups: int, taps: int,
                 read_only: bool = False) -> None:
    """What :func:`mamba_scan` computes, for prompt portions in bfloat16: the rows of every request are cut into chunks
    of ``MAMBA_CHUNK_TOKENS`` tokens that run in parallel on the tensor cores (each chunk's own contribution to the
    state, then the states before every chunk in order, then the results).  ``xbc``: bfloat16, what :func:`mamba_conv`
    wrote; ``chunks``: the number of chunks of the step, sum over the requests of ceil(rows / MAMBA_CHUNK_TOKENS), or more."""
    _mamba_args(proj, state, heads, vdim, nstate, groups, taps)
    rows, inner = proj.shape[0], heads * vdim
    _need(proj, "proj", torch.bfloat16); _need(xbc, "xbc", torch.bfloat16); _need(y, "y", torch.float32)
    for name, t in (("a_log", a_log), ("d_skip", d_skip), ("dt_bias", dt_bias)):
        _need(t, name, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"mamba_chunks: {name} needs one entry per head")
    for name, t in (("positions", positions), ("cu_rows", cu_rows), ("state_slots", state_slots)):
        _need(t, name, torch.int32)
    if xbc.shape != (rows, inner + 2 * groups * nstate) or not xbc.is_contiguous() or y.shape != (rows, inner):
        raise KernelError("mamba_chunks: shapes of the convolved inputs and the output do not agree")
    if not mamba_chunks_takes(proj.dtype, vdim, nstate):
        raise KernelError(f"mamba_chunks: a state of {nstate} x {vdim} per head is not taken")
    chunks = max(int(chunks), 1)
    scratch = torch.empty((chunks * heads * (nstate * vdim + 1),), dtype=torch.float32, device=proj.device)
    lib = load_library("mamba")
    _check(lib, lib.srb_mamba_chunks(_ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(xbc), _ptr(a_log), _ptr(d_skip),
                                     _ptr(dt_bias), _ptr(positions), _ptr(cu_rows), _ptr(state_slots), _ptr(state),
                                     ctypes.c_longlong(state.stride(0)), _ptr(scratch), _ptr(y), rows, int(num_requests), chunks,
                                     heads, vdim, nstate, groups, taps, int(not read_only), _stream()), launches=3)


@traced("mamba_gate_norm")
def mamba_gate_norm(y: torch.Tensor, proj: torch.Tensor, weight: torch.Tensor, eps: float, norm_groups: int,
                    out: torch.Tensor) -> None:
    """out = rms_in_parts(y * silu(z)) * weight with z the first entries of ``proj``'s rows and the RMS norm taken in
    ``norm_groups`` equal consecutive parts; y float32 [rows, inner], out [rows, inner] of proj's dtype."""
    _need(y, "y", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out", proj.dtype)
    rows, inner = y.shape
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[0] != rows or proj.shape[1] < inner or weight.numel() != inner \
            or out.shape != (rows, inner):
        raise KernelError("mamba_gate_norm: shapes do not agree")
    lib = load_library("mamba")
    _check(lib, lib.srb_mamba_gate_norm(_ptr(y), _ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(weight), ctypes.c_float(eps),
                                        rows, inner, int(norm_groups), _ptr(out), dtype_code(proj.dtype), _stream()))


# --------------------------------------------------------------------------- sublayers side by side, a token's own input

@traced("residual")
def scaled_sum(residual: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], mult: float,
               rounded: Optional[torch.Tensor] = None) -> None:
    """residual += mult * (a + b) in 32-bit, in place.  ``a``: [rows, width] of the compute dtype or float32, or float32
    [parts, rows, width] (partial sums, added in order), or None; ``b``: float32 [rows, width] or None.  ``rounded``
    ([rows, width]) receives the new residual rounded to its dtype."""
    _need(residual, "residual", torch.float32)
    rows, width = residual.shape
    whole = parts = None
    num_parts = stride = 0
    dtype = rounded.dtype if rounded is not None else (a.dtype if a is not None else torch.float32)
    if a is not None:
        _need(a, "a")
        if a.dtype == torch.float32:
            parts = a if a.dim() == 3 else a.unsqueeze(0)
            if parts.shape[1:] != residual.shape:
                raise KernelError("scaled_sum: a and the residual differ in shape")
            num_parts, stride = parts.shape[0], parts.stride(0)
        else:
            if a.shape != residual.shape or a.dtype != dtype:
                raise KernelError("scaled_sum: a must be shaped like the residual, of the rounded copy's dtype")
            whole = a
    if b is not None:
        _need(b, "b", torch.float32)
        if b.shape != residual.shape:
            raise KernelError("scaled_sum: b and the residual differ in shape")
    if rounded is not None:
        _need(rounded, "rounded")
        if rounded.shape != residual.shape:
            raise KernelError("scaled_sum: the rounded copy and the residual differ in shape")
    lib = load_library("elementwise")
    _check(lib, lib.srb_scaled_sum(_ptr(residual), _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(stride), _ptr(b),
                                   ctypes.c_float(mult), _ptr(rounded), rows, width, dtype_code(dtype), _stream()))


@traced("activation")
def token_gate(gate: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, offset: int, out: torch.Tensor, error_word: torch.Tensor,
               activation: str = "gelu_tanh") -> None:
    """out[r, j] = act(gate[r, j]) * table[ids[r], offset + j]: a gate multiplied by a slice of the row that the token
    chooses in ``table`` [vocab, >= offset + dim]."""
    _need(gate, "gate"); _need(out, "out", gate.dtype); _need(table, "table", gate.dtype); _need(ids, "ids", torch.int32)
    rows, dim = gate.shape
    if out.shape != gate.shape or ids.numel() != rows or table.dim() != 2 or offset < 0 or offset + dim > table.shape[1]:
        raise KernelError("token_gate: shapes do not agree")
    lib = load_library("elementwise")
    _check(lib, lib.srb_token_gate(_ptr(gate), _ptr(ids), _ptr(table), ctypes.c_longlong(table.stride(0)), int(offset),
                                   table.shape[0], rows, dim, activation_code(activation), _ptr(out), _ptr(error_word),
                                   dtype_code(gate.dtype), _stream()))


@traced("logits")
def scale_values(values: torch.Tensor, factor: float) -> None:
    """values *= factor, float32, in place."""
    _need(values, "values", torch.float32)
    lib = load_library("elementwise")
    _check(lib, lib.srb_scale_values(_ptr(values), ctypes.c_longlong(values.numel()), ctypes.c_float(factor), _stream()))


@traced("sampling")
def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of 32-bit logits: argmax where temperature is None or <= 0, else
    inverse-CDF sampling of softmax(logits / temperature) with the row's uniform number."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32)
    if temperature is not None:
        _need(temperature, "temperature", torch.float32); _need(uniform, "uniform", torch.float32)
    lib = load_library("sampling")
    scratch = torch.empty(lib.srb_sample_scratch_floats(rows), dtype=torch.float32, device=logits.device)
    _check(lib, lib.srb_sample(_ptr(logits), rows, vocab, logits.stride(0), _ptr(temperature), _ptr(uniform),
                               _ptr(out), _ptr(scratch), _stream()), launches=2)
    return out


@traced("sampling")
def sample_filtered(logits: torch.Tensor, rows_index: Optional[torch.Tensor], temperature: torch.Tensor,
                    top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor,
                    out: torch.Tensor) -> None:
    """Sampling with top-k, top-p and min-p for the rows named in ``rows_index`` (int32; None: all rows),
    into ``out[row]``.  The option tensors hold one entry per row of ``logits``: temperature > 0, top_k
    (int32; <= 0: off), top_p (>= 1: off), min_p (<= 0: off), uniform in [0, 1)."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32); _need(min_p, "min_p", torch.float32); _need(uniform, "uniform", torch.float32)
    rows, vocab = logits.shape
    for name, tensor in (("temperature", temperature), ("top_k", top_k), ("top_p", top_p), ("min_p", min_p),
                         ("uniform", uniform), ("out", out)):
        if tensor.numel() < rows:
            raise KernelError(f"sample_filtered: {name} needs one entry per row")
    count = rows
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32)
        count = rows_index.numel()
    if count == 0:
        return
    lib = load_library("sampling")
    # the rows' probabilities, each row padded to a multiple of four
    scratch = torch.empty(count * ((vocab + 3) & ~3), dtype=torch.float32, device=logits.device)
    _check(lib, lib.srb_sample_filtered(_ptr(logits), vocab, ctypes.c_longlong(logits.stride(0)), _ptr(rows_index), count,
                                        _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform),
                                        _ptr(scratch), _ptr(out), _stream()))


@traced("sampling")
def count_tokens(counts_row: torch.Tensor, tokens: torch.Tensor) -> None:
    """``counts_row[t] += 1`` for every token id in ``tokens`` (int32, on the device)."""
    _need(counts_row, "counts_row", torch.int32); _need(tokens, "tokens", torch.int32)
    lib = load_library("sampling")
    _check(lib, lib.srb_count_tokens(_ptr(counts_row), _ptr(tokens), tokens.numel(), counts_row.numel(), _stream()))


@traced("sampling")
def apply_penalties(logits: torch.Tensor, counts: torch.Tensor, index: torch.Tensor, presence: torch.Tensor,
                    frequency: torch.Tensor, repetition: torch.Tensor) -> None:
    """Penalises ``logits`` in place: row r uses the counts of ``counts[index[r]]`` (``index[r] < 0``: none).
    A token seen c > 0 times: divided by ``repetition[r]`` if positive, multiplied if negative, then
    lowered by ``presence[r] + frequency[r] * c``."""
    _need(logits, "logits", torch.float32); _need(counts, "counts", torch.int32); _need(index, "index", torch.int32)
    _need(presence, "presence", torch.float32); _need(frequency, "frequency", torch.float32)
    _need(repetition, "repetition", torch.float32)
    rows, vocab = logits.shape
    if counts.dim() != 2 or counts.shape[1] != vocab:
        raise KernelError("apply_penalties: counts must be [table rows, vocab]")
    lib = load_library("sampling")
    _check(lib, lib.srb_apply_penalties(_ptr(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _ptr(counts),
                                        _ptr(index), _ptr(presence), _ptr(frequency), _ptr(repetition), _stream()))


@traced("sampling")
def count_picked(counts: torch.Tensor, index: torch.Tensor, picked: torch.Tensor) -> None:
    """``counts[index[r], picked[r]] += 1`` for every row with ``index[r] >= 0``."""
    _need(counts, "counts", torch.int32); _need(index, "index", torch.int32); _need(picked, "picked", torch.int32)
    lib = load_library("sampling")
    _check(lib, lib.srb_count_picked(_ptr(counts), counts.shape[1], _ptr(index), _ptr(picked), picked.numel(), _stream()))
