"""Validated configuration of a ``Titatar`` checkpoint.

The document is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (one entry per layer: ``type``
``attention`` or ``latent_attention``, the mixer's sizes under ``mixer``, the feed-forward under ``mlp`` or null) and
``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1 are walked ``times`` times in a row).  A mixer's rotation
is ``rot`` (``base``, ``dims`` and, optionally, ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``); the window
of the ``attention`` mixer is ``mask.size``.  A feed-forward is ``kind`` ``dense`` (``ff``) or ``moe`` (``expert.ff``,
``router.experts``, ``router.top``, ``router.identity``, ``shared.ff``).  Every size and every constant that can differ
between checkpoints is read here, layer by layer; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

from ..config.model_config import ConfigError, RawConfig, missing_field, required_positive_int

ARCHITECTURE = "Titatar"
ATTENTION_TYPE, LATENT_TYPE = "attention", "latent_attention"
#: positions a request may reach when the document gives no limit (every position is exact in 32-bit floats)
DEFAULT_MAX_POSITIONS = 1 << 24


def _section(document: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = document.get(key)
    if not isinstance(value, dict):
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be an object")
    return value


def _number(document: Mapping[str, Any], key: str, where: str) -> float:
    value = document.get(key)
    if value is None:
        raise missing_field(ARCHITECTURE, where + key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be a number, found {value!r}")
    return float(value)


def _count(document: Mapping[str, Any], key: str, where: str, least: int = 1, default: Optional[int] = None) -> int:
    value = document.get(key)
    if value is None:
        if default is not None:
            return default
        raise missing_field(ARCHITECTURE, where + key)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be an integer of at least {least}, found {value!r}")
    return value


@dataclass(frozen=True)
class RotationSpec:
    base: float
    dims: int                                   # leading entries of the rotated vector that turn; the rest pass
    #: (factor, original, fast, slow) of the stretching of long wavelengths, or None
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class WindowedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot: Optional[RotationSpec]


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int                 # unrotated query/key entries per head
    rot_dim: int             # rotated query/key entries per head (the key's are shared by all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[RotationSpec]


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class RoutedSizes:
    experts: int             # experts with tensors
    identity: int            # router outputs behind them that stand for experts returning their input
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class LayerSpec:
    kind: str
    mixer: Union[WindowedAttentionSizes, LatentAttentionSizes]
    mlp: Union[DenseSizes, RoutedSizes, None]


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TitatarConfig:
    ARCHITECTURE = ARCHITECTURE

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    loop: Optional[LoopSpec]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Sequence[int] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "TitatarConfig":
        doc = raw.document
        vocab = required_positive_int(ARCHITECTURE, doc, "vocab")
        width = required_positive_int(ARCHITECTURE, doc, "width")
        scale = _number(_section(doc, "embedding", ""), "scale", "embedding.")
        eps = _number(_section(doc, "norm", ""), "eps", "norm.")
        if not eps >= 0:
            raise ConfigError(ARCHITECTURE, "`norm.eps` must be non-negative")
        entries = doc.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(ARCHITECTURE, "`layers` must be a list with at least one layer")
        layers = tuple(_layer(entry, f"layers[{i}].") for i, entry in enumerate(entries))
        loop = None
        if doc.get("loop") is not None:
            section = _section(doc, "loop", "")
            loop = LoopSpec(_count(section, "start", "loop.", 0), _count(section, "stop", "loop.", 0),
                            _count(section, "times", "loop."))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(ARCHITECTURE, f"`loop` must name a stretch of the {len(layers)} layers, "
                                                f"found {loop.start} .. {loop.stop}")
        limit = doc.get("max_position_embeddings")
        if limit is not None:
            limit = required_positive_int(ARCHITECTURE, doc, "max_position_embeddings")
        return cls(vocab, width, scale, eps, layers, loop, limit or DEFAULT_MAX_POSITIONS, tuple(raw.eos_token_ids), doc)


def _rotation(mixer: Mapping[str, Any], where: str, most: int) -> Optional[RotationSpec]:
    """``rot`` of a mixer; None if the document has none or it turns no entries."""
    if mixer.get("rot") is None:
        return None
    rot = _section(mixer, "rot", where)
    inside = where + "rot."
    dims = _count(rot, "dims", inside, 0)
    if dims == 0:
        return None
    base = _number(rot, "base", inside)
    if dims % 2 or dims > most or not base > 0:
        raise ConfigError(ARCHITECTURE, f"`{inside[:-1]}` must rotate an even number of at most {most} entries with a positive base")
    scaling = None
    if rot.get("scaling") is not None:
        s = _section(rot, "scaling", inside)
        scaling = tuple(_number(s, key, inside + "scaling.") for key in ("factor", "original", "fast", "slow"))
        if not all(value > 0 for value in scaling) or not base > 1:
            raise ConfigError(ARCHITECTURE, f"`{inside}scaling` needs positive numbers and a base above 1")
    return RotationSpec(base, dims, scaling)


def _layer(entry: Any, where: str) -> LayerSpec:
    if not isinstance(entry, dict):
        raise ConfigError(ARCHITECTURE, f"`{where[:-1]}` must be an object")
    kind = entry.get("type")
    m = _section(entry, "mixer", where)
    inside = where + "mixer."
    if kind == ATTENTION_TYPE:
        heads, kv_heads = _count(m, "heads", inside), _count(m, "kv_heads", inside)
        if heads % kv_heads:
            raise ConfigError(ARCHITECTURE, f"`{inside}heads` {heads} is not a multiple of `kv_heads` {kv_heads}")
        dim = _count(m, "dim", inside)
        window = None
        if m.get("mask") is not None:
            window = _count(_section(m, "mask", inside), "size", inside + "mask.")
        mixer = WindowedAttentionSizes(heads, kv_heads, dim, _count(m, "vdim", inside), _number(m, "scale", inside), window,
                                       _rotation(m, inside, dim))
    elif kind == LATENT_TYPE:
        rot_dim = _count(m, "rot_dim", inside, 0)
        mixer = LatentAttentionSizes(
            heads=_count(m, "heads", inside), dim=_count(m, "dim", inside), rot_dim=rot_dim, vdim=_count(m, "vdim", inside),
            q_rank=_count(m, "q_rank", inside), kv_rank=_count(m, "kv_rank", inside), scale=_number(m, "scale", inside),
            rot=_rotation(m, inside, rot_dim) if rot_dim else None)
    else:
        raise ConfigError(ARCHITECTURE, f"`{where}type` {kind!r} is not a mixer of this design ({ATTENTION_TYPE}, {LATENT_TYPE})")
    mlp = None
    if entry.get("mlp") is not None:
        f = _section(entry, "mlp", where)
        inside = where + "mlp."
        if f.get("kind") == "dense":
            mlp = DenseSizes(_count(f, "ff", inside))
        elif f.get("kind") == "moe":
            router = _section(f, "router", inside)
            shared = None
            if f.get("shared") is not None:
                shared = _count(_section(f, "shared", inside), "ff", inside + "shared.")
            mlp = RoutedSizes(_count(router, "experts", inside + "router."),
                              _count(router, "identity", inside + "router.", 0, default=0),
                              _count(router, "top", inside + "router."),
                              _count(_section(f, "expert", inside), "ff", inside + "expert."), shared)
            if mlp.top > mlp.experts + mlp.identity:
                raise ConfigError(ARCHITECTURE, f"`{inside}router.top` exceeds the number of router outputs")
        else:
            raise ConfigError(ARCHITECTURE, f"`{inside}kind` {f.get('kind')!r} is not a feed-forward of this design (dense, moe)")
    return LayerSpec(kind, mixer, mlp)
