"""Validated configuration of a ``Desarax`` checkpoint.

The document is nested: ``vocab``, ``width``, ``residual_mult`` (the factor on every term that joins the residual
stream), ``logit_scale``, ``norm`` (``eps``, ``groups``: the model's RMS norm is taken in that many equal parts of the
row), ``token_side`` (``dim``: per layer a slice of that many entries of a second table indexed by the token; absent or
null: no such input) and ``layers``: one entry per layer with ``type`` (``mamba2`` or ``mamba2_2``: the state-space
mixer; ``latent_attention``), the mixer's sizes under ``mixer`` and the feed-forward under ``mlp`` (``kind`` ``moe``;
null: none).  An attention layer may name, as ``kv_from``, an earlier attention layer whose cached latents it reads.
Every size and every constant that can differ between checkpoints is read here, per layer; nothing is assumed equal
between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

from ..config.model_config import ConfigError, RawConfig, missing_field, required_positive_int

ARCHITECTURE = "Desarax"
#: positions a request may reach when the document gives no limit (every position is exact in 32-bit floats)
DEFAULT_MAX_POSITIONS = 1 << 24
STATE_SPACE_TYPES = ("mamba2", "mamba2_2")
ATTENTION_TYPE = "latent_attention"


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


def _count(document: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    value = document.get(key)
    if value is None:
        raise missing_field(ARCHITECTURE, where + key)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be an integer of at least {least}, found {value!r}")
    return value


@dataclass(frozen=True)
class StateSpaceSizes:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int               # tokens the causal convolution spans
    norm_groups: int


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]    # a row sees itself and window - 1 rows before it; None: every earlier row
    kv_from: Optional[int]   # the layer whose cached latents this layer reads; None: its own


@dataclass(frozen=True)
class RoutedSizes:
    experts: int
    top: int
    ff: int
    limit: float
    scale: float


@dataclass(frozen=True)
class LayerSpec:
    kind: str
    mixer: Union[StateSpaceSizes, LatentAttentionSizes]
    mlp: Optional[RoutedSizes]


@dataclass(frozen=True)
class DesaraxConfig:
    ARCHITECTURE = ARCHITECTURE

    vocab: int
    width: int
    residual_mult: float
    logit_scale: float
    norm_eps: float
    norm_groups: int
    side_dim: Optional[int]
    layers: Tuple[LayerSpec, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Sequence[int] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "DesaraxConfig":
        doc = raw.document
        vocab = required_positive_int(ARCHITECTURE, doc, "vocab")
        width = required_positive_int(ARCHITECTURE, doc, "width")
        norm = _section(doc, "norm", "")
        eps, groups = _number(norm, "eps", "norm."), _count(norm, "groups", "norm.") if norm.get("groups") is not None else 1
        if not eps >= 0:
            raise ConfigError(ARCHITECTURE, "`norm.eps` must be non-negative")
        if width % groups:
            raise ConfigError(ARCHITECTURE, f"`norm.groups` {groups} does not divide the width {width}")
        side_dim = None
        if doc.get("token_side") is not None:
            side_dim = _count(_section(doc, "token_side", ""), "dim", "token_side.")
        entries = doc.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(ARCHITECTURE, "`layers` must be a list with at least one layer")
        layers = tuple(_layer(entry, f"layers[{i}].") for i, entry in enumerate(entries))
        for i, layer in enumerate(layers):
            source = getattr(layer.mixer, "kv_from", None)
            if source is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if not 0 <= source < i or layers[source].kind != ATTENTION_TYPE:
                raise ConfigError(ARCHITECTURE, f"`{where}` must name an earlier {ATTENTION_TYPE} layer, found {source}")
            if layers[source].mixer.kv_from is not None:
                raise ConfigError(ARCHITECTURE, f"`{where}` names layer {source}, which keeps no latents of its own")
            if layers[source].mixer.kv_rank != layer.mixer.kv_rank:
                raise ConfigError(ARCHITECTURE, f"`{where}`: layer {source} keeps latents of {layers[source].mixer.kv_rank} "
                                                f"entries, this layer reads {layer.mixer.kv_rank}")
        limit = doc.get("max_position_embeddings")
        if limit is not None:
            limit = required_positive_int(ARCHITECTURE, doc, "max_position_embeddings")
        mult = _number(doc, "residual_mult", "") if doc.get("residual_mult") is not None else 1.0
        logit_scale = _number(doc, "logit_scale", "") if doc.get("logit_scale") is not None else 1.0
        return cls(vocab, width, mult, logit_scale, eps, groups, side_dim, layers, limit or DEFAULT_MAX_POSITIONS,
                   tuple(raw.eos_token_ids), doc)

    def cache_windows(self) -> Tuple[Optional[int], ...]:
        """Per layer, how many rows the layer's cache must keep: the widest window among the layer itself and the layers
        that read its latents (None: every row, or no cache of latents at all)."""
        keep = [getattr(layer.mixer, "window", None) for layer in self.layers]
        unbounded = [layer.kind == ATTENTION_TYPE and layer.mixer.window is None for layer in self.layers]
        for layer in self.layers:
            source = getattr(layer.mixer, "kv_from", None)
            if source is None:
                continue
            if layer.mixer.window is None or unbounded[source]:
                unbounded[source], keep[source] = True, None
            else:
                keep[source] = max(keep[source], layer.mixer.window)
        return tuple(keep[layer.mixer.kv_from] if getattr(layer.mixer, "kv_from", None) is not None else keep[i]
                     for i, layer in enumerate(self.layers))


def _layer(entry: Any, where: str) -> LayerSpec:
    if not isinstance(entry, dict):
        raise ConfigError(ARCHITECTURE, f"`{where[:-1]}` must be an object")
    kind = entry.get("type")
    m = _section(entry, "mixer", where)
    inside = where + "mixer."
    if kind in STATE_SPACE_TYPES:
        mixer = StateSpaceSizes(heads=_count(m, "heads", inside), vdim=_count(m, "vdim", inside), state=_count(m, "state", inside),
                                groups=_count(m, "groups", inside), conv=_count(m, "conv", inside),
                                norm_groups=_count(m, "norm_groups", inside))
        if mixer.heads % mixer.groups:
            raise ConfigError(ARCHITECTURE, f"`{inside}groups` {mixer.groups} does not divide the {mixer.heads} heads")
        if (mixer.heads * mixer.vdim) % mixer.norm_groups:
            raise ConfigError(ARCHITECTURE, f"`{inside}norm_groups` {mixer.norm_groups} does not divide heads * vdim")
    elif kind == ATTENTION_TYPE:
        window = None
        if m.get("mask") is not None:
            window = _count(_section(m, "mask", inside), "size", inside + "mask.")
        kv_from = _count(m, "kv_from", inside, 0) if m.get("kv_from") is not None else None
        mixer = LatentAttentionSizes(heads=_count(m, "heads", inside), dim=_count(m, "dim", inside), vdim=_count(m, "vdim", inside),
                                     kv_rank=_count(m, "kv_rank", inside), scale=_number(m, "scale", inside), window=window,
                                     kv_from=kv_from)
    else:
        raise ConfigError(ARCHITECTURE, f"`{where}type` {kind!r} is not a mixer of this design "
                                        f"({', '.join(STATE_SPACE_TYPES)}, {ATTENTION_TYPE})")
    mlp = None
    if entry.get("mlp") is not None:
        f = _section(entry, "mlp", where)
        if f.get("kind") != "moe":
            raise ConfigError(ARCHITECTURE, f"`{where}mlp.kind` {f.get('kind')!r} is not a feed-forward of this design (moe)")
        router, expert = _section(f, "router", where + "mlp."), _section(f, "expert", where + "mlp.")
        mlp = RoutedSizes(experts=_count(router, "experts", where + "mlp.router."), top=_count(router, "top", where + "mlp.router."),
                          ff=_count(expert, "ff", where + "mlp.expert."), limit=_number(expert, "limit", where + "mlp.expert."),
                          scale=_number(router, "scale", where + "mlp.router.") if router.get("scale") is not None else 1.0)
        if mlp.top > mlp.experts:
            raise ConfigError(ARCHITECTURE, f"`{where}mlp.router.top` exceeds the number of experts")
        if not mlp.limit > 0:
            raise ConfigError(ARCHITECTURE, f"`{where}mlp.expert.limit` must be positive")
    return LayerSpec(kind, mixer, mlp)
