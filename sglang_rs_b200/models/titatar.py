"""Titatar put together from the parts.

A decoder whose layers each hold a mixer and, unless the layer has none, a feed-forward, with an RMS norm ahead of and
behind each sublayer (``parts.SandwichBlock``); the norms' weights are stored around zero and multiply as 1 + w
(``parts.GroupedRmsNorm(weight_offset=1)``).  The embedding is scaled.  The mixer is

* ``attention`` (``parts.GroupedQueryAttention``): grouped heads, q and k normed over the whole projection with a weight
  per entry, the leading entries of every head rotated in half-split pairs, values of their own width, a sliding window,
  one added to the softmax's denominator (a sink of score 0), a sigmoid gate per head on the result; or
* ``latent_attention`` (``parts.LatentAttention``): queries through a normed latent, keys and values from one normed
  latent per token plus one rotated key part that all heads share, the rotation in interleaved pairs with its long
  wavelengths stretched, a learned sink per head, a sigmoid gate per entry of the joined heads, no window.

The feed-forward is a gated one with SiLU (``parts.GatedMlp``) or routed experts (``parts.RoutedExperts``): softmax over
all router outputs, a correction per output added for the choice only, the chosen scores as weights without
renormalising, the last router outputs standing for experts that return their input, and an expert that all rows share.
A stretch of layers may be walked several times with the same weights, each pass with caches of its own; every pass but
the first is opened by adding the embedding output to the stream (``parts.PassSum``).  The final norm is of the same kind
and the head a matrix of its own.

Checkpoint names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b``,
``l<i>.mix.{q, k, v, q.norm, k.norm, g, o}`` or ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, g, o}``,
``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{router, correction}``, ``l<i>.mlp.e<j>.{gate, up, down}`` and
``l<i>.mlp.shared.{gate, up, down}``.
Fixed by the design, not by config.json: SiLU in every feed-forward, unnormalised router weights, the pairings of the
two rotations, the sink of score 0 in the windowed attention, the offset 1 of the norms' weights.
"""
from __future__ import annotations

from ..config.model_config import ConfigError
from ..config.registry import register_architecture
from ..parts import (AttentionNames, GatedMlp, GatedMlpNames, GroupedQueryAttention, GroupedRmsNorm, LatentAttention,
                     LatentAttentionNames, NoPositionEncoding, OutputHead, PassSum, RotaryEncoding, RoutedExperts,
                     SandwichBlock, TokenEmbedding, WavelengthScaling)
from .decoder import DecoderModel, LayerCall
from .titatar_config import ARCHITECTURE, ATTENTION_TYPE, DenseSizes, TitatarConfig

#: what the norms' stored weights are short of
NORM_WEIGHT_OFFSET = 1.0
#: the score of the sink in the windowed attention's softmax: exp(0) = 1 joins the denominator
WINDOWED_SINK = 0.0


def layer_program(config: TitatarConfig):
    """The layer calls of one forward pass: the layers ahead of the stretch, the stretch ``times`` times (the first call
    of every walk but the first opens the pass), the layers behind it."""
    count, loop = len(config.layers), config.loop
    if loop is None:
        return [LayerCall(i) for i in range(count)]
    calls = [LayerCall(i) for i in range(loop.start)]
    for t in range(loop.times):
        for i in range(loop.start, loop.stop):
            calls.append(LayerCall(i, entry=0 if (t > 0 and i == loop.start) else None, pass_index=t))
    calls += [LayerCall(i) for i in range(loop.stop, count)]
    return calls


def build_titatar(config: TitatarConfig) -> DecoderModel:
    try:
        return _build(config)
    except ValueError as error:
        if isinstance(error, ConfigError):
            raise
        raise ConfigError(ARCHITECTURE, str(error)) from None


def _build(config: TitatarConfig) -> DecoderModel:
    width, eps = config.width, config.norm_eps
    embedding = TokenEmbedding(config.vocab, width, "embed", scale=config.embedding_scale)

    def norm(name: str) -> GroupedRmsNorm:
        return GroupedRmsNorm(width, eps, name, weight_offset=NORM_WEIGHT_OFFSET)
    rotations = {}          # layers with the same rotation share one table of frequencies

    def rotation(spec, head_dim: int, interleaved: bool):
        if spec is None:
            return None
        key = (head_dim, spec, interleaved)
        if key not in rotations:
            scaling = WavelengthScaling(*spec.scaling) if spec.scaling else None
            rotations[key] = RotaryEncoding(head_dim, spec.base, rotary_dim=spec.dims, interleaved=interleaved, scaling=scaling)
        return rotations[key]
    layers = []
    for index, spec in enumerate(config.layers):
        p, m = f"l{index}.", spec.mixer
        if spec.kind == ATTENTION_TYPE:
            mixer = GroupedQueryAttention(
                width, m.heads, m.kv_heads, m.dim, m.scale, rotation(m.rot, m.dim, False) or NoPositionEncoding(),
                AttentionNames(q=p + "mix.q", k=p + "mix.k", v=p + "mix.v", o=p + "mix.o", q_norm=p + "mix.q.norm",
                               k_norm=p + "mix.k.norm", gate=p + "mix.g"),
                qk_norm_eps=eps, window=m.window, whole_norm=True, value_dim=m.vdim, sink=WINDOWED_SINK)
        else:
            mixer = LatentAttention(
                width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, eps, rotation(m.rot, m.rot_dim, True),
                LatentAttentionNames(q_down=p + "mix.dq", q_norm=p + "mix.dq.norm", q_up=p + "mix.uq", kv_down=p + "mix.dkv",
                                     kv_norm=p + "mix.dkv.norm", k_up=p + "mix.uk", v_up=p + "mix.uv", o=p + "mix.o",
                                     sink=p + "mix.sink", gate=p + "mix.g"),
                gate_per_entry=True, partial_sums=True)
        f = spec.mlp
        if f is None:
            layers.append(SandwichBlock(norm(p + "norm1"), mixer, norm(p + "norm1b")))
            continue
        if isinstance(f, DenseSizes):
            feed_forward = GatedMlp(width, f.ff, "silu", GatedMlpNames(gate=p + "mlp.gate", up=p + "mlp.up", down=p + "mlp.down"))
        else:
            shared = None
            if f.shared_ff:
                shared = GatedMlp(width, f.shared_ff, "silu",
                                  GatedMlpNames(gate=p + "mlp.shared.gate", up=p + "mlp.shared.up", down=p + "mlp.shared.down"),
                                  float_result=True)
            feed_forward = RoutedExperts(
                width, f.ff, f.experts, f.top, "silu", p + "mlp.router",
                lambda e, p=p: GatedMlpNames(gate=f"{p}mlp.e{e}.gate", up=f"{p}mlp.e{e}.up", down=f"{p}mlp.e{e}.down"),
                renormalize=False, choice_bias_name=p + "mlp.correction", shared=shared, identity=f.identity)
        layers.append(SandwichBlock(norm(p + "norm1"), mixer, norm(p + "norm1b"), norm(p + "norm2"), feed_forward,
                                    norm(p + "norm2b")))
    entries = [PassSum()] if config.loop is not None and config.loop.times > 1 else []
    program = layer_program(config)
    if not entries:
        program = [LayerCall(call.layer) for call in program]
    # a layer without a feed-forward has no second pair of norms; checkpoints may carry them all the same
    ignored = [f"l{i}.norm2*" for i, spec in enumerate(config.layers) if spec.mlp is None]
    return DecoderModel(embedding, layers, norm("final.norm"), OutputHead(config.vocab, width, "head"),
                        vocab_size=config.vocab, max_positions=config.max_positions, eos_token_ids=config.eos_token_ids,
                        program=program, pass_entries=entries, ignored_tensors=ignored)


register_architecture(ARCHITECTURE, TitatarConfig.from_raw, build_titatar, replace=True)
