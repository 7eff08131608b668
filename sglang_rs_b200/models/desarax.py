"""Desarax put together from the parts.

A decoder whose layers each run a mixer and, unless the layer has none, a feed-forward of routed experts side by side
from ONE norm of the stream (``parts.ParallelBlock``): x <- x + mult * (mixer(h) + experts(h)), h = norm(x), the norm an
RMS norm in equal parts of the row (``parts.GroupedRmsNorm``).  After that every layer adds the token's own input
(``parts.TokenSideInput``: a gate of the stream times the layer's slice of a second table's row, projected, RMS-normed
with a plain weight, times mult), unless the document has no such table.  The mixer is a state-space mixer
(``parts.MambaMixer``) or attention through latents without positions (``parts.LatentAttention`` with queries straight
from the input, no rotated part, no sink, no gate, a sliding window); an attention layer may read the latents that an
earlier attention layer caches, which is a layer call on that layer's cache (``LayerCall.cache_from``).  The experts
(``parts.RoutedExperts``) score with a sigmoid, choose with a correction per expert, renormalise the chosen scores and
scale them; an expert clamps gate and up.  The head is the embedding table, its logits times a constant.

Checkpoint names: ``embed``, ``side.embed``, ``final.norm`` and per layer ``l<i>.norm1``, ``l<i>.mix.{in, conv, conv.b,
dt_bias, A_log, D, norm, o}`` or ``l<i>.mix.{q, dkv, dkv.norm, uk, uv, o}``, ``l<i>.mlp.{router, correction}``,
``l<i>.mlp.e<j>.{gate, up, down}`` and ``l<i>.side.{gate, proj, norm}``.
Fixed by the design, not by config.json: the experts' activation and its 1.702, the 1e-20 beside the sum of the chosen
scores, SiLU around the convolution and in the state-space gate, the tanh form of GELU in the token's gate.
"""
from __future__ import annotations

from ..config.model_config import ConfigError
from ..config.registry import register_architecture
from ..parts import (GatedMlpNames, GroupedRmsNorm, LatentAttention, LatentAttentionNames, MambaMixer, MambaNames,
                     OutputHead, ParallelBlock, RoutedExperts, TokenEmbedding, TokenSideInput, TokenSideNames)
from .decoder import DecoderModel, LayerCall
from .desarax_config import ARCHITECTURE, ATTENTION_TYPE, DesaraxConfig

#: added to the sum of the chosen scores before they are divided by it
CHOSEN_SUM_EPS = 1e-20
SIDE_TABLE = "side.embed"


def build_desarax(config: DesaraxConfig) -> DecoderModel:
    try:
        return _build(config)
    except ValueError as error:
        if isinstance(error, ConfigError):
            raise
        raise ConfigError(ARCHITECTURE, str(error)) from None


def _build(config: DesaraxConfig) -> DecoderModel:
    width, eps, mult = config.width, config.norm_eps, config.residual_mult
    count = len(config.layers)
    tables = {SIDE_TABLE: count * config.side_dim} if config.side_dim else None
    embedding = TokenEmbedding(config.vocab, width, "embed", side_tables=tables)
    keep = config.cache_windows()
    layers, program, call_of = [], [], {}
    for index, spec in enumerate(config.layers):
        p, m = f"l{index}.", spec.mixer
        if spec.kind == ATTENTION_TYPE:
            own = m.kv_from is None
            mixer = LatentAttention(
                width, m.heads, m.dim, 0, m.vdim, 0, m.kv_rank, m.scale, eps, None,
                LatentAttentionNames(q_down=None, q_norm=None, q_up=p + "mix.q", kv_down=p + "mix.dkv" if own else None,
                                     kv_norm=p + "mix.dkv.norm" if own else None, k_up=p + "mix.uk", v_up=p + "mix.uv",
                                     o=p + "mix.o"),
                window=m.window, cache_window=keep[index])
            call_of[index] = len(program)
            program.append(LayerCall(index, cache_from=None if own else call_of[m.kv_from]))
        else:
            mixer = MambaMixer(width, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, eps,
                               MambaNames(w_in=p + "mix.in", conv=p + "mix.conv", conv_bias=p + "mix.conv.b",
                                          dt_bias=p + "mix.dt_bias", a_log=p + "mix.A_log", d=p + "mix.D", norm=p + "mix.norm",
                                          o=p + "mix.o"))
            program.append(LayerCall(index))
        feed_forward = None
        if spec.mlp is not None:
            f = spec.mlp
            feed_forward = RoutedExperts(
                width, f.ff, f.experts, f.top, "swiglu_clamp", p + "mlp.router",
                lambda e, p=p: GatedMlpNames(gate=f"{p}mlp.e{e}.gate", up=f"{p}mlp.e{e}.up", down=f"{p}mlp.e{e}.down"),
                renormalize=True, scoring="sigmoid", choice_bias_name=p + "mlp.correction", weight_scale=f.scale,
                norm_eps=CHOSEN_SUM_EPS, activation_param=f.limit)
        side = None
        if config.side_dim:
            side = TokenSideInput(width, config.side_dim, index * config.side_dim, embedding, SIDE_TABLE,
                                  GroupedRmsNorm(width, eps, p + "side.norm", groups=1, scale=mult),
                                  TokenSideNames(gate=p + "side.gate", proj=p + "side.proj"))
        layers.append(ParallelBlock(GroupedRmsNorm(width, eps, p + "norm1", groups=config.norm_groups), mixer, feed_forward,
                                    mult=mult, side=side))
    final_norm = GroupedRmsNorm(width, eps, "final.norm", groups=config.norm_groups)
    head = OutputHead(config.vocab, width, None, embedding=embedding, scale=config.logit_scale)
    return DecoderModel(embedding, layers, final_norm, head, vocab_size=config.vocab, max_positions=config.max_positions,
                        eos_token_ids=config.eos_token_ids, program=program)


register_architecture(ARCHITECTURE, DesaraxConfig.from_raw, build_desarax, replace=True)
