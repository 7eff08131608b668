"""A feed-forward of routed experts.

Router logits z = W_router h in 32-bit, scores s = softmax(z) over all experts; the ``top`` experts with
the largest scores are chosen (ties: the lower index) and the result is sum_e s_e * expert_e(h) over the
chosen ones, with the scores as they are or, with ``renormalize``, divided by their sum.  An expert is a
gated feed-forward without biases: W_down (act(W_gate h) * (W_up h)).  The experts' matrices are stacked at
load ([experts, ...]; gate rows over up rows); the whole part is a handful of launches that decide nothing on the host (``ops.routed_experts``),
so decode steps can be captured.  The result is 32-bit: the weighted sum is taken in 32-bit and goes to
the residual sum (or the norm ahead of it) unrounded.

Variations, all off by default: experts without a gate, W_down act(W_up h) (``expert_names`` then gives
``GatedMlpNames`` with ``gate`` None); a bias on the router's logits (``router_bias_name``), added before the
choice; an expert that every row shares (``shared``: a feed-forward whose 32-bit result is the first term of
the sum).  A softmax over the chosen logits only is the same as ``renormalize`` over the softmax of all.
Scores may be the sigmoid of each logit instead of the softmax over all (``scoring="sigmoid"``); a correction per expert
(``choice_bias_name``) may be added to the scores for the choice alone, the weights using the scores without it; with
``renormalize`` the chosen scores are divided by their sum plus ``norm_eps``; ``weight_scale`` multiplies the weights.
An activation with a parameter (``swiglu_clamp``: g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit) and
u' = clamp(u, -limit, limit)) takes it as ``activation_param``.
``identity``: the router has this many outputs behind the experts' that stand for experts without tensors, whose result is
their input: a row that chooses one gets weight * h as that term.  Scores, the correction and the choice run over all
router outputs alike (the router matrix and the correction have experts + identity rows).
"""
from __future__ import annotations

from typing import Callable, Dict, Mapping, Optional

import torch

from .. import ops
from .base import FeedForward, TensorSpec, matrix_to, scale_to
from .mlp import GatedMlpNames


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, inner: int, experts: int, top: int, activation: str, router_name: str,
                 expert_names: Callable[[int], GatedMlpNames], renormalize: bool = False, *,
                 router_bias_name: Optional[str] = None, shared: Optional[FeedForward] = None,
                 scoring: str = "softmax", choice_bias_name: Optional[str] = None, weight_scale: float = 1.0,
                 norm_eps: float = 0.0, activation_param: float = 0.0, identity: int = 0):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unsupported activation {activation}; available: {sorted(ops.ACTIVATIONS)}")
        if scoring not in ops.ROUTER_SCORING:
            raise ValueError(f"unsupported scoring {scoring}; available: {sorted(ops.ROUTER_SCORING)}")
        if identity < 0:
            raise ValueError(f"{identity} experts that return their input")
        if not 0 < top <= experts + identity or experts <= 0:
            raise ValueError(f"{top} chosen experts of {experts + identity}")
        if experts + identity > 1024 or top > 32:
            raise ValueError(f"the router kernel takes at most 1024 experts and 32 chosen ones, not {experts + identity} and {top}")
        self.identity = int(identity)
        self.hidden, self.inner, self.experts, self.top = int(hidden), int(inner), int(experts), int(top)
        self.activation, self.router_name, self.renormalize = activation, router_name, bool(renormalize)
        self.names = [expert_names(e) for e in range(self.experts)]
        self.gated = self.names[0].gate is not None
        if any((n.gate is not None) != self.gated for n in self.names):
            raise ValueError("the experts of one layer have a gate or have none, all alike")
        self.router_bias_name, self.shared = router_bias_name, shared
        self.scoring, self.choice_bias_name = scoring, choice_bias_name
        self.weight_scale, self.norm_eps, self.activation_param = float(weight_scale), float(norm_eps), float(activation_param)
        self.router = self.w_gate_up = self.w_down = self.router_bias = self.choice_bias = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        routes = self.experts + self.identity
        specs = {self.router_name: TensorSpec((routes, self.hidden))}
        if self.router_bias_name:
            specs[self.router_bias_name] = TensorSpec((routes,))
        if self.choice_bias_name:
            specs[self.choice_bias_name] = TensorSpec((routes,))
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
        for n in self.names:
            if self.gated:
                specs[n.gate] = TensorSpec((self.inner, self.hidden))
            specs[n.up] = TensorSpec((self.inner, self.hidden))
            specs[n.down] = TensorSpec((self.hidden, self.inner))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.router = matrix_to(tensors[self.router_name], device, dtype)
        # per expert the gate rows over the up rows: the two matrices of a tile then lie a fixed distance apart
        if self.gated:
            stacked = [torch.cat([tensors[n.gate], tensors[n.up]], dim=0) for n in self.names]
        else:
            stacked = [tensors[n.up] for n in self.names]
        self.w_gate_up = matrix_to(torch.stack(stacked), device, dtype)
        self.router_bias = scale_to(tensors[self.router_bias_name], device) if self.router_bias_name else None
        self.choice_bias = scale_to(tensors[self.choice_bias_name], device) if self.choice_bias_name else None
        if self.shared is not None:
            self.shared.load(tensors, device, dtype)
        self.w_down = matrix_to(torch.stack([tensors[n.down] for n in self.names]), device, dtype)

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        base = self.shared.forward(ctx, x) if self.shared is not None else None
        if base is not None and (base.dtype != torch.float32 or base.dim() != 2):
            raise TypeError("the shared expert must give a 32-bit result [rows, width]")
        return ops.routed_experts(x, self.router, self.w_gate_up, self.w_down, self.top, self.activation,
                                  self.renormalize, ctx.error_word, gated=self.gated, router_bias=self.router_bias,
                                  base=base, scoring=self.scoring, choice_bias=self.choice_bias,
                                  weight_scale=self.weight_scale, norm_eps=self.norm_eps,
                                  activation_param=self.activation_param, identity=self.identity)
