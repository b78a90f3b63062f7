"""A feed-forward of routed experts.

Router logits z = W_router h in 32-bit, scores s = softmax(z) over all experts; the ``top`` experts with
the largest scores are chosen (ties: the lower index) and the result is sum_e s_e * expert_e(h) over the
chosen ones, with the scores as they are or, with ``renormalize``, divided by their sum.  An expert is a
gated feed-forward without biases: W_down (act(W_gate h) * (W_up h)).  The experts' matrices are stacked at
load ([experts, ...]; gate rows over up rows); the whole part is a handful of launches that decide nothing on the host (``ops.routed_experts``),
so decode steps can be captured.  The result is 32-bit: the weighted sum is taken in 32-bit and goes to
the residual sum (or the norm ahead of it) unrounded.
"""
from __future__ import annotations

from typing import Callable, Dict, Mapping

import torch

from .. import ops
from .base import FeedForward, TensorSpec, matrix_to
from .mlp import GatedMlpNames


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, inner: int, experts: int, top: int, activation: str, router_name: str,
                 expert_names: Callable[[int], GatedMlpNames], renormalize: bool = False):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unsupported activation {activation}; available: {sorted(ops.ACTIVATIONS)}")
        if not 0 < top <= experts:
            raise ValueError(f"{top} chosen experts of {experts}")
        if experts > 1024 or top > 32:
            raise ValueError(f"the router kernel takes at most 1024 experts and 32 chosen ones, not {experts} and {top}")
        self.hidden, self.inner, self.experts, self.top = int(hidden), int(inner), int(experts), int(top)
        self.activation, self.router_name, self.renormalize = activation, router_name, bool(renormalize)
        self.names = [expert_names(e) for e in range(self.experts)]
        self.router = self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.router_name: TensorSpec((self.experts, self.hidden))}
        for n in self.names:
            specs[n.gate] = TensorSpec((self.inner, self.hidden))
            specs[n.up] = TensorSpec((self.inner, self.hidden))
            specs[n.down] = TensorSpec((self.hidden, self.inner))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.router = matrix_to(tensors[self.router_name], device, dtype)
        # per expert the gate rows over the up rows: the two matrices of a tile then lie a fixed distance apart
        self.w_gate_up = matrix_to(torch.stack([torch.cat([tensors[n.gate], tensors[n.up]], dim=0) for n in self.names]),
                                   device, dtype)
        self.w_down = matrix_to(torch.stack([tensors[n.down] for n in self.names]), device, dtype)

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return ops.routed_experts(x, self.router, self.w_gate_up, self.w_down, self.top, self.activation,
                                  self.renormalize, ctx.error_word)
