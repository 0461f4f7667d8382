"""A mixture of experts as a feed-forward part.

    z      = W_router h + b_router               float32 logits, one per expert
    chosen = the ``top`` experts with the largest z;  w = softmax over the chosen z alone
    y      = sum_e w_e W_down,e (act(W_gate,e h) * (W_up,e h)),   act = silu

Tensors: ``.router`` [X, E], ``.router.b`` [X], ``.e<i>.gate`` / ``.up`` [F, E], ``.e<i>.down`` [E, F]
(no biases in the experts).  The experts' matrices are stacked when they are bound (gate and up of a
feature as neighbouring rows), so that a kernel finds expert e at a fixed stride.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


class RoutedExperts(Part):
    graph_safe = True

    def __init__(self, width: int, inner: int, n_experts: int, top: int, router_bias: bool = True):
        if not 0 < top <= n_experts:
            raise ValueError(f"{top} of {n_experts} experts cannot be chosen")
        self.width, self.inner, self.n_experts, self.top = width, inner, n_experts, top
        self.router_bias = bool(router_bias)
        self.w_router = self.b_router = self.w_gu = self.wd = None

    def tensor_specs(self, prefix):
        E, F = self.width, self.inner
        # the router stays float32 (its logits decide which experts run)
        specs = [TensorSpec(prefix + ".router", (self.n_experts, E), VECTOR)]
        if self.router_bias:
            specs.append(TensorSpec(prefix + ".router.b", (self.n_experts,), VECTOR))
        for e in range(self.n_experts):
            specs += [TensorSpec(f"{prefix}.e{e}.gate", (F, E)), TensorSpec(f"{prefix}.e{e}.up", (F, E)), TensorSpec(f"{prefix}.e{e}.down", (E, F))]
        return specs

    def bind(self, prefix, tensors, rt):
        self.w_router = tensors[prefix + ".router"].contiguous()
        self.b_router = tensors[prefix + ".router.b"] if self.router_bias else None
        # gate and up of an expert as one matrix [2 F, E], the gate row of a feature followed by its up row: a product's
        # epilogue, and a warp of the row form, then has both of a feature
        pairs = lambda e: torch.stack([tensors[f"{prefix}.e{e}.gate"], tensors[f"{prefix}.e{e}.up"]], dim=1).reshape(2 * self.inner, self.width)
        self.w_gu = torch.stack([pairs(e) for e in range(self.n_experts)], dim=0).contiguous()
        self.wd = torch.stack([tensors[f"{prefix}.e{e}.down"] for e in range(self.n_experts)], dim=0).contiguous()
        for e in range(self.n_experts):      # the stacked copies are what runs
            for name in ("gate", "up", "down"):
                tensors.pop(f"{prefix}.e{e}.{name}", None)

    def forward(self, rt, h):
        ids, wts = ops.moe_router(h, self.w_router, self.b_router, self.top)
        return rt.moe_experts(h, ids, wts, self.w_gu, self.wd)


register_part("feed_forward", "routed_experts", RoutedExperts)
