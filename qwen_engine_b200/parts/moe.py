"""Routed experts: a mixture of small gated feed-forwards of which every token uses a few.

    z = W_router h + b                      float32, one logit per expert
    the `top` experts with the largest logits are chosen; their weights are the softmax over the chosen logits alone
    out = sum over the chosen e of weight_e * W_down,e glu(W_gate,e h, W_up,e h)

The experts' weights are stacked ([E, 2 ff, W] gate rows then up rows, and [E, W, ff]); the (token, choice) pairs
are ordered by expert on the device and run as tiles of two grouped products, the activation in the first one's
epilogue.  Nothing of the launches depends on the routing, so steps are replayed from CUDA graphs like any other.

``scoring`` = "softmax_all": s = softmax(z) over all router outputs; the `top` largest of s + correction (a stored
vector) are chosen and their weights are their s as it is.  ``num_identity``: the router's last outputs stand for
experts without weights that hand their input on (times the weight).  ``router_bias_name`` None: no router bias.

``scoring`` = "sigmoid": every router output is scored alone, s = sigmoid(z); the `top` largest are chosen and their
weights are their s, not made to sum to one.  ``weight_inputs``: the weight multiplies what an expert reads, not what it
returns: out = sum over the chosen e of expert_e(weight_e * h).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, WeightSpec
from .base import FeedForward, StepContext, register


@register("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, activation="silu",
                 names: tuple = ("gate", "up", "down"), router_name: str = "router", router_bias_name: Optional[str] = "router.b",
                 expert_prefix: str = "e", scoring: str = "softmax_chosen", correction_name: Optional[str] = None,
                 num_identity: int = 0, weight_inputs: bool = False):
        if not ops.gate_activation_known(activation):
            raise ValueError(f"unknown activation {activation!r}")
        if not (1 <= top <= num_experts + num_identity):
            raise ValueError(f"top = {top} of {num_experts + num_identity} experts")
        if scoring not in ops.ROUTER_SCORINGS or (correction_name is not None and scoring != "softmax_all"):
            raise ValueError(f"unknown scoring {scoring!r}, or a correction without scores over all experts")
        self.scoring, self.correction_name, self.num_identity = scoring, correction_name, int(num_identity)
        self.correction = None
        self.weight_inputs = bool(weight_inputs)
        if self.weight_inputs and num_identity:
            raise ValueError("weighted inputs and identity experts do not go together")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top = num_experts, top
        self.activation = tuple(activation) if isinstance(activation, (tuple, list)) else activation
        self.names, self.router_name, self.router_bias_name, self.expert_prefix = tuple(names), router_name, router_bias_name, expert_prefix
        self.w_router = self.router_bias = self.w_gate_up = self.w_down = None

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        I, W = self.intermediate_size, self.hidden_size
        gate, up, down = self.names
        specs = []
        for e in range(self.num_experts):
            p = f"{prefix}{self.expert_prefix}{e}."
            specs += [WeightSpec(p + gate, (I, W), MATRIX), WeightSpec(p + up, (I, W), MATRIX), WeightSpec(p + down, (W, I), MATRIX)]
        outputs = self.num_experts + self.num_identity
        specs.append(WeightSpec(prefix + self.router_name, (outputs, W), MATRIX))
        if self.router_bias_name is not None:
            specs.append(WeightSpec(prefix + self.router_bias_name, (outputs,), VECTOR))
        if self.correction_name is not None:
            specs.append(WeightSpec(prefix + self.correction_name, (outputs,), VECTOR))
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        gate, up, down = self.names
        gu, dn = [], []
        for e in range(self.num_experts):
            p = f"{prefix}{self.expert_prefix}{e}."
            gu.append(torch.cat([source.get(p + gate), source.get(p + up)], dim=0))
            dn.append(source.get(p + down))
        self.w_gate_up = torch.stack(gu).to(dtype).to(device).contiguous()
        self.w_down = torch.stack(dn).to(dtype).to(device).contiguous()
        # the router works in float32 whatever the compute type
        self.w_router = source.get(prefix + self.router_name).to(torch.float32).to(device).contiguous()
        if self.router_bias_name is not None:
            self.router_bias = source.get(prefix + self.router_bias_name).to(torch.float32).to(device).contiguous()
        if self.correction_name is not None:
            self.correction = source.get(prefix + self.correction_name).to(torch.float32).to(device).contiguous()

    def first_weights(self):
        return None

    def forward(self, ctx: StepContext, x, out) -> None:
        T = ctx.num_tokens
        top_idx = ctx.arena.alloc((T, self.top), torch.int32)
        top_w = ctx.arena.alloc((T, self.top), torch.float32)
        ops.moe_route(x, self.w_router, self.router_bias, top_idx, top_w, scoring=self.scoring, correction=self.correction)
        ops.moe_experts(x, top_idx, top_w, self.w_gate_up, self.w_down, out, self.activation, ctx.arena.alloc,
                        num_identity=self.num_identity, weight_inputs=self.weight_inputs)
