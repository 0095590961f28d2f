"""The gated delta rule with a decay per head and key channel, behind short causal convolutions.

For the mixer's input h, H heads over G query/key heads (head h reads group h // (H / G)), dk key and dv value channels:

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     conv: per channel over the last `taps` tokens
    q <- q / sqrt(sum q^2 + 1e-6) dk^-1/2,   k <- k / sqrt(sum k^2 + 1e-6)          per head
    beta = sigmoid(W_b h)                                                   one per head
    g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias))                one per head and key channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q      per head, S: dk x dv, float32

Each head's o is RMS-normed over dv (one weight for all heads), multiplied by sigmoid(W_g2 (W_g1 h)) and projected by
W_o.  Two states of fixed size per request: S, and the last taps - 1 inputs of the convolutions.  q, k, v, beta and
the first half of the decay's pair are one product over stacked weights; what follows the convolution is float32.

``decay_per`` = "head": one decay per head and token instead, g = exp(-exp(A_log_h) softplus(W_a h + dt_bias_h)) with
W_a of one row per head; the scan forms it from the product's output itself.  ``gate_form`` = "silu": the output gate is
silu(W_g h) with a whole matrix W_g in the place of the low-rank pair and the sigmoid.  With both, every projection of
the mixer is one product over stacked weights.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import FixedStateSpec
from ..weights.spec import MATRIX, NORM, VECTOR, WeightSpec
from .base import Mixer, StepContext, register

_NAMES = dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", rate="A_log", norm="norm",
              decay_in="a1", decay_out="a2", decay_bias="dt_bias", gate_in="g1", gate_out="g2", gate="g", out="o")
UNIT_NORM_EPS = 1e-6


@register("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    writes_through_linear = True  # out is the out of the last product

    def __init__(self, hidden_size: int, num_heads: int, num_key_heads: int, key_dim: int, value_dim: int, conv_taps: int,
                 norm_eps: float, low_rank: Optional[int] = None, random_low_rank: int = 16, names: Optional[dict] = None,
                 decay_per: str = "channel", gate_form: str = "low_rank_sigmoid"):
        """``low_rank`` None: the ranks of the two low-rank pairs are whatever the checkpoint stores (random weights are
        drawn with ``random_low_rank``)."""
        if num_heads % num_key_heads:
            raise ValueError("num_heads must be a multiple of num_key_heads")
        if conv_taps < 1:
            raise ValueError("conv_taps must be positive")
        if decay_per not in ("channel", "head") or gate_form not in ("low_rank_sigmoid", "silu"):
            raise ValueError(f"unknown decay {decay_per!r} or gate {gate_form!r}")
        self.decay_per, self.gate_form = decay_per, gate_form
        self.hidden_size, self.num_heads, self.num_key_heads = hidden_size, num_heads, num_key_heads
        self.key_dim, self.value_dim, self.conv_taps = key_dim, value_dim, conv_taps
        self.norm_eps = float(norm_eps)
        self.low_rank = low_rank
        self.random_low_rank = low_rank or random_low_rank
        self.names = dict(_NAMES, **(names or {}))
        self.qk_width = num_key_heads * key_dim
        self.v_width = num_heads * value_dim
        self.g_width = num_heads * key_dim
        self.conv_width = 2 * self.qk_width + self.v_width
        self.inner_width = self.v_width
        self.q_scale = float(key_dim) ** -0.5
        self.decay_rank = self.gate_rank = low_rank
        self.w_in = self.w_conv = self.w_a2 = self.decay_bias = self.log_rate = None
        self.w_g1 = self.w_g2 = self.norm_w = self.w_o = None

    def cache_specs(self):
        # the recurrence's state (a value channel's key channels side by side), and the convolutions' last inputs
        return [FixedStateSpec((self.num_heads, self.value_dim, self.key_dim), torch.float32),
                FixedStateSpec((self.conv_taps - 1, self.conv_width), torch.float32)]

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        n, W, r, H = self.names, self.hidden_size, self.low_rank, self.num_heads
        rr = self.random_low_rank
        fill = (lambda a, b: None) if r is not None else (lambda a, b: (a, b))
        specs = [
            WeightSpec(prefix + n["q"], (self.qk_width, W), MATRIX),
            WeightSpec(prefix + n["q_conv"], (self.qk_width, self.conv_taps), MATRIX),
            WeightSpec(prefix + n["k"], (self.qk_width, W), MATRIX),
            WeightSpec(prefix + n["k_conv"], (self.qk_width, self.conv_taps), MATRIX),
            WeightSpec(prefix + n["v"], (self.v_width, W), MATRIX),
            WeightSpec(prefix + n["v_conv"], (self.v_width, self.conv_taps), MATRIX),
            WeightSpec(prefix + n["beta"], (H, W), MATRIX),
            WeightSpec(prefix + n["rate"], (H,), VECTOR),
            WeightSpec(prefix + n["norm"], (self.value_dim,), NORM),
            WeightSpec(prefix + n["out"], (W, self.v_width), MATRIX),
        ]
        if self.decay_per == "head":
            specs += [WeightSpec(prefix + n["decay_in"], (H, W), MATRIX), WeightSpec(prefix + n["decay_bias"], (H,), VECTOR)]
        else:
            specs += [WeightSpec(prefix + n["decay_in"], (r, W), MATRIX, fill=fill(rr, W)),
                      WeightSpec(prefix + n["decay_out"], (self.g_width, r), MATRIX, fill=fill(self.g_width, rr)),
                      WeightSpec(prefix + n["decay_bias"], (self.g_width,), VECTOR)]
        if self.gate_form == "silu":
            specs.append(WeightSpec(prefix + n["gate"], (self.v_width, W), MATRIX))
        else:
            specs += [WeightSpec(prefix + n["gate_in"], (r, W), MATRIX, fill=fill(rr, W)),
                      WeightSpec(prefix + n["gate_out"], (self.v_width, r), MATRIX, fill=fill(self.v_width, rr))]
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        n = self.names
        a1 = source.get(prefix + n["decay_in"])
        stacked = [source.get(prefix + n[x]) for x in ("q", "k", "v", "beta")] + [a1]
        if self.decay_per == "head":
            self.decay_rank = self.num_heads            # the decay's input: one column per head
        else:
            a2 = source.get(prefix + n["decay_out"])
            if a1.shape[0] != a2.shape[1]:
                raise ValueError(f"{prefix}: a low-rank pair does not fit: {tuple(a1.shape)}, {tuple(a2.shape)}")
            self.decay_rank = int(a1.shape[0])
            self.w_a2 = a2.to(dtype).to(device).contiguous()
        if self.gate_form == "silu":
            stacked.append(source.get(prefix + n["gate"]))       # the gate rides in the stacked product
        else:
            g1, g2 = source.get(prefix + n["gate_in"]), source.get(prefix + n["gate_out"])
            if g1.shape[0] != g2.shape[1]:
                raise ValueError(f"{prefix}: a low-rank pair does not fit: {tuple(g1.shape)}, {tuple(g2.shape)}")
            self.gate_rank = int(g1.shape[0])
            self.w_g1 = ops.prepare_matrix(g1.to(dtype).to(device))
            self.w_g2 = ops.prepare_matrix(g2.to(dtype).to(device))
        self.w_in = ops.prepare_matrix(torch.cat(stacked, dim=0).to(dtype).to(device))
        conv = torch.cat([source.get(prefix + n[x]) for x in ("q_conv", "k_conv", "v_conv")], dim=0)
        self.w_conv = conv.to(torch.float32).to(device).contiguous()
        self.decay_bias = source.get(prefix + n["decay_bias"]).to(torch.float32).to(device).contiguous()
        self.log_rate = source.get(prefix + n["rate"]).to(torch.float32).to(device).contiguous()
        self.norm_w = source.get(prefix + n["norm"]).to(torch.float32).to(device).contiguous()
        self.w_o = ops.prepare_matrix(source.get(prefix + n["out"]).to(dtype).to(device))

    def first_weights(self):
        return self.w_in

    def output_weight(self):
        return self.w_o

    def mix_into(self, ctx: StepContext, x, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        T, H, G, dk, dv = ctx.num_tokens, self.num_heads, self.num_key_heads, self.key_dim, self.value_dim
        state, conv_state = cache
        C, qk = self.conv_width, self.qk_width
        silu_gate = self.gate_form == "silu"
        n_dec = C + H + self.decay_rank
        proj = ctx.arena.alloc((T, n_dec + (self.v_width if silu_gate else 0)), ctx.dtype)
        ops.linear(x, self.w_in, proj)
        if silu_gate:
            gate = proj[:, n_dec:]
        else:
            gate_in = ctx.arena.alloc((T, self.gate_rank), ctx.dtype)
            ops.linear(x, self.w_g1, gate_in)
            gate = ctx.arena.alloc((T, self.v_width), ctx.dtype)
            ops.linear(gate_in, self.w_g2, gate)
        qkv = ctx.arena.alloc((T, C), torch.float32)
        ops.short_conv(proj[:, :C], self.w_conv, conv_state, ctx, qkv, write_state=write_cache, silu=True)
        ops.unit_norm(qkv[:, :qk], G, dk, UNIT_NORM_EPS, self.q_scale)
        ops.unit_norm(qkv[:, qk:2 * qk], G, dk, UNIT_NORM_EPS, 1.0)
        o = ctx.arena.alloc((T, self.v_width), torch.float32)
        if self.decay_per == "head":
            # the scan forms the heads' decays from the product's output while it stages the tokens
            ops.delta_rule_scan(qkv[:, :qk], qkv[:, qk:2 * qk], qkv[:, 2 * qk:], None, proj[:, C:C + H], state, ctx, o,
                                H, G, dk, dv, write_state=write_cache,
                                head_decay=(proj[:, C + H:n_dec], self.log_rate, self.decay_bias))
        else:
            decay = ctx.arena.alloc((T, self.g_width), torch.float32)
            ops.channel_decay(proj[:, C + H:n_dec], self.w_a2, self.decay_bias, 1.0, decay, log_rate=self.log_rate)
            ops.delta_rule_scan(qkv[:, :qk], qkv[:, qk:2 * qk], qkv[:, 2 * qk:], decay, proj[:, C:C + H], state, ctx, o,
                                H, G, dk, dv, write_state=write_cache)
        ops.head_norm_gate(o, gate, self.norm_w, self.norm_eps, inner, H, dv, gate_kind="silu" if silu_gate else "sigmoid",
                           scale=scale)

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        inner = ctx.arena.alloc((ctx.num_tokens, self.inner_width), ctx.dtype)
        self.mix_into(ctx, x, cache, group, inner, write_cache)
        ops.linear(inner, self.w_o, out)
