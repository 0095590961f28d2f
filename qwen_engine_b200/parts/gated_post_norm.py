"""A residual block that norms what a sublayer returns, not what it reads.

For the float32 stream x of a layer, with a sublayer f (the mixer, then the feed-forward):

    h  = x + conv(x)                         a short causal convolution over time on each channel (``conv_taps`` taps;
                                             tap taps - 1 multiplies the token itself); the last taps - 1 rows of x
                                             are state of the request, one state per sublayer
    x <- x + norm(f(h) * sigmoid(W_r x + b)) the gate reads x itself, not h

and then, optionally,

    x <- x + rmsnorm(W_p (gelu_tanh(W_s x) * e)) * w     ``token_side``: e is this layer's ``dim`` columns of a second
                                                         embedding table's row of the token
    x <- sum_j a[j] X_j                                  ``depth_mix``: X_0 the embedding output, X_(j+1) the result of
                                                         layer run j (before this sum), a of one weight per X so far

The sublayers' inputs are rounded once to the compute type; the stream, the convolution, the gates, the norms and the
sums are float32.  The weighted sum needs the model to keep its runs' results (``ModelLayout.layer_history``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import FixedStateSpec
from ..weights.spec import MATRIX, NORM, VECTOR, WeightSpec
from .base import Block, PartSpec, StepContext, register, step_hint

_NAMES = dict(norm1="norm1", norm2="norm2", conv1="canon1", conv2="canon2", gate1="rg1", gate1_bias="rg1.b", gate2="rg2",
              gate2_bias="rg2.b", side_gate="side.gate", side_proj="side.proj", side_norm="side.norm", depth="dwa")


@register("block", "gated_post_norm")
class GatedPostNormBlock(Block):
    def __init__(self, hidden_size: int, mixer: PartSpec, feed_forward: Optional[PartSpec], norm: PartSpec, conv_taps: int,
                 mixer_prefix: str = "mix.", ffn_prefix: str = "mlp.", token_side: Optional[dict] = None,
                 depth_mix: Optional[int] = None, names: Optional[dict] = None):
        """``token_side``: dict(dim, table (the table's tensor name, without the layer's prefix), columns (of the whole
        table), first (this layer's first column), vocab, eps).  ``depth_mix``: how many results the layer's weighted sum
        runs over (the embedding output and every run up to this one)."""
        if conv_taps < 1:
            raise ValueError("conv_taps must be positive")
        self.hidden_size, self.conv_taps = hidden_size, conv_taps
        self.mixer = mixer.build("mixer")
        self.ffn = feed_forward.build("feed_forward") if feed_forward is not None else None
        self.norm1 = norm.build("norm")
        self.norm2 = norm.build("norm") if self.ffn is not None else None
        self.mixer_prefix, self.ffn_prefix = mixer_prefix, ffn_prefix
        self.token_side = dict(token_side) if token_side else None
        self.depth_mix = depth_mix
        self.names = dict(_NAMES, **(names or {}))
        self.n_mixer_caches = len(self.mixer.cache_specs())
        self.w_conv1 = self.w_conv2 = self.w_gate1 = self.w_gate2 = self.b_gate1 = self.b_gate2 = None
        self.side_table = self.w_side_gate = self.w_side_proj = self.side_norm_w = self.depth_w = None

    @property
    def capturable(self) -> bool:
        return all(getattr(p, "capturable", True) for p in (self.mixer, self.ffn) if p is not None)

    def cache_specs(self) -> list:
        # behind the mixer's caches: the last taps - 1 rows of the stream, for each sublayer
        specs = list(self.mixer.cache_specs())
        if self.conv_taps > 1:
            specs += [FixedStateSpec((self.conv_taps - 1, self.hidden_size), torch.float32)
                      for _ in range(1 if self.ffn is None else 2)]
        return specs

    def weight_specs(self, prefix: str):
        n, W = self.names, self.hidden_size
        specs = self.mixer.weight_specs(prefix + self.mixer_prefix) + self.norm1.weight_specs(prefix + n["norm1"])
        specs += [WeightSpec(prefix + n["conv1"], (W, self.conv_taps), MATRIX), WeightSpec(prefix + n["gate1"], (W, W), MATRIX),
                  WeightSpec(prefix + n["gate1_bias"], (W,), VECTOR)]
        if self.ffn is not None:
            specs += self.ffn.weight_specs(prefix + self.ffn_prefix) + self.norm2.weight_specs(prefix + n["norm2"])
            specs += [WeightSpec(prefix + n["conv2"], (W, self.conv_taps), MATRIX), WeightSpec(prefix + n["gate2"], (W, W), MATRIX),
                      WeightSpec(prefix + n["gate2_bias"], (W,), VECTOR)]
        if self.token_side:
            ts = self.token_side
            specs += [WeightSpec(ts["table"], (ts["vocab"], ts["columns"]), MATRIX),
                      WeightSpec(prefix + n["side_gate"], (ts["dim"], W), MATRIX),
                      WeightSpec(prefix + n["side_proj"], (W, ts["dim"]), MATRIX),
                      WeightSpec(prefix + n["side_norm"], (W,), NORM)]
        if self.depth_mix:
            specs.append(WeightSpec(prefix + n["depth"], (self.depth_mix,), VECTOR))
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        n = self.names

        def f32(name):
            return source.get(name).to(torch.float32).to(device).contiguous()

        def matrix(name):
            return ops.prepare_matrix(source.get(name).to(dtype).to(device))

        self.mixer.load(prefix + self.mixer_prefix, source, dtype, device)
        self.norm1.load(prefix + n["norm1"], source, dtype, device)
        self.w_conv1, self.w_gate1, self.b_gate1 = f32(prefix + n["conv1"]), matrix(prefix + n["gate1"]), f32(prefix + n["gate1_bias"])
        if self.ffn is not None:
            self.ffn.load(prefix + self.ffn_prefix, source, dtype, device)
            self.norm2.load(prefix + n["norm2"], source, dtype, device)
            self.w_conv2, self.w_gate2, self.b_gate2 = f32(prefix + n["conv2"]), matrix(prefix + n["gate2"]), f32(prefix + n["gate2_bias"])
        if self.token_side:
            ts = self.token_side
            # this layer's columns of the table, as a table of its own
            self.side_table = source.get(ts["table"])[:, ts["first"]:ts["first"] + ts["dim"]].to(dtype).to(device).contiguous()
            self.w_side_gate, self.w_side_proj = matrix(prefix + n["side_gate"]), matrix(prefix + n["side_proj"])
            self.side_norm_w = f32(prefix + n["side_norm"])
        if self.depth_mix:
            self.depth_w = f32(prefix + n["depth"])

    def first_weights(self):
        return None

    def _sublayer(self, ctx: StepContext, src, dst, part, run, norm, w_conv, state, w_gate, b_gate, write_cache, cast=None):
        """dst = src + norm(part(src + conv(src)) * sigmoid(W_gate src + b_gate)); ``run(h, out)`` runs the part."""
        T, W = ctx.num_tokens, self.hidden_size
        plain = ctx.arena.alloc((T, W), ctx.dtype)
        convolved = ctx.arena.alloc((T, W), ctx.dtype)
        ops.stream_conv(src, w_conv, state, ctx, plain, convolved, write_state=write_cache)
        gate = ctx.arena.alloc((T, W), ctx.dtype)
        ops.linear(plain, w_gate, gate)
        out = ctx.arena.alloc((T, W), ctx.dtype)
        run(convolved, out)
        norm.norm_add(ctx, src, out, dst, gate=gate, gate_bias=b_gate, cast=cast)

    def forward(self, ctx: StepContext, stream, cache, group, write_cache) -> None:
        T, W = ctx.num_tokens, self.hidden_size
        caches = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        groups = group if isinstance(group, tuple) else (() if group is None else (group,))
        nm = self.n_mixer_caches
        m_cache = None if nm == 0 else caches[0] if nm == 1 else tuple(caches[:nm])
        m_group = None if nm == 0 else groups[0] if nm == 1 else tuple(groups[:nm])
        conv_states = list(caches[nm:]) + [None, None]
        if stream.has_delta:
            raise RuntimeError("gated_post_norm: the stream carries a branch output that nobody added")
        history = step_hint(ctx, "layer_history")
        mark = ctx.arena.mark()
        x = stream.resid
        # the layer's result is built in its own row of the runs' results when the model keeps them, else in place
        y = history.results[history.run + 1] if history is not None else x
        cast = ctx.arena.alloc((T, W), ctx.dtype) if (self.token_side and self.ffn is None) else None
        self._sublayer(ctx, x, y, self.mixer, lambda h, out: self.mixer.forward(ctx, h, m_cache, m_group, out, write_cache),
                       self.norm1, self.w_conv1, conv_states[0], self.w_gate1, self.b_gate1, write_cache, cast=cast)
        if self.ffn is not None:
            cast = ctx.arena.alloc((T, W), ctx.dtype) if self.token_side else None
            self._sublayer(ctx, y, y, self.ffn, lambda h, out: self.ffn.forward(ctx, h, out),
                           self.norm2, self.w_conv2, conv_states[1], self.w_gate2, self.b_gate2, write_cache, cast=cast)
        if self.token_side:
            d = self.token_side["dim"]
            side_gate = ctx.arena.alloc((T, d), ctx.dtype)
            ops.linear(cast, self.w_side_gate, side_gate)
            gated = ctx.arena.alloc((T, d), ctx.dtype)
            ops.token_side_gate(side_gate, self.side_table, ctx.token_ids, gated)
            side = ctx.arena.alloc((T, W), ctx.dtype)
            ops.linear(gated, self.w_side_proj, side)
        if self.depth_mix:
            if history is None:
                raise RuntimeError("gated_post_norm: a weighted sum over the runs' results needs a model that keeps them")
            if history.run + 2 != self.depth_mix:
                raise RuntimeError(f"gated_post_norm: run {history.run} sums {history.run + 2} results, the layer has {self.depth_mix} weights")
        mix = (history.results, self.depth_w, self.depth_mix, history.mixed) if self.depth_mix else None
        if self.token_side:
            # the layer's last add also forms the weighted sum over the results so far
            ops.gated_norm_add(y, side, None, None, self.side_norm_w, self.token_side["eps"], y, depth_mix=mix)
        elif mix is not None:
            ops.depth_mix(*mix)
        if mix is not None:
            stream.resid = history.mixed
        elif history is not None:
            stream.resid = y
        stream.has_delta, stream.n_ssq = False, 0
        ctx.arena.release(mark)
