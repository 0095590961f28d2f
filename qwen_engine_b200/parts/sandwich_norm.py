"""A residual block that norms a sublayer's input and its result.

For the float32 stream x of a layer, with a sublayer f (the mixer, then the feed-forward) and the norms n and nb:

    x <- x + m * nb(f(n(x)))

m is folded into nb's weights (the norm part's ``output_scale``).  The mixer may read its normed input through a short
causal convolution over time on each channel (``input_conv_taps`` taps; tap taps - 1 multiplies the token itself):

    h = n(x);  h <- h + conv(h),   conv(h)_t = sum_j c[:, j] * h_(t - taps + 1 + j), rows before the request's start zero

The last taps - 1 rows of h are state of the request (float32, one slot per request and layer).  The norms, the
convolution and the sums are float32; what a sublayer reads is rounded once to the compute type.

The add of a sublayer's result and the norm of the new stream row for the sublayer after it are one pass where the norm
part offers it (``fuses_with``): within the layer, and into the next layer's first norm when the model names it
(``ctx.extras["norm_after_block"]``; the normed rows then wait in ``ctx.extras["normed_ahead"]``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import FixedStateSpec
from ..weights.spec import MATRIX, WeightSpec
from .base import Block, PartSpec, StepContext, register, step_hint

_NAMES = dict(norm1="norm1", norm1b="norm1b", norm2="norm2", norm2b="norm2b", conv="canon1")


@register("block", "sandwich_norm")
class SandwichNormBlock(Block):
    def __init__(self, hidden_size: int, mixer: PartSpec, feed_forward: Optional[PartSpec], norm: PartSpec, post_norm: PartSpec,
                 input_conv_taps: Optional[int] = None, mixer_prefix: str = "mix.", ffn_prefix: str = "mlp.",
                 names: Optional[dict] = None):
        if input_conv_taps is not None and input_conv_taps < 1:
            raise ValueError("input_conv_taps must be positive")
        self.hidden_size, self.conv_taps = hidden_size, input_conv_taps
        self.mixer = mixer.build("mixer")
        self.ffn = feed_forward.build("feed_forward") if feed_forward is not None else None
        self.norm1, self.norm1b = norm.build("norm"), post_norm.build("norm")
        self.norm2 = norm.build("norm") if self.ffn is not None else None
        self.norm2b = post_norm.build("norm") if self.ffn is not None else None
        self.mixer_prefix, self.ffn_prefix = mixer_prefix, ffn_prefix
        self.names = dict(_NAMES, **(names or {}))
        self.n_mixer_caches = len(self.mixer.cache_specs())
        self.w_conv = None

    @property
    def capturable(self) -> bool:
        return all(getattr(p, "capturable", True) for p in (self.mixer, self.ffn) if p is not None)

    def cache_specs(self) -> list:
        # behind the mixer's caches: the last taps - 1 normed rows that the mixer's convolution reads
        specs = list(self.mixer.cache_specs())
        if self.conv_taps is not None and self.conv_taps > 1:
            specs.append(FixedStateSpec((self.conv_taps - 1, self.hidden_size), torch.float32))
        return specs

    def _norms(self):
        n = self.names
        pairs = [(self.norm1, n["norm1"]), (self.norm1b, n["norm1b"])]
        if self.ffn is not None:
            pairs += [(self.norm2, n["norm2"]), (self.norm2b, n["norm2b"])]
        return pairs

    def weight_specs(self, prefix: str):
        specs = self.mixer.weight_specs(prefix + self.mixer_prefix)
        for norm, name in self._norms():
            specs += norm.weight_specs(prefix + name)
        if self.ffn is not None:
            specs += self.ffn.weight_specs(prefix + self.ffn_prefix)
        if self.conv_taps is not None:
            specs.append(WeightSpec(prefix + self.names["conv"], (self.hidden_size, self.conv_taps), MATRIX))
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        self.mixer.load(prefix + self.mixer_prefix, source, dtype, device)
        for norm, name in self._norms():
            norm.load(prefix + name, source, dtype, device)
        if self.ffn is not None:
            self.ffn.load(prefix + self.ffn_prefix, source, dtype, device)
        if self.conv_taps is not None:
            self.w_conv = source.get(prefix + self.names["conv"]).to(torch.float32).to(device).contiguous()

    def first_weights(self):
        return None

    def first_norm(self):
        """The norm that reads the stream first and the type its reader wants (None: the compute type): the block before
        this one may form it in its last add."""
        return self.norm1, (torch.float32 if self.conv_taps is not None else None)

    def _way_back(self, ctx: StepContext, post_norm, x, branch, next_norm, next_dtype, step_lived: bool = False):
        """x += post_norm(branch); returns next_norm(x) from the same pass where the two norms fit, else None."""
        fuse = next_norm is not None and getattr(post_norm, "fuses_with", lambda other: False)(next_norm)
        next_out = None
        if fuse:
            shape = (ctx.num_tokens, self.hidden_size)
            if step_lived:
                # two buffers a step, taken in turn: what a layer leaves for the next one outlives its own scratch
                pool = ctx.extras.setdefault("normed_ahead_buffers", [])
                turn = ctx.extras.get("normed_ahead_turn", 0)
                if len(pool) <= turn:
                    pool.append(ctx.arena.alloc_step(shape, next_dtype))
                next_out = pool[turn]
                ctx.extras["normed_ahead_turn"] = 1 - turn
            else:
                next_out = ctx.arena.alloc(shape, next_dtype)
            post_norm.norm_add(ctx, x, branch, x, next_norm=next_norm, next_out=next_out)
        else:
            post_norm.norm_add(ctx, x, branch, x)
        return next_out

    def forward(self, ctx: StepContext, stream, cache, group, write_cache) -> None:
        T, W = ctx.num_tokens, self.hidden_size
        caches = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        groups = group if isinstance(group, tuple) else (() if group is None else (group,))
        nm = self.n_mixer_caches
        m_cache = None if nm == 0 else caches[0] if nm == 1 else tuple(caches[:nm])
        m_group = None if nm == 0 else groups[0] if nm == 1 else tuple(groups[:nm])
        conv_state = caches[nm] if len(caches) > nm else None
        if stream.has_delta:
            raise RuntimeError("sandwich_norm: the stream carries a branch output that nobody added")
        extras = getattr(ctx, "extras", None)
        ahead = extras.pop("normed_ahead", None) if extras else None
        after, after_dtype = step_hint(ctx, "norm_after_block") or (None, None)
        after_dtype = after_dtype or ctx.dtype
        mark = ctx.arena.mark()
        x = stream.resid
        conv = self.conv_taps is not None
        # the mixer's input: the normed rows (float32 where the convolution reads them), then rows + convolution, rounded once
        h_dtype = torch.float32 if conv else ctx.dtype
        if ahead is not None and ahead[0] is self.norm1 and ahead[1].dtype == h_dtype:
            h = ahead[1]
        else:
            h = ctx.arena.alloc((T, W), h_dtype)
            self.norm1.add_norm(ctx, x, None, h)
        if conv:
            read = ctx.arena.alloc((T, W), ctx.dtype)
            ops.stream_conv(h, self.w_conv, conv_state, ctx, None, read, write_state=write_cache)
            h = read
        out = ctx.arena.alloc((T, W), ctx.dtype)
        self.mixer.forward(ctx, h, m_cache, m_group, out, write_cache)
        if self.ffn is None:
            left = self._way_back(ctx, self.norm1b, x, out, after, after_dtype, step_lived=True)
        else:
            h2 = self._way_back(ctx, self.norm1b, x, out, self.norm2, ctx.dtype)
            if h2 is None:
                h2 = ctx.arena.alloc((T, W), ctx.dtype)
                self.norm2.add_norm(ctx, x, None, h2)
            out2 = ctx.arena.alloc((T, W), ctx.dtype)
            self.ffn.forward(ctx, h2, out2)
            left = self._way_back(ctx, self.norm2b, x, out2, after, after_dtype, step_lived=True)
        if left is not None and extras is not None:
            extras["normed_ahead"] = (after, left)
        stream.has_delta, stream.n_ssq = False, 0
        ctx.arena.release(mark)
