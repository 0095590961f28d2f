"""RMS norm over the width of the residual stream, with the add of the
previous branch fused in.

y = x * rsqrt(mean(x^2) + eps) * w, all in float32
(reference src/layers/ops/layernorm.py:50-88).  The reference adds residuals
with a separate ``+`` in the model's dtype (src/models/qwen3/model.py:291, 296);
here the stream is float32 and the add happens inside the norm kernel.

``weight_offset``: a design may store the scale around zero and multiply by
(offset + w); the sum is formed once, in float32, when the weights are loaded.
``output_scale``: a constant that multiplies the normed rows (a model's scale of
its logits, on the final norm), folded into the weight in float32 at load.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights.spec import NORM, NORM_ZERO, WeightSpec
from .base import Norm, StepContext, register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str = "weight", weight_offset: float = 0.0,
                 output_scale: float = 1.0):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight_offset = float(weight_offset)
        self.output_scale = float(output_scale)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        return [WeightSpec(prefix + self.weight_name, (self.width,), NORM_ZERO if self.weight_offset else NORM)]

    def load(self, prefix, source, dtype, device) -> None:
        # scale vectors are float32 on the device whatever the compute dtype
        w = source.get(prefix + self.weight_name).to(torch.float32)
        if self.weight_offset:
            w = w + self.weight_offset
        if self.output_scale != 1.0:
            w = w * self.output_scale
        self.weight = w.to(device).contiguous()

    def normed(self, ctx: StepContext, stream, lazy: bool = False):
        x = ops.NormedInput(stream, self.weight, self.eps, ctx.arena.alloc, ctx.dtype)
        return x if lazy else x.materialize()

    def add_norm(self, ctx: StepContext, resid, delta, out):
        ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)
        return out

    def add_norm_rows(self, ctx: StepContext, resid, delta, rows, out):
        ops.add_rmsnorm_rows(resid, delta, rows, self.weight, self.eps, out)
        return out

    def norm_add(self, ctx: StepContext, src, branch, dst, gate=None, gate_bias=None, cast=None) -> None:
        ops.gated_norm_add(src, branch, gate, gate_bias, self.weight, self.eps, dst, cast)


@register("norm", "group_rmsnorm")
class GroupRMSNorm(Norm):
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, every part is divided by its own
    sqrt(mean(part^2) + eps), and the whole row is multiplied by the weight vector.  One group is the plain RMS norm.
    ``output_scale`` multiplies the normed rows (a block's multiplier on what its sublayers return); it is folded
    into the weight in float32 at load."""

    def __init__(self, width: int, eps: float, groups: int = 1, weight_name: str = "weight", output_scale: float = 1.0):
        if groups < 1 or width % groups:
            raise ValueError(f"a width of {width} does not split into {groups} equal parts")
        self.width, self.eps, self.groups = width, float(eps), int(groups)
        self.weight_name, self.output_scale = weight_name, float(output_scale)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        return [WeightSpec(prefix + self.weight_name, (self.width,), NORM)]

    def load(self, prefix, source, dtype, device) -> None:
        w = source.get(prefix + self.weight_name).to(torch.float32)
        if self.output_scale != 1.0:
            w = w * self.output_scale
        self.weight = w.to(device).contiguous()

    def normed(self, ctx: StepContext, stream, lazy: bool = False):
        out = ctx.arena.alloc(tuple(stream.resid.shape), ctx.dtype)
        self.add_norm(ctx, stream.resid, stream.delta if stream.has_delta else None, out)
        if stream.has_delta:
            stream.has_delta, stream.n_ssq = False, 0
        return out

    def add_norm(self, ctx: StepContext, resid, delta, out):
        """``out`` may be float32 (for a reader that works on the normed rows in float32) or the compute type."""
        if delta is not None:
            ops.scaled_add(resid, delta, 1.0)
        ops.group_rmsnorm(resid, None, self.weight, self.eps, self.groups, out)
        return out

    def add_norm_rows(self, ctx: StepContext, resid, delta, rows, out):
        if delta is not None:
            raise NotImplementedError("group_rmsnorm: chosen rows of a stream with a pending branch output")
        ops.group_rmsnorm(resid, rows, self.weight, self.eps, self.groups, out)
        return out

    def fuses_with(self, other) -> bool:
        """Whether ``other``'s norm of the stream can ride in this norm's add (one pass over the row)."""
        return isinstance(other, GroupRMSNorm) and (other.width, other.eps, other.groups) == (self.width, self.eps, self.groups)

    def norm_add(self, ctx: StepContext, src, branch, dst, gate=None, gate_bias=None, cast=None, next_norm=None,
                 next_out=None) -> None:
        """dst = src + norm(branch); with ``next_norm`` (see ``fuses_with``) and ``next_out``, next_out = next_norm(dst)
        in the same pass."""
        if gate is not None or cast is not None:
            raise NotImplementedError("group_rmsnorm: no gate and no rounded copy on a sublayer's way back")
        if next_out is not None and not self.fuses_with(next_norm):
            raise ValueError("group_rmsnorm: the following norm does not fit this one's pass")
        ops.group_norm_add(src, branch, self.weight, self.eps, self.groups, dst,
                           next_norm.weight if next_out is not None else None, next_out)
