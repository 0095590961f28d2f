"""Rotary position encoding with half-split ("neox") pairs.

inv_freq[j] = theta^(-2j/rotary_dim); angle = position * inv_freq[j] in
float32; out = [cos*x1 - sin*x2 | sin*x1 + cos*x2] with x1, x2 the two halves of
the rotated dimensions (reference src/models/qwen3/model.py:75-84,
src/layers/ops/rope.py:37-121).  The reference keeps a float32 cos/sin table
of max_position rows in every layer; here one inv_freq vector is kept and the
angle, its cosine and its sine are computed in float32 inside the kernel that
also norms q and k and writes the cache.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding, StepContext, register


@register("position_encoding", "rope_neox")
class NeoxRope(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {head_dim}")
        # the same float32 arithmetic as model.py:77-79
        self._inv_freq_cpu = 1.0 / (self.theta ** (
            torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
        self.inv_freq: torch.Tensor | None = None

    def load(self, prefix, source, dtype, device) -> None:
        self.inv_freq = self._inv_freq_cpu.to(device).contiguous()

    def step_table(self, ctx: StepContext):
        """The cosines and sines of this step's angles [T, rotary_dim / 2, 2], computed once per step
        and shared by every layer with the same frequencies; None for small steps (the kernel then
        computes them itself) and where the fused kernel takes no table."""
        if not ops.rope_table_applies(ctx.num_tokens, ctx.dtype, self.head_dim, self.rotary_dim):
            return None
        key = ("rope_table", self.theta, self.rotary_dim)
        table = ctx.extras.get(key)
        if table is None:
            # (for the whole step: a layer's own scratch is handed to the next layer when the layer is done)
            table = ctx.arena.alloc_step((ctx.num_tokens, self.rotary_dim // 2, 2), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, table)
            ctx.extras[key] = table
        return table

    def rotate(self, ctx: StepContext, q, k) -> None:
        ops.rope_neox(q, k, ctx.positions, self.inv_freq, self.rotary_dim)

    def half_split_rotation(self):
        return self


def banded_frequencies(inv_freq: torch.Tensor, factor: float, low: float, high: float, original: int) -> torch.Tensor:
    """Frequencies scaled by wavelength bands (float64 in, float64 out): with l = 2 pi / f, f stays where
    l < original / high, becomes f / factor where l > original / low, and between the two is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    f = inv_freq.to(torch.float64)
    wavelength = 2.0 * math.pi / f
    blend = (original / wavelength - low) / (high - low)
    mixed = (1.0 - blend) * f / factor + blend * f
    return torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, mixed))


def ramped_frequencies(inv_freq: torch.Tensor, base: float, rotary_dim: int, factor: float, original: int, fast: float,
                       slow: float) -> torch.Tensor:
    """Frequencies blended along a ramp over the pair index i (float64): with index(t) = rotary_dim ln(original /
    (2 pi t)) / (2 ln base), lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), rotary_dim - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is f_i / factor * r_i + f_i (1 - r_i)."""
    f = inv_freq.to(torch.float64)

    def index_of(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), rotary_dim - 1)
    ramp = ((torch.arange(f.numel(), dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp)


@register("position_encoding", "rope_scaled")
class ScaledRope(NeoxRope):
    """Rotation of the first ``rotary_dim`` channels of a head with scaled frequencies.

    ``scaling``: None, or ("bands", factor, low, high, original) (``banded_frequencies``), or ("ramp", factor, original,
    fast, slow) (``ramped_frequencies``, with which cosines and sines are also multiplied by 0.1 ln(factor) + 1).
    ``pairing``: "half" pairs channel i with i + rotary_dim / 2; "interleaved" pairs 2 i with 2 i + 1.  The kernels
    rotate half-split pairs; for interleaved pairs the mixer reorders the rows of W_q and W_k within every head when it
    loads them (``row_permutation``), which leaves every q.k as it was.  Frequencies are formed in float64 and rounded
    once; angles, cosines and sines are float32."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, scaling=None, pairing: str = "half"):
        super().__init__(head_dim, theta, rotary_dim)
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown pairing {pairing!r}")
        self.pairing, self.scaling = pairing, None if scaling is None else tuple(scaling)
        self.magnitude = 1.0
        base = torch.tensor([self.theta ** (-2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)], dtype=torch.float64)
        if self.scaling is None:
            f = base
        elif self.scaling[0] == "bands":
            _, factor, low, high, original = self.scaling
            f = banded_frequencies(base, float(factor), float(low), float(high), original)
        elif self.scaling[0] == "ramp":
            _, factor, original, fast, slow = self.scaling
            f = ramped_frequencies(base, self.theta, self.rotary_dim, float(factor), original, float(fast), float(slow))
            self.magnitude = 0.1 * math.log(float(factor)) + 1.0
        else:
            raise ValueError(f"unknown frequency scaling {self.scaling[0]!r}")
        self._inv_freq_cpu = f.to(torch.float32)

    def step_table(self, ctx: StepContext):
        return None           # (the table of a step's angles serves whole heads of 128 channels without a magnitude)

    def row_permutation(self):
        """None, or the order in which a head's rows of W_q and W_k are to be stacked so that the kernels' half-split
        rotation is the design's: new row i is old row 2 i, new row i + rotary_dim / 2 is old row 2 i + 1."""
        if self.pairing == "half":
            return None
        half = self.rotary_dim // 2
        return [2 * i for i in range(half)] + [2 * i + 1 for i in range(half)] + list(range(self.rotary_dim, self.head_dim))

    def rotate(self, ctx: StepContext, q, k) -> None:
        raise NotImplementedError("rope_scaled rotates inside the kernel that writes the cache")
