"""Grouped-query attention over the paged cache.

q, k, v projections (one product over the stacked weights), per-head RMS norm
of q and k, position encoding, write of k and v into the request's pages,
attention of the new queries over all keys of the request that the mask
allows, output projection (reference src/models/qwen3/model.py:200-213).
Query head h reads key/value head h // (heads / kv_heads)
(src/layers/fused_ops/attn.py:181-182); key j is allowed for the query at
position i iff j <= i (attn.py:195, 239) and, with a window w, j > i - w.

Options that other designs use (all off for Qwen3):

* ``value_dim``: values of another size than keys.  The smaller of the two is
  padded with zero channels up to the larger when the weights are loaded
  (zero rows of W_q, W_k or W_v, zero columns of W_o), so the cache and the
  kernels see one head size; the q/k norm's mean runs over the real channels.
* ``distance_slopes``: one slope per query head; slope * (i - j) is taken off
  the score of query i and key j before the softmax.
* ``output_gate`` = "sigmoid": the joined heads are multiplied by
  sigmoid(W_g x) before the output projection; W_g rides in the stacked product.
* no position encoding at all (``position_encoding`` None).
* ``tied_values``: there is no W_v; the values are the keys as projected (with their bias, before their
  norm).  The cache's value plane takes the projected keys and its key plane the normed ones, so the
  attention kernels see an ordinary cache.  Comes with ``qk_bias`` (biases of the q and k projections),
  a q/k norm without weights (``qk_norm_eps`` is its eps), and
  ``query_temperature`` = (coef, every): the query at position p is multiplied by
  1 + coef ln(floor((p + 1) / every) + 1).
* ``names``: the tensors' names in the checkpoint.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import PagedKVSpec
from ..weights.spec import MATRIX, NORM, VECTOR, WeightSpec
from .base import Mixer, PartSpec, StepContext, register, step_hint

_NAMES = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", out="o_proj.weight",
              q_norm="q_norm.weight", k_norm="k_norm.weight", gate="g_proj.weight",
              q_bias="q_proj.bias", k_bias="k_proj.bias")


def _pad_rows(w: torch.Tensor, heads: int, dim: int, padded: int) -> torch.Tensor:
    """[heads * dim, W] -> [heads * padded, W] with zero rows after each head's own."""
    if dim == padded:
        return w
    out = w.new_zeros((heads, padded, w.shape[1]))
    out[:, :dim] = w.reshape(heads, dim, w.shape[1])
    return out.reshape(heads * padded, w.shape[1])


@register("mixer", "gqa_attention")
class GQAAttention(Mixer):
    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, qk_norm_eps: Optional[float] = None,
                 position_encoding: Optional[PartSpec] = None, window: Optional[int] = None,
                 value_dim: Optional[int] = None, distance_slopes=None, output_gate: Optional[str] = None,
                 names: Optional[dict] = None, tied_values: bool = False, qk_bias: bool = False,
                 query_temperature=None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if output_gate not in (None, "sigmoid"):
            raise ValueError(f"unknown output gate {output_gate!r}")
        if distance_slopes is not None and len(distance_slopes) != num_heads:
            raise ValueError("one distance slope per query head")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.pos = position_encoding.build("position_encoding") if position_encoding else None
        self.key_dim = head_dim                              # the checkpoint's sizes
        self.value_dim = value_dim if value_dim is not None else head_dim
        self.head_dim = max(self.key_dim, self.value_dim)    # what the cache and the kernels see
        self.q_width = num_heads * self.head_dim
        self.kv_width = num_kv_heads * self.head_dim
        self.output_gate = output_gate
        self.tied_values = bool(tied_values)
        self.qk_bias = bool(qk_bias)
        self.query_temperature = None if query_temperature is None else (float(query_temperature[0]), int(query_temperature[1]))
        if self.tied_values:
            if self.value_dim != self.key_dim or self.pos is not None or distance_slopes is not None or window:
                raise ValueError("values that are the keys: one head size, no rotation, no distance bias, no window")
            if qk_norm_eps is None:
                raise ValueError("values that are the keys: the q/k norm's eps is needed")
        elif self.qk_bias or self.query_temperature is not None:
            raise ValueError("q/k biases and a query temperature come with values that are the keys")
        self.distance_slopes = None if distance_slopes is None else tuple(float(x) for x in distance_slopes)
        self.names = dict(_NAMES, **(names or {}))
        # the step takes the route of separate operations (one stacked product, norm and cache write, attention, gate,
        # output product) when any of the options above is on
        self.extended = bool(output_gate or self.distance_slopes is not None or self.value_dim != self.key_dim or self.tied_values)
        self.inner_width = self.q_width
        self.input_width = self.q_width + (1 if self.tied_values else 2) * self.kv_width + (self.q_width if output_gate else 0)
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = self.slopes = self.q_bias = self.k_bias = None

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def attention_geometry(self):
        geo = (self.num_heads, self.num_kv_heads, self.head_dim, self.window or 0)
        return geo + (True,) if self.distance_slopes is not None else geo

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        n, H, G, W = self.names, self.num_heads, self.num_kv_heads, self.hidden_size
        specs = [
            WeightSpec(prefix + n["q"], (H * self.key_dim, W), MATRIX),
            WeightSpec(prefix + n["k"], (G * self.key_dim, W), MATRIX),
        ]
        if not self.tied_values:
            specs.append(WeightSpec(prefix + n["v"], (G * self.value_dim, W), MATRIX))
        specs.append(WeightSpec(prefix + n["out"], (W, H * self.value_dim), MATRIX))
        if self.output_gate:
            specs.append(WeightSpec(prefix + n["gate"], (H * self.value_dim, W), MATRIX))
        if self.qk_bias:
            specs += [WeightSpec(prefix + n["q_bias"], (H * self.key_dim,), VECTOR),
                      WeightSpec(prefix + n["k_bias"], (G * self.key_dim,), VECTOR)]
        if self.qk_norm_eps is not None and not self.tied_values:
            specs += [WeightSpec(prefix + n["q_norm"], (self.key_dim,), NORM),
                      WeightSpec(prefix + n["k_norm"], (self.key_dim,), NORM)]
        if self.pos is not None:
            specs += self.pos.weight_specs(prefix)
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        n, H, G, D = self.names, self.num_heads, self.num_kv_heads, self.head_dim
        # q, k and v rows stacked (and the gate's behind them): one product gives [T, q_width + 2 kv_width (+ q_width)]
        rows = [_pad_rows(source.get(prefix + n["q"]), H, self.key_dim, D),
                _pad_rows(source.get(prefix + n["k"]), G, self.key_dim, D)]
        if not self.tied_values:
            rows.append(_pad_rows(source.get(prefix + n["v"]), G, self.value_dim, D))
        if self.output_gate:
            rows.append(_pad_rows(source.get(prefix + n["gate"]), H, self.value_dim, D))
        self.w_qkv = ops.prepare_matrix(torch.cat(rows, dim=0).to(dtype).to(device))
        w_o = source.get(prefix + n["out"])
        if self.value_dim != D:                      # zero columns where the attention's output is padding
            w_o = _pad_rows(w_o.t().contiguous(), H, self.value_dim, D).t()
        self.w_o = ops.prepare_matrix(w_o.to(dtype).to(device))
        if self.qk_bias:
            self.q_bias = source.get(prefix + n["q_bias"]).to(torch.float32).to(device).contiguous()
            self.k_bias = source.get(prefix + n["k_bias"]).to(torch.float32).to(device).contiguous()
        if self.qk_norm_eps is not None and not self.tied_values:
            def norm_weight(name):
                w = source.get(prefix + name).to(torch.float32)
                return torch.nn.functional.pad(w, (0, D - self.key_dim)).to(device).contiguous()
            self.q_norm_w, self.k_norm_w = norm_weight(n["q_norm"]), norm_weight(n["k_norm"])
        if self.distance_slopes is not None:
            self.slopes = torch.tensor(self.distance_slopes, dtype=torch.float32).to(device)
        if self.pos is not None:
            self.pos.load(prefix, source, dtype, device)

    def first_weights(self):
        return self.w_qkv

    def output_weight(self):
        return self.w_o

    def input_weight(self):
        return self.w_qkv

    def mix_into(self, ctx: StepContext, x, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        """Everything before the output projection, as separate operations; serves every option."""
        proj = ctx.arena.alloc((ctx.num_tokens, self.input_width), ctx.dtype)
        ops.linear(x, self.w_qkv, proj)
        self.mix_projected(ctx, proj, cache, group, inner, write_cache, scale)

    def mix_projected(self, ctx: StepContext, proj, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        T = ctx.num_tokens
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        view = ctx.groups[group]
        if self.tied_values:
            # q and k lead the rows; the cache's value plane gets the keys as projected, its key plane the normed ones
            n_qk = self.q_width + self.kv_width
            ops.qk_bias_norm_kv_write(proj, ctx.positions, self.q_bias, self.k_bias, self.qk_norm_eps, self.query_temperature,
                                      cache, view.slot_mapping, H, Hkv, D, write_kv=write_cache)
            attn = ctx.arena.alloc((T, self.q_width), ctx.dtype) if (self.output_gate or scale != 1.0 or not inner.is_contiguous()) else inner
            ops.paged_attention(proj, cache, view.block_tables, ctx, attn, self.scale, 0, H, Hkv, D)
            if attn is not inner:
                ops.head_norm_gate(attn, proj[:, n_qk:n_qk + self.q_width] if self.output_gate else None, None, 0.0, inner, H, D,
                                   gate_kind=self.output_gate, scale=scale)
            return
        n_qkv = self.q_width + 2 * self.kv_width
        qkv = proj[:, :n_qkv]
        if self.pos is not None:
            # norm, then the part's own rotation, then the plain cache write (the order of model.py:204-208)
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0, None, 0,
                                      cache, view.slot_mapping, H, Hkv, D, write_kv=False, norm_dim=self.key_dim)
            self.pos.rotate(ctx, qkv[:, :self.q_width].unflatten(1, (H, D)),
                            qkv[:, self.q_width:self.q_width + self.kv_width].unflatten(1, (Hkv, D)))
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, None, None, 0.0, None, 0, cache, view.slot_mapping,
                                      H, Hkv, D, write_kv=write_cache)
        else:
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0, None, 0,
                                      cache, view.slot_mapping, H, Hkv, D, write_kv=write_cache, norm_dim=self.key_dim)
        gated = bool(self.output_gate) or scale != 1.0
        attn = ctx.arena.alloc((T, self.q_width), ctx.dtype) if gated or not inner.is_contiguous() else inner
        ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale, self.window or 0, H, Hkv, D,
                            slopes=self.slopes)
        if attn is not inner:
            ops.head_norm_gate(attn, proj[:, n_qkv:n_qkv + self.q_width] if self.output_gate else None, None, 0.0, inner, H, D,
                               gate_kind=self.output_gate, scale=scale)

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        T = ctx.num_tokens
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        if self.extended:
            inner = ctx.arena.alloc((T, self.inner_width), ctx.dtype)
            self.mix_into(ctx, x, cache, group, inner, write_cache)
            ops.linear(inner, self.w_o, out)
            return
        view = ctx.groups[group]
        qkv = ctx.arena.alloc((T, self.q_width + 2 * self.kv_width), ctx.dtype)
        rot = self.pos.half_split_rotation() if self.pos is not None else None
        fused_rope = rot is not None
        attn = ctx.arena.alloc((T, self.q_width), ctx.dtype)
        if fused_rope and ops.qkv_rope_fused_applies(T, qkv.shape[1], self.hidden_size, ctx.dtype, D, rot.rotary_dim):
            table = rot.step_table(ctx)
            if table is not None:
                # many rows: norm, rotation and cache write happen in the epilogue of the QKV product
                if isinstance(x, ops.NormedInput):
                    x = x.materialize()
                ops.linear_qkv_rope(x, self.w_qkv, qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0, table,
                                    cache, view.slot_mapping, H, Hkv, write_kv=write_cache)
                ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale,
                                    self.window or 0, H, Hkv, D, next_pages=step_hint(ctx, "next_cache"))
                ops.linear(attn, self.w_o, out)
                return
        if fused_rope and ops.qkv_rope_small_applies(T, qkv.shape[1], self.hidden_size, ctx.dtype, D, rot.rotary_dim):
            # a few rows: the same in the epilogue of the product that streams the weights (a cluster of CTAs per head)
            ops.prefetch_next(self.w_o)
            ops.linear_qkv_rope_small(x, self.w_qkv, qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0,
                                      ctx.positions, rot.inv_freq, rot.step_table(ctx), cache, view.slot_mapping, H, Hkv,
                                      write_kv=write_cache)
            ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale,
                                self.window or 0, H, Hkv, D, next_pages=step_hint(ctx, "next_cache"))
            ops.prefetch_next(step_hint(ctx, "weights_after_mixer"))
            ops.linear(attn, self.w_o, out)
            ops.prefetch_next(None)
            return
        ops.prefetch_next(self.w_o)
        ops.linear(x, self.w_qkv, qkv)
        if self.pos is not None and not fused_rope:
            # another position encoding: norm first (the order of model.py:204-208),
            # then the part's own rotation, then the plain cache write
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, self.q_norm_w, self.k_norm_w,
                                      self.qk_norm_eps or 0.0, None, 0, cache, view.slot_mapping,
                                      H, Hkv, D, write_kv=False)
            q3 = qkv[:, :self.q_width].unflatten(1, (H, D))
            k3 = qkv[:, self.q_width:self.q_width + self.kv_width].unflatten(1, (Hkv, D))
            self.pos.rotate(ctx, q3, k3)
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, None, None, 0.0, None, 0, cache,
                                      view.slot_mapping, H, Hkv, D, write_kv=write_cache)
        else:
            ops.qk_norm_rope_kv_write(
                qkv, ctx.positions, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0,
                rot.inv_freq if fused_rope else None,
                rot.rotary_dim if fused_rope else 0,
                cache, view.slot_mapping, H, Hkv, D, write_kv=write_cache,
                cos_sin=rot.step_table(ctx) if fused_rope else None)
        ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale,
                            self.window or 0, H, Hkv, D, next_pages=step_hint(ctx, "next_cache"))
        ops.prefetch_next(step_hint(ctx, "weights_after_mixer"))
        ops.linear(attn, self.w_o, out)
        ops.prefetch_next(None)
