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
* ``softcap``: the scaled score s becomes softcap * tanh(s / softcap) before the mask and the softmax.
* ``sink``: one stored number per query head; exp(sink_h) joins head h's softmax denominator.  It has no key and no
  value, is not scaled and counts once.
* ``head_mixing``: a stored matrix M [H, H]; head h's attention weights become sum_g M[h, g] weights_g (after the
  softmax, sink included in the denominators) and meet the values of h's own kv head.  The sum over keys is linear, so
  the attention kernel runs once per kv-head shift and ``ops.head_mix_gate`` forms the sums over g.
* ``output_gate`` = "sigmoid_head": every head's output is multiplied by sigmoid(W_g x)_h, one number per head; W_g [H,
  hidden] rides in the stacked product.
* ``value_mix``: values shared across layers.  "keep": this layer's values of the step's tokens are kept for the layers
  after it (``ctx.extras["shared_values"]``); "blend": v <- (1 - lam) v + lam v_kept with the stored scalar lam, and
  the blended v is what is cached.  The kept values are as projected (the keeping layer blends nothing).
* a position encoding with ``row_permutation()`` (pairs that the kernels do not rotate as stored): the rows of W_q
  and W_k are reordered within every head at load; ``magnitude`` multiplies its cosines and sines.
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
              q_bias="q_proj.bias", k_bias="k_proj.bias", sink="sinks", head_mix="head_mix", value_mix="value_mix")


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
                 query_temperature=None, softcap: Optional[float] = None, sink: bool = False, head_mixing: bool = False,
                 value_mix: Optional[str] = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if output_gate not in (None, "sigmoid", "sigmoid_head"):
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
        if value_mix not in (None, "keep", "blend"):
            raise ValueError(f"unknown value_mix {value_mix!r}")
        self.softcap = None if not softcap else float(softcap)
        self.sink, self.head_mixing, self.value_mix = bool(sink), bool(head_mixing), value_mix
        self.per_head = bool(self.softcap or self.sink or self.head_mixing or value_mix or output_gate == "sigmoid_head"
                             or getattr(self.pos, "row_permutation", None) is not None)
        if self.per_head and (self.tied_values or self.distance_slopes is not None or window or qk_norm_eps is not None):
            raise ValueError("bent scores, sinks, mixed heads, shared values and a gate per head go without a window, a distance "
                             "bias, a q/k norm or tied values")
        if self.per_head and output_gate == "sigmoid":
            raise ValueError("with these options the output gate is one number per head ('sigmoid_head') or absent")
        if self.per_head and self.pos is not None and self.pos.half_split_rotation() is None:
            raise ValueError("these options rotate q and k inside the kernel that writes the cache")
        self.gate_width = 0
        if output_gate == "sigmoid_head":
            self.gate_width = -(-num_heads // 8) * 8        # padded with zero rows, so that the stacked product's rows stay aligned
        self.sinks = self.head_mix = self.mix_lambda = None
        # the step takes the route of separate operations (one stacked product, norm and cache write, attention, gate,
        # output product) when any of the options above is on
        self.extended = bool(output_gate or self.distance_slopes is not None or self.value_dim != self.key_dim or self.tied_values
                             or self.per_head)
        self.inner_width = self.q_width
        self.input_width = (self.q_width + (1 if self.tied_values else 2) * self.kv_width
                            + (self.gate_width if output_gate == "sigmoid_head" else self.q_width if output_gate else 0))
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
        if self.output_gate == "sigmoid_head":
            specs.append(WeightSpec(prefix + n["gate"], (H, W), MATRIX))
        elif self.output_gate:
            specs.append(WeightSpec(prefix + n["gate"], (H * self.value_dim, W), MATRIX))
        if self.sink:
            specs.append(WeightSpec(prefix + n["sink"], (H,), VECTOR))
        if self.head_mixing:
            specs.append(WeightSpec(prefix + n["head_mix"], (H, H), MATRIX))
        if self.value_mix:
            # (the keeping layer's scalar is stored and not used)
            specs.append(WeightSpec(prefix + n["value_mix"], (), VECTOR, optional=self.value_mix == "keep"))
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
        perm = getattr(self.pos, "row_permutation", lambda: None)() if self.pos is not None else None

        def qk_rows(name, heads):
            w = source.get(prefix + name)
            if perm is not None:                     # the same reordering of q's and k's channels leaves every q.k as it was
                w = w.reshape(heads, self.key_dim, w.shape[1])[:, perm].reshape(heads * self.key_dim, w.shape[1])
            return _pad_rows(w, heads, self.key_dim, D)

        rows = [qk_rows(n["q"], H), qk_rows(n["k"], G)]
        if not self.tied_values:
            rows.append(_pad_rows(source.get(prefix + n["v"]), G, self.value_dim, D))
        if self.output_gate == "sigmoid_head":
            w_g = source.get(prefix + n["gate"])
            rows.append(torch.cat([w_g, w_g.new_zeros((self.gate_width - H, w_g.shape[1]))], dim=0))
        elif self.output_gate:
            rows.append(_pad_rows(source.get(prefix + n["gate"]), H, self.value_dim, D))
        if self.sink:
            self.sinks = source.get(prefix + n["sink"]).to(torch.float32).to(device).contiguous()
        if self.head_mixing:
            self.head_mix = source.get(prefix + n["head_mix"]).to(torch.float32).to(device).contiguous()
        if self.value_mix == "blend":
            self.mix_lambda = float(source.get(prefix + n["value_mix"]).to(torch.float32))
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
        if self.per_head:
            self._mix_per_head(ctx, proj, qkv, cache, view, inner, write_cache, scale)
            return
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

    def _mix_per_head(self, ctx: StepContext, proj, qkv, cache, view, inner, write_cache: bool, scale: float) -> None:
        """Rotation (inside the kernel that blends and writes the cache), attention with bent scores or a sink, the heads'
        weights mixed, a gate per head."""
        T = ctx.num_tokens
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        if scale != 1.0:
            raise NotImplementedError("gqa_attention: no output scale with these options")
        shared = None
        if self.value_mix:
            first = step_hint(ctx, "shared_values")
            if self.value_mix == "keep":
                first = ctx.arena.alloc_step((T, Hkv * self.value_dim), ctx.dtype)     # (the heads' own channels: layers pad differently)
                ctx.extras["shared_values"] = first
                shared = ("keep", first)
            else:
                if first is None or first.shape != (T, Hkv * self.value_dim):
                    raise RuntimeError("gqa_attention: values to blend with, but no layer before this one kept its own")
                shared = ("blend", first, self.mix_lambda)
        rot = self.pos.half_split_rotation() if self.pos is not None else None
        ops.qk_norm_rope_kv_write(qkv, ctx.positions, None, None, 0.0, rot.inv_freq if rot is not None else None,
                                  rot.rotary_dim if rot is not None else 0, cache, view.slot_mapping, H, Hkv, D,
                                  write_kv=write_cache, magnitude=getattr(rot, "magnitude", 1.0) if rot is not None else 1.0,
                                  value_mix=shared)
        shifts = Hkv if self.head_mixing else 1
        gate = proj[:, self.q_width + 2 * self.kv_width:self.q_width + 2 * self.kv_width + H] if self.output_gate else None
        direct = shifts == 1 and gate is None and inner.is_contiguous()
        partial = inner.unsqueeze(0) if direct else ctx.arena.alloc((shifts, T, self.q_width), ctx.dtype)
        if shifts > 1:
            ops.paged_attention(qkv, cache, view.block_tables, ctx, partial, self.scale, 0, H, Hkv, D,
                                softcap=self.softcap or 0.0, sinks=self.sinks, value_shifts=shifts)
        else:
            ops.paged_attention(qkv, cache, view.block_tables, ctx, partial[0], self.scale, 0, H, Hkv, D,
                                softcap=self.softcap or 0.0, sinks=self.sinks)
        if not direct:
            ops.head_mix_gate(partial, self.head_mix, gate, inner, H, Hkv, D)

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
