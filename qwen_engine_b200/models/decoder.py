"""The generic decoder: embedding, a plan of layers, final norm, output head.

Which layers exist, what each is made of, and in which order they run is data
(``ModelLayout``), written by an architecture's layout function from its
configuration.  The plan is a list of entries; an entry names the layer to run,
the cache slot it uses, and whether it writes that slot (a layer may run twice
under two slots, or read the slot another layer wrote).  A mixer made of
several mixers names one slot for each (a tuple); an entry may also ask for
the embedding output to be added to the stream before it runs (a pass over the
same layers that starts again from the tokens).

The reference's model runs embedding, its layers in order, the final norm and
the head over every row (src/models/qwen3/model.py:347-360, 420-422); here the
final norm and the head run on the rows whose logits are wanted only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..cache.spec import CacheSpec
from ..parts.base import Block, PartSpec, StepContext
from ..weights.loader import check_against_manifest
from ..weights.spec import MATRIX, TensorSource, WeightSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement with which parameters, and the prefix
    of its tensors in the checkpoint."""

    block: PartSpec
    weight_prefix: str


@dataclass(frozen=True)
class PlanEntry:
    layer: int                  # index into ModelLayout.layers
    cache_slot: object          # which cache slot this run uses (None: the mixer keeps nothing; a tuple: one per
                                # cache description of a mixer that has several, in the order of its cache_specs())
    write_cache: bool = True    # False: read what another entry wrote into the slot
    add_embedding: bool = False  # the embedding output (token rows x the model's scale) is added to the stream first

    @property
    def slots(self) -> tuple:
        if self.cache_slot is None:
            return ()
        return tuple(self.cache_slot) if isinstance(self.cache_slot, (tuple, list)) else (self.cache_slot,)


@dataclass(frozen=True)
class ModelLayout:
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    plan: tuple[PlanEntry, ...]
    final_norm: PartSpec
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: Optional[str] = "lm_head.weight"      # None: the model has no head tensor (the embedding table serves)
    tie_head: bool = True
    max_positions: Optional[int] = None
    embed_scale: float = 1.0    # the embedding output is the table's row times this (the head uses the table as it is)
    embed_norm: Optional[PartSpec] = None         # a norm that the embedding output passes before the first layer ...
    embed_norm_prefix: str = "embed.norm"         # ... and the prefix of its tensors
    layer_history: bool = False                   # a step keeps the embedding output and every layer run's result (blocks
                                                  # that read earlier layers' results find them in ctx.extras)


@dataclass
class LayerHistory:
    """The results of a step's layer runs so far, for arrangements that read them again: ``results`` float32
    [runs + 1, T, H] (entry 0 is the embedding output, entry i + 1 the result of run i, written by its block),
    ``run`` the index of the run in progress, ``mixed`` a float32 [T, H] buffer for what goes on to the next run."""

    results: torch.Tensor
    mixed: torch.Tensor
    run: int = 0


class DecoderModel:
    def __init__(self, layout: ModelLayout):
        self.layout = layout
        self.blocks: list[Block] = [ls.block.build("block") for ls in layout.layers]
        self.final_norm = layout.final_norm.build("norm")
        self.embed_norm = layout.embed_norm.build("norm") if layout.embed_norm is not None else None
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.device = None
        n_slots = 1 + max((s for e in layout.plan for s in e.slots), default=-1)
        specs: list[Optional[CacheSpec]] = [None] * n_slots
        writers = [0] * n_slots
        for e in layout.plan:
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"plan names layer {e.layer}, the model has {len(self.blocks)}")
            if not e.slots:
                continue
            needs = self.blocks[e.layer].cache_specs()
            if len(needs) != len(e.slots):
                raise ValueError(f"plan gives layer {e.layer} {len(e.slots)} cache slot(s) but it keeps {len(needs)} cache(s)")
            for slot, spec in zip(e.slots, needs):
                if specs[slot] is not None and specs[slot] != spec:
                    raise ValueError(f"cache slot {slot} is used by layers with different needs")
                specs[slot] = spec
                writers[slot] += int(e.write_cache)
        for slot, n in enumerate(writers):
            if specs[slot] is not None and n != 1:
                raise ValueError(f"cache slot {slot} must be written by exactly one plan entry, not {n}")
        self._cache_specs = specs
        geos = []
        for b in self.blocks:
            for geo in b.mixer.attention_geometries():
                if geo not in geos:
                    geos.append(geo)
        self.attention_geometries = tuple(geos)
        self.capturable = all(getattr(b, "capturable", True) and getattr(b.mixer, "capturable", True) for b in self.blocks)

    # ---- what the cache manager and the loader ask --------------------------------------
    def cache_specs(self) -> list[Optional[CacheSpec]]:
        return list(self._cache_specs)

    def weight_manifest(self) -> list[WeightSpec]:
        lo = self.layout
        specs = [WeightSpec(lo.embed_name, (lo.vocab_size, lo.hidden_size), MATRIX)]
        if self.embed_norm is not None:
            specs += self.embed_norm.weight_specs(lo.embed_norm_prefix)
        for ls, block in zip(lo.layers, self.blocks):
            specs += block.weight_specs(ls.weight_prefix)
        specs += self.final_norm.weight_specs(lo.final_norm_prefix)
        if lo.head_name is not None:
            specs.append(WeightSpec(lo.head_name, (lo.vocab_size, lo.hidden_size), MATRIX,
                                    optional=lo.tie_head))
        elif not lo.tie_head:
            raise ValueError("a model without a head tensor must tie its head to the embedding")
        return specs

    def load_weights(self, source: TensorSource, dtype: torch.dtype, device, where: str = "checkpoint") -> None:
        check_against_manifest(source, self.weight_manifest(), where)
        lo = self.layout
        self.dtype, self.device = dtype, torch.device(device)
        self.embed = ops.prepare_matrix(source.get(lo.embed_name).to(dtype).to(device))
        for ls, block in zip(lo.layers, self.blocks):
            block.load(ls.weight_prefix, source, dtype, device)
        self.final_norm.load(lo.final_norm_prefix, source, dtype, device)
        if self.embed_norm is not None:
            self.embed_norm.load(lo.embed_norm_prefix, source, dtype, device)
        if lo.tie_head:
            self.head = self.embed            # the same storage (model.py:417-418)
            if lo.head_name is not None and lo.head_name in set(source.names()):
                # the reference lets such a tensor overwrite the shared storage (whichever of the two is read
                # last wins); here the embedding is the one that counts, and the user is told
                import warnings
                warnings.warn(f"{where}: the model ties its output head to the embedding; the stored "
                              f"{lo.head_name!r} is not used", stacklevel=2)
        else:
            self.head = ops.prepare_matrix(source.get(lo.head_name).to(dtype).to(device))

    def weight_bytes(self) -> int:
        """Bytes of every weight a decode step reads once (a tied head counts once)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_floating_point():
                    key = v.untyped_storage().data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += v.numel() * v.element_size()
                elif hasattr(v, "weight_specs"):
                    visit(v)
        total += self.embed.numel() * self.embed.element_size()
        seen.add(self.embed.untyped_storage().data_ptr())
        if self.head is not None and self.head.untyped_storage().data_ptr() not in seen:
            total += self.head.numel() * self.head.element_size()
        for b in self.blocks:
            visit(b)
        visit(self.final_norm)
        if self.embed_norm is not None:
            visit(self.embed_norm)
        return total

    # ---- one step ---------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache: CacheManager) -> Optional[torch.Tensor]:
        """Run the tokens of ``ctx`` through the plan; float32 logits
        [num_logit_rows, vocab] (None when no logits are wanted)."""
        lo = self.layout
        T, H = ctx.num_tokens, lo.hidden_size
        stream = ops.ResidualStream.for_step(ctx.arena.alloc, T, H, ctx.dtype)
        history = None
        if lo.layer_history:
            # the stream starts as entry 0 of the runs' results; a block that mixes them hands on ``mixed``
            history = LayerHistory(ctx.arena.alloc_step((len(lo.plan) + 1, T, H), torch.float32),
                                   ctx.arena.alloc_step((T, H), torch.float32))
            stream.resid, stream.ssq = history.results[0], None
            ctx.extras["layer_history"] = history
        if self.embed_norm is None:
            ops.embedding(ctx.token_ids, self.embed, stream, scale=lo.embed_scale)
        else:
            # the table's rows, normed in float32, are what the stream starts from
            rows = ctx.arena.alloc((T, H), torch.float32)
            ops.embedding(ctx.token_ids, self.embed, rows, scale=lo.embed_scale)
            self.embed_norm.add_norm(ctx, rows, None, stream.resid)
            stream.has_delta, stream.n_ssq = False, 0
        views = []
        for e in lo.plan:
            if not e.slots:
                views.append((None, None))
            elif isinstance(e.cache_slot, (tuple, list)):
                views.append((tuple(cache.layer_view(s) for s in e.slots), tuple(cache.group_of_slot[s][0] for s in e.slots)))
            else:
                views.append((cache.layer_view(e.cache_slot), cache.group_of_slot[e.cache_slot][0]))
        for i, entry in enumerate(lo.plan):
            view, group = views[i]
            # a hint for mixers that can ask for it ahead of time: the cache that the next entry of the plan
            # with a cache of the same group will read (the same pages at the same places)
            ctx.extras["next_cache"] = None if isinstance(view, tuple) else next(
                (v for v, g in views[i + 1:] if v is not None and not isinstance(v, tuple) and g == group and v is not view), None)
            if entry.add_embedding:
                # a pass that starts again from the tokens: the rows of the table, scaled, are added to the stream
                ops.embedding(ctx.token_ids, self.embed, stream, scale=lo.embed_scale, accumulate=True)
            # and the weights that the step reads first after this block
            nxt = lo.plan[i + 1].layer if i + 1 < len(lo.plan) else None
            ctx.extras["weights_after_ffn"] = self.blocks[nxt].first_weights() if nxt is not None else None
            # and the norm that reads the stream first after this block, where the next block names it
            ctx.extras["norm_after_block"] = self.blocks[nxt].first_norm() if nxt is not None else None
            if history is not None:
                history.run = i
            self.blocks[entry.layer].forward(ctx, stream, view, group, entry.write_cache)
        ctx.extras["next_cache"] = ctx.extras["weights_after_ffn"] = ctx.extras["norm_after_block"] = None
        if ctx.num_logit_rows == 0:
            return None
        N = ctx.num_logit_rows
        normed = ctx.arena.alloc((N, H), ctx.dtype)
        self.final_norm.add_norm_rows(ctx, stream.resid, stream.delta if stream.has_delta else None,
                                      ctx.logit_rows, normed)
        logits = ctx.arena.alloc((N, lo.vocab_size), torch.float32)
        ops.linear(normed, self.head, logits)
        return logits
