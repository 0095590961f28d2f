"""Merudra as a layout of parts.

Layers in the order config.json gives, each a ``gated_post_norm`` block (the
sublayers read the stream through a short causal convolution, their results are
gated, normed and added; a gated row of a second embedding table is added per
layer; what goes on is a weighted sum of all layers' results so far) with one of
two mixers: ``attention`` (softmax attention without rotation whose values are
the keys as projected, biased projections, weightless q/k norm, a query
temperature that grows with the position, a sigmoid output gate) and ``delta``
(the gated delta rule with one decay per head behind short convolutions, a silu
output gate); the feed-forward is absent or a mixture of routed experts scored
by a softmax over all of them, some of which hand their input on.

Tensor names: ``embed``, ``side.embed``, ``final.norm``, ``head``, and per layer
``l<i>.norm1/2``, ``l<i>.canon1/2``, ``l<i>.rg1/2`` (+ ``.b``), ``l<i>.dwa``,
``l<i>.side.gate/proj/norm``, ``l<i>.mix.*``, ``l<i>.mlp.*`` (experts
``l<i>.mlp.e<j>.*``).
"""
from __future__ import annotations

from ..config.merudra_config import MerudraConfig
from ..parts.base import PartSpec
from .decoder import LayerSpec, ModelLayout, PlanEntry


def _mixer(cfg: MerudraConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "attention":
        temp = m.get("q_temp")
        return PartSpec("gqa_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], scale=m["scale"],
            qk_norm_eps=cfg.norm_eps, position_encoding=None, output_gate="sigmoid", tied_values=True, qk_bias=True,
            query_temperature=None if temp is None else (temp["coef"], temp["every"]),
            names=dict(q="q", k="k", gate="g", out="o", q_bias="q.b", k_bias="k.b")))
    return PartSpec("gated_delta_rule", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_key_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
        conv_taps=m["conv"], norm_eps=cfg.norm_eps, low_rank=None, decay_per="head", gate_form="silu",
        names=dict(decay_in="a", gate="g")))


def _feed_forward(cfg: MerudraConfig, mlp):
    if mlp is None:
        return None
    r = mlp["router"]
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, intermediate_size=mlp["expert"]["ff"], num_experts=r["experts"], top=r["top"],
        activation="silu", router_bias_name=None, scoring="softmax_all", correction_name="correction",
        num_identity=r.get("identity", 0)))


def merudra_layout(cfg: MerudraConfig) -> ModelLayout:
    norm = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=""))
    n_layers = len(cfg.layers)
    layers, plan, slot = [], [], 0
    for i, layer in enumerate(cfg.layers):
        block = PartSpec("gated_post_norm", dict(
            hidden_size=cfg.width, mixer=_mixer(cfg, layer), feed_forward=_feed_forward(cfg, layer.get("mlp")), norm=norm,
            conv_taps=cfg.canon_taps,
            token_side=dict(dim=cfg.side_dim, table="side.embed", columns=n_layers * cfg.side_dim, first=i * cfg.side_dim,
                            vocab=cfg.vocab, eps=cfg.norm_eps),
            depth_mix=i + 2))
        layers.append(LayerSpec(block, f"l{i}."))
        n_caches = len(block.build("block").cache_specs())
        plan.append(PlanEntry(i, tuple(range(slot, slot + n_caches)) if n_caches != 1 else slot, True))
        slot += n_caches
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), plan=tuple(plan), final_norm=norm,
        embed_name="embed", final_norm_prefix="final.norm", head_name="head", tie_head=False, max_positions=None,
        layer_history=True)
