"""Pufivik as a layout of parts.

Layers in the order config.json gives, each a ``sandwich_norm`` block (a group RMS norm before and after every
sublayer, the result times the model's multiplier; the mixer reads its normed input through a short causal convolution)
with one of two mixers, both ``gqa_attention`` with its options: ``attention`` (half-split rotation of the head's first
channels with frequencies scaled by wavelength bands, a sink per head in the softmax, the heads' weights mixed by a
matrix, a sigmoid gate per head) and ``attention_2`` (interleaved rotation with frequencies scaled along a ramp, scores
bent by a tanh).  Keys and values have sizes of their own; layers that say so blend their values with those of the
first such layer.  The feed-forward is absent or a mixture of routed experts scored by sigmoids, whose weights
multiply what the experts read.  The embedding output is scaled; the head is the embedding table as it is.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1/norm1b/norm2/norm2b``, ``l<i>.canon1``,
``l<i>.mix.q/k/v/o/vmix`` (+ ``sink``, ``talk``, ``g``), ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate/up/down``.
"""
from __future__ import annotations

from ..config.pufivik_config import PufivikConfig
from ..parts.base import PartSpec
from .decoder import LayerSpec, ModelLayout, PlanEntry


def _position_encoding(kind: str, m: dict) -> PartSpec:
    rot = m["rot"]
    s = rot.get("scaling")
    if kind == "attention":
        scaling = None if s is None else ("bands", s["factor"], s["low"], s["high"], s["original"])
        pairing = "half"
    else:
        scaling = None if s is None else ("ramp", s["factor"], s["original"], s["fast"], s["slow"])
        pairing = "interleaved"
    return PartSpec("rope_scaled", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"], scaling=scaling, pairing=pairing))


def _mixer(cfg: PufivikConfig, layer: dict, value_mix) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    names = dict(q="q", k="k", v="v", out="o", gate="g", sink="sink", head_mix="talk", value_mix="vmix")
    common = dict(hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                  scale=m["scale"], position_encoding=_position_encoding(kind, m), value_mix=value_mix, names=names)
    if kind == "attention":
        return PartSpec("gqa_attention", dict(common, sink=True, head_mixing=True, output_gate="sigmoid_head"))
    return PartSpec("gqa_attention", dict(common, softcap=m.get("softcap")))


def _feed_forward(cfg: PufivikConfig, mlp):
    if mlp is None:
        return None
    r = mlp["router"]
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, intermediate_size=mlp["expert"]["ff"], num_experts=r["experts"], top=r["top"],
        activation="silu", router_bias_name=None, scoring="sigmoid", weight_inputs=True))


def pufivik_layout(cfg: PufivikConfig) -> ModelLayout:
    norm = PartSpec("group_rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, groups=cfg.norm_groups, weight_name=""))
    post_norm = PartSpec("group_rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, groups=cfg.norm_groups, weight_name="",
                                               output_scale=cfg.residual_mult))
    layers, plan, slot = [], [], 0
    kept = False
    for i, layer in enumerate(cfg.layers):
        value_mix = None
        if layer["mixer"].get("v_mix"):
            value_mix, kept = ("blend" if kept else "keep"), True
        block = PartSpec("sandwich_norm", dict(
            hidden_size=cfg.width, mixer=_mixer(cfg, layer, value_mix), feed_forward=_feed_forward(cfg, layer.get("mlp")),
            norm=norm, post_norm=post_norm, input_conv_taps=cfg.canon_taps))
        layers.append(LayerSpec(block, f"l{i}."))
        n_caches = len(block.build("block").cache_specs())
        plan.append(PlanEntry(i, tuple(range(slot, slot + n_caches)) if n_caches != 1 else slot, True))
        slot += n_caches
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), plan=tuple(plan), final_norm=norm,
        embed_name="embed", final_norm_prefix="final.norm", head_name=None, tie_head=True, max_positions=None,
        embed_scale=cfg.embed_scale)
