"""Configuration of the Pufivik design, from the keys of its ``config.json``.

A Pufivik model is a list of layers, each with one of two attention mixers and an optional mixture of routed experts;
every sublayer is normed in groups on its way in and on its way back, and the mixer reads its normed input through a
short causal convolution:

    {"architecture": "Pufivik", "vocab": V, "width": W, "norm": {"eps": e, "groups": g}, "canon": {"taps": n},
     "embedding": {"scale": s}, "residual_mult": m,
     "layers": [{"type": "attention" | "attention_2",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix",
                           "rot": {"base", "dims", "scaling": {...}}, "softcap" (attention_2)},
                 "mlp": null | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}}}, ...]}

``attention``: half-split rotation whose frequencies are scaled by wavelength bands (``scaling``: factor, low, high,
original), a sink per head in the softmax, the heads' weights mixed by a matrix, a sigmoid gate per head.
``attention_2``: interleaved rotation whose frequencies are scaled along a ramp (``scaling``: factor, original, fast,
slow), scores bent by softcap * tanh(score / softcap).
Every size and constant is read from here.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .ganidra_config import _number
from .model_config import ConfigError, ModelConfig, _require_int

_MIXERS = ("attention", "attention_2")
_SCALING_KEYS = {"attention": ("factor", "low", "high", "original"), "attention_2": ("factor", "original", "fast", "slow")}


def _check_mixer(where: str, kind: str, m: Any) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _require_int(f"{where}.{key}", m.get(key))
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
    _number(f"{where}.scale", m.get("scale"))
    if not isinstance(m.get("v_mix", False), bool):
        raise ConfigError(f"config.json: {where}.v_mix must be true or false")
    rot = m.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
    _number(f"{where}.rot.base", rot.get("base"))
    dims = _require_int(f"{where}.rot.dims", rot.get("dims"), 2)
    if dims % 2 or dims > m["dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims ({dims}) must be even and at most dim ({m['dim']})")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, dict):
            raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
        for key in _SCALING_KEYS[kind]:
            _number(f"{where}.rot.scaling.{key}", scaling.get(key))
        if kind == "attention" and scaling["high"] == scaling["low"]:
            raise ConfigError(f"config.json: {where}.rot.scaling.high and .low must differ")
    if m.get("softcap") is not None:                # (absent or null: the scores stay as they are)
        if kind != "attention_2":
            raise ConfigError(f"config.json: {where}.softcap belongs to the mixer 'attention_2'")
        _number(f"{where}.softcap", m["softcap"])


def _check_mlp(where: str, mlp: Any) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where} must be null or a 'moe' feed-forward, got {mlp!r}")
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, dict) or not isinstance(router, dict):
        raise ConfigError(f"config.json: {where} needs 'expert' and 'router' objects")
    _require_int(f"{where}.expert.ff", expert.get("ff"))
    experts = _require_int(f"{where}.router.experts", router.get("experts"))
    top = _require_int(f"{where}.router.top", router.get("top"))
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top ({top}) exceeds its experts ({experts})")


@dataclass
class PufivikConfig(ModelConfig):
    architecture: ClassVar[str] = "Pufivik"

    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    norm_groups: int = 1
    canon_taps: int = 1
    embed_scale: float = 1.0
    residual_mult: float = 1.0
    layers: tuple = ()                  # the config.json entries, checked
    eos_token_ids: tuple = field(default_factory=tuple)

    # what the engine asks of every configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "PufivikConfig":
        for key in ("vocab", "width", "layers", "norm", "canon", "embedding", "residual_mult"):
            if key not in raw:
                raise ConfigError(f"config.json: '{key}' is missing")
        for key, sub in (("norm", "eps"), ("norm", "groups"), ("canon", "taps"), ("embedding", "scale")):
            if not isinstance(raw[key], dict) or sub not in raw[key]:
                raise ConfigError(f"config.json: {key}.{sub} is missing")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        eos = raw.get("eos_token_id")
        eos_all = tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        cfg = cls(vocab=_require_int("vocab", raw["vocab"]), width=_require_int("width", raw["width"]),
                  norm_eps=_number("norm.eps", raw["norm"]["eps"]),
                  norm_groups=_require_int("norm.groups", raw["norm"]["groups"]),
                  canon_taps=_require_int("canon.taps", raw["canon"]["taps"]),
                  embed_scale=_number("embedding.scale", raw["embedding"]["scale"], positive=False),
                  residual_mult=_number("residual_mult", raw["residual_mult"], positive=False),
                  layers=tuple(copy.deepcopy(raw["layers"])), eos_token_ids=eos_all)
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "canon": {"taps": self.canon_taps},
                               "embedding": {"scale": self.embed_scale}, "residual_mult": self.residual_mult,
                               "layers": copy.deepcopy(list(self.layers))}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def validate(self) -> None:
        if self.width % self.norm_groups:
            raise ConfigError(f"config.json: width ({self.width}) must be a multiple of norm.groups ({self.norm_groups})")
        shared = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = layer.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design; known: {list(_MIXERS)}")
            _check_mixer(f"{where}.mixer", kind, layer.get("mixer"))
            _check_mlp(f"{where}.mlp", layer.get("mlp"))
            m = layer["mixer"]
            if m.get("v_mix"):
                # values shared across layers: one shape for all of them
                shape = (m["kv_heads"], m["vdim"])
                if shared is not None and shape != shared:
                    raise ConfigError(f"config.json: {where}.mixer shares values of {shape[0]} kv heads x {shape[1]}, "
                                      f"the first such layer has {shared[0]} x {shared[1]}")
                shared = shape
