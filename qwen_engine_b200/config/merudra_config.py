"""Configuration of the Merudra design, from the keys of its ``config.json``.

A Merudra model is a list of layers, each with one of two mixers and an
optional mixture of routed experts; every sublayer reads the residual stream
through a short causal convolution and is gated and normed on its way back:

    {"architecture": "Merudra", "vocab": V, "width": W, "norm": {"eps": e}, "canon": {"taps": n},
     "token_side": {"dim": d},
     "layers": [{"type": "attention" | "delta", "mixer": {...},
                 "mlp": null | {"kind": "moe", "expert": {"ff": F},
                                "router": {"experts": E, "identity": I, "top": k}}}, ...]}

Mixer sizes:
``attention``: heads, kv_heads, dim, vdim (the values are the keys, so vdim = dim), scale,
q_temp {coef, every}.
``delta``: heads, kv_heads, dim, vdim, conv (taps of the short convolution).
Every size and constant is read from here.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .ganidra_config import _number
from .model_config import ConfigError, ModelConfig, _require_int

_MIXERS = ("attention", "delta")


def _check_mixer(where: str, kind: str, m: Any) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _require_int(f"{where}.{key}", m.get(key))
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
    if kind == "attention":
        _number(f"{where}.scale", m.get("scale"))
        if m["vdim"] != m["dim"]:
            raise ConfigError(f"config.json: {where}.vdim ({m['vdim']}) must equal dim ({m['dim']}): the values are the keys")
        temp = m.get("q_temp")
        if temp is not None:
            if not isinstance(temp, dict):
                raise ConfigError(f"config.json: {where}.q_temp must be an object with 'coef' and 'every'")
            _number(f"{where}.q_temp.coef", temp.get("coef"), positive=False)
            _require_int(f"{where}.q_temp.every", temp.get("every"))
    else:
        _require_int(f"{where}.conv", m.get("conv"))


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
    identity = _require_int(f"{where}.router.identity", router.get("identity", 0), 0)
    top = _require_int(f"{where}.router.top", router.get("top"))
    if top > experts + identity:
        raise ConfigError(f"config.json: {where}.router.top ({top}) exceeds its router outputs ({experts + identity})")


@dataclass
class MerudraConfig(ModelConfig):
    architecture: ClassVar[str] = "Merudra"

    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    canon_taps: int = 1
    side_dim: int = 1
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
    def from_dict(cls, raw: dict[str, Any]) -> "MerudraConfig":
        for key in ("vocab", "width", "layers", "norm", "canon", "token_side"):
            if key not in raw:
                raise ConfigError(f"config.json: '{key}' is missing")
        for key, sub in (("norm", "eps"), ("canon", "taps"), ("token_side", "dim")):
            if not isinstance(raw[key], dict) or sub not in raw[key]:
                raise ConfigError(f"config.json: {key}.{sub} is missing")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        eos = raw.get("eos_token_id")
        eos_all = tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        cfg = cls(vocab=_require_int("vocab", raw["vocab"]), width=_require_int("width", raw["width"]),
                  norm_eps=_number("norm.eps", raw["norm"]["eps"]),
                  canon_taps=_require_int("canon.taps", raw["canon"]["taps"]),
                  side_dim=_require_int("token_side.dim", raw["token_side"]["dim"]),
                  layers=tuple(copy.deepcopy(raw["layers"])), eos_token_ids=eos_all)
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
                               "token_side": {"dim": self.side_dim}, "layers": copy.deepcopy(list(self.layers))}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = layer.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design; known: {list(_MIXERS)}")
            _check_mixer(f"{where}.mixer", kind, layer.get("mixer"))
            _check_mlp(f"{where}.mlp", layer.get("mlp"))
