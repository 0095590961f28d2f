"""Named configurations: each is the content of a ``config.json``.

The sizes are data here, not constants of the code: a preset is turned into a
model folder (config.json + model.safetensors) by the random-weights writer
and read back like any other model.  ``init`` gives the spread of the random
weights and the page size the configuration is usually run with.
"""
from __future__ import annotations

from typing import Any

_QWEN3_COMMON = dict(
    architectures=["Qwen3ForCausalLM"], hidden_act="silu", attention_bias=False,
    head_dim=128, vocab_size=151936, rope_theta=1_000_000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=40960,
)

PRESETS: dict[str, dict[str, Any]] = {
    "tiny-a": dict(
        config=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                    rms_norm_eps=1e-6, tie_word_embeddings=True,
                    max_position_embeddings=512),
        init=dict(seed=0, std=0.02, norm_std=0.1, block_size=4)),
    "tiny-b": dict(
        config=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=80,
                    num_attention_heads=4, num_key_value_heads=1, head_dim=32,
                    intermediate_size=224, vocab_size=389, rope_theta=1_000_000.0,
                    rms_norm_eps=1e-5, tie_word_embeddings=False,
                    max_position_embeddings=512),
        init=dict(seed=1, std=0.05, norm_std=0.2, block_size=8)),
    "qwen3-0.6b": dict(
        config=dict(_QWEN3_COMMON, num_hidden_layers=28, hidden_size=1024,
                    num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072),
        init=dict(seed=2, std=0.02, norm_std=0.1, block_size=16)),
    "qwen3-1.7b": dict(
        config=dict(_QWEN3_COMMON, num_hidden_layers=28, hidden_size=2048,
                    num_attention_heads=16, num_key_value_heads=8, intermediate_size=6144),
        init=dict(seed=3, std=0.02, norm_std=0.1, block_size=16)),
    "qwen3-4b": dict(
        config=dict(_QWEN3_COMMON, num_hidden_layers=36, hidden_size=2560,
                    num_attention_heads=32, num_key_value_heads=8, intermediate_size=9728),
        init=dict(seed=4, std=0.02, norm_std=0.1, block_size=16)),
    # a small model of the Ganidra design: gated linear attention, and windowed softmax attention beside it, the
    # first two layers passed twice
    "ganidra-tiny": dict(
        config=dict(architecture="Ganidra", vocab=320, width=128, embedding=dict(scale=2.0), norm=dict(eps=1e-6),
                    layers=[dict(type="gla", mixer=dict(heads=4, dim=16, vdim=32, tau=8.0, rank=8), mlp=None),
                            dict(type="parallel",
                                 mixer=dict(left=dict(heads=4, kv_heads=2, dim=32, vdim=32, mask=dict(size=48), scale=0.17),
                                            right=dict(heads=2, dim=16, vdim=32, tau=8.0, rank=8),
                                            left_scale=0.7, right_scale=0.7),
                                 mlp=dict(kind="dense", ff=256)),
                            dict(type="gla", mixer=dict(heads=4, dim=16, vdim=32, tau=4.0, rank=8), mlp=dict(kind="dense", ff=192))],
                    loop=dict(start=0, stop=2, times=2)),
        init=dict(seed=5, std=0.08, norm_std=0.1, block_size=16)),
    # a small model of the Besavik design: linear attention with a constant decay per head, latent attention, the gated
    # delta rule behind short convolutions; a dense feed-forward and two mixtures of routed experts
    "besavik-tiny": dict(
        config=dict(architecture="Besavik", vocab=320, width=128, logit_scale=0.5, norm=dict(eps=1e-6),
                    layers=[dict(type="lightning", mixer=dict(heads=2, dim=16, vdim=32, decay=[0.9, 0.99]),
                                 mlp=dict(kind="dense", ff=256, limit=2.0)),
                            dict(type="latent_attention",
                                 mixer=dict(heads=4, dim=16, rot_dim=16, vdim=32, kv_rank=48, q_rank=32, scale=0.18,
                                            rot=dict(base=10000.0, dims=16)),
                                 mlp=dict(kind="moe", expert=dict(ff=64, limit=2.0), router=dict(experts=4, top=2))),
                            dict(type="channel_delta", mixer=dict(heads=4, kv_heads=2, dim=16, vdim=32, conv=4, rank=8),
                                 mlp=dict(kind="moe", expert=dict(ff=64, limit=2.0), router=dict(experts=4, top=2)))]),
        init=dict(seed=7, std=0.08, norm_std=0.1, block_size=16)),
    # a small model of the Merudra design: attention whose values are its keys, the delta rule with one decay per head,
    # experts scored over all of them with two that hand their input on; the stream read through convolutions of 3 taps
    "merudra-tiny": dict(
        config=dict(architecture="Merudra", vocab=320, width=128, norm=dict(eps=1e-6), canon=dict(taps=3), token_side=dict(dim=16),
                    layers=[dict(type="attention",
                                 mixer=dict(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.18, q_temp=dict(coef=0.3, every=16)),
                                 mlp=dict(kind="moe", expert=dict(ff=64), router=dict(experts=4, identity=2, top=2))),
                            dict(type="delta", mixer=dict(heads=4, kv_heads=2, dim=16, vdim=32, conv=4),
                                 mlp=dict(kind="moe", expert=dict(ff=64), router=dict(experts=4, identity=1, top=2))),
                            dict(type="attention",
                                 mixer=dict(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.18, q_temp=dict(coef=0.3, every=16)),
                                 mlp=None)]),
        init=dict(seed=11, std=0.08, norm_std=0.1, block_size=16)),
    # a small model of the Pufivik design: norms in two groups around every sublayer, the mixers' input through
    # convolutions of 3 taps, attention with bent scores and attention with a sink, mixed heads and a gate per head, keys
    # of 32 and values of 16 channels, values blended with the first layer's, experts scored by sigmoids
    "pufivik-tiny": dict(
        config=dict(architecture="Pufivik", vocab=320, width=128, norm=dict(eps=1e-6, groups=2), canon=dict(taps=3),
                    embedding=dict(scale=4.0), residual_mult=0.6,
                    layers=[dict(type="attention_2",
                                 mixer=dict(heads=4, kv_heads=2, dim=32, vdim=16, scale=0.18, softcap=20.0, v_mix=True,
                                            rot=dict(base=10000.0, dims=16, scaling=dict(factor=4.0, original=64, fast=16.0, slow=1.0))),
                                 mlp=dict(kind="moe", expert=dict(ff=64), router=dict(experts=4, top=2))),
                            dict(type="attention",
                                 mixer=dict(heads=4, kv_heads=2, dim=32, vdim=16, scale=0.18, v_mix=True,
                                            rot=dict(base=50000.0, dims=32, scaling=dict(factor=8.0, low=1.0, high=4.0, original=128))),
                                 mlp=dict(kind="moe", expert=dict(ff=64), router=dict(experts=4, top=1))),
                            dict(type="attention_2",
                                 mixer=dict(heads=2, kv_heads=2, dim=16, vdim=16, scale=0.25, softcap=8.0, v_mix=True,
                                            rot=dict(base=10000.0, dims=8, scaling=None)),
                                 mlp=None)]),
        init=dict(seed=17, std=0.08, norm_std=0.1, block_size=16)),
}


def preset_config_dict(name: str) -> dict[str, Any]:
    try:
        import copy
        return copy.deepcopy(dict(PRESETS[name]["config"]))
    except KeyError:
        raise ValueError(f"unknown preset {name!r}; known: {sorted(PRESETS)}") from None


def preset_init(name: str) -> dict[str, Any]:
    preset_config_dict(name)
    return dict(PRESETS[name]["init"])
