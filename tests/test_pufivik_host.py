"""Pufivik on the host side of the engine: configuration, registry, weights and caches, and replay and generation on
the CPU with the plain operations in the place of the kernels, against the plain restatement of the design
(tests/plain_pufivik.py).  The same traces run on the GPU in test_pufivik_gpu.py."""
import copy
import math

import pytest
import torch

import plain_pufivik
import pufivik_helpers as ph
from helpers import random_tokens
from qwen_engine_b200.config import ConfigError, PufivikConfig
from qwen_engine_b200.registry import architecture_of, build_model, config_from_dict
from qwen_engine_b200.weights import SafetensorsSource, WeightError, check_against_manifest

F32 = torch.float32


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pufivik")
    return {name: ph.make_folder(str(root / name), name) for name in ("p-a", "p-b", "p-c")}


def test_config_reads_its_own_keys_and_round_trips():
    raw = ph.PUFIVIK["p-a"]["cfg"]
    assert architecture_of(raw).name == "Pufivik"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, PufivikConfig)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.norm_groups, cfg.canon_taps, cfg.embed_scale, cfg.residual_mult) == (211, 64, 1e-6, 2, 2, 3.0, 0.7)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="delta"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=3.0), "belongs to"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("high"), "scaling.high"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=4), "shares values"),
    (lambda c: c["layers"][1].update(mlp=dict(kind="dense", ff=8)), "feed-forward"),
    (lambda c: c.pop("canon"), "'canon' is missing"),
    (lambda c: c["norm"].pop("groups"), "norm.groups is missing"),
    (lambda c: c["norm"].update(groups=3), "multiple of norm.groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "exceeds"),
])
def test_config_refuses_what_it_cannot_run(change, text):
    raw = copy.deepcopy(ph.PUFIVIK["p-a"]["cfg"])
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_caches_of_the_layers():
    """A layer keeps pages of keys and values, padded to the larger of the two sizes, and the last taps - 1 normed rows
    that its mixer's convolution reads; with one tap nobody keeps rows."""
    model = build_model(config_from_dict(ph.PUFIVIK["p-a"]["cfg"]))
    specs = model.cache_specs()
    assert [type(s).__name__ for s in specs] == ["PagedKVSpec", "FixedStateSpec"] * 3
    assert (specs[0].num_kv_heads, specs[0].head_dim, specs[0].planes) == (2, 16, 2) and specs[1].shape == (1, 64)
    assert (specs[4].num_kv_heads, specs[4].head_dim) == (1, 32)
    assert model.attention_geometries == ((4, 2, 16, 0), (4, 2, 24, 0), (2, 1, 32, 0)) and specs[2].head_dim == 24
    model = build_model(config_from_dict(ph.PUFIVIK["p-b"]["cfg"]))
    assert model.cache_specs()[0].head_dim == 32 and model.cache_specs()[1].shape == (3, 96)
    model = build_model(config_from_dict(ph.PUFIVIK["p-c"]["cfg"]))
    assert [type(s).__name__ for s in model.cache_specs()] == ["PagedKVSpec", "PagedKVSpec"]


def test_tensor_names(folders):
    src = SafetensorsSource(folders["p-a"])
    names = set(src.names())
    assert {"embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.canon1", "l0.mix.q", "l0.mix.k", "l0.mix.v",
            "l0.mix.o", "l0.mlp.e4.down", "l0.mlp.router", "l1.mix.sink", "l1.mix.talk", "l1.mix.g", "l1.mix.vmix", "l2.norm1b"} <= names
    assert not {"head", "l0.mix.sink", "l0.mix.g", "l2.norm2", "l2.norm2b", "l2.mix.vmix", "l0.mlp.e5.gate", "l0.canon2"} & names
    assert src.shape("l1.mix.vmix") == () and src.shape("l1.mix.talk") == (4, 4) and src.shape("l1.mix.g") == (4, 64)
    assert src.shape("l0.mix.v") == (16, 64) and src.shape("l0.mix.o") == (64, 32) and src.shape("l0.canon1") == (64, 2)
    raw = copy.deepcopy(ph.PUFIVIK["p-a"]["cfg"])
    check_against_manifest(src, build_model(config_from_dict(raw)).weight_manifest(), "folder")
    raw["canon"]["taps"] = 3
    with pytest.raises(WeightError, match="wrong shapes"):
        check_against_manifest(src, build_model(config_from_dict(raw)).weight_manifest(), "folder")


def test_scaled_frequencies_against_the_plain_functions():
    """The frequencies the position encoding hands to the kernels, against the plain functions, for both scalings, for
    no scaling, and with bands and ramps that leave every frequency on one side."""
    from qwen_engine_b200.parts.rope import ScaledRope
    for rot in (dict(base=5000.0, dims=16, scaling=dict(factor=8.0, low=1.0, high=4.0, original=32)),
                dict(base=100.0, dims=8, scaling=dict(factor=2.0, low=1.0, high=2.0, original=8)),
                dict(base=1e6, dims=64, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)),
                dict(base=10.0, dims=6, scaling=dict(factor=3.0, low=0.5, high=1000.0, original=4))):
        s = rot["scaling"]
        pe = ScaledRope(rot["dims"] + 4, rot["base"], rot["dims"], ("bands", s["factor"], s["low"], s["high"], s["original"]))
        want, mag = plain_pufivik.banded_frequencies(rot)
        assert torch.allclose(pe._inv_freq_cpu.double(), want, rtol=1e-7, atol=0) and pe.magnitude == mag == 1.0
        assert pe.row_permutation() is None
    for rot in (dict(base=10000.0, dims=8, scaling=dict(factor=8.0, original=64, fast=16.0, slow=2.0)),
                dict(base=7.0, dims=4, scaling=dict(factor=3.0, original=8, fast=2.0, slow=1.0)),
                dict(base=1e6, dims=128, scaling=dict(factor=32.0, original=4096, fast=32.0, slow=1.0)),
                dict(base=50.0, dims=10, scaling=dict(factor=1.5, original=1 << 20, fast=1.0, slow=1.0))):
        s = rot["scaling"]
        pe = ScaledRope(rot["dims"], rot["base"], rot["dims"], ("ramp", s["factor"], s["original"], s["fast"], s["slow"]), "interleaved")
        want, mag = plain_pufivik.ramped_frequencies(rot)
        assert torch.allclose(pe._inv_freq_cpu.double(), want, rtol=1e-7, atol=0)
        assert math.isclose(pe.magnitude, mag) and mag == 0.1 * math.log(s["factor"]) + 1.0
        half = rot["dims"] // 2
        assert pe.row_permutation()[:half] == list(range(0, rot["dims"], 2)) and pe.row_permutation()[half:] == list(range(1, rot["dims"], 2))
    pe = ScaledRope(12, 300.0, 8, None, "half")
    assert torch.allclose(pe._inv_freq_cpu.double(), plain_pufivik.base_frequencies(dict(base=300.0, dims=8)), rtol=1e-7)


@pytest.mark.parametrize("name", ["p-a", "p-b", "p-c"])
def test_replay_on_the_host(folders, cpu_ops, name):
    folder = folders[name]
    ph.replay_cases(lambda n: ph.make_replayer(folder, name, F32, n, device="cpu", poison=True), folder, name, F32,
                    f"host {name}")


def test_greedy_generation_through_the_engine_on_the_host(folders, cpu_ops):
    from qwen_engine_b200.sampling.params import SamplingParams
    name = "p-a"
    folder = folders[name]
    cfg, w = ph.plain_model(folder)
    V = ph.vocab_of(name)
    prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26])]
    eng = ph.make_engine(folder, name, F32, device="cpu", max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=6, temperature=0.0)) for p in prompts]
    outs = {o.request_id: o for o in eng.serving()}
    for rid, p in zip(ids, prompts):
        assert list(outs[rid].output_token_ids) == plain_pufivik.greedy(cfg, w, p, 6), f"prompt of {len(p)} tokens"
    assert eng.cache.slots.num_free == eng.cache.slots.num_slots


def test_a_stored_scalar_of_the_keeping_layer_is_ignored(folders, tmp_path, cpu_ops):
    """The layer that keeps its values blends nothing; a checkpoint that stores its scalar all the same loads, and the
    logits do not depend on it."""
    import shutil

    from safetensors.torch import load_file, save_file
    from helpers import run_steps
    src = folders["p-a"]
    dst = str(tmp_path / "with_scalar")
    shutil.copytree(src, dst)
    tensors = load_file(dst + "/model.safetensors")
    tensors["l0.mix.vmix"] = torch.tensor(0.9, dtype=torch.bfloat16)
    save_file(tensors, dst + "/model.safetensors", metadata={"format": "pt"})
    toks = random_tokens(ph.vocab_of("p-a"), 21, 8)
    steps = [{"entries": [{"id": "a", "tokens": toks, "want": [20]}], "end": ["a"]}]
    a = run_steps(ph.make_replayer(src, "p-a", F32, 64, device="cpu"), steps)["a"][20]
    b = run_steps(ph.make_replayer(dst, "p-a", F32, 64, device="cpu"), steps)["a"][20]
    assert torch.equal(a, b)
