"""Merudra on the host side of the engine: configuration, registry, weights and caches, and replay and generation on
the CPU with the plain operations in the place of the kernels, against the plain restatement of the design
(tests/plain_merudra.py).  The same traces run on the GPU in test_merudra_gpu.py."""
import copy

import pytest
import torch

import merudra_helpers as mh
import plain_merudra
from helpers import random_tokens
from qwen_engine_b200.config import ConfigError, MerudraConfig
from qwen_engine_b200.registry import architecture_of, build_model, config_from_dict
from qwen_engine_b200.weights import SafetensorsSource, WeightError, check_against_manifest

F32 = torch.float32


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("merudra")
    return {name: mh.make_folder(str(root / name), name) for name in ("m-a", "m-b", "m-c")}


def test_config_reads_its_own_keys_and_round_trips():
    raw = mh.MERUDRA["m-a"]["cfg"]
    assert architecture_of(raw).name == "Merudra"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, MerudraConfig)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.canon_taps, cfg.side_dim) == (211, 64, 1e-6, 2, 5)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="gla"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "values are the keys"),
    (lambda c: c["layers"][1].update(mlp=dict(kind="dense", ff=8)), "feed-forward"),
    (lambda c: c.pop("canon"), "'canon' is missing"),
    (lambda c: c["token_side"].pop("dim"), "token_side.dim is missing"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "exceeds"),
])
def test_config_refuses_what_it_cannot_run(change, text):
    raw = copy.deepcopy(mh.MERUDRA["m-a"]["cfg"])
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_caches_of_the_layers():
    """An attention layer keeps pages and the two sublayers' last rows of the stream; a delta layer its recurrence's
    state, its convolutions' inputs and the same rows; with one tap nobody keeps rows."""
    model = build_model(config_from_dict(mh.MERUDRA["m-a"]["cfg"]))
    kinds = [type(s).__name__ for s in model.cache_specs()]
    assert kinds == ["PagedKVSpec", "FixedStateSpec", "FixedStateSpec", "FixedStateSpec", "FixedStateSpec", "FixedStateSpec",
                     "FixedStateSpec", "PagedKVSpec", "FixedStateSpec"]
    specs = model.cache_specs()
    assert (specs[0].num_kv_heads, specs[0].head_dim, specs[0].planes) == (2, 16, 2)
    assert specs[1].shape == (1, 64) and specs[3].shape == (4, 12, 8) and specs[4].shape == (2, 2 * 2 * 8 + 4 * 12)
    assert model.attention_geometries == ((4, 2, 16, 0), (2, 1, 32, 0))
    model = build_model(config_from_dict(mh.MERUDRA["m-c"]["cfg"]))
    assert [type(s).__name__ for s in model.cache_specs()] == ["PagedKVSpec", "FixedStateSpec", "FixedStateSpec"]
    assert model.cache_specs()[2].shape == (0, 2 * 2 * 12 + 2 * 4)


def test_tensor_names(folders):
    src = SafetensorsSource(folders["m-a"])
    names = set(src.names())
    assert {"embed", "side.embed", "final.norm", "head", "l0.norm1", "l0.canon2", "l0.rg1", "l0.rg1.b", "l0.dwa", "l0.side.gate",
            "l0.side.proj", "l0.side.norm", "l0.mix.q.b", "l0.mix.k.b", "l0.mix.g", "l0.mlp.e4.down", "l0.mlp.router",
            "l0.mlp.correction", "l1.mix.q.conv", "l1.mix.A_log", "l1.mix.dt_bias", "l1.mix.a", "l1.mix.b", "l1.mix.norm"} <= names
    assert not {"l0.mix.v", "l0.mlp.e5.gate", "l2.norm2", "l2.canon2", "l2.rg2", "l1.mix.a1"} & names
    assert src.shape("side.embed") == (211, 3 * 5) and src.shape("l2.dwa") == (4,) and src.shape("l0.mlp.router") == (7, 64)
    raw = copy.deepcopy(mh.MERUDRA["m-a"]["cfg"])
    model = build_model(config_from_dict(raw))
    check_against_manifest(src, model.weight_manifest(), "folder")
    raw["token_side"]["dim"] = 6
    with pytest.raises(WeightError, match="wrong shapes"):
        check_against_manifest(src, build_model(config_from_dict(raw)).weight_manifest(), "folder")


@pytest.mark.parametrize("name", ["m-a", "m-b", "m-c"])
def test_replay_on_the_host(folders, cpu_ops, name):
    folder = folders[name]
    mh.replay_cases(lambda n: mh.make_replayer(folder, name, F32, n, device="cpu", poison=True), folder, name, F32,
                    f"host {name}")


def test_greedy_generation_through_the_engine_on_the_host(folders, cpu_ops):
    from qwen_engine_b200.sampling.params import SamplingParams
    name = "m-a"
    folder = folders[name]
    cfg, w = mh.plain_model(folder)
    V = mh.vocab_of(name)
    prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26])]
    eng = mh.make_engine(folder, name, F32, device="cpu", max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=6, temperature=0.0)) for p in prompts]
    outs = {o.request_id: o for o in eng.serving()}
    for rid, p in zip(ids, prompts):
        assert list(outs[rid].output_token_ids) == plain_merudra.greedy(cfg, w, p, 6), f"prompt of {len(p)} tokens"
    assert eng.cache.slots.num_free == eng.cache.slots.num_slots


def test_state_keeps_requests_from_sharing_pages(folders, cpu_ops):
    """Every layer keeps rows of the stream per request, so equal prefixes share no pages: a second request with the
    same first tokens runs them again."""
    from helpers import run_steps
    name = "m-a"
    folder = folders[name]
    toks = random_tokens(mh.vocab_of(name), 40, 5)
    rep = mh.make_replayer(folder, name, F32, 192, device="cpu")
    steps = [{"entries": [{"id": "a", "tokens": toks, "want": [39]}]},
             {"entries": [{"id": "b", "tokens": toks, "want": [7, 39]}], "end": ["a", "b"]}]
    got = run_steps(rep, steps)
    assert rep.cache.prefix_hit_tokens == 0
    mh.check_requests(got, folder, {"a": toks, "b": toks}, F32, "no sharing")
