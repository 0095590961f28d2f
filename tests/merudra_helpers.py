"""Shared by the Merudra tests: small configurations that differ in every size and constant, model folders with
seeded random weights, and the plain implementation's logits."""
from __future__ import annotations

import torch

import plain_merudra
from ganidra_helpers import ROW_TOL, ROW_WORST
from qwen_engine_b200.registry import config_from_dict
from qwen_engine_b200.weights import write_model_folder


def _attn(heads, kv_heads, dim, scale, coef, every):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, q_temp=dict(coef=coef, every=every))


def _delta(heads, kv_heads, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def _moe(experts, identity, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top))


def _layer(kind, mixer, mlp=None):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def _model(vocab, width, eps, taps, side, layers):
    return dict(architecture="Merudra", vocab=vocab, width=width, norm=dict(eps=eps), canon=dict(taps=taps),
                token_side=dict(dim=side), layers=layers)


MERUDRA = {
    # grouped key heads in both mixers, a temperature that steps every fourth position, identity experts among three
    # choices, a last layer without feed-forward
    "m-a": dict(cfg=_model(211, 64, 1e-6, 2, 5, [
        _layer("attention", _attn(4, 2, 16, 0.2, 0.3, 4), _moe(5, 2, 3, 24)),
        _layer("delta", _delta(4, 2, 8, 12, 3), _moe(3, 1, 1, 16)),
        _layer("attention", _attn(2, 1, 32, 0.1, 1.0, 7), None)]), seed=3, std=0.12, norm_std=0.2, page=4),
    # the delta mixer first and without feed-forward; a head size that is no multiple of 16; all experts chosen and
    # none of them an identity; more identity experts than others; a temperature that steps at every position
    "m-b": dict(cfg=_model(300, 96, 1e-5, 4, 8, [
        _layer("delta", _delta(2, 2, 16, 16, 2), None),
        _layer("attention", _attn(3, 3, 24, 0.15, 0.7, 1), _moe(4, 0, 4, 32)),
        _layer("delta", _delta(3, 1, 6, 10, 5), _moe(2, 3, 2, 20)),
        _layer("attention", _attn(1, 1, 48, 0.3, 0.05, 30), _moe(6, 1, 2, 8))]), seed=5, std=0.1, norm_std=0.1, page=16),
    # one tap: the stream is read as it is and the sublayers keep no rows; sizes that are no multiples of four or eight;
    # convolutions of one tap in the delta mixer too
    "m-c": dict(cfg=_model(97, 40, 3e-6, 1, 3, [
        _layer("attention", _attn(2, 2, 20, 0.25, 2.0, 3), _moe(3, 2, 2, 12)),
        _layer("delta", _delta(2, 2, 12, 4, 1), _moe(2, 1, 3, 28))]), seed=9, std=0.15, norm_std=0.3, page=8),
    # sizes of real heads: head size 128 (the kernels' fast paths), 128 key channels in the delta mixer
    "m-d": dict(cfg=_model(513, 384, 1e-6, 3, 16, [
        _layer("attention", _attn(4, 2, 128, 0.09, 0.4, 64), _moe(8, 2, 2, 128)),
        _layer("delta", _delta(4, 2, 128, 64, 4), _moe(8, 1, 3, 64)),
        _layer("attention", _attn(4, 2, 128, 0.09, 0.4, 64), _moe(6, 3, 2, 96)),
        _layer("attention", _attn(2, 2, 64, 0.125, 0.25, 100), None)]), seed=13, std=0.05, norm_std=0.1, page=16),
}


def assert_close_rows(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    """Row by row, the root mean square of the logits' difference (means taken off) against that of the logits.  float32 is
    the sharp test (1e-4).  In bfloat16 these narrow random models with queries that grow with the position make sharp
    softmaxes, and a lone position moves by 10 to 20 % whichever way the request is cut (whole, token by token and mixed
    give the same rows to 4 %: measured); so a few rows may pass the bound that most keep, none the worst one."""
    got = got.detach().to("cpu", torch.float64)
    want = want.to(torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    d = got - want
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / (want - want.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt()
    worst = int(torch.argmax(err))
    assert float(err[worst]) <= ROW_WORST[dtype], f"{what}: row {worst} is off by {float(err[worst]):.3e} > {ROW_WORST[dtype]}"
    over = int((err > ROW_TOL[dtype]).sum())
    assert over <= max(2, err.numel() // 12), f"{what}: {over} of {err.numel()} rows are off by more than {ROW_TOL[dtype]}"


def make_folder(path: str, name: str) -> str:
    spec = MERUDRA[name]
    write_model_folder(config_from_dict(spec["cfg"]), path, spec["seed"], spec["std"], spec["norm_std"], torch.bfloat16)
    return path


_plain: dict = {}


def plain_model(folder: str):
    if folder not in _plain:
        _plain[folder] = plain_merudra.read_model_folder(folder)
    return _plain[folder]


def plain_logits(folder: str, tokens) -> torch.Tensor:
    key = (folder, tuple(tokens))
    if key not in _plain:
        cfg, w = plain_model(folder)
        margins: list = []
        _plain[key] = plain_merudra.forward(cfg, w, list(tokens), margins=margins).to(torch.float32)
        _plain[("margin",) + key] = torch.stack(margins).min(dim=0).values if margins else torch.full((len(tokens),), float("inf"))
    return _plain[key]


CLOSE_CALL = 0.02


def settled_positions(folder: str, tokens, dtype) -> set:
    """The positions at which no router of the plain model makes a close call (the last chosen expert beats the first one
    left out by less than CLOSE_CALL): bfloat16 rounding may decide such a call the other way, and then the row is another
    expert's, so in bfloat16 rows are judged at the other positions only.  In float32 every position counts."""
    plain_logits(folder, tokens)
    m = _plain[("margin", folder, tuple(tokens))]
    if dtype == torch.float32:
        return set(range(len(tokens)))
    return {i for i in range(len(tokens)) if float(m[i]) >= CLOSE_CALL}


def vocab_of(name: str) -> int:
    return MERUDRA[name]["cfg"]["vocab"]


def make_replayer(folder, name, dtype, max_tokens, device="cuda:0", slots=4, poison=False):
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.trace import TraceReplayer
    page = MERUDRA[name]["page"]
    unit = max(64, page)
    unit = -(-unit // page) * page
    num_pages = -(-max_tokens // unit) * (unit // page)
    loaded = load_model(folder, dtype, device, page, num_pages, slots, poison_cache=poison, check_device=(device != "cpu"))
    return TraceReplayer(folder, dtype, max_tokens, page_size=page, loaded=loaded)


def check_requests(got, folder, requests, dtype, what):
    for rid, toks in requests.items():
        want = plain_logits(folder, toks)
        rows = got[rid]
        settled = settled_positions(folder, toks, dtype)
        idx = [i for i in sorted(rows) if i in settled]
        assert len(rows) < 10 or len(idx) >= 0.5 * len(rows), f"{what} {rid}: too many close calls to judge"
        if not idx:
            continue
        assert_close_rows(torch.stack([rows[i] for i in idx]), want[idx], dtype, f"{what} {rid} (positions {idx[0]}..)")


def make_engine(folder, name, dtype, device="cuda:0", **engine_kwargs):
    from qwen_engine_b200.config import EngineConfig
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    kw = dict(dtype=dtype, device=device, block_size=MERUDRA[name]["page"], max_model_len=160, max_num_seqs=4,
              max_num_batched_tokens=48)
    kw.update(engine_kwargs)
    ec = EngineConfig(**kw)
    loaded = load_model(folder, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(), ec.max_num_seqs,
                        ec.enable_prefix_cache, check_device=(device != "cpu"))
    return LLMEngine(loaded, ec)


def replay_cases(rep_factory, folder, name, dtype, what):
    """The ways of cutting requests into steps, each against the plain implementation: whole prompts; a prompt and
    then single tokens; from the first token one by one; portions of changing sizes down to two tokens; up to four
    live requests mixed, with pages and slots that come back and go out again."""
    from helpers import live_tokens_needed, mixed_steps, random_tokens, run_steps
    V = vocab_of(name)
    reqs = {"w0": random_tokens(V, 61, 1), "w1": random_tokens(V, 9, 2), "w2": random_tokens(V, 1, 3)}
    steps = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]} for r, t in reqs.items()]
    check_requests(run_steps(rep_factory(128), steps), folder, reqs, dtype, f"{what} whole")
    toks = random_tokens(V, 75, 3)
    steps = [{"entries": [{"id": "d", "tokens": toks[:35], "want": [0, 17, 34]}]}]
    steps += [{"entries": [{"id": "d", "tokens": [t], "want": [0]}]} for t in toks[35:]]
    check_requests(run_steps(rep_factory(128), steps), folder, {"d": toks}, dtype, f"{what} decode")
    steps = [{"entries": [{"id": "s", "tokens": [t], "want": [0]}]} for t in toks[:20]]
    check_requests(run_steps(rep_factory(64), steps), folder, {"s": toks[:20]}, dtype, f"{what} single tokens")
    toks = random_tokens(V, 90, 4)
    steps, p = [], 0
    for n in [2, 7, 3, 2, 16, 5, 2, 13, 9, 2, 11] + [1] * 18:
        steps.append({"entries": [{"id": "c", "tokens": toks[p:p + n], "want": list(range(n))}]})
        p += n
    assert p == len(toks)
    check_requests(run_steps(rep_factory(128), steps), folder, {"c": toks}, dtype, f"{what} portions")
    reqs = {f"m{i}": random_tokens(V, n, 20 + i) for i, n in enumerate([40, 64, 23, 90, 17, 55, 70, 33])}
    steps = mixed_steps(reqs, seed=7)
    rep = rep_factory(live_tokens_needed(steps, 64))
    check_requests(run_steps(rep, steps), folder, reqs, dtype, f"{what} mixed")
    assert rep.cache.pages_in_use() == 0 and rep.cache.slots.num_free == rep.cache.slots.num_slots
