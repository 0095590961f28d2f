"""Pufivik on the GPU: each new kernel or kernel option alone against the plain function of its mechanism
(tests/plain_pufivik.py, tests/ref_ops.py), the mixers through their cache with inputs made so that a far key, a sink, a
bent score or a mixed head shows, then whole models through replay, the engine and the command line."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import plain_pufivik as plain
import pufivik_helpers as ph
import ref_ops
from helpers import random_tokens, run_steps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64
DTYPES = [F32, BF16]


@pytest.fixture(scope="module")
def ops():
    from qwen_engine_b200 import ops as _ops
    _ops.lib()
    return _ops


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pufivik_gpu")
    return {name: ph.make_folder(str(root / name), name) for name in ph.PUFIVIK}


def _close(got, want, dtype, what="", tol=None):
    got, want = got.detach().to("cpu", F64), want.to(F64)
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    tol = tol if tol is not None else {F32: 2e-5, BF16: 1.5e-2}[dtype]
    err = float((got - want).abs().max())
    scale = max(1e-6, float(want.abs().max()))
    assert err <= tol * scale, f"{what}: max |diff| {err:.3e} > {tol} * {scale:.3e}"


# ---- the norm in groups ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,groups", [(1, 40, 5), (9, 256, 4), (70, 1024, 1), (5, 3000, 3), (33, 97, 97), (3, 96, 2), (600, 384, 3)])
def test_group_norm_of_rows_and_of_chosen_rows(ops, dtype, T, W, groups):
    """Every part is divided by its own root mean square: a part a hundred times as large as the others comes out as
    large as they do.  Whole rows and chosen rows, into float32 and into the compute type."""
    g = torch.Generator().manual_seed(T + W)
    x = torch.randn(T, W, generator=g)
    x[:, :W // groups] *= 100.0
    w = 1.0 + 0.3 * torch.randn(W, generator=g)
    eps = 1e-5
    want = plain.group_rms_norm(x.double(), w.double(), groups, eps)
    for out_dtype in (F32, dtype):
        out = torch.empty(T, W, dtype=out_dtype, device=DEV)
        ops.group_rmsnorm(x.to(DEV), None, w.to(DEV), eps, groups, out)
        _close(out, want, out_dtype, f"rows into {out_dtype}")
    if groups > 1:
        assert float(out[:, :W // groups].float().abs().mean()) < 3.0 * float(out[:, W // groups:].float().abs().mean())
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    out = torch.empty(3, W, dtype=dtype, device=DEV)
    ops.group_rmsnorm(x.to(DEV), rows, w.to(DEV), eps, groups, out)
    _close(out, want[[T - 1, 0, T // 2]], dtype, "chosen rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,groups", [(1, 40, 5), (9, 256, 4), (70, 1024, 1), (5, 3000, 3), (33, 97, 1), (520, 384, 6)])
def test_a_sublayers_way_back_with_the_next_norm_in_the_same_pass(ops, dtype, T, W, groups):
    g = torch.Generator().manual_seed(T * W)
    src = torch.randn(T, W, generator=g)
    branch = (3.0 * torch.randn(T, W, generator=g)).to(dtype)
    w = 0.5 * (1.0 + 0.3 * torch.randn(W, generator=g))
    w2 = 1.0 + 0.3 * torch.randn(W, generator=g)
    eps = 1e-6
    res = src.double() + plain.group_rms_norm(branch.double(), w.double(), groups, eps)
    nxt = plain.group_rms_norm(res, w2.double(), groups, eps)
    for next_dtype in (None, F32, dtype):
        dst = src.clone().to(DEV)
        out = None if next_dtype is None else torch.empty(T, W, dtype=next_dtype, device=DEV)
        ops.group_norm_add(dst, branch.to(DEV), w.to(DEV), eps, groups, dst, w2.to(DEV) if out is not None else None, out)
        _close(dst, res, F32, "the stream", tol=2e-6)
        if out is not None:
            _close(out, nxt, next_dtype, f"the next norm into {next_dtype}")
    other = torch.empty(T, W, device=DEV)
    ops.group_norm_add(src.to(DEV), branch.to(DEV), w.to(DEV), eps, groups, other)
    _close(other, res, F32, "not in place", tol=2e-6)


# ---- heads mixed and gated ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,G,D", [(1, 4, 2, 16), (9, 3, 3, 24), (70, 8, 4, 128), (33, 6, 1, 20), (5, 2, 2, 80)])
def test_heads_mixed_and_gated(ops, dtype, T, H, G, D):
    g = torch.Generator().manual_seed(T + H + D)
    partial = torch.randn(G, T, H * D, generator=g).to(dtype)
    mix = torch.randn(H, H, generator=g)
    wide = torch.randn(T, H + 11, generator=g).to(dtype)          # the gate's columns sit inside a wider row
    gate = wide[:, 3:3 + H]
    for use_mix, use_gate in ((True, True), (True, False), (False, True)):
        p = partial if use_mix else partial[:1]
        want = torch.empty(T, H * D, dtype=F32)
        ref_ops.head_mix_gate(p.float(), mix if use_mix else None, gate.float() if use_gate else None, want, H, G, D)
        out = torch.zeros(T, H * D + 8, dtype=dtype, device=DEV)[:, :H * D]
        ops.head_mix_gate(p.contiguous().to(DEV), mix.to(DEV) if use_mix else None, wide.to(DEV)[:, 3:3 + H] if use_gate else None,
                          out, H, G, D)
        _close(out, want, dtype, f"mix {use_mix} gate {use_gate}")


# ---- the router and the experts ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,E,top", [(1, 40, 2, 1), (9, 64, 7, 3), (70, 96, 20, 2), (33, 50, 200, 8), (5, 32, 4, 4)])
def test_router_that_scores_every_expert_alone(ops, dtype, T, W, E, top):
    g = torch.Generator().manual_seed(E + top)
    x = torch.randn(T, W, generator=g).to(dtype)
    w = torch.randn(E, W, generator=g) * 0.3
    z = x.double() @ w.double().t()
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(T, top, dtype=F32, device=DEV)
    ops.moe_route(x.to(DEV), w.to(DEV), None, idx, wt, scoring="sigmoid")
    val, want_idx = torch.topk(z, top, dim=-1)
    assert torch.equal(idx.cpu().long(), want_idx)
    _close(wt, torch.sigmoid(val), F32, "weights", tol=1e-5)
    assert top == 1 or float(wt.sum(dim=-1).sub(1.0).abs().max()) > 1e-3      # the weights do not sum to one


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,I,E,top", [(1, 40, 12, 2, 2), (9, 64, 24, 5, 3), (300, 96, 72, 3, 1), (70, 128, 64, 16, 2), (33, 50, 20, 4, 4)])
def test_experts_that_read_their_weighted_input(ops, dtype, T, W, I, E, top):
    """expert(w h) is not w expert(h): weights far from one show which of the two is computed."""
    from qwen_engine_b200.parts.base import Arena
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    wgu = (torch.randn(E, 2 * I, W, generator=g) * 0.2).to(dtype)
    wd = (torch.randn(E, W, I, generator=g) * 0.2).to(dtype)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wt = 0.2 + 2.5 * torch.rand(T, top, generator=g)
    want = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            h = float(wt[t, j]) * x[t].double()
            gu = wgu[e].double() @ h
            want[t] += wd[e].double() @ (plain.silu(gu[:I]) * gu[I:])
    out = torch.empty(T, W, dtype=dtype, device=DEV)
    arena = Arena(DEV, 1 << 24)
    ops.moe_experts(x.to(DEV), idx.to(DEV), wt.to(DEV), wgu.to(DEV), wd.to(DEV), out, "silu", arena.alloc, weight_inputs=True)
    _close(out, want, dtype, "experts", tol={F32: 5e-5, BF16: 3e-2}[dtype])
    other = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.moe_experts(x.to(DEV), idx.to(DEV), wt.to(DEV), wgu.to(DEV), wd.to(DEV), other, "silu", arena.alloc)
    assert float((other.float() - out.float()).abs().max()) > 0.05 * float(want.abs().max())


# ---- rotation with a magnitude, values shared across layers, the cache write -------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,R,P", [(4, 2, 16, 8, 4), (3, 3, 24, 24, 8), (2, 1, 80, 40, 16), (4, 2, 128, 128, 16), (1, 1, 20, 6, 8)])
def test_rotation_magnitude_and_blended_values_into_the_cache(ops, dtype, H, G, D, R, P):
    T, pages = 37, 16           # (pages x P slots: more than tokens for every P)
    g = torch.Generator().manual_seed(D + R)
    qkv = torch.randn(T, (H + 2 * G) * D + 8, generator=g).to(dtype)
    pos = torch.randint(0, 5000, (T,), generator=g).to(torch.int32)
    inv = torch.rand(R // 2, generator=g)
    slots = torch.randperm(pages * P, generator=g)[:T].to(torch.int32)
    mag, lam = 1.27, 0.35
    dv = D // 2 if P == 4 or D == 80 else D               # kept values may have fewer channels than the padded head
    first = torch.randn(T, G * dv, generator=g).to(dtype)
    for mode in ("keep", "blend", None):
        cache = torch.full((pages, 2, G, P, D), 7.0, dtype=dtype, device=DEV)
        rows = qkv.clone().to(DEV)
        kept = torch.zeros(T, G * dv, dtype=dtype, device=DEV) if mode == "keep" else first.clone().to(DEV)
        vm = None if mode is None else ("keep", kept) if mode == "keep" else ("blend", kept, lam)
        ops.qk_norm_rope_kv_write(rows[:, :(H + 2 * G) * D], pos.to(DEV), None, None, 0.0, inv.to(DEV), R, cache, slots.to(DEV), H, G, D,
                                  magnitude=mag, value_mix=vm)
        q = qkv[:, :H * D].reshape(T, H, D).double()
        k = qkv[:, H * D:(H + G) * D].reshape(T, G, D).double()
        v = qkv[:, (H + G) * D:(H + 2 * G) * D].reshape(T, G, D).double()
        want_q = plain.rotate(q, pos, inv.double(), mag, R, interleaved=False)
        want_k = plain.rotate(k, pos, inv.double(), mag, R, interleaved=False)
        tol = {F32: 2e-4, BF16: 1.5e-2}[dtype]              # (float32 angles of positions in the thousands)
        _close(rows[:, :H * D], want_q.reshape(T, H * D), dtype, "q", tol=tol)
        _close(rows[:, H * D:(H + G) * D], want_k.reshape(T, G * D), dtype, "k", tol=tol)
        want_v = v
        if mode == "blend":
            padded = torch.zeros(T, G, D, dtype=F64)
            padded[:, :, :dv] = first.double().reshape(T, G, dv)
            want_v = plain.mixed_values(v, padded, lam)
        page, off = slots.long() // P, slots.long() % P
        _close(cache[page, 0, :, off], want_k, dtype, "cached keys", tol=tol)
        _close(cache[page, 1, :, off], want_v, dtype, f"cached values ({mode})")
        if mode == "keep":
            assert torch.equal(kept.cpu().reshape(T, G, dv), qkv[:, (H + G) * D:(H + 2 * G) * D].reshape(T, G, D)[:, :, :dv])
        untouched = torch.ones(pages * P, dtype=torch.bool)
        untouched[slots.long()] = False
        assert bool((cache.reshape(pages, 2, G, P, D).permute(0, 3, 1, 2, 4).reshape(pages * P, -1)[untouched.to(DEV)] == 7.0).all())


# ---- attention's scores: bent, with a sink, over another kv head's values ----------------------------------------------
def _attention_case(ops, dtype, H, G, D, P, q_lens, ctx_lens, softcap, sink, shift, seed, sharp=None):
    """Requests with contexts in the cache and new queries; the kernels against the plain operation.  ``sharp``:
    (request, key position): that key is made to point where the request's last query points, five times as long."""
    from qwen_engine_b200.engine.runner import ModelRunner
    from qwen_engine_b200.parts.base import Arena
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    blocks = [-(-t // P) for t in totals]
    pages = sum(blocks) + 3
    order = torch.randperm(pages, generator=g).tolist()
    tables = torch.full((R, max(blocks)), -1, dtype=torch.int32)
    cache = torch.zeros(pages, 2, G, P, D, dtype=dtype)
    T = sum(q_lens)
    qkv = torch.randn(T, (H + 2 * G) * D, generator=g).to(dtype)
    at = 0
    for r in range(R):
        tables[r, :blocks[r]] = torch.tensor([order.pop() for _ in range(blocks[r])], dtype=torch.int32)
        kv = torch.randn(totals[r], 2, G, D, generator=g)
        if sharp is not None and sharp[0] == r:
            last_q = qkv[sum(q_lens[:r + 1]) - 1, :H * D].float().reshape(H, D)
            for c in range(G):
                kv[sharp[1], 0, c] = 5.0 * last_q[c * (H // G)]
            kv[sharp[1], 1] = 3.0
        for j in range(totals[r]):
            cache[tables[r, j // P], :, :, j % P] = kv[j].to(dtype)
    geo = (H, G, D, 0)
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, (geo,), dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    devplan = ModelRunner._device_plan(plan, {"plan_" + k: i32(v) for k, v in plan.items()}, (geo,))
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    ctx = SimpleNamespace(cu_q=i32(cu), ctx_lens=i32(list(ctx_lens)), q_lens_host=list(q_lens), ctx_lens_host=list(ctx_lens),
                          attn_plan=devplan, arena=Arena(DEV, 1 << 26))
    sinks = torch.randn(H, generator=g) * 2.0 if sink else None
    out = torch.empty(T, H * D, dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(D)
    ops.paged_attention(qkv.to(DEV), cache.to(DEV), tables.to(DEV), ctx, out, scale, 0, H, G, D, softcap=softcap,
                        sinks=None if sinks is None else sinks.to(DEV), value_shift=shift)
    torch.cuda.synchronize()
    want = torch.empty(T, H * D, dtype=F32)
    cpu_ctx = SimpleNamespace(cu_q=torch.tensor(cu), ctx_lens=torch.tensor(list(ctx_lens)))
    ref_ops.paged_attention(qkv.float(), cache.float(), tables, cpu_ctx, want, scale, 0, H, G, D, softcap=softcap, sinks=sinks,
                            value_shift=shift)
    return out, want, ops.last_attention_kernel


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 80, 16), (8, 4, 128, 16), (3, 3, 32, 8), (6, 1, 64, 4), (2, 2, 20, 8)])
@pytest.mark.parametrize("softcap,sink,shift", [(0.0, False, 0), (1.5, False, 0), (0.0, True, 0), (0.0, True, 1), (2.0, True, 0)])
def test_attention_scores_bent_sunk_and_shifted(ops, dtype, H, G, D, P, softcap, sink, shift):
    """Prompt portions behind contexts beside decoded tokens (one far back in a long context, which the kernels cut into
    parts), with a key five times as long as the others where a query points: unbent it takes the whole row, bent it
    takes a share that the cap decides."""
    shift = shift % G
    q_lens, ctx_lens = [70, 1, 5, 1, 33], [0, 900, 61, 15, 200]
    out, want, kernel = _attention_case(ops, dtype, H, G, D, P, q_lens, ctx_lens, softcap, sink, shift, 11, sharp=(1, 3 * P))
    _close(out, want, dtype, f"{kernel}", tol={F32: 3e-5, BF16: 2e-2}[dtype])
    if dtype == BF16 and D % 16 == 0:
        assert kernel != "paged_attention_generic"
    # the row of the sharpened key: unbent and without a sink it is that key's value; a cap or a sink takes its share
    row = want[70, :D]
    if softcap == 0.0 and not sink:
        assert float((row - 3.0).abs().max()) < 1e-3
    elif softcap > 0.0:
        assert float(row.abs().max()) < 2.0


@pytest.mark.parametrize("softcap,sink,shift", [(0.0, False, 0), (4.0, False, 0), (0.0, True, 3), (2.5, True, 1)])
def test_long_portions_at_head_size_128_on_the_tensor_memory_kernel(ops, softcap, sink, shift):
    """Portions long enough for the tcgen05 kernel, whose tiles are cut into parts behind long contexts and merged (the
    sink joins the merged denominator once), beside decoded tokens on the kernel for few rows; the same options."""
    from helpers import LaunchSpy
    H, G, D, P = 8, 4, 128, 16
    with LaunchSpy() as spy:
        out, want, kernel = _attention_case(ops, BF16, H, G, D, P, [300, 64, 1, 130, 1], [1000, 0, 3000, 77, 40], softcap, sink, shift, 21,
                                            sharp=(0, 5 * P))
    _close(out, want, BF16, kernel, tol=2e-2)
    assert spy.count("qe_flash_attention_tc") == 1 and spy.count("qe_decode_attention_mma") + spy.count("qe_flash_attention_fused_merge") == 1


@pytest.mark.parametrize("H,G,D,P", [(8, 4, 128, 16), (4, 2, 80, 16), (6, 3, 32, 8)])
def test_all_shifts_of_decoded_tokens_in_one_launch(ops, H, G, D, P):
    """Steps without a long portion: every shift of the values' kv head as one launch, each with its own output, parts and
    counters, what one launch per shift gives; contexts short, split into parts, and of a few rows."""
    from helpers import LaunchSpy
    from qwen_engine_b200.engine.runner import ModelRunner
    from qwen_engine_b200.parts.base import Arena
    g = torch.Generator().manual_seed(D)
    q_lens, ctx_lens = [1, 1, 3, 1, 2], [0, 2700, 40, 600, 1300]
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    blocks = [-(-t // P) for t in totals]
    tables = torch.full((len(q_lens), max(blocks)), -1, dtype=torch.int32)
    at = 0
    for r, b in enumerate(blocks):
        tables[r, :b] = torch.arange(at, at + b, dtype=torch.int32)
        at += b
    cache = torch.randn(at, 2, G, P, D, generator=g).to(BF16).to(DEV)
    T = sum(q_lens)
    qkv = torch.randn(T, (H + 2 * G) * D, generator=g).to(BF16).to(DEV)
    sinks = (torch.randn(H, generator=g) * 2.0).to(DEV)
    geo = (H, G, D, 0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    outs = []
    for one in (True, False):
        ops.SHIFTS_IN_ONE_LAUNCH = one
        try:
            for splits in (None, {geo: 4}):
                plan = ops.plan_attention(q_lens, ctx_lens, P, (geo,), BF16, uniform_splits=splits)
                devplan = ModelRunner._device_plan(plan, {"plan_" + k: i32(v) for k, v in plan.items()}, (geo,))
                ctx = SimpleNamespace(cu_q=i32(cu), ctx_lens=i32(ctx_lens), q_lens_host=q_lens, ctx_lens_host=ctx_lens, attn_plan=devplan,
                                      arena=Arena(DEV, 1 << 26))
                out = torch.zeros(G, T, H * D, dtype=BF16, device=DEV)
                with LaunchSpy() as spy:
                    ops.paged_attention(qkv, cache, tables.to(DEV), ctx, out, D ** -0.5, 0, H, G, D, softcap=5.0, sinks=sinks, value_shifts=G)
                torch.cuda.synchronize()
                assert spy.count("qe_decode_attention_mma") + spy.count("qe_flash_attention_fused_merge") == (1 if one else G)
                outs.append(out.float().cpu())
        finally:
            ops.SHIFTS_IN_ONE_LAUNCH = True
    # (to rounding: with more CTAs in the launch the kernel may take CTAs of fewer warps, which add a context's keys in another order)
    _close(outs[0], outs[2], BF16, "one launch against one a shift", tol=1e-2)
    _close(outs[1], outs[3], BF16, "one launch against one a shift, four parts a request", tol=1e-2)
    want = torch.empty(G, T, H * D, dtype=F32)
    cpu_ctx = SimpleNamespace(cu_q=torch.tensor(cu), ctx_lens=torch.tensor(ctx_lens))
    ref_ops.paged_attention(qkv.float().cpu(), cache.float().cpu(), tables, cpu_ctx, want, D ** -0.5, 0, H, G, D, softcap=5.0, sinks=sinks.cpu(),
                            value_shifts=G)
    _close(outs[0], want, BF16, "one launch", tol=2e-2)
    _close(outs[1], want, BF16, "one launch, four parts a request", tol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_single_decoded_tokens_alone_and_from_the_first_token(ops, dtype):
    """Steps of single tokens only (the kernels' layout for few rows, contexts in parts that are merged with the sink):
    contexts of 0, 1, a page less one, a page, and thousands of keys."""
    for H, G, D, P in ((4, 2, 80, 16), (8, 2, 128, 16), (2, 1, 48, 8)):
        ctx_lens = [0, 1, P - 1, P, 2500, 700]
        out, want, kernel = _attention_case(ops, dtype, H, G, D, P, [1] * 6, ctx_lens, 3.0, True, 0, 5, sharp=(4, P))
        _close(out, want, dtype, kernel, tol={F32: 3e-5, BF16: 2e-2}[dtype])
        out, want, kernel = _attention_case(ops, dtype, H, G, D, P, [1] * 6, ctx_lens, 0.0, True, G - 1, 6, sharp=(5, 2 * P - 1))
        _close(out, want, dtype, kernel, tol={F32: 3e-5, BF16: 2e-2}[dtype])


# ---- the mixers through their cache ----------------------------------------------------------------------------------------
class _Dict:
    def __init__(self, d):
        self.d = d

    def names(self):
        return self.d.keys()

    def shape(self, n):
        return tuple(self.d[n].shape)

    def get(self, n):
        return self.d[n]


def _run_mixer(ops, mixer, x, dtype, P, portions, extras_in=None):
    """The mixer alone over one request cut into ``portions``, through a cache of its own; its output rows."""
    from qwen_engine_b200.cache.manager import CacheManager
    from qwen_engine_b200.engine.runner import ModelRunner
    from qwen_engine_b200.parts.base import Arena, GroupStepView, StepContext
    cache = CacheManager([mixer.cache_spec()], P, -(-sum(portions) // P) + 2, 4, dtype, DEV, poison=1.0e4)
    rc = cache.open("r")
    geo = mixer.attention_geometry()
    rows, done = [], 0
    for n in portions:
        toks = [0] * n
        cache.append(rc, toks)
        plan = ops.plan_attention([n], [done], P, (geo,), dtype)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        devplan = ModelRunner._device_plan(plan, {"plan_" + k: i32(v) for k, v in plan.items()}, (geo,))
        table = rc.tables[0]
        ctx = StepContext(num_tokens=n, num_reqs=1, dtype=dtype, device=torch.device(DEV), page_size=P, token_ids=i32(toks),
                          positions=i32(list(range(done, done + n))), cu_q=i32([0, n]), ctx_lens=i32([done]), slot_ids=i32([0]),
                          logit_rows=i32([0]), num_logit_rows=0,
                          groups={0: GroupStepView(i32(table).view(1, len(table)), i32(cache.slot_mapping(rc, 0)), len(table))},
                          q_lens_host=[n], ctx_lens_host=[done], arena=Arena(DEV, 1 << 26), attn_plan=devplan)
        if extras_in is not None:
            ctx.extras["shared_values"] = extras_in[done:done + n].to(DEV).contiguous()
        out = torch.empty(n, x.shape[1], dtype=dtype, device=DEV)
        mixer.forward(ctx, x[done:done + n].to(DEV), cache.layer_view(0), 0, out, True)
        torch.cuda.synchronize()
        cache.commit(rc)
        rows.append(out.float().cpu())
        done += n
    return torch.cat(rows)


def _mixer_and_weights(kind, m, W, dtype, seed, value_mix):
    from qwen_engine_b200.config.pufivik_config import PufivikConfig
    from qwen_engine_b200.models.pufivik import _mixer
    cfg = PufivikConfig(vocab=10, width=W)
    mixer = _mixer(cfg, dict(type=kind, mixer=m), value_mix).build("mixer")
    g = torch.Generator().manual_seed(seed)
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    std = 1.0 / math.sqrt(W)
    w = {"q": torch.randn(H * D, W, generator=g) * std, "k": torch.randn(G * D, W, generator=g) * std,
         "v": torch.randn(G * Dv, W, generator=g) * std, "o": torch.randn(W, H * Dv, generator=g) / math.sqrt(H * Dv),
         "vmix": torch.tensor(0.4)}
    if kind == "attention":
        w.update(sink=torch.randn(H, generator=g) * 2.0, talk=torch.eye(H) + 0.5 * torch.randn(H, H, generator=g),
                 g=torch.randn(H, W, generator=g) * std * 3.0)
    w = {k: v.to(BF16).float() for k, v in w.items()}
    mixer.load("", _Dict(w), dtype, DEV)
    return mixer, w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,H,G,D,Dv,R,P", [("attention", 4, 2, 80, 48, 40, 16), ("attention", 8, 4, 128, 128, 64, 16), ("attention", 3, 3, 16, 40, 16, 8),
                                               ("attention_2", 4, 2, 80, 48, 40, 16), ("attention_2", 4, 1, 128, 64, 128, 16), ("attention_2", 2, 2, 24, 8, 6, 4)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_mixer_through_its_cache_with_a_far_key_that_stands_out(ops, dtype, kind, H, G, D, Dv, R, P, decoded):
    """Every row of 700 tokens against the plain mixer, cut into a long portion and a short one or into a prompt and
    single tokens; the input of one token far back (a page's first place) is made so that its keys point where the last
    token's queries point and are several times as long, so the last row is decided by that key, by the cap on its
    score and by the sink.  Values are blended with given ones (a layer that shares them)."""
    W, total, far = 160, 700, 3 * P
    rot = (dict(base=10000.0, dims=R, scaling=dict(factor=4.0, low=1.0, high=4.0, original=256)) if kind == "attention" else
           dict(base=10000.0, dims=R, scaling=dict(factor=4.0, original=256, fast=32.0, slow=1.0)))
    m = dict(heads=H, kv_heads=G, dim=D, vdim=Dv, scale=4.0 / math.sqrt(D), rot=rot, v_mix=True)
    if kind == "attention_2":
        m["softcap"] = 6.0
    mixer, w = _mixer_and_weights(kind, m, W, dtype, D + Dv, "blend")
    g = torch.Generator().manual_seed(H)
    x = torch.randn(total, W, generator=g)
    # the far token's input: the one whose keys (before rotation) equal the last token's queries of each group's first head
    q_last = (w["q"].double() @ x[-1].double()).reshape(H, D)[::H // G].reshape(G * D)
    x[far] = 3.0 * torch.linalg.lstsq(w["k"].double(), q_last[:, None]).solution[:, 0].float()
    x = x.to(dtype)
    shared_first = torch.randn(total, G, Dv, generator=g).to(dtype)
    shared = {"v_first": shared_first.double()}
    fn = plain.sink_talking_attention if kind == "attention" else plain.capped_attention
    want = fn(x.double(), {k: v.double() for k, v in w.items()}, "", m, shared)
    portions = [total - 25] + [1] * 25 if decoded else [40, total - 42, 2]
    got = _run_mixer(ops, mixer, x, dtype, P, portions, extras_in=shared_first.reshape(total, -1))
    _close(got, want, dtype, f"{kind} {ops.last_attention_kernel}", tol={F32: 1e-4, BF16: 4e-2}[dtype])


# ---- whole models ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,name", [(d, n) for n in ph.PUFIVIK for d in DTYPES])
def test_replay_against_the_plain_model(folders, dtype, name):
    folder = folders[name]
    ph.replay_cases(lambda n: ph.make_replayer(folder, name, dtype, n, poison=1.0e4), folder, name, dtype, f"{name}")


@pytest.mark.parametrize("name", ["p-a", "p-d"])
def test_bfloat16_rows_do_not_depend_on_the_schedule(folders, name):
    """In bfloat16 a row is judged loosely against the plain model; against the engine's own rows of the whole prompt the
    rows of a mixed schedule (portions beside single tokens, slots and pages used again) are judged tightly."""
    from helpers import live_tokens_needed, mixed_steps
    folder = folders[name]
    V = ph.vocab_of(name)
    reqs = {f"m{i}": random_tokens(V, n, 60 + i) for i, n in enumerate([40, 64, 23, 90, 17, 55])}
    steps = mixed_steps(reqs, seed=11)
    got = run_steps(ph.make_replayer(folder, name, BF16, live_tokens_needed(steps, 64), poison=1.0e4), steps)
    for rid, toks in reqs.items():
        whole = run_steps(ph.make_replayer(folder, name, BF16, 128),
                          [{"entries": [{"id": "a", "tokens": toks, "want": list(range(len(toks)))}], "end": ["a"]}])["a"]
        settled = ph.settled_positions(folder, toks, BF16)
        idx = [i for i in sorted(got[rid]) if i in settled]
        if not idx:
            continue
        a, b = torch.stack([got[rid][i] for i in idx]).double(), torch.stack([whole[i] for i in idx]).double()
        d = a - b
        d = d - d.mean(dim=-1, keepdim=True)
        err = d.pow(2).mean(dim=-1).sqrt() / (b - b.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt()
        assert float(err.max()) < 0.1, f"{name} {rid}: position {idx[int(err.argmax())]} differs by {float(err.max()):.3f}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_position_of_a_long_prompt_whole_and_decoded(folders, dtype):
    """Prompts of several pages at all positions: whole, and from the first token on one by one (the steps of single
    tokens are replayed from a CUDA graph): first tokens and pages' borders lie among them, in prompts and in decoding."""
    for name, n in (("p-b", 120), ("p-d", 330)):
        folder = folders[name]
        toks = random_tokens(ph.vocab_of(name), n, 31)
        whole = [{"entries": [{"id": "a", "tokens": toks, "want": list(range(n))}], "end": ["a"]}]
        ph.check_requests(run_steps(ph.make_replayer(folder, name, dtype, 384), whole), folder, {"a": toks}, dtype, f"{name} whole")
        single = [{"entries": [{"id": "a", "tokens": [t], "want": [0]}]} for t in toks]
        rep = ph.make_replayer(folder, name, dtype, 384)
        ph.check_requests(run_steps(rep, single), folder, {"a": toks}, dtype, f"{name} decoded")
        assert rep.runner.num_graph_replays > n // 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions_then_decoded(folders, dtype):
    """600 tokens: whole; and in portions of changing sizes (two tokens among them, cuts inside pages) with the last 40
    tokens one by one, beside a second request that comes and goes (its slot and pages are used again)."""
    name = "p-d"
    folder = folders[name]
    V = ph.vocab_of(name)
    toks, other = random_tokens(V, 600, 3), random_tokens(V, 50, 4)
    want = sorted(set(range(0, 600, 7)) | set(range(560, 600)))
    whole = [{"entries": [{"id": "a", "tokens": toks, "want": want}], "end": ["a"]}]
    ph.check_requests(run_steps(ph.make_replayer(folder, name, dtype, 640), whole), folder, {"a": toks}, dtype, "whole")
    steps, p = [], 0
    for i, n in enumerate([64, 64, 100, 2, 30, 129, 16, 3, 95, 57] + [1] * 40):
        entries = [{"id": "a", "tokens": toks[p:p + n], "want": [w - p for w in want if p <= w < p + n]}]
        if i in (1, 5, 12):
            entries.append({"id": f"b{i}", "tokens": other, "want": [49]})
        steps.append({"entries": entries, "end": [f"b{i}"] if i in (1, 5, 12) else []})
        p += n
    assert p == 600
    rep = ph.make_replayer(folder, name, dtype, 704)
    got = run_steps(rep, steps)
    ph.check_requests(got, folder, {"a": toks, "b1": other, "b5": other, "b12": other}, dtype, "portions")


def test_greedy_generation_through_the_engine(folders):
    from qwen_engine_b200.sampling.params import SamplingParams
    for name in ("p-a", "p-c"):
        folder = folders[name]
        cfg, w = ph.plain_model(folder)
        V = ph.vocab_of(name)
        prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26, 47])]
        eng = ph.make_engine(folder, name, F32, max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
        ids = [eng.add_request(p, SamplingParams(max_new_tokens=8, temperature=0.0)) for p in prompts]
        outs = {o.request_id: o for o in eng.serving()}
        for rid, p in zip(ids, prompts):
            assert list(outs[rid].output_token_ids) == plain.greedy(cfg, w, p, 8), f"{name}: prompt of {len(p)} tokens"
        assert eng.cache.slots.num_free == eng.cache.slots.num_slots and eng.cache.pages_in_use() == 0


def test_the_command_line_replays_a_trace(folders, tmp_path):
    name = "p-c"
    folder = folders[name]
    toks = random_tokens(ph.vocab_of(name), 30, 8)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[21:23], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[23:], "want": [6]}, {"id": "y", "tokens": toks[:4], "want": [3]}],
              "end": ["x", "y"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    V = ph.vocab_of(name)
    want = ph.plain_logits(folder, toks)
    first = torch.frombuffer(bytearray((out / "0.f32").read_bytes()), dtype=F32).reshape(-1, V)
    last = torch.frombuffer(bytearray((out / "2.f32").read_bytes()), dtype=F32).reshape(-1, V)
    ph.assert_close_rows(first, want[[0, 20]], F32, "step 0")
    ph.assert_close_rows(last, torch.stack([want[29], want[3]]), F32, "step 2")
