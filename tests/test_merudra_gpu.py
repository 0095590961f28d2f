"""Merudra on the GPU: each new kernel alone against the plain function of its mechanism
(tests/plain_merudra.py), then whole models through replay, the engine and the command line."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import merudra_helpers as mh
import plain_merudra as plain
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
    root = tmp_path_factory.mktemp("merudra_gpu")
    return {name: mh.make_folder(str(root / name), name) for name in mh.MERUDRA}


def _close(got, want, dtype, what="", tol=None):
    got, want = got.detach().to("cpu", F64), want.to(F64)
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    tol = tol if tol is not None else {F32: 2e-5, BF16: 1.5e-2}[dtype]
    err = float((got - want).abs().max())
    scale = max(1e-6, float(want.abs().max()))
    assert err <= tol * scale, f"{what}: max |diff| {err:.3e} > {tol} * {scale:.3e}"


def _ctx(q_lens, ctx_lens, slots, plan=None):
    from qwen_engine_b200.parts.base import Arena
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(cu_q=i32(cu), ctx_lens=i32(ctx_lens), slot_ids=i32(slots), num_reqs=len(q_lens),
                           max_q_len=max(q_lens), q_lens_host=list(q_lens), ctx_lens_host=list(ctx_lens),
                           attn_plan=plan, arena=Arena(DEV))


# three steps that cut four unequal requests differently: (tokens of each request in the step)
CUTS = [[5, 1, 40, 2], [1, 33, 2, 0], [17, 1, 1, 9]]
SLOTS = [2, 0, 3, 1]


def _rows_of(cuts, r):
    return [(sum(step[:r]), step[r]) for step in cuts], sum(step[r] for step in cuts)


# ---- what a sublayer reads: the stream and its short convolution ------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps", [(5, 1), (40, 2), (130, 3), (132, 4), (24, 5), (300, 16)])
def test_stream_convolution_in_portions_through_used_slots(ops, dtype, C, taps):
    """Four unequal requests cut differently into three steps (portions shorter than the window among them), through
    slots that held other requests' rows: every row is the stream plus its convolution over the request's own rows."""
    g = torch.Generator().manual_seed(C + taps)
    w = torch.randn(C, taps, generator=g)
    state = torch.full((4, taps - 1, C), 50.0, device=DEV) if taps > 1 else None
    seqs = [torch.randn(_rows_of(CUTS, r)[1], C, generator=g) for r in range(4)]
    done = [0] * 4
    got, got_plain = [[] for _ in range(4)], [[] for _ in range(4)]
    for step in CUTS:
        live = [r for r in range(4) if step[r] > 0]
        x = torch.cat([seqs[r][done[r]:done[r] + step[r]] for r in live]).to(DEV)
        ctx = _ctx([step[r] for r in live], [done[r] for r in live], [SLOTS[r] for r in live])
        out_plain = torch.empty(x.shape, dtype=dtype, device=DEV)
        out_conv = torch.empty(x.shape, dtype=dtype, device=DEV)
        ops.stream_conv(x, w.to(DEV), state, ctx, out_plain, out_conv)
        row = 0
        for r in live:
            got[r].append(out_conv[row:row + step[r]].float().cpu())
            got_plain[r].append(out_plain[row:row + step[r]].float().cpu())
            row += step[r]
            done[r] += step[r]
    for r in range(4):
        want = seqs[r].double() + plain.causal_conv(seqs[r].double(), w.double())
        _close(torch.cat(got[r]), want, dtype, f"request {r}", tol={F32: 3e-6, BF16: 8e-3}[dtype])
        assert torch.equal(torch.cat(got_plain[r]), seqs[r].to(dtype).float())
        if taps > 1:
            tail = seqs[r][-(taps - 1):]
            assert torch.equal(state[SLOTS[r]].cpu()[-tail.shape[0]:], tail)


def test_stream_convolution_reads_a_state_it_does_not_write(ops):
    C, taps = 64, 4
    g = torch.Generator().manual_seed(1)
    w, x = torch.randn(C, taps, generator=g).to(DEV), torch.randn(6, C, generator=g).to(DEV)
    state = torch.randn(2, taps - 1, C, generator=g).to(DEV)
    before = state.clone()
    out = torch.empty(6, C, dtype=F32, device=DEV)
    ops.stream_conv(x, w, state, _ctx([6], [9], [1]), None, out, write_state=False)
    assert torch.equal(state, before)
    seq = torch.cat([before[1].cpu(), x.cpu()]).double()
    _close(out, (seq + plain.causal_conv(seq, w.cpu().double()))[taps - 1:], F32, "behind a state", tol=3e-6)


# ---- a sublayer's way back --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,gated", [(1, 40, True), (9, 256, True), (70, 1024, True), (5, 3000, True), (33, 97, False),
                                         (700, 512, True), (530, 2048, True), (600, 136, False), (513, 4100, True)])
def test_gated_norm_add(ops, dtype, T, W, gated):
    g = torch.Generator().manual_seed(T + W)
    src = torch.randn(T, W, generator=g)
    branch = (3.0 * torch.randn(T, W, generator=g)).to(dtype)
    gate = (2.0 * torch.randn(T, W, generator=g)).to(dtype) if gated else None
    bias = torch.randn(W, generator=g) if gated else None
    weight = 1.0 + 0.3 * torch.randn(W, generator=g)
    eps = 1e-5
    dst = torch.empty(T, W, dtype=F32, device=DEV)
    cast = torch.empty(T, W, dtype=dtype, device=DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    ops.gated_norm_add(dev(src), dev(branch), dev(gate), dev(bias), dev(weight), eps, dst, cast)
    v = branch.double()
    if gated:
        v = v * torch.sigmoid(gate.double() + bias.double())
    want = src.double() + plain.rms(v, eps) * weight.double()
    _close(dst, want, F32, "dst", tol=2e-6)
    assert torch.equal(cast.float(), dst.to(dtype).float())
    # in place: the source is the destination
    both = dev(src).clone()
    ops.gated_norm_add(both, dev(branch), dev(gate), dev(bias), dev(weight), eps, both)
    assert torch.equal(both, dst)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("L,T,W", [(1, 3, 40), (4, 9, 256), (7, 33, 97), (3, 70, 1024), (2, 520, 256)])
def test_the_last_add_of_a_layer_also_forms_the_weighted_sum(ops, dtype, L, T, W):
    """The add into entry L of the layers' results, and the weighted sum over entries 0 .. L in the same launch: as the
    add alone followed by the sum alone, to the bit."""
    g = torch.Generator().manual_seed(L + T + W)
    hist = torch.randn(L + 2, T, W, generator=g).to(DEV)
    branch = torch.randn(T, W, generator=g).to(dtype).to(DEV)
    weight = (1.0 + 0.3 * torch.randn(W, generator=g)).to(DEV)
    wts = torch.randn(L + 1, generator=g).to(DEV)
    apart = hist.clone()
    ops.gated_norm_add(apart[L], branch, None, None, weight, 1e-6, apart[L])
    want = torch.empty(T, W, dtype=F32, device=DEV)
    ops.depth_mix(apart, wts, L + 1, want)
    mixed = torch.empty(T, W, dtype=F32, device=DEV)
    ops.gated_norm_add(hist[L], branch, None, None, weight, 1e-6, hist[L], depth_mix=(hist, wts, L + 1, mixed))
    assert torch.equal(hist, apart) and torch.equal(mixed, want)
    ref = sum(wts[j].double().cpu() * apart[j].double().cpu() for j in range(L + 1))
    _close(mixed, ref, F32, "sum", tol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,d,V", [(1, 3, 7), (40, 24, 100), (300, 64, 50), (1, 8, 9), (2500, 16, 33), (40000, 64, 1000)])
def test_token_side_gate(ops, dtype, T, d, V):
    g = torch.Generator().manual_seed(T + d)
    gate = (2.0 * torch.randn(T, d, generator=g)).to(dtype)
    table = torch.randn(V, d, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    out = torch.empty(T, d, dtype=dtype, device=DEV)
    ops.token_side_gate(gate.to(DEV), table.to(DEV), ids.to(DEV), out)
    _close(out, plain.gelu_tanh(gate.double()) * table[ids.long()].double(), dtype, "side", tol={F32: 2e-6, BF16: 8e-3}[dtype])


@pytest.mark.parametrize("L,T,W", [(2, 1, 40), (5, 33, 64), (9, 7, 97), (3, 130, 256)])
def test_weighted_sum_over_the_layers_results(ops, L, T, W):
    g = torch.Generator().manual_seed(L + T)
    hist = torch.randn(L + 2, T, W, generator=g)
    wts = torch.randn(L + 2, generator=g)
    for count in (1, L):
        out = torch.empty(T, W, dtype=F32, device=DEV)
        ops.depth_mix(hist.to(DEV), wts.to(DEV), count, out)
        want = sum(wts[j].double() * hist[j].double() for j in range(count))
        _close(out, want, F32, f"{count} results", tol=2e-6)


# ---- attention whose values are its keys -------------------------------------------------------------------------
def _plain_qk(proj, pos, qb, kb, eps, temp, H, G, D):
    T = proj.shape[0]
    q = (proj[:, :H * D].double() + qb.double()).reshape(T, H, D)
    k = (proj[:, H * D:(H + G) * D].double() + kb.double()).reshape(T, G, D)
    qn = plain.rms(q, eps) * plain.query_temperature(pos, temp[0], temp[1])[:, None, None]
    return qn, plain.rms(k, eps), k


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,P,every", [(4, 2, 16, 4, 4), (3, 3, 24, 8, 1), (2, 1, 64, 16, 7), (4, 2, 128, 16, 64), (1, 1, 200, 16, 1000)])
def test_bias_norm_temperature_and_the_two_planes(ops, dtype, H, G, D, P, every):
    """Positions on both sides of every step of the temperature; the value plane takes the keys with their bias and
    before their norm, the key plane the normed ones; columns behind q and k stay as they are."""
    g = torch.Generator().manual_seed(H * D + every)
    pos = torch.tensor(sorted({0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 2 * every, 5 * every - 1, 900} - {-1, -2}),
                       dtype=torch.int32)
    T = pos.numel()
    extra = 8
    proj = (2.0 * torch.randn(T, (H + G) * D + extra, generator=g)).to(dtype)
    qb, kb = torch.randn(H * D, generator=g), torch.randn(G * D, generator=g)
    n_pages = 6
    pages = torch.full((n_pages, 2, G, P, D), 7.0, dtype=dtype, device=DEV)
    slots = torch.randperm(n_pages * P, generator=g)[:T].to(torch.int32)
    eps, temp = 1e-5, (0.6, every)
    dproj = proj.to(DEV)
    ops.qk_bias_norm_kv_write(dproj, pos.to(DEV), qb.to(DEV), kb.to(DEV), eps, temp, pages, slots.to(DEV), H, G, D)
    qn, kn, kraw = _plain_qk(proj.float(), pos, qb, kb, eps, temp, H, G, D)
    tol = {F32: 3e-6, BF16: 1.2e-2}[dtype]
    _close(dproj[:, :H * D].reshape(T, H, D), qn, dtype, "q", tol=tol)
    _close(dproj[:, H * D:(H + G) * D].reshape(T, G, D), kn, dtype, "k", tol=tol)
    assert torch.equal(dproj[:, (H + G) * D:].cpu(), proj[:, (H + G) * D:])
    page, off = (slots // P).long(), (slots % P).long()
    _close(pages[page, 0, :, off], kn, dtype, "key plane", tol=tol)
    _close(pages[page, 1, :, off], kraw, dtype, "value plane", tol=tol)
    untouched = torch.ones(n_pages, P, dtype=torch.bool)
    untouched[page, off] = False
    assert bool((pages.cpu()[untouched.nonzero()[:, 0], :, :, untouched.nonzero()[:, 1]] == 7.0).all())
    # without the cache write nothing lands in the pages
    fresh = torch.full_like(pages, 7.0)
    ops.qk_bias_norm_kv_write(proj.to(DEV), pos.to(DEV), qb.to(DEV), kb.to(DEV), eps, None, fresh, slots.to(DEV), H, G, D, write_kv=False)
    assert bool((fresh == 7.0).all())


def _attention_mixer(H, G, D, scale, temp, dtype, seed, hidden=64):
    """The mixer alone with weights of its own making: the projections are set so that a test decides q and k."""
    from qwen_engine_b200.parts.base import PartSpec
    spec = PartSpec("gqa_attention", dict(hidden_size=hidden, num_heads=H, num_kv_heads=G, head_dim=D, scale=scale, qk_norm_eps=1e-6,
                                          position_encoding=None, output_gate="sigmoid", tied_values=True, qk_bias=True,
                                          query_temperature=temp, names=dict(q="q", k="k", gate="g", out="o", q_bias="q.b", k_bias="k.b")))
    return spec.build("mixer")


class _Dict:
    def __init__(self, d):
        self.d = d

    def names(self):
        return self.d.keys()

    def shape(self, n):
        return tuple(self.d[n].shape)

    def get(self, n):
        return self.d[n]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 128, 16), (2, 2, 64, 16), (3, 1, 48, 8)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_far_key_decides_the_row_and_its_value_is_the_key_before_the_norm(ops, dtype, H, G, D, P, decoded):
    """Through the mixer and its cache, with weights made so that it shows: the input's first D channels are the query of
    head 0, its next D channels the key of kv head 0.  One key far back (at a page's first place) is five times as long as the others and
    points where the last query points: normed, it is as long as any key, so only its direction wins the softmax; the row's
    output is then the key as projected, five times as long.  In a prompt's portion and for a decoded token."""
    from qwen_engine_b200.cache.manager import CacheManager
    from qwen_engine_b200.engine.runner import ModelRunner
    from qwen_engine_b200.parts.base import Arena, GroupStepView, StepContext
    W = 2 * D
    scale = 30.0 / D                                  # unit-RMS vectors: q . k = D for equal directions
    mixer = _attention_mixer(H, G, D, scale, (0.0, 1), dtype, 1, hidden=W)
    eye = torch.zeros(D, W)
    eye[:, :D] = torch.eye(D)
    wq = torch.zeros(H * D, W)
    wq[:D] = eye
    wk = torch.zeros(G * D, W)
    wk[:D, D:2 * D] = torch.eye(D)
    wo = torch.zeros(W, H * D)
    wo[:D, :D] = torch.eye(D)                          # the output's first D channels are head 0's
    tensors = {"q": wq, "k": wk, "g": torch.zeros(H * D, W), "o": wo, "q.b": torch.zeros(H * D), "k.b": torch.zeros(G * D)}
    mixer.load("", _Dict(tensors), dtype, DEV)
    far, total = 3 * P, 731
    g = torch.Generator().manual_seed(D)
    x = torch.randn(total, W, generator=g)
    d = torch.randn(D, generator=g)
    d = d / d.norm() * math.sqrt(D)
    x[far, D:2 * D] = 5.0 * d
    x[total - 1, :D] = d
    x = x.to(dtype)
    cache = CacheManager([mixer.cache_spec()], P, 128, 4, dtype, DEV, poison=1.0e4)
    rc = cache.open("r")
    out_rows = []
    portions = [total - 1, 1] if decoded else [40, total - 40]
    done = 0
    for n in portions:
        toks = [0] * n
        cache.append(rc, toks)
        plan = ops.plan_attention([n], [done], P, (mixer.attention_geometry(),), dtype)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        devplan = ModelRunner._device_plan(plan, {"plan_" + k: i32(v) for k, v in plan.items()}, (mixer.attention_geometry(),))
        table = rc.tables[0]
        ctx = StepContext(num_tokens=n, num_reqs=1, dtype=dtype, device=torch.device(DEV), page_size=P, token_ids=i32(toks),
                          positions=i32(list(range(done, done + n))), cu_q=i32([0, n]), ctx_lens=i32([done]), slot_ids=i32([0]),
                          logit_rows=i32([0]), num_logit_rows=0,
                          groups={0: GroupStepView(i32(table).view(1, len(table)), i32(cache.slot_mapping(rc, 0)), len(table))},
                          q_lens_host=[n], ctx_lens_host=[done], arena=Arena(DEV, 1 << 26), attn_plan=devplan)
        out = torch.empty(n, W, dtype=dtype, device=DEV)
        mixer.forward(ctx, x[done:done + n].to(DEV), cache.layer_view(0), 0, out, True)
        torch.cuda.synchronize()
        cache.commit(rc)
        out_rows.append(out.float().cpu())
        done += n
    last = torch.cat(out_rows)[-1, :D]
    want = 0.5 * 5.0 * d                               # the gate's weights are zero: sigmoid(0)
    assert float((last - want).abs().max()) < 0.05 * float(want.abs().max()), ops.last_attention_kernel


# ---- the delta rule with one decay per head ----------------------------------------------------------------------
def _delta_inputs(H, G, dk, dv, T, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    wide = torch.randn(T, 2 * G * dk + H * dv + 3, generator=g)
    q = wide[:, 1:1 + G * dk].reshape(T, G, dk)
    q /= q.norm(dim=-1, keepdim=True) * math.sqrt(dk)
    k = wide[:, 1 + G * dk:1 + 2 * G * dk].reshape(T, G, dk)
    k /= k.norm(dim=-1, keepdim=True)
    small = (1.5 * torch.randn(T, 2 * H + 2, generator=g)).to(dtype)          # beta's and the decay's inputs, side by side
    rate, bias = torch.randn(H, generator=g) - 1.0, torch.randn(H, generator=g)
    return wide, small, rate, bias


def _plain_delta(wide, small, rate, bias, H, G, dk, dv):
    T = wide.shape[0]
    rep = H // G
    q = wide[:, 1:1 + G * dk].double().reshape(T, G, dk).repeat_interleave(rep, dim=1)
    k = wide[:, 1 + G * dk:1 + 2 * G * dk].double().reshape(T, G, dk).repeat_interleave(rep, dim=1)
    v = wide[:, 1 + 2 * G * dk:1 + 2 * G * dk + H * dv].double().reshape(T, H, dv)
    beta = torch.sigmoid(small[:, 1:1 + H].double())
    decay = torch.exp(-torch.exp(rate.double()) * torch.nn.functional.softplus(small[:, 1 + H:1 + 2 * H].double() + bias.double()))
    return plain.delta_recurrence(q, k, v, decay, beta)


def _scan(ops, wide, small, rate, bias, state, ctx, out, H, G, dk, dv, **kw):
    qk = G * dk
    ops.delta_rule_scan(wide[:, 1:1 + qk], wide[:, 1 + qk:1 + 2 * qk], wide[:, 1 + 2 * qk:1 + 2 * qk + H * dv], None,
                        small[:, 1:1 + H], state, ctx, out, H, G, dk, dv, head_decay=(small[:, 1 + H:1 + 2 * H], rate, bias), **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dk,dv", [(2, 2, 64, 64), (4, 2, 8, 12), (3, 1, 6, 10), (2, 2, 12, 4), (4, 2, 128, 64), (1, 1, 40, 130)])
def test_delta_rule_with_a_decay_per_head_in_portions(ops, dtype, H, G, dk, dv):
    state = torch.full((4, H, dv, dk), 9.0, device=DEV)                      # what other requests left in the slots
    ins = [_delta_inputs(H, G, dk, dv, _rows_of(CUTS, r)[1], 10 * r + dk, dtype) for r in range(4)]
    rate, bias = ins[0][2], ins[0][3]
    done = [0] * 4
    got = [[] for _ in range(4)]
    for step in CUTS:
        live = [r for r in range(4) if step[r] > 0]
        cat = lambda i: torch.cat([ins[r][i][done[r]:done[r] + step[r]] for r in live]).to(DEV)
        wide, small = cat(0), cat(1)
        ctx = _ctx([step[r] for r in live], [done[r] for r in live], [SLOTS[r] for r in live])
        out = torch.empty(wide.shape[0], H * dv, dtype=F32, device=DEV)
        _scan(ops, wide, small, rate.to(DEV), bias.to(DEV), state, ctx, out, H, G, dk, dv)
        row = 0
        for r in live:
            got[r].append(out[row:row + step[r]].cpu())
            row += step[r]
            done[r] += step[r]
    for r in range(4):
        o = _plain_delta(ins[r][0], ins[r][1], rate, bias, H, G, dk, dv)
        _close(torch.cat(got[r]).reshape(-1, H, dv), o, F32, f"request {r}", tol=3e-5)


def test_delta_rule_with_a_decay_per_head_long_whole_and_token_by_token_to_the_bit(ops):
    H, G, dk, dv, T = 2, 1, 64, 32, 600
    wide, small, rate, bias = _delta_inputs(H, G, dk, dv, T, 3, F32)
    bias[0], rate[0] = -40.0, -3.0                       # a head that forgets next to nothing: the first tokens stay in its state
    dev = lambda t: t.to(DEV)
    w, s, rt, bs = dev(wide), dev(small), dev(rate), dev(bias)
    state = torch.zeros(1, H, dv, dk, device=DEV)
    whole = torch.empty(T, H * dv, dtype=F32, device=DEV)
    _scan(ops, w, s, rt, bs, state, _ctx([T], [0], [0]), whole, H, G, dk, dv)
    _close(whole.reshape(T, H, dv), _plain_delta(wide, small, rate, bias, H, G, dk, dv), F32, "600 tokens", tol=5e-5)
    state2 = torch.full((1, H, dv, dk), 4.0, device=DEV)
    single = torch.empty(T, H * dv, dtype=F32, device=DEV)
    for t in range(T):
        _scan(ops, w[t:t + 1], s[t:t + 1], rt, bs, state2, _ctx([1], [t], [0]), single[t:t + 1], H, G, dk, dv)
    assert torch.equal(single, whole) and torch.equal(state, state2)


# ---- the router that scores all experts, and experts that hand their input on ------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,E,top", [(1, 40, 2, 1), (9, 64, 7, 3), (70, 96, 20, 2), (33, 50, 200, 8), (5, 32, 4, 4)])
def test_router_over_all_experts_with_a_correction(ops, dtype, T, W, E, top):
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    w = torch.randn(E, W, generator=g) * 0.3
    corr = torch.randn(E, generator=g) * 0.2            # as large as the scores: it changes who is chosen
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wgt = torch.empty(T, top, dtype=F32, device=DEV)
    ops.moe_route(x.to(DEV), w.to(DEV), None, idx, wgt, scoring="softmax_all", correction=corr.to(DEV))
    s = torch.softmax(x.double() @ w.double().T, dim=-1)
    want_idx = torch.topk(s + corr.double(), top, dim=-1).indices
    assert torch.equal(idx.cpu().long(), want_idx)
    _close(wgt, torch.gather(s, 1, want_idx), F32, "weights", tol=1e-5)       # the scores as they are: they do not sum to one
    plain_choice = torch.topk(s, top, dim=-1).indices
    if T * top >= 20 and top < E:
        assert not torch.equal(plain_choice, want_idx)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,I,E,n_id,top", [(1, 40, 12, 2, 1, 2), (9, 64, 24, 5, 2, 3), (300, 96, 72, 3, 4, 2), (70, 128, 64, 16, 4, 2),
                                              (5, 32, 16, 1, 3, 4), (40, 256, 1536, 8, 1, 2)])
def test_experts_among_which_some_hand_their_input_on(ops, dtype, T, W, I, E, n_id, top):
    from qwen_engine_b200.parts.base import Arena
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    w_gate_up = (torch.randn(E, 2 * I, W, generator=g) / math.sqrt(W) * 2).to(dtype)
    w_down = (torch.randn(E, W, I, generator=g) / math.sqrt(I)).to(dtype)
    rows = [torch.randperm(E + n_id, generator=g)[:top].tolist() for _ in range(T)]
    rows[0] = list(range(E + n_id - 1, E + n_id - 1 - top, -1))[:top]            # the first token: identity experts first
    idx = torch.tensor(rows, dtype=torch.int32)
    wgt = torch.rand(T, top, generator=g)
    out = torch.empty(T, W, dtype=dtype, device=DEV)
    arena = Arena(DEV, 1 << 24)
    ops.moe_experts(x.to(DEV), idx.to(DEV), wgt.to(DEV), w_gate_up.to(DEV), w_down.to(DEV), out, "silu", arena.alloc, num_identity=n_id)
    want = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            h = x[t].double()
            y = h if e >= E else (plain.silu(h @ w_gate_up[e, :I].double().T) * (h @ w_gate_up[e, I:].double().T)) @ w_down[e].double().T
            want[t] += wgt[t, j].double() * y
    _close(out, want, dtype, "experts", tol={F32: 2e-5, BF16: 2e-2}[dtype])


# ---- whole models ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,name", [(d, n) for n in mh.MERUDRA for d in DTYPES])
def test_replay_against_the_plain_model(folders, dtype, name):
    folder = folders[name]
    mh.replay_cases(lambda n: mh.make_replayer(folder, name, dtype, n, poison=1.0e4), folder, name, dtype, f"{name}")


@pytest.mark.parametrize("name", ["m-a", "m-d"])
def test_bfloat16_rows_do_not_depend_on_the_schedule(folders, name):
    """In bfloat16 a row is judged loosely against the plain model; against the engine's own rows of the whole prompt the
    rows of a mixed schedule (portions beside single tokens, slots and pages used again) are judged tightly."""
    from helpers import live_tokens_needed, mixed_steps
    folder = folders[name]
    V = mh.vocab_of(name)
    reqs = {f"m{i}": random_tokens(V, n, 60 + i) for i, n in enumerate([40, 64, 23, 90, 17, 55])}
    steps = mixed_steps(reqs, seed=11)
    got = run_steps(mh.make_replayer(folder, name, BF16, live_tokens_needed(steps, 64), poison=1.0e4), steps)
    for rid, toks in reqs.items():
        whole = run_steps(mh.make_replayer(folder, name, BF16, 128),
                          [{"entries": [{"id": "a", "tokens": toks, "want": list(range(len(toks)))}], "end": ["a"]}])["a"]
        settled = mh.settled_positions(folder, toks, BF16)
        idx = [i for i in sorted(got[rid]) if i in settled]
        a, b = torch.stack([got[rid][i] for i in idx]).double(), torch.stack([whole[i] for i in idx]).double()
        d = a - b
        d = d - d.mean(dim=-1, keepdim=True)
        err = d.pow(2).mean(dim=-1).sqrt() / (b - b.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt()
        assert float(err.max()) < 0.1, f"{name} {rid}: position {idx[int(err.argmax())]} differs by {float(err.max()):.3f}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_position_of_a_long_prompt_whole_and_decoded(folders, dtype):
    """Prompts of several pages at all positions: whole, and from the first token on one by one (the steps of single
    tokens are replayed from a CUDA graph): first tokens, pages' borders and the steps of the queries' temperature lie
    among them, in prompts and in decoding."""
    for name, n in (("m-b", 120), ("m-d", 330)):
        folder = folders[name]
        toks = random_tokens(mh.vocab_of(name), n, 31)
        whole = [{"entries": [{"id": "a", "tokens": toks, "want": list(range(n))}], "end": ["a"]}]
        mh.check_requests(run_steps(mh.make_replayer(folder, name, dtype, 384), whole), folder, {"a": toks}, dtype, f"{name} whole")
        single = [{"entries": [{"id": "a", "tokens": [t], "want": [0]}]} for t in toks]
        rep = mh.make_replayer(folder, name, dtype, 384)
        mh.check_requests(run_steps(rep, single), folder, {"a": toks}, dtype, f"{name} decoded")
        assert rep.runner.num_graph_replays > n // 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions_then_decoded(folders, dtype):
    """600 tokens: whole; and in portions of changing sizes (two tokens among them, cuts inside pages) with the last 40
    tokens one by one, beside a second request that comes and goes (its slot and pages are used again)."""
    name = "m-d"
    folder = folders[name]
    V = mh.vocab_of(name)
    toks, other = random_tokens(V, 600, 3), random_tokens(V, 50, 4)
    want = sorted(set(range(0, 600, 7)) | set(range(560, 600)))
    whole = [{"entries": [{"id": "a", "tokens": toks, "want": want}], "end": ["a"]}]
    mh.check_requests(run_steps(mh.make_replayer(folder, name, dtype, 640), whole), folder, {"a": toks}, dtype, "whole")
    steps, p = [], 0
    for i, n in enumerate([64, 64, 100, 2, 30, 129, 16, 3, 95, 57] + [1] * 40):
        entries = [{"id": "a", "tokens": toks[p:p + n], "want": [w - p for w in want if p <= w < p + n]}]
        if i in (1, 5, 12):
            entries.append({"id": f"b{i}", "tokens": other, "want": [49]})
        steps.append({"entries": entries, "end": [f"b{i}"] if i in (1, 5, 12) else []})
        p += n
    assert p == 600
    rep = mh.make_replayer(folder, name, dtype, 704)
    got = run_steps(rep, steps)
    mh.check_requests(got, folder, {"a": toks, "b1": other, "b5": other, "b12": other}, dtype, "portions")


def test_greedy_generation_through_the_engine(folders):
    from qwen_engine_b200.sampling.params import SamplingParams
    for name in ("m-a", "m-c"):
        folder = folders[name]
        cfg, w = mh.plain_model(folder)
        V = mh.vocab_of(name)
        prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26, 47])]
        eng = mh.make_engine(folder, name, F32, max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
        ids = [eng.add_request(p, SamplingParams(max_new_tokens=8, temperature=0.0)) for p in prompts]
        outs = {o.request_id: o for o in eng.serving()}
        for rid, p in zip(ids, prompts):
            assert list(outs[rid].output_token_ids) == plain.greedy(cfg, w, p, 8), f"{name}: prompt of {len(p)} tokens"
        assert eng.cache.slots.num_free == eng.cache.slots.num_slots and eng.cache.pages_in_use() == 0


def test_the_command_line_replays_a_trace(folders, tmp_path):
    name = "m-c"
    folder = folders[name]
    toks = random_tokens(mh.vocab_of(name), 30, 8)
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
    V = mh.vocab_of(name)
    want = mh.plain_logits(folder, toks)
    first = torch.frombuffer(bytearray((out / "0.f32").read_bytes()), dtype=F32).reshape(-1, V)
    last = torch.frombuffer(bytearray((out / "2.f32").read_bytes()), dtype=F32).reshape(-1, V)
    mh.assert_close_rows(first, want[[0, 20]], F32, "step 0")
    mh.assert_close_rows(last, torch.stack([want[29], want[3]]), F32, "step 2")
