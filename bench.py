"""Benchmark of the engine on one B200: decode tokens a second at a fixed batch and context,
prefill tokens a second at 2,048 tokens, for Qwen3-0.6B-shaped random weights.

    python bench.py --gpus 1 --steps K --warmup W        # prints ONE JSON line

A step is one decode step of the whole batch.  ``value`` is timed on the device over the step
function (tokens already on the host side of the step function, no sampling read-back);
``e2e`` is the same through the Python entry point (LLMEngine.step: host tokens in, sampled
tokens out, every step).  ``prefill`` is one 2,048-token prompt to its last logits;
``roofline`` is the decode step's bytes (every weight once, the cache of the live requests)
over its time; ``points`` holds batch 1 and 64.  The step's inputs (1.2 GB of weights plus the
cache) are larger than L2, so successive steps do not find them there.

``--impl reference`` would run kzw3933/Qwen-Engine itself from baseline/_ref; see
``reference_arm``.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(raw)
            peaks = dict(FALLBACK_PEAKS)
            for k in FALLBACK_PEAKS:
                if k in flat:
                    peaks[k] = flat[k]
            return peaks, "measured"
        except Exception:       # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def config_record(model, layers, layers_of_config, hidden, heads, kv_heads, head_dim, intermediate, vocab, batch, context,
                  page_size, prefill_tokens) -> dict:
    """The ``config`` of the JSON line: every size, flat, the same keys for both arms."""
    return {"model": model, "layers": layers, "layers_of_config": layers_of_config, "hidden": hidden, "heads": heads,
            "kv_heads": kv_heads, "head_dim": head_dim, "intermediate": intermediate, "vocab": vocab,
            "global_batch": batch, "seq_len": context, "page_size": page_size, "prefill_tokens": prefill_tokens,
            "l2": "inputs larger than L2", "parallelism": "single GPU"}


class ClockSampler:
    """nvidia-smi in the background during the timed regions (read-only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def mark(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, spans: list[tuple[int, int]]) -> dict:
        rows = [r for a, b in spans for r in self.rows[a:b]] or self.rows
        sm = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(rows)}


def reference_arm(args) -> int:
    """The reference arm: the unmodified kzw3933/Qwen-Engine as installed into baseline/_ref
    (pip install --no-deps --target), through its own classes and stock code path in
    ``mode="triton"``: Qwen3Config defaults (Qwen3-0.6B) -> Qwen3ForCausalLM with its own random
    initialisation -> KVCachePool -> ModelExecutor.run_prefill / run_decode_step -> its argmax
    sampler, i.e. the body of its LLMEngine.serving loop (src/engine/llm_engine.py:101-145) with
    the step count under the benchmark's control.  Token ids stand in for its tokenizer, which needs
    the network.  Nothing of this repository's engine is imported."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "engine")) or not os.path.isdir(os.path.join(ref, "models")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref does not hold the reference's engine and models packages (not installed)"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference is single-GPU"}))
        return 0
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        sys.path.insert(0, ref)
        from engine import KVCachePool                       # the reference's own packages
        from engine.executor import ModelExecutor
        from engine.sequence import Sequence
        from models import Qwen3Config, Qwen3ForCausalLM
        args.warmup = max(args.warmup, 3)
        rng = random.Random(0)
        cfg = Qwen3Config()
        dev = torch.device("cuda:0")
        torch.manual_seed(2)
        t0 = time.time()
        model = Qwen3ForCausalLM(**cfg.to_model_kwargs(), dtype=torch.bfloat16).to(dev).eval()
        print(f"[bench reference] model ready in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
        V, block = cfg.vocab_size, 16
        extra = args.warmup + args.steps + 4
        big = args.batch if args.no_points else max(args.batch, 64)
        blocks = big * (-(-(args.context + 3 * extra) // block) + 1) + args.prefill_tokens // block + 8
        pool = KVCachePool(num_layers=cfg.num_hidden_layers, num_blocks=blocks, block_size=block,
                           num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, dtype=torch.bfloat16, device=dev)
        ex = ModelExecutor(model, pool, dev, mode="triton")
        sid = [0]

        def new_seq(n):
            sid[0] += 1
            return Sequence(sid[0], "", [rng.randrange(V) for _ in range(n)])

        def decode_step(seqs):
            logits = ex.run_decode_step(seqs)                 # llm_engine.py:132-143
            toks = ex.sample_next_tokens(logits)
            for s, t in zip(seqs, toks):
                s.output_token_ids.append(t)
                s.num_computed_tokens += 1
                s.num_kv_tokens += 1
            ex.register_shared_blocks(seqs)

        clocks = ClockSampler()
        clocks.start()
        spans = []
        with torch.no_grad():
            # prefill of one 2,048-token prompt (its executor computes logits for every row)
            def prefill_once():
                s = new_seq(args.prefill_tokens)
                logits, ctx = ex.run_prefill([s])
                ex.sample_next_tokens(ex.gather_prefill_last_logits(logits, ctx.cu_seqlens))
                ex.release_sequence(s)
            for _ in range(2):
                prefill_once()
            torch.cuda.synchronize()
            m0 = clocks.mark()
            t0 = time.perf_counter()
            for _ in range(3):
                prefill_once()
            torch.cuda.synchronize()
            prefill_ms = (time.perf_counter() - t0) / 3 * 1e3
            spans.append((m0, clocks.mark()))

            def decode_rate(batch, steps, warmup):
                seqs = [new_seq(args.context) for _ in range(batch)]
                for i in range(0, batch, 8):
                    group = seqs[i:i + 8]
                    logits, ctx = ex.run_prefill(group)
                    toks = ex.sample_next_tokens(ex.gather_prefill_last_logits(logits, ctx.cu_seqlens))
                    for s, t in zip(group, toks):                # llm_engine.py:115-119
                        s.output_token_ids.append(t)
                        s.num_computed_tokens = s.num_kv_tokens = s.prompt_len
                for _ in range(warmup):
                    decode_step(seqs)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                m = clocks.mark()
                t0 = time.perf_counter()
                a.record()
                for _ in range(steps):
                    decode_step(seqs)
                b.record()
                torch.cuda.synchronize()
                wall = time.perf_counter() - t0
                spans.append((m, clocks.mark()))
                for s in seqs:
                    ex.release_sequence(s)
                return batch * steps / (a.elapsed_time(b) / 1e3), a.elapsed_time(b) / steps, batch * steps / wall
            value, ms_per_step, e2e_value = decode_rate(args.batch, args.steps, args.warmup)
            points = {}
            if not args.no_points:
                points["decode_b1"] = round(decode_rate(1, args.steps, 3)[0], 1)
                points["decode_b64"] = round(decode_rate(64, max(3, args.steps // 4), 2)[0], 1)
        clocks.stop()
        print(json.dumps({
            "metric": "decode tok/s (Qwen3-0.6B, batch 8, context 1024)", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic: uniform random token ids, the reference's own random initialisation",
            "config": config_record("qwen3-0.6b", cfg.num_hidden_layers, cfg.num_hidden_layers, cfg.hidden_size,
                                    cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size,
                                    cfg.vocab_size, args.batch, args.context, block, args.prefill_tokens),
            "mode": "triton",
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s"},
            "prefill": {"value": round(args.prefill_tokens / (prefill_ms / 1e3), 1), "tokens": args.prefill_tokens,
                        "ms": round(prefill_ms, 3)},
            "points": points, "clocks": clocks.summary(spans)}))
        return 0
    except Exception as e:          # noqa: BLE001 - the arm reports instead of failing the round
        msg = f"{type(e).__name__}: {e}".replace("\n", " ")[:300]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference did not run here: {msg}"}))
        return 0



def capture_context(runner, entries):
    """Run one step eagerly and hand back the StepContext the model saw (index data, block tables and the
    attention work lists on the device), for timing single kernels on a real step's data."""
    seen = []
    real = runner.model.forward
    graphs = runner.use_cuda_graphs
    runner.use_cuda_graphs = False
    runner.model.forward = lambda ctx, cache: (seen.append(ctx), real(ctx, cache))[1]
    try:
        runner.step(entries)
    finally:
        runner.model.forward = real
        runner.use_cuda_graphs = graphs
    return seen[0]


def kernel_chains(loaded, cfg, peaks, tag, ctx, torch, ops, out) -> None:
    """Each kernel class of the step alone: one launch per layer, back to back over the layers' own weights and
    caches (more bytes than L2 holds, as in the step), timed with CUDA events; microseconds a launch and the
    launch's bytes (decode: weights or keys and values read once) or flops (prompt portions) over the measured
    peak.  ``tag`` "decode": the classes of a decode step at the benchmark's batch; "prefill": those of its prompt.
    ``ctx`` must be the context of the step that ran last (its index data lives in the step function's buffer)."""
    model, cache = loaded.model, loaded.cache
    blocks = model.blocks
    L = len(blocks)
    H, Hq, Hkv, D, I = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    dev = "cuda:0"
    bf = torch.bfloat16
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def chain(fn, reps=5):
        """us a launch of the chain's L launches, replayed from a CUDA graph (so that the host's launch rate,
        a few microseconds a call from Python, does not show)."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / reps / L

    def record(name, us, nbytes=None, flops=None):
        e = {"us": round(us, 2)}
        if nbytes is not None:
            e["gbs"] = round(nbytes / us / 1e3, 1)
            e["frac"] = round(nbytes / (us * 1e-6) / hbm, 3)
        if flops is not None:
            e["tflops"] = round(flops / us / 1e6, 1)
            e["frac"] = round(flops / (us * 1e-6) / tflops, 3)
        out[name] = e

    T = ctx.num_tokens
    g = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.5).to(bf)      # noqa: E731
    x, attn, act = rnd(T, H), rnd(T, Hq * D), rnd(T, I)
    qkv, gate_up = rnd(T, (Hq + 2 * Hkv) * D), rnd(T, 2 * I)
    y_qkv, y_h, y_gu = torch.empty_like(qkv), torch.empty(T, H, dtype=bf, device=dev), torch.empty_like(gate_up)
    resid = torch.zeros(T, H, dtype=torch.float32, device=dev)
    a_out = torch.empty(T, Hq * D, dtype=bf, device=dev)
    dec = tag == "decode"
    tokens_kv = sum(ctx.ctx_lens_host) + T
    view = ctx.groups[cache.group_of_slot[0][0]]
    mixers = [b.mixer for b in blocks]
    ffns = [b.ffn for b in blocks]
    ctx.arena.reset()

    def products(name, ws, xin, yout, N, K):
        us = chain(lambda: [ops.linear(xin, w, yout) for w in ws])
        record(f"{tag}_{name}", us, nbytes=N * K * 2 if dec else None, flops=None if dec else 2.0 * T * N * K)
    rot0 = mixers[0].pos.half_split_rotation()
    if not dec and ops.qkv_rope_fused_applies(T, qkv.shape[1], H, bf, D, rot0.rotary_dim):
        # as the step runs it: per-head norm, rotation and cache write in the product's epilogue
        table = torch.empty(T, D // 2, 2, dtype=torch.float32, device=dev)
        ops.rope_table(ctx.positions, rot0.inv_freq, table)
        us = chain(lambda: [ops.linear_qkv_rope(x, m.w_qkv, y_qkv, m.q_norm_w, m.k_norm_w, cfg.rms_norm_eps, table,
                                                cache.layer_view(i), view.slot_mapping, Hq, Hkv) for i, m in enumerate(mixers)])
        record(f"{tag}_qkv_rope", us, flops=2.0 * T * (Hq + 2 * Hkv) * D * H)
    else:
        products("qkv", [m.w_qkv for m in mixers], x, y_qkv, (Hq + 2 * Hkv) * D, H)
    products("o", [m.w_o for m in mixers], attn, y_h, H, Hq * D)
    if not dec and ops.swiglu_fused_applies(T, I, H, bf):
        us = chain(lambda: [ops.linear_swiglu(x, f.w_gate_up, act) for f in ffns])
        record(f"{tag}_gate_up_swiglu", us, flops=2.0 * T * 2 * I * H)
    elif dec and ops.swiglu_small_applies(T, I, H, bf):
        us = chain(lambda: [ops.linear_swiglu_small(x, f.w_gate_up, act) for f in ffns])
        record(f"{tag}_gate_up_swiglu", us, nbytes=2 * I * H * 2)
    else:
        products("gate_up", [f.w_gate_up for f in ffns], x, y_gu, 2 * I, H)
    products("down", [f.w_down for f in ffns], act, y_h, H, I)

    def attention():
        for i, m in enumerate(mixers):
            mark = ctx.arena.mark()
            ops.paged_attention(qkv, cache.layer_view(i), view.block_tables, ctx, a_out, m.scale, 0, Hq, Hkv, D)
            ctx.arena.release(mark)
    us = chain(attention)
    kv_bytes = tokens_kv * 2 * Hkv * D * 2
    if dec:
        record("decode_attention", us, nbytes=kv_bytes)
    else:
        flops = sum(4.0 * Hq * D * n * (c + (n + 1) / 2) for n, c in zip(ctx.q_lens_host, ctx.ctx_lens_host))
        record("prefill_attention", us, flops=flops)
    out[f"{tag}_attention"]["kernel"] = ops.last_attention_kernel

    w_norm = blocks[0].norm1.weight
    us = chain(lambda: [ops.add_rmsnorm(resid, y_h, b.norm1.weight, cfg.rms_norm_eps, x) for b in blocks])
    record(f"{tag}_add_rmsnorm", us, nbytes=T * H * (4 + 4 + 2 + 2))
    del w_norm

    def rotary():
        for i, m in enumerate(mixers):
            rot = m.pos.half_split_rotation()
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, m.q_norm_w, m.k_norm_w, cfg.rms_norm_eps, rot.inv_freq, rot.rotary_dim,
                                      cache.layer_view(i), view.slot_mapping, Hq, Hkv, D)
    us = chain(rotary)
    record(f"{tag}_qk_norm_rope_kv_write", us, nbytes=T * (Hq + 2 * Hkv) * D * 2 * 2)
    if tag == "decode":
        # the output head on the wanted rows, alone (one launch: the matrix is larger than L2 by itself)
        N = ctx.num_logit_rows
        normed = torch.randn(N, H, device=dev).to(bf)
        logits = torch.empty(N, cfg.vocab_size, dtype=torch.float32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        times = []
        for _ in range(4):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            ops.linear(normed, model.head, logits)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        us = sorted(times[1:])[1]
        out["decode_lm_head"] = {"us": round(us, 2), "gbs": round(cfg.vocab_size * H * 2 / us / 1e3, 1),
                                 "frac": round(cfg.vocab_size * H * 2 / (us * 1e-6) / hbm, 3)}


def run_workload(name: str, torch, peaks) -> dict:
    """A scheduler workload at the sizes of a larger model, end to end through ``LLMEngine.serving`` with random
    weights: generated tokens a second (wall clock from the first step to the last), prompt tokens found in shared
    pages, preemptions, and steps, tokens and device time by kind of step."""
    from qwen_engine_b200.config import EngineConfig, preset_config_dict, preset_init
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.registry import config_from_dict
    from qwen_engine_b200.sampling import SamplingParams
    rng = random.Random(11)
    if name == "mixed-1.7b":
        preset, n_req, new_tokens, chunk, max_len = "qwen3-1.7b", 32, 256, 512, 2048 + 256 + 16
        lens = [rng.randint(128, 2048) for _ in range(n_req)]
        shared = 0
    elif name == "shared-prefix-4b":
        preset, n_req, new_tokens, chunk, max_len = "qwen3-4b", 16, 512, 2048, 4096
        lens = [1024 + 256] * n_req
        shared = 1024
    else:
        raise ValueError(f"unknown workload {name!r}")
    cfg = config_from_dict(preset_config_dict(preset))
    init = preset_init(preset)
    page = init["block_size"]
    V = cfg.vocab_size
    common = [rng.randrange(V) for _ in range(shared)]
    prompts = [common + [rng.randrange(V) for _ in range(n - shared)] for n in lens]
    pages = sum(-(-(n + new_tokens) // page) + 1 for n in lens) + 64
    t0 = time.time()
    loaded = load_model(None, torch.bfloat16, "cuda:0", page, pages, n_req, enable_prefix_cache=True, config=cfg,
                        random_seed=init["seed"], random_std=init["std"], random_norm_std=init["norm_std"])
    print(f"[bench] {name}: model ready in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
    ec = EngineConfig(dtype=torch.bfloat16, device="cuda:0", block_size=page, num_blocks=pages, max_model_len=max_len,
                      max_num_seqs=n_req, max_num_batched_tokens=chunk + n_req, prefill_chunk_size=chunk,
                      enable_prefix_cache=True, profile=True)
    eng = LLMEngine(loaded, ec)
    sp = SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)
    # warm-up outside the timed run: one short request through prompt and decoding (kernels loaded, arena sized)
    eng.add_request(prompts[0][:64] if not shared else [rng.randrange(V) for _ in range(64)], SamplingParams(max_new_tokens=4, ignore_eos=True))
    eng.serving()
    eng.stats.__init__()
    hit0, pre0 = eng.scheduler.prefix_hit_tokens, eng.scheduler.num_preemptions
    for p in prompts:
        eng.add_request(p, sp)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.serving()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    generated = sum(len(o.output_token_ids) for o in outs)
    st = eng.stats
    rec = {"model": preset, "layers": cfg.num_hidden_layers, "requests": n_req, "prompt_tokens": sum(lens),
           "new_tokens_each": new_tokens, "prefill_chunk": chunk, "value": round(generated / wall, 1), "unit": "generated tokens/s",
           "seconds": round(wall, 3), "generated_tokens": generated, "steps": st.steps,
           "prefix_hit_tokens": eng.scheduler.prefix_hit_tokens - hit0, "preemptions": eng.scheduler.num_preemptions - pre0,
           "graph_replays": loaded.runner.num_graph_replays, "graph_captures": loaded.runner.num_graph_captures,
           "capture_seconds": round(loaded.runner.graph_capture_seconds, 3),
           "by_kind": {k: {"steps": v["steps"], "tokens": v["tokens"], "device_ms": round(v["device_ms"], 1)}
                       for k, v in (st.profile or {}).items()}}
    del eng, loaded
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return rec


# ---- two designs side by side ---------------------------------------------------------------------------------------------
# Sizes that resemble real models' layers.  A Ganidra model alternates a layer with a gated-linear-attention mixer and a
# layer with windowed softmax attention beside such a mixer, each with its gated feed-forward; the Qwen3 model beside it
# has the same width, feed-forward, heads and number of layers.
COMPARE_SIZES = {
    "w1024": dict(width=1024, ff=3072, heads=16, kv_heads=8, head_dim=128, gla_heads=8, gla_dk=64, gla_dv=128, window=1024,
                  layers=8, vocab=32768, preset="qwen3-0.6b"),
    "w2048": dict(width=2048, ff=6144, heads=16, kv_heads=8, head_dim=128, gla_heads=16, gla_dk=64, gla_dv=128, window=1024,
                  layers=8, vocab=32768, preset="qwen3-1.7b"),
}
_TIMED_OPS = ("embedding", "linear", "linear_swiglu", "linear_swiglu_small", "linear_silu_mul", "linear_qkv_rope", "act_mul",
              "qk_norm_rope_kv_write", "paged_attention", "channel_decay", "linear_attention_scan", "head_norm_gate",
              "add_rmsnorm", "add_rmsnorm_rows", "rope_table", "latent_prepare", "head_linear", "short_conv", "unit_norm",
              "delta_rule_scan", "moe_route", "moe_experts", "qk_bias_norm_kv_write", "stream_conv", "gated_norm_add",
              "token_side_gate", "depth_mix", "group_rmsnorm", "group_norm_add", "head_mix_gate")


def ganidra_config_of(sz: dict) -> dict:
    gla = dict(heads=sz["gla_heads"], dim=sz["gla_dk"], vdim=sz["gla_dv"], tau=16.0, rank=16)
    left = dict(heads=sz["heads"], kv_heads=sz["kv_heads"], dim=sz["head_dim"], vdim=sz["head_dim"],
                mask=dict(size=sz["window"]), scale=sz["head_dim"] ** -0.5)
    mlp = dict(kind="dense", ff=sz["ff"])
    pair = [dict(type="gla", mixer=gla, mlp=mlp),
            dict(type="parallel", mixer=dict(left=left, right=dict(gla, heads=max(1, sz["gla_heads"] // 2)),
                                             left_scale=0.7, right_scale=0.7), mlp=mlp)]
    return dict(architecture="Ganidra", vocab=sz["vocab"], width=sz["width"], embedding=dict(scale=1.0), norm=dict(eps=1e-6),
                layers=pair * (sz["layers"] // 2), loop=dict(start=0, stop=0, times=1))


def besavik_config_of(sz: dict) -> dict:
    """A Besavik model at the sizes of ``sz``: lightning, latent attention, the delta mixer and latent attention again,
    twice over; a dense feed-forward behind the lightning layers and eight experts of half its width, two per token,
    behind the others (the same weights at work per token as the dense one)."""
    D = sz["head_dim"]
    lightning = dict(heads=sz["gla_heads"], dim=sz["gla_dk"], vdim=sz["gla_dv"],
                     decay=[1.0 - 2.0 ** (-5.0 - 4.0 * h / sz["gla_heads"]) for h in range(sz["gla_heads"])])
    latent = dict(heads=sz["heads"], dim=D, rot_dim=D // 2, vdim=D, kv_rank=D + D // 2, q_rank=sz["width"] // 2,
                  scale=(D + D // 2) ** -0.5, rot=dict(base=1000000.0, dims=D // 2))
    delta = dict(heads=sz["gla_heads"], kv_heads=max(1, sz["gla_heads"] // 2), dim=sz["gla_dk"], vdim=sz["gla_dv"], conv=4, rank=64)
    dense = dict(kind="dense", ff=sz["ff"], limit=7.0)
    moe = dict(kind="moe", expert=dict(ff=sz["ff"] // 2, limit=7.0), router=dict(experts=8, top=2))
    four = [dict(type="lightning", mixer=lightning, mlp=dense), dict(type="latent_attention", mixer=latent, mlp=moe),
            dict(type="channel_delta", mixer=delta, mlp=moe), dict(type="latent_attention", mixer=latent, mlp=moe)]
    return dict(architecture="Besavik", vocab=sz["vocab"], width=sz["width"], logit_scale=1.0, norm=dict(eps=1e-6),
                layers=four * (sz["layers"] // 4))


def merudra_config_of(sz: dict) -> dict:
    """A Merudra model at the sizes of ``sz``: attention whose values are its keys twice, the delta mixer with one decay
    per head, attention again, twice over; behind every mixer eight experts of half the dense feed-forward's width and two
    that hand their input on, two per token; streams read through convolutions of four taps; a token input of 64 columns
    per layer."""
    D = sz["head_dim"]
    attn = dict(heads=sz["heads"], kv_heads=sz["kv_heads"], dim=D, vdim=D, scale=D ** -0.5, q_temp=dict(coef=0.1, every=512))
    delta = dict(heads=sz["gla_heads"], kv_heads=max(1, sz["gla_heads"] // 2), dim=sz["gla_dk"], vdim=sz["gla_dv"], conv=4)
    moe = dict(kind="moe", expert=dict(ff=sz["ff"] // 2), router=dict(experts=8, identity=2, top=2))
    four = [dict(type="attention", mixer=attn, mlp=moe), dict(type="attention", mixer=attn, mlp=moe),
            dict(type="delta", mixer=delta, mlp=moe), dict(type="attention", mixer=attn, mlp=moe)]
    return dict(architecture="Merudra", vocab=sz["vocab"], width=sz["width"], norm=dict(eps=1e-6), canon=dict(taps=4),
                token_side=dict(dim=64), layers=four * (sz["layers"] // 4))


def pufivik_config_of(sz: dict) -> dict:
    """A Pufivik model at the sizes of ``sz``: three layers of attention with bent scores and one with a sink, mixed heads
    and a gate per head, twice over; half of every head rotated, with scaled frequencies; values blended with the first
    layer's; behind every mixer eight experts of half the dense feed-forward's width, two per token, scored by sigmoids;
    norms in four groups around every sublayer; the mixers read their input through convolutions of four taps."""
    D = sz["head_dim"]
    common = dict(heads=sz["heads"], kv_heads=sz["kv_heads"], dim=D, vdim=D, scale=D ** -0.5, v_mix=True)
    capped = dict(common, softcap=30.0, rot=dict(base=1000000.0, dims=D // 2, scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0)))
    sunk = dict(common, rot=dict(base=500000.0, dims=D // 2, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    moe = dict(kind="moe", expert=dict(ff=sz["ff"] // 2), router=dict(experts=8, top=2))
    four = [dict(type="attention_2", mixer=capped, mlp=moe), dict(type="attention_2", mixer=capped, mlp=moe),
            dict(type="attention_2", mixer=capped, mlp=moe), dict(type="attention", mixer=sunk, mlp=moe)]
    return dict(architecture="Pufivik", vocab=sz["vocab"], width=sz["width"], norm=dict(eps=1e-6, groups=4), canon=dict(taps=4),
                embedding=dict(scale=1.0), residual_mult=0.5, layers=four * (sz["layers"] // 4))


def pufivik_kernels_alone(torch, ops, peaks) -> dict:
    """The kernels and kernel options that Pufivik adds, each alone on rows that do not fit in L2 (16 384 tokens of width
    2 048: a float32 stream of 134 MB), beside the like kernel of the other models on the same rows: device time (CUDA
    events, ten launches after three), the bytes the operation has to move, and their rate over the measured copy rate;
    for attention the multiply-adds over the time instead."""
    from types import SimpleNamespace
    from qwen_engine_b200.engine.runner import ModelRunner
    from qwen_engine_b200.parts.base import Arena
    dev, bf, f32 = "cuda:0", torch.bfloat16, torch.float32
    T, W, reqs = 16384, 2048, 8
    hbm = float(peaks["hbm_gbs"])
    g = torch.Generator(device=dev).manual_seed(5)
    rnd = lambda *shape, dtype=f32, std=1.0: (torch.randn(*shape, device=dev, dtype=f32, generator=g) * std).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    per = T // reqs
    out: dict = {}

    def timed(name, fn, nbytes, like=None, flops=None):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 100.0
        out[name] = {"us": round(us, 1), "mb": round(nbytes / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1),
                     "frac_of_copy": round(nbytes / us / 1e3 / hbm, 3)}
        if flops:
            out[name]["tflops"] = round(flops / us / 1e6, 1)
        if like:
            out[name]["like"] = like

    n = T * W
    stream, stream2 = rnd(T, W), rnd(T, W)
    branch, cast, cast32 = rnd(T, W, dtype=bf), torch.empty(T, W, device=dev, dtype=bf), torch.empty(T, W, device=dev, dtype=f32)
    wt, wt2 = rnd(W) + 1.0, rnd(W) + 1.0
    timed("add_rmsnorm", lambda: ops.add_rmsnorm(stream, branch, wt, 1e-6, cast), n * 12)
    timed("group_rmsnorm into the compute type", lambda: ops.group_rmsnorm(stream, None, wt, 1e-6, 4, cast), n * 6, like="add_rmsnorm")
    timed("group_rmsnorm into float32", lambda: ops.group_rmsnorm(stream, None, wt, 1e-6, 4, cast32), n * 8, like="add_rmsnorm")
    timed("group_norm_add", lambda: ops.group_norm_add(stream, branch, wt, 1e-6, 4, stream2), n * 10, like="add_rmsnorm, gated_norm_add")
    timed("group_norm_add with the next norm (compute type)", lambda: ops.group_norm_add(stream, branch, wt, 1e-6, 4, stream2, wt2, cast),
          n * 12, like="add_rmsnorm, gated_norm_add")
    timed("group_norm_add with the next norm (float32)", lambda: ops.group_norm_add(stream, branch, wt, 1e-6, 4, stream2, wt2, cast32),
          n * 14, like="add_rmsnorm, gated_norm_add")
    timed("gated_norm_add without gate", lambda: ops.gated_norm_add(stream, branch, None, None, wt, 1e-6, stream2), n * 10)
    del stream2, cast32, branch
    Hq, Hkv, D, page = 16, 8, 128, 16
    pos = torch.arange(T, device=dev, dtype=torch.int32) % per
    slots = torch.arange(T, device=dev, dtype=torch.int32)
    pages = rnd(T // page, 2, Hkv, page, D, dtype=bf)
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=bf)
    nw = rnd(D) + 1.0
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=dev, dtype=f32) / D))
    inv_half = inv[:D // 4].contiguous()
    first = rnd(T, Hkv * D, dtype=bf)
    moved = T * ((Hq + Hkv) * D * 2 * 2 + Hkv * D * 2 + 2 * Hkv * D * 2)
    timed("qk_norm_rope_kv_write", lambda: ops.qk_norm_rope_kv_write(qkv, pos, nw, nw, 1e-6, inv, D, pages, slots, Hq, Hkv, D), moved)
    timed("rotation of half a head with a magnitude, values blended, cache write",
          lambda: ops.qk_norm_rope_kv_write(qkv, pos, None, None, 0.0, inv_half, D // 2, pages, slots, Hq, Hkv, D, magnitude=1.14,
                                            value_mix=("blend", first, 0.3)), moved + T * Hkv * D * 2, like="qk_norm_rope_kv_write")
    E, top = 8, 2
    rx, rw = rnd(T, W, dtype=bf), rnd(E, W, std=0.05)
    ti, tw = torch.empty(T, top, device=dev, dtype=torch.int32), torch.empty(T, top, device=dev, dtype=f32)
    timed("moe_route by sigmoids", lambda: ops.moe_route(rx, rw, None, ti, tw, "sigmoid"), n * 2, like="moe_route over the chosen")
    timed("moe_route over the chosen", lambda: ops.moe_route(rx, rw, None, ti, tw, "softmax_chosen"), n * 2)
    del rx
    partial = rnd(Hkv, T // 4, Hq * D, dtype=bf)
    mix = rnd(Hq, Hq)
    inner = torch.empty(T // 4, Hq * D, device=dev, dtype=bf)
    gate_rows = rnd(T // 4, 16, dtype=bf)
    timed("head_mix_gate over eight kv heads", lambda: ops.head_mix_gate(partial, mix, gate_rows, inner, Hq, Hkv, D),
          (T // 4) * Hq * D * 2 * (Hkv + 1), like="head_norm_gate")
    one = partial[:1].contiguous()
    timed("head_mix_gate, the gate alone", lambda: ops.head_mix_gate(one, None, gate_rows, inner, Hq, Hkv, D), (T // 4) * Hq * D * 4, like="head_norm_gate")
    full_gate = rnd(T // 4, Hq * D, dtype=bf)
    timed("head_norm_gate", lambda: ops.head_norm_gate(one[0], full_gate, None, 0.0, inner, Hq, D, gate_kind="sigmoid"), (T // 4) * Hq * D * 6)
    del partial, one, full_gate
    # attention: eight prompts of 2 048 tokens; the same rows through the tcgen05 kernel (the other models' route at this
    # head size), the flash kernel as it was, and the flash kernel with bent scores and with a sink
    q_lens, ctx_lens = [per] * reqs, [0] * reqs
    blocks = per // page
    tables = torch.arange(reqs * blocks, device=dev, dtype=torch.int32).view(reqs, blocks).contiguous()
    attn_out = torch.empty(T, Hq * D, device=dev, dtype=bf)
    sinks = rnd(Hq)
    macs = reqs * Hq * D * 2 * (per * (per + 1) // 2)              # q.k and p.v over the allowed pairs
    cu = [r * per for r in range(reqs + 1)]
    geo = (Hq, Hkv, D, 0)
    for label, flash, kw in (("paged_attention, tcgen05 kernel", False, {}),
                             ("paged_attention, tcgen05 kernel, bent scores", False, dict(softcap=30.0)),
                             ("paged_attention, tcgen05 kernel, sink and values of the next kv head", False, dict(sinks=sinks, value_shift=1)),
                             ("paged_attention, flash kernel", True, {}),
                             ("paged_attention, flash kernel, bent scores", True, dict(softcap=30.0))):
        saved = ops.TC_MIN_ROWS
        ops.TC_MIN_ROWS = 1 << 30 if flash else saved          # (the flash kernel serves where no portion is long enough for the other)
        try:
            plan = ops.plan_attention(q_lens, ctx_lens, page, (geo,), bf)
        finally:
            ops.TC_MIN_ROWS = saved
        devplan = ModelRunner._device_plan(plan, {"plan_" + k: i32(v) for k, v in plan.items()}, (geo,))
        actx = SimpleNamespace(cu_q=i32(cu), ctx_lens=i32(ctx_lens), q_lens_host=q_lens, ctx_lens_host=ctx_lens, attn_plan=devplan,
                               arena=Arena(dev, 1 << 28))
        timed(label, lambda: ops.paged_attention(qkv, pages, tables, actx, attn_out, D ** -0.5, 0, Hq, Hkv, D, **kw),
              T * (Hq + 2 * Hkv + Hq) * D * 2, flops=2 * macs, like=None if not kw else label.split(",")[0] + "," + label.split(",")[1])
        out[label]["kernel"] = ops.last_attention_kernel
    ops.check_device_status()
    return {"rows": T, "width": W, "kernels": out}


def merudra_kernels_alone(torch, ops, peaks) -> dict:
    """The kernels that Merudra's arrangement adds, each alone on rows that do not fit in L2 (16 384 tokens of width
    2 048: a float32 stream of 134 MB), beside the like kernel of the other models on the same rows: device time (CUDA
    events, ten launches after three), the bytes the operation has to move, and their rate over the measured copy rate."""
    from types import SimpleNamespace
    dev, bf, f32 = "cuda:0", torch.bfloat16, torch.float32
    T, W, taps, reqs = 16384, 2048, 4, 8
    hbm = float(peaks["hbm_gbs"])
    g = torch.Generator(device=dev).manual_seed(5)
    rnd = lambda *shape, dtype=f32, std=1.0: (torch.randn(*shape, device=dev, dtype=f32, generator=g) * std).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    per = T // reqs
    ctx = SimpleNamespace(cu_q=i32([r * per for r in range(reqs + 1)]), ctx_lens=i32([0] * reqs), slot_ids=i32(list(range(reqs))),
                          num_reqs=reqs, max_q_len=per)
    out: dict = {}

    def timed(name, fn, nbytes, like=None):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 100.0
        out[name] = {"us": round(us, 1), "mb": round(nbytes / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1),
                     "frac_of_copy": round(nbytes / us / 1e3 / hbm, 3)}
        if like:
            out[name]["like"] = like

    n = T * W
    stream, stream2 = rnd(T, W), rnd(T, W)
    branch, gate, cast, plain = rnd(T, W, dtype=bf), rnd(T, W, dtype=bf), torch.empty(T, W, device=dev, dtype=bf), torch.empty(T, W, device=dev, dtype=bf)
    wt, gb = rnd(W) + 1.0, rnd(W)
    cw = rnd(W, taps, std=0.3)
    state = torch.zeros(reqs, taps - 1, W, device=dev, dtype=f32)
    timed("add_rmsnorm", lambda: ops.add_rmsnorm(stream, branch, wt, 1e-6, cast), n * 12)
    timed("gated_norm_add", lambda: ops.gated_norm_add(stream, branch, gate, gb, wt, 1e-6, stream2, cast), n * 14, like="add_rmsnorm")
    timed("gated_norm_add without the rounded copy", lambda: ops.gated_norm_add(stream, branch, gate, gb, wt, 1e-6, stream2), n * 12,
          like="add_rmsnorm")
    timed("stream_conv", lambda: ops.stream_conv(stream, cw, state, ctx, plain, cast), n * 8, like="add_rmsnorm, short_conv")
    xin, conv_out = rnd(T, W, dtype=bf), stream2
    timed("short_conv", lambda: ops.short_conv(xin, cw, state, ctx, conv_out), n * 6)
    count = 5
    hist = rnd(count, T // 2, W)
    dw, mixed = rnd(count), torch.empty(T // 2, W, device=dev, dtype=f32)
    timed("depth_mix of five results", lambda: ops.depth_mix(hist, dw, count, mixed), (n // 2) * 4 * (count + 1), like="add_rmsnorm")
    half = n // 2
    timed("gated_norm_add with the weighted sum of five results",
          lambda: ops.gated_norm_add(hist[count - 1], branch[:T // 2], None, None, wt, 1e-6, hist[count - 1], None,
                                     depth_mix=(hist, dw, count, mixed)),
          half * (4 + 2 + 4 + 4 * (count - 1) + 4), like="add_rmsnorm")
    del hist, mixed
    d, V = 64, 32768
    Tt = T * 16
    tg, table, tout = rnd(Tt, d, dtype=bf), rnd(V, d, dtype=bf), torch.empty(Tt, d, device=dev, dtype=bf)
    ids = torch.randint(0, V, (Tt,), device=dev, dtype=torch.int32, generator=g)
    timed("token_side_gate", lambda: ops.token_side_gate(tg, table, ids, tout), Tt * (d * 6 + 4), like="act_mul")
    a_in, a_out = rnd(T, 2 * W, dtype=bf), torch.empty(T, W, device=dev, dtype=bf)
    timed("act_mul", lambda: ops.act_mul(a_in, a_out), n * 6)
    del tg, tout, a_in, a_out
    Hq, Hkv, D, page = 16, 8, 128, 16
    pos = torch.arange(T, device=dev, dtype=torch.int32) % per
    slots = torch.arange(T, device=dev, dtype=torch.int32)
    pages = torch.empty(T // page, 2, Hkv, page, D, device=dev, dtype=bf)
    proj = rnd(T, (2 * Hq + Hkv) * D, dtype=bf)
    qb, kb = rnd(Hq * D), rnd(Hkv * D)
    moved = T * ((Hq + Hkv) * D * 2 * 2 + 2 * Hkv * D * 2)
    timed("qk_bias_norm_kv_write", lambda: ops.qk_bias_norm_kv_write(proj, pos, qb, kb, 1e-6, (0.1, 512), pages, slots, Hq, Hkv, D),
          moved, like="qk_norm_rope_kv_write")
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=bf)
    nw = rnd(D) + 1.0
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=dev, dtype=f32) / D))
    moved = T * ((Hq + Hkv) * D * 2 * 2 + Hkv * D * 2 + 2 * Hkv * D * 2)
    timed("qk_norm_rope_kv_write", lambda: ops.qk_norm_rope_kv_write(qkv, pos, nw, nw, 1e-6, inv, D, pages, slots, Hq, Hkv, D), moved)
    E, top = 10, 2
    rx, rw, corr = rnd(T, W, dtype=bf), rnd(E, W, std=0.05), rnd(E, std=0.01)
    ti, tw = torch.empty(T, top, device=dev, dtype=torch.int32), torch.empty(T, top, device=dev, dtype=f32)
    timed("moe_route over all outputs", lambda: ops.moe_route(rx, rw, None, ti, tw, "softmax_all", corr), n * 2, like="moe_route over the chosen")
    timed("moe_route over the chosen", lambda: ops.moe_route(rx, rw, None, ti, tw, "softmax_chosen"), n * 2)
    ops.check_device_status()
    return {"rows": T, "width": W, "kernels": out}


def compare_designs(args) -> int:
    """``--compare ganidra``: prefill and decode of a Ganidra model beside a Qwen3 model of equal sizes (random weights,
    bfloat16), and the device time of every class of operation in one eager step of each (CUDA events around every
    call, the calls of a class added up).  ``--compare besavik``: a Besavik model beside both.  ``--compare merudra``: a
    Merudra model beside a Besavik and a Qwen3 model.  ``--compare pufivik``: a Pufivik model beside a Merudra and a Qwen3
    model.  Prints one JSON line."""
    import torch
    from qwen_engine_b200 import ops
    from qwen_engine_b200.config import preset_config_dict
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.runner import StepEntry
    from qwen_engine_b200.registry import config_from_dict
    peaks, peaks_src = load_peaks()
    P, B, C = args.prefill_tokens, args.batch, args.context
    page = 16
    rng = random.Random(0)
    clocks = ClockSampler()
    clocks.start()
    m_start = clocks.mark()

    def events_time(fn, n):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    def by_operation(runner, entries_fn):
        """Device microseconds by class of operation in one eager step."""
        spans = []
        saved = {name: getattr(ops, name) for name in _TIMED_OPS}

        def wrap(name, fn):
            def timed_call(*a, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = fn(*a, **k)
                e1.record()
                spans.append((name, e0, e1))
                return r
            return timed_call
        graphs = runner.use_cuda_graphs
        runner.use_cuda_graphs = False
        for name, fn in saved.items():
            setattr(ops, name, wrap(name, fn))
        try:
            runner.step(entries_fn())
            torch.cuda.synchronize()
        finally:
            for name, fn in saved.items():
                setattr(ops, name, fn)
            runner.use_cuda_graphs = graphs
        out: dict = {}
        for name, e0, e1 in spans:
            rec = out.setdefault(name, {"calls": 0, "us": 0.0})
            rec["calls"] += 1
            rec["us"] += e0.elapsed_time(e1) * 1e3
        return {k: {"calls": v["calls"], "us": round(v["us"], 1)} for k, v in sorted(out.items(), key=lambda kv: -kv[1]["us"])}

    def measure(cfg, tag):
        V = cfg.vocab_size
        pages = (B + 1) * (-(-(C + 64 * (args.steps + args.warmup + 8)) // page) + 1) + -(-P // page) + 8
        loaded = load_model(None, torch.bfloat16, "cuda:0", page, pages, B + 2, enable_prefix_cache=False, config=cfg,
                            random_seed=2, random_std=0.02, random_norm_std=0.1)
        runner, cache = loaded.runner, loaded.cache
        toks = lambda n: [rng.randrange(V) for _ in range(n)]
        prompt = toks(P)

        def prefill_once():
            rc = cache.open("p")
            runner.step([StepEntry(rc, prompt, [P - 1])])
            cache.close(rc)
        for _ in range(args.warmup):
            prefill_once()
        prefill_ms = events_time(prefill_once, 5)

        def prefill_entries():
            rc = cache.open("p")
            return [StepEntry(rc, prompt, [P - 1])]
        prefill_ops = by_operation(runner, prefill_entries)
        cache.close(cache.live["p"])
        reqs = [cache.open(f"d{i}") for i in range(B)]
        for i in range(0, B, max(1, 4096 // C)):
            runner.step([StepEntry(rc, toks(C), []) for rc in reqs[i:i + max(1, 4096 // C)]])
        one = lambda: runner.step([StepEntry(rc, [rng.randrange(V)], [0]) for rc in reqs])
        for _ in range(args.warmup):
            one()
        decode_ms = events_time(one, args.steps)
        decode_ops = by_operation(runner, lambda: [StepEntry(rc, [rng.randrange(V)], [0]) for rc in reqs])
        for rc in reqs:
            cache.close(rc)
        weight_bytes = loaded.model.weight_bytes()
        state_bytes = sum(g.tensor[:, 0].numel() * g.tensor.element_size() for g in cache.groups if not g.is_paged)
        rec = {"layers": len(loaded.model.layout.plan), "weight_mb": round(weight_bytes / 2**20, 1),
               "prefill": {"tokens": P, "ms": round(prefill_ms, 3), "tokens_per_s": round(P / prefill_ms * 1e3, 1)},
               "decode": {"batch": B, "context": C, "ms": round(decode_ms, 4), "tokens_per_s": round(B / decode_ms * 1e3, 1)},
               "state_bytes_per_request": state_bytes, "prefill_ops_us": prefill_ops, "decode_ops_us": decode_ops}
        ops.check_device_status()
        del loaded, runner, cache, reqs
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        return rec

    out = {}
    for name in ([args.compare_size] if args.compare_size else list(COMPARE_SIZES)):
        sz = COMPARE_SIZES[name]
        qraw = preset_config_dict(sz["preset"])
        qraw.update(num_hidden_layers=sz["layers"], vocab_size=sz["vocab"])
        out[name] = {"sizes": sz}
        if args.compare == "pufivik":
            out[name]["pufivik"] = measure(config_from_dict(pufivik_config_of(sz)), "pufivik")
        if args.compare in ("merudra", "pufivik"):
            out[name]["merudra"] = measure(config_from_dict(merudra_config_of(sz)), "merudra")
        if args.compare in ("besavik", "merudra"):
            out[name]["besavik"] = measure(config_from_dict(besavik_config_of(sz)), "besavik")
        if args.compare not in ("merudra", "pufivik"):
            out[name]["ganidra"] = measure(config_from_dict(ganidra_config_of(sz)), "ganidra")
        out[name]["qwen3"] = measure(config_from_dict(qraw), "qwen3")
        designs = [d for d in ("pufivik", "merudra", "besavik", "ganidra", "qwen3") if d in out[name]]
        for other in designs[1:]:
            g, q = out[name][designs[0]], out[name][other]
            out[name][f"{designs[0]}_over_{other}"] = {"prefill": round(g["prefill"]["tokens_per_s"] / q["prefill"]["tokens_per_s"], 3),
                                                      "decode": round(g["decode"]["tokens_per_s"] / q["decode"]["tokens_per_s"], 3)}
    alone = None
    if not args.compare_size and args.compare in ("merudra", "pufivik"):
        alone = (merudra_kernels_alone if args.compare == "merudra" else pufivik_kernels_alone)(torch, ops, peaks)
    clocks.stop()
    title = {"besavik": "Besavik beside Ganidra and Qwen3", "merudra": "Merudra beside Besavik and Qwen3",
             "pufivik": "Pufivik beside Merudra and Qwen3"}.get(args.compare, "Ganidra beside Qwen3")
    print(json.dumps({"metric": f"prefill and decode tok/s, {title} at equal sizes", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights N(0, 0.02) seed 2",
                      "steps": args.steps, "warmup": args.warmup, "peaks": peaks_src, "sizes": out,
                      **({"kernels_alone": alone} if alone else {}), "clocks": clocks.summary([(m_start, clocks.mark())])}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="qwen3-0.6b")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--workload", choices=["mixed-1.7b", "shared-prefix-4b"], default=None,
                    help="run only this scheduler workload (32 requests with prompts of 128..2048 tokens and 256 new tokens at "
                         "Qwen3-1.7B sizes in portions of 512; 16 requests sharing 1,024 of 1,280 prompt tokens with 512 new "
                         "tokens at Qwen3-4B sizes) and print its record as one JSON line")
    ap.add_argument("--no-workloads", action="store_true", help="skip the two scheduler workloads at the end of the default run")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel-class timings")
    ap.add_argument("--profile", choices=["decode", "prefill"], default=None,
                    help="bracket that timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--compare", choices=["ganidra", "besavik", "merudra", "pufivik"], default=None,
                    help="instead of the default workload: prefill and decode of a Ganidra model beside a Qwen3 model of equal "
                         "sizes (besavik: a Besavik model beside both; merudra: a Merudra model beside a Besavik and a Qwen3 model; pufivik: a Pufivik model beside a Merudra and a Qwen3 model), with the device time of every class of operation "
                         "(one JSON line)")
    ap.add_argument("--compare-size", choices=sorted(COMPARE_SIZES), default=None, help="with --compare: one size only")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.compare:
        return compare_designs(args)

    import torch
    from qwen_engine_b200 import ops
    if args.workload:
        peaks, _ = load_peaks()
        print(json.dumps({"metric": f"generated tok/s, workload {args.workload}", "impl": "ours", "n_gpus": 1,
                          **run_workload(args.workload, torch, peaks)}))
        return 0
    from qwen_engine_b200.config import EngineConfig, parse_dtype, preset_config_dict, preset_init
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.runner import StepEntry
    from qwen_engine_b200.registry import config_from_dict
    from qwen_engine_b200.sampling import SamplingParams

    peaks, peaks_src = load_peaks()
    dtype = parse_dtype(args.dtype)
    raw = preset_config_dict(args.preset)
    layers_of_config = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    init = preset_init(args.preset)
    page = init["block_size"]
    big_batch = args.batch if args.no_points else max(args.batch, 64)
    extra = args.warmup + args.steps + 8
    per_req = -(-(args.context + 3 * extra) // page) + 1
    pages = big_batch * per_req + -(-args.prefill_tokens // page) + 8
    t_load = time.time()
    loaded = load_model(None, dtype, "cuda:0", page, pages, big_batch + 2, enable_prefix_cache=False, config=cfg,
                        random_seed=init["seed"], random_std=init["std"], random_norm_std=init["norm_std"])
    print(f"[bench] model ready in {time.time() - t_load:.1f}s", file=sys.stderr, flush=True)
    runner, cache, model = loaded.runner, loaded.cache, loaded.model
    rng = random.Random(0)
    V = cfg.vocab_size

    def tokens(n):
        return [rng.randrange(V) for _ in range(n)]

    def timed(fn, n_iter, what=None):
        if what is not None and what == args.profile:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            try:
                return timed(fn, n_iter)
            finally:
                torch.cuda.profiler.stop()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_iter):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n_iter

    clocks = ClockSampler()
    clocks.start()
    spans = []

    # ---- prefill: one prompt of 2,048 tokens to its last logits ----------------------------------
    P = args.prefill_tokens
    prompt = tokens(P)

    def prefill_once():
        rc = cache.open("prefill")
        runner.step([StepEntry(rc, prompt, [P - 1])])
        cache.close(rc)
    for _ in range(args.warmup):
        prefill_once()
    m0 = clocks.mark()
    prefill_ms = timed(prefill_once, 5 if args.profile is None else 1, "prefill")
    spans.append((m0, clocks.mark()))
    # the first, eager run of a prompt length that has not come before (recurring shapes are replayed from a graph)
    def prefill_eager(n):
        rc = cache.open("prefill")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        runner.step([StepEntry(rc, prompt[:n], [n - 1])])
        torch.cuda.synchronize()
        cache.close(rc)
        return (time.perf_counter() - t0) * 1e3
    eager_ms = min(prefill_eager(P - 16 * k) for k in (1, 2, 3)) if args.profile is None else None
    c = cfg
    gemm_params = c.num_hidden_layers * (c.hidden_size * (c.q_width + 2 * c.kv_width) + c.q_width * c.hidden_size
                                         + 3 * c.hidden_size * c.intermediate_size)
    prefill_flops = 2.0 * P * gemm_params + c.num_hidden_layers * 4.0 * c.num_attention_heads * c.head_dim * P * P / 2 \
        + 2.0 * c.vocab_size * c.hidden_size
    prefill = {"value": round(P / (prefill_ms / 1e3), 1), "tokens": P, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
               "first_run_ms": None if eager_ms is None else round(eager_ms, 3)}

    # ---- decode at batch 64, 8, 1 over real, scattered pages ----------------------------------------
    reqs = [cache.open(f"d{i}") for i in range(big_batch)]
    per_step = max(1, 4096 // args.context)
    for i in range(0, big_batch, per_step):
        runner.step([StepEntry(rc, tokens(args.context), []) for rc in reqs[i:i + per_step]])
    torch.cuda.synchronize()
    weight_bytes = model.weight_bytes()
    kv_bytes_per_token = sum(g.tensor[:, 0].numel() // g.tensor.shape[4] * g.tensor.element_size()
                             for g in cache.paged_groups)      # all layers, K and V, one token

    def decode_rate(batch, steps, warmup, record=None, what=None):
        live = reqs[:batch]

        def one():
            runner.step([StepEntry(rc, [rng.randrange(V)], [0]) for rc in live])
        for _ in range(warmup):
            one()
        l0, m = ops.launch_count, clocks.mark()
        ms = timed(one, steps, what)
        if record is not None:
            record["launches"] = ops.launch_count - l0
            spans.append((m, clocks.mark()))
        return batch * 1e3 / ms, ms

    points = {}
    points_detail = {}

    def point(name, batch, steps):
        rate, ms = decode_rate(batch, steps, 3)
        nbytes = weight_bytes + batch * reqs[0].num_tokens * kv_bytes_per_token
        points[name] = round(rate, 1)
        points_detail[name] = {"ms": round(ms, 4), "context": reqs[0].num_tokens, "gbs": round(nbytes / ms / 1e6, 1),
                               "frac": round(nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)}
    if not args.no_points and big_batch >= 64:
        point("decode_b64", 64, max(5, args.steps // 2))
    rec = {}
    value, ms_per_step = decode_rate(args.batch, args.steps, args.warmup, rec, "decode")
    ctx_now = reqs[0].num_tokens
    step_bytes = weight_bytes + args.batch * ctx_now * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    if not args.no_points:
        point("decode_b1", 1, args.steps)
    kernels = {}
    if not args.no_kernels and args.profile is None and dtype == torch.bfloat16:
        dctx = capture_context(runner, [StepEntry(rc, [rng.randrange(V)], [0]) for rc in reqs[:args.batch]])
        kernel_chains(loaded, cfg, peaks, "decode", dctx, torch, ops, kernels)
        rc = cache.open("prefill")
        pctx = capture_context(runner, [StepEntry(rc, prompt, [P - 1])])
        kernel_chains(loaded, cfg, peaks, "prefill", pctx, torch, ops, kernels)
        cache.close(rc)
    for rc in reqs:
        cache.close(rc)

    # ---- end to end through the Python entry point ----------------------------------------------------
    ec = EngineConfig(dtype=dtype, device="cuda:0", block_size=page, num_blocks=pages, max_model_len=args.context + 4 * extra,
                      max_num_seqs=args.batch, max_num_batched_tokens=4096, enable_prefix_cache=False)
    eng = LLMEngine(loaded, ec)
    # (at least 5 untimed decode steps: a step launched ahead is a shape of its own, run eagerly at first sight
    # and captured in a CUDA graph at the second, after the one decode step that is not launched ahead)
    e2e_warmup = max(args.warmup, 5)
    sp = SamplingParams(max_new_tokens=e2e_warmup + args.steps + 8, ignore_eos=True)    # (the requests' ends lie outside the timed steps)
    for _ in range(args.batch):
        eng.add_request(tokens(args.context), sp)
    while eng.stats.decode_tokens < args.batch * e2e_warmup:      # prompts, then the warm-up decode steps
        eng.step()
    torch.cuda.synchronize()
    import gc
    gc.collect()
    gc.disable()                 # (a collection of the benchmark's own heap in mid-loop would stall the host for longer than a step)
    m0 = clocks.mark()
    t0 = time.perf_counter()
    call_s = []
    for _ in range(args.steps):
        t1 = time.perf_counter()
        eng.step()                                                  # host tokens in, sampled tokens out
        call_s.append(time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    gc.enable()
    print(f"[bench] end to end: {e2e_s / args.steps * 1e3:.3f} ms a step; calls (ms): " + " ".join(f"{c * 1e3:.2f}" for c in call_s), file=sys.stderr)
    spans.append((m0, clocks.mark()))
    e2e = {"value": round(args.batch * args.steps / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": runner.last_h2d_bytes, "d2h_bytes_per_step": 4 * args.batch}
    while eng.has_work():
        eng.step()
    eng.check_device()               # no bounded wait inside a kernel ran out during any of the above
    workloads = {}
    if not args.no_workloads and args.profile is None and dtype == torch.bfloat16 and args.preset == "qwen3-0.6b" and not args.layers:
        del eng, reqs, runner, cache, model
        loaded.runner = loaded.cache = loaded.model = None
        import gc as _gc
        _gc.collect()
        torch.cuda.empty_cache()
        for w in ("mixed-1.7b", "shared-prefix-4b"):
            try:
                workloads[w] = run_workload(w, torch, peaks)
            except Exception as e:      # noqa: BLE001 - the headline stands without them
                workloads[w] = {"failed": f"{type(e).__name__}: {e}"[:200]}
    clocks.stop()

    line = {
        "metric": "decode tok/s (Qwen3-0.6B, batch 8, context 1024)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "fp32",
        "data": "synthetic: uniform random token ids, random weights N(0, 0.02) seed 2", "impl": "ours",
        "config": config_record(args.preset, cfg.num_hidden_layers, layers_of_config, c.hidden_size, c.num_attention_heads,
                                c.num_key_value_heads, c.head_dim, c.intermediate_size, c.vocab_size, args.batch,
                                args.context, page, P),
        "context_at_timing": ctx_now, "peaks": peaks_src,
        "e2e": e2e, "gpu_launches": rec.get("launches", 0),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points, "points_detail": points_detail,
        "kernels": kernels, "workloads": workloads,
        "clocks": clocks.summary(spans),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
