#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second of a Qwen3-8B-shaped model in bfloat16
with random weights (batch 8, context up to 4096), plus a 2,048-token prefill, decode at batch 1 and 64,
the same decode measured end to end through the Python entry point, and roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Prompts are 2,048 seeded uniform-random token ids per
request; the requests are decoded (untimed) until W + K steps before the context length 4096, then W
warm-up steps and exactly K timed steps follow, bracketed by CUDA events.  Every step reads all weights
(15 GB), far more than the 126 MB L2, so no flush is needed between steps.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the Qwen3-8B shape
SHAPE = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
             intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
             max_position_embeddings=40960)
FULL_LAYERS = 36
CONTEXT = 4096
PROMPT = 2048
PAGE = 16
PREFILL_IDLE_S = 2.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PROFILER_RANGE = False      # --only: bracket the timed steps with cudaProfilerStart/Stop (ncu --profile-from-start off)


def _profiler(start: bool) -> None:
    if PROFILER_RANGE:
        import torch
        (torch.cuda.profiler.start if start else torch.cuda.profiler.stop)()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks, source = dict(FALLBACK_PEAKS), "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                obj = json.load(fh)
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(obj.get(key), (int, float)):
                    peaks[key] = float(obj[key])
            source = "measured"
        except (OSError, ValueError):
            pass
    return peaks, source


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.monotonic(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [l for t, l in self.samples if t0 <= t <= t1] or [l for _, l in self.samples[-3:]]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in rows:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_config(layers: int, shape: dict | None = None):
    from pulse_infer_b200.config import Qwen3Config
    return Qwen3Config(architecture="Qwen3ForCausalLM", torch_dtype="bfloat16", eos_token_ids=(),
                       **{**(shape or SHAPE), "num_hidden_layers": layers})


def weight_bytes_per_step(cfg) -> int:
    """Bytes of weights a decode step reads once: every layer's matrices and norms, the final norm, the head."""
    H, Q, KV, I, V, L = cfg.hidden_size, cfg.q_size, cfg.kv_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    per_layer = H * (Q + 2 * KV) + Q * H + 3 * H * I + 2 * H + 2 * cfg.head_dim
    return 2 * (L * per_layer + H + V * H)


def kv_bytes(cfg, batch: int, ctx: float) -> float:
    return batch * ctx * 2 * cfg.num_hidden_layers * cfg.kv_size * 2


def prefill_flops(cfg, T: int) -> float:
    H, Q, KV, I, V, L = cfg.hidden_size, cfg.q_size, cfg.kv_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    linear = 2.0 * T * L * (H * (Q + 2 * KV) + Q * H + 3 * H * I) + 2.0 * H * V
    attention = 4.0 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) / 2) * L
    return linear + attention


def timed_decode(engine, batch: int, steps: int, warmup: int, rng, through_api: bool, context: int | None = None,
                 prompt: int | None = None):
    """``steps`` timed decode steps of ``batch`` requests whose prompts were 2,048 random ids, ending at
    context 4096.  through_api=False: the step function with device-side argmax and pre-drawn input
    tokens (no host round trip between steps).  through_api=True: Engine.step() - every step takes host
    tokens in (pinned metadata buffer, one copy) and brings the sampled tokens back to the host.
    Returns (ms per step, launches of own kernels, mean context, h2d bytes, d2h bytes per step)."""
    import torch
    from pulse_infer_b200 import ops
    from pulse_infer_b200.engine import Segment
    from pulse_infer_b200.engine.context import StepContext
    vocab = engine.config.vocab_size
    runner = engine.runner
    CONTEXT = context or globals()["CONTEXT"]
    PROMPT = prompt or globals()["PROMPT"]
    prompts = [[int(t) for t in rng.randint(0, vocab, size=PROMPT)] for _ in range(batch)]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h2d = StepContext.layout(batch, batch, batch)["_total"][1] * 4
    if through_api:
        ids = [engine.add_request(p, CONTEXT, ignore_eos=True) for p in prompts]
        reqs = [engine.get_request(i) for i in ids]
        # requests finish their prompts in different steps, so they stay a few tokens apart
        while any(r.is_prefill() for r in reqs):
            engine.step()
        lead = max(r.total_input_tokens() for r in reqs)
        while lead < CONTEXT - (steps + warmup):
            engine.step()
            lead += 1
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        ctx_before = sum(r.total_input_tokens() for r in reqs) / batch
        before = ops.kernels.LAUNCHES
        ev0.record()
        for _ in range(steps):
            engine.step()
        ev1.record()
        torch.cuda.synchronize()
        mean_ctx = ctx_before + steps / 2.0
        d2h = batch * 4
        for i in ids:
            engine.abort(i)
    else:
        rids = [("bench", j) for j in range(batch)]
        for rid, p in zip(rids, prompts):
            runner.open(rid)
            runner.step([Segment(rid, p, [])])                       # one prompt per step
        advance = CONTEXT - (steps + warmup) - PROMPT
        draws = rng.randint(0, vocab, size=(advance + steps + warmup, batch))
        out = torch.empty(batch, dtype=torch.int32, device=runner.runtime.device)

        def one(k):
            logits = runner.step([Segment(rid, [int(draws[k, j])], [0]) for j, rid in enumerate(rids)])
            ops.argmax(logits, out)
        for k in range(advance + warmup):
            one(k)
        torch.cuda.synchronize()
        before = ops.kernels.LAUNCHES
        _profiler(True)
        ev0.record()
        for k in range(advance + warmup, advance + warmup + steps):
            one(k)
        ev1.record()
        torch.cuda.synchronize()
        _profiler(False)
        assert all(runner.cache.length(rid) == CONTEXT for rid in rids)
        mean_ctx = CONTEXT - steps / 2.0
        d2h = 0
        for rid in rids:
            runner.close(rid)
    launches = ops.kernels.LAUNCHES - before
    ms = ev0.elapsed_time(ev1) / steps
    return ms, launches, mean_ctx, h2d, d2h


def timed_prefill(engine, rng, repeats: int = 3, prompt: int | None = None, cached: int = 0):
    """Milliseconds of one step that feeds ``prompt`` tokens of one request (median of ``repeats`` after a warm-up);
    ``cached``: tokens of that request already in the cache (fed before, untimed, in portions of 2,048)."""
    import torch
    from pulse_infer_b200.engine import Segment
    runner = engine.runner
    PROMPT = prompt or globals()["PROMPT"]
    tokens = [int(t) for t in rng.randint(0, engine.config.vocab_size, size=PROMPT)]
    earlier = [int(t) for t in rng.randint(0, engine.config.vocab_size, size=cached)]
    times = []
    for i in range(repeats + 1):
        runner.open(("prefill", i))
        for at in range(0, cached, 2048):
            runner.step([Segment(("prefill", i), earlier[at:at + 2048], [])])
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if i == repeats:
            _profiler(True)
        ev0.record()
        runner.step([Segment(("prefill", i), tokens, [PROMPT - 1])])
        ev1.record()
        torch.cuda.synchronize()
        if i == repeats:
            _profiler(False)
        runner.close(("prefill", i))
        if i > 0:                       # the first run warms up
            times.append(ev0.elapsed_time(ev1))
    return statistics.median(times)


def make_engine(cfg, max_batch: int, graphs: bool = True, context: int | None = None, prompt: int | None = None):
    from pulse_infer_b200 import Engine
    context, prompt = context or CONTEXT, prompt or PROMPT
    return Engine(None, config=cfg, seed=0, dtype="bfloat16", page_size=PAGE, max_tokens=max_batch * (context + 256),
                  max_batch_size=max_batch, chunk_size=prompt, max_tokens_per_step=prompt + max_batch,
                  max_tokens_per_request=context + 256, use_cuda_graphs=graphs)


def run_part(args) -> dict:
    """A short run of one phase only (for profilers): --only decode | prefill, usually with few layers."""
    import numpy as np
    global PROFILER_RANGE
    PROFILER_RANGE = True
    shape = WORKLOADS[args.shape]["shape"] if args.shape else SHAPE
    cfg = make_config(args.layers or shape["num_hidden_layers"], shape)
    rng = np.random.RandomState(0)
    if args.only == "prefill":
        T = args.prompt_len or PROMPT
        engine = make_engine(cfg, args.batch, graphs=not args.no_graphs, context=max(CONTEXT, T + args.cached), prompt=max(T, 2048))
        ms = timed_prefill(engine, rng, repeats=max(1, args.steps), prompt=T, cached=args.cached)
        peaks, _ = load_peaks()
        flops = prefill_flops(cfg, T) + 4.0 * cfg.num_attention_heads * cfg.head_dim * T * args.cached * cfg.num_hidden_layers
        return {"only": "prefill", "shape": args.shape or "bench", "layers": cfg.num_hidden_layers, "tokens": T, "cached": args.cached, "ms": round(ms, 3),
                "tokens_per_s": round(T / ms * 1e3, 1), "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
    prompt = args.prompt_len or min(PROMPT, args.context - args.steps - args.warmup - 1)
    engine = make_engine(cfg, args.batch, graphs=not args.no_graphs, context=args.context, prompt=prompt)
    ms, launches, ctx, _, _ = timed_decode(engine, args.batch, args.steps, args.warmup, rng, False, context=args.context,
                                           prompt=prompt)
    return {"only": "decode", "shape": args.shape or "bench", "layers": cfg.num_hidden_layers, "batch": args.batch, "context": args.context,
            "ms_per_step": round(ms, 4), "tokens_per_s": round(args.batch / ms * 1e3, 1), "gpu_launches": launches,
            "cuda_graphs": not args.no_graphs}


def run_ours(args) -> dict:
    import numpy as np
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    peaks, peak_source = load_peaks()
    layers = args.layers or FULL_LAYERS
    cfg = make_config(layers)
    rng = np.random.RandomState(0)
    batches = sorted({1, 8, 64} | {args.batch})
    max_batch = max(batches)
    t_build = time.time()
    engine = make_engine(cfg, max_batch)
    build_s = time.time() - t_build
    wbytes = weight_bytes_per_step(cfg)

    # The headline first, on a GPU that has done nothing but the untimed steps that bring the batch to its context;
    # the prefill and the other batch sizes (batch 64 runs under the power cap) follow.
    points = {}
    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)
    t0 = time.monotonic()
    ms, launches, mean_ctx, h2d, _ = timed_decode(engine, args.batch, args.steps, args.warmup, rng, through_api=False)
    t1 = time.monotonic()
    clock_info = clocks.stop(t0, t1)
    points[f"decode_b{args.batch}"] = round(args.batch * 1000.0 / ms, 1)
    e2e_ms, _, _, h2d_e, d2h_e = timed_decode(engine, args.batch, args.steps, args.warmup, rng, through_api=True)

    # a prompt step is a burst of 26 ms and is held against the burst peak: it starts from an idle GPU, not from the
    # power cap that thousands of decode steps leave behind
    torch.cuda.synchronize()
    time.sleep(PREFILL_IDLE_S)
    prefill_ms = timed_prefill(engine, rng)
    pf = prefill_flops(cfg, PROMPT)
    for b in batches:
        if b == args.batch:
            continue
        b_ms, _, _, _, _ = timed_decode(engine, b, min(args.steps, 32), args.warmup, rng, through_api=False)
        points[f"decode_b{b}"] = round(b * 1000.0 / b_ms, 1)

    value = args.batch * 1000.0 / ms
    step_bytes = wbytes + kv_bytes(cfg, args.batch, mean_ctx)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {
        "metric": "decode tok/s (Qwen3-8B shape, bf16, batch 8, context to 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, seeded random weights",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (every step reads 15 GB of weights)", "cuda_graphs": True,
                   "peaks": peak_source, "prefill_idle_s": PREFILL_IDLE_S},
        "clocks": clock_info,
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d_e, "d2h_bytes_per_step": d2h_e,
                "note": "Engine.step() with lookahead: each call launches a step and reads the ids of the step before"},
        "gpu_launches": launches,
        "prefill": {"value": round(PROMPT * 1000.0 / prefill_ms, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(pf / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "build_s": round(build_s, 1),
    }


WORKLOADS = {
    # Qwen3-14B shape: a continuous batch of 32 requests, prompt lengths uniform in [128, 2048], 256 new tokens each
    "serve14b": dict(shape=dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                                head_dim=128, intermediate_size=17408, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                                tie_word_embeddings=False, max_position_embeddings=40960),
                     requests=32, prompt_range=(128, 2048), new_tokens=256, max_batch=32),
    # Qwen3-32B shape (q width 8192 != hidden): 16 requests reaching context 8192, prompts fed in portions beside the
    # decode tokens of the requests that are already generating
    "mixed32b": dict(shape=dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                                head_dim=128, intermediate_size=25600, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                                tie_word_embeddings=False, max_position_embeddings=40960),
                     requests=16, prompt_range=(7936, 7936), new_tokens=256, max_batch=16),
}


def run_workload(args) -> dict:
    """A whole serving run through the Python entry point and the scheduler: requests in, generated ids out.
    Reports the throughput, the mix of steps, and per kind of step the host time spent inside ``Engine.step()``
    next to the GPU time of the step's kernels (CUDA events around each call)."""
    import numpy as np
    import torch
    from pulse_infer_b200 import Engine
    from pulse_infer_b200.config import Qwen3Config
    w = WORKLOADS[args.workload]
    shape = dict(w["shape"])
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", torch_dtype="bfloat16", eos_token_ids=(), **shape)
    rng = np.random.RandomState(0)
    lo, hi = w["prompt_range"]
    lengths = [int(rng.randint(lo, hi + 1)) for _ in range(w["requests"])]
    prompts = [[int(t) for t in rng.randint(0, cfg.vocab_size, size=n)] for n in lengths]
    pool_tokens = sum(n + w["new_tokens"] + PAGE for n in lengths)
    t_build = time.time()
    engine = Engine(None, config=cfg, seed=0, dtype="bfloat16", page_size=PAGE, max_tokens=pool_tokens,
                    max_batch_size=w["max_batch"], chunk_size=args.chunk, max_tokens_per_step=args.budget,
                    max_tokens_per_request=max(lengths) + w["new_tokens"] + PAGE, use_cuda_graphs=not args.no_graphs)
    build_s = time.time() - t_build
    # warm-up: one short request end to end (library start-up, first recordings), not timed
    wid = engine.add_request(prompts[0][:64], 4, ignore_eos=True)
    engine.run_until_complete()
    assert len(engine.get_result(wid)) == 4
    t_warm = time.time()
    recorded_before = 0 if args.no_warm_up else engine.warm_up()      # decode steps of every batch size, as a server does at start
    torch.cuda.synchronize()
    warm_s = time.time() - t_warm

    ids = [engine.add_request(p, w["new_tokens"], ignore_eos=True) for p in prompts]
    graphs = engine.runner.graphs
    rec0, rec_s0 = (graphs.recordings, graphs.record_seconds) if graphs is not None else (0, 0.0)
    kinds, host_ms, events = [], [], []
    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)
    c0 = time.monotonic()
    t0 = time.perf_counter()
    first, last = ([int(v) for v in args.profile_steps.split(":")] if args.profile_steps else (-1, -1))
    while engine.has_work():
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if len(kinds) == first:
            torch.cuda.profiler.start()
        h0 = time.perf_counter()
        a.record()
        engine.step()
        b.record()
        if len(kinds) == last:
            torch.cuda.profiler.stop()
        host_ms.append((time.perf_counter() - h0) * 1e3)
        batch = engine.engine.last_batch
        sizes = [n for _, n in batch.entries]
        kinds.append("idle" if not sizes else "decode" if max(sizes) == 1 else "mixed" if min(sizes) == 1 else "prompt")
        events.append((a, b))
    torch.cuda.synchronize()
    wall_s = time.perf_counter() - t0
    clock_info = clocks.stop(c0, time.monotonic())
    generated = sum(len(engine.get_result(i)) for i in ids)
    assert generated == w["requests"] * w["new_tokens"]
    gpu_ms = [a.elapsed_time(b) for a, b in events]
    per_kind = {}
    for kind in ("decode", "mixed", "prompt"):
        idx = [i for i, k in enumerate(kinds) if k == kind]
        if idx:
            per_kind[kind] = {"steps": len(idx), "host_ms": round(sum(host_ms[i] for i in idx) / len(idx), 3),
                              "gpu_ms": round(sum(gpu_ms[i] for i in idx) / len(idx), 3),
                              "gpu_ms_median": round(statistics.median(gpu_ms[i] for i in idx), 3)}
    st = engine.get_stats()
    prompt_tokens = sum(lengths)
    return {"workload": args.workload, "impl": "ours", "dtype": "bf16", "layers": cfg.num_hidden_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "intermediate": cfg.intermediate_size, "requests": w["requests"], "prompt_tokens": prompt_tokens,
            "prompt_range": [lo, hi], "new_tokens_each": w["new_tokens"], "chunk": args.chunk, "budget": args.budget,
            "seconds": round(wall_s, 3), "generated_tokens_per_s": round(generated / wall_s, 1),
            "all_tokens_per_s": round((generated + prompt_tokens) / wall_s, 1), "steps": len(kinds), "step_kinds": per_kind,
            "gpu_busy_frac": round(sum(gpu_ms) / (wall_s * 1e3), 3), "preemptions": st.num_preemptions,
            "graphs_recorded_at_start": recorded_before, "warm_up_s": round(warm_s, 2),
            "graphs_recorded": graphs.recordings - rec0 if graphs is not None else 0,
            "graph_record_s": round(graphs.record_seconds - rec_s0, 3) if graphs is not None else 0.0,
            "weight_gb": round(engine.runner.model.weight_bytes() / 1e9, 2), "clocks": clock_info, "build_s": round(build_s, 1),
            "data": "synthetic: seeded uniform-random token ids, seeded random weights"}


def run_reference(args) -> dict:
    """The reference engine itself on the same shape, batch, context, steps and warm-up: ``baseline/_ref/ref_bench`` is
    the reference's unmodified sources built for sm_100 by ``baseline/build_reference.py`` plus a driver that calls its
    ``init_paged_cache`` and ``forward_batched``; nothing of this repository's engine or kernels is on that path."""
    exe = os.path.join(ROOT, "baseline", "_ref", "ref_bench")
    if not os.path.isfile(exe):
        ref = os.environ.get("PULSE_REFERENCE", "/root/reference")
        if os.path.isdir(os.path.join(ref, "src")):
            subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--reference", ref],
                           stdout=sys.stderr, stderr=sys.stderr)
    if not os.path.isfile(exe):
        return {"impl": "reference", "unavailable": "baseline/_ref/ref_bench is not built and no checkout of the reference "
                "is at hand to build it from (python baseline/build_reference.py --reference DIR)"}
    layers = args.layers or FULL_LAYERS
    warmup = max(args.warmup, 3)
    cmd = [exe, "--layers", str(layers), "--hidden", str(SHAPE["hidden_size"]), "--heads", str(SHAPE["num_attention_heads"]),
           "--kv-heads", str(SHAPE["num_key_value_heads"]), "--head-dim", str(SHAPE["head_dim"]),
           "--intermediate", str(SHAPE["intermediate_size"]), "--vocab", str(SHAPE["vocab_size"]),
           "--max-position", str(SHAPE["max_position_embeddings"]), "--theta", repr(SHAPE["rope_theta"]),
           "--eps", repr(SHAPE["rms_norm_eps"]), "--batch", str(args.batch), "--context", str(CONTEXT),
           "--prompt", str(PROMPT), "--steps", str(args.steps), "--warmup", str(warmup), "--page", str(PAGE)]
    clocks = ClockSampler()
    clocks.start()
    t0 = time.monotonic()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=args.reference_timeout)
    except subprocess.TimeoutExpired:
        clocks.stop(t0, time.monotonic())
        return {"impl": "reference", "unavailable": f"the reference did not finish its run within {args.reference_timeout} s"}
    clock_info = clocks.stop(t0, time.monotonic())
    try:
        out = json.loads(proc.stdout.strip().splitlines()[-1])
    except (ValueError, IndexError):
        out = {"error": (proc.stderr or proc.stdout)[-300:]}
    if proc.returncode != 0 or "error" in out:
        return {"impl": "reference", "unavailable": f"the reference's run failed (code {proc.returncode}): {out.get('error')}"}
    peaks, peak_source = load_peaks()
    cfg = make_config(layers)
    ms, e2e_ms, prefill_ms = out["decode_ms_per_step"], out["e2e_ms_per_step"], out["prefill_ms"]
    step_bytes = weight_bytes_per_step(cfg) + kv_bytes(cfg, args.batch, CONTEXT - args.steps / 2.0)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {
        "metric": "decode tok/s (Qwen3-8B shape, bf16, batch 8, context to 4096)",
        "value": round(args.batch * 1000.0 / ms, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, seeded random weights",
        "impl": "reference",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (every step reads 15 GB of weights)", "cuda_graphs": False,
                   "peaks": peak_source},
        "clocks": clock_info,
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": out["h2d_bytes_per_step"], "d2h_bytes_per_step": out["d2h_bytes_per_step"],
                "note": "forward_batched + per-request last-row logits to the host + host argmax, as the reference's engine does"},
        "gpu_launches": None,
        "prefill": {"value": round(PROMPT * 1000.0 / prefill_ms, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops(cfg, PROMPT) / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": {f"decode_b{args.batch}": round(args.batch * 1000.0 / ms, 2)},
        "fill_s": out.get("fill_s"),
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the 36 of the shape (named in config)")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None, help="run one phase only (for profilers)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only decode: the context the timed steps end at")
    ap.add_argument("--prompt-len", type=int, default=None, help="with --only: tokens of each prompt (default 2048)")
    ap.add_argument("--cached", type=int, default=0, help="with --only prefill: tokens of the request already in the cache")
    ap.add_argument("--no-graphs", action="store_true", help="with --only: launch decode steps eagerly")
    ap.add_argument("--shape", choices=sorted(WORKLOADS), default=None,
                    help="with --only: the layer sizes of that workload's model instead of the Qwen3-8B shape")
    ap.add_argument("--reference-timeout", type=int, default=1500, help="seconds the reference arm may take")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="a whole serving run through Engine and the scheduler instead of the decode benchmark")
    ap.add_argument("--profile-steps", default=None, metavar="A:B",
                    help="with --workload: cudaProfilerStart before step A, cudaProfilerStop after step B "
                         "(ncu --profile-from-start off)")
    ap.add_argument("--no-warm-up", action="store_true",
                    help="with --workload: do not record the decode steps of all batch sizes before the timed run")
    ap.add_argument("--chunk", type=int, default=1024, help="with --workload: longest prompt portion of one request")
    ap.add_argument("--budget", type=int, default=2048, help="with --workload: tokens of one step")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.gpus != 1:
            print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, only --gpus 1")
            return 2
        print(json.dumps(run_reference(args)))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, only --gpus 1")
        return 2
    if args.only:
        print(json.dumps(run_part(args)))
        return 0
    if args.workload:
        print(json.dumps(run_workload(args)))
        return 0
    args.warmup = max(args.warmup, 3)
    result = run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
