"""Command line, in the manner of the reference's two demo programs.

``qwen3_infer [model_dir]`` (``demo/qwen3_infer.cpp:539-676``): single-stream generation, one prompt after
the other, with the demo's sampler - its constants are the defaults here: 32 new tokens
(``kMaxNewTokens``, 542), temperature / top-k / top-p from generation_config.json else 0.6 / 20 / 0.95
(590-592), presence penalty 1.5 (469), a tokens-per-second line at the end (669-673).

``qwen3_continuous_batch_demo [model_dir]`` (``demo/qwen3_continuous_batch_demo.cpp:99-180``): several
prompts through the continuous-batching engine, greedy, with its constants as defaults: batch 2, chunk
64, pages of 16 tokens, ``max(64, ceil(sum(prompt + max_new + 16) / 16))`` pages (146-157).

Both take the model folder as their one positional argument, as the reference does; prompts are token
ids (``--prompt-ids 1,2,3``, repeatable) or seeded random ids (``--prompt-len N``), since text is outside
this engine.  ``--random-config FILE --seed N`` runs random weights of a config.json instead of a folder.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np


def _find_default_model_dir() -> str | None:
    """The nearest ``model/`` folder upward from the working directory (qwen3_infer.cpp:42-60)."""
    here = os.path.abspath(os.getcwd())
    while True:
        cand = os.path.join(here, "model")
        if os.path.isfile(os.path.join(cand, "config.json")):
            return cand
        parent = os.path.dirname(here)
        if parent == here:
            return None
        here = parent


def _common(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("model_dir", nargs="?", default=None, help="model folder (default: nearest model/ upward)")
    ap.add_argument("--random-config", help="a config.json; weights are random (with --seed) instead of loaded")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and of the sampler")
    ap.add_argument("--dtype", choices=["bfloat16", "float32", "bf16", "fp32"], default="bfloat16")
    ap.add_argument("--rope-style", choices=["interleaved", "half"], default="interleaved",
                    help="which elements form a rotated pair: interleaved (2i, 2i+1) as the reference, or halves")
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeatable")
    ap.add_argument("--prompt-len", type=int, action="append", default=[], help="a seeded random prompt; repeatable")
    ap.add_argument("--prompt-seed", type=int, default=0)
    ap.add_argument("--max-new-tokens", type=int, default=None)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--kv-gb", type=float, default=None, help="size the page pool by memory (GiB) instead of --num-pages")
    ap.add_argument("--max-tokens-per-step", type=int, default=None, help="token budget of one step (default: batch x chunk)")
    ap.add_argument("--print-logits-topk", type=int, default=0, metavar="K",
                    help="with every generated token, print the K largest logits it was chosen from")
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--device", default="cuda:0")


def _prompts(args, vocab: int) -> list:
    prompts = [[int(t) for t in text.split(",") if t.strip()] for text in args.prompt_ids]
    for i, n in enumerate(args.prompt_len):
        rng = np.random.RandomState(args.prompt_seed + i)
        prompts.append([int(t) for t in rng.randint(0, vocab, size=n)])
    return prompts


def _make_engine(args, max_batch_size: int, chunk_size: int, num_pages: int | None, max_tokens: int | None):
    from .api import Engine
    from .config.registry import get_architecture, load_config
    from .config.base import read_json_file
    pairing = "adjacent" if args.rope_style == "interleaved" else "half"
    kv_bytes = int(args.kv_gb * (1 << 30)) if args.kv_gb and not num_pages else None
    kw = dict(dtype=args.dtype, device=args.device, page_size=args.page_size, num_pages=num_pages,
              max_tokens=None if kv_bytes else max_tokens, kv_bytes=kv_bytes,
              max_batch_size=max_batch_size, chunk_size=chunk_size, use_cuda_graphs=not args.no_cuda_graphs,
              rope_pairing=pairing, max_tokens_per_step=args.max_tokens_per_step)
    if args.random_config:
        from .config.registry import architecture_name_of
        obj = read_json_file(args.random_config)
        arch = get_architecture(architecture_name_of(obj, args.random_config))
        config = arch.config_class.from_json_dict(obj, args.random_config)
        return Engine(None, config=config, seed=args.seed, **kw), config
    model_dir = args.model_dir or _find_default_model_dir()
    if model_dir is None:
        raise SystemExit("no model folder given and no model/ folder found upward from here")
    return Engine(model_dir, **kw), load_config(model_dir)


def _topk_recorder(engine, k: int) -> dict:
    """Make the engine note, for every token it samples, the k largest logits of that position:
    request id -> list (one entry per generated token) of [[token id, logit], ...]."""
    import torch
    seen: dict = {}

    def hook(requests, logits):
        values, ids = torch.topk(logits, min(k, logits.shape[1]), dim=-1)
        values, ids = values.tolist(), ids.tolist()
        for req, v, i in zip(requests, values, ids):
            seen.setdefault(req.request_id, []).append([[int(t), round(float(x), 5)] for t, x in zip(i, v)])
    engine.engine.logits_hook = hook
    return seen


def _config_first(args):
    from .config.base import read_json_file
    from .config.registry import architecture_name_of, get_architecture, load_config
    if args.random_config:
        obj = read_json_file(args.random_config)
        return get_architecture(architecture_name_of(obj, args.random_config)).config_class.from_json_dict(obj)
    model_dir = args.model_dir or _find_default_model_dir()
    if model_dir is None:
        raise SystemExit("no model folder given and no model/ folder found upward from here")
    return load_config(model_dir)


def qwen3_infer(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="qwen3_infer", description="single-stream generation")
    _common(ap)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--presence-penalty", type=float, default=1.5)
    ap.add_argument("--greedy", action="store_true")
    args = ap.parse_args(argv)
    cfg = _config_first(args)
    prompts = _prompts(args, cfg.vocab_size) or [[int(t) for t in np.random.RandomState(0).randint(0, cfg.vocab_size, 16)]]
    max_new = 32 if args.max_new_tokens is None else args.max_new_tokens
    temperature = args.temperature if args.temperature is not None else (cfg.temperature if cfg.temperature > 0 else 0.6)
    top_k = args.top_k if args.top_k is not None else (cfg.top_k if cfg.top_k > 0 else 20)
    top_p = args.top_p if args.top_p is not None else (cfg.top_p if cfg.top_p > 0 else 0.95)
    if args.greedy:
        temperature = 0.0
    longest = max(len(p) for p in prompts) + max_new
    engine, _ = _make_engine(args, 1, 256, args.num_pages, None if args.num_pages else longest + args.page_size)
    topk = _topk_recorder(engine, args.print_logits_topk) if args.print_logits_topk > 0 else None
    generated, t0 = 0, time.perf_counter()
    for i, prompt in enumerate(prompts):
        rid = engine.add_request(prompt, max_new, temperature=temperature, top_k=top_k, top_p=top_p,
                                 presence_penalty=args.presence_penalty, seed=args.seed + i, ignore_eos=args.ignore_eos)
        engine.run_until_complete()
        out = engine.get_result(rid)
        generated += len(out)
        line = {"prompt": i, "prompt_tokens": len(prompt), "generated": out}
        if topk is not None:
            line["logits_topk"] = topk.get(rid, [])[:len(out)]
        print(json.dumps(line))
    dt = time.perf_counter() - t0
    print(f"Generated {generated} tokens in {dt:.3f}s ({generated / dt:.2f} tokens/s)")
    return 0


def _bench(engine, kind: str, prompts: list, max_new: list, args) -> int:
    """``--bench``: time the given prompts through the engine instead of printing what it generates; one JSON line.
    serve: the whole run, requests in to last token out.  prefill: until every request has its first token (prompt
    tokens per second).  decode: from the step after the last prompt portion to the end (generated tokens per second
    while nothing but single tokens is in flight).  The decode steps of all batch sizes are recorded beforehand
    (``Engine.warm_up``), no request stops early, and the clock is read with the device idle."""
    import torch
    recorded = engine.warm_up()
    if kind == "prefill":
        max_new = [1] * len(prompts)
    ids = [engine.add_request(p, m, temperature=args.temperature, seed=args.seed + i, ignore_eos=True)
           for i, (p, m) in enumerate(zip(prompts, max_new))]
    reqs = [engine.get_request(rid) for rid in ids]
    steps0 = engine.get_stats().num_steps
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    already = 0
    if kind == "decode":
        while engine.has_work() and any(r.is_prefill() for r in reqs):
            engine.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        already = sum(len(engine.get_result(rid)) for rid in ids)
        steps0 = engine.get_stats().num_steps
    engine.run_until_complete()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    generated = sum(len(engine.get_result(rid)) for rid in ids)
    prompt_tokens = sum(len(p) for p in prompts)
    st = engine.get_stats()
    line = {"bench": kind, "requests": len(prompts), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "seconds": round(dt, 4), "steps": st.num_steps - steps0, "preemptions": st.num_preemptions,
            "max_batch_size": args.max_batch_size, "chunk_size": args.chunk_size, "dtype": args.dtype,
            "decode_steps_recorded_before": recorded}
    if kind == "prefill":
        line["prompt_tokens_per_s"] = round(prompt_tokens / dt, 1)
    elif kind == "decode":
        line["timed_tokens"] = generated - already
        line["generated_tokens_per_s"] = round((generated - already) / dt, 1)
    else:
        line["generated_tokens_per_s"] = round(generated / dt, 1)
        line["all_tokens_per_s"] = round((generated + prompt_tokens) / dt, 1)
    print(json.dumps(line))
    return 0


def qwen3_continuous_batch_demo(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="qwen3_continuous_batch_demo", description="continuous batching, greedy")
    _common(ap)
    ap.add_argument("--max-batch-size", type=int, default=2)
    ap.add_argument("--chunk-size", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--bench", choices=["decode", "prefill", "serve"], default=None,
                    help="time the prompts through the engine (one JSON line) instead of printing the generated ids")
    args = ap.parse_args(argv)
    cfg = _config_first(args)
    prompts = _prompts(args, cfg.vocab_size)
    if not prompts:
        prompts = [[int(t) for t in np.random.RandomState(i).randint(0, cfg.vocab_size, n)] for i, n in enumerate((24, 9, 40))]
    max_new = [96, 72, 96] if args.max_new_tokens is None else [args.max_new_tokens]
    max_new = [max_new[i % len(max_new)] for i in range(len(prompts))]
    estimate = sum(len(p) + m + 16 for p, m in zip(prompts, max_new))
    num_pages = args.num_pages or (None if args.kv_gb else max(64, (estimate + args.page_size - 1) // args.page_size))
    engine, _ = _make_engine(args, args.max_batch_size, args.chunk_size, num_pages, None)
    if args.bench:
        return _bench(engine, args.bench, prompts, max_new, args)
    topk = _topk_recorder(engine, args.print_logits_topk) if args.print_logits_topk > 0 else None
    ids = [engine.add_request(p, m, temperature=args.temperature, seed=args.seed + i, ignore_eos=args.ignore_eos)
           for i, (p, m) in enumerate(zip(prompts, max_new))]
    t0 = time.perf_counter()

    def on_step(eng, out):
        st = eng.get_stats()
        if st.num_steps % 10 == 0:      # continuous_batch_engine.cpp:89-96
            print(f"step {st.num_steps}: running={st.num_running} waiting={st.num_waiting} "
                  f"finished={st.num_finished}/{st.total_requests} free_pages={list(st.free_pages)}", file=sys.stderr)
    engine.run_until_complete(on_step)
    dt = time.perf_counter() - t0
    total = 0
    for i, rid in enumerate(ids):
        out = engine.get_result(rid)
        total += len(out)
        line = {"request": rid, "prompt_tokens": len(prompts[i]), "generated": out,
                "finish_reason": engine.get_request(rid).finish_reason}
        if topk is not None:
            line["logits_topk"] = topk.get(rid, [])[:len(out)]
        print(json.dumps(line))
    st = engine.get_stats()
    print(f"Generated {total} tokens in {dt:.3f}s ({total / dt:.2f} tokens/s); steps={st.num_steps} "
          f"preemptions={st.num_preemptions}")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("infer", "qwen3_infer"):
        return qwen3_infer(argv[1:])
    if argv and argv[0] in ("batch", "qwen3_continuous_batch_demo"):
        return qwen3_continuous_batch_demo(argv[1:])
    print("usage: python -m pulse_infer_b200.cli {infer|batch} [model_dir] [options]", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
