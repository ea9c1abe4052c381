"""The engine against the plain implementation: every way of cutting the same requests into steps,
in 32-bit and in bfloat16, on tiny configurations that differ in every size and option."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
from gpu_util import need_gpu
from helpers import load_plain, random_tokens
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# max |logit difference| allowed, as a fraction of the largest |logit| of the sequence
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def _runner(folder, dtype, **kw):
    from pulse_infer_b200.engine import build_runner
    args = dict(dtype=dtype, device="cuda:0", page_size=16, num_pages=64, max_requests=4, max_tokens_per_request=512)
    args.update(kw)
    return build_runner(folder, **args)


def _check(got, want, dtype, what):
    got = got.detach().cpu().double().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    scale = np.abs(want).max()
    err = np.abs(got - want)
    bad = np.argwhere(err > TOL[dtype] * scale)
    assert bad.size == 0, (f"{what}: {len(bad)} logits off by up to {err.max():.3e} (scale {scale:.3f}); "
                           f"first wrong position {bad[0][0]}")


@pytest.fixture(scope="module")
def plain_cache():
    return {}


def _plain(plain_cache, folder, tokens):
    key = (folder, tuple(tokens))
    if key not in plain_cache:
        cfg, w = load_plain(folder)
        plain_cache[key] = plain_model.forward(cfg, w, tokens)
    return plain_cache[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_then_last_32_one_by_one_then_portions(name, dtype, model_folders, plain_cache):
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders[name], CONFIGS[name]
    runner = _runner(folder, dtype)
    for seed, n in ((1, 100), (2, 33), (3, 1)):
        toks = random_tokens(seed, n, cfg.vocab_size)
        want = _plain(plain_cache, folder, toks)
        # whole, logits at every place
        runner.open("w")
        _check(runner.step([Segment("w", toks, list(range(n)))]), want, dtype, f"{name} whole n={n}")
        runner.check_device_errors()
        runner.close("w")
        # most of it in one step, the last 32 tokens one by one
        head = max(0, n - 32)
        runner.open("d")
        outs = []
        if head:
            outs.append(runner.step([Segment("d", toks[:head], [head - 1])]))
            _check(outs[0], want[head - 1:head], dtype, f"{name} head of {head}")
        for i in range(head, n):
            _check(runner.step([Segment("d", [toks[i]], [0])]), want[i:i + 1], dtype, f"{name} decode at {i}")
        runner.check_device_errors()
        runner.close("d")
        # portions of changing size, down to two tokens
        runner.open("p")
        at, k = 0, 0
        sizes = [7, 2, 13, 2, 5, 3, 2, 31, 2, 17]
        while at < n:
            c = min(sizes[k % len(sizes)], n - at)
            k += 1
            got = runner.step([Segment("p", toks[at:at + c], list(range(c)))])
            _check(got, want[at:at + c], dtype, f"{name} portion [{at}, {at + c})")
            at += c
        runner.close("p")
        runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_long_prompt_in_large_portions(name, dtype, model_folders, plain_cache):
    """Portions of several hundred tokens: several query tiles over several key tiles, a window that ends inside
    a key tile (head sizes 64 and 128: the tcgen05 attention kernel in bfloat16), then single tokens."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders[name], CONFIGS[name]
    toks = random_tokens(77, 600, cfg.vocab_size)
    want = _plain(plain_cache, folder, toks)
    runner = _runner(folder, dtype, num_pages=48, max_tokens_per_request=768)
    runner.open("r")
    at = 0
    for c in (257, 130, 200, 1, 1, 9, 1, 1):
        got = runner.step([Segment("r", toks[at:at + c], list(range(c)))])
        _check(got, want[at:at + c], dtype, f"portion [{at}, {at + c})")
        at += c
    runner.check_device_errors()
    runner.close("r")
    runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_batches_with_reused_pages(name, dtype, model_folders, plain_cache):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool so small
    that pages of finished requests are handed to the next ones at once."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders[name], CONFIGS[name]
    lengths = [90, 41, 64, 17, 75, 30, 52]
    reqs = {f"r{i}": random_tokens(10 + i, n, cfg.vocab_size) for i, n in enumerate(lengths)}
    want = {rid: _plain(plain_cache, folder, t) for rid, t in reqs.items()}
    # pool: four live requests need at most 90+75+64+52 tokens -> 6+5+4+4 = 19 pages of 16; give 20
    runner = _runner(folder, dtype, num_pages=20, max_requests=4)
    waiting = list(reqs)
    live, done_at = {}, {}
    rng = np.random.RandomState(0)
    steps = 0
    freed_pages = [set() for _ in range(8)]
    reused = False
    while waiting or live:
        while waiting and len(live) < 4:
            rid = waiting[0]
            need = (len(reqs[rid]) + 15) // 16
            held = sum((len(reqs[r]) + 15) // 16 for r in live)
            if held + need > 20:
                break
            waiting.pop(0)
            runner.open(rid)
            live[rid] = 0
        segs, spans = [], []
        for rid, at in live.items():
            n = len(reqs[rid])
            prompt_end = n - 8                      # the last 8 tokens of every request go one by one
            if at < prompt_end:
                c = min(int(rng.choice([2, 3, 5, 11, 24])), prompt_end - at)
            else:
                c = 1
            if rng.rand() < 0.2 and len(live) > 1 and segs:
                continue                            # this request sits the step out
            segs.append(Segment(rid, reqs[rid][at:at + c], list(range(c))))
            spans.append((rid, at, c))
        if not segs:
            continue
        logits = runner.step(segs)
        runner.check_device_errors()
        row = 0
        for rid, at, c in spans:
            _check(logits[row:row + c], want[rid][at:at + c], dtype, f"{name} mixed step {steps} {rid}[{at}:{at + c}]")
            row += c
            live[rid] = at + c
        for gi, g in enumerate(runner.cache.groups):
            now = {int(p) for r in live for p in g.table.row(runner.cache.slot(r)) if p >= 0}
            reused = reused or bool(now & freed_pages[gi])
        for rid in [r for r, at in live.items() if at == len(reqs[r])]:
            for gi, g in enumerate(runner.cache.groups):
                freed_pages[gi] |= {int(p) for p in g.table.row(runner.cache.slot(rid)) if p >= 0}
            runner.close(rid)
            del live[rid]
        runner.cache.check_invariants()
        steps += 1
    assert steps > 20 and reused
    assert all(g.allocator.num_free == 20 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, model_folders, plain_cache):
    """300 tokens one by one: crosses many pages and, in bfloat16, the boundary where the keys are split."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders["C"], CONFIGS["C"]
    toks = random_tokens(77, 300, cfg.vocab_size)
    want = _plain(plain_cache, folder, toks)
    runner = _runner(folder, dtype)
    runner.open("x")
    for i, t in enumerate(toks):
        _check(runner.step([Segment("x", [t], [0])]), want[i:i + 1], dtype, f"long decode at {i}")
    runner.close("x")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_against_reference_golden(dtype, model_folders):
    """The engine against the logits of the reference's own CPU model (tests/golden)."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    for name in ("A", "B"):
        gold = np.load(os.path.join(ROOT, "tests", "golden", f"tiny_{name}.npz"))
        runner = _runner(model_folders[name], dtype)
        i = 0
        while f"tokens_{i}" in gold:
            toks = [int(t) for t in gold[f"tokens_{i}"]]
            runner.open("g")
            got = runner.step([Segment("g", toks, list(range(len(toks))))])
            runner.close("g")
            want = gold[f"logits_{i}"].astype(np.float64)
            tol = 6e-5 if dtype == "float32" else TOL["bfloat16"]     # the reference itself sums in float32
            assert np.abs(got.cpu().double().numpy() - want).max() <= tol * np.abs(want).max()
            if dtype == "float32":
                assert (got.argmax(-1).cpu().numpy() == want.argmax(-1)).all()
            i += 1


def test_weights_stored_in_32bit_stay_32bit_in_bfloat16_mode(model_folders, plain_cache, tmp_path):
    """A folder whose tensors are stored as F32: in bfloat16 mode they stay 32-bit (products with them run
    in 32-bit), in float32 mode nothing changes; both match the plain implementation."""
    import shutil
    from pulse_infer_b200.engine import Segment
    from pulse_infer_b200.weights import SafetensorsFile, write_safetensors
    need_gpu()
    src = model_folders["A"]
    folder = str(tmp_path / "f32")
    shutil.copytree(src, folder)
    f = SafetensorsFile(os.path.join(src, "model.safetensors"))
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: f.tensor(n).float() for n in f.names()})
    toks = random_tokens(9, 50, CONFIGS["A"].vocab_size)
    want = _plain(plain_cache, src, toks)
    for dtype in ("bfloat16", "float32"):
        runner = _runner(folder, dtype)
        assert runner.model.layers[0].mixer.qkv.dtype == torch.float32
        runner.open("x")
        got = torch.cat([runner.step([Segment("x", toks[:37], list(range(37)))]),
                         runner.step([Segment("x", toks[37:], list(range(13)))])])
        _check(got, want, dtype, f"F32 storage, {dtype} mode")


def test_step_refuses_bad_batches(model_folders):
    from pulse_infer_b200.cache import CacheError, OutOfPages
    from pulse_infer_b200.engine import Segment, StepError
    need_gpu()
    runner = _runner(model_folders["A"], "float32", num_pages=2, max_tokens_per_request=128)
    runner.open("a")
    with pytest.raises(StepError):
        runner.step([Segment("a", [1, 2, 256], [0])])             # token outside the vocabulary
    with pytest.raises(StepError):
        runner.step([Segment("a", [], [])])
    with pytest.raises(StepError):
        runner.step([Segment("a", [1], [0]), Segment("a", [2], [0])])
    with pytest.raises(CacheError):
        runner.step([Segment("nobody", [1], [0])])
    with pytest.raises(OutOfPages):
        runner.step([Segment("a", list(range(40)), [39])])        # 3 pages wanted, 2 exist
    assert runner.cache.length("a") == 0
    out = runner.step([Segment("a", list(range(30)), [29])])      # still usable afterwards
    assert out.shape == (1, 256) and torch.isfinite(out).all()
    with pytest.raises(StepError):
        runner.step([Segment("a", list(range(99)), [0])])         # beyond max_position_embeddings = 128


def _trace_lines(reqs, plan):
    lines = []
    for step, (entries, end) in enumerate(plan):
        lines.append(json.dumps({"step": step, "entries": [
            {"id": rid, "tokens": reqs[rid][a:b], "want": list(range(b - a))} for rid, a, b in entries], "end": end}))
    return "\n".join(lines) + "\n"


@pytest.mark.parametrize("dtype, pool", [("float32", ["--max-tokens", "192"]), ("bfloat16", ["--max-tokens", "192"]),
                                         ("bfloat16", ["--page-size", "8", "--num-pages", "23"])])
def test_trace_run_program(dtype, pool, model_folders, plain_cache, tmp_path):
    """bin/trace_run as a user runs it: a subprocess, steps on standard input, logits in files."""
    need_gpu()
    folder, cfg = model_folders["B"], CONFIGS["B"]
    reqs = {"a": random_tokens(1, 70, cfg.vocab_size), "b": random_tokens(2, 50, cfg.vocab_size),
            "c": random_tokens(3, 64, cfg.vocab_size)}
    plan = [([("a", 0, 38)], []), ([("a", 38, 40), ("b", 0, 20)], []), ([("b", 20, 50), ("a", 40, 41)], []),
            ([("a", 41, 70)], ["b"]), ([("c", 0, 64)], ["a"]), ([], ["c"])]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), *pool], input=_trace_lines(reqs, plan),
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(plan))]
    for step, (entries, _) in enumerate(plan):
        path = out / f"{step}.f32"
        if not entries:
            assert not path.exists()
            continue
        got = np.fromfile(path, dtype="<f4").reshape(-1, cfg.vocab_size)
        want = np.concatenate([_plain(plain_cache, folder, reqs[rid])[a:b] for rid, a, b in entries])
        _check(got, want, dtype, f"trace step {step}")
    # the index names every row: (step, request, position, row)
    with open(out / "index.json") as fh:
        index = json.load(fh)
    assert index["page_size"] == (8 if "--page-size" in pool else 16)
    rows = {(r["step"], r["row"]): (r["request"], r["position"]) for r in index["rows"]}
    for step, (entries, _) in enumerate(plan):
        row = 0
        for rid, a, b in entries:
            for pos in range(a, b):
                assert rows[(step, row)] == (rid, pos)
                row += 1
    assert len(rows) == sum(b - a for entries, _ in plan for _, a, b in entries)
