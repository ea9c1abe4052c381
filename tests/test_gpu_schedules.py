"""The engine against the plain implementation on the code paths that large models take: head size 128 with four query
heads per key/value head, steps recorded as CUDA graphs (their logits, not only their tokens), more than four and more
than sixteen live requests, contexts of thousands of tokens cut into several key ranges, pages of 8 tokens, and one
check at the real widths of the 8B shape."""
import numpy as np
import pytest
import torch

import plain_model
from gpu_util import need_gpu
from helpers import load_plain, random_tokens
from test_gpu_engine import TOL, _check, _plain, _runner, plain_cache  # noqa: F401  (plain_cache is a fixture)
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu


# ---- recorded steps ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_recorded_steps_give_the_plain_logits(name, dtype, model_folders, plain_cache):
    """Steps of single tokens run as CUDA graph replays: the logits of every replay are compared, at batch sizes 3, 2
    and 1, with requests of different lengths, and once with the input ids taken from a device tensor."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders[name], CONFIGS[name]
    runner = _runner(folder, dtype, use_cuda_graphs=True, num_pages=96, max_tokens_per_request=640)
    assert runner.model.capturable
    reqs = {"a": random_tokens(31, 330, cfg.vocab_size), "b": random_tokens(32, 75, cfg.vocab_size),
            "c": random_tokens(33, 140, cfg.vocab_size)}
    want = {r: _plain(plain_cache, folder, t) for r, t in reqs.items()}
    at = {}
    for rid, toks in reqs.items():
        runner.open(rid)
        head = len(toks) - 40
        got = runner.step([Segment(rid, toks[:head], [head - 1])])
        _check(got, want[rid][head - 1:head], dtype, f"{name} prompt of {rid}")
        at[rid] = head
    replays = 0
    for k in range(40):
        live = [r for r in reqs if not (r == "b" and k >= 30) and not (r == "c" and k >= 35)]    # batch 3, then 2, then 1
        segs = [Segment(r, [reqs[r][at[r]]], [0]) for r in live]
        assert runner.takes_device_tokens(segs)
        if k % 7 == 3:
            # the ids come from the device (what the step before sampled); the segments carry placeholders
            ids = torch.tensor([reqs[r][at[r]] for r in live], dtype=torch.int32, device="cuda:0")
            for s in segs:
                s.tokens = [0]
            got = runner.step(segs, tokens_from=ids)
        else:
            got = runner.step(segs)
        replays += 1
        for i, r in enumerate(live):
            _check(got[i:i + 1], want[r][at[r]:at[r] + 1], dtype, f"{name} recorded step {k} {r}@{at[r]}")
            at[r] += 1
    runner.check_device_errors()
    assert len(runner.graphs.graphs) >= 3 and replays == 40
    for r in reqs:
        runner.close(r)
    runner.cache.check_invariants()


# ---- many live requests ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("live", [12, 20])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_live_requests(dtype, live, graphs, model_folders, plain_cache):
    """12 live requests: decode steps of 9 to 16 rows (the fused chain of the weight-streaming products in its
    two-tile form).  20: steps of more than 16 rows (library products, norm kernels, the tcgen05 product).  Two waves
    of requests in a pool that holds one, so the second wave gets the first one's pages; portions of prompts run
    beside single tokens, and some steps hold single tokens only (recorded when ``graphs``)."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders["E"], CONFIGS["E"]
    rng = np.random.RandomState(live)
    lengths = [int(rng.randint(24, 70)) for _ in range(2 * live)]
    reqs = {f"r{i}": random_tokens(200 + i, n, cfg.vocab_size) for i, n in enumerate(lengths)}
    want = {rid: _plain(plain_cache, folder, t) for rid, t in reqs.items()}
    waves = [list(reqs)[:live], list(reqs)[live:]]
    pages = max(sum((len(reqs[r]) + 15) // 16 for r in wave) for wave in waves)
    runner = _runner(folder, dtype, num_pages=pages, max_requests=live, max_tokens_per_request=128,
                     use_cuda_graphs=graphs)
    steps = decode_only = mixed = 0
    first_wave_pages, reused = set(), False
    for wave in waves:
        at = {}
        for rid in wave:
            runner.open(rid)
            at[rid] = 0
        while any(a < len(reqs[r]) for r, a in at.items()):
            everyone_at_the_tail = all(a >= len(reqs[r]) - 8 for r, a in at.items())
            segs, spans = [], []
            for rid, a in at.items():
                n = len(reqs[rid])
                if a < n - 12:
                    c = min(int(rng.choice([5, 9, 16])), n - 12 - a)       # a portion of the prompt
                elif a < n - 8 or everyone_at_the_tail:
                    c = 1                                                # one token: beside portions, or all together
                else:
                    continue                                             # waits for the others to reach their tails
                if a == n:
                    continue
                segs.append(Segment(rid, reqs[rid][a:a + c], [c - 1]))
                spans.append((rid, a, c))
            logits = runner.step(segs)
            runner.check_device_errors()
            for row, (rid, a, c) in enumerate(spans):
                _check(logits[row:row + 1], want[rid][a + c - 1:a + c], dtype,
                       f"{live} live, step {steps}, {rid}[{a}:{a + c}]")
                at[rid] = a + c
            sizes = {c for _, _, c in spans}
            decode_only += int(sizes == {1} and len(spans) == live)
            mixed += int(1 in sizes and len(sizes) > 1)
            held = {int(p) for g in runner.cache.groups for r in at for p in g.table.row(runner.cache.slot(r)) if p >= 0}
            if wave is waves[0]:
                first_wave_pages |= held
            else:
                reused = reused or bool(held & first_wave_pages)
            runner.cache.check_invariants()
            steps += 1
        for rid in wave:
            runner.close(rid)
    assert decode_only >= 16 and mixed >= 2 and reused
    assert all(g.allocator.num_free == pages for g in runner.cache.groups)
    if graphs:
        assert any(key[0] == live for key in runner.graphs.graphs)


# ---- thousands of tokens -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype, split_keys, graphs", [("bfloat16", None, False), ("bfloat16", "512", True),
                                                       ("bfloat16", "2048", False), ("float32", None, False)])
def test_decoding_one_by_one_beyond_2600_tokens(dtype, split_keys, graphs, model_folders, plain_cache, monkeypatch):
    """A prompt of 2,000 tokens in three portions, then 640 tokens one by one: positions in the thousands with
    theta = 1e6, key ranges of 256 (eleven of them), 512 and 2,048 keys (several tiles a range), queries sharp enough
    that single far keys carry the result."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    if split_keys is None:
        monkeypatch.delenv("PULSE_SPLIT_KEYS", raising=False)
    else:
        monkeypatch.setenv("PULSE_SPLIT_KEYS", split_keys)
    folder, cfg = model_folders["E"], CONFIGS["E"]
    toks = random_tokens(91, 2640, cfg.vocab_size)
    want = _plain(plain_cache, folder, toks)
    runner = _runner(folder, dtype, num_pages=170, max_requests=2, max_tokens_per_request=2704, use_cuda_graphs=graphs)
    runner.open("x")
    at = 0
    for c in (700, 650, 650):
        got = runner.step([Segment("x", toks[at:at + c], [0, c // 2, c - 1])])
        _check(got, want[[at, at + c // 2, at + c - 1]], dtype, f"portion [{at}, {at + c})")
        at += c
    worst = 0.0
    for i in range(at, len(toks)):
        got = runner.step([Segment("x", [toks[i]], [0])])
        _check(got, want[i:i + 1], dtype, f"decode at {i} (ranges of {split_keys or 'default'} keys)")
        worst = max(worst, float(np.abs(got.cpu().double().numpy() - want[i]).max()))
    runner.check_device_errors()
    runner.close("x")
    runner.cache.check_invariants()
    assert worst > 0.0 or dtype == "float32"


def test_sharp_queries_make_far_keys_matter(model_folders, plain_cache):
    """The premise of the test above: in the last layer's input, dropping the 64 oldest keys of a 2,000-token context
    must move the logits by more than the bfloat16 tolerance; otherwise a kernel that skips them would pass."""
    folder, cfg = model_folders["E"], CONFIGS["E"]
    toks = random_tokens(91, 2640, cfg.vocab_size)[:2000]
    full = _plain(plain_cache, folder, toks)[-1]
    cfg_d, w = load_plain(folder)
    cut = plain_model.forward({**cfg_d, "use_sliding_window": True, "sliding_window": 2000 - 64,
                               "layer_types": ["sliding_attention"] * cfg.num_hidden_layers}, w, toks)[-1]
    assert np.abs(full - cut).max() > 2 * TOL["bfloat16"] * np.abs(full).max()


# ---- pages of 8 tokens ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D", "E"])
def test_the_four_schedules_with_pages_of_8_tokens(name, dtype, model_folders, plain_cache):
    """Whole, last 32 one by one, changing portions, and mixed with reused pages - with 8-token pages."""
    from pulse_infer_b200.engine import Segment
    need_gpu()
    folder, cfg = model_folders[name], CONFIGS[name]
    runner = _runner(folder, dtype, page_size=8, num_pages=30, max_requests=4, max_tokens_per_request=128)
    toks = random_tokens(41, 100, cfg.vocab_size)
    want = _plain(plain_cache, folder, toks)
    runner.open("w")
    _check(runner.step([Segment("w", toks, list(range(100)))]), want, dtype, f"{name} whole")
    runner.close("w")
    runner.open("d")
    _check(runner.step([Segment("d", toks[:68], [67])]), want[67:68], dtype, f"{name} head")
    for i in range(68, 100):
        _check(runner.step([Segment("d", [toks[i]], [0])]), want[i:i + 1], dtype, f"{name} decode at {i}")
    runner.close("d")
    runner.open("p")
    at, k, sizes = 0, 0, [7, 2, 13, 2, 5, 3, 2, 31, 2, 17]
    while at < 100:
        c = min(sizes[k % len(sizes)], 100 - at)
        k += 1
        _check(runner.step([Segment("p", toks[at:at + c], list(range(c)))]), want[at:at + c], dtype, f"{name} portion at {at}")
        at += c
    runner.close("p")
    runner.check_device_errors()
    # mixed: five requests through a pool of 30 pages (240 tokens), at most four live
    lengths = [90, 41, 64, 33, 75]
    reqs = {f"m{i}": random_tokens(50 + i, n, cfg.vocab_size) for i, n in enumerate(lengths)}
    wants = {rid: _plain(plain_cache, folder, t) for rid, t in reqs.items()}
    rng = np.random.RandomState(3)
    waiting, live, freed, reused, steps = list(reqs), {}, set(), False, 0
    while waiting or live:
        while waiting and len(live) < 4:
            need = (len(reqs[waiting[0]]) + 7) // 8
            if sum((len(reqs[r]) + 7) // 8 for r in live) + need > 30:
                break
            rid = waiting.pop(0)
            runner.open(rid)
            live[rid] = 0
        segs, spans = [], []
        for rid, a in live.items():
            n = len(reqs[rid])
            c = min(int(rng.choice([2, 3, 5, 11, 24])), n - 8 - a) if a < n - 8 else 1
            segs.append(Segment(rid, reqs[rid][a:a + c], list(range(c))))
            spans.append((rid, a, c))
        logits = runner.step(segs)
        row = 0
        for rid, a, c in spans:
            _check(logits[row:row + c], wants[rid][a:a + c], dtype, f"{name} mixed step {steps} {rid}[{a}:{a + c}]")
            row += c
            live[rid] = a + c
        g = runner.cache.groups[0]
        reused = reused or bool({int(p) for r in live for p in g.table.row(runner.cache.slot(r)) if p >= 0} & freed)
        for rid in [r for r, a in live.items() if a == len(reqs[r])]:
            freed |= {int(p) for p in g.table.row(runner.cache.slot(rid)) if p >= 0}
            runner.close(rid)
            del live[rid]
        runner.cache.check_invariants()
        steps += 1
    runner.check_device_errors()
    assert reused


# ---- the real widths ---------------------------------------------------------------------------------------------------
def test_two_layers_at_the_widths_of_the_8b_shape():
    """Hidden 4096, 32 / 8 heads of 128, intermediate 12288, vocabulary 151,936 - two layers of it, in bfloat16: a
    prompt of 64 tokens, then 8 tokens one by one (recorded steps), against the plain implementation in float32
    numpy on the same weights (the seeded generator gives the same values on the device and on the host)."""
    from pulse_infer_b200.config import Qwen3Config
    from pulse_infer_b200.engine import Segment, build_runner
    from pulse_infer_b200.weights.random_init import _spec_only_model, random_tensors
    need_gpu()
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                      max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
                      torch_dtype="bfloat16", eos_token_ids=())
    runner = build_runner(None, config=cfg, seed=11, dtype="bfloat16", device="cuda:0", page_size=16, num_pages=16,
                          max_requests=2, max_tokens_per_request=128, use_cuda_graphs=True)
    dev = torch.device("cuda:0")
    w = {name: t.float().cpu().numpy() for name, _, _, t in random_tensors(_spec_only_model(cfg), 11, torch.bfloat16, dev)}
    toks = random_tokens(12, 72, cfg.vocab_size)
    want = plain_model.forward(cfg.to_json_dict(), w, toks, dtype=np.float32).astype(np.float64)
    runner.open("x")
    got = [runner.step([Segment("x", toks[:64], [0, 31, 63])]).cpu()]
    rows = [0, 31, 63]
    for i in range(64, 72):
        got.append(runner.step([Segment("x", [toks[i]], [0])]).cpu())
        rows.append(i)
    runner.check_device_errors()
    _check(torch.cat(got), want[rows], "bfloat16", "8B widths, two layers")
    assert (torch.cat(got).argmax(-1).numpy() == want[rows].argmax(-1)).mean() >= 0.7      # near-ties aside


# ---- a window as long as a key range ---------------------------------------------------------------------------------
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_of_256_keys_with_requests_either_side_of_a_range_boundary(dtype, graphs, plain_cache, tmp_path_factory):
    """With a window the number of key ranges is not monotone in the position (the window's first key is rounded down
    to a multiple of 64): at a window of 256 keys and ranges of 256 keys, the request at position 511 needs one range
    and the one at 300 needs two.  Both decode in the same steps, the longer one crossing positions 500 to 530."""
    import dataclasses
    from pulse_infer_b200.engine import Segment
    from pulse_infer_b200.weights import write_random_model
    from tiny_configs import TINY_D
    need_gpu()
    cfg = dataclasses.replace(TINY_D, sliding_window=256, layer_types=("sliding_attention", "sliding_attention"))
    folder = str(tmp_path_factory.mktemp("tiny_D_window256"))
    write_random_model(cfg, 8, folder, dtype="bfloat16")
    reqs = {"far": random_tokens(61, 531, cfg.vocab_size), "near": random_tokens(62, 321, cfg.vocab_size),
            "short": random_tokens(63, 71, cfg.vocab_size)}
    want = {r: _plain(plain_cache, folder, t) for r, t in reqs.items()}
    runner = _runner(folder, dtype, num_pages=80, max_requests=4, max_tokens_per_request=640, use_cuda_graphs=graphs)
    at = {}
    for rid, toks in reqs.items():
        runner.open(rid)
        head = len(toks) - 31
        _check(runner.step([Segment(rid, toks[:head], [head - 1])]), want[rid][head - 1:head], dtype, f"prompt {rid}")
        at[rid] = head
    from pulse_infer_b200 import ops
    assert ops.attention_num_splits(511, 256, 256) == 1 and ops.attention_num_splits(300, 256, 256) == 2
    for k in range(31):
        order = ["far", "near", "short"] if k % 2 else ["short", "near", "far"]
        segs = [Segment(r, [reqs[r][at[r]]], [0]) for r in order]
        got = runner.step(segs)
        for i, r in enumerate(order):
            _check(got[i:i + 1], want[r][at[r]:at[r] + 1], dtype, f"window 256, step {k}, {r}@{at[r]}")
            at[r] += 1
    runner.check_device_errors()
    for r in reqs:
        runner.close(r)
    runner.cache.check_invariants()
