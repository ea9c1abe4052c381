"""Generation through the Python entry point and the command line, the parts of a layer alone, and a
toy mixer with state of its own that is registered from here without touching the framework."""
import dataclasses
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
from gpu_util import need_gpu
from helpers import load_plain, random_tokens
from tiny_configs import CONFIGS, SEEDS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plain_generate(cfg, w, prompt, max_new, temperature=0.0, top_k=0, top_p=0.0, seed=0, eos=()):
    toks, out = list(prompt), []
    for i in range(max_new):
        logits = plain_model.forward(cfg, w, toks)[-1]
        t = plain_model.sample(logits, temperature, top_k, top_p, seed, i)
        out.append(t); toks.append(t)
        if t in eos:
            break
    return out


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_float32_config_a(model_folders, graphs):
    """Tiny A: prompts of 5 and 17 tokens, 8 greedy steps, through Engine.generate."""
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["A"], CONFIGS["A"]
    pc, pw = load_plain(folder)
    prompts = [random_tokens(1, 5, cfg.vocab_size), random_tokens(2, 17, cfg.vocab_size)]
    engine = Engine(folder, dtype="float32", page_size=8, num_pages=16, max_batch_size=2, chunk_size=256,
                    use_cuda_graphs=graphs)
    got = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    want = [_plain_generate(pc, pw, p, 8) for p in prompts]
    assert got == want
    st = engine.get_stats()
    assert st.num_finished == 2 and st.decode_tokens == 14 and list(st.free_pages) == [16]


@pytest.mark.parametrize("graphs", [False, True])
def test_sampled_generation_mixed_batch_config_b(model_folders, graphs):
    """Tiny B: three requests (prompts 1, 23, 40), portions of 7, 12 tokens at temperature 0.8, seeded."""
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["B"], CONFIGS["B"]
    pc, pw = load_plain(folder)
    prompts = [random_tokens(s, n, cfg.vocab_size) for s, n in ((1, 1), (2, 23), (3, 40))]
    engine = Engine(folder, dtype="float32", page_size=16, num_pages=12, max_batch_size=3, chunk_size=7,
                    use_cuda_graphs=graphs)
    ids = [engine.add_request(p, 12, temperature=0.8, seed=100 + i, ignore_eos=True) for i, p in enumerate(prompts)]
    engine.run_until_complete()
    for i, (rid, p) in enumerate(zip(ids, prompts)):
        assert engine.get_result(rid) == _plain_generate(pc, pw, p, 12, temperature=0.8, seed=100 + i)


def test_lookahead_gives_the_same_tokens_as_reading_every_step(model_folders):
    """bfloat16, head size 64, requests of different lengths that end at different steps (length limits and EOS
    ids): with a decode step kept in flight the results are those of the plain loop, and steps did stay in flight."""
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["D"], CONFIGS["D"]
    prompts = [random_tokens(20 + i, n, cfg.vocab_size) for i, n in enumerate((5, 33, 70, 18, 51))]
    limits = [9, 30, 17, 40, 25]
    results, in_flight = {}, {}
    for lookahead in (False, True):
        engine = Engine(folder, dtype="bfloat16", page_size=16, num_pages=40, max_batch_size=4, chunk_size=32,
                        lookahead=lookahead)
        engine.engine.eos_token_ids = (7, 100, 200, 287)          # ids this random model does produce
        ids = [engine.add_request(p, m, temperature=0.7 if i % 2 else 0.0, top_k=50, seed=5 + i)
               for i, (p, m) in enumerate(zip(prompts, limits))]
        count = 0
        while engine.has_work():
            engine.step()
            count += engine.engine._inflight is not None
        results[lookahead] = [(engine.get_result(i), engine.get_request(i).finish_reason) for i in ids]
        in_flight[lookahead] = count
        engine.runner.check_device_errors()
        engine.runner.cache.check_invariants()
        assert engine.runner.cache.free_pages() == [40] * len(engine.runner.cache.free_pages())
    assert results[True] == results[False]
    assert in_flight[False] == 0 and in_flight[True] >= 10
    assert {r for _, r in results[True]} <= {"eos", "length"}


def test_warm_up_records_every_batch_size_once(model_folders):
    """After ``Engine.warm_up()`` the decode steps of all batch sizes are recorded: a run whose batch shrinks request by
    request records nothing more, leaves every page free, and gives the tokens of an engine that was not warmed up."""
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["D"], CONFIGS["D"]
    prompts = [random_tokens(40 + i, n, cfg.vocab_size) for i, n in enumerate((9, 21, 14, 30))]
    limits = [6, 11, 16, 21]
    results = {}
    for warm in (False, True):
        engine = Engine(folder, dtype="bfloat16", page_size=16, num_pages=40, max_batch_size=4, chunk_size=32)
        graphs = engine.runner.graphs
        if warm:
            assert engine.warm_up() == 4 and graphs.recordings == 4
            assert engine.warm_up() == 0                                   # nothing left to record
            assert engine.runner.cache.free_pages() == [40] * len(engine.runner.cache.free_pages())
        before = graphs.recordings
        ids = [engine.add_request(p, m, ignore_eos=True) for p, m in zip(prompts, limits)]
        engine.run_until_complete()
        results[warm] = [engine.get_result(i) for i in ids]
        assert (graphs.recordings - before == 0) if warm else (graphs.recordings - before >= 3)
        engine.runner.check_device_errors()
        engine.runner.cache.check_invariants()
    assert results[True] == results[False]
    no_graphs = Engine(folder, dtype="bfloat16", page_size=16, num_pages=40, max_batch_size=4, use_cuda_graphs=False)
    assert no_graphs.warm_up() == 0


def test_engine_run_and_replay_through_the_python_entry_point(model_folders):
    """``Engine.run()`` returns what every request generated; ``Engine.replay(trace)`` feeds given ids through the same
    engine's step function and returns the logits at the wanted places - those of the plain implementation, whatever
    the cut - and leaves the engine ready to generate."""
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["B"], CONFIGS["B"]
    pc, pw = load_plain(folder)
    engine = Engine(folder, dtype="float32", page_size=16, num_pages=24, max_batch_size=3, chunk_size=16)
    a, b = random_tokens(71, 37, cfg.vocab_size), random_tokens(72, 12, cfg.vocab_size)
    trace = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [19]}, {"id": "b", "tokens": b[:5], "want": []}]},
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": a[20:22], "want": [0, 1]}, {"id": "b", "tokens": b[5:], "want": [6]}], "end": ["b"]}),
             {"step": 2, "entries": [{"id": "a", "tokens": a[22:], "want": [14]}], "end": ["a"]},
             {"step": 3, "entries": [], "end": []}]
    got = engine.replay(trace)
    assert sorted(got) == [0, 1, 2]
    wa, wb = plain_model.forward(pc, pw, a), plain_model.forward(pc, pw, b)
    for step, want in ((0, wa[[19]]), (1, np.concatenate([wa[[20, 21]], wb[[11]]])), (2, wa[[36]])):
        assert got[step].shape == want.shape and got[step].dtype == np.float32
        assert np.abs(got[step] - want).max() <= 2e-5 * np.abs(want).max()
    assert engine.runner.cache.free_pages() == [24] * len(engine.runner.cache.free_pages())
    ids = [engine.add_request(p, 5, ignore_eos=True) for p in (a[:9], b)]
    with pytest.raises(RuntimeError):
        engine.replay(trace)                                  # requests in flight
    done = engine.run()
    assert done == {ids[0]: _plain_generate(pc, pw, a[:9], 5), ids[1]: _plain_generate(pc, pw, b, 5)}


def test_generation_survives_preemption_and_eos(model_folders):
    """So few pages that requests are preempted and recomputed; tokens are the same as with plenty."""
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["C"], CONFIGS["C"]
    prompts = [random_tokens(20 + i, n, cfg.vocab_size) for i, n in enumerate((30, 18, 25, 9))]
    outs = {}
    for pages in (64, 7):
        engine = Engine(folder, dtype="float32", page_size=8, num_pages=pages, max_batch_size=3, chunk_size=16,
                        max_tokens_per_request=128)
        ids = [engine.add_request(p, 20, temperature=0.7, top_k=50, top_p=0.9, seed=i, ignore_eos=True)
               for i, p in enumerate(prompts)]
        engine.run_until_complete()
        outs[pages] = [engine.get_result(i) for i in ids]
        if pages == 7:
            assert engine.get_stats().num_preemptions > 0
        engine.runner.cache.check_invariants()
    assert outs[64] == outs[7] and all(len(o) == 20 for o in outs[64])
    # EOS: take a token the first request generates and declare it the stop token
    stop = outs[64][0][5]
    engine = Engine(folder, dtype="float32", page_size=8, num_pages=64, max_batch_size=3, max_tokens_per_request=128)
    engine.engine.eos_token_ids = (stop,)
    rid = engine.add_request(prompts[0], 20, temperature=0.7, top_k=50, top_p=0.9, seed=0)
    engine.run_until_complete()
    first = outs[64][0].index(stop)
    assert engine.get_result(rid) == outs[64][0][:first + 1] and engine.get_request(rid).finish_reason == "eos"


def test_bfloat16_greedy_tokens_are_top_tokens(model_folders):
    need_gpu()
    from pulse_infer_b200 import Engine
    folder, cfg = model_folders["B"], CONFIGS["B"]
    pc, pw = load_plain(folder)
    prompts = [random_tokens(5, 33, cfg.vocab_size), random_tokens(6, 4, cfg.vocab_size)]
    for graphs in (False, True):
        engine = Engine(folder, dtype="bfloat16", page_size=16, num_pages=16, max_batch_size=2, use_cuda_graphs=graphs)
        outs = engine.generate(prompts, max_new_tokens=10, ignore_eos=True)
        for p, o in zip(prompts, outs):
            ref = plain_model.forward(pc, pw, p + o)
            for i, t in enumerate(o):
                row = ref[len(p) + i - 1]
                assert row[t] >= row.max() - 0.02 * np.abs(row).max()


def test_command_line_programs(model_folders, tmp_path):
    need_gpu()
    folder = model_folders["A"]
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_continuous_batch_demo"), folder,
                          "--dtype", "float32", "--prompt-len", "9", "--prompt-len", "21", "--max-new-tokens", "6",
                          "--ignore-eos", "--chunk-size", "8"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    pc, pw = load_plain(folder)
    for i, (rec, n) in enumerate(zip(lines, (9, 21))):
        prompt = [int(t) for t in np.random.RandomState(i).randint(0, CONFIGS["A"].vocab_size, size=n)]
        assert rec["generated"] == _plain_generate(pc, pw, prompt, 6)
    assert "tokens/s" in out.stdout
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_infer"), folder, "--prompt-ids", "1,2,3,4",
                          "--max-new-tokens", "5", "--ignore-eos", "--seed", "3"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][0])
    assert len(rec["generated"]) == 5 and "tokens/s" in out.stdout
    # the pool sized by memory, a token budget per step, and the largest logits behind every token (greedy: the first
    # of them is the token, and they are the plain implementation's)
    prompt = [5, 6, 7, 8, 9, 10, 11, 12, 13]
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_infer"), folder, "--dtype", "float32",
                          "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "4", "--ignore-eos", "--greedy",
                          "--presence-penalty", "0", "--kv-gb", "0.001", "--max-tokens-per-step", "4",
                          "--print-logits-topk", "3"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][0])
    want = _plain_generate(pc, pw, prompt, 4)
    assert rec["generated"] == want and len(rec["logits_topk"]) == 4
    toks = list(prompt)
    for tok, top in zip(want, rec["logits_topk"]):
        row = plain_model.forward(pc, pw, toks)[-1]
        assert top[0][0] == tok and len(top) == 3
        assert [t for t, _ in top] == [int(i) for i in np.argsort(-row, kind="stable")[:3]]
        assert abs(top[0][1] - row[tok]) <= 2e-5 * np.abs(row).max() + 1e-5
        toks.append(tok)
    # --bench: the same prompts timed instead of printed, one JSON line per kind
    for kind in ("serve", "prefill", "decode"):
        out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_continuous_batch_demo"), model_folders["D"],
                              "--prompt-len", "40", "--prompt-len", "9", "--prompt-len", "70", "--max-new-tokens", "12",
                              "--max-batch-size", "3", "--chunk-size", "32", "--bench", kind],
                             capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        recs = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
        assert len(recs) == 1
        rec = recs[0]
        assert rec["bench"] == kind and rec["requests"] == 3 and rec["prompt_tokens"] == 119 and rec["seconds"] > 0
        assert rec["decode_steps_recorded_before"] == 3 and rec["preemptions"] == 0
        if kind == "serve":
            assert rec["generated_tokens"] == 36 and rec["generated_tokens_per_s"] > 0 and rec["all_tokens_per_s"] > rec["generated_tokens_per_s"]
        elif kind == "prefill":
            assert rec["generated_tokens"] == 3 and rec["prompt_tokens_per_s"] > 0
        else:
            # timed from the step after the last prompt portion: the tokens sampled by then are not counted
            assert rec["generated_tokens"] == 36 and 30 <= rec["timed_tokens"] <= 35 and rec["steps"] <= 12


# ---- each part of a layer alone ----------------------------------------------------------------------------
def _ctx_for(segs, cache_specs, runtime, page_size=8, state_specs=None):
    """A cache manager and a step context for hand-made segments [(request id, start, tokens)]."""
    from pulse_infer_b200.cache import CacheManager
    from pulse_infer_b200.engine import Segment, StepContext
    cm = CacheManager(cache_specs, state_specs or [None] * len(cache_specs), page_size, 32, 4, 256,
                      dtype=runtime.act_dtype, device=runtime.device)
    segments = []
    for rid, start, toks in segs:
        cm.open(rid); cm.reserve(rid, start + len(toks)); cm.commit(rid, start)
        s = Segment(rid, toks, [len(toks) - 1]); s.slot = cm.slot(rid); s.start = start
        segments.append(s)
    cm.sync_tables()
    return cm, StepContext.build(segments, runtime, cm)


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_parts_alone(mode):
    dev = need_gpu()
    from pulse_infer_b200.parts import Runtime, build_part
    rt = Runtime(dev, mode)
    dt = rt.act_dtype
    tol = 1e-5 if mode == "float32" else 2e-2
    g = torch.Generator().manual_seed(0)
    H, I, nq, nkv, d, T = 72, 200, 6, 3, 32, 11
    _, ctx = _ctx_for([("a", 0, list(range(T)))], [None], rt)

    norm = build_part("norm", "rmsnorm", dict(size=H, eps=1e-5))
    wn = (1 + 0.1 * torch.randn(H, generator=g)).to(dt)
    norm.load({"weight": wn.to(dev)}, rt)
    h = torch.randn(T, H, generator=g)
    got = norm.forward(h.clone().to(dev), ctx).cpu().double().numpy()
    want = plain_model.rms_norm(h.double().numpy(), wn.double().numpy(), 1e-5)
    assert np.abs(got - want).max() <= tol * np.abs(want).max()

    ff = build_part("feed_forward", "swiglu", dict(hidden_size=H, intermediate_size=I))
    ws = {k: (torch.randn(*shape, generator=g) * 0.1).to(dt) for k, shape in
          (("gate_proj.weight", (I, H)), ("up_proj.weight", (I, H)), ("down_proj.weight", (H, I)))}
    ff.load({k: v.to(dev) for k, v in ws.items()}, rt)
    x = torch.randn(T, H, generator=g).to(dt)
    got = ff.forward(x.to(dev), ctx).cpu().double().numpy()
    want = plain_model.swiglu(x.double().numpy(), *[ws[k].double().numpy() for k in ws])
    assert np.abs(got - want).max() <= tol * np.abs(want).max()

    rope = build_part("position_encoding", "rotary", dict(theta=5000.0, rotary_dim=d, pairing="half"))
    _, ctx2 = _ctx_for([("a", 37, list(range(T)))], [None], rt)
    tab = rope.prepare(ctx2)
    ang = np.arange(37, 37 + T)[:, None] / np.power(5000.0, 2.0 * np.arange(d // 2) / d)[None, :]
    assert np.abs(tab["cos"].cpu().numpy() - np.cos(ang)).max() < 1e-6 and tab["adjacent"] is False

    # attention part: a portion of 11 tokens at position 37 of a request whose first 37 tokens are in the cache
    from pulse_infer_b200.parts.base import CacheSpec
    for pairing, window in (("adjacent", None), ("half", 9)):
        attn = build_part("mixer", "attention", dict(hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                                                    qk_norm=True, norm_eps=1e-5, position="rot", window=window))
        aw = {k: (torch.randn(*shape, generator=g) * 0.15).to(dt) for k, shape in
              (("q_proj.weight", (nq * d, H)), ("k_proj.weight", (nkv * d, H)), ("v_proj.weight", (nkv * d, H)),
               ("o_proj.weight", (H, nq * d)))}
        aw["q_norm.weight"] = (1 + 0.1 * torch.randn(d, generator=g)).to(dt)
        aw["k_norm.weight"] = (1 + 0.1 * torch.randn(d, generator=g)).to(dt)
        attn.load({k: v.to(dev) for k, v in aw.items()}, rt)
        rope = build_part("position_encoding", "rotary", dict(theta=5000.0, rotary_dim=d, pairing=pairing))
        xs = torch.randn(48, H, generator=g).to(dt)
        cm, ctx_a = _ctx_for([("a", 0, list(range(37)))], [attn.cache_spec()], rt)
        ctx_a.position_data = {"rot": rope.prepare(ctx_a)}
        y1 = attn.forward(xs[:37].to(dev), ctx_a, ctx_a.cache_view(0, 0))
        cm.commit("a", 37)
        from pulse_infer_b200.engine import Segment, StepContext
        seg = Segment("a", list(range(11)), [10]); seg.slot = cm.slot("a"); seg.start = 37
        cm.reserve("a", 48); cm.sync_tables()
        ctx_b = StepContext.build([seg], rt, cm)
        ctx_b.position_data = {"rot": rope.prepare(ctx_b)}
        y2 = attn.forward(xs[37:].to(dev), ctx_b, ctx_b.cache_view(0, 0))
        got = torch.cat([y1, y2]).cpu().double().numpy()
        xd = xs.double().numpy()
        wd = {k: v.double().numpy() for k, v in aw.items()}
        pos = np.arange(48)
        q = plain_model.rope(plain_model.rms_norm((xd @ wd["q_proj.weight"].T).reshape(48, nq, d), wd["q_norm.weight"], 1e-5), pos, 5000.0, d, pairing)
        k = plain_model.rope(plain_model.rms_norm((xd @ wd["k_proj.weight"].T).reshape(48, nkv, d), wd["k_norm.weight"], 1e-5), pos, 5000.0, d, pairing)
        v = (xd @ wd["v_proj.weight"].T).reshape(48, nkv, d)
        want = plain_model.attention(q, k, v, window).reshape(48, nq * d) @ wd["o_proj.weight"].T
        assert np.abs(got - want).max() <= tol * np.abs(want).max(), (pairing, window)


# ---- a toy mixer with state, registered from the test ----------------------------------------------------------
def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A new architecture whose second layer's mixer is a decaying running sum kept in the per-request
    state slot.  Nothing under pulse_infer_b200/ is changed: the mixer, the architecture and its
    configuration are registered here."""
    dev = need_gpu()
    from pulse_infer_b200 import ops
    from pulse_infer_b200.config import Qwen3Config, register_architecture
    from pulse_infer_b200.engine import Segment, build_runner
    from pulse_infer_b200.models.qwen3 import build_qwen3_spec
    from pulse_infer_b200.models.spec import PartSpec
    from pulse_infer_b200.parts.base import MIXERS, Mixer, StateSpec, TensorSpec, register_part
    from pulse_infer_b200.weights import write_random_model

    DECAY = 0.75

    class DecaySum(Mixer):
        """s_t = decay * s_(t-1) + x_t per request; y_t = W s_t.  State: s, one vector per request."""

        def __init__(self, hidden_size, decay):
            self.hidden_size, self.decay = hidden_size, decay

        def tensor_specs(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def state_spec(self):
            return StateSpec((self.hidden_size,), torch.float32)

        def load(self, tensors, runtime):
            self.w = tensors["mix.weight"]
            self._tensors = {"w": self.w}

        def forward(self, x, ctx, cache):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for seg in ctx.segments:
                s = cache.state[seg.slot]
                for i in range(len(seg.tokens)):
                    s = self.decay * s + x[seg.offset + i].float()
                    out[seg.offset + i] = s
                cache.state[seg.slot] = s
            return ops.linear(out.to(x.dtype), self.w, ctx.act_dtype)

    if "decay_sum" not in MIXERS:
        register_part("mixer", "decay_sum")(DecaySum)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(Qwen3Config):
        pass

    def build_toy_spec(config):
        spec = build_qwen3_spec(config)
        layers = list(spec.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=PartSpec(
            "decay_sum", dict(hidden_size=config.hidden_size, decay=DECAY), "model.layers.1.toy."))
        order = tuple(dataclasses.replace(e, cache=None) if e.layer == 1 else e for e in spec.order)
        return dataclasses.replace(spec, layers=tuple(layers), order=order)

    register_architecture("ToyStateForCausalLM", ToyConfig, build_toy_spec, replace=True)
    cfg = dataclasses.replace(CONFIGS["B"], architecture="ToyStateForCausalLM")
    cfg = ToyConfig(**{f.name: getattr(cfg, f.name) for f in dataclasses.fields(cfg)})
    folder = write_random_model(cfg, 5, str(tmp_path / "toy"), dtype="bfloat16")
    pc, pw = load_plain(folder)
    assert "model.layers.1.toy.mix.weight" in pw and "model.layers.1.self_attn.q_proj.weight" not in pw

    def plain_toy(tokens):
        w = {k: np.asarray(v, dtype=np.float64) for k, v in pw.items()}
        positions = np.arange(len(tokens))
        h = plain_model.embedding(w["model.embed_tokens.weight"], tokens)
        for layer in range(pc["num_hidden_layers"]):
            prefix = f"model.layers.{layer}."
            if layer != 1:
                h, _ = plain_model.decoder_layer(h, w, prefix, pc, positions)
                continue
            x = plain_model.rms_norm(h, w[prefix + "input_layernorm.weight"], pc["rms_norm_eps"])
            s, ys = np.zeros(h.shape[1]), []
            for t in range(len(tokens)):
                s = DECAY * s + x[t]
                ys.append(s.copy())
            h = h + plain_model.linear(np.stack(ys), w[prefix + "toy.mix.weight"])
            x = plain_model.rms_norm(h, w[prefix + "post_attention_layernorm.weight"], pc["rms_norm_eps"])
            h = h + plain_model.swiglu(x, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                                       w[prefix + "mlp.down_proj.weight"])
        x = plain_model.rms_norm(h, w["model.norm.weight"], pc["rms_norm_eps"])
        return plain_model.linear(x, w["lm_head.weight"])

    runner = build_runner(folder, dtype="float32", device="cuda:0", page_size=8, num_pages=32, max_requests=3,
                          max_tokens_per_request=128)
    assert 1 in runner.cache.state and runner.cache.state[1].shape == (3, cfg.hidden_size)
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].cache_indices == [0, 2]
    reqs = {"a": random_tokens(1, 40, cfg.vocab_size), "b": random_tokens(2, 23, cfg.vocab_size)}
    want = {k: plain_toy(v) for k, v in reqs.items()}
    runner.open("a"); runner.open("b")
    plan = [[("a", 0, 13), ("b", 0, 2)], [("a", 13, 14), ("b", 2, 20)], [("a", 14, 15)], [("b", 20, 21), ("a", 15, 40)],
            [("b", 21, 23)]]
    for step in plan:
        logits = runner.step([Segment(r, reqs[r][a:b], list(range(b - a))) for r, a, b in step]).cpu().double().numpy()
        ref = np.concatenate([want[r][a:b] for r, a, b in step])
        assert np.abs(logits - ref).max() <= 2e-5 * np.abs(ref).max()
    # a slot that is reused starts from zero state
    runner.close("a"); runner.open("c")
    logits = runner.step([Segment("c", reqs["b"], list(range(23)))]).cpu().double().numpy()
    assert np.abs(logits - want["b"]).max() <= 2e-5 * np.abs(want["b"]).max()

    # ---- through the entry point, where recording of decode steps is on by default ---------------------------------
    # Three requests of different lengths and limits: the set of slots in a two-request decode step changes while
    # steps of that shape have already run.  DecaySum walks ctx.segments on the host, so it does not declare itself
    # capturable and its steps are launched kernel by kernel; the tokens are the plain implementation's.
    from pulse_infer_b200 import Engine
    prompts = [random_tokens(7, 5, cfg.vocab_size), random_tokens(8, 11, cfg.vocab_size), random_tokens(9, 17, cfg.vocab_size)]
    limits = [12, 7, 15]

    def plain_greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(plain_model.greedy(plain_toy(toks)[-1]))
        return toks[len(prompt):]
    want_tokens = [plain_greedy(p, n) for p, n in zip(prompts, limits)]
    eng = Engine(folder, dtype="float32", page_size=8, num_pages=32, max_batch_size=3, use_cuda_graphs=True)
    assert not eng.runner.model.capturable
    ids = [eng.add_request(p, n, ignore_eos=True) for p, n in zip(prompts, limits)]
    eng.run_until_complete()
    assert [eng.get_result(i) for i in ids] == want_tokens
    assert not eng.runner.graphs.graphs                      # nothing was recorded

    # The same mixer written so that a recorded step stays right: for steps of single tokens it reads the slots from
    # the device (ctx.seg_slot) and updates the state with device-side gathers and scatters; it says capturable.
    # The engine's warm-up run before the recording must not advance the state twice.
    class DecaySumDevice(DecaySum):
        capturable = True

        def forward(self, x, ctx, cache):
            if ctx.max_seg_len > 1:                           # portions: not recorded, the host loop will do
                return DecaySum.forward(self, x, ctx, cache)
            slots = ctx.seg_slot.long()
            s = self.decay * cache.state.index_select(0, slots) + x.float()
            cache.state.index_copy_(0, slots, s)
            return ops.linear(s.to(x.dtype), self.w, ctx.act_dtype)

    if "decay_sum_device" not in MIXERS:
        register_part("mixer", "decay_sum_device")(DecaySumDevice)

    def build_toy_device_spec(config):
        spec = build_toy_spec(config)
        layers = list(spec.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=dataclasses.replace(layers[1].mixer, kind="decay_sum_device"))
        return dataclasses.replace(spec, layers=tuple(layers))

    register_architecture("ToyStateDeviceForCausalLM", ToyConfig, build_toy_device_spec, replace=True)
    cfg2 = dataclasses.replace(cfg, architecture="ToyStateDeviceForCausalLM")
    folder2 = write_random_model(cfg2, 5, str(tmp_path / "toy_device"), dtype="bfloat16")
    eng = Engine(folder2, dtype="float32", page_size=8, num_pages=32, max_batch_size=3, use_cuda_graphs=True)
    assert eng.runner.model.capturable
    ids = [eng.add_request(p, n, ignore_eos=True) for p, n in zip(prompts, limits)]
    eng.run_until_complete()
    assert [eng.get_result(i) for i in ids] == want_tokens
    assert {key[0] for key in eng.runner.graphs.graphs} >= {1, 2, 3}      # decode steps of 3, 2 and 1 requests were recorded


# ---- a toy feed-forward with routing and a toy position encoding, registered from the test ------------------------
def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path):
    """A new architecture: the first layer's feed-forward routes every token to one of four small experts
    (router logits and softmax in 32-bit, top 1), and positions rotate only the first half of each head, with
    angles that grow linearly in the pair index and 'half' pairing.  Both parts, the architecture and its
    configuration are registered here; nothing under pulse_infer_b200/ is changed."""
    dev = need_gpu()
    from pulse_infer_b200.config import Qwen3Config, register_architecture
    from pulse_infer_b200.engine import Segment, build_runner
    from pulse_infer_b200.models.qwen3 import build_qwen3_spec
    from pulse_infer_b200.models.spec import PartSpec
    from pulse_infer_b200.parts.base import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding, TensorSpec,
                                             register_part)
    from pulse_infer_b200.weights import write_random_model

    EXPERTS, WIDTH, ALPHA = 4, 40, 0.013

    class Top1Experts(FeedForward):
        """y = p_e * W_out[e] relu(W_in[e] x), e = argmax of the router's logits, p = their softmax."""

        def __init__(self, hidden_size, experts, width):
            self.hidden_size, self.experts, self.width = hidden_size, experts, width

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.experts, self.hidden_size))}
            for e in range(self.experts):
                specs[f"experts.{e}.in.weight"] = TensorSpec((self.width, self.hidden_size))
                specs[f"experts.{e}.out.weight"] = TensorSpec((self.hidden_size, self.width))
            return specs

        def load(self, tensors, runtime):
            self.router = tensors["router.weight"].float()
            self.w_in = torch.stack([tensors[f"experts.{e}.in.weight"].float() for e in range(self.experts)])
            self.w_out = torch.stack([tensors[f"experts.{e}.out.weight"].float() for e in range(self.experts)])
            self._tensors = {"router": self.router, "w_in": self.w_in, "w_out": self.w_out}

        def first_weights(self):
            return None

        def forward(self, x, ctx):
            xf = x.float()
            probs = torch.softmax(xf @ self.router.t(), dim=-1)
            p, e = probs.max(dim=-1)
            hid = torch.relu(torch.einsum("tfh,th->tf", self.w_in[e], xf))
            return (torch.einsum("thf,tf->th", self.w_out[e], hid) * p[:, None]).to(x.dtype)

    class LinearRotary(PositionEncoding):
        """angle(pos, i) = pos * alpha * (i + 1) for pair i of the first ``rotary_dim`` elements, pairs (i, i + rot/2)."""

        def __init__(self, alpha, rotary_dim):
            self.alpha, self.rotary_dim = alpha, rotary_dim

        def prepare(self, ctx):
            i = torch.arange(1, self.rotary_dim // 2 + 1, dtype=torch.float64, device=ctx.positions.device)
            ang = ctx.positions.double()[:, None] * (self.alpha * i)[None, :]
            return {"cos": torch.cos(ang).float().contiguous(), "sin": torch.sin(ang).float().contiguous(), "adjacent": False}

    if "top1_experts" not in FEED_FORWARDS:
        register_part("feed_forward", "top1_experts")(Top1Experts)
    if "linear_rotary" not in POSITION_ENCODINGS:
        register_part("position_encoding", "linear_rotary")(LinearRotary)

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig(Qwen3Config):
        pass

    def build_routed_spec(config):
        spec = build_qwen3_spec(config)
        layers = list(spec.layers)
        layers[0] = dataclasses.replace(layers[0], feed_forward=PartSpec(
            "top1_experts", dict(hidden_size=config.hidden_size, experts=EXPERTS, width=WIDTH), "model.layers.0.moe."))
        positions = {"rotary": PartSpec("linear_rotary", dict(alpha=ALPHA, rotary_dim=config.head_dim // 2))}
        return dataclasses.replace(spec, layers=tuple(layers), positions=positions)

    register_architecture("RoutedForCausalLM", RoutedConfig, build_routed_spec, replace=True)
    base = CONFIGS["B"]
    cfg = RoutedConfig(**{**{f.name: getattr(base, f.name) for f in dataclasses.fields(base)},
                          "architecture": "RoutedForCausalLM"})
    folder = write_random_model(cfg, 11, str(tmp_path / "routed"), dtype="bfloat16")
    pc, pw = load_plain(folder)
    assert "model.layers.0.moe.router.weight" in pw and "model.layers.0.mlp.gate_proj.weight" not in pw

    def toy_rope(x, positions):
        rot = pc["head_dim"] // 2
        pairs = rot // 2
        ang = np.asarray(positions, dtype=np.float64)[:, None] * (ALPHA * np.arange(1, pairs + 1))[None, :]
        cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        out = x.copy()
        a, b = x[..., :pairs], x[..., pairs:rot]
        out[..., :pairs] = a * cos - b * sin
        out[..., pairs:rot] = a * sin + b * cos
        return out

    margins = []

    def plain_routed(tokens):
        w = {k: np.asarray(v, dtype=np.float64) for k, v in pw.items()}
        T, positions = len(tokens), np.arange(len(tokens))
        nq, nkv, d, eps = pc["num_attention_heads"], pc["num_key_value_heads"], pc["head_dim"], pc["rms_norm_eps"]
        h = plain_model.embedding(w["model.embed_tokens.weight"], tokens)
        for layer in range(pc["num_hidden_layers"]):
            pre = f"model.layers.{layer}."
            x = plain_model.rms_norm(h, w[pre + "input_layernorm.weight"], eps)
            q = plain_model.linear(x, w[pre + "self_attn.q_proj.weight"]).reshape(T, nq, d)
            k = plain_model.linear(x, w[pre + "self_attn.k_proj.weight"]).reshape(T, nkv, d)
            v = plain_model.linear(x, w[pre + "self_attn.v_proj.weight"]).reshape(T, nkv, d)
            q = toy_rope(plain_model.rms_norm(q, w[pre + "self_attn.q_norm.weight"], eps), positions)
            k = toy_rope(plain_model.rms_norm(k, w[pre + "self_attn.k_norm.weight"], eps), positions)
            h = h + plain_model.linear(plain_model.attention(q, k, v).reshape(T, nq * d), w[pre + "self_attn.o_proj.weight"])
            x = plain_model.rms_norm(h, w[pre + "post_attention_layernorm.weight"], eps)
            if layer == 0:
                logits = x @ w[pre + "moe.router.weight"].T
                srt = np.sort(logits, axis=-1)
                margins.append(float((srt[:, -1] - srt[:, -2]).min()))
                y = np.zeros_like(h)
                for t in range(T):
                    e = int(np.argmax(logits[t]))
                    p = plain_model.softmax(logits[t])[e]
                    hid = np.maximum(w[pre + f"moe.experts.{e}.in.weight"] @ x[t], 0.0)
                    y[t] = p * (w[pre + f"moe.experts.{e}.out.weight"] @ hid)
                h = h + y
            else:
                h = h + plain_model.swiglu(x, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"],
                                           w[pre + "mlp.down_proj.weight"])
        x = plain_model.rms_norm(h, w["model.norm.weight"], eps)
        return plain_model.linear(x, w["lm_head.weight"])

    reqs = {"a": random_tokens(4, 45, cfg.vocab_size), "b": random_tokens(5, 19, cfg.vocab_size)}
    want = {k: plain_routed(v) for k, v in reqs.items()}
    assert min(margins) > 1e-4, "a router decision of this seed is too close to call; pick another seed"
    runner = build_runner(folder, dtype="float32", device="cuda:0", page_size=8, num_pages=32, max_requests=2,
                          max_tokens_per_request=128)
    runner.open("a"); runner.open("b")
    plan = [[("a", 0, 17), ("b", 0, 2)], [("a", 17, 18), ("b", 2, 19)], [("a", 18, 45)]]
    for step in plan:
        logits = runner.step([Segment(r, reqs[r][a:b], list(range(b - a))) for r, a, b in step]).cpu().double().numpy()
        ref = np.concatenate([want[r][a:b] for r, a, b in step])
        assert np.abs(logits - ref).max() <= 2e-5 * np.abs(ref).max()
    # the same model in bfloat16 steps too (routing may differ there, so only the shape and finiteness are checked)
    runner16 = build_runner(folder, dtype="bfloat16", device="cuda:0", page_size=8, num_pages=32, max_requests=2,
                            max_tokens_per_request=128)
    runner16.open("a")
    out = runner16.step([Segment("a", reqs["a"][:20], [19])])
    out = runner16.step([Segment("a", reqs["a"][20:21], [0])])
    assert out.shape == (1, cfg.vocab_size) and bool(torch.isfinite(out).all())
    runner16.check_device_errors()


def test_layer_order_as_data_repeat_and_shared_cache(model_folders, tmp_path):
    """The order in which layers run is a list: here layer 0 runs twice (with a cache of its own each
    time) and a last layer without key/value projections reads the cache that layer 1 filled."""
    dev = need_gpu()
    from pulse_infer_b200.config import Qwen3Config, register_architecture
    from pulse_infer_b200.engine import Segment, build_runner
    from pulse_infer_b200.models.qwen3 import build_qwen3_spec
    from pulse_infer_b200.models.spec import ScheduleEntry
    from pulse_infer_b200.weights import write_random_model

    @dataclasses.dataclass(frozen=True)
    class LoopConfig(Qwen3Config):
        pass

    def build_loop_spec(config):
        spec = build_qwen3_spec(config)
        layers = list(spec.layers)
        last = len(layers) - 1
        reader = dataclasses.replace(layers[last].mixer, params={**layers[last].mixer.params, "writes_cache": False})
        layers[last] = dataclasses.replace(layers[last], mixer=reader)
        order = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(last, 1))
        return dataclasses.replace(spec, layers=tuple(layers), order=order)

    register_architecture("LoopForCausalLM", LoopConfig, build_loop_spec, replace=True)
    base = CONFIGS["B"]
    cfg = LoopConfig(**{**{f.name: getattr(base, f.name) for f in dataclasses.fields(base)},
                        "architecture": "LoopForCausalLM"})
    folder = write_random_model(cfg, 9, str(tmp_path / "loop"), dtype="bfloat16")
    pc, pw = load_plain(folder)
    assert "model.layers.2.self_attn.k_proj.weight" not in pw
    toks = random_tokens(4, 45, cfg.vocab_size)
    want = plain_model.forward(pc, pw, toks, order=[(0, 0), (1, 1), (0, 2), (2, 1)])
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 2e-2)):
        runner = build_runner(folder, dtype=dtype, device="cuda:0", page_size=16, num_pages=16, max_requests=2,
                              max_tokens_per_request=64)
        runner.open("a")
        got = [runner.step([Segment("a", toks[a:b], list(range(b - a)))]) for a, b in ((0, 19), (19, 21), (21, 44), (44, 45))]
        got = torch.cat(got).cpu().double().numpy()
        assert np.abs(got - want).max() <= tol * np.abs(want).max()
