"""The scheduler's decisions and the generation loop, on the CPU with a stand-in model.

The stand-in model keeps every request's token history and checks that each step brings exactly the
next tokens at the right positions; its "logits" are a one-hot of a hash of the history, so outputs are
a deterministic function of the tokens fed - any scheduling mistake (wrong portion, lost token after a
preemption) changes them."""
import numpy as np
import pytest
import torch

from pulse_infer_b200.cache import CacheManager
from pulse_infer_b200.engine.engine import ContinuousBatchEngine
from pulse_infer_b200.engine.request import InferenceRequest, RequestState
from pulse_infer_b200.engine.scheduler import ContinuousBatchScheduler
from pulse_infer_b200.engine.step import ModelRunner
from pulse_infer_b200.parts.base import CacheSpec
from pulse_infer_b200.parts.model import Runtime
from pulse_infer_b200.sampling import SamplingParams

VOCAB = 97


class _Spec:
    vocab_size = VOCAB
    max_position = 4096


class StandInModel:
    spec = _Spec()

    def __init__(self):
        self.history = {}
        self.steps = []           # per step: [(request id, start, number of tokens)]

    def forward(self, ctx):
        rows, record = [], []
        for s in ctx.segments:
            if s.start == 0:
                self.history[s.request_id] = []
            h = self.history[s.request_id]
            assert s.start == len(h), f"request {s.request_id}: step starts at {s.start}, history has {len(h)}"
            record.append((s.request_id, s.start, len(s.tokens)))
            for j, t in enumerate(s.tokens):
                h.append(t)
                if j in s.want:
                    nxt = (sum((i + 1) * v for i, v in enumerate(h)) * 31 + len(h)) % VOCAB
                    row = torch.zeros(VOCAB)
                    row[nxt] = 1.0
                    rows.append(row)
        self.steps.append(record)
        return torch.stack(rows) if rows else torch.zeros(0, VOCAB)


class ArgmaxSampler:
    def sample(self, logits, params, draw_index, history=None):
        return logits.argmax(-1).tolist()


def make_engine(num_pages=64, page_size=4, max_batch_size=4, chunk_size=8, max_tokens_per_step=None, eos=(),
                slots=8, per_request=256):
    cache = CacheManager([CacheSpec(1, 16, None)], [None], page_size, num_pages, slots, per_request, allocate_pools=False)
    model = StandInModel()
    runner = ModelRunner(model, cache, Runtime(torch.device("cpu"), "float32"))
    engine = ContinuousBatchEngine(runner, ArgmaxSampler(), eos, max_batch_size=max_batch_size, chunk_size=chunk_size,
                                   max_tokens_per_step=max_tokens_per_step)
    return engine, model, cache


def expected_output(prompt, max_new, eos=()):
    h, out = list(prompt), []
    for _ in range(max_new):
        nxt = (sum((i + 1) * v for i, v in enumerate(h)) * 31 + len(h)) % VOCAB
        out.append(nxt); h.append(nxt)
        if nxt in eos:
            break
    return out


def test_request_state_machine_and_chunks():
    """Prompt portions, then single tokens, then EOS (tests/scheduler/test_continuous_batch_scheduler.cpp:10-40)."""
    r = InferenceRequest(0, [5, 6, 7, 8, 9], max_new_tokens=3)
    assert r.state == RequestState.WAITING and r.is_prefill() and r.get_next_chunk_size(2) == 2
    assert r.get_next_chunk_tokens(2) == [5, 6]
    r.start_running(); r.add_computed_tokens(2)
    assert r.get_next_chunk_tokens(8) == [7, 8, 9]
    r.add_computed_tokens(3)
    assert not r.has_pending_input() and r.can_generate_more()
    assert r.add_sampled_token(11, [42]) is True
    assert not r.is_prefill() and r.get_next_chunk_tokens(8) == [11] and r.total_input_tokens() == 6
    r.add_computed_tokens(1)
    with pytest.raises(ValueError):
        r.add_computed_tokens(1)
    assert r.add_sampled_token(42, [42]) is False and r.is_finished() and r.finish_reason == "eos"
    assert r.generated_tokens == [11, 42]            # the EOS token stays in the output
    r2 = InferenceRequest(1, [1], max_new_tokens=2)
    r2.add_sampled_token(3, []); assert r2.add_sampled_token(4, []) is False and r2.finish_reason == "length"
    # after a preemption everything is fed again, and nothing is sampled before the last known token is in
    r3 = InferenceRequest(2, [1, 2, 3], max_new_tokens=5, generated_tokens=[9, 8])
    r3.num_computed_tokens = 4
    r3.preempt()
    assert r3.state == RequestState.WAITING and r3.pending_tokens() == 5 and r3.is_prefill()
    assert r3.get_next_chunk_tokens(4) == [1, 2, 3, 9]


def test_one_request_prefill_decode_eos():
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    want = expected_output(prompt, 6)
    eos = (want[3],)
    engine, model, cache = make_engine(chunk_size=4, eos=eos)
    rid = engine.add_request(prompt, 6)
    engine.run_until_complete()
    assert engine.get_result(rid) == expected_output(prompt, 6, eos) == want[:4]
    assert engine.get_request(rid).finish_reason == "eos"
    assert [s[0][2] for s in model.steps] == [4, 4, 3, 1, 1, 1]         # portions, then one token a step
    assert cache.free_pages() == [64] and cache.num_free_slots == 8


def test_slot_passes_to_the_next_request_when_one_finishes():
    """tests/scheduler/test_continuous_batch_scheduler.cpp:42-66."""
    engine, model, cache = make_engine(max_batch_size=2, chunk_size=16)
    ids = [engine.add_request([i + 1, i + 2, i + 3], n) for i, n in enumerate((1, 4, 2))]
    engine.step()
    st = engine.get_stats()
    assert (st.num_running, st.num_waiting, st.num_finished) == (1, 1, 1)    # request 0 sampled its one token
    engine.step()
    assert {r for r, _, _ in model.steps[1]} == {ids[1], ids[2]}
    engine.run_until_complete()
    for i, n in enumerate((1, 4, 2)):
        assert engine.get_result(ids[i]) == expected_output([i + 1, i + 2, i + 3], n)
    st = engine.get_stats()
    assert st.num_finished == 3 and st.total_requests == 3 and st.num_running == 0


def test_token_budget_decodes_first_then_cuts_portions():
    engine, model, _ = make_engine(max_batch_size=3, chunk_size=100, max_tokens_per_step=10)
    a = engine.add_request(list(range(1, 5)), 20)          # 4 tokens: decoding from the second step on
    engine.step()
    b = engine.add_request(list(range(1, 31)), 2)          # 30 tokens
    c = engine.add_request(list(range(1, 8)), 2)           # 7 tokens
    engine.step()
    assert model.steps[1] == [(a, 4, 1), (b, 0, 9)]        # the decode token first, the rest of the budget to b
    engine.step()
    assert model.steps[2] == [(a, 5, 1), (b, 9, 9)]
    engine.step(); engine.step()
    assert model.steps[4] == [(a, 7, 1), (b, 27, 3), (c, 0, 6)]      # b's tail, then c admitted with what is left
    assert all(sum(n for _, _, n in s) <= 10 for s in model.steps)
    engine.run_until_complete()
    assert engine.get_result(b) == expected_output(list(range(1, 31)), 2)
    assert engine.get_result(c) == expected_output(list(range(1, 8)), 2)


def test_admission_waits_for_pages():
    # 6 pages of 4 tokens; a request of 14 + 6 tokens needs 5 pages in the end
    engine, model, cache = make_engine(num_pages=6, page_size=4, max_batch_size=2, chunk_size=16)
    a = engine.add_request(list(range(1, 15)), 3)
    b = engine.add_request(list(range(2, 16)), 3)
    engine.step()
    assert [r for r, _, _ in model.steps[0]] == [a]         # b's first portion (4 pages) does not fit beside a's 4
    assert engine.get_stats().num_waiting == 1
    engine.run_until_complete()
    assert engine.get_result(a) == expected_output(list(range(1, 15)), 3)
    assert engine.get_result(b) == expected_output(list(range(2, 16)), 3)
    assert engine.get_stats().num_preemptions == 0 and cache.free_pages() == [6]


def test_preemption_when_a_decode_needs_a_page():
    # both fit at first (2 + 2 pages of 5); when a needs a third page none is free: b, the newest, gives way
    engine, model, cache = make_engine(num_pages=5, page_size=4, max_batch_size=2, chunk_size=16)
    a = engine.add_request(list(range(1, 8)), 12)            # 7 tokens -> 19
    b = engine.add_request(list(range(3, 10)), 12)
    seen_preempted = []
    while engine.has_work():
        engine.step()
        seen_preempted += [r.request_id for r in engine.last_batch.preempted]
        cache.check_invariants()
    assert seen_preempted and set(seen_preempted) == {b}
    assert engine.get_request(b).num_preemptions >= 1 and engine.get_request(a).num_preemptions == 0
    # the outcome is what it would have been without the shortage
    assert engine.get_result(a) == expected_output(list(range(1, 8)), 12)
    assert engine.get_result(b) == expected_output(list(range(3, 10)), 12)
    # b came back to the front of the queue and recomputed prompt + generated tokens from position 0
    restarts = [s for step in model.steps for s in step if s[0] == b and s[1] == 0]
    assert len(restarts) == 1 + engine.get_request(b).num_preemptions
    assert cache.free_pages() == [5]


def test_request_that_can_never_fit_is_finished_not_stalled():
    engine, _, cache = make_engine(num_pages=3, page_size=4, max_batch_size=2, chunk_size=64)
    big = engine.add_request(list(range(1, 11)), 20)         # would reach 30 tokens, the pool holds 12
    small = engine.add_request([1, 2, 3], 2)
    engine.run_until_complete()
    assert engine.get_request(big).finish_reason == "out_of_pages"
    assert len(engine.get_result(big)) < 20
    assert engine.get_result(small) == expected_output([1, 2, 3], 2)
    assert cache.free_pages() == [3] and cache.num_free_slots == 8


def test_zero_new_tokens_finishes_after_the_prompt():
    engine, model, cache = make_engine()
    rid = engine.add_request([1, 2, 3, 4, 5], 0)
    engine.run_until_complete()
    assert engine.get_result(rid) == [] and engine.get_request(rid).is_finished() and cache.free_pages() == [64]


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_match_an_unconstrained_run(seed):
    rng = np.random.RandomState(seed)
    reqs = [([int(t) for t in rng.randint(1, VOCAB, size=rng.randint(1, 40))], int(rng.randint(1, 25)))
            for _ in range(12)]
    engine, model, cache = make_engine(num_pages=int(rng.randint(17, 30)), page_size=4, max_batch_size=4,
                                       chunk_size=int(rng.choice([3, 8, 32])), max_tokens_per_step=int(rng.choice([6, 16, 64])))
    ids = []
    pending = list(reqs)
    while pending or engine.has_work():
        while pending and rng.rand() < 0.5:
            p, m = pending.pop(0)
            ids.append(engine.add_request(p, m))
        if engine.has_work():
            engine.step()
            cache.check_invariants()
            assert engine.last_batch.num_tokens <= engine.scheduler.max_tokens_per_step
    for rid, (p, m) in zip(ids, reqs):
        assert engine.get_result(rid) == expected_output(p, m), f"request {rid}"
    assert cache.free_pages() == [cache.num_pages] and cache.num_free_slots == 8


# ---- lookahead: a step of single tokens stays in flight, its ids are read a step later -----------------------------
class LookaheadRunner(ModelRunner):
    """The stand-in's version of a captured step that takes its input ids from the device: the ids of the step
    before arrive as a tensor and replace the places kept in the segments."""

    def takes_device_tokens(self, segments):
        return all(len(s.tokens) == 1 and list(s.want) == [0] for s in segments)

    def step(self, segments, tokens_from=None):
        if tokens_from is not None:
            assert self.takes_device_tokens(segments) and tokens_from.numel() == len(segments)
            for s, t in zip(segments, tokens_from.tolist()):
                s.tokens = [int(t)]
        return super().step(segments)


class DeviceArgmaxSampler(ArgmaxSampler):
    reads = 0

    def sample_device(self, logits, params, draw_index, history=None):
        return logits.argmax(-1).to(torch.int32)


def make_lookahead_engine(num_pages=64, page_size=4, max_batch_size=4, chunk_size=8, max_tokens_per_step=None, eos=()):
    cache = CacheManager([CacheSpec(1, 16, None)], [None], page_size, num_pages, 8, 256, allocate_pools=False)
    model = StandInModel()
    runner = LookaheadRunner(model, cache, Runtime(torch.device("cpu"), "float32"))
    engine = ContinuousBatchEngine(runner, DeviceArgmaxSampler(), eos, max_batch_size=max_batch_size, chunk_size=chunk_size,
                                   max_tokens_per_step=max_tokens_per_step, lookahead=True)
    return engine, model, cache


def test_lookahead_keeps_a_decode_step_in_flight_and_returns_its_tokens_a_step_later():
    prompt = [3, 1, 4, 1, 5]
    want = expected_output(prompt, 5)
    engine, model, cache = make_lookahead_engine(chunk_size=16)
    rid = engine.add_request(prompt, 5)
    assert engine.step() == [(rid, want[0])]          # the prompt step samples; it is not a step of single tokens
    assert engine.step() == []                        # first decode step: launched, its token stays on the device
    assert engine.get_result(rid) == want[:1] and engine.get_request(rid).unresolved == 1
    assert engine.step() == [(rid, want[1])]          # second decode step launched on the device token; first one read
    assert [s for s in model.steps[-1]] == [(rid, 6, 1)] and model.history[rid][-1] == want[1]
    outs = []
    while engine.has_work():
        outs += engine.step()
    assert [t for _, t in outs] == want[2:] and engine.get_result(rid) == want
    assert engine.get_request(rid).finish_reason == "length" and engine.get_request(rid).unresolved == 0
    assert cache.free_pages() == [64]
    # the last allowed token is not fed back: 5 prompt tokens + 4 fed samples
    assert len(model.history[rid]) == 9


def test_lookahead_eos_read_late_drops_the_extra_token():
    prompt = [2, 7, 1, 8, 2, 8]
    free_run = expected_output(prompt, 12)
    eos = (free_run[4],)
    want = expected_output(prompt, 12, eos)
    assert len(want) == 5
    engine, model, cache = make_lookahead_engine(chunk_size=16, eos=eos)
    rid = engine.add_request(prompt, 12)
    engine.run_until_complete()
    assert engine.get_result(rid) == want and engine.get_request(rid).finish_reason == "eos"
    assert engine.get_request(rid).generated_tokens == want and cache.free_pages() == [64]
    assert len(model.history[rid]) == len(prompt) + len(want)        # one step ran past the end; its token is dropped


def test_lookahead_request_preempted_while_its_last_token_is_in_flight():
    """The newest request is preempted in the very plan that runs while the id that ends it (its length limit) is
    still on the device: it must finish from the waiting queue, holding no slot, and nothing may be freed twice."""
    hit = 0
    for pages in range(4, 12):
        for new_b in (2, 3, 4):
            engine, model, cache = make_lookahead_engine(num_pages=pages, page_size=4, chunk_size=16, max_batch_size=2)
            a = engine.add_request([1, 2, 3, 4, 5, 6, 7], 14)
            b = engine.add_request([9, 8, 7, 6, 5], new_b)
            while engine.has_work():
                engine.step()
                cache.check_invariants()
            rb = engine.get_request(b)
            hit += int(rb.num_preemptions > 0 and rb.finish_reason == "length" and rb.num_computed_tokens == 0)
            for rid, (p, m) in ((a, ([1, 2, 3, 4, 5, 6, 7], 14)), (b, ([9, 8, 7, 6, 5], new_b))):
                r = engine.get_request(rid)
                want = expected_output(p, m)
                got = engine.get_result(rid)
                assert got == (want if r.finish_reason != "out_of_pages" else want[:len(got)]), (pages, new_b, rid)
            assert not engine.scheduler.waiting_queue and not engine.scheduler.running_requests
            assert cache.free_pages() == [pages] and cache.num_free_slots == 8
    assert hit > 0, "no case preempted a request that then ended by its length limit"


@pytest.mark.parametrize("seed", range(40))
def test_lookahead_random_workloads_match_an_unconstrained_run(seed):
    """Admissions, portions, preemptions, EOS and length limits while steps are in flight: the results are those of
    the plain loop.  Small pools (from 11 pages) preempt requests whose sampled id has not been read yet."""
    rng = np.random.RandomState(100 + seed)
    reqs = [([int(t) for t in rng.randint(1, VOCAB, size=rng.randint(1, 40))], int(rng.randint(1, 25)))
            for _ in range(12)]
    eos = tuple(int(t) for t in rng.randint(1, VOCAB, size=3)) if seed % 2 else ()
    engine, model, cache = make_lookahead_engine(num_pages=int(rng.randint(11, 30)), page_size=4, max_batch_size=4,
                                                 chunk_size=int(rng.choice([3, 8, 32])),
                                                 max_tokens_per_step=int(rng.choice([6, 16, 64])), eos=eos)
    ids, seen = [], {}
    pending = list(reqs)
    while pending or engine.has_work():
        while pending and rng.rand() < 0.5:
            p, m = pending.pop(0)
            ids.append(engine.add_request(p, m))
        if engine.has_work():
            for rid, tok in engine.step():
                seen.setdefault(rid, []).append(tok)
            cache.check_invariants()
    for rid, (p, m) in zip(ids, reqs):
        want, got = expected_output(p, m, eos), engine.get_result(rid)
        if engine.get_request(rid).finish_reason == "out_of_pages":      # longer than the whole pool: cut short
            want = want[:len(got)]
        assert got == want, f"request {rid}"
        assert seen.get(rid, []) == engine.get_result(rid)             # every token was handed out once, in order
        assert engine.get_request(rid).unresolved == 0
    assert cache.free_pages() == [cache.num_pages] and cache.num_free_slots == 8


def test_small_budget_rotates_over_decoding_requests_and_stats_count_what_ran():
    """Four decoding requests under a budget of two tokens a step: nobody starves, and the counters equal the tokens
    that the model really saw."""
    engine, model, cache = make_engine(max_batch_size=4, chunk_size=8, max_tokens_per_step=2)
    prompts = [[1 + i, 2, 3] for i in range(4)]
    ids = [engine.add_request(p, 6) for p in prompts]
    served = {rid: 0 for rid in ids}
    while engine.has_work():
        engine.step()
        assert engine.last_batch.num_tokens <= 2
        decoding = [r for r in engine.last_batch.requests if r.num_generated() > 1]
        for r in decoding:
            served[r.request_id] += 1
    for rid, p in zip(ids, prompts):
        assert engine.get_result(rid) == expected_output(p, 6)
    st = engine.get_stats()
    ran = sum(n for step in model.steps for _, _, n in step)
    assert st.prefill_tokens + st.decode_tokens == ran
    assert st.prefill_tokens == sum(len(p) for p in prompts) and st.decode_tokens == 4 * 5
    # while all four were decoding, consecutive steps served different pairs
    pairs = [tuple(sorted(r for r, s, n in step)) for step in model.steps if all(n == 1 and s >= 3 for r, s, n in step)]
    assert len(set(pairs[:4])) > 1


def test_preempting_a_request_already_in_the_step_gives_its_token_back():
    """Pages run out while the decode loop plans: a victim that already had its token in this step is taken out, and
    both the step's budget and the counters forget that token."""
    engine, model, cache = make_engine(num_pages=5, page_size=4, max_batch_size=3, chunk_size=16, max_tokens_per_step=3)
    a = engine.add_request([1, 2, 3, 4, 5, 6, 7], 9)      # 2 pages, a third at length 9
    b = engine.add_request([9, 8, 7, 6, 5, 4, 3], 9)
    engine.run_until_complete()
    for rid, p in ((a, [1, 2, 3, 4, 5, 6, 7]), (b, [9, 8, 7, 6, 5, 4, 3])):
        r = engine.get_request(rid)
        want = expected_output(p, 9)
        got = engine.get_result(rid)
        assert got == (want if r.finish_reason != "out_of_pages" else want[:len(got)])
    st = engine.get_stats()
    assert st.num_preemptions > 0
    assert st.prefill_tokens + st.decode_tokens == sum(n for step in model.steps for _, _, n in step)
