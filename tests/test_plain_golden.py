"""The plain implementation against the golden logits of the reference's own CPU model code."""
import os

import numpy as np
import pytest

import plain_model
from helpers import load_plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_cpu_model(name, model_folders):
    cfg, w = load_plain(model_folders[name])
    gold = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    checksum = float(sum(np.abs(a).sum() for a in w.values()))
    if "lm_head.weight" not in w:    # the golden run had to add a copy of the embedding
        checksum += float(np.abs(w["model.embed_tokens.weight"]).sum())
    assert checksum == pytest.approx(float(gold["weight_checksum"][0]), rel=1e-12), "random weights changed"
    i = 0
    while f"tokens_{i}" in gold:
        tokens = [int(t) for t in gold[f"tokens_{i}"]]
        want = gold[f"logits_{i}"]
        got64 = plain_model.forward(cfg, w, tokens, dtype=np.float64)
        got32 = plain_model.forward(cfg, w, tokens, dtype=np.float32)
        scale = np.abs(want).max()
        # the reference sums products and attention in float32: agreement to float32 rounding
        assert np.abs(got64 - want).max() <= 2e-5 * scale + 1e-6
        assert np.abs(got32 - want).max() <= 4e-5 * scale + 1e-6
        assert (got64.argmax(-1) == want.argmax(-1)).all()
        i += 1
    assert i >= 2


def test_plain_parts_small_cases():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain_model.rms_norm(x, np.array([1.0, 2.0]), 0.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])
    # rotation by pos=1 with theta=1: angle 1 for every pair
    v = np.array([[[1.0, 0.0, 0.0, 1.0]]])
    r = plain_model.rope(v, [1], 1.0, 4, "adjacent")
    assert np.allclose(r[0, 0], [np.cos(1), np.sin(1), -np.sin(1), np.cos(1)])
    r = plain_model.rope(v, [1], 1.0, 4, "half")   # pairs (0,2) and (1,3)
    assert np.allclose(r[0, 0], [np.cos(1), -np.sin(1), np.sin(1), np.cos(1)])
    # one key: attention returns its value
    q = np.ones((1, 2, 4)); k = np.ones((1, 1, 4)); vv = np.arange(4.0).reshape(1, 1, 4)
    assert np.allclose(plain_model.attention(q, k, vv)[0, 1], np.arange(4.0))
    # window of 1: every query sees only itself
    q = np.random.RandomState(0).randn(5, 2, 4); k = np.random.RandomState(1).randn(5, 1, 4)
    vv = np.random.RandomState(2).randn(5, 1, 4)
    out = plain_model.attention(q, k, vv, window=1)
    assert np.allclose(out[:, 0], vv[:, 0])
    assert plain_model.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 1


def test_plain_sampler_kept_set_and_draw():
    logits = np.array([0.0, 2.0, 1.0, 2.0, -1.0, 0.5])
    order, weights = plain_model.kept_set(logits, 1.0, 3, 0.0)
    assert order == [1, 3, 2]
    order, _ = plain_model.kept_set(logits, 1.0, 0, 0.5)
    assert order == [1, 3]          # ties of the last kept logit stay
    picks = {plain_model.sample(logits, 0.7, 3, 0.9, seed=11, counter=c) for c in range(200)}
    assert picks <= {1, 2, 3} and len(picks) >= 2
    assert plain_model.sample(logits, 0.0, 0, 0.0, 1, 1) == 1
    u = [plain_model.uniform_from(5, c) for c in range(1000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and 0.4 < np.mean(u) < 0.6
