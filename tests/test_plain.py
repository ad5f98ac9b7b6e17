"""The plain implementation itself: against the outputs of the reference's own model code stored
under tests/golden/ (made by tests/golden/make_golden.py), and its extensions (window, schedule,
sampler) against first principles."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests import tiny

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_outputs(tmp_path, name):
    g = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    cfg, w = plain.read_folder(tiny.make_tiny_folder(name, tmp_path))
    for n, v in zip(g["fingerprint_names"], g["fingerprint"]):
        assert float(w[str(n)].double().abs().sum()) == pytest.approx(float(v), rel=1e-12), \
            "the random-weights writer no longer makes the model the stored outputs belong to"
    ids = g["ids"].tolist()
    logits, hidden = plain.forward(cfg, w, ids, return_hidden=True)
    assert np.abs(logits.numpy() - g["logits"]).max() < 1e-5
    assert np.abs(np.stack([h.numpy() for h in hidden]) - g["hidden"]).max() < 1e-5
    if len(g["greedy"]):
        assert plain.greedy(cfg, w, ids[:9], 8) == g["greedy"].tolist()


def test_window_mask_and_prefix_independence(tmp_path):
    cfg, w = plain.read_folder(tiny.make_tiny_folder("W", tmp_path))
    ids = tiny.random_ids(90, cfg["vocab_size"], 3)
    full = plain.forward(cfg, w, ids)
    # causal: logits at position p do not depend on later tokens
    assert torch.allclose(plain.forward(cfg, w, ids[:50]), full[:50], atol=1e-5)
    # the window matters: without it the late logits differ
    nowin = plain.forward({**cfg, "use_sliding_window": False}, w, ids)
    assert torch.allclose(nowin[:24], full[:24], atol=1e-5) and not torch.allclose(nowin[60:], full[60:], atol=1e-3)
    q = torch.randn(40, 2, 8)
    k, v = torch.randn(40, 1, 8), torch.randn(40, 1, 8)
    a = plain.attention(q, k, v, 0.3, window=5)
    # last row by hand: keys 35..39 only
    s = (q[39, 0] @ k[35:, 0].T) * 0.3
    want = torch.softmax(s, -1) @ v[35:, 0]
    assert torch.allclose(a[39, :8], want, atol=1e-6)


def test_schedule_semantics(tmp_path):
    cfg, w = plain.read_folder(tiny.make_tiny_folder("B", tmp_path))
    ids = tiny.random_ids(30, cfg["vocab_size"], 4)
    base = plain.forward(cfg, w, ids)
    assert torch.equal(plain.forward(cfg, w, ids, schedule=[(0, None), (1, None), (2, None)]), base)
    twice = plain.forward(cfg, w, ids, schedule=[(0, None), (1, None), (1, None), (2, None)])
    shared = plain.forward(cfg, w, ids, schedule=[(0, None), (1, None), (2, 1)])
    assert not torch.allclose(twice, base, atol=1e-3) and not torch.allclose(shared, base, atol=1e-4)


def test_philox_known_answer_and_noise_range():
    assert int(plain._philox_first_word((0, 0, 0, 0), (0, 0))) == 0x6627E8D5
    assert int(plain._philox_first_word((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2)) == 0x408F276D
    e = plain.exponential_noise(7, 3, 100000)
    assert e.min() > 0 and np.isfinite(e).all() and abs(e.mean() - 1.0) < 0.02
    assert not np.array_equal(e[:100], plain.exponential_noise(8, 3, 100))


def test_filtered_probs_and_penalties():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 0.0])
    p = plain.filtered_probs(logits, 1.0, 2, 1.0)
    assert (p > 0).tolist() == [True, True, False, False, False] and float(p.sum()) == pytest.approx(1.0)
    p = plain.filtered_probs(logits, 1.0, -1, 0.6)              # 0.57 first, then 0.21: the second is kept too
    assert (p > 0).tolist() == [True, True, False, False, False]
    p = plain.filtered_probs(logits, 1.0, -1, 0.5)
    assert (p > 0).tolist() == [True, False, False, False, False]
    out = plain.penalize(torch.tensor([2.0, -2.0, 1.0, 1.0]), [0], [1, 1, 2], 2.0, 0.5, 0.25)
    assert out.tolist() == [1.0, -4.0 - 0.5 - 0.5, 0.5 - 0.25 - 0.5, 1.0]
    tok, scores = plain.sample(logits, 0.0, -1, 1.0, 1, 0)
    assert tok == 0 and scores is None
