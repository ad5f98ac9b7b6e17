"""The sampling kernels against the plain sampler (tests/plain_qwen2.py), after the reference's
tests/unit/test_sampler.py:34-118."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from turingserve_b200.sampling import Sampler, SampleRow, SamplingParams

pytestmark = pytest.mark.gpu


def _rows(params, seeds, drawn=None, prompts=None, outputs=None, stop=()):
    n = len(params)
    return [SampleRow(params[i], seeds[i], 0 if drawn is None else drawn[i],
                      [] if prompts is None else prompts[i], [] if outputs is None else outputs[i], stop)
            for i in range(n)]


def _agree(token, scores):
    """The engine's token is the plain argmax, or ties with it within float rounding."""
    return token == int(scores.argmax()) or float(scores[token]) >= float(scores.max()) * (1 - 1e-5)


def test_greedy_is_first_maximum():
    s = Sampler("cuda")
    logits = torch.randn(5, 1000)
    logits[2, 77] = logits[2, 500] = 9.0
    toks, bad = s.sample(logits.cuda(), _rows([SamplingParams(temperature=0.0)] * 5, [0] * 5))
    assert toks.tolist() == logits.argmax(-1).tolist() and toks[2] == 77
    assert not bad.any()


@pytest.mark.parametrize("S,V", [(1, 7), (8, 151936), (3, 4097), (64, 32000), (5, 262147)])
def test_all_greedy_rows_take_the_many_block_path(S, V):
    """A step whose rows are all greedy goes to the kernel that cuts each row into parts; it answers
    as the one-block-per-row kernel does: first index of the maximum (ties across part edges, -inf
    entries), a NaN or +inf anywhere flags the row, and repeated calls leave the counters clean."""
    from turingserve_b200 import kernels
    ops = kernels.ops()
    g = torch.Generator().manual_seed(S * 1000 + V)
    logits = torch.randn(S, V, generator=g)
    parts = ops.lib.ts_sample_greedy_parts(V)
    edge = -(-V // parts)
    if V > 10:
        logits[0, min(edge, V - 1)] = logits[0, min(edge, V - 1) - 1] = logits[0, 3] = 50.0     # a tie across a part edge
        logits[S - 1, : V // 2] = float("-inf")
    dev = logits.cuda()
    s = Sampler("cuda")
    for _ in range(3):
        toks, bad = s.sample(dev, _rows([SamplingParams(temperature=0.0)] * S, [0] * S))
        assert toks.tolist() == logits.argmax(-1).tolist() and not bad.any()
    if V > 10:
        assert toks[0] == 3
    general = torch.empty((2, S), dtype=torch.int32, device="cuda")
    ops.sample(general, dev, torch.zeros((S, 2), device="cuda"), torch.zeros((S, 4), dtype=torch.int64, device="cuda"))
    assert general[0].cpu().tolist() == toks.tolist()
    if S >= 3:
        logits[1, V - 1] = float("inf")
        logits[2, V // 3] = float("nan")
        toks, bad = s.sample(logits.cuda(), _rows([SamplingParams(temperature=0.0)] * S, [0] * S))
        assert bad.tolist() == [False, True, True] + [False] * (S - 3) and toks[1] == 0 and toks[2] == 0
        assert toks[0] == logits[0].argmax()
    # one row with a temperature: the whole step goes to the general kernel, greedy rows unchanged
    mixed = [SamplingParams(temperature=0.0)] * (S - 1) + [SamplingParams(temperature=0.8)]
    logits2 = torch.randn(S, V, generator=g)
    toks2, _ = s.sample(logits2.cuda(), _rows(mixed, list(range(S))))
    assert toks2[: S - 1].tolist() == logits2[: S - 1].argmax(-1).tolist()


@pytest.mark.parametrize("V", [256, 301, 151936])
def test_temperature_matches_plain(V):
    s = Sampler("cuda")
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(6, V, generator=g) * 3
    params = [SamplingParams(temperature=t) for t in (1.0, 0.5, 0.7, 2.0, 0.0, 1.3)]
    seeds = [1, 2, 3, 2 ** 63 + 5, 4, 99]
    drawn = [0, 5, 17, 3, 0, 2 ** 33]
    toks, bad = s.sample(logits.cuda(), _rows(params, seeds, drawn))
    for i in range(6):
        tok, scores = plain.sample(logits[i], params[i].temperature, -1, 1.0, seeds[i], drawn[i])
        assert toks[i] == tok if scores is None else _agree(int(toks[i]), scores), i


@pytest.mark.parametrize("V", [301, 32000])
def test_top_k_top_p_match_plain(V):
    s = Sampler("cuda")
    g = torch.Generator().manual_seed(V + 1)
    logits = torch.randn(8, V, generator=g) * 2
    combos = [(1, 1.0), (5, 1.0), (-1, 0.5), (40, 0.9), (-1, 0.05), (V, 0.999), (3, 0.3), (1000, 0.8)]
    for drawn in range(4):
        params = [SamplingParams(temperature=0.8, top_k=k, top_p=p) for k, p in combos]
        toks, _ = s.sample(logits.cuda(), _rows(params, list(range(10, 18)), [drawn] * 8))
        for i, (k, p) in enumerate(combos):
            probs = plain.filtered_probs(logits[i], 0.8, k, p)
            assert probs[int(toks[i])] > 0, f"row {i}: token outside the kept set (k={k}, p={p})"
            tok, scores = plain.sample(logits[i], 0.8, k, p, 10 + i, drawn)
            assert _agree(int(toks[i]), scores), (i, k, p)
    toks, _ = s.sample(logits.cuda(), _rows([SamplingParams(temperature=1.0, top_k=1)] * 8, [5] * 8))
    assert toks.tolist() == logits.argmax(-1).tolist()      # top_k = 1 is greedy


def test_seeded_stream_independent_of_batch_mates():
    s = Sampler("cuda")
    logits = torch.randn(4, 500)
    p = SamplingParams(temperature=1.0, seed=123)
    alone, _ = s.sample(logits[1:2].cuda(), _rows([p], [123], [7]))
    together, _ = s.sample(logits.cuda(), _rows([SamplingParams(temperature=0.9)] * 1 + [p] + [SamplingParams()] * 2,
                                                [5, 123, 6, 7], [0, 7, 1, 2]))
    assert alone[0] == together[1]
    again, _ = s.sample(logits[1:2].cuda(), _rows([p], [123], [8]))
    # a different stream position gives different noise (equal tokens only by chance; check noise)
    assert not np.array_equal(plain.exponential_noise(123, 7, 500), plain.exponential_noise(123, 8, 500))
    assert again.shape == (1,)


@pytest.mark.parametrize("temperature", [1.0, 0.5])
def test_distribution_chi_square(temperature):
    """20 000 draws from a 4-way distribution (reference tests/unit/test_sampler.py:54-60,79-85)."""
    s = Sampler("cuda")
    base = torch.tensor([1.0, 2.0, 0.5, -1.0])
    n = 20000
    logits = base[None].repeat(n, 1).cuda()
    params = [SamplingParams(temperature=temperature)] * n
    toks, _ = s.sample(logits, _rows(params, list(range(1000, 1000 + n))))
    p = torch.softmax(base / temperature, -1).numpy()
    counts = np.bincount(toks, minlength=4)
    chi2 = float(((counts - n * p) ** 2 / (n * p)).sum())
    assert chi2 < 16.27, (chi2, counts)          # 3 degrees of freedom, p = 0.001
    same, _ = s.sample(logits[:64], _rows(params[:64], [42] * 64, list(range(64))))
    assert len(set(same.tolist())) > 1


def test_bad_row_is_flagged():
    s = Sampler("cuda")
    logits = torch.randn(3, 300)
    logits[1, 17] = float("nan")
    toks, bad = s.sample(logits.cuda(), _rows([SamplingParams(temperature=0.0)] * 3, [0] * 3))
    assert bad.tolist() == [False, True, False]
    assert toks[0] == logits[0].argmax() and toks[2] == logits[2].argmax()


def test_penalties_and_min_tokens_match_plain():
    s = Sampler("cuda")
    V = 400
    logits = torch.randn(3, V) * 2
    prompts = [[1, 2, 3, 3, 50], [], [7, 8]]
    outputs = [[3, 9, 9, 9, 100], [5], []]
    params = [SamplingParams(temperature=0.0, repetition_penalty=1.3, presence_penalty=0.4, frequency_penalty=0.2),
              SamplingParams(temperature=0.0, min_tokens=3, max_tokens=8),
              SamplingParams(temperature=0.0, repetition_penalty=0.8)]
    stop = (int(logits[1].argmax()), 11)
    rows = [SampleRow(params[i], 0, 0, prompts[i], outputs[i], stop) for i in range(3)]
    toks, _ = s.sample(logits.cuda(), rows)
    exp0 = plain.penalize(logits[0], prompts[0], outputs[0], 1.3, 0.4, 0.2)
    exp1 = logits[1].clone()
    exp1[list(stop)] = float("-inf")
    exp2 = plain.penalize(logits[2], prompts[2], outputs[2], 0.8, 0.0, 0.0)
    assert toks.tolist() == [int(exp0.argmax()), int(exp1.argmax()), int(exp2.argmax())]
    # and the edited logits themselves
    from turingserve_b200 import kernels
    edited = logits.clone().cuda()
    s._edit_logits(kernels.ops(), edited, rows)
    torch.testing.assert_close(edited[0].cpu(), exp0, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(edited[2].cpu(), exp2, atol=1e-6, rtol=1e-6)
    assert torch.isinf(edited[1, list(stop)]).all()


def test_status_words_travel_with_the_tokens():
    """The draw copies the status words of the kernels with bounded waits out beside the tokens: all
    zero after healthy kernels; a word that a kernel set (here: set through the test hook, in stream
    order, as a block that gave up would) arrives with the very next draw, greedy or not."""
    from turingserve_b200 import kernels
    kernels.use(None)
    ops = kernels.ops()
    s = Sampler("cuda")
    logits = torch.randn(3, 1000)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for params in ([SamplingParams(temperature=0.0)] * 3, [SamplingParams(temperature=0.7)] * 3):
            p = s.launch(logits.cuda(), _rows(params, [0] * 3))
            s.finish(p)
            assert list(p.status()) == [0, 0, 0, 0]
            assert ops.lib.ts_poke_status(2, 7, stream) == 0
            p = s.launch(logits.cuda(), _rows(params, [0] * 3))
            toks, bad = s.finish(p)
            assert list(p.status()) == [0, 0, 7, 0] and not bad.any()
            assert ops.lib.ts_clear_status(stream) == 0
        p = s.launch(logits.cuda(), _rows([SamplingParams(temperature=0.0)] * 3, [0] * 3))
        s.finish(p)
        assert list(p.status()) == [0, 0, 0, 0]
    finally:
        ops.lib.ts_clear_status(stream)
