"""The scheduler's decisions, with a model-free runner (after the reference's
tests/unit/test_scheduler.py:13-120)."""

from __future__ import annotations

import random

import pytest

from tests.fakes import expected_output, make_fake_engine
from turingserve_b200.sampling import SamplingParams


def greedy(n, **kw):
    return SamplingParams(temperature=0.0, max_tokens=n, **kw)


def check_invariants(eng, plan_items=None):
    eng.cache.check()
    s = eng.scheduler
    assert len(s.running) <= s.max_num_seqs
    assert all(r.cache is not None for r in s.running) and all(r.cache is None for r in s.waiting)


def run(eng, reqs, check=True):
    for rid, (p, sp) in reqs.items():
        eng.add_request(rid, p, sp)
    out = {rid: [] for rid in reqs}
    reasons = {}
    steps = 0
    while eng.has_unfinished():
        for o in eng.step():
            out[o.request_id] += o.delta_token_ids
            if o.finished:
                reasons[o.request_id] = o.finish_reason
        if check:
            check_invariants(eng)
        steps += 1
        assert steps < 100000
    return out, reasons, steps


def test_chunked_prefill_takes_ceil_steps_and_samples_once():
    eng = make_fake_engine(num_pages=128, budget=64)
    prompt = list(range(1000))
    out, reasons, steps = run(eng, {"a": (prompt, greedy(1))})
    assert steps == 16                                             # ceil(1000 / 64)
    sizes = [n for st in eng.runner.steps for _, n in st]
    assert sizes == [64] * 15 + [40]
    assert out["a"] == expected_output(prompt, 1) and reasons["a"] == "length"


def test_decodes_first_and_budget_respected():
    eng = make_fake_engine(num_pages=256, budget=48, max_seqs=8)
    reqs = {f"r{i}": (list(range(i, i + 30 + 17 * i)), greedy(12)) for i in range(5)}
    for rid, (p, sp) in reqs.items():
        eng.add_request(rid, p, sp)
    while eng.has_unfinished():
        plan = eng.scheduler.schedule()
        assert plan.num_tokens <= 48
        kinds = [it.num_tokens == 1 and it.request.num_uncomputed == 1 for it in plan.items]
        assert kinds == sorted(kinds, reverse=True), "decodes come first"
        assert plan.num_decode == sum(kinds)
        eng._run(plan)
        eng.step_count += 1
        check_invariants(eng)


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_match_solo_runs_and_free_everything(seed):
    rng = random.Random(seed)
    eng = make_fake_engine(num_pages=rng.choice([24, 40, 200]), budget=rng.choice([16, 48, 200]),
                           max_seqs=rng.choice([2, 4, 8]), window=rng.choice([None, 40]))
    reqs = {}
    for i in range(12):
        p = [rng.randrange(1000) for _ in range(rng.choice([1, 5, 17, 60, 130]))]
        reqs[f"r{i}"] = (p, greedy(rng.choice([1, 4, 20])))
    out, reasons, _ = run(eng, reqs)
    for rid, (p, sp) in reqs.items():
        if reasons[rid] == "error":
            assert len(p) + sp.max_tokens > (eng.cache.num_pages - 1) * 16 - 16
            continue
        assert out[rid] == expected_output(p, sp.max_tokens), rid
    assert not eng.cache.live and eng.cache.min_free() == eng.cache.num_pages - 1


def test_pages_run_out_newest_is_preempted_and_outputs_do_not_change():
    reqs = {f"r{i}": (list(range(10 * i, 10 * i + 40)), greedy(60)) for i in range(4)}
    big, _, _ = run(make_fake_engine(num_pages=400), dict(reqs))
    small_eng = make_fake_engine(num_pages=16)                      # 15 pages = 240 tokens < 4 x 100
    small, reasons, _ = run(small_eng, dict(reqs))
    assert small == big and set(reasons.values()) == {"length"}
    assert small_eng.scheduler.num_preemptions > 0
    # the victim was the newest running request, and it went back to the FRONT of the queue
    eng = make_fake_engine(num_pages=10, budget=256)                # 9 pages
    for i in range(2):
        eng.add_request(f"r{i}", list(range(60)), greedy(40))       # 4 pages each at admission, 7 at the end
    for _ in range(200):
        if eng.scheduler.num_preemptions:
            break
        eng.step()
    assert eng.scheduler.num_preemptions == 1
    assert [r.request_id for r in eng.scheduler.waiting] == ["r1"]
    assert [r.request_id for r in eng.scheduler.running] == ["r0"]
    assert eng.requests["r1"].num_computed == 0 and eng.requests["r1"].num_output > 0
    check_invariants(eng)


def test_no_admission_in_a_step_that_preempted_and_watermark():
    eng = make_fake_engine(num_pages=9, budget=256, watermark=0.3)  # keeps 2 pages free at admission
    assert eng.scheduler.watermark_pages == 2
    eng.add_request("a", list(range(16 * 6)), greedy(4))             # 6 pages: fits with 2 left
    eng.add_request("b", list(range(16)), greedy(4))                 # 1 page would leave 1 < watermark
    eng.step()
    assert [r.request_id for r in eng.scheduler.running] == ["a"]
    assert [r.request_id for r in eng.scheduler.waiting] == ["b"]


def test_unschedulable_request_errors_others_go_on():
    eng = make_fake_engine(num_pages=5, budget=32)                   # 64 tokens of cache
    out, reasons, _ = run(eng, {"big": (list(range(100)), greedy(4)), "ok": (list(range(10)), greedy(4))})
    assert reasons == {"big": "error", "ok": "length"}
    assert out["ok"] == expected_output(list(range(10)), 4) and out["big"] == []
    assert not eng.cache.live


def test_two_prompts_that_block_each_other_are_untangled():
    """Both running requests are in the middle of their prompts and neither portion fits: the newest
    gives its pages to the other (the reference would wait forever)."""
    from turingserve_b200.engine.request import Status
    eng = make_fake_engine(num_pages=9, budget=48, max_seqs=4)       # 8 pages = 128 tokens
    reqs = {"a": (list(range(100)), greedy(3)), "b": (list(range(5, 105)), greedy(3))}
    for rid, (p, sp) in reqs.items():
        r = eng.add_request(rid, p, sp)
        eng.scheduler.waiting.remove(r)
        r.status = Status.RUNNING
        r.cache = eng.cache.admit(rid)
        eng.runner.step([type("E", (), {"cache": r.cache, "tokens": p[:60], "want": []})()])   # 4 pages each
        eng.scheduler.running.append(r)
    assert eng.cache.min_free() == 0
    plan = eng.scheduler.schedule()
    assert [it.request.request_id for it in plan.items] == ["a"] and plan.items[0].num_tokens == 40
    assert [r.request_id for r in plan.preempted] == ["b"] and eng.scheduler.waiting[0].request_id == "b"
    eng._run(plan)
    out = {"a": [], "b": []}
    reasons = {}
    for _ in range(100):
        for o in eng.step():
            out[o.request_id] += o.delta_token_ids
            if o.finished:
                reasons[o.request_id] = o.finish_reason
        check_invariants(eng)
    assert reasons == {"a": "length", "b": "length"}
    for rid, (p, sp) in reqs.items():
        assert (expected_output(p, 3)[-len(out[rid]):] == out[rid]) and len(out[rid]) >= 2
    # a lone request whose prompt can never fit is handed back as failed, not retried forever
    eng = make_fake_engine(num_pages=5, budget=48)                   # 64 tokens of cache
    r = eng.add_request("big", list(range(100)), greedy(2))
    outs = []
    for _ in range(10):
        outs += eng.step()
    assert [(o.request_id, o.finish_reason) for o in outs] == [("big", "error")] and not eng.cache.live


def test_abort_and_stop_rules():
    eng = make_fake_engine()
    eng.add_request("a", [1, 2, 3], greedy(50))
    eng.add_request("b", [4, 5, 6], greedy(50))
    eng.step()
    eng.abort("a")
    outs = eng.step()
    assert any(o.request_id == "a" and o.finish_reason == "abort" for o in outs)
    assert "a" not in eng.requests
    check_invariants(eng)
    while eng.has_unfinished():
        eng.step()
    assert not eng.cache.live
    # stop tokens: eos unless ignore_eos; stop_token_ids always; max_model_len
    first = expected_output([7, 8, 9], 3)
    eng = make_fake_engine(eos=(first[1],))
    out, reasons, _ = run(eng, {"x": ([7, 8, 9], greedy(10)), "y": ([7, 8, 9], greedy(10, ignore_eos=True)),
                                "z": ([7, 8, 9], greedy(10, stop_token_ids=[first[0]]))})
    assert out["x"] == first[:2] and reasons["x"] == "stop"
    assert len(out["y"]) == 10 and reasons["y"] == "length"
    assert out["z"] == first[:1] and reasons["z"] == "stop"
    eng = make_fake_engine(max_model_len=8)
    out, reasons, _ = run(eng, {"m": ([1, 2, 3, 4, 5], greedy(10))})
    assert len(out["m"]) == 3 and reasons["m"] == "length"


def test_duplicate_and_empty_requests_are_refused():
    eng = make_fake_engine()
    eng.add_request("a", [1], greedy(1))
    with pytest.raises(ValueError, match="duplicate"):
        eng.add_request("a", [1], greedy(1))
    with pytest.raises(ValueError, match="at least one"):
        eng.add_request("b", [], greedy(1))


def test_requests_are_checked_when_they_are_added():
    """A prompt that leaves no room within max_model_len, or a token id outside the vocabulary, is
    refused at add_request: the other requests never see it."""
    eng = make_fake_engine(max_model_len=32)
    eng.vocab_size = 1000
    with pytest.raises(ValueError, match="max_model_len"):
        eng.add_request("long", list(range(32)), greedy(3))
    with pytest.raises(ValueError, match="outside"):
        eng.add_request("bad", [1, 2, 1000], greedy(3))
    with pytest.raises(ValueError, match="outside"):
        eng.add_request("neg", [1, -2, 3], greedy(3))
    out, reasons, _ = run(eng, {"ok": (list(range(10)), greedy(3))})
    assert reasons == {"ok": "length"} and out["ok"] == expected_output(list(range(10)), 3)
    assert not eng.cache.live and not eng.requests


def test_a_kernel_fault_ends_the_steps_requests_and_switches_the_kernel_off():
    """A status word that is not zero beside a step's tokens (a block of a kernel gave up on a
    bounded wait): every request of that step finishes with "error", the kernel object is told, and
    requests that arrive afterwards run normally."""
    from tests.fakes import FakeSampler
    from turingserve_b200 import kernels

    class Pending:
        def __init__(self, tokens, bad, status):
            self.tokens, self.bad, self._status = tokens, bad, status
            self.device_out = None

        def status(self):
            return self._status

    class StatusSampler(FakeSampler):
        calls = 0

        def launch(self, logits, rows):
            StatusSampler.calls += 1
            tokens, bad = self.sample(logits, rows)
            return Pending(tokens, bad, [0, 0, 7, 0] if StatusSampler.calls == 3 else [0, 0, 0, 0])

        def finish(self, pending):
            return pending.tokens, pending.bad

    class FakeOps:
        reported = []

        def fault_reported(self, status):
            FakeOps.reported.append(list(status))
            return "decode attention gave up"

    eng = make_fake_engine(budget=8)
    eng.sampler = StatusSampler()
    eng.cfg.async_decode = False
    kernels.use(FakeOps())
    try:
        eng.add_request("a", [1, 2, 3], greedy(10))
        eng.add_request("b", [4, 5, 6], greedy(10))
        eng.add_request("c", list(range(30)), greedy(10))         # still in the middle of its prompt at step 3
        reasons = {}
        for _ in range(3):
            for o in eng.step():
                if o.finished:
                    reasons[o.request_id] = o.finish_reason
        assert reasons == {"a": "error", "b": "error", "c": "error"}
        assert FakeOps.reported == [[0, 0, 7, 0]] and eng.faults == ["decode attention gave up"]
        assert not eng.cache.live
        out, reasons, _ = run(eng, {"d": ([7, 8, 9], greedy(4))})
        assert reasons == {"d": "length"} and out["d"] == expected_output([7, 8, 9], 4)
    finally:
        kernels.use(None)


@pytest.mark.parametrize("padded", [True, False])
def test_padding_rows_of_captured_steps_count_against_the_budget(padded):
    """Where the runner fills decoding requests up to a captured number of rows, those rows come out of the
    token budget, so that the prompt portion beside them has the budget less a captured size: 3 decoding
    requests are 4 rows, a budget of 32 leaves 28 for the portion (29 without).  The tokens are the same."""
    eng = make_fake_engine(num_pages=256, budget=32, max_seqs=8)
    if padded:
        eng.scheduler.padded_decodes = lambda n: next((s for s in (1, 2, 4, 8) if s >= n), None)
    for i in range(3):
        eng.add_request(f"d{i}", [i + 1, i + 2, i + 3], greedy(40))
    eng.step()
    long_prompt = list(range(100))
    eng.add_request("long", long_prompt, greedy(5))
    plan = eng.scheduler.schedule()
    assert plan.num_decode == 3
    assert [p.num_tokens for p in plan.items] == [1, 1, 1, 28 if padded else 29]
    out = {}
    for o in eng._run(plan):
        out.setdefault(o.request_id, []).extend(o.delta_token_ids)
    while eng.has_unfinished():
        for o in eng.step():
            out.setdefault(o.request_id, []).extend(o.delta_token_ids)
        check_invariants(eng)
    assert out["long"] == expected_output(long_prompt, 5)
    for i in range(3):
        assert out[f"d{i}"][-1] == expected_output([i + 1, i + 2, i + 3], 40)[-1]


def test_padding_rows_never_starve_a_prompt():
    """5 decoding requests would be filled up to 8 rows: under a budget of 20 that would leave a prompt 12
    tokens, fewer than any captured portion, so the padding is not charged and the prompt gets all 15."""
    eng = make_fake_engine(num_pages=256, budget=20, max_seqs=8)
    eng.scheduler.padded_decodes = lambda n: next((s for s in (1, 2, 4, 8) if s >= n), None)
    for i in range(5):
        eng.add_request(f"d{i}", [i + 1, i + 2], greedy(30))
    eng.step()
    eng.add_request("long", list(range(60)), greedy(2))
    plan = eng.scheduler.schedule()
    assert [p.num_tokens for p in plan.items] == [1, 1, 1, 1, 1, 15]
