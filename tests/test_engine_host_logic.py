"""The engine's host logic (cache manager, batch builder, step function, replay) on the CPU, with
the plain torch twins standing in for the CUDA kernels: every way of cutting the work must give
the plain whole-sequence logits."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests import schedules, tiny
from tests.twin_ops import TwinOps
from turingserve_b200 import kernels
from turingserve_b200.engine.replay import Replayer


@pytest.fixture()
def twin_ops():
    kernels.use(TwinOps())
    yield
    kernels.use(None)


def _requests(name, cfg, lengths):
    return {f"r{i}": tiny.random_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(lengths)}


LENGTHS = {"A": [5, 17, 33, 70, 41, 64], "B": [1, 9, 40, 70, 97, 33], "W": [3, 50, 77, 120, 64, 31],
           "X": [2, 33, 100, 64, 7, 129]}


@pytest.mark.parametrize("name", ["A", "B", "W", "X"])
@pytest.mark.parametrize("schedule", ["whole", "decode_tail", "portions", "mixed"])
def test_schedules_match_plain(tmp_path, twin_ops, name, schedule):
    folder = tiny.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    reqs = _requests(name, cfg, LENGTHS[name])
    expected = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    steps = getattr(schedules, schedule)(reqs)
    rp = Replayer(folder, torch.float32, schedules.peak_tokens(steps), "cpu", page_size=tiny.page_size(name))
    outs = {}
    with torch.inference_mode():
        for s in steps:
            o = rp.step(s)
            if o is not None:
                outs[s["step"]] = o
            rp.cache.check()
    got = schedules.collect(steps, outs)
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    bad = schedules.first_bad(got, expected, 1e-4)
    assert bad is None, f"first wrong place {bad}"
    assert not rp.cache.live
    for g in rp.cache.groups:
        assert g.allocator.num_free == g.allocator.num_usable


@pytest.mark.parametrize("name", ["A", "W"])
def test_steps_laid_out_as_captured_shapes_match_plain(tmp_path, twin_ops, name):
    """The layout a captured step has (single-token requests filled up to 1, 2 or 4 rows with empty rows,
    one prompt portion behind them, block tables at full width, the logits of every single-token row and
    of the portion's last row) run eagerly with the kernel twins: the rows handed back are the plain
    logits, whatever the padding, and which steps take that layout is decided as documented."""
    from turingserve_b200.engine.batch import StepEntry
    from turingserve_b200.engine.runner import _StepGraph
    folder = tiny.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    reqs = _requests(name, cfg, LENGTHS[name])
    expected = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    steps = schedules.served(reqs, portion=16)
    rp = Replayer(folder, torch.float32, schedules.peak_tokens(steps), "cpu", page_size=tiny.page_size(name),
                  graph_batch_sizes=(1, 2, 4), graph_portion_sizes=(16,))
    runner, shapes, outs = rp.runner, set(), {}
    live = {}
    with torch.inference_mode():
        for s in steps:
            entries = []
            for e in s["entries"]:
                rc = live.get(e["id"]) or live.setdefault(e["id"], rp.cache.admit(e["id"]))
                entries.append(StepEntry(rc, list(e["tokens"]), list(e["want"])))
            for e in entries:
                rp.cache.grow(e.cache, len(e.tokens))
            shape = runner._graph_shape(entries)
            if shape is None:
                logits = runner.forward(runner.builder.build(entries))
            else:
                shapes.add(shape)
                g = _StepGraph(runner, shape[0], shape[1], False)
                step = g._build(entries)
                assert step.num_requests == shape[0] + (1 if shape[1] else 0) and step.num_decode == shape[0]
                assert step.num_tokens == shape[0] + shape[1]
                g.logits = runner.forward(step)
                assert g.logits.shape[0] == shape[0] + (1 if shape[1] else 0)
                logits = g._wanted(entries)
            for e in entries:
                rp.cache.advance(e.cache, len(e.tokens))
            for rid in s["end"]:
                rp.cache.release(live.pop(rid))
            if logits is not None:
                outs[s["step"]] = logits.float().numpy()
            rp.cache.check()
    assert {p for _, p in shapes} == {0, 16} and {sz for sz, p in shapes if p} >= {2, 4}, shapes
    bad = schedules.first_bad(schedules.collect(steps, outs), expected, 1e-4)
    assert bad is None, f"first wrong place {bad}"
    # which steps take the layout
    rc = rp.cache.admit("x")
    one = lambda want=(0,): StepEntry(rc, [1], list(want))
    assert runner._graph_shape([one()] * 3) == (4, 0)
    assert runner._graph_shape([one(), StepEntry(rc, [1] * 16, [])]) == (1, 16)
    assert runner._graph_shape([StepEntry(rc, [1] * 16, [15])]) == (0, 16)
    assert runner._graph_shape([one(), StepEntry(rc, [1] * 16, [3])]) is None          # logits wanted inside the portion
    assert runner._graph_shape([one(), StepEntry(rc, [1] * 15, [])]) is None           # a length that is not captured
    assert runner._graph_shape([StepEntry(rc, [1] * 16, []), StepEntry(rc, [1] * 16, [])]) is None
    assert runner._graph_shape([one(()), one()]) is None                               # a single token whose logits nobody wants
    assert runner._graph_shape([one()] * 5) is None                                    # more than the largest captured size
    assert runner._graph_shape([one(), StepEntry(rc, [1] * 16, [], feedback=0)]) is None
