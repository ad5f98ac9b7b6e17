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
