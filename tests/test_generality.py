"""(c)'s generality: parts chosen layer by layer, a mixer with state of its own registered from
the test, a feed-forward that routes and a position encoding registered from the test, a
position-free layer, partial rotary, a layer that runs twice, a run that reads another
run's cache, two cache groups.  Runs on the CPU with the kernel twins and, marked gpu, on the GPU."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests import schedules, tiny, toy
from tests.twin_ops import TwinOps
from turingserve_b200 import kernels
from turingserve_b200.engine.replay import Replayer
from turingserve_b200.weights import write_random_model


def _toy_folder(tmp_path, c=toy.TOY):
    folder = str(tmp_path / "toy")
    write_random_model(folder, toy.make(c), seed=5, std=0.1)
    return folder


def _run_toy(folder, device, dtype, tol, c=toy.TOY, groups=2, states=2):
    cfg_json, w = plain.read_folder(folder)
    reqs = {f"r{i}": tiny.random_ids(n, c["vocab"], 50 + i) for i, n in enumerate([40, 7, 61, 23, 35])}
    expected = {rid: toy.plain_forward(c, w, t).numpy() for rid, t in reqs.items()}
    for sched in ("whole", "decode_tail", "portions", "mixed"):
        steps = getattr(schedules, sched)(reqs)
        rp = Replayer(folder, dtype, schedules.peak_tokens(steps), device, page_size=8)
        assert len(rp.cache.groups) == groups, "full and windowed attention runs live in separate groups"
        assert sum(s is not None for s in rp.cache.states) == states, "one state per run of a running-mean layer"
        outs = {}
        with torch.inference_mode():
            for s in steps:
                o = rp.step(s)
                if o is not None:
                    outs[s["step"]] = o
                rp.cache.check()
        got = schedules.collect(steps, outs)
        bad = schedules.first_bad(got, expected, tol)
        assert bad is None, f"{sched}: first wrong place {bad}"


def test_toy_architecture_on_cpu(tmp_path):
    kernels.use(TwinOps())
    try:
        _run_toy(_toy_folder(tmp_path), "cpu", torch.float32, 1e-4)
    finally:
        kernels.use(None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 0.06)])
def test_toy_architecture_on_gpu(tmp_path, dtype, tol):
    kernels.use(None)
    _run_toy(_toy_folder(tmp_path), "cuda", dtype, tol)


def test_toy_with_routed_feed_forward_and_its_own_position_encoding_on_cpu(tmp_path):
    """A feed-forward with routing and a position encoding, both registered by the test, are built from
    the configuration layer by layer and stepped like the built-in parts."""
    kernels.use(TwinOps())
    try:
        _run_toy(_toy_folder(tmp_path, toy.TOY_ROUTED), "cpu", torch.float32, 1e-4, toy.TOY_ROUTED, groups=1, states=1)
    finally:
        kernels.use(None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 0.06)])
def test_toy_with_routed_feed_forward_and_its_own_position_encoding_on_gpu(tmp_path, dtype, tol):
    """The same toy through the CUDA kernels: its routed feed-forward and its position encoding are the
    test's own code between the framework's attention, norm and step function."""
    kernels.use(None)
    _run_toy(_toy_folder(tmp_path, toy.TOY_ROUTED), "cuda", dtype, tol, toy.TOY_ROUTED, groups=1, states=1)


def test_toy_with_a_third_norm_and_a_model_class_of_its_own_on_cpu(tmp_path):
    """A block arrangement that names a part in a role the built-in one does not have (a third norm,
    with its own checkpoint prefix), and a model class registered with the architecture that scales the
    embeddings and caps the logits: built, loaded and stepped without a change to the framework."""
    kernels.use(TwinOps())
    try:
        c = toy.TOY_SANDWICH
        folder = _toy_folder(tmp_path, c)
        from safetensors import safe_open
        with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
            assert "blocks.1.norm_mid.weight" in set(f.keys())
        _run_toy(folder, "cpu", torch.float32, 1e-4, c, groups=1, states=1)
    finally:
        kernels.use(None)


@pytest.mark.gpu
def test_toy_with_a_third_norm_and_a_model_class_of_its_own_on_gpu(tmp_path):
    kernels.use(None)
    c = toy.TOY_SANDWICH
    _run_toy(_toy_folder(tmp_path, c), "cuda", torch.float32, 1e-4, c, groups=1, states=1)
    _run_toy(_toy_folder(tmp_path, c), "cuda", torch.bfloat16, 0.06, c, groups=1, states=1)


def test_padding_rows_of_a_captured_batch_leave_live_state_alone(tmp_path):
    """A decode batch padded to a captured size: the padding rows carry the null state slot, so a
    mixer with state of its own neither reads nor resets the state of the request in slot 0."""
    from turingserve_b200.engine.batch import StepEntry
    from turingserve_b200.engine.runner import ModelRunner, run_needs
    from turingserve_b200.cache import CacheManager
    from turingserve_b200.weights.loader import load_model
    kernels.use(TwinOps())
    try:
        c = toy.TOY
        folder = _toy_folder(tmp_path)
        _, w = plain.read_folder(folder)
        model, cfg = load_model(folder, torch.float32, "cpu")
        cache = CacheManager(run_needs(model), 8, 40, 4, torch.float32, "cpu")
        runner = ModelRunner(model, cache, 64, 4, 128)
        ids = tiny.random_ids(12, c["vocab"], 3)
        rc = cache.admit("a")
        assert rc.slot == 0 and cache.null_slot == 4
        with torch.inference_mode():
            runner.step([StepEntry(rc, ids[:9], [])])
            rows = []
            for t in ids[9:]:
                entries = [StepEntry(rc, [t], [0])]
                cache.grow(rc, 1)
                step = runner.builder.build(entries, pad_requests=3)
                assert step.state_slots.tolist() == [0, 4, 4, 4] and step.num_requests == 4
                rows.append(runner.forward(step)[0])
                cache.advance(rc, 1)
        want = toy.plain_forward(c, w, ids)[9:]
        assert (torch.stack(rows) - want).abs().max() < 1e-4
    finally:
        kernels.use(None)


def test_schedule_that_repeats_and_shares_on_qwen2(tmp_path):
    """The run order is data: the same Qwen2 weights with a layer run twice and a shared cache."""
    from turingserve_b200.config import LayerRun
    from turingserve_b200.engine.batch import StepEntry
    from turingserve_b200.engine.runner import ModelRunner, run_needs
    from turingserve_b200.cache import CacheManager
    from turingserve_b200.parts.model import DecoderModel
    from turingserve_b200.weights.loader import load_into
    kernels.use(TwinOps())
    try:
        folder = tiny.make_tiny_folder("B", tmp_path)
        cfg_json, w = plain.read_folder(folder)
        sched = [(0, None), (1, None), (1, None), (2, 1), (0, None)]
        cfg = tiny.tiny_config("B").with_schedule([LayerRun(l, f) for l, f in sched])
        model = DecoderModel(cfg, torch.float32, "cpu", 256)
        load_into(model, folder)
        cache = CacheManager(run_needs(model), 8, 40, 2, torch.float32, "cpu")
        runner = ModelRunner(model, cache, 128, 2, 256)
        ids = tiny.random_ids(45, cfg.vocab_size, 9)
        rc = cache.admit("a")
        with torch.inference_mode():
            a = runner.step([StepEntry(rc, ids[:17], list(range(17)))])
            b = runner.step([StepEntry(rc, ids[17:19], [0, 1])])
            c = runner.step([StepEntry(rc, ids[19:], list(range(26)))])
        got = torch.cat([a, b, c])
        want = plain.forward(cfg_json, w, ids, schedule=sched)
        assert (got - want).abs().max() < 1e-4
        assert len(cache.groups[0].runs) == 4                       # run 3 reads run 1's cache and owns none
    finally:
        kernels.use(None)
