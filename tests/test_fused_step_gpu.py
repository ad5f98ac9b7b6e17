"""The decode step as one persistent kernel (csrc/decode_step.cu, parts/fused_decode.py), switched on
for the test: the same requests through the same schedules as the chain of kernels, against the plain
implementation.  The kernel is off by default (it does not yet beat the chain), so nothing else in the
suite runs it."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests import schedules, tiny
from tests.test_replay_gpu import BF16_REL, expected_logits, requests_for

pytestmark = pytest.mark.gpu


def _replay(folder, page, steps, graphs=()):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    kernels.use(None)
    rp = Replayer(folder, torch.bfloat16, schedules.peak_tokens(steps), "cuda", page_size=page, graph_batch_sizes=graphs)
    outs = {}
    with torch.inference_mode():
        for s in steps:
            o = rp.step(s)
            if o is not None:
                outs[s["step"]] = o
            rp.cache.check()
    return schedules.collect(steps, outs), rp


@pytest.fixture()
def fused(monkeypatch):
    from turingserve_b200 import kernels
    from turingserve_b200.parts.fused_decode import FusedDecodeStep
    monkeypatch.setattr(FusedDecodeStep, "enabled", True)
    yield
    assert kernels.ops().tc_status() == 0


@pytest.mark.parametrize("graphs", [(), (1, 2, 4)])
@pytest.mark.parametrize("schedule", ["batched_tail", "decode_tail", "mixed"])
def test_fused_step_on_the_tiny_model_with_heads_of_128(tmp_path, fused, schedule, graphs):
    folder = tiny.make_tiny_folder("K", tmp_path)
    reqs = requests_for("K", folder)
    steps = getattr(schedules, schedule)(reqs)
    got, rp = _replay(folder, tiny.page_size("K"), steps, graphs)
    assert rp.runner.fused is not None and rp.runner.fused.runs > 0, "the fused step did not run"
    expected = expected_logits(folder, reqs)
    _, w16 = plain.read_folder(folder, torch.bfloat16)
    cfg, _ = plain.read_folder(folder)
    for rid, toks in reqs.items():
        scale = float(np.abs(expected[rid]).max())
        yard = np.abs(plain.forward(cfg, w16, toks).float().numpy() - expected[rid]).max(1) / scale
        errs = np.array([np.abs(got[rid][p] - expected[rid][p]).max() for p in range(len(toks))]) / scale
        assert np.isfinite(errs).all()
        assert errs.max() <= 1.5 * yard.max() + 1e-3, (rid, int(errs.argmax()), float(errs.max()), float(yard.max()))


@pytest.mark.parametrize("page", [16, 64])
def test_fused_step_at_real_layer_sizes_and_long_contexts(tmp_path, fused, page):
    """Two layers of the Qwen2.5-1.5B shape; contexts long enough that a block's share of the keys is as
    many stages as the ring has (where a waiter that skipped those stages once fell two phases behind),
    eight requests decoding together, the new token's key in the first, a middle and the last row of a
    page."""
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.weights import write_random_model
    folder = str(tmp_path / "real")
    write_random_model(folder, make_config(hidden_size=1536, intermediate_size=8960, num_layers=2, num_heads=12,
                                           num_kv_heads=2, vocab_size=2000, rope_theta=1e6, rms_norm_eps=1e-6,
                                           tie_word_embeddings=True, max_position_embeddings=4096), seed=4)
    cfg, w = plain.read_folder(folder)
    lens = [2090, 700, 1290, 65, 2100, 130, 515, 33]
    reqs = {f"r{i}": tiny.random_ids(n, 2000, 300 + i) for i, n in enumerate(lens)}
    expected = {k: plain.forward(cfg, w, v).numpy() for k, v in reqs.items()}
    # all eight live at once: heads one by one, then 20 tokens each decoded together
    steps = schedules.batched_tail(reqs, tail=20, max_live=8)
    from turingserve_b200.engine import replay
    old = replay.MAX_LIVE
    replay.MAX_LIVE = 8
    try:
        got, rp = _replay(folder, page, steps)
    finally:
        replay.MAX_LIVE = old
    assert rp.runner.fused is not None and rp.runner.fused.runs >= 20
    for rid, rows in got.items():
        tol = BF16_REL * float(np.abs(expected[rid]).max())
        bad = schedules.first_bad({rid: rows}, expected, tol)
        assert bad is None, (page, bad, tol)
