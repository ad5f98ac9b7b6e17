"""The engine on the GPU against the plain implementation: the same requests whole, with the last
32 tokens decoded one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again; in 32-bit and in bfloat16; in-process and through
``bin/trace_run`` as a user starts it."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests import schedules, tiny

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": [5, 17, 33, 70, 41, 64], "B": [1, 9, 40, 70, 97, 33], "W": [3, 50, 77, 120, 64, 31],
           "K": [5, 130, 200, 70, 257, 64], "L": [3, 150, 77, 260, 128, 31], "X": [2, 33, 100, 64, 7, 129]}
# float32: the reference's own bound for logits (tests/correctness/test_vs_hf.py:40-48).
# bfloat16: 8 bits of mantissa; logits of these models reach |2.5|; the bound is 3% of the largest
# expected logit of the request, about eight bfloat16 roundings.
F32_TOL = 1e-4
BF16_REL = 3e-2


def expected_logits(folder, reqs):
    cfg, w = plain.read_folder(folder)
    return {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def requests_for(name, folder):
    cfg, _ = plain.read_folder(folder)
    return {f"r{i}": tiny.random_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])}


def check(got, expected, dtype):
    if dtype == "float32":
        bad = schedules.first_bad(got, expected, F32_TOL)
        assert bad is None, f"first wrong place (request, position, error): {bad}"
    else:
        for rid, rows in got.items():
            tol = BF16_REL * float(np.abs(expected[rid]).max())
            bad = schedules.first_bad({rid: rows}, expected, tol)
            assert bad is None, f"first wrong place (request, position, error): {bad}, bound {tol}"


def replay_in_process(folder, name, steps, dtype, gemm="library", fresh_ops=True, graphs=(), replayer=None, portions=()):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    if fresh_ops:
        kernels.use(None)
    kernels.ops().gemm_mode = gemm
    rp = Replayer(folder, getattr(torch, dtype), schedules.peak_tokens(steps), "cuda", page_size=tiny.page_size(name),
                  graph_batch_sizes=graphs, graph_portion_sizes=portions)
    if replayer is not None:
        replayer.append(rp)
    outs = {}
    with torch.inference_mode():
        for s in steps:
            o = rp.step(s)
            if o is not None:
                outs[s["step"]] = o
            rp.cache.check()
    assert not rp.cache.live
    kernels.ops().gemm_mode = "auto"
    return schedules.collect(steps, outs)


@pytest.mark.parametrize("dtype,gemm", [("float32", "library"), ("bfloat16", "library"), ("bfloat16", "auto"),
                                        ("bfloat16", "tc")])
@pytest.mark.parametrize("name", ["A", "B", "W", "X"])
@pytest.mark.parametrize("schedule", ["whole", "decode_tail", "portions", "mixed"])
def test_schedules_match_plain(tmp_path, name, schedule, dtype, gemm):
    """``gemm``: which bfloat16 products run on this library's tcgen05 kernel (none, the few-token
    ones, all); the float32 path always uses the FFMA kernel."""
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = getattr(schedules, schedule)(reqs)
    got = replay_in_process(folder, name, steps, dtype, gemm)
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    check(got, expected_logits(folder, reqs), dtype)


@pytest.mark.parametrize("decode", ["cp", "tma"])
@pytest.mark.parametrize("portions", ["tc", "mma"])
@pytest.mark.parametrize("name", ["K", "L"])
@pytest.mark.parametrize("schedule", ["whole", "decode_tail", "portions", "mixed"])
def test_schedules_on_the_tensor_core_attention_kernels(tmp_path, monkeypatch, name, schedule, decode, portions):
    """Models whose head size and pages the fast bfloat16 attention kernels take, through every
    schedule: both decode kernels (the chain-length one, the streaming one with TMA) and both
    prompt-portion kernels (tcgen05 where the head size is 128, mma.sync)."""
    from turingserve_b200 import kernels
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = getattr(schedules, schedule)(reqs)
    kernels.use(None)
    ops = kernels.ops()
    monkeypatch.setattr(ops, "decode_kernel", decode)
    monkeypatch.setattr(ops, "use_tc_attention", portions == "tc")
    before = ops.launches
    got = replay_in_process(folder, name, steps, "bfloat16", "auto", fresh_ops=False)
    assert ops.launches > before and ops.tc_status() == 0
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    check(got, expected_logits(folder, reqs), "bfloat16")


@pytest.mark.parametrize("name", ["K", "L"])
@pytest.mark.parametrize("schedule", ["whole", "portions", "mixed"])
def test_schedules_with_the_many_row_products_on_pairs_of_sms(tmp_path, monkeypatch, name, schedule):
    """Steps of more than four tokens with the q/k/v product (bias, rotation and cache write in
    its epilogue) and the gate/up product (activation in its epilogue) on the kernel for pairs of SMs,
    which the cost rule would not pick for models this small: heads of 128 and of 64, steps in which
    single decoded tokens of other requests sit in front of the portion's rows."""
    from turingserve_b200 import kernels
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = getattr(schedules, schedule)(reqs)
    kernels.use(None)
    ops = kernels.ops()
    monkeypatch.setattr(ops, "pair_wins", lambda *a: True)
    monkeypatch.setattr(ops, "fused_qkv_tokens", 4)            # every step of more than four tokens takes them
    monkeypatch.setattr(ops, "fused_gate_tokens", 4)
    used = []
    monkeypatch.setattr(ops, "linear_pair", lambda *a, _f=ops.linear_pair: (used.append("gated"), _f(*a))[1])
    qkv = ops.lib.ts_linear_pair_qkv
    monkeypatch.setattr(ops.lib, "ts_linear_pair_qkv", lambda *a: (used.append("qkv"), qkv(*a))[1])
    got = replay_in_process(folder, name, steps, "bfloat16", "auto", fresh_ops=False)
    assert "qkv" in used and ("gated" in used) == (name == "K"), "a feed-forward width of 272 has no blocks of 64 gates"
    assert ops.tc_status() == 0
    check(got, expected_logits(folder, reqs), "bfloat16")


@pytest.mark.parametrize("graphs", [(), (1,)])
def test_long_context_on_the_kernels_a_long_context_picks(tmp_path, graphs):
    """One request of 3,900 tokens and a second of 700 on the K model: the prompt attention with several
    waves of blocks, then decoding where the split rule by itself asks for sixteen pieces (the blocks of
    8 warps) and, under a captured graph, launch geometry for the longest context; logits of the last 32
    positions one by one against the plain implementation."""
    from turingserve_b200 import kernels
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.weights import write_random_model
    folder = str(tmp_path / "long")
    write_random_model(folder, make_config(hidden_size=192, intermediate_size=320, num_layers=2, num_heads=4, num_kv_heads=2,
                                           head_dim=128, vocab_size=300, rope_theta=1e6, rms_norm_eps=1e-6,
                                           tie_word_embeddings=True, max_position_embeddings=4096), seed=9, std=0.03)
    cfg, _ = plain.read_folder(folder)
    reqs = {"long": tiny.random_ids(3900, cfg["vocab_size"], 7), "short": tiny.random_ids(700, cfg["vocab_size"], 8)}
    steps = schedules.decode_tail(reqs)
    kernels.use(None)
    got = replay_in_process(folder, "K", steps, "bfloat16", "auto", graphs=graphs)
    assert kernels.ops().tc_status() == 0
    check(got, expected_logits(folder, reqs), "bfloat16")


@pytest.mark.parametrize("schedule", ["batched_tail", "decode_tail", "mixed"])
@pytest.mark.parametrize("graphs", [(), (1, 2, 4)])
def test_decode_attention_cut_into_sixteen(tmp_path, monkeypatch, schedule, graphs):
    """What a step of few requests with long contexts runs (the split rule asks for 16 pieces, the kernel
    then takes 8 pieces of 8 warps and tiles of 128 keys), here forced on the short contexts of the K
    model so that most pieces hold no key at all and the others end anywhere in a tile: logits at every
    position against the plain implementation, with and without captured graphs."""
    from turingserve_b200 import kernels
    folder = tiny.make_tiny_folder("K", tmp_path)
    reqs = requests_for("K", folder)
    steps = getattr(schedules, schedule)(reqs)
    kernels.use(None)
    ops = kernels.ops()
    monkeypatch.setattr(ops, "decode_kernel", "cp")
    monkeypatch.setattr(ops, "decode_splits", lambda *a: 16)
    got = replay_in_process(folder, "K", steps, "bfloat16", "auto", fresh_ops=False, graphs=graphs)
    assert ops.tc_status() == 0
    check(got, expected_logits(folder, reqs), "bfloat16")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16"),
                                        ("K", "bfloat16"), ("L", "bfloat16")])
@pytest.mark.parametrize("schedule", ["batched_tail", "decode_tail", "mixed"])
def test_captured_decode_graphs_give_the_same_logits(tmp_path, monkeypatch, name, schedule, dtype):
    """The step that generation and the benchmark run: single-token steps replayed from captured CUDA
    graphs of sizes 1, 2 and 4 (padding rows when 3 decode together, block tables at full width, launch
    geometry for the longest context), the decode-attention choice flipping in the middle (one graph per
    size and choice).  Logits at every position against the plain implementation, same bounds as without
    graphs."""
    from turingserve_b200 import kernels
    from turingserve_b200.engine import batch
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = getattr(schedules, schedule)(reqs)
    monkeypatch.setattr(batch, "STREAMING_DECODE_KEYS", 150)
    held = []
    got = replay_in_process(folder, name, steps, dtype, "auto", graphs=(1, 2, 4), replayer=held)
    captured = set(held[0].runner._graphs)
    sizes = {len(s["entries"]) for s in steps if all(len(e["tokens"]) == 1 for e in s["entries"])}
    assert {sz for sz, _, _ in captured} >= {1 if 1 in sizes else min(sizes)}, captured
    if schedule == "batched_tail":
        assert 3 in sizes and {sz for sz, _, _ in captured} >= {1, 2, 4}, (sizes, captured)
        assert {st for _, _, st in captured} == {False, True}, captured
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    check(got, expected_logits(folder, reqs), dtype)
    assert kernels.ops().tc_status() == 0


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("K", "bfloat16"), ("L", "bfloat16")])
def test_captured_steps_of_decodes_beside_a_prompt_portion(tmp_path, monkeypatch, name, dtype):
    """Steps as a serving engine cuts them (decoding requests, filled up to 1, 2 or 4 rows, beside one prompt
    portion of 16 tokens) replayed from captured graphs, one per (rows, portion length, decode-attention
    choice); the last, shorter portion of a prompt and the first steps run kernel by kernel.  The logits of
    every decoded token and of every prompt's last token against the plain implementation: the portions'
    keys and values, written by replayed graphs, are what the decoded tokens read."""
    from turingserve_b200 import kernels
    from turingserve_b200.engine import batch
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = schedules.served(reqs, portion=16)
    monkeypatch.setattr(batch, "STREAMING_DECODE_KEYS", 150)
    held = []
    got = replay_in_process(folder, name, steps, dtype, "auto", graphs=(1, 2, 4), replayer=held, portions=(16,))
    captured = set(held[0].runner._graphs)
    beside = {sz for sz, p, _ in captured if p == 16}
    assert len(beside) >= 2 and 4 in beside and any(p == 0 for _, p, _ in captured), captured
    expected = expected_logits(folder, reqs)
    assert sum(len(v) for v in got.values()) > sum(min(20, len(t) - 1) for t in reqs.values())
    check(got, expected, dtype)
    assert kernels.ops().tc_status() == 0


@pytest.mark.parametrize("name", ["K", "L"])
@pytest.mark.parametrize("schedule", ["whole", "decode_tail", "portions", "mixed", "batched_tail"])
def test_fast_kernels_are_as_close_as_a_plain_bfloat16_run(tmp_path, name, schedule):
    """The models that reach the tensor-core and TMA attention kernels cannot show their faults in
    32-bit (those kernels are bfloat16 only), and 3 % of the largest logit is a loose bound on its own.
    The yardstick here is the plain implementation itself run with bfloat16 weights and activations: the
    engine's error against the 32-bit plain logits (median and 95th percentile over positions, and the
    worst position) may not exceed 1.5 times that run's."""
    from turingserve_b200 import kernels
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    cfg, w = plain.read_folder(folder)
    _, w16 = plain.read_folder(folder, torch.bfloat16)
    expected = expected_logits(folder, reqs)
    steps = getattr(schedules, schedule)(reqs)
    got = replay_in_process(folder, name, steps, "bfloat16", "auto",
                            graphs=(1, 2, 4) if schedule == "batched_tail" else ())
    for rid, toks in reqs.items():
        scale = float(np.abs(expected[rid]).max())
        yard = np.abs(plain.forward(cfg, w16, toks).float().numpy() - expected[rid]).max(1) / scale
        errs = np.array([np.abs(got[rid][p] - expected[rid][p]).max() for p in range(len(toks))]) / scale
        assert np.isfinite(errs).all()
        if len(toks) >= 8:
            assert np.median(errs) <= 1.5 * np.median(yard), (rid, float(np.median(errs)), float(np.median(yard)))
            assert np.percentile(errs, 95) <= 1.5 * np.percentile(yard, 95), (rid, int(errs.argmax()))
        assert errs.max() <= 1.5 * yard.max() + 1e-3, (rid, int(errs.argmax()), float(errs.max()), float(yard.max()))
    assert kernels.ops().tc_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a subprocess: steps on stdin, `done <step>` after each, files in --out."""
    name = "B"
    folder = tiny.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = schedules.mixed(reqs, seed=3)
    out = tmp_path / f"out_{dtype}"
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                          "--out", str(out), "--max-tokens", str(schedules.peak_tokens(steps)),
                          "--block-size", str(tiny.page_size(name))] + (["--graphs", "1,2"] if dtype == "bfloat16" else []),
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {s['step']}"
    p.stdin.close()
    assert p.wait(timeout=120) == 0
    V = plain.read_folder(folder)[0]["vocab_size"]
    outs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, V) for s in steps}
    check(schedules.collect(steps, outs), expected_logits(folder, reqs), dtype)
