#!/usr/bin/env python3
"""Benchmark: decode tokens/s (default batch 8), prefill tokens/s at 2,048 tokens and roofline
fractions for a Qwen2.5-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model qwen2.5-1.5b|qwen2.5-7b|qwen2.5-14b] [--batch 8] [--kv-block 16] [--phases ...]

One JSON line.  Beside the contract's keys: ``prefill``, ``roofline`` (the whole decode step against
the copy bandwidth), ``points`` (batch 1 and 64, and the headline batch with pages of 64 tokens),
``kernels`` (each dominant kernel alone against its roofline), ``graph_check`` (the captured decode
step against the same step launched kernel by kernel) and ``mixed`` (the Qwen2.5-14B shape with 32
decodes beside a 2,048-token prompt in portions of 512).

A "step" is one decode step of the whole batch.  ``value`` times K decode steps of the engine's
step function with CUDA events (inputs built on the host, copied to the device each step);
``e2e`` times the same through ``LLMEngine.step`` (scheduler, step function, sampler; host tokens
in, sampled tokens out).  The method follows the reference's micro benchmark
(benchmarks/micro/decode_speed.py:42-64: warm-up steps dropped, speed of light = bandwidth /
bytes per step), on synthetic uniform token ids and N(0, 0.02) weights.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE configs[2]: Qwen2.5-1.5B shape
SHAPES = {
    "qwen2.5-0.5b": dict(hidden_size=896, intermediate_size=4864, num_layers=24, num_heads=14, num_kv_heads=2,
                         head_dim=64, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-1.5b": dict(hidden_size=1536, intermediate_size=8960, num_layers=28, num_heads=12, num_kv_heads=2,
                         head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-3b": dict(hidden_size=2048, intermediate_size=11008, num_layers=36, num_heads=16, num_kv_heads=2,
                       head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-7b": dict(hidden_size=3584, intermediate_size=18944, num_layers=28, num_heads=28, num_kv_heads=4,
                       head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=False, max_position_embeddings=32768),
    "qwen2.5-14b": dict(hidden_size=5120, intermediate_size=13824, num_layers=48, num_heads=40, num_kv_heads=8,
                        head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                        tie_word_embeddings=False, max_position_embeddings=32768),
    "qwen2.5-32b": dict(hidden_size=5120, intermediate_size=27648, num_layers=64, num_heads=40, num_kv_heads=8,
                        head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-5,
                        tie_word_embeddings=False, max_position_embeddings=32768),
}
SHAPE_NAMES = {"qwen2.5-0.5b": "Qwen2.5-0.5B", "qwen2.5-1.5b": "Qwen2.5-1.5B", "qwen2.5-3b": "Qwen2.5-3B",
               "qwen2.5-7b": "Qwen2.5-7B", "qwen2.5-14b": "Qwen2.5-14B", "qwen2.5-32b": "Qwen2.5-32B"}


def metric_name(a) -> str:
    """The same words in both arms: the driver divides two lines only when their metrics read alike.
    The precision each arm computes in is in its ``dtype``."""
    return f"decode tok/s at batch {a.batch} ({SHAPE_NAMES[a.model]} shape, {a.prompt_len:,}-token prompts)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(p.get(k), (int, float)):
                    out[k] = float(p[k])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.samples: list[list[str]] = []
        self.index = index
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                r = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                    "-i", str(self.index)], capture_output=True, text=True, timeout=5)
                if r.returncode == 0 and r.stdout.strip():
                    self.samples.append([x.strip() for x in r.stdout.strip().splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        mhz = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:]) if v.lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_numbers(kw: dict, layers: int) -> dict:
    h, I, H, KVH, D, V = (kw["hidden_size"], kw["intermediate_size"], kw["num_heads"], kw["num_kv_heads"],
                          kw["head_dim"], kw["vocab_size"])
    per_layer = h * (H + 2 * KVH) * D + (H + 2 * KVH) * D + H * D * h + 3 * h * I + 2 * h
    linear_params = layers * (h * (H + 2 * KVH) * D + H * D * h + 3 * h * I)
    head = V * h
    return dict(weight_bytes_decode=2 * (layers * per_layer + h + head),      # every weight a decode step reads
                kv_bytes_per_token=2 * layers * KVH * D * 2, linear_params=linear_params, head_params=head,
                attn_flops_per_layer=lambda T: 2.0 * T * T * D * H)             # causal: QK^T and PV, half each


def make_model(shape: str, layers: int, tmp: str) -> str:
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.weights.random_init import write_random_model
    kw = dict(SHAPES[shape])
    kw["num_layers"] = layers
    folder = os.path.join(tmp, f"{shape}-L{layers}")
    t0 = time.time()
    write_random_model(folder, make_config(**kw), seed=0)
    print(f"[bench] wrote random {shape} ({layers} layers) in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return folder


def build_engine_on_device(shape: str, layers: int, *, ctx_len: int, page: int, max_seqs: int, max_tokens: int,
                           graph_sizes: tuple[int, ...], model=None, portion_budget: int | None = None):
    """An engine around a model whose N(0, 0.02) weights are drawn on the device (no checkpoint file:
    the 14B shape would be 30 GB of it); everything else as ``LLMEngine.from_config`` builds it."""
    import torch

    from turingserve_b200 import EngineConfig, LLMEngine
    from turingserve_b200.cache.manager import CacheManager
    from turingserve_b200.engine.runner import ModelRunner, run_needs
    from turingserve_b200.engine.scheduler import Scheduler
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.sampling.sampler import Sampler
    from turingserve_b200.weights.random_init import random_model_on_device

    kw = dict(SHAPES[shape])
    kw["num_layers"] = layers
    mcfg = make_config(**kw)
    device = torch.device("cuda", 0)
    if model is None:
        t0 = time.time()
        model = random_model_on_device(mcfg, torch.bfloat16, device, seed=0, max_positions=ctx_len)
        torch.cuda.synchronize()
        print(f"[bench] random {shape} ({layers} layers) on the device in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    cfg = EngineConfig(model=f"<random {shape}>", dtype="bfloat16", max_model_len=ctx_len, block_size=page,
                       num_blocks=max_seqs * (-(-ctx_len // page)) + 8, max_num_seqs=max_seqs,
                       max_num_batched_tokens=max_tokens, graph_batch_sizes=graph_sizes, watermark=0.0)
    if portion_budget is not None:
        cfg.graph_portion_budget = portion_budget
    cfg.validate(mcfg.max_position_embeddings)
    cache = CacheManager(run_needs(model), page, cfg.num_blocks, max_seqs, torch.bfloat16, device)
    portions = cfg.graph_portion_sizes() if graph_sizes else ()
    runner = ModelRunner(model, cache, max(max_tokens, max_seqs), max_seqs, ctx_len, cfg.graph_batch_sizes, portions)
    sched = Scheduler(cache, max_tokens, max_seqs, 0.0, runner.padded_decodes if portions else None)
    return LLMEngine(cfg, runner, cache, sched, Sampler(device), mcfg.eos_token_ids, ctx_len, mcfg.vocab_size)


def graph_check(runner, cache, rcs, tokens) -> dict:
    """One decode step replayed from its captured graph, then the same tokens at the same positions
    launched kernel by kernel (the cache is told to forget the step, whose keys and values are simply
    written again): the logits must agree to within bfloat16 rounding of a step's different split of
    the keys.  A wrong-but-finite output head or a stale graph input would show here."""
    import torch

    from turingserve_b200.engine.batch import StepEntry
    entries = [StepEntry(rc, [int(t)], [0]) for rc, t in zip(rcs, tokens)]
    with_graph = runner.step(entries).clone()
    for rc in rcs:
        rc.num_tokens -= 1
    sizes, runner.graph_batch_sizes = runner.graph_batch_sizes, ()
    try:
        without = runner.step([StepEntry(rc, [int(t)], [0]) for rc, t in zip(rcs, tokens)])
    finally:
        runner.graph_batch_sizes = sizes
    err = float((with_graph - without).abs().max())
    top = float(without.abs().max())
    rel = float((with_graph - without).norm() / without.norm())
    same = int((with_graph.argmax(-1) == without.argmax(-1)).sum())
    # The two runs split the keys differently (a captured step sizes its launch for the longest context),
    # so they differ by bfloat16 roundings carried through every layer: a few percent of the largest logit
    # at the worst of a million entries and about 3 % in the root mean square after 28 layers (some 200
    # roundings of 2^-9 each, added like a random walk).  A stale graph input or a wrong head gives
    # unrelated rows: a relative difference near 1.4.
    if not (rel <= 0.15):
        raise RuntimeError(f"the captured decode step disagrees with the same step launched kernel by kernel: "
                           f"relative difference {rel:.4g} (largest {err:.4g} against a largest logit of {top:.4g})")
    return {"rel_l2_diff": round(rel, 5), "max_abs_diff": round(err, 5), "max_logit": round(top, 3),
            "same_argmax": same, "rows": len(rcs)}


def run_ours(a) -> dict:
    import numpy as np
    import torch

    from turingserve_b200 import SamplingParams, kernels
    from turingserve_b200.engine.batch import StepEntry

    torch.cuda.set_device(0)
    ops = kernels.ops()
    pk, pk_src = peaks()
    kw = SHAPES[a.model]
    layers = a.layers or kw["num_layers"]
    nums = model_numbers(kw, layers)
    B, prompt_len, ctx_len = a.batch, a.prompt_len, a.context
    rng = np.random.default_rng(0)
    V = kw["vocab_size"]

    max_b = max(B, 64)
    ctx_len = max(ctx_len, a.prefill_tokens + 64, prompt_len + a.steps + max(3, a.warmup) + 64)
    eng = build_engine_on_device(a.model, layers, ctx_len=ctx_len, page=a.kv_block, max_seqs=max_b,
                                 max_tokens=max(2048, max_b, a.prefill_tokens), graph_sizes=(1, 8, 64, B))
    runner, cache = eng.runner, eng.cache

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill: one 2,048-token prompt in one step ------------------------------------------------
    def prefill_once(tokens):
        rc = cache.admit("prefill")
        e0, e1 = ev(), ev()
        e0.record()
        runner.step([StepEntry(rc, tokens, [len(tokens) - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.release(rc)
        return e0.elapsed_time(e1)

    phases = set(a.phases.split(","))
    prefill = None
    if "prefill" in phases:
        ptoks = rng.integers(0, V, size=a.prefill_tokens).tolist()
        for _ in range(3):
            prefill_once(ptoks)
        pms = sorted(prefill_once(ptoks) for _ in range(5))[2]
        T = a.prefill_tokens
        pflops = 2.0 * T * nums["linear_params"] + layers * nums["attn_flops_per_layer"](T) + 2.0 * nums["head_params"]
        prefill = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(pflops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "tflop": round(pflops / 1e12, 3)}

    # ---- decode through the step function -----------------------------------------------------------
    def decode_run(batch: int, steps: int, warmup: int):
        rcs = [cache.admit(f"d{i}") for i in range(batch)]
        for rc in rcs:                                           # prompts, one request per step
            runner.step([StepEntry(rc, rng.integers(0, V, size=prompt_len).tolist(), [])])
        toks = rng.integers(0, V, size=(warmup + steps, batch))
        if batch == B and not checks:
            checks.update(graph_check(runner, cache, rcs, rng.integers(0, V, size=batch)))
        for s in range(warmup):
            runner.step([StepEntry(rc, [int(toks[s, i])], [0]) for i, rc in enumerate(rcs)])
        torch.cuda.synchronize()
        l0 = ops.launches
        e0, e1 = ev(), ev()
        e0.record()
        for s in range(warmup, warmup + steps):
            runner.step([StepEntry(rc, [int(toks[s, i])], [0]) for i, rc in enumerate(rcs)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = ops.launches - l0
        ctx_mid = prompt_len + warmup + steps / 2.0
        for rc in rcs:
            cache.release(rc)
        return ms, launches, ctx_mid

    steps, warmup = a.steps, max(3, a.warmup)
    checks: dict = {}
    with ClockSampler() as clocks:
        ms, launches, ctx_mid = decode_run(B, steps, warmup)
    value = B / (ms / 1e3)
    step_bytes = nums["weight_bytes_decode"] + B * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms / 1e3) / 1e9
    points = {}
    if "points" in phases:
        for b in (1, 64):
            pms_, _, _ = decode_run(b, min(steps, 64), 3)
            points[f"decode_b{b}"] = round(b / (pms_ / 1e3), 1)

    # ---- end to end: LLMEngine.step with scheduler and sampler, host tokens in and out ----------------
    e2e = None
    if "e2e" in phases:
        prompts = [rng.integers(0, V, size=prompt_len).tolist() for _ in range(B)]
        params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + B + 8, ignore_eos=True)
        for i, p in enumerate(prompts):
            eng.add_request(f"e{i}", p, params)
        while any(r.num_uncomputed > 1 for r in eng.requests.values()) or len(eng.scheduler.waiting):
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(steps):
            n_tok += sum(len(o.delta_token_ids) for o in eng.step())
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        if n_tok != steps * B:
            raise RuntimeError(f"end-to-end run produced {n_tok} tokens in {steps} steps of {B} requests: a request "
                               "stopped early (bad logits?)")
        for rid in list(eng.requests):
            eng.abort(rid)
        eng.step()
        # per step: the input arena (ids, positions, request index, starts, lengths, slots, rows, slot
        # map, block tables) goes up (greedy rows need no sampler parameters); tokens and flags come back
        width = runner.max_pages
        h2d = 4 * (4 * B + (B + 1) + 3 * B + B * width)
        d2h = (2 * B + ops.STATUS_WORDS) * 4
        e2e = {"value": round(n_tok / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(1e3 * e2e_s / steps, 4)}

    kernel_points = None
    if "kernels" in phases:
        kernel_points = per_kernel(ops, kw, B, prompt_len + warmup + steps // 2, a.kv_block, a.prefill_tokens, pk)
    if "points" in phases and a.kv_block != 64:
        # the same decode step with pages of 64 tokens (one TMA box of the attention kernels a page)
        model = runner.model
        del eng, runner, cache
        torch.cuda.empty_cache()
        eng = build_engine_on_device(a.model, layers, ctx_len=ctx_len, page=64, max_seqs=B, max_tokens=max(2048, B),
                                     graph_sizes=(B,), model=model)
        runner, cache = eng.runner, eng.cache
        pms_, _, _ = decode_run(B, min(steps, 64), 3)
        points[f"decode_b{B}_page64"] = round(B / (pms_ / 1e3), 1)
    mixed = None
    if "mixed" in phases:
        del eng, runner, cache
        torch.cuda.empty_cache()
        try:
            mixed = run_mixed(a, pk)
        except Exception as e:                              # the 14B point must not take the headline down
            mixed = {"error": f"{type(e).__name__}: {str(e).splitlines()[0][:160] if str(e) else ''}"}

    return {
        "metric": metric_name(a),
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, N(0,0.02) random weights", "impl": "ours",
        "config": {"model": a.model, "layers": layers, "layers_of_model": kw["num_layers"],
                   "hidden": kw["hidden_size"], "heads": kw["num_heads"], "kv_heads": kw["num_kv_heads"],
                   "head_dim": kw["head_dim"], "intermediate": kw["intermediate_size"], "vocab": V,
                   "global_batch": B, "seq_len": ctx_len, "prompt_len": prompt_len, "new_tokens": warmup + steps,
                   "kv_block": a.kv_block, "parallelism": "single GPU", "cuda_graphs": True,
                   "l2": "inputs larger than L2 (weights %.2f GB per step)" % (nums["weight_bytes_decode"] / 1e9),
                   "peaks": pk_src},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "graph_check": checks,
        "kernels": kernel_points,
        "mixed": mixed,
    }


def per_kernel(ops, kw: dict, B: int, ctx: int, page: int, prefill_tokens: int, pk: dict) -> dict:
    """Each dominant kernel alone at the step's shapes: mean time per launch with CUDA events around a
    CUDA graph of launches that rotate over enough copies of the weights (or caches) that they come from
    DRAM, the bytes (or FLOPs) the launch must move, and that rate over the measured peak (copy bandwidth;
    burst cuBLAS rate for the prompt attention, which is timed in isolation).  Inside a step the same
    kernels overlap their neighbours through programmatic dependent launch, so these times do not add up
    to the step; they say how far each is from its own roofline."""
    import torch

    from turingserve_b200 import kernels
    from turingserve_b200.engine.batch import streaming_decode

    h, I, H, KVH, D, V = (kw["hidden_size"], kw["intermediate_size"], kw["num_heads"], kw["num_kv_heads"],
                          kw["head_dim"], kw["vocab_size"])
    dev, bf = "cuda", torch.bfloat16
    out: dict = {"method": "CUDA events around a graph of rotating launches, each kernel alone"}

    def timed_graph(fn, copies: int) -> float:
        for i in range(copies):
            fn(i)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(copies):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * copies) * 1e3            # us per launch

    def record(name: str, us: float, nbytes: float = 0.0, flops: float = 0.0) -> None:
        r = {"us": round(us, 2)}
        if nbytes:
            r["GBps"] = round(nbytes / us / 1e3, 1)
            r["frac_hbm"] = round(nbytes / us / 1e3 / pk["hbm_gbs"], 4)
        if flops:
            r["TFLOPs"] = round(flops / us / 1e6, 1)
            r["frac_bf16"] = round(flops / us / 1e6 / pk["bf16_tflops"], 4)
        out[name] = r

    def weights(n: int, k: int):
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        return [torch.randn(n, k, device=dev, dtype=bf) * 0.02 for _ in range(copies)]

    x = torch.randn(B, h, device=dev, dtype=bf)
    positions = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    half = D // 2
    cos, sin = torch.ones(ctx + 8, half, device=dev), torch.zeros(ctx + 8, half, device=dev)
    slots = torch.full((B,), -1, dtype=torch.int32, device=dev)
    # K3: q/k/v product with bias, rotation and cache write (slots -1: nothing is written)
    nqkv = (H + 2 * KVH) * D
    ws, bias = weights(nqkv, h), torch.zeros(nqkv, device=dev, dtype=bf)
    qkv = torch.empty(B, nqkv, device=dev, dtype=bf)
    kc1 = torch.zeros(2, KVH, page, D, device=dev, dtype=bf)
    us = timed_graph(lambda i: ops.qkv_rope(qkv, x, ws[i % len(ws)], bias, positions, cos, sin, H, KVH, D, D, kc1, kc1,
                                            slots, page), len(ws))
    record("qkv_rope", us, nqkv * h * 2)
    del ws
    # K7, K10: output and down projections as the step runs them: a few tokens add themselves to the residual
    # rows (their K splits summed on chip), more leave partial sums for the norm kernel
    resid = torch.randn(B, h, device=dev, dtype=bf)
    for name, n, k in (("o_proj", h, H * D), ("down_proj", h, I)):
        ws = weights(n, k)
        xin = torch.randn(B, k, device=dev, dtype=bf) * 0.02
        o = torch.empty(B, n, device=dev, dtype=bf)

        def product(i):
            p = ops.linear(o, xin, ws[i % len(ws)], None, may_defer=True)
            if isinstance(p, kernels.LazyProduct) and not ops._into_residual(p, resid):
                ops._settle(p)

        record(name, timed_graph(product, len(ws)), n * k * 2)
        del ws
    # K8: gate/up product with the activation in its epilogue
    ws = weights(2 * I, h)
    act = torch.empty(B, I, device=dev, dtype=bf)
    group = 64 if I % 64 == 0 else 0
    record("gate_up_silu", timed_graph(lambda i: ops.gated_linear(act, x, ws[i % len(ws)], None, group), len(ws)), 2 * I * h * 2)
    del ws
    # K11: output head, 32-bit logits
    ws = weights(V, h)
    logits = torch.empty(B, V, device=dev, dtype=torch.float32)
    record("lm_head", timed_graph(lambda i: ops.linear(logits, x, ws[i % len(ws)], None), len(ws)), V * h * 2)
    del ws
    torch.cuda.empty_cache()

    class Step:
        pass

    def caches(batch: int, tokens: int, copies: int):
        per = -(-tokens // page)
        pages = batch * per + 1
        kv = [(torch.randn(pages, KVH, page, D, device=dev, dtype=bf), torch.randn(pages, KVH, page, D, device=dev, dtype=bf))
              for _ in range(copies)]
        table = (torch.randperm(pages - 1, device=dev).to(torch.int32) + 1).view(batch, per)
        return kv, table

    # K5: decode attention over the cache
    kv_bytes = B * (ctx + 1) * KVH * D * 2 * 2
    copies = max(2, min(28, int(300e6 // kv_bytes) + 1))
    kv, table = caches(B, ctx + 1, copies)
    st = Step()
    st.q_start = torch.arange(B + 1, dtype=torch.int32, device=dev)
    st.seq_lens = torch.full((B,), ctx + 1, dtype=torch.int32, device=dev)
    st.num_requests, st.max_q_len, st.max_seq_len, st.num_decode = B, 1, max(4096, ctx + 1), B
    st.streaming_decode = streaming_decode(B, ctx + 1)
    ao = torch.empty(B, H * D, device=dev, dtype=bf)
    record("decode_attention", timed_graph(lambda i: ops.attention(ao, qkv, kv[i % copies][0], kv[i % copies][1], table, st,
                                                                   H, KVH, D, page, D ** -0.5, None), copies), kv_bytes)
    del kv
    # K6: prompt attention, one prompt
    T = prefill_tokens
    kv, table = caches(1, T, 4)
    pq = torch.randn(T, nqkv, device=dev, dtype=bf)
    st = Step()
    st.q_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
    st.seq_lens = torch.tensor([T], dtype=torch.int32, device=dev)
    st.num_requests, st.max_q_len, st.max_seq_len, st.num_decode, st.streaming_decode = 1, T, T, 0, False
    po = torch.empty(T, H * D, device=dev, dtype=bf)
    # pages shorter than a tile of 64 keys are fetched as one box where they lie one after the other
    # in the pool (a fresh pool hands them out so) and page by page where they do not
    in_order = torch.arange(1, table.numel() + 1, dtype=torch.int32, device=dev).view_as(table)
    for name, tab in (("prefill_attention", in_order), ("prefill_attention_shuffled_pages", table)):
        record(name, timed_graph(lambda i: ops.attention(po, pq, kv[i % 4][0], kv[i % 4][1], tab, st, H, KVH, D,
                                                         page, D ** -0.5, None), 4), flops=2.0 * T * T * D * H)
    return out


def run_mixed(a, pk: dict) -> dict:
    """The Qwen2.5-14B shape under a mixed step: 32 requests decode at about 2,048 tokens of context
    while a 2,048-token prompt arrives in portions of 512 (four steps a prompt).  Times the steps with
    CUDA events through the step function, and the same through ``LLMEngine.step`` with its scheduler
    (token budget 544: the decodes first, then the portion)."""
    import numpy as np
    import torch

    from turingserve_b200 import SamplingParams
    from turingserve_b200.engine.batch import StepEntry

    shape, nd, plen, chunk, ctx_len = "qwen2.5-14b", 32, 2048, 512, 4096
    kw = SHAPES[shape]
    layers = kw["num_layers"]
    V = kw["vocab_size"]
    rng = np.random.default_rng(1)
    # (steps of 32 decoding requests beside a 512-token portion are one captured graph, as in serving)
    eng = build_engine_on_device(shape, layers, ctx_len=ctx_len, page=a.kv_block, max_seqs=nd + 2, max_tokens=nd + chunk,
                                 graph_sizes=(nd,))
    runner, cache = eng.runner, eng.cache
    rcs = [cache.admit(f"d{i}") for i in range(nd)]
    for rc in rcs:
        for at in range(0, plen, chunk):
            runner.step([StepEntry(rc, rng.integers(0, V, size=chunk).tolist(), [])])

    def prompt_round(tag: str) -> float:
        rc = cache.admit(tag)
        ptoks = rng.integers(0, V, size=plen).tolist()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for at in range(0, plen, chunk):
            entries = [StepEntry(r, [int(rng.integers(0, V))], [0]) for r in rcs]
            entries.append(StepEntry(rc, ptoks[at:at + chunk], [chunk - 1] if at + chunk == plen else []))
            runner.step(entries)
        e1.record()
        torch.cuda.synchronize()
        cache.release(rc)
        return e0.elapsed_time(e1) / (plen // chunk)

    prompt_round("w0")
    prompt_round("w1")
    ms = sorted(prompt_round(f"p{i}") for i in range(3))[1]
    for rc in rcs:
        cache.release(rc)
    # the same through the engine: 32 running requests, prompts arriving one after the other
    # (while the later prompts arrive in portions the earlier requests already decode: a budget that lasts)
    params = SamplingParams(temperature=0.0, max_tokens=1024, ignore_eos=True)
    for i in range(nd):
        eng.add_request(f"e{i}", rng.integers(0, V, size=plen).tolist(), params)
    while any(r.num_uncomputed > 1 for r in eng.requests.values()) or len(eng.scheduler.waiting):
        eng.step()
    eng.add_request("x0", rng.integers(0, V, size=plen).tolist(), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    for _ in range(4):
        eng.step()
    eng.add_request("x1", rng.integers(0, V, size=plen).tolist(), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(4):
        n_tok += sum(len(o.delta_token_ids) for o in eng.step())
    torch.cuda.synchronize()
    wall_ms = 1e3 * (time.perf_counter() - t0) / 4
    if n_tok < 4 * nd:
        raise RuntimeError(f"the mixed run through the engine produced {n_tok} tokens in 4 steps of {nd} decoding requests")
    for rid in list(eng.requests):
        eng.abort(rid)
    eng.step()
    nums = model_numbers(kw, layers)
    flops = 2.0 * (nd + chunk) * (nums["linear_params"] + 0) + 2.0 * (nd + 1) * nums["head_params"]
    return {"model": shape, "layers": layers, "decodes": nd, "prompt_tokens": plen, "portion": chunk,
            "ms_per_step": round(ms, 3), "tok_per_s": round((nd + chunk) / (ms / 1e3), 1),
            "e2e_ms_per_step": round(wall_ms, 3), "e2e_tokens_out": n_tok,
            "frac_bf16_products": round(flops / (ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}


class _StubTokenizer:
    """The reference's engine wants a tokenizer object; token ids go in and out, text is unused."""

    def decode(self, ids, skip_special_tokens=True):
        return ""


def run_reference(a) -> dict:
    """The unmodified reference from baseline/_ref through its own ``build_engine`` /
    ``LLMEngine.step``: float16 (it has no bfloat16), Triton kernels, CUDA graphs, same workload."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "turingserve")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed"}
    sys.path.insert(0, ref)
    import numpy as np
    import torch

    kw = SHAPES[a.model]
    layers = a.layers or kw["num_layers"]
    B, prompt_len, ctx_len = a.batch, a.prompt_len, a.context
    rng = np.random.default_rng(0)
    try:
        from turingserve.config import EngineConfig as RefConfig
        from turingserve.engine.builder import build_engine
        from turingserve.engine.sampling_params import SamplingParams as RefParams
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_model(a.model, layers, tmp)
            cfg = RefConfig(model=folder, dtype="float16", device="cuda", kernels="triton", max_model_len=ctx_len,
                            num_blocks=B * (-(-ctx_len // 16)) + 64, max_num_seqs=B, max_num_batched_tokens=2048,
                            cuda_graphs=True, graph_batch_sizes=(B,), prefix_caching=False, autopilot="off",
                            log_level="warning")
            eng = build_engine(cfg, tokenizer=_StubTokenizer())
        steps, warmup = a.steps, max(3, a.warmup)
        params = RefParams(temperature=0.0, max_tokens=warmup + steps + B + 8, ignore_eos=True)
        for i in range(B):
            eng.add_request(f"r{i}", rng.integers(0, kw["vocab_size"], size=prompt_len).tolist(), params)
        while eng.scheduler.waiting or any(s.num_uncomputed > 1 for s in eng.scheduler.running):
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        with ClockSampler() as clocks:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            n_tok = 0
            for _ in range(steps):
                n_tok += sum(len(o.delta_token_ids) for o in eng.step())
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1) / steps
        # per step its input builder copies ids, positions, slots and sample rows (int64), query starts and
        # lengths (int32), the block table at its live width, and the all-greedy flag; tokens and bad flags
        # (int64) and that flag's answer come back (turingserve/runner/input_builder.py:138-144,
        # turingserve/sampling/sampler.py:88-89,105-106)
        width = -(-(prompt_len + warmup + steps) // 16)
        h2d = 8 * 4 * B + 4 * (B + 1) + 4 * B + 4 * B * width + B
        d2h = 2 * 8 * B + 1
        return {"metric": metric_name(a),
                "value": round(n_tok / (ms * steps / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
                "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "fp16", "data": "synthetic: uniform random token ids, N(0,0.02) random weights",
                "impl": "reference",
                "config": {"model": a.model, "layers": layers, "global_batch": B, "seq_len": ctx_len,
                           "prompt_len": prompt_len, "parallelism": "single GPU", "cuda_graphs": True,
                           "kernels": "triton"},
                "clocks": clocks.summary(),
                "e2e": {"value": round(n_tok / wall, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h}}
    except Exception as e:                                   # the reference targets Turing + torch 2.6/triton 3.2
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e).splitlines()[0][:200] if str(e) else ''}"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen2.5-1.5b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--kv-block", type=int, default=16, help="tokens per cache page (the reference's 16)")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--phases", default="prefill,decode,points,e2e,kernels,mixed",
                    help="which measurements to run (decode always runs); fewer for a profiler capture")
    a = ap.parse_args()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    out = run_reference(a) if a.impl == "reference" else run_ours(a)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
