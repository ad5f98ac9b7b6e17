#!/usr/bin/env python3
"""Benchmark: decode tokens/s (default batch 8), prefill tokens/s at 2,048 tokens and roofline
fractions for a Qwen2.5-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

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
    "qwen2.5-1.5b": dict(hidden_size=1536, intermediate_size=8960, num_layers=28, num_heads=12, num_kv_heads=2,
                         head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-7b": dict(hidden_size=3584, intermediate_size=18944, num_layers=28, num_heads=28, num_kv_heads=4,
                       head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=False, max_position_embeddings=32768),
}
SHAPE_NAMES = {"qwen2.5-1.5b": "Qwen2.5-1.5B", "qwen2.5-7b": "Qwen2.5-7B"}
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


def run_ours(a) -> dict:
    import numpy as np
    import torch

    from turingserve_b200 import EngineConfig, LLMEngine, SamplingParams, kernels
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

    with tempfile.TemporaryDirectory() as tmp:
        folder = make_model(a.model, layers, tmp)
        max_b = max(B, 64)
        pages = max_b * (-(-ctx_len // a.kv_block)) + 8
        eng = LLMEngine.from_config(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=ctx_len, block_size=a.kv_block, num_blocks=pages,
            max_num_seqs=max_b, max_num_batched_tokens=max(2048, max_b), graph_batch_sizes=(1, 8, 64, B),
            watermark=0.0))
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
        d2h = 2 * B * 4
        e2e = {"value": round(n_tok / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(1e3 * e2e_s / steps, 4)}

    return {
        "metric": f"decode tok/s at batch {B} ({SHAPE_NAMES[a.model]} shape, {prompt_len:,}-token prompts, bf16)",
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
    }


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
        return {"metric": f"decode tok/s at batch {B} ({SHAPE_NAMES[a.model]} shape, {prompt_len:,}-token prompts)",
                "value": round(n_tok / (ms * steps / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
                "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "fp16", "data": "synthetic: uniform random token ids, N(0,0.02) random weights",
                "impl": "reference",
                "config": {"model": a.model, "layers": layers, "global_batch": B, "seq_len": ctx_len,
                           "prompt_len": prompt_len, "parallelism": "single GPU", "cuda_graphs": True,
                           "kernels": "triton"},
                "clocks": clocks.summary(),
                "e2e": {"value": round(n_tok / wall, 1), "unit": "tok/s"}}
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
    ap.add_argument("--kv-block", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--phases", default="prefill,decode,points,e2e",
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
