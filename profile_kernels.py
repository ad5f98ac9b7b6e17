#!/usr/bin/env python3
"""Single-kernel workloads at the layer sizes of one of bench.py's model shapes (--model), small
enough for a profiler capture that ends by itself (a few hundred MB on the device, a few dozen
launches), and the kernel-by-kernel timeline of one captured decode step.

    python profile_kernels.py decode_attention [--model qwen2.5-1.5b] [--batch 8] [--context 2048] [--page 16] [--graph]
    python profile_kernels.py prefill_attention [--tokens 2048] [--prefix 0] [--page 16] [--in-order]
    python profile_kernels.py timeline --prefill 2048
    python profile_kernels.py gemm [--tokens 8] [--n 17920] [--k 1536] [--mode auto|tc|library] [--gated|--resid] [--pair] [--qkv] [--graph]
    python profile_kernels.py timeline [--batch 8] [--context 2048] [--layers 0] [--page 16]
    python profile_kernels.py fused_step [--batch 8] [--context 2048] [--layers 4] [--page 16]

Each prints the launches it made and, timed with CUDA events, the mean time per launch.
"""

from __future__ import annotations

import argparse
import dataclasses
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from bench import SHAPES                                    # noqa: E402
from turingserve_b200 import kernels                        # noqa: E402
from turingserve_b200.engine.batch import streaming_decode  # noqa: E402

PAGE = 16
H = KVH = D = LAYERS = 0            # set from --model in main()
SHAPE: dict = {}


@dataclasses.dataclass
class Step:
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    num_requests: int
    max_q_len: int
    max_seq_len: int
    num_decode: int
    streaming_decode: bool | None = None     # which decode kernel, as the engine decides it from the live contexts


def timed(fn, n: int) -> float:
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def paged(batch: int, tokens_per_request: int, layers: int, PAGE: int = PAGE):
    per = -(-tokens_per_request // PAGE)
    pages = batch * per + 1
    caches = [(torch.randn(pages, KVH, PAGE, D, device="cuda", dtype=torch.bfloat16),
               torch.randn(pages, KVH, PAGE, D, device="cuda", dtype=torch.bfloat16)) for _ in range(layers)]
    table = (torch.randperm(pages - 1, device="cuda").to(torch.int32) + 1).view(batch, per)
    return caches, table


def decode_attention(a) -> None:
    ops = kernels.ops()
    B, ctx = a.batch, a.context
    kv = B * (ctx + 1) * KVH * D * 2 * 2
    layers = max(2, min(LAYERS, int(500e6 // kv) + 1))            # rotate caches so that keys come from DRAM
    PAGE = a.page
    caches, table = paged(B, ctx + 1, layers, PAGE)
    qkv = torch.randn(B, (H + 2 * KVH) * D, device="cuda", dtype=torch.bfloat16)
    longest = max(4096, ctx + 1)
    step = Step(torch.arange(B + 1, dtype=torch.int32, device="cuda"),
                torch.full((B,), ctx + 1, dtype=torch.int32, device="cuda"), B, 1, longest, B,
                streaming_decode(B, ctx + 1))
    out = torch.empty(B, H * D, device="cuda", dtype=torch.bfloat16)
    if a.splits:                                                   # instead of the rule's own count
        ops.decode_splits = lambda *args: a.splits
        ops.decode_splits_tma = lambda *args: a.splits

    def f(i):
        kc, vc = caches[i % layers]
        ops.attention(out, qkv, kc, vc, table, step, H, KVH, D, PAGE, D ** -0.5, None)

    for i in range(layers):
        f(i)
    if a.graph:                                                    # as inside a captured decode step: no launch gaps
        reps = max(layers, 24 // layers * layers)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps):
                f(i)
        g.replay()
        us = timed(lambda i: g.replay(), 3) / reps
    else:
        us = timed(f, max(3 * layers, 24))
    print(f"decode_attention batch {B} context {ctx} page {PAGE}{' (graph)' if a.graph else ''}: "
          f"{us:.2f} us per launch, {kv / us / 1e6:.2f} TB/s of keys and values")


def prefill_attention(a) -> None:
    ops = kernels.ops()
    T, S = a.tokens, a.prefix + a.tokens                          # a portion of T tokens after `prefix` cached ones
    PAGE = a.page
    caches, table = paged(1, S, 4, PAGE)
    if a.in_order:                                                 # as a fresh pool hands its pages out
        table = torch.arange(1, table.numel() + 1, dtype=torch.int32, device="cuda").view_as(table)
    qkv = torch.randn(T, (H + 2 * KVH) * D, device="cuda", dtype=torch.bfloat16)
    step = Step(torch.tensor([0, T], dtype=torch.int32, device="cuda"),
                torch.tensor([S], dtype=torch.int32, device="cuda"), 1, T, S, 0)
    out = torch.empty(T, H * D, device="cuda", dtype=torch.bfloat16)

    def f(i):
        kc, vc = caches[i % 4]
        ops.attention(out, qkv, kc, vc, table, step, H, KVH, D, PAGE, D ** -0.5, None)

    for i in range(4):
        f(i)
    us = timed(f, 12)
    flops = 4.0 * D * H * (T * a.prefix + T * (T + 1) / 2)         # scores and values over the keys each token sees
    print(f"prefill_attention {T} tokens after {a.prefix} page {PAGE}{' in order' if a.in_order else ' shuffled'}: "
          f"{us:.1f} us per launch, {flops / us / 1e6:.1f} TFLOP/s")


def gemm(a) -> None:
    ops = kernels.ops()
    ops.gemm_mode = a.mode
    M, N, K = a.tokens, a.n, a.k
    copies = max(2, int(400e6 // (N * K * 2)) + 1)               # rotate weights so they come from DRAM
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

    act = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
    resid = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)

    if a.qkv:        # the q/k/v product of the model's heads with bias, rotation and cache write in its epilogue (pairs of SMs)
        N = (H + 2 * KVH) * D
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        bias = torch.randn(N, device="cuda", dtype=torch.bfloat16) * 0.1
        freqs = torch.outer(torch.arange(M + 1).float(), 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D)))
        cos, sin = freqs.cos().cuda().contiguous(), freqs.sin().cuda().contiguous()
        pos = torch.arange(M, dtype=torch.int32, device="cuda")
        slots = pos + PAGE
        kc = torch.zeros((M // PAGE + 2, KVH, PAGE, D), device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)

    def f(i):
        if a.qkv:
            rc = ops.lib.ts_linear_pair_qkv(out.data_ptr(), x.data_ptr(), ws[i % copies].data_ptr(), bias.data_ptr(), pos.data_ptr(),
                                            cos.data_ptr(), sin.data_ptr(), slots.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                            M, H, KVH, D, PAGE, K, None)
            if rc:
                raise SystemExit(f"ts_linear_pair_qkv refused: {rc}")
        elif a.pair:                                              # the many-row kernel on pairs of SMs, whatever the cost rule says
            if not ops.linear_pair(act if a.gated else out, x, ws[i % copies], None, ops.PAIR_GATED if a.gated else ops.PAIR_PLAIN):
                raise SystemExit("the pair kernel does not take this shape")
        elif a.gated:                                             # block-interleaved gate/up rows, SiLU*mul in the epilogue
            ops.gated_linear(act, x, ws[i % copies], None, 64)
        elif a.resid:                                             # the product adds itself to the residual rows
            p = ops.linear(out, x, ws[i % copies], None, may_defer=True)
            if not (isinstance(p, kernels.LazyProduct) and ops._into_residual(p, resid)):
                raise SystemExit("this shape does not take the product that adds itself to the residual")
        else:
            ops.linear(out, x, ws[i % copies], None)

    for i in range(copies):
        f(i)
    if a.graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(copies):
                f(i)
        g.replay()
        us = timed(lambda i: g.replay(), 5) / copies
    else:
        us = timed(f, 3 * copies)
    print(f"gemm {M}x{N}x{K} mode {a.mode}{' on pairs of SMs' if a.pair else ''}{' gated' if a.gated else ''}{' into the residual' if a.resid else ''}{' (graph)' if a.graph else ''}: {us:.2f} us per launch, "
          f"{N * K * 2 / us / 1e6:.2f} TB/s of weights, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")


def timeline(a) -> None:
    """Where a captured decode step's time goes: every kernel of one graph replay with the moment
    it ended (CUPTI through torch.profiler), and per kernel the increment of the end time over the
    kernel that ended before it.  With programmatic dependent launch kernels start long before
    their predecessor ends, so durations overlap; the end-time increments add up to the step."""
    import collections
    import re
    import tempfile

    import numpy as np
    from torch.profiler import ProfilerActivity, profile

    from turingserve_b200 import EngineConfig, LLMEngine, SamplingParams
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.weights.random_init import write_random_model

    if a.prefill:
        return prefill_timeline(a)
    B, ctx = a.batch, a.context
    with tempfile.TemporaryDirectory() as tmp:
        kw = dict(SHAPE)
        kw["num_layers"] = a.layers or LAYERS
        write_random_model(tmp, make_config(**kw), seed=0)
        eng = LLMEngine.from_config(EngineConfig(model=tmp, dtype="bfloat16", max_model_len=2 * ctx, block_size=a.page,
                                                 num_blocks=B * (2 * ctx // a.page) + 8, max_num_seqs=B,
                                                 max_num_batched_tokens=max(2048, B), graph_batch_sizes=(B,), watermark=0.0))
    rng = np.random.default_rng(0)
    params = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True)
    for i in range(B):
        eng.add_request(f"r{i}", rng.integers(0, SHAPE["vocab_size"], size=ctx).tolist(), params)
    while any(r.num_uncomputed > 1 for r in eng.requests.values()) or len(eng.scheduler.waiting):
        eng.step()
    for _ in range(8):
        eng.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(5):
            eng.step()
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                 key=lambda e: e.time_range.start)
    firsts = [i for i, e in enumerate(evs) if "embedding_kernel" in e.name]
    step = sorted(evs[firsts[2]:firsts[3]], key=lambda e: e.time_range.end)

    def short(name: str) -> str:
        m = re.search(r"(gemm_tc_kernel<[^>]*>|attention_\w+_kernel|reduce_rmsnorm_kernel|rope_kv_write\w*|rmsnorm\w*|"
                      r"silu_mul\w*|embedding_kernel|gather_rows_kernel|feed_tokens_kernel|sample\w*|splitk_reduce_kernel|"
                      r"Memcpy \w+|nvjet\w*)", name)
        return m.group(1) if m else name[:50]

    t0 = min(e.time_range.start for e in step)
    prev, share, rows = t0, collections.OrderedDict(), []
    for e in step:
        d = e.time_range.end - prev
        prev = e.time_range.end
        n = short(e.name)
        share.setdefault(n, [0, 0.0])
        share[n][0] += 1
        share[n][1] += d
        rows.append((e.time_range.start - t0, e.time_range.end - t0, d, n))
    print(f"timeline batch {B} context {ctx} layers {a.layers or LAYERS} page {a.page}: one step = {prev - t0:.1f} us, {len(step)} kernels and copies")
    print("end-time increments, summed per kernel:")
    for n, (c, d) in sorted(share.items(), key=lambda kv: -kv[1][1]):
        print(f"  {d:8.1f} us  {c:4d} x {d / c:6.2f}  {n}")
    print("second layer (start, end, increment):")
    per_layer = (len(step) - 10) // max(a.layers or LAYERS, 1)
    for r in rows[3 + per_layer: 3 + 2 * per_layer]:
        print(f"  {r[0]:8.2f} {r[1]:8.2f}  +{r[2]:5.2f}  {r[3]}")


def prefill_timeline(a) -> None:
    """One prompt of ``--prefill`` tokens in one step, launched kernel by kernel: the duration of every
    kernel (CUPTI through torch.profiler), summed per kernel, and the layers' share of the step.  The
    profiler slows the host, so the step's own time comes from CUDA events without it."""
    import collections
    import re

    import numpy as np
    from torch.profiler import ProfilerActivity, profile

    import bench
    from turingserve_b200.engine.batch import StepEntry

    T, L = a.prefill, a.layers or LAYERS
    eng = bench.build_engine_on_device(a.model, L, ctx_len=T + 64, page=a.page, max_seqs=8, max_tokens=T, graph_sizes=())
    runner, cache = eng.runner, eng.cache
    toks = np.random.default_rng(0).integers(0, SHAPE["vocab_size"], size=T).tolist()

    def once(i=0):
        rc = cache.admit("p")
        runner.step([StepEntry(rc, toks, [T - 1])])
        cache.release(rc)

    for _ in range(4):
        once()
    us = timed(once, 5)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        once()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]

    def short(name: str) -> str:
        m = re.search(r"(gemm_pair_kernel<[^>]*>|gemm_tc_kernel<[^>]*>|attention_\w+_kernel|rope_kv_write\w*|rmsnorm\w*|"
                      r"silu_mul\w*|embedding_kernel|gather_rows_kernel|Memcpy \w+|nvjet\w*)", name)
        return m.group(1) if m else name[:50]

    share = collections.OrderedDict()
    for e in evs:
        d = e.time_range.end - e.time_range.start
        share.setdefault(short(e.name), [0, 0.0])
        share[short(e.name)][0] += 1
        share[short(e.name)][1] += d
    total = sum(d for _, d in share.values())
    print(f"prefill timeline {T} tokens layers {L} page {a.page}: one step = {us:.1f} us (CUDA events), "
          f"kernel durations add up to {total:.1f} us, {len(evs)} kernels and copies")
    for n, (c, d) in sorted(share.items(), key=lambda kv: -kv[1][1]):
        print(f"  {d:8.1f} us  {c:4d} x {d / c:7.2f}  {n}")


def fused_step(a) -> None:
    """The whole decode step as one persistent kernel (off by default in the engine), phase by phase:
    the kernel stamps the clock when a block arrives at a grid barrier and when it leaves it, so a
    phase's work (arrival minus the leave before) and its wait show per block.  Also times the same
    step as the chain of kernels, both eagerly launched, for comparison."""
    import numpy as np

    import bench
    from turingserve_b200.engine.batch import StepEntry
    from turingserve_b200.parts.fused_decode import FusedDecodeStep

    FusedDecodeStep.enabled = True
    B, ctx, L = a.batch, a.context, a.layers
    eng = bench.build_engine_on_device(a.model, L, ctx_len=2 * ctx, page=a.page, max_seqs=B, max_tokens=2048, graph_sizes=())
    runner, cache, ops = eng.runner, eng.cache, kernels.ops()
    fused = runner.fused
    if fused is None:
        raise SystemExit("the fused step does not take this model")
    rng = np.random.default_rng(0)
    V = SHAPE["vocab_size"]
    rcs = [cache.admit(f"d{i}") for i in range(B)]
    for rc in rcs:
        runner.step([StepEntry(rc, rng.integers(0, V, size=ctx).tolist(), [])])

    def step(i=0):
        runner.step([StepEntry(rc, [int(rng.integers(0, V))], [0]) for rc in rcs])

    for use in (False, True):
        ops.use_fused_step = use
        for _ in range(3):
            step()
        print(f"fused_step batch {B} context {ctx} layers {L} page {a.page}: {'one kernel' if use else 'chain of kernels'} "
              f"{timed(step, 10):.1f} us a step (host work of an eager step included)")
    assert ops.lib.ts_decode_step_status() == 0
    nbar = 5 * L + 1
    fused.trace = torch.zeros((fused.blocks, nbar + 1, 8), dtype=torch.int64, device="cuda")
    step()
    torch.cuda.synchronize()
    t = fused.trace.cpu().numpy().astype(np.float64)[:, :nbar]
    fused.trace = None
    arrive, leave = t[:, :, 0], t[:, :, 1]
    mhz = 1965                                                     # the clock a decode step runs at (it is far from the power cap)
    work = arrive[:, 1:] - leave[:, :-1]
    wait = (leave - arrive)[:, 1:]
    length = leave[:, 1:].max(0) - leave[:, :-1].max(0)
    print(f"phases (us at {mhz} MHz, mean over layers 1..{L - 1}): work of the slowest / median block, wait of the last / median block at the barrier, length")
    for j, name in enumerate(("q/k/v", "attention", "output", "gate/up", "down")):
        cols = [5 * l + j for l in range(1, L)]
        print(f"  {name:10s} work {work[:, cols].max(0).mean() / mhz:6.2f} / {np.median(work[:, cols], 0).mean() / mhz:6.2f}   "
              f"wait {wait[:, cols].min(0).mean() / mhz:5.2f} / {np.median(wait[:, cols], 0).mean() / mhz:5.2f}   "
              f"length {length[cols].mean() / mhz:6.2f}")
    print(f"  a layer: {(leave[:, 5 * L].max() - leave[:, 5].max()) / mhz / (L - 1):.2f} us")


def main() -> int:
    ap = argparse.ArgumentParser(prog="python profile_kernels.py")
    ap.add_argument("--model", default="qwen2.5-1.5b", choices=sorted(SHAPES), help="whose layer sizes to use")
    sub = ap.add_subparsers(dest="workload", required=True)
    s = sub.add_parser("decode_attention")
    s.add_argument("--batch", type=int, default=8)
    s.add_argument("--context", type=int, default=2048)
    s.add_argument("--page", type=int, default=PAGE)
    s.add_argument("--graph", action="store_true", help="time the launches inside one CUDA graph")
    s.add_argument("--splits", type=int, default=0, help="key splits per request (0: the rule's count)")
    s = sub.add_parser("prefill_attention")
    s.add_argument("--tokens", type=int, default=2048)
    s.add_argument("--page", type=int, default=PAGE)
    s.add_argument("--prefix", type=int, default=0, help="tokens of the request already in the cache")
    s.add_argument("--in-order", action="store_true", help="page ids one after the other instead of shuffled")
    s = sub.add_parser("gemm")
    s.add_argument("--tokens", type=int, default=8)
    s.add_argument("--n", type=int, default=17920)
    s.add_argument("--k", type=int, default=1536)
    s.add_argument("--mode", default="auto", choices=["auto", "tc", "library"])
    s.add_argument("--gated", action="store_true", help="gate/up product with the activation in its epilogue")
    s.add_argument("--pair", action="store_true", help="the many-row kernel whose tiles are computed by two SMs together")
    s.add_argument("--qkv", action="store_true", help="that kernel as the q/k/v product of the model's heads: bias, rotation, cache write (--n is ignored)")
    s.add_argument("--resid", action="store_true", help="the product that sums its splits on chip and adds itself to residual rows")
    s.add_argument("--graph", action="store_true", help="time the launches inside one CUDA graph")
    s = sub.add_parser("timeline")
    s.add_argument("--batch", type=int, default=8)
    s.add_argument("--context", type=int, default=2048)
    s.add_argument("--layers", type=int, default=0, help="0: as many as the model has")
    s.add_argument("--page", type=int, default=PAGE)
    s.add_argument("--prefill", type=int, default=0, help="instead: one prompt of this many tokens in one step")
    s = sub.add_parser("fused_step")
    s.add_argument("--batch", type=int, default=8)
    s.add_argument("--context", type=int, default=2048)
    s.add_argument("--layers", type=int, default=4)
    s.add_argument("--page", type=int, default=PAGE)
    a = ap.parse_args()
    global H, KVH, D, LAYERS, SHAPE
    SHAPE = SHAPES[a.model]
    H, KVH, D, LAYERS = SHAPE["num_heads"], SHAPE["num_kv_heads"], SHAPE["head_dim"], SHAPE["num_layers"]
    {"decode_attention": decode_attention, "prefill_attention": prefill_attention, "gemm": gemm,
     "timeline": timeline, "fused_step": fused_step}[a.workload](a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
