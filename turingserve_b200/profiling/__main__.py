"""Single-kernel workloads at the sizes of a Qwen2.5-1.5B-shaped step, small enough for a profiler
capture that ends by itself (a few hundred MB on the device, a few dozen launches).

    python -m turingserve_b200.profiling decode_attention [--batch 8] [--context 2048] [--page 16] [--graph]
    python -m turingserve_b200.profiling prefill_attention [--tokens 2048] [--page 16]
    python -m turingserve_b200.profiling gemm [--tokens 8] [--n 17920] [--k 1536] [--mode auto|tc|library]

Each prints the launches it made and, timed with CUDA events, the mean time per launch.
"""

from __future__ import annotations

import argparse
import dataclasses

import torch

from turingserve_b200 import kernels

H, KVH, D, PAGE, LAYERS = 12, 2, 128, 16, 28


@dataclasses.dataclass
class Step:
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    num_requests: int
    max_q_len: int
    max_seq_len: int
    num_decode: int


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
                torch.full((B,), ctx + 1, dtype=torch.int32, device="cuda"), B, 1, longest, B)
    out = torch.empty(B, H * D, device="cuda", dtype=torch.bfloat16)

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
    T = a.tokens
    PAGE = a.page
    caches, table = paged(1, T, 4, PAGE)
    qkv = torch.randn(T, (H + 2 * KVH) * D, device="cuda", dtype=torch.bfloat16)
    step = Step(torch.tensor([0, T], dtype=torch.int32, device="cuda"),
                torch.tensor([T], dtype=torch.int32, device="cuda"), 1, T, T, 0)
    out = torch.empty(T, H * D, device="cuda", dtype=torch.bfloat16)

    def f(i):
        kc, vc = caches[i % 4]
        ops.attention(out, qkv, kc, vc, table, step, H, KVH, D, PAGE, D ** -0.5, None)

    for i in range(4):
        f(i)
    us = timed(f, 12)
    print(f"prefill_attention {T} tokens page {PAGE}: {us:.1f} us per launch, {2.0 * T * T * D * H / us / 1e6:.1f} TFLOP/s (causal)")


def gemm(a) -> None:
    ops = kernels.ops()
    ops.gemm_mode = a.mode
    M, N, K = a.tokens, a.n, a.k
    copies = max(2, int(400e6 // (N * K * 2)) + 1)               # rotate weights so they come from DRAM
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

    def f(i):
        ops.linear(out, x, ws[i % copies], None)

    for i in range(copies):
        f(i)
    us = timed(f, 3 * copies)
    print(f"gemm {M}x{N}x{K} mode {a.mode}: {us:.2f} us per launch, {N * K * 2 / us / 1e6:.2f} TB/s of weights, "
          f"{2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")


def main() -> int:
    ap = argparse.ArgumentParser(prog="python -m turingserve_b200.profiling")
    sub = ap.add_subparsers(dest="workload", required=True)
    s = sub.add_parser("decode_attention")
    s.add_argument("--batch", type=int, default=8)
    s.add_argument("--context", type=int, default=2048)
    s.add_argument("--page", type=int, default=PAGE)
    s.add_argument("--graph", action="store_true", help="time the launches inside one CUDA graph")
    s = sub.add_parser("prefill_attention")
    s.add_argument("--tokens", type=int, default=2048)
    s.add_argument("--page", type=int, default=PAGE)
    s = sub.add_parser("gemm")
    s.add_argument("--tokens", type=int, default=8)
    s.add_argument("--n", type=int, default=17920)
    s.add_argument("--k", type=int, default=1536)
    s.add_argument("--mode", default="auto", choices=["auto", "tc", "library"])
    a = ap.parse_args()
    {"decode_attention": decode_attention, "prefill_attention": prefill_attention, "gemm": gemm}[a.workload](a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
