"""Launches the split-key decode attention kernel the way a Qwen2.5-1.5B decode step does (batch 8,
context 2,048, 12 heads over 2 kv heads of 128, 28 layers' caches so that keys come from DRAM), for
a profiler capture.  Usage: python profiles/run_decode_attention.py [batch] [context] [rounds]"""
import dataclasses
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from turingserve_b200 import kernels  # noqa: E402

B = int(sys.argv[1]) if len(sys.argv) > 1 else 8
ctx = int(sys.argv[2]) if len(sys.argv) > 2 else 2048
rounds = int(sys.argv[3]) if len(sys.argv) > 3 else 3
H, KVH, D, page, layers = 12, 2, 128, 16, 28
ops = kernels.ops()
pages_per = -(-(ctx + 1) // page)
pages = B * pages_per + 1
caches = [(torch.randn(pages, KVH, page, D, device="cuda", dtype=torch.bfloat16),
           torch.randn(pages, KVH, page, D, device="cuda", dtype=torch.bfloat16)) for _ in range(layers)]
bt = (torch.randperm(pages - 1, device="cuda").to(torch.int32) + 1).view(B, pages_per)
qkv = torch.randn(B, (H + 2 * KVH) * D, device="cuda", dtype=torch.bfloat16)


@dataclasses.dataclass
class Step:
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    num_requests: int
    max_q_len: int
    max_seq_len: int
    num_decode: int


step = Step(torch.arange(B + 1, dtype=torch.int32, device="cuda"),
            torch.full((B,), ctx + 1, dtype=torch.int32, device="cuda"), B, 1, 4096, B)
out = torch.empty(B, H * D, device="cuda", dtype=torch.bfloat16)
for _ in range(rounds):
    for kc, vc in caches:
        ops.attention(out, qkv, kc, vc, bt, step, H, KVH, D, page, D ** -0.5, None)
torch.cuda.synchronize()
print("done", B, ctx, "splits", ops.decode_splits(B, KVH, 4096))
