"""Engine options and the command-line parser.

Option names and meanings follow the reference's ``EngineConfig`` / ``build_parser``
(turingserve/config.py:10-47,107-156) for every option this engine has; the server, speculative,
quantization and autopilot flags of the reference have no counterpart here.  Differences:
``--dtype`` is bfloat16|float32 (the reference: float16|float32, config.py:56-60), and
``--block-size`` is free and defaults to 64 (the reference fixes 16, config.py:74-75): a page of 64
tokens is one TMA box of the attention kernels, which a page of 16 needs four of.
"""

from __future__ import annotations

import argparse
from dataclasses import dataclass, fields

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineConfig:
    model: str = ""
    dtype: str = "bfloat16"
    device: str = "cuda"
    max_model_len: int | None = None          # None: the model's max_position_embeddings, at most 4096
    block_size: int = 64
    num_blocks: int | None = None             # pages per cache group (None: from free memory)
    gpu_memory_utilization: float = 0.85
    max_num_seqs: int = 128
    max_num_batched_tokens: int = 2048
    watermark: float = 0.01
    cuda_graphs: bool = True
    graph_batch_sizes: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128)
    # Steps of decoding requests beside one prompt portion are captured too where the token budget is
    # at most this: launched kernel by kernel such a step costs the host about 3 ms whatever its size, more
    # than the GPU needs for a few hundred tokens.  The portion then has the budget less the (padded)
    # decoding rows.  0: never.
    graph_portion_budget: int = 1024
    # launch the next decode step before the host has read the current step's tokens (they are fed
    # back on the device); a request that stops on a token then runs one step in vain
    async_decode: bool = True
    seed: int = 0

    @property
    def torch_dtype(self):
        import torch

        return {"bfloat16": torch.bfloat16, "float32": torch.float32}[self.dtype]

    def graph_portion_sizes(self) -> tuple[int, ...]:
        """Lengths of the prompt portions whose steps are captured: the token budget less each captured
        number of decoding rows (and less none)."""
        budget = self.max_num_batched_tokens
        if not self.cuda_graphs or budget > self.graph_portion_budget:
            return ()
        from turingserve_b200.engine.scheduler import Scheduler
        least = Scheduler.SMALLEST_CAPTURED_PORTION
        return tuple(sorted({budget - s for s in (0, *self.graph_batch_sizes) if budget - s >= least}))

    def resolve_max_model_len(self, max_position_embeddings: int) -> int:
        if self.max_model_len is None:
            return min(4096, max_position_embeddings)
        return self.max_model_len

    def validate(self, max_position_embeddings: int | None = None) -> None:
        """Same checks as turingserve/config.py:62-100, for the options kept."""
        def bad(msg: str):
            raise ValueError(msg)

        if not self.model:
            bad("--model is required")
        if self.dtype not in DTYPES:
            bad("--dtype must be bfloat16 or float32")
        if self.device != "cuda":
            bad("--device must be cuda (this engine has no CPU path)")
        if self.block_size < 1:
            bad("--block-size must be >= 1")
        if self.max_model_len is not None:
            if self.max_model_len < 1:
                bad("--max-model-len must be >= 1")
            if max_position_embeddings is not None and self.max_model_len > max_position_embeddings:
                bad(f"--max-model-len {self.max_model_len} exceeds the model's "
                    f"max_position_embeddings {max_position_embeddings}")
        if self.max_num_batched_tokens < 1:
            bad("--max-num-batched-tokens must be >= 1")
        if self.max_num_seqs < 1:
            bad("--max-num-seqs must be >= 1")
        if not 0.0 <= self.watermark < 1.0:
            bad("--watermark must be in [0, 1)")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            bad("--gpu-memory-utilization must be in (0, 1]")
        if self.num_blocks is not None and self.num_blocks < 2:
            bad("--num-blocks must be >= 2 (page 0 is the null page)")
        self.graph_batch_sizes = tuple(s for s in self.graph_batch_sizes if s <= self.max_num_seqs)

    def max_blocks_per_seq(self, max_model_len: int) -> int:
        return -(-max_model_len // self.block_size)


def add_engine_arguments(s: argparse.ArgumentParser) -> None:
    d = EngineConfig()
    s.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    s.add_argument("--dtype", default=d.dtype, choices=list(DTYPES))
    s.add_argument("--device", default=d.device, choices=["cuda"])
    s.add_argument("--max-model-len", type=int, default=None)
    s.add_argument("--block-size", type=int, default=d.block_size)
    s.add_argument("--num-blocks", type=int, default=None)
    s.add_argument("--gpu-memory-utilization", type=float, default=d.gpu_memory_utilization)
    s.add_argument("--max-num-seqs", type=int, default=d.max_num_seqs)
    s.add_argument("--max-num-batched-tokens", type=int, default=d.max_num_batched_tokens)
    s.add_argument("--watermark", type=float, default=d.watermark)
    g = s.add_mutually_exclusive_group()
    g.add_argument("--cuda-graphs", dest="cuda_graphs", action="store_true",
                   help="graph replay for pure-decode steps")
    g.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false")
    s.set_defaults(cuda_graphs=d.cuda_graphs)
    s.add_argument("--graph-batch-sizes", default=",".join(map(str, d.graph_batch_sizes)))
    s.add_argument("--graph-portion-budget", type=int, default=d.graph_portion_budget,
                   help="token budgets up to this also capture steps of decoding requests beside one prompt portion")
    g2 = s.add_mutually_exclusive_group()
    g2.add_argument("--async-decode", dest="async_decode", action="store_true",
                    help="launch the next decode step before reading this step's tokens")
    g2.add_argument("--no-async-decode", dest="async_decode", action="store_false")
    s.set_defaults(async_decode=d.async_decode)
    s.add_argument("--seed", type=int, default=d.seed)


def engine_config_from_namespace(ns: argparse.Namespace) -> EngineConfig:
    kw = {f.name: getattr(ns, f.name) for f in fields(EngineConfig) if hasattr(ns, f.name)}
    if isinstance(kw.get("graph_batch_sizes"), str):
        kw["graph_batch_sizes"] = tuple(int(x) for x in kw["graph_batch_sizes"].split(",") if x)
    return EngineConfig(**kw)
