"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and schedules nothing; it drives the same model, cache manager and step
function that generation uses.  The reference has no such tool; its tests hand-build
``BatchItem``s and call the runner with ``sample="all"``
(tests/correctness/test_paged_engine.py:46-63 of the reference).

Input: one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: ``<out>/<step>.f32`` (little-endian float32 [wanted, vocab]) for steps that want logits,
and a line ``done <step>`` on stdout after every step.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

from turingserve_b200.cache.manager import CacheManager
from turingserve_b200.engine.batch import StepEntry
from turingserve_b200.engine.runner import ModelRunner, run_needs
from turingserve_b200.weights.loader import load_model

MAX_LIVE = 4
ROUND_TO = 64


class Replayer:
    def __init__(self, model_dir: str, dtype: torch.dtype, max_tokens: int, device,
                 page_size: int = 64, max_step_tokens: int | None = None,
                 graph_batch_sizes: tuple[int, ...] = (), graph_portion_sizes: tuple[int, ...] = ()) -> None:
        """``graph_batch_sizes``: steps made of single tokens whose logits are wanted replay a captured
        CUDA graph of the smallest of these sizes that holds them, as generation does; empty: none.
        ``graph_portion_sizes``: so do steps of such tokens beside one prompt portion of one of these lengths
        of which the last logits, or none, are wanted."""
        if ROUND_TO % page_size:
            raise ValueError(f"page size {page_size} must divide {ROUND_TO}")
        self.model, self.cfg = load_model(model_dir, dtype, device)
        needs = run_needs(self.model)
        max_tokens = -(-max_tokens // ROUND_TO) * ROUND_TO
        num_pages = max_tokens // page_size + 1                      # + the null page
        self.cache = CacheManager(needs, page_size, num_pages, MAX_LIVE, dtype, device)
        max_len = min(self.cfg.max_position_embeddings, max_tokens)
        self.runner = ModelRunner(self.model, self.cache, max_step_tokens or max_tokens, MAX_LIVE, max_len,
                                  tuple(s for s in graph_batch_sizes if s <= MAX_LIVE), tuple(graph_portion_sizes))
        self.live: dict[str, object] = {}

    def step(self, record: dict) -> np.ndarray | None:
        entries = []
        for e in record.get("entries", []):
            rid = str(e["id"])
            rc = self.live.get(rid)
            if rc is None:
                rc = self.live[rid] = self.cache.admit(rid)
            entries.append(StepEntry(rc, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = self.runner.step(entries) if entries else None
        for rid in record.get("end", []):
            rc = self.live.pop(str(rid), None)
            if rc is not None:
                self.cache.release(rc)
        if logits is None:
            return None
        return logits.float().cpu().numpy()


def run(model_dir: str, dtype_name: str, out_dir: str, max_tokens: int, stdin=None, stdout=None,
        device=None, page_size: int = 64, graph_batch_sizes: tuple[int, ...] = ()) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype_name]
    if device is None:
        from turingserve_b200 import kernels
        kernels.ops()                                   # builds at the first call; raises without a GPU
        device = torch.device("cuda", torch.cuda.current_device())
    os.makedirs(out_dir, exist_ok=True)
    rp = Replayer(model_dir, dtype, max_tokens, device, page_size, graph_batch_sizes=graph_batch_sizes)
    with torch.inference_mode():
        for line in stdin:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            logits = rp.step(rec)
            if logits is not None:
                logits.astype("<f4").tofile(os.path.join(out_dir, f"{rec['step']}.f32"))
            stdout.write(f"done {rec['step']}\n")
            stdout.flush()
    return 0
