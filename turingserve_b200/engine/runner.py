"""The step function: run a batch of (request, its next tokens) from the cache and return the
logits at the wanted places.

One call = one forward pass over a flat token batch that may mix portions of prompts with single
decoded tokens (turingserve/runner/model_runner.py:20-32; design in docs/ARCHITECTURE.md:224-237 of
the reference).  It runs only the tokens it is given; everything earlier comes from the cache.

Pure-decode steps whose request count fits a captured size are replayed from a CUDA graph (the
reference captures the decode forward per batch size, turingserve/runner/cuda_graphs.py:44-78).  So
are steps of decoding requests beside ONE prompt portion of a captured length (``graph_portion_sizes``):
launched kernel by kernel, a step of a few hundred tokens costs the host more time than the GPU.
"""

from __future__ import annotations

import dataclasses
import gc

import torch

from turingserve_b200 import kernels
from turingserve_b200.cache.manager import CacheManager, RunNeeds
from turingserve_b200.engine.batch import StepEntry, StepInputBuilder, StepInputs, streaming_decode
from turingserve_b200.parts.model import DecoderModel


def run_needs(model: DecoderModel) -> list[RunNeeds]:
    """What each run of the model's schedule needs from the cache manager."""
    out = []
    for r, run in enumerate(model.cfg.schedule):
        mixer = model.run_mixer(r)
        out.append(RunNeeds(cache=mixer.cache_need(), state=mixer.state_need(), cache_from=run.cache_from))
    return out


class ModelRunner:
    supports_feedback = True            # entries may take their token id from the previous sampler output

    def __init__(self, model: DecoderModel, cache: CacheManager, max_tokens: int, max_requests: int,
                 max_model_len: int, graph_batch_sizes: tuple[int, ...] = (),
                 graph_portion_sizes: tuple[int, ...] = ()) -> None:
        self.model, self.cache = model, cache
        self.max_model_len = max_model_len
        self.max_pages = -(-max_model_len // cache.page_size)
        # (rows of a captured step: the decoding requests filled up to a captured size, and the portion's)
        rows = max_requests + (1 if graph_portion_sizes else 0)
        self.builder = StepInputBuilder(cache, max_tokens, rows, self.max_pages, model.device)
        self.views = cache.views()
        self.graph_batch_sizes = tuple(sorted(graph_batch_sizes))
        self.graph_portion_sizes = frozenset(graph_portion_sizes)
        # a step of a few single tokens as ONE kernel, where the model's parts are the ones it is written for
        from turingserve_b200.parts.fused_decode import FusedDecodeStep
        self.fused = FusedDecodeStep.try_build(model, self.views) if hasattr(model, "blocks") else None
        self._graphs: dict[tuple[int, int, bool], _StepGraph] = {}

    # -- the step ---------------------------------------------------------------------------------
    def step(self, entries: list[StepEntry], prev_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """Logits [sum(len(e.want)), vocab] fp32 in the order of ``entries`` and of each ``want``
        (None when nothing is wanted).  Grows each request's pages, runs, then advances the cache.
        ``prev_tokens``: the previous step's sampled tokens on the device, for entries whose token
        is fed back there (``StepEntry.feedback``)."""
        self._check(entries)
        if prev_tokens is None and any(e.feedback is not None for e in entries):
            raise ValueError("entries with device feedback need the previous step's tokens")
        for e in entries:
            self.cache.grow(e.cache, len(e.tokens))
        shape = self._graph_shape(entries)
        if shape is not None:
            logits = self._replay(shape, entries, prev_tokens)
        else:
            step = self.builder.build(entries)
            self._feed(step, prev_tokens)
            logits = self.forward(step)
        for e in entries:
            self.cache.advance(e.cache, len(e.tokens))
        return logits

    def _feed(self, step: StepInputs, prev_tokens: torch.Tensor | None) -> None:
        if step.feedback_rows.shape[0]:
            kernels.ops().feed_tokens(step.input_ids, step.feedback_rows, step.feedback_src, prev_tokens,
                                      self.model.cfg.vocab_size)

    def forward(self, step: StepInputs) -> torch.Tensor | None:
        if self.fused is not None and getattr(kernels.ops(), "use_fused_step", False) and self.fused.takes(step):
            logits = self.fused.run(step)
            if step.all_rows_sampled:
                return logits
            if step.sample_rows.shape[0] == 0:
                return None
            wanted = torch.empty((step.sample_rows.shape[0], logits.shape[1]), dtype=logits.dtype, device=logits.device)
            kernels.ops().gather_rows(wanted, logits, step.sample_rows)
            return wanted
        hidden = self.model.forward(step, self.views, self.cache.states)
        if step.sample_rows.shape[0] == 0:
            return None
        # a captured decode step samples every row in order: no rows to pick out
        return self.model.logits(hidden, None if step.all_rows_sampled else step.sample_rows)

    def _check(self, entries: list[StepEntry]) -> None:
        seen = set()
        vocab = self.model.cfg.vocab_size
        for e in entries:
            if id(e.cache) in seen:
                raise ValueError(f"request {e.cache.request_id!r} appears twice in one step")
            seen.add(id(e.cache))
            if not e.tokens:
                raise ValueError(f"request {e.cache.request_id!r} brings no tokens")
            if e.cache.num_tokens + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.cache.request_id!r} would exceed max_model_len {self.max_model_len}")
            if e.feedback is not None:
                continue
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise ValueError(f"request {e.cache.request_id!r}: token id outside [0, {vocab})")

    # -- CUDA graphs -------------------------------------------------------------------------------
    def padded_decodes(self, n: int) -> int | None:
        """The captured batch size that ``n`` decoding requests are filled up to (None: none takes them)."""
        if n == 0:
            return 0
        for s in self.graph_batch_sizes:
            if s >= n:
                return s
        return None

    def _graph_shape(self, entries: list[StepEntry]) -> tuple[int, int] | None:
        """(decode rows after padding, tokens of the one prompt portion or 0) when the step is one that
        graphs are kept for: single tokens whose logits are wanted, and at most one portion of a captured
        length whose last logits, or none, are wanted."""
        if not self.graph_batch_sizes:
            return None
        n_dec, portion = 0, 0
        for e in entries:
            n = len(e.tokens)
            if n == 1 and e.want == [0]:
                n_dec += 1
            elif (n > 1 and portion == 0 and n in self.graph_portion_sizes and e.feedback is None
                    and (not e.want or e.want == [n - 1])):
                portion = n
            else:
                return None
        size = self.padded_decodes(n_dec)
        if size is None or size + (1 if portion else 0) > self.builder.max_requests or size + portion > self.builder.max_tokens:
            return None
        return size, portion

    def _replay(self, shape: tuple[int, int], entries: list[StepEntry], prev_tokens=None) -> torch.Tensor | None:
        # which attention kernel the decode rows get is part of what a graph captures
        decodes = [e for e in entries if len(e.tokens) == 1]
        streaming = bool(decodes) and streaming_decode(len(decodes), max(e.cache.num_tokens for e in decodes) + 1)
        key = (*shape, streaming)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _StepGraph(self, shape[0], shape[1], streaming)
        return g.run(entries, prev_tokens)


class _StepGraph:
    """One captured step for ``size`` single-token requests (fewer are filled up with empty rows) and, when
    ``portion`` is not 0, one prompt portion of that many tokens behind them, with one choice of
    decode-attention kernel: static input arena, static logits (a row per single-token request in batch
    order, then the portion's last row)."""

    def __init__(self, runner: ModelRunner, size: int, portion: int, streaming: bool) -> None:
        self.runner, self.size, self.portion, self.streaming = runner, size, portion, streaming
        b = runner.builder
        dev = runner.model.device
        self.arena = torch.zeros(b.capacity, dtype=torch.int32, device=dev)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        # in a captured decode step every row is sampled: row b of the logits is request b
        rows = list(range(size)) + ([size + portion - 1] if portion else [])
        self.rows = torch.tensor(rows, dtype=torch.int32, device=dev)
        self.kernels_per_replay = 0

    def _build(self, entries: list[StepEntry]) -> StepInputs:
        r = self.runner
        n_dec = sum(1 for e in entries if len(e.tokens) == 1)
        step = r.builder.build(entries, fixed_width=r.max_pages, pad_requests=self.size - n_dec, arena=self.arena)
        # launch geometry must not depend on this step's lengths: size it for the longest context
        return dataclasses.replace(step, sample_rows=self.rows, max_seq_len=r.max_model_len,
                                   streaming_decode=self.streaming, all_rows_sampled=self.portion == 0)

    def _wanted(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """The caller's rows (order of ``entries`` and of their ``want``) out of the static logits."""
        idx, n_dec = [], 0
        for e in entries:
            if len(e.tokens) == 1:
                idx.append(n_dec)                   # single-token requests keep the caller's order among themselves
                n_dec += 1
            elif e.want:
                idx.append(self.size)
        if not idx:
            return None
        if idx == list(range(len(idx))):
            return self.logits[:len(idx)]
        if idx[:-1] == list(range(len(idx) - 1)) and idx[-1] == self.size:
            # the single tokens first, then the portion, as a scheduler orders them: two slices, no index
            # tensor (made on the host, it would be a copy from pageable memory, which waits for the stream)
            return torch.cat([self.logits[:len(idx) - 1], self.logits[self.size:self.size + 1]])
        return self.logits[torch.tensor(idx, dtype=torch.long, device=self.logits.device)]

    def run(self, entries: list[StepEntry], prev_tokens=None) -> torch.Tensor | None:
        step = self._build(entries)
        self.runner._feed(step, prev_tokens)
        ops = kernels.ops()
        if self.graph is None:
            r = self.runner
            # warm up outside capture (lazy set-up, allocator pools), then capture
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                r.forward(step)
            torch.cuda.current_stream().wait_stream(s)
            graph = torch.cuda.CUDAGraph()
            before = getattr(ops, "launches", 0)
            # No garbage collection while the stream captures: a finaliser that gives pinned host memory or
            # an event back to the driver in the middle of it is a call the capture does not allow, and
            # the capture is then lost (seen once in a long test session, never alone).
            was_collecting = gc.isenabled()
            gc.collect()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    self.logits = r.forward(step)
            finally:
                if was_collecting:
                    gc.enable()
            self.kernels_per_replay = getattr(ops, "launches", 0) - before
            self.graph = graph
        self.graph.replay()
        if hasattr(ops, "launches"):
            ops.launches += self.kernels_per_replay
        return self._wanted(entries)
