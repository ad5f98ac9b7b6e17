"""LLMEngine: add requests, step until they finish.

One step = schedule -> one forward over the flat batch -> sample -> commit tokens -> finish and
free (turingserve/engine/engine.py:96-184).  Finish rules in the reference's order
(turingserve/engine/output_processor.py:26-44, turingserve/engine/stop.py:8-11): a stop token
(``stop_token_ids``, or an end-of-sequence id unless ``ignore_eos``) -> "stop"; ``max_tokens``
produced or ``max_model_len`` reached -> "length".  A row of non-finite logits, or a request that
can never be scheduled, finishes with "error" (engine.py:142-146,199-208); so does every request
of a step in which a kernel reported that one of its blocks gave up on a bounded wait (the step's
logits cannot be trusted; the kernel concerned is taken off the path for the steps that follow).
"""

from __future__ import annotations

import time
from dataclasses import dataclass

import torch

from turingserve_b200.cache.manager import CacheManager
from turingserve_b200.config.engine_config import EngineConfig
from turingserve_b200.engine.batch import StepEntry
from turingserve_b200.engine.request import Request, RequestOutput, Status
from turingserve_b200.engine.scheduler import Scheduler, StepPlan
from turingserve_b200.engine.runner import ModelRunner, run_needs

from turingserve_b200.sampling.params import SamplingParams
from turingserve_b200.sampling.sampler import Sampler, SampleRow, derive_seed


@dataclass
class FinalOutput:
    request_id: str
    token_ids: list[int]
    finish_reason: str | None
    prompt_tokens: int


@dataclass
class _Sampled:
    """Tokens a sampler without a launch/finish split returned at once."""

    tokens: object
    bad: object


@dataclass
class _InFlight:
    """A step that has been launched and whose tokens have not been committed yet."""

    plan: StepPlan
    sampling: list
    pending: object                      # PendingSample | _Sampled | None


class StepTimer:
    """Wall-clock seconds per phase of the last step (turingserve/utils/timing.py:9-24)."""

    def __init__(self) -> None:
        self.t: dict[str, float] = {}
        self._t0: dict[str, float] = {}

    def reset(self) -> None:
        self.t.clear()

    def start(self, name: str) -> None:
        self._t0[name] = time.perf_counter()

    def stop(self, name: str) -> None:
        self.t[name] = self.t.get(name, 0.0) + time.perf_counter() - self._t0.pop(name)


class LLMEngine:
    def __init__(self, cfg: EngineConfig, runner, cache: CacheManager, scheduler: Scheduler,
                 sampler, eos_ids: tuple[int, ...], max_model_len: int, vocab_size: int | None = None) -> None:
        self.cfg, self.runner, self.cache = cfg, runner, cache
        self.scheduler, self.sampler = scheduler, sampler
        self.eos_ids = tuple(eos_ids)
        self.max_model_len = max_model_len
        self.vocab_size = vocab_size
        self.faults: list[str] = []          # what kernels reported through their status words
        self.requests: dict[str, Request] = {}
        self._inflight: _InFlight | None = None
        self._aborts: list[str] = []
        self._arrivals = 0
        self.timer = StepTimer()
        self.step_count = 0

    # -- construction ---------------------------------------------------------------------------
    @classmethod
    def from_config(cls, cfg: EngineConfig) -> LLMEngine:
        """Start-up order of turingserve/engine/builder.py:29-135: config -> weights -> model ->
        number of pages (flag, or from free memory) -> cache -> runner, scheduler, sampler."""
        from turingserve_b200 import kernels
        from turingserve_b200.config.registry import load_model_config
        from turingserve_b200.weights.loader import load_model

        mcfg = load_model_config(cfg.model)
        cfg.validate(mcfg.max_position_embeddings)
        max_len = cfg.resolve_max_model_len(mcfg.max_position_embeddings)
        kernels.ops()                                   # build/load the CUDA library; fails loudly
        device = torch.device("cuda", torch.cuda.current_device())
        model, mcfg = load_model(cfg.model, cfg.torch_dtype, device, max_len)
        needs = run_needs(model)
        num_pages = cfg.num_blocks
        if num_pages is None:
            free, total = torch.cuda.mem_get_info(device)
            per_page = max(1, CacheManager.bytes_per_page(needs, cfg.block_size, cfg.torch_dtype))
            budget = free - (1.0 - cfg.gpu_memory_utilization) * total - (2 << 30)
            wanted = cfg.max_num_seqs * cfg.max_blocks_per_seq(max_len) + 1
            num_pages = int(max(2, min(budget // per_page, wanted)))
        cache = CacheManager(needs, cfg.block_size, num_pages, cfg.max_num_seqs, cfg.torch_dtype, device)
        runner = ModelRunner(model, cache, max(cfg.max_num_batched_tokens, cfg.max_num_seqs),
                             cfg.max_num_seqs, max_len,
                             cfg.graph_batch_sizes if cfg.cuda_graphs else (), cfg.graph_portion_sizes())
        scheduler = Scheduler(cache, cfg.max_num_batched_tokens, cfg.max_num_seqs, cfg.watermark,
                              runner.padded_decodes if cfg.graph_portion_sizes() else None)
        return cls(cfg, runner, cache, scheduler, Sampler(device), mcfg.eos_token_ids, max_len, mcfg.vocab_size)

    # -- requests -----------------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt_token_ids: list[int], params: SamplingParams) -> Request:
        if request_id in self.requests:
            raise ValueError(f"duplicate request id {request_id}")
        if not prompt_token_ids:
            raise ValueError("a request needs at least one prompt token")
        # refused here, where only this request is concerned: inside a step the same fault would take
        # the whole batch down, after pages were grown for it
        if len(prompt_token_ids) >= self.max_model_len:
            raise ValueError(f"request {request_id!r}: a prompt of {len(prompt_token_ids)} tokens leaves no room "
                             f"to generate within max_model_len {self.max_model_len}")
        if self.vocab_size is not None:
            lo, hi = min(prompt_token_ids), max(prompt_token_ids)
            if lo < 0 or hi >= self.vocab_size:
                raise ValueError(f"request {request_id!r}: token id {lo if lo < 0 else hi} outside "
                                 f"[0, {self.vocab_size})")
        seed = params.seed if params.seed is not None else derive_seed(self.cfg.seed, self._arrivals)
        self._arrivals += 1
        req = Request(request_id, list(prompt_token_ids), len(prompt_token_ids), params, seed=seed)
        self.requests[request_id] = req
        self.scheduler.add(req)
        return req

    def abort(self, request_id: str) -> None:
        self._aborts.append(request_id)

    def has_unfinished(self) -> bool:
        return bool(self._aborts) or self._inflight is not None or self.scheduler.has_unfinished()

    # -- one step -----------------------------------------------------------------------------------
    def step(self) -> list[RequestOutput]:
        """Commit one step's tokens and return what they produced.

        With ``async_decode`` the engine keeps one step in flight: before it waits for the current
        step's tokens it schedules and launches the next one, whose input ids for the requests that
        just sampled are taken from the sampler's output on the device.  The host work and the launch
        of step N+1 so overlap the GPU's work on step N.  A request that stops on a token (as opposed
        to its length, which is known beforehand) has then run one step in vain; its row is dropped."""
        t = self.timer
        t.reset()
        outputs = self._process_aborts()
        cur, self._inflight = self._inflight, None
        if cur is None:
            cur, outs = self._schedule_and_launch(None)
            outputs += outs
            if cur is None:
                return outputs + self._fail_unschedulable()
        nxt = None
        if self._may_look_ahead(cur):
            self._mark_pending(cur)
            nxt, outs = self._schedule_and_launch(cur)
            outputs += outs
        outputs += self._finish_step(cur)
        self._inflight = nxt
        self.step_count += 1
        return outputs

    def _schedule_and_launch(self, prev: _InFlight | None) -> tuple[_InFlight | None, list[RequestOutput]]:
        t = self.timer
        t.start("schedule")
        plan = self.scheduler.schedule()
        t.stop("schedule")
        outputs = [self._finish(req, "error", []) for req in plan.failed]
        self._finalize(outputs)
        if not plan.items:
            return None, outputs
        return self._launch(plan, prev), outputs

    def _run(self, plan: StepPlan) -> list[RequestOutput]:
        """Run one given plan to the end (launch, wait, commit)."""
        return self._finish_step(self._launch(plan, None))

    def _launch(self, plan: StepPlan, prev: _InFlight | None) -> _InFlight:
        t = self.timer
        t.start("forward")
        entries = []
        prev_row = {id(r): i for i, r in enumerate(prev.sampling)} if prev is not None else {}
        for it in plan.items:
            r = it.request
            start = r.num_computed
            toks = r.token_ids[start:start + it.num_tokens]
            feedback = None
            if r.pending and start + it.num_tokens == len(r.token_ids):
                feedback = prev_row[id(r)]                        # the stand-in: its id is still on the device
            entries.append(StepEntry(r.cache, toks, [it.num_tokens - 1] if it.samples else [], feedback))
        if prev is not None and prev.pending is not None and any(e.feedback is not None for e in entries):
            logits = self.runner.step(entries, prev.pending.device_out[0])
        else:
            logits = self.runner.step(entries)
        t.stop("forward")
        sampling = [it.request for it in plan.items if it.samples]
        pending = None
        t.start("sample")
        if sampling:
            rows = [SampleRow(r.params, r.seed, r.num_drawn + (1 if r.pending else 0),
                              r.token_ids[:r.num_prompt_tokens], r.output_ids, self._stop_ids(r)) for r in sampling]
            if hasattr(self.sampler, "launch"):
                pending = self.sampler.launch(logits, rows)
            else:
                pending = _Sampled(*self.sampler.sample(logits, rows))
        t.stop("sample")
        return _InFlight(plan, sampling, pending)

    def _may_look_ahead(self, cur: _InFlight) -> bool:
        if not (self.cfg.async_decode and getattr(self.runner, "supports_feedback", False)):
            return False
        if cur.pending is None or isinstance(cur.pending, _Sampled):
            return False
        for r in cur.sampling:
            p = r.params
            if p.uses_penalties or p.min_tokens > 0:
                return False                                      # these read the tokens produced so far
        return any(self._continues_after_next_token(r) for r in cur.sampling)

    def _continues_after_next_token(self, req: Request) -> bool:
        """Whether the request goes on after the token now in flight, as far as its length decides."""
        return (req.num_output + 1 < req.params.max_tokens and len(req.token_ids) + 1 < self.max_model_len
                and not req.finished)

    def _mark_pending(self, cur: _InFlight) -> None:
        for r in cur.sampling:
            if self._continues_after_next_token(r):
                r.token_ids.append(-1)                            # stand-in until the token arrives
                r.pending = True

    def _finish_step(self, cur: _InFlight) -> list[RequestOutput]:
        t = self.timer
        outputs: list[RequestOutput] = []
        if cur.pending is None:
            return outputs
        t.start("sample")
        if isinstance(cur.pending, _Sampled):
            tokens, bad = cur.pending.tokens, cur.pending.bad
        else:
            tokens, bad = self.sampler.finish(cur.pending)
            status = cur.pending.status() if hasattr(cur.pending, "status") else None
            if status is not None and any(int(v) for v in status):
                from turingserve_b200 import kernels
                self.faults.append(kernels.ops().fault_reported(status))
                bad = [True] * len(cur.sampling)
                # portions that drew nothing wrote keys and values of the same untrustworthy step
                for p in cur.plan.items:
                    if not p.samples and not p.request.finished:
                        if p.request.pending:
                            p.request.token_ids.pop()
                            p.request.pending = False
                        outputs.append(self._finish(p.request, "error", []))
        t.stop("sample")
        t.start("output")
        for row, req in enumerate(cur.sampling):
            if req.finished:                                      # stopped or aborted while this step ran
                continue
            if req.pending:
                req.token_ids.pop()
                req.pending = False
            if bad[row]:
                outputs.append(self._finish(req, "error", []))
                continue
            outputs.append(self._commit(req, int(tokens[row])))
        self._finalize(outputs)
        t.stop("output")
        return outputs

    def _stop_ids(self, req: Request) -> tuple[int, ...]:
        return tuple(self.eos_ids) + tuple(req.params.stop_token_ids)

    def _commit(self, req: Request, token: int) -> RequestOutput:
        req.token_ids.append(token)
        req.num_drawn += 1
        p = req.params
        if token in p.stop_token_ids or ((not p.ignore_eos) and token in self.eos_ids):
            return self._finish(req, "stop", [token])
        if req.num_output >= p.max_tokens or len(req.token_ids) >= self.max_model_len:
            return self._finish(req, "length", [token])
        return self._output(req, [token])

    def _output(self, req: Request, tokens: list[int]) -> RequestOutput:
        return RequestOutput(req.request_id, tokens, req.finished, req.finish_reason,
                             req.num_prompt_tokens, req.num_output)

    def _finish(self, req: Request, reason: str, tokens: list[int]) -> RequestOutput:
        req.status = Status.FINISHED
        req.finish_reason = reason
        return self._output(req, tokens)

    def _finalize(self, outputs: list[RequestOutput]) -> None:
        for out in outputs:
            if not out.finished:
                continue
            req = self.requests.pop(out.request_id, None)
            if req is not None:
                self.scheduler.finish(req)

    def _process_aborts(self) -> list[RequestOutput]:
        outs = []
        ids, self._aborts = self._aborts, []
        for rid in ids:
            req = self.requests.get(rid)
            if req is None or req.finished:
                continue
            outs.append(self._finish(req, "abort", []))
        self._finalize(outs)
        return outs

    def _fail_unschedulable(self) -> list[RequestOutput]:
        req = self.scheduler.unschedulable()
        if req is None:
            return []
        out = self._finish(req, "error", [])
        self._finalize([out])
        return [out]

    # -- offline helper -----------------------------------------------------------------------------
    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams]
                 ) -> list[FinalOutput]:
        """Run ``prompts`` (lists of token ids) to completion (turingserve/engine/engine.py:237-259)."""
        plist = params if isinstance(params, list) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or a single one for all")
        ids = [f"gen-{id(self)}-{i}-{time.monotonic_ns()}" for i in range(len(prompts))]
        for rid, p, sp in zip(ids, prompts, plist):
            self.add_request(rid, p, sp)
        finals = {rid: FinalOutput(rid, [], None, len(p)) for rid, p in zip(ids, prompts)}
        while self.has_unfinished():
            for out in self.step():
                f = finals.get(out.request_id)
                if f is None:
                    continue
                f.token_ids += out.delta_token_ids
                if out.finished:
                    f.finish_reason = out.finish_reason
        return [finals[r] for r in ids]

