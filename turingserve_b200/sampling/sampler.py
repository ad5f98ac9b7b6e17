"""Sampler: penalties -> min_tokens -> greedy / temperature -> top-k -> top-p -> exponential-race
draw, all in device kernels, one device-to-host copy at the end
(turingserve/sampling/sampler.py:68-107, turingserve/sampling/penalties.py:20-45).

The draw is ``argmax(probs / E)`` with E ~ Exp(1) per vocabulary entry, as the reference
(sampler.py:95-103).  Where the reference takes E from a ``torch.Generator`` per seeded request
and a shared one for the rest, here E comes from a counter-based generator keyed by
(the request's seed, how many tokens it has drawn so far, the vocabulary index): a request's
stream never depends on its batch-mates, seeded or not.  Requests without a seed get one derived
from the engine seed and their arrival number.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from turingserve_b200 import kernels
from turingserve_b200.sampling.params import SamplingParams

_MASK64 = (1 << 64) - 1


def derive_seed(engine_seed: int, ordinal: int) -> int:
    """splitmix64 of (engine seed, arrival number): the seed of a request that brought none."""
    z = (engine_seed * 0x9E3779B97F4A7C15 + ordinal + 0x632BE59BD9B4E019) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return (z ^ (z >> 31)) & _MASK64


@dataclass
class SampleRow:
    """What the sampler needs to know about the request behind one logits row."""

    params: SamplingParams
    seed: int                       # 64-bit seed of this request's stream
    num_drawn: int                  # tokens this request has sampled so far (the stream position)
    prompt_ids: list[int]
    output_ids: list[int]
    stop_ids: tuple[int, ...] = ()  # eos + stop_token_ids, masked while num_output < min_tokens


@dataclass
class PendingSample:
    """A draw that has been launched: tokens and flags are on their way to the host."""

    device_out: torch.Tensor        # [2, S] int32 on the device: tokens, then bad flags
    host_out: torch.Tensor          # the same, in pinned host memory (valid after ``event``)
    event: object
    count: int
    host_status: torch.Tensor | None = None     # the kernels' status words, copied with the tokens

    def status(self):
        """The status words of the kernels with bounded waits as the draw saw them (all zero: every
        block of the step ran to its end); None when the kernel object reports none.  Valid after
        ``Sampler.finish``."""
        return None if self.host_status is None else self.host_status.numpy()


class Sampler:
    def __init__(self, device) -> None:
        self.device = torch.device(device)
        self._host_ring: list[torch.Tensor] = []
        self._turn = 0
        # parameter staging: pinned host memory (a copy from pageable memory would first wait for
        # everything queued on the stream, and so undo the overlap of steps)
        self._param_ring: list[tuple[torch.Tensor, torch.Tensor, object]] = []
        self._param_turn = 0

    def sample(self, logits: torch.Tensor, rows: list[SampleRow]) -> tuple[np.ndarray, np.ndarray]:
        """logits [S, V] fp32 on the device -> (tokens[S], bad[S]) on the host.  ``bad`` marks rows
        with a NaN or +inf logit; their token is 0 (the reference zeroes such rows, sampler.py:73-74)."""
        return self.finish(self.launch(logits, rows))

    def finish(self, pending: PendingSample) -> tuple[np.ndarray, np.ndarray]:
        """Wait for a launched draw (only for it, not for work queued after it)."""
        if pending.event is not None:
            pending.event.synchronize()
        host = pending.host_out.numpy()
        return host[0, :pending.count].astype(np.int64), host[1, :pending.count].astype(bool)

    def _param_buffers(self, S: int) -> tuple[torch.Tensor, torch.Tensor]:
        pin = self.device.type == "cuda"
        if len(self._param_ring) < 4:
            self._param_ring.append((torch.zeros((max(S, 256), 2), dtype=torch.float32, pin_memory=pin),
                                     torch.zeros((max(S, 256), 4), dtype=torch.int64, pin_memory=pin), None))
        k = self._param_turn % len(self._param_ring)
        fh, ih, ev = self._param_ring[k]
        if ev is not None:
            ev.synchronize()                                       # the copy that last used these has run
        if fh.shape[0] < S:
            fh = torch.zeros((S, 2), dtype=torch.float32, pin_memory=pin)
            ih = torch.zeros((S, 4), dtype=torch.int64, pin_memory=pin)
        self._param_ring[k] = (fh, ih, None)
        return fh, ih

    def _param_copied(self) -> None:
        k = self._param_turn % len(self._param_ring)
        fh, ih, _ = self._param_ring[k]
        ev = None
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
        self._param_ring[k] = (fh, ih, ev)
        self._param_turn += 1

    def _host_buffer(self, n: int) -> torch.Tensor:
        """A contiguous pinned int32 buffer of ``n`` elements (contiguous, so that the copy into it
        is one asynchronous transfer)."""
        if len(self._host_ring) < 4:
            pin = self.device.type == "cuda"
            self._host_ring.append(torch.empty(max(n, 516), dtype=torch.int32, pin_memory=pin))
        k = self._turn % len(self._host_ring)
        if self._host_ring[k].numel() < n:
            self._host_ring[k] = torch.empty(n, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self._turn += 1
        return self._host_ring[k][:n]

    @torch.inference_mode()
    def launch(self, logits: torch.Tensor, rows: list[SampleRow]) -> PendingSample:
        """Edit the logits, draw, and start the copy of tokens and flags to the host; no waiting."""
        ops = kernels.ops()
        S, V = logits.shape
        assert S == len(rows)
        dev = self.device
        if any(r.params.uses_penalties or len(r.output_ids) < r.params.min_tokens for r in rows):
            logits = logits.clone()
            self._edit_logits(ops, logits, rows)
        # tokens, flags and (where the kernel object reports them) the kernels' status words leave in
        # one buffer and one copy
        W = int(getattr(ops, "STATUS_WORDS", 0))
        buf = torch.empty(2 * S + W, dtype=torch.int32, device=dev)
        out, status = buf[: 2 * S].view(2, S), (buf[2 * S:] if W else None)
        extra = (status,) if W else ()
        if all(r.params.greedy for r in rows) and hasattr(ops, "sample_greedy"):
            # no parameters to send, and the rows spread over many blocks instead of one each
            ops.sample_greedy(out, logits, *extra)
            return self._copy_out(buf, S, W)
        fh, ih = self._param_buffers(S)
        f, i = fh.numpy()[:S], ih.numpy()[:S]
        f[:] = 0
        i[:] = 0
        for n, r in enumerate(rows):
            p = r.params
            f[n, 0] = 0.0 if p.greedy else p.temperature
            f[n, 1] = p.top_p
            i[n, 0] = p.top_k
            i[n, 1] = np.int64(np.uint64(r.seed & _MASK64).astype(np.int64))
            i[n, 2] = r.num_drawn
        fp = fh[:S].to(dev, non_blocking=True)
        ip = ih[:S].to(dev, non_blocking=True)
        self._param_copied()
        ops.sample(out, logits, fp, ip, *extra)
        return self._copy_out(buf, S, W)

    def _copy_out(self, buf: torch.Tensor, S: int, W: int) -> PendingSample:
        host = self._host_buffer(2 * S + W)
        host.copy_(buf, non_blocking=True)             # the one device-to-host copy of the step
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        return PendingSample(buf[: 2 * S].view(2, S), host[: 2 * S].view(2, S), event, S,
                             host[2 * S:] if W else None)

    def _edit_logits(self, ops, logits: torch.Tensor, rows: list[SampleRow]) -> None:
        """Penalties (penalties.py:20-45), then stop tokens masked to -inf while fewer than
        ``min_tokens`` were produced (sampler.py:24-28,84-86).  Token lists travel as one flat
        int32 array with offsets."""
        flat: list[int] = []
        meta = np.zeros((len(rows), 8), dtype=np.int32)
        pen = np.zeros((len(rows), 4), dtype=np.float32)
        for n, r in enumerate(rows):
            p = r.params
            a = len(flat)
            if p.uses_penalties:
                flat += r.prompt_ids
            b = len(flat)
            if p.uses_penalties:
                flat += r.output_ids
            c = len(flat)
            if len(r.output_ids) < p.min_tokens:
                flat += list(r.stop_ids)
            d = len(flat)
            meta[n, :4] = (a, b, c, d)
            pen[n, :3] = (p.repetition_penalty, p.presence_penalty, p.frequency_penalty)
        dev = self.device
        ids = torch.tensor(flat if flat else [0], dtype=torch.int32).to(dev, non_blocking=True)
        ops.penalize(logits, ids, torch.from_numpy(meta).to(dev, non_blocking=True),
                     torch.from_numpy(pen).to(dev, non_blocking=True))
