"""The flat token batch of one step, on the device.

Same content as the reference's ``ModelInput`` / ``AttentionMetadata``
(turingserve/runner/attention_metadata.py:10-27, built in turingserve/runner/input_builder.py:105-150):
ids, positions, per-token cache slots, cumulative query starts, context lengths after the step,
padded block tables, rows whose logits are wanted.  Differences: everything is int32; there is one
slot mapping and one block table per cache GROUP; each request also brings its state slot; and the
whole step travels in ONE pinned buffer and ONE host-to-device copy.

Requests with a single token (decodes) are placed first (input_builder.py:41-48), whatever order
the caller gave; ``sample_rows`` keeps the caller's order.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from turingserve_b200.cache.manager import CacheManager, RequestCache


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the places among them (``want``)
    whose logits are asked for."""

    cache: RequestCache
    tokens: list[int]
    want: list[int] = field(default_factory=list)
    # When set, the (single) token is not known to the host yet: its id is row ``feedback`` of the
    # previous step's sampler output and is put in place on the device (``tokens`` holds a stand-in).
    feedback: int | None = None


@dataclass
class GroupInputs:
    block_tables: torch.Tensor      # [B, W] int32, padded with the null page 0
    slot_mapping: torch.Tensor      # [T] int32, -1 = do not write
    table_width: int


@dataclass
class StepInputs:
    num_tokens: int
    num_requests: int
    num_decode: int                 # leading requests with exactly one token
    input_ids: torch.Tensor         # [T] int32
    positions: torch.Tensor         # [T] int32
    token_request: torch.Tensor     # [T] int32: index of the request a token belongs to
    q_start: torch.Tensor           # [B+1] int32
    seq_lens: torch.Tensor          # [B] int32: context length after this step
    state_slots: torch.Tensor       # [B] int32
    sample_rows: torch.Tensor       # [S] int32 rows of the flat batch
    groups: list[GroupInputs]
    feedback_rows: torch.Tensor     # [F] int32 rows of the flat batch whose id comes from the device
    feedback_src: torch.Tensor      # [F] int32 rows of the previous sampler output
    # host copies, for launch geometry and for parts written in plain torch
    q_lens: list[int]
    starts: list[int]
    max_q_len: int
    max_seq_len: int
    # The single-token requests together read this many keys or more: their attention should be the
    # kernel built for streaming, not the one built for the shortest chain.  Set from the real
    # lengths; a captured step keeps one graph for each value.
    streaming_decode: bool = False
    # every row of the batch is wanted, in batch order (a captured decode step)
    all_rows_sampled: bool = False


# From about this many keys under the decode rows of a step (requests x longest context), reading them
# takes longer than the fixed chain of a decode-attention launch, and the kernel built for streaming wins
# (measured at 12 heads over 2 kv heads of 128: 4 x 16,384 keys 23 against 26 us for the short-chain kernel,
# 8 x 16,384 keys 38 against 32 us).  The kernels' front adds its own rule for many requests.
STREAMING_DECODE_KEYS = 98304


def streaming_decode(num_decode: int, longest_context: int) -> bool:
    return num_decode * longest_context >= STREAMING_DECODE_KEYS


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class StepInputBuilder:
    """Fills a pinned host arena and copies it to a persistent device arena."""

    def __init__(self, cache: CacheManager, max_tokens: int, max_requests: int,
                 max_pages_per_request: int, device) -> None:
        self.cache = cache
        self.max_tokens, self.max_requests = max_tokens, max_requests
        self.max_pages = max_pages_per_request
        self.device = device
        g = len(cache.groups)
        cap = (_align(max_tokens) * (3 + g) + _align(max_requests + 1) + 4 * _align(max_requests)
               + _align(max_tokens) + g * _align(max_requests * max_pages_per_request) + 64)
        self.capacity = cap
        pin = device is not None and torch.device(device).type == "cuda"
        self._host = [torch.empty(cap, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._events = [None, None]
        self._turn = 0
        self._dev = torch.empty(cap, dtype=torch.int32, device=device)

    def order(self, entries: list[StepEntry]) -> list[int]:
        """Indices of ``entries`` in batch order: single-token requests first, stable."""
        dec = [i for i, e in enumerate(entries) if len(e.tokens) == 1]
        rest = [i for i, e in enumerate(entries) if len(e.tokens) != 1]
        return dec + rest

    def build(self, entries: list[StepEntry], *, fixed_width: int | None = None,
              pad_requests: int = 0, arena: torch.Tensor | None = None) -> StepInputs:
        """Lay out the step.  ``pad_requests`` puts that many empty decode rows (context 0, slot -1,
        null pages) behind the single-token requests: used to fill a captured batch size.  ``fixed_width`` forces the
        block-table width; ``arena`` is an alternative device buffer (static addresses)."""
        order = self.order(entries)
        n_dec = sum(1 for e in entries if len(e.tokens) == 1)
        # batch order: single-token requests, the padding rows, then the rest
        order = order[:n_dec] + [None] * pad_requests + order[n_dec:]
        rows_e = [None if i is None else entries[i] for i in order]
        ents = [e for e in rows_e if e is not None]
        B = len(rows_e)
        q_lens = [1 if e is None else len(e.tokens) for e in rows_e]
        T = sum(q_lens)
        if B > self.max_requests:
            raise ValueError(f"step has {B} requests, the engine was sized for {self.max_requests}")
        if T > self.max_tokens:
            raise ValueError(f"step has {T} tokens, the engine was sized for {self.max_tokens}")
        if T == 0:
            raise ValueError("empty step")
        starts = [0 if e is None else e.cache.num_tokens for e in rows_e]
        num_decode = n_dec + pad_requests
        ps = self.cache.page_size
        widths = []
        for gi in range(len(self.cache.groups)):
            w = max([len(e.cache.tables[gi]) for e in ents] + [1])
            if fixed_width is not None:
                if w > fixed_width:
                    raise ValueError("block table wider than the fixed width")
                w = fixed_width
            widths.append(w)

        # caller-order sample rows
        row_of = {}
        off = 0
        for i, n in zip(order, q_lens):
            if i is not None:
                row_of[i] = off
            off += n
        sample = []
        for i, e in enumerate(entries):
            for w_ in e.want:
                if not 0 <= w_ < len(e.tokens):
                    raise ValueError(f"request {e.cache.request_id!r}: wanted place {w_} outside its {len(e.tokens)} tokens")
                sample.append(row_of[i] + w_)
        S = len(sample)

        host_t = self._host[self._turn]
        ev = self._events[self._turn]
        if ev is not None:
            ev.synchronize()
        host = host_t.numpy()
        cursor = 0

        def take(n: int):
            nonlocal cursor
            a = cursor
            cursor += _align(n)
            return a

        # With a caller-owned arena (a captured graph reads it at fixed addresses) the layout may depend
        # only on T, B and the table widths, never on how many rows are wanted or fed back.
        static = arena is not None
        o_ids, o_pos, o_req = take(T), take(T), take(T)
        o_qs, o_sl, o_ss, o_sr = take(B + 1), take(B), take(B), take(T if static else max(S, 1))
        fb = [(b, e.feedback) for b, e in enumerate(rows_e) if e is not None and e.feedback is not None]
        F = len(fb)
        o_fr, o_fs = take(B if static else max(F, 1)), take(B if static else max(F, 1))
        o_slot = [take(T) for _ in widths]
        o_bt = [take(B * w) for w in widths]
        used = cursor
        if used > self.capacity:
            raise ValueError("step does not fit the input arena")

        ids = host[o_ids:o_ids + T]
        pos = host[o_pos:o_pos + T]
        req = host[o_req:o_req + T]
        qs = host[o_qs:o_qs + B + 1]
        sl = host[o_sl:o_sl + B]
        ss = host[o_ss:o_ss + B]
        qs[0] = 0
        t = 0
        for b, e in enumerate(rows_e):
            if e is None:                           # a padding row: no context, nothing written
                ids[t] = 0
                pos[t] = 0
                req[t] = b
                t += 1
                qs[b + 1] = t
                sl[b] = 0
                ss[b] = self.cache.null_slot
                continue
            n = len(e.tokens)
            ids[t:t + n] = e.tokens
            pos[t:t + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            req[t:t + n] = b
            t += n
            qs[b + 1] = t
            sl[b] = starts[b] + n
            ss[b] = e.cache.slot
        host[o_sr:o_sr + S] = sample
        for i, (b, src) in enumerate(fb):
            if q_lens[b] != 1:
                raise ValueError("a token fed back on the device must be a request's only token in the step")
            host[o_fr + i] = qs[b]
            host[o_fs + i] = src
            ids[qs[b]] = 0
        for gi, w in enumerate(widths):
            bt = host[o_bt[gi]:o_bt[gi] + B * w].reshape(B, w)
            bt[:] = 0
            sm = host[o_slot[gi]:o_slot[gi] + T]
            t = 0
            for b, e in enumerate(rows_e):
                if e is None:
                    sm[t] = -1
                    t += 1
                    continue
                table = e.cache.tables[gi]
                bt[b, :len(table)] = table
                n = len(e.tokens)
                p = pos[t:t + n]
                tab = np.asarray(table, dtype=np.int32)
                sm[t:t + n] = tab[p // ps] * ps + p % ps
                t += n

        dev = self._dev if arena is None else arena
        dev[:used].copy_(host_t[:used], non_blocking=True)
        if torch.device(self.device).type == "cuda":
            e_ = torch.cuda.Event()
            e_.record()
            self._events[self._turn] = e_
        self._turn ^= 1

        def d(o, n):
            return dev[o:o + n]

        groups = [GroupInputs(d(o_bt[gi], B * w).view(B, w), d(o_slot[gi], T), w)
                  for gi, w in enumerate(widths)]
        return StepInputs(
            num_tokens=T, num_requests=B, num_decode=num_decode, input_ids=d(o_ids, T),
            positions=d(o_pos, T), token_request=d(o_req, T), q_start=d(o_qs, B + 1),
            seq_lens=d(o_sl, B), state_slots=d(o_ss, B), sample_rows=d(o_sr, S), groups=groups,
            feedback_rows=d(o_fr, F), feedback_src=d(o_fs, F),
            q_lens=q_lens, starts=starts, max_q_len=max(q_lens), max_seq_len=int(sl.max()) if B else 0,
            streaming_decode=streaming_decode(num_decode, int(sl[:num_decode].max()) if num_decode else 0))
