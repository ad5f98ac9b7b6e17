"""Traces for the replay tests: the same requests cut into steps in four ways.

Every trace wants the logits of every token it feeds, so each schedule can be compared position
by position with the plain whole-sequence implementation.
"""

from __future__ import annotations

import numpy as np


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, whole, in one step."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: dict[str, list[int]], sizes=(7, 2, 16, 3, 2, 5, 11, 2, 9, 4)) -> list[dict]:
    """Portions of changing size, down to two tokens, crossing page edges."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            if len(toks) - at - n == 1:          # never leave a single token for last: take it along
                n += 1
            k += 1
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
    return steps


def mixed(requests: dict[str, list[int]], seed: int = 0, max_live: int = 4, tail: int = 12) -> list[dict]:
    """Up to ``max_live`` requests at a time: prompt portions of some beside single decoded tokens of
    others, some requests left out of a step; finished requests make room for waiting ones, so
    their pages are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = {"toks": toks, "at": 0}
        entries, end = [], []
        ids = list(live)
        for rid in ids:
            st = live[rid]
            toks, at = st["toks"], st["at"]
            if len(ids) > 1 and rng.random() < 0.2:
                continue                              # left out of this step
            left = len(toks) - at
            if left <= tail:
                n = 1
            else:
                n = int(rng.integers(2, 14))
                n = min(n, left - tail) if left - tail >= 2 else left - tail
                n = max(n, 1)
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            st["at"] = at + n
            if st["at"] == len(toks):
                end.append(rid)
        if not entries:
            continue
        for rid in end:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def batched_tail(requests: dict[str, list[int]], tail: int = 24, seed: int = 0, max_live: int = 4) -> list[dict]:
    """Up to ``max_live`` requests at a time: each one's head in a step of its own, then their last
    ``tail`` tokens one a step, all live requests of a step decoding together but for some left out at
    random.  These are the steps a captured decode graph serves: 1 to ``max_live`` single tokens, so a
    graph of 4 is also run with 3 (a padding row)."""
    rng = np.random.default_rng(seed)
    steps = []
    items = list(requests.items())
    for base in range(0, len(items), max_live):
        group = items[base:base + max_live]
        at = {}
        for rid, toks in group:
            head = max(1, len(toks) - tail)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                          "end": [rid] if head == len(toks) else []})
            if head < len(toks):
                at[rid] = head
        toks_of = dict(group)
        while at:
            ids = [rid for rid in at if len(at) == 1 or rng.random() < 0.8] or [next(iter(at))]
            entries, end = [], []
            for rid in ids:
                entries.append({"id": rid, "tokens": [toks_of[rid][at[rid]]], "want": [0]})
                at[rid] += 1
                if at[rid] == len(toks_of[rid]):
                    end.append(rid)
                    del at[rid]
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def served(requests: dict[str, list[int]], portion: int = 16, tail: int = 20, max_live: int = 4) -> list[dict]:
    """As a serving engine cuts its steps: every live request that is past its prompt (all but its last
    ``tail`` tokens) brings one token and wants its logits; beside them ONE request still in its prompt
    brings a portion of exactly ``portion`` tokens (its last portion: what is left) and wants the logits
    of the prompt's last token only.  These are the steps a captured graph of (decoding rows, portion
    length) serves."""
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = {"toks": toks, "at": 0, "prompt": max(1, len(toks) - tail)}
        entries, end = [], []
        in_prompt = [rid for rid, st in live.items() if st["at"] < st["prompt"]]
        for rid, st in live.items():
            if st["at"] >= st["prompt"]:
                entries.append({"id": rid, "tokens": [st["toks"][st["at"]]], "want": [0]})
                st["at"] += 1
        if in_prompt:
            rid = in_prompt[0]
            st = live[rid]
            n = min(portion, st["prompt"] - st["at"])
            last = st["at"] + n == st["prompt"]
            entries.append({"id": rid, "tokens": st["toks"][st["at"]:st["at"] + n], "want": [n - 1] if last else []})
            st["at"] += n
        for rid, st in live.items():
            if st["at"] == len(st["toks"]):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: list[dict], outputs: dict[int, np.ndarray]) -> dict[str, dict[int, np.ndarray]]:
    """{request: {position: logits row}} from the per-step arrays a replay wrote."""
    at: dict[str, int] = {}
    got: dict[str, dict[int, np.ndarray]] = {}
    for s in steps:
        row = 0
        arr = outputs.get(s["step"])
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = arr[row]
                row += 1
            at[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            at.pop(rid, None)
    return got


def max_error(got: dict[str, dict[int, np.ndarray]], expected: dict[str, np.ndarray]):
    """(largest abs difference, where) over every collected row."""
    worst, where = 0.0, None
    for rid, rows in got.items():
        for pos, row in rows.items():
            err = float(np.abs(row - expected[rid][pos]).max())
            if not np.isfinite(err):
                return float("inf"), (rid, pos)
            if err > worst:
                worst, where = err, (rid, pos)
    return worst, where


def first_bad(got, expected, tol: float):
    """The first (request, position) whose error exceeds ``tol``: the place to look at."""
    for rid, rows in got.items():
        for pos in sorted(rows):
            err = float(np.abs(rows[pos] - expected[rid][pos]).max())
            if not err <= tol:
                return rid, pos, err
    return None
