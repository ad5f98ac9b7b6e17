"""Command line: ``python -m turingserve_b200.cli generate|random-model ...``.

Engine options carry the reference's names and meanings (turingserve/config.py:114-156).  The
reference's ``serve`` starts an HTTP server (turingserve/cli.py:12-19), which this engine does not
have; ``generate`` is the offline counterpart of ``LLMEngine.generate``, and ``random-model`` is
the random-weights mode (in place of the reference's scripts/make_tiny_model.py).
"""

from __future__ import annotations

import argparse
import json
import sys

from turingserve_b200.config.engine_config import add_engine_arguments, engine_config_from_namespace


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="turingserve_b200")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids for prompts given as token ids")
    add_engine_arguments(g)
    g.add_argument("--prompt-ids", action="append", default=[],
                   help="comma-separated token ids; repeat for several prompts")
    g.add_argument("--prompt-len", type=int, action="append", default=[],
                   help="a random prompt of this many tokens (seeded by --seed); repeatable")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--min-tokens", type=int, default=0)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--sampling-seed", type=int, default=None, help="per-request seed")
    g.add_argument("--ignore-eos", action="store_true")

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    return p


def main(argv: list[str] | None = None) -> int:
    ns = build_parser().parse_args(argv)
    if ns.command == "random-model":
        import torch

        from turingserve_b200.config.registry import architecture_of
        from turingserve_b200.weights.random_init import write_random_model
        with open(ns.config, encoding="utf-8") as f:
            cj = json.load(f)
        cfg = architecture_of(cj).parse_config(cj, None)
        write_random_model(ns.out, cfg, ns.seed, ns.std, getattr(torch, ns.dtype))
        print(ns.out)
        return 0

    import numpy as np

    from turingserve_b200.config.registry import load_model_config
    from turingserve_b200.engine.engine import LLMEngine
    from turingserve_b200.sampling.params import SamplingParams

    cfg = engine_config_from_namespace(ns)
    prompts = [[int(t) for t in s.split(",") if t.strip()] for s in ns.prompt_ids]
    if ns.prompt_len:
        vocab = load_model_config(cfg.model).vocab_size
        rng = np.random.default_rng(cfg.seed)
        prompts += [rng.integers(0, vocab, size=n).tolist() for n in ns.prompt_len]
    if not prompts:
        print("give --prompt-ids or --prompt-len", file=sys.stderr)
        return 2
    params = SamplingParams(
        temperature=ns.temperature, top_k=ns.top_k, top_p=ns.top_p, seed=ns.sampling_seed,
        max_tokens=ns.max_tokens, min_tokens=ns.min_tokens, ignore_eos=ns.ignore_eos,
        repetition_penalty=ns.repetition_penalty, presence_penalty=ns.presence_penalty,
        frequency_penalty=ns.frequency_penalty)
    engine = LLMEngine.from_config(cfg)
    for out in engine.generate(prompts, params):
        print(json.dumps({"token_ids": out.token_ids, "finish_reason": out.finish_reason,
                          "prompt_tokens": out.prompt_tokens}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
