"""Python entry points in the reference's manner: ``LLMEngine.from_config(cfg).generate(...)``
(turingserve/engine/engine.py:59-63,237-259) and the minimal greedy helper
(turingserve/simple_generate.py:10-31)."""

from __future__ import annotations

from turingserve_b200.config.engine_config import EngineConfig
from turingserve_b200.sampling.params import SamplingParams


def generate(model: str, prompts: list[list[int]], params: SamplingParams | list[SamplingParams] | None = None,
             **engine_options) -> list[list[int]]:
    """Generate continuations (token ids) for ``prompts`` with the model folder ``model``.
    ``engine_options`` are ``EngineConfig`` fields (dtype, block_size, num_blocks, ...)."""
    from turingserve_b200.engine.engine import LLMEngine

    engine = LLMEngine.from_config(EngineConfig(model=model, **engine_options))
    outs = engine.generate(prompts, params if params is not None else SamplingParams())
    return [o.token_ids for o in outs]


def generate_greedy(model: str, prompt_ids: list[int], max_new_tokens: int, eos_ids: tuple[int, ...] = (),
                    **engine_options) -> list[int]:
    """Greedy continuation of one prompt; stops at ``max_new_tokens`` or at one of ``eos_ids``."""
    params = SamplingParams(temperature=0.0, max_tokens=max_new_tokens, stop_token_ids=list(eos_ids))
    return generate(model, [prompt_ids], params, **engine_options)[0]
