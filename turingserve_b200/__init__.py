"""turingserve_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

    from turingserve_b200 import EngineConfig, LLMEngine, SamplingParams
    engine = LLMEngine.from_config(EngineConfig(model="/path/to/model"))
    outs = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=8))
"""

from turingserve_b200.config.engine_config import EngineConfig
from turingserve_b200.sampling.params import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("LLMEngine", "FinalOutput"):
        from turingserve_b200.engine import engine as _e
        return getattr(_e, name)
    if name in ("generate", "generate_greedy"):
        from turingserve_b200 import entry as _entry
        return getattr(_entry, name)
    raise AttributeError(name)


__all__ = ["EngineConfig", "SamplingParams", "LLMEngine", "FinalOutput", "generate", "generate_greedy"]
