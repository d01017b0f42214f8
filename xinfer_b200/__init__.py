"""xinfer_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

Public entry points, in the manner of the reference's Python package (xinfer.pyi):
``Engine(EngineConfig, dtype)`` with ``generate_sync`` / ``generate_stream``, ``SamplingParams``,
``GenerationOutput``; plus ``ModelRunner.step`` for callers that drive steps themselves.
"""
from .config import EngineConfig, GenerationConfig, Qwen3Config, ConfigError, register_architecture

__version__ = "0.1.0"


def __getattr__(name):
    # heavier parts are imported on first use so that configuration-only users stay light
    if name in ("Engine", "GenerationOutput", "StreamItem"):
        from .engine import llm
        return getattr(llm, name)
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    if name in ("ModelRunner", "StepInput", "StepError"):
        from .engine import runner
        return getattr(runner, name)
    raise AttributeError(f"module 'xinfer_b200' has no attribute '{name}'")


__all__ = ["EngineConfig", "GenerationConfig", "Qwen3Config", "ConfigError", "register_architecture", "Engine",
           "GenerationOutput", "StreamItem", "SamplingParams", "ModelRunner", "StepInput", "StepError"]
