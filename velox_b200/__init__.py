"""velox_b200: a single-GPU inference engine for sm_100a, built from parts.

    from velox_b200 import Engine, EngineConfig, SamplingParams
"""
from .config import EngineConfig, Qwen3Config, register_architecture
from .sampling.params import SamplingParams

__all__ = ["Engine", "EngineConfig", "Qwen3Config", "SamplingParams", "register_architecture"]
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
