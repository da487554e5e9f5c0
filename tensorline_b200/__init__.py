"""tensorline_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a)."""
from .config import EngineConfig, Qwen2Config, ConfigError
from .sampling import SamplingParams, GenStats

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "Output"):
        from .engine import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)


__all__ = ["Engine", "Output", "EngineConfig", "Qwen2Config", "ConfigError", "SamplingParams", "GenStats"]
