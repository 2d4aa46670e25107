"""A small, whole, single-GPU inference engine for Qwen3 dense on B200 (sm_100a):
typed configuration and registry, safetensors weights, a model put together from
parts, a paged cache manager, one step function over mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels.

    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams
    out = Engine(EngineConfig(model_path=DIR)).generate([[1, 2, 3]], SamplingParams())
"""

from .config import ConfigError, EngineConfig, Qwen3Config, SamplingParams, preset, preset_names

__all__ = ["Engine", "EngineConfig", "SamplingParams", "Qwen3Config", "ConfigError", "preset",
           "preset_names", "RequestOutput"]


def __getattr__(name):
    # the engine imports torch and the kernels; keep ``import package`` light
    if name in ("Engine", "RequestOutput"):
        from .engine import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)
