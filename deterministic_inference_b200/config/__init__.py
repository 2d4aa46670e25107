from .engine_config import EngineConfig, SamplingParams
from .model_config import ConfigError, Qwen3Config, preset, preset_names
