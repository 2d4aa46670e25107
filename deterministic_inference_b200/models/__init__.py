from .decoder import DecoderModel
from .registry import MODEL_REGISTRY, UnknownArchitecture, build_model, config_from_dir, register_architecture
