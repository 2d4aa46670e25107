"""One registry from an architecture's name (``architectures[0]`` of config.json)
to its configuration class.  The reference has none: it asserts
``model_type == "qwen3"`` and imports its model class (sid/model/loader.py:32,
sid/engine/model_runner.py:23).

A configuration class has ``from_json(dir)``, ``from_dict(d)``, ``to_dict()`` and
``plan() -> ModelPlan``; the model itself is always the generic ``DecoderModel``
built from that plan.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.model_config import Qwen3Config
from .decoder import DecoderModel


class UnknownArchitecture(ValueError):
    pass


MODEL_REGISTRY: dict[str, type] = {}


def register_architecture(name: str, config_class: type) -> None:
    MODEL_REGISTRY[name] = config_class


register_architecture("Qwen3ForCausalLM", Qwen3Config)


def config_from_dir(model_dir):
    """The typed configuration of the folder's model, chosen by config.json."""
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"{path} does not exist")
    raw = json.loads(path.read_text())
    archs = raw.get("architectures") or []
    if not archs:
        raise UnknownArchitecture(f"{path} names no architecture; known: {sorted(MODEL_REGISTRY)}")
    if archs[0] not in MODEL_REGISTRY:
        raise UnknownArchitecture(f"architecture {archs[0]!r} is not registered; "
                                  f"known: {sorted(MODEL_REGISTRY)}")
    return MODEL_REGISTRY[archs[0]].from_json(model_dir)


def build_model(config, dtype: torch.dtype, device) -> DecoderModel:
    return DecoderModel(config.plan(), dtype, device)
