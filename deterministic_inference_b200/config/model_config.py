"""Typed model configuration for Qwen3 dense, read from the keys of config.json.

The reference fills a ``ModelConfig`` dataclass from config.json
(sid/config.py:33-57, sid/model/loader.py:30-55) and asserts
``model_type == "qwen3"``.  Here the configuration is a typed dataclass with
validation; no size and no constant that config.json gives stands anywhere else
in the package.  The class also turns itself into a ``ModelPlan``: the list of
parts (mixer, feed-forward, norm, position encoding) of each layer and the order
in which layers run, which is all the generic decoder knows of this
architecture.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Optional

from ..parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


_REQUIRED = (
    "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
    "head_dim", "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta",
    "max_position_embeddings",
)


@dataclass(frozen=True)
class Qwen3Config:
    """Every field is a key of Qwen3's config.json (same names).

    Required keys are the ones the reference reads without a default
    (sid/model/loader.py:40-52).  ``tie_word_embeddings`` defaults to False and
    ``eos_token_id`` to 151645 as there (:34,:53).  The window keys are read too
    (the reference ignores them): layers with index >= ``max_window_layers`` use
    a window of ``sliding_window`` keys when ``use_sliding_window`` is true.
    """

    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    eos_token_ids: tuple = (151645,)
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    hidden_act: str = "silu"
    attention_bias: bool = False
    architectures: tuple = ("Qwen3ForCausalLM",)
    model_type: str = "qwen3"

    # ---- construction -----------------------------------------------------

    @classmethod
    def from_dict(cls, cfg: dict, generation_config: Optional[dict] = None) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in cfg]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if cfg.get("model_type", "qwen3") != "qwen3":
            raise ConfigError(f"model_type must be 'qwen3', got {cfg.get('model_type')!r}")
        if cfg.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"rope_scaling is not supported: {cfg['rope_scaling']!r}")
        if cfg.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported (Qwen3 dense has no biases)")
        if cfg.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act must be 'silu', got {cfg.get('hidden_act')!r}")

        eos = cfg.get("eos_token_id", 151645)
        if generation_config is not None and "eos_token_id" in generation_config:
            # generation_config.json overrides (sid/model/loader.py:35-39)
            eos = generation_config["eos_token_id"]
        eos_ids = tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)

        out = cls(
            num_hidden_layers=int(cfg["num_hidden_layers"]),
            hidden_size=int(cfg["hidden_size"]),
            num_attention_heads=int(cfg["num_attention_heads"]),
            num_key_value_heads=int(cfg["num_key_value_heads"]),
            head_dim=int(cfg["head_dim"]),
            intermediate_size=int(cfg["intermediate_size"]),
            vocab_size=int(cfg["vocab_size"]),
            rms_norm_eps=float(cfg["rms_norm_eps"]),
            rope_theta=float(cfg["rope_theta"]),
            max_position_embeddings=int(cfg["max_position_embeddings"]),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            eos_token_ids=tuple(int(e) for e in eos_ids),
            use_sliding_window=bool(cfg.get("use_sliding_window", False)),
            sliding_window=(None if cfg.get("sliding_window") is None else int(cfg["sliding_window"])),
            max_window_layers=(None if cfg.get("max_window_layers") is None
                               else int(cfg["max_window_layers"])),
            hidden_act=cfg.get("hidden_act", "silu"),
            attention_bias=False,
            architectures=tuple(cfg.get("architectures", ("Qwen3ForCausalLM",))),
            model_type="qwen3",
        )
        out.validate()
        return out

    @classmethod
    def from_json(cls, model_dir) -> "Qwen3Config":
        model_dir = Path(model_dir)
        cfg = json.loads((model_dir / "config.json").read_text())
        gen = None
        gen_path = model_dir / "generation_config.json"
        if gen_path.exists():
            gen = json.loads(gen_path.read_text())
        return cls.from_dict(cfg, gen)

    def validate(self) -> None:
        pos = {k: getattr(self, k) for k in (
            "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
            "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings")}
        bad = {k: v for k, v in pos.items() if v < 1}
        if bad:
            raise ConfigError(f"sizes must be positive: {bad}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotate-half RoPE")
        if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window < 1:
                raise ConfigError("use_sliding_window=true needs a positive sliding_window")

    def to_dict(self) -> dict:
        """The config.json content that ``from_dict`` reads back unchanged."""
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = eos[0] if len(eos) == 1 else list(eos)
        d["architectures"] = list(d["architectures"])
        d["torch_dtype"] = "bfloat16"
        return d

    # ---- derived -----------------------------------------------------------

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of a layer, or None for all keys."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        full = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return None if layer < full else self.sliding_window

    def num_parameters(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        per_layer = (self.q_size + 2 * self.kv_size) * h + h * self.q_size + 3 * h * i \
            + 2 * h + 2 * self.head_dim
        n = self.num_hidden_layers * per_layer + self.vocab_size * h + h
        if not self.tie_word_embeddings:
            n += self.vocab_size * h
        return n

    # ---- the plan: parts layer by layer, and the order of layers ------------

    def plan(self) -> ModelPlan:
        """Qwen3 dense as parts (sid/model/qwen3.py:43-115): every layer is a
        pre-norm block of a grouped-query attention mixer with per-head q/k
        RMSNorm and full-width rotate-half RoPE, and a SiLU-gated dense
        feed-forward; layers run once each, in order, each on its own cache."""
        rope = PartSpec("rope", dict(
            head_dim=self.head_dim, rotary_dim=self.head_dim, theta=self.rope_theta,
            max_positions=self.max_position_embeddings))
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            norm = dict(size=self.hidden_size, eps=self.rms_norm_eps)
            layers.append(LayerSpec(
                block=PartSpec("pre_norm", {}),
                mixer=PartSpec("gqa_attention", dict(
                    prefix=p + "self_attn.",
                    hidden_size=self.hidden_size,
                    num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads,
                    head_dim=self.head_dim,
                    scale=self.head_dim ** -0.5,
                    qk_norm_eps=self.rms_norm_eps,
                    window=self.layer_window(i),
                    position_encoding=rope)),
                feed_forward=PartSpec("gated_mlp", dict(
                    prefix=p + "mlp.",
                    hidden_size=self.hidden_size,
                    intermediate_size=self.intermediate_size,
                    activation=self.hidden_act)),
                mixer_norm=PartSpec("rms_norm", dict(name=p + "input_layernorm.weight", **norm)),
                feed_forward_norm=PartSpec("rms_norm", dict(
                    name=p + "post_attention_layernorm.weight", **norm)),
            ))
        return ModelPlan(
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            embedding=PartSpec("token_embedding", dict(
                name="model.embed_tokens.weight", vocab_size=self.vocab_size, hidden_size=self.hidden_size)),
            head=PartSpec("linear_head", dict(
                name=None if self.tie_word_embeddings else "lm_head.weight",
                vocab_size=self.vocab_size, hidden_size=self.hidden_size)),
            ignored_names=("lm_head.weight",) if self.tie_word_embeddings else (),
            ignored_substrings=("rotary",),
            final_norm=PartSpec("rms_norm", dict(
                name="model.norm.weight", size=self.hidden_size, eps=self.rms_norm_eps)),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i, cache=i, writes_cache=True)
                           for i in range(self.num_hidden_layers)),
            max_positions=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids,
        )


# Named shapes (``--preset``) are data: one config.json-style file each under
# ``presets/`` beside this module.  The engine itself only ever sees a Qwen3Config.
_PRESET_DIR = Path(__file__).resolve().parent / "presets"


def preset_names() -> list[str]:
    return sorted(p.stem for p in _PRESET_DIR.glob("*.json"))


def preset(name: str, **overrides) -> Qwen3Config:
    path = _PRESET_DIR / f"{name}.json"
    if not path.exists():
        raise ConfigError(f"unknown preset {name!r}; known: {preset_names()}")
    d = json.loads(path.read_text())
    d.update(overrides)
    return Qwen3Config.from_dict(d)
