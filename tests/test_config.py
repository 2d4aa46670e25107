"""Configuration: reading config.json keys, validation, presets, registry."""

import json

import pytest

from deterministic_inference_b200.config import (ConfigError, EngineConfig, Qwen3Config,
                                                 SamplingParams, preset, preset_names)
from deterministic_inference_b200.models.registry import (MODEL_REGISTRY, UnknownArchitecture,
                                                          config_from_dir)

BASE = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=3,
            hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
            intermediate_size=160, vocab_size=512, rms_norm_eps=1e-5, rope_theta=1e6,
            max_position_embeddings=512)


def test_reads_every_key_and_round_trips():
    cfg = Qwen3Config.from_dict({**BASE, "tie_word_embeddings": True, "eos_token_id": [7, 9]})
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads) == (3, 96, 6)
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size) == (2, 32, 160)
    assert cfg.q_size == 192 and cfg.kv_size == 64        # head_dim is explicit: q_size != hidden
    assert cfg.eos_token_ids == (7, 9) and cfg.tie_word_embeddings
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


def test_defaults_follow_the_reference():
    cfg = Qwen3Config.from_dict(BASE)
    assert cfg.tie_word_embeddings is False          # sid/model/loader.py:53
    assert cfg.eos_token_ids == (151645,)            # sid/model/loader.py:34


def test_generation_config_overrides_eos(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({**BASE, "eos_token_id": 1}))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 4]}))
    assert Qwen3Config.from_json(tmp_path).eos_token_ids == (3, 4)   # sid/model/loader.py:35-39


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 4}, "multiple"),
    ({"head_dim": 31}, "even"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"model_type": "llama"}, "model_type"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"vocab_size": 0}, "positive"),
])
def test_rejects_what_it_cannot_run(change, match):
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict({**BASE, **change})


def test_missing_keys_are_listed():
    d = dict(BASE)
    del d["head_dim"], d["rope_theta"]
    with pytest.raises(ConfigError, match="head_dim.*rope_theta"):
        Qwen3Config.from_dict(d)


def test_window_layers():
    cfg = Qwen3Config.from_dict({**BASE, "use_sliding_window": True, "sliding_window": 24,
                                 "max_window_layers": 2})
    assert [cfg.layer_window(i) for i in range(3)] == [None, None, 24]
    plan = cfg.plan()
    assert [l.mixer.params["window"] for l in plan.layers] == [None, None, 24]


def test_plan_is_data():
    plan = preset("tiny_a").plan()
    plan.validate()
    assert [e.layer for e in plan.schedule] == [0, 1] and all(e.writes_cache for e in plan.schedule)
    m = plan.layers[0].mixer
    assert m.kind == "gqa_attention" and m.params["head_dim"] == 16 and m.params["scale"] == 16 ** -0.5
    assert plan.head.params["name"] is None              # tied
    assert preset("tiny_b").plan().head.params["name"] == "lm_head.weight"


def test_presets_and_parameter_counts():
    assert {"tiny_a", "tiny_b", "qwen3_0_6b", "qwen3_8b", "qwen3_32b"} <= set(preset_names())
    assert preset("qwen3_0_6b").num_parameters() == 596_049_920
    assert preset("qwen3_8b").num_parameters() == 8_190_735_360
    with pytest.raises(ConfigError, match="unknown preset"):
        preset("nope")


def test_registry(tmp_path):
    assert MODEL_REGISTRY["Qwen3ForCausalLM"] is Qwen3Config
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    assert isinstance(config_from_dir(tmp_path), Qwen3Config)
    (tmp_path / "config.json").write_text(json.dumps({**BASE, "architectures": ["LlamaForCausalLM"]}))
    with pytest.raises(UnknownArchitecture, match="Qwen3ForCausalLM"):
        config_from_dir(tmp_path)


def test_engine_config_and_sampling_params():
    with pytest.raises(ValueError):
        EngineConfig()
    with pytest.raises(ValueError):
        EngineConfig(model_path="x", dtype="fp16")
    assert EngineConfig(model_path="x", dtype="fp32").dtype == "float32"
    assert EngineConfig(model_path="x", kv_pool_tokens=100, page_size=16).num_pages == 6
    for bad in (dict(temperature=-1), dict(top_p=0.0), dict(top_p=1.5), dict(max_new_tokens=0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)            # sid/config.py:101-107
