"""Weights: binding by name, the one error that lists every problem, dtype policy,
random-weights mode."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from deterministic_inference_b200.config import preset
from deterministic_inference_b200.models.registry import build_model
from deterministic_inference_b200.weights import (WeightsError, load_weights, random_tensors,
                                                  write_random_model)


def _model(name="tiny_a"):
    cfg = preset(name)
    return cfg, build_model(cfg, torch.bfloat16, "cpu")


def test_random_model_folder_loads_and_is_reproducible(tmp_path):
    cfg, model = _model()
    a = write_random_model(cfg, 5, tmp_path / "a")
    b = write_random_model(cfg, 5, tmp_path / "b")
    c = write_random_model(cfg, 6, tmp_path / "c")
    ta, tb, tc = (load_file(str(d / "model.safetensors")) for d in (a, b, c))
    assert set(ta) == {s.name for s in model.tensor_specs()}
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert any(not torch.equal(ta[k], tc[k]) for k in ta)
    assert all(v.dtype == torch.bfloat16 for v in ta.values())
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    # laws: matrices N(0, 0.02), norm weights 1 + N(0, 0.1)
    emb = ta["model.embed_tokens.weight"].float()
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(emb.mean())) < 0.002
    nw = torch.cat([v.float() for k, v in ta.items() if "norm" in k])
    assert abs(float(nw.mean()) - 1.0) < 0.05 and 0.05 < float(nw.std()) < 0.15


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dtype_policy(tmp_path, dtype):
    cfg, model = _model("tiny_b")
    d = write_random_model(cfg, 1, tmp_path)
    w = load_weights(d, model.tensor_specs(), model.plan, dtype, "cpu")
    assert w["model.embed_tokens.weight"].dtype == dtype
    assert w["model.layers.0.mlp.down_proj.weight"].dtype == dtype
    # norm weights stay float32 in both paths
    assert w["model.norm.weight"].dtype == torch.float32
    assert w["model.layers.1.self_attn.q_norm.weight"].dtype == torch.float32
    # the 32-bit path holds exactly the stored (bfloat16) values
    raw = load_file(str(d / "model.safetensors"))
    assert torch.equal(w["lm_head.weight"].float(), raw["lm_head.weight"].float())
    model.load(w)
    assert model.blocks[0].mixer.w_qkv.shape == (cfg.q_size + 2 * cfg.kv_size, cfg.hidden_size)
    assert model.blocks[0].feed_forward.w_gate_up.shape == (2 * cfg.intermediate_size, cfg.hidden_size)


def test_one_error_lists_missing_unexpected_shapes_and_types(tmp_path):
    cfg, model = _model("tiny_b")
    d = write_random_model(cfg, 1, tmp_path)
    t = load_file(str(d / "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    t["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    t["model.layers.0.self_attn.o_proj.weight"] = t["model.layers.0.self_attn.o_proj.weight"].T.contiguous()
    t["lm_head.weight"] = torch.zeros(512, 96, dtype=torch.int32)
    save_file(t, str(d / "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_weights(d, model.tensor_specs(), model.plan, torch.bfloat16, "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg \
        and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.extra.weight" in msg
    assert "wrong shapes (2)" in msg and "expected [32], found [16]" in msg \
        and "expected [96, 192], found [192, 96]" in msg
    assert "wrong types (1)" in msg and "lm_head.weight: stored as I32" in msg


def test_tied_head_ignores_a_stray_lm_head_and_rotary_buffers(tmp_path):
    cfg, model = _model("tiny_a")                   # tied (sid/model/loader.py:76-80,105)
    d = write_random_model(cfg, 1, tmp_path)
    t = load_file(str(d / "model.safetensors"))
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(t, str(d / "model.safetensors"))
    w = load_weights(d, model.tensor_specs(), model.plan, torch.bfloat16, "cpu")
    model.load(w)
    assert model.head.tied and model.head.weight is model.embedding.table()


def test_no_safetensors(tmp_path):
    cfg, model = _model()
    with pytest.raises(WeightsError, match="no \\*.safetensors"):
        load_weights(tmp_path, model.tensor_specs(), model.plan, torch.bfloat16, "cpu")


def test_sharded_checkpoint(tmp_path):
    cfg, model = _model("tiny_b")
    specs = model.tensor_specs()
    t = random_tensors(specs, 2)
    names = sorted(t)
    save_file({k: t[k] for k in names[::2]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in names[1::2]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    w = load_weights(tmp_path, specs, model.plan, torch.bfloat16, "cpu")
    assert all(torch.equal(w[k].float(), t[k].float()) for k in names)
