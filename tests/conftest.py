"""Shared fixtures: the ``gpu`` marker, tiny model folders with random weights
(made in a temporary folder, never committed), and the ``torch_ops`` fixture that
lets the engine's host logic run on a machine without a GPU."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations of the architecture that differ in every size and
# option: head counts and group ratio, head size, hidden width (HqD == H or not),
# intermediate size, vocabulary, number of layers, eps, theta, tied or untied
# head, window or none.
TINY = {
    "a": dict(preset="tiny_a", seed=0, page_size=16),
    "b": dict(preset="tiny_b", seed=3, page_size=32),
    # Tiny B with a window on its last layer: two cache groups (all keys / window)
    "bw": dict(preset="tiny_b", seed=5, page_size=16,
               overrides=dict(use_sliding_window=True, sliding_window=24, max_window_layers=2)),
    # odd sizes: hidden 80 (no power of two), 5 heads in 5 groups (ratio 1), head_dim 48
    "c": dict(preset="tiny_a", seed=9, page_size=16,
              overrides=dict(hidden_size=80, num_attention_heads=5, num_key_value_heads=5,
                             head_dim=48, intermediate_size=112, vocab_size=300,
                             num_hidden_layers=1, rms_norm_eps=1e-4, rope_theta=5e4,
                             tie_word_embeddings=False, eos_token_id=299)),
    # Heads of 128, the head size of the benchmark shapes: the tcgen05 prompt kernel, the
    # page-wise TMA decode kernels and the eight-lane q/k kernel run inside these models.
    # "d": group ratio 2, page 16, tied head; "e": ratio 8 (one kv head), page 32, untied
    # head, other eps / theta, and a window on its last layer.
    "d": dict(preset="tiny_a", seed=11, page_size=16,
              overrides=dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                             head_dim=128, intermediate_size=384, vocab_size=320,
                             num_hidden_layers=2, max_position_embeddings=1024, eos_token_id=319)),
    "e": dict(preset="tiny_b", seed=13, page_size=32,
              overrides=dict(hidden_size=384, num_attention_heads=8, num_key_value_heads=1,
                             head_dim=128, intermediate_size=640, vocab_size=704,
                             num_hidden_layers=3, max_position_embeddings=1024, eos_token_id=703,
                             use_sliding_window=True, sliding_window=200, max_window_layers=2)),
    # The layer sizes of the smallest benchmark shape (width 1,024, 16 + 8 heads of 128,
    # intermediate 3,072) with two layers, a small vocabulary (the plain implementation must
    # stay fast) and a window on the second layer: the matrix-product shapes, split counts
    # and attention launch forms of the benchmark run inside the parity tests.
    "f": dict(preset="qwen3_0_6b", seed=17, page_size=16,
              overrides=dict(num_hidden_layers=2, vocab_size=2048, max_position_embeddings=4096,
                             eos_token_id=2047, use_sliding_window=True, sliding_window=600,
                             max_window_layers=1)),
}


@pytest.fixture(scope="session")
def tiny_model_dirs(tmp_path_factory):
    from deterministic_inference_b200.config import preset
    from deterministic_inference_b200.weights import write_random_model

    out = {}
    for name, spec in TINY.items():
        cfg = preset(spec["preset"], **spec.get("overrides", {}))
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(cfg, spec["seed"], d)
        sharpen(d)
        out[name] = d
    return out


def sharpen(model_dir, qk_scale: float = 2.5, final_scale: float = 6.0, o_scale: float = 6.0) -> None:
    """Random weights give nearly uniform attention and tiny logits, which would
    hide a wrong key under the rounding tolerance.  Scale the per-head q/k norm
    weights (scores grow by qk_scale^2, attention becomes sharp) and the final
    norm weight (logits reach unit scale); scale the attention output projection
    so that what attention computes weighs in the residual stream."""
    from safetensors.torch import load_file, save_file

    path = Path(model_dir) / "model.safetensors"
    tensors = load_file(str(path))
    for name in list(tensors):
        if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
            tensors[name] = (tensors[name].float() * qk_scale).to(tensors[name].dtype)
        if name.endswith("o_proj.weight"):
            tensors[name] = (tensors[name].float() * o_scale).to(tensors[name].dtype)
        if name == "model.norm.weight":
            tensors[name] = (tensors[name].float() * final_scale).to(tensors[name].dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})


@pytest.fixture
def torch_ops(monkeypatch):
    """Replace every kernel wrapper by its plain PyTorch restatement (CPU tests
    of host logic only)."""
    from deterministic_inference_b200.kernels import ops
    from tests import torch_kernels

    for name in torch_kernels.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_kernels, name))
    return ops
