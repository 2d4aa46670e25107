"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed.  The reference has no such mode (its tests download a
checkpoint, tests/test_05_model_vs_hf.py:14,45).

Law: matrices and the embedding N(0, std), norm weights 1 + N(0, norm_std), drawn
in float32 from ONE ``torch.Generator`` seeded once, in the fixed order in which
the model lists its tensors, then stored as bfloat16 like a published
checkpoint.  Both engine dtypes therefore run the same values (the 32-bit path
upcasts them exactly).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts.spec import TensorSpec


def random_tensors(specs: list[TensorSpec], seed: int, std: float = 0.02, norm_std: float = 0.1,
                   store_dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    out = {}
    for s in specs:
        x = torch.randn(tuple(s.shape), generator=g, dtype=torch.float32)
        if s.init == "one_plus_normal":
            x = 1.0 + norm_std * x
        elif s.init == "normal":
            x = std * x
        else:
            raise ValueError(f"{s.name}: unknown init law {s.init!r}")
        out[s.name] = x.to(store_dtype).contiguous()
    return out


def random_tensors_on_device(specs: list[TensorSpec], seed: int, dtype: torch.dtype, device,
                             std: float = 0.02, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    """The same laws drawn on the device, one generator seed per tensor
    (seed + index); for shapes too large to draw on the host and write to disk.
    The values differ from ``random_tensors``; they are rounded to bfloat16 like
    stored ones."""
    out = {}
    for i, s in enumerate(specs):
        g = torch.Generator(device=device).manual_seed(int(seed) * 1_000_003 + i)
        x = torch.randn(tuple(s.shape), generator=g, dtype=torch.float32, device=device)
        if s.init == "one_plus_normal":
            x = 1.0 + norm_std * x
        else:
            x = std * x
        x = x.to(torch.bfloat16)
        out[s.name] = x.to(torch.float32 if s.role == "vector" else dtype).contiguous()
    return out


def write_random_model(config, seed: int, out_dir, std: float = 0.02, norm_std: float = 0.1) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (any
    registered architecture's configuration object) under ``out_dir``."""
    from safetensors.torch import save_file

    from ..models.decoder import DecoderModel

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    specs = DecoderModel(config.plan(), torch.bfloat16, "cpu").tensor_specs()
    tensors = random_tensors(specs, seed, std, norm_std)
    (out_dir / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    save_file(tensors, str(out_dir / "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed), "std": str(std), "norm_std": str(norm_std)})
    return out_dir
