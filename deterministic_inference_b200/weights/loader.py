"""Weights from safetensors, bound by tensor name.

The reference reads every ``*.safetensors`` of the folder into one dict and pops
each tensor by its checkpoint name, casting to bfloat16; a missing name is a
``KeyError`` and leftovers an assertion (sid/model/loader.py:58-107).  Here the
model's parts say which tensors they need (name and shape); the headers of the
files are compared with that list before any data is read, and ONE error lists
everything that is missing, unexpected or of the wrong shape or type.

dtype: matrices and the embedding are cast to the engine dtype (bfloat16, or
float32 for the 32-bit path, which upcasts exactly); norm weights are kept in
float32 whatever they are stored as, because norm arithmetic is float32; an
integer tensor would be kept as int32.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import torch

from ..parts.spec import ModelPlan, TensorSpec


class WeightsError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem."""


_FLOAT_CODES = {"F32", "BF16", "F16", "F64"}
_INT_CODES = {"I8", "I16", "I32", "I64", "U8"}


def read_header(path: Path) -> dict[str, dict]:
    """{name: {"dtype", "shape"}} of one safetensors file, without its data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    header.pop("__metadata__", None)
    return header


def checkpoint_files(model_dir: Path) -> list[Path]:
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise WeightsError(f"no *.safetensors file in {model_dir}")
    return files


def check_checkpoint(headers: dict[str, dict], specs: list[TensorSpec], plan: ModelPlan) -> None:
    """Raise one ``WeightsError`` that lists all missing and unexpected tensors,
    wrong shapes and wrong types; return silently if the checkpoint fits."""
    expected = {s.name: s for s in specs}
    missing = [n for n in expected if n not in headers]
    unexpected = [n for n in headers
                  if n not in expected and n not in plan.ignored_names
                  and not any(sub in n for sub in plan.ignored_substrings)]
    wrong_shape, wrong_type = [], []
    for n, s in expected.items():
        if n not in headers:
            continue
        got = tuple(headers[n]["shape"])
        if got != tuple(s.shape):
            wrong_shape.append(f"{n}: expected {list(s.shape)}, found {list(got)}")
        if headers[n]["dtype"] not in _FLOAT_CODES:
            wrong_type.append(f"{n}: stored as {headers[n]['dtype']}, expected a floating type")
    if missing or unexpected or wrong_shape or wrong_type:
        lines = ["checkpoint does not match the model:"]
        for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                             ("wrong shapes", wrong_shape), ("wrong types", wrong_type)):
            if items:
                lines.append(f"  {title} ({len(items)}):")
                lines.extend(f"    {i}" for i in sorted(items))
        raise WeightsError("\n".join(lines))


def target_dtype(spec: TensorSpec, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if spec.role == "vector":
        return torch.float32
    return engine_dtype


def load_weights(model_dir, specs: list[TensorSpec], plan: ModelPlan, dtype: torch.dtype,
                 device) -> dict[str, torch.Tensor]:
    """{name: tensor on ``device``} for every spec, read file by file."""
    from safetensors import safe_open

    files = checkpoint_files(Path(model_dir))
    headers: dict[str, dict] = {}
    where: dict[str, Path] = {}
    for f in files:
        for name, meta in read_header(f).items():
            headers[name] = meta
            where[name] = f
    check_checkpoint(headers, specs, plan)

    by_file: dict[Path, list[TensorSpec]] = {}
    for s in specs:
        by_file.setdefault(where[s.name], []).append(s)
    out: dict[str, torch.Tensor] = {}
    for f, wanted in by_file.items():
        with safe_open(str(f), framework="pt", device="cpu") as reader:
            for s in wanted:
                t = reader.get_tensor(s.name)
                out[s.name] = t.to(device=device, dtype=target_dtype(s, t.dtype, dtype)).contiguous()
    return out
