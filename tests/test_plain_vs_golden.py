"""The plain implementation against the reference's own model code.

tests/golden/make_golden.py ran the reference's ``Qwen3Model.forward`` and
``sample`` once on the CPU (its GPU kernels replaced, for that run, by the float32
PyTorch references of its own tests) and stored the outputs; here the plain
implementation of tests/plain_qwen3.py must reproduce them."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from deterministic_inference_b200.config import preset
from deterministic_inference_b200.weights import write_random_model
from tests import plain_qwen3

GOLDEN = Path(__file__).resolve().parent / "golden"
META = json.loads((GOLDEN / "golden.json").read_text())


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_forward_reproduces_the_reference(name, tmp_path):
    m = META[name]
    write_random_model(preset(name), m["weight_seed"], tmp_path)
    cfg, w = plain_qwen3.read_model_dir(tmp_path)
    checksum = float(sum(v.double().abs().sum() for v in w.values()))
    if abs(checksum - m["weights_abs_sum"]) > 1e-6 * m["weights_abs_sum"]:
        pytest.skip("the seeded CPU generator gives other weights than when the golden files were made")
    want = torch.from_numpy(np.load(GOLDEN / f"{name}_logits.npy"))
    got = plain_qwen3.forward(cfg, w, m["tokens"])
    assert got.shape == want.shape
    torch.testing.assert_close(got, want, atol=5e-6, rtol=1e-5)


def test_plain_sampler_reproduces_the_reference():
    m = META["sampler"]
    logits = torch.from_numpy(np.load(GOLDEN / "sampler_logits.npy"))
    for i in range(logits.shape[0]):
        tok = plain_qwen3.sample_token(logits[i], m["temperatures"][i], m["seeds"][i],
                                       m["positions"][i], m["top_ks"][i], m["top_ps"][i])
        assert tok == m["tokens"][i], i
