"""The plain implementation by itself: each part against an independent
formulation, and the properties the engine relies on."""

import math

import torch

from tests import plain_qwen3 as P
from tests import torch_kernels as K


def test_rms_norm_formula():
    x = torch.randn(5, 12)
    w = torch.randn(12)
    want = torch.stack([r / math.sqrt(float((r * r).mean()) + 1e-3) * w for r in x])
    torch.testing.assert_close(P.rms_norm(x, w, 1e-3), want)


def test_rope_is_a_rotation_by_position_times_frequency():
    d, theta = 8, 100.0
    ang = P.rope_angles(torch.tensor([0, 3]), d, theta)
    assert ang.shape == (2, 4) and float(ang[0].abs().sum()) == 0.0
    assert abs(float(ang[1, 1]) - 3 * theta ** (-1 / 4)) < 1e-6
    x = torch.randn(2, 3, d)
    y = P.apply_rope(x, ang)
    torch.testing.assert_close(y[0], x[0])                                # position 0: identity
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))            # rotations keep the norm
    c, s = math.cos(float(ang[1, 2])), math.sin(float(ang[1, 2]))
    torch.testing.assert_close(y[1, :, 2], x[1, :, 2] * c - x[1, :, 6] * s)   # pairs (i, i + d/2)
    torch.testing.assert_close(y[1, :, 6], x[1, :, 6] * c + x[1, :, 2] * s)


def test_attention_is_causal_grouped_and_windowed():
    t, hq, hkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(t, hq, d), torch.randn(t, hkv, d), torch.randn(t, hkv, d)
    out = P.attention(q, k, v, 0.5)
    # position p depends on keys 0..p only
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 7.0, -3.0
    torch.testing.assert_close(P.attention(q, k2, v2, 0.5)[:5], out[:5])
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.clone()
    v3[:, 1] += 1.0
    o3 = P.attention(q, k, v3, 0.5)
    torch.testing.assert_close(o3[:, :2], out[:, :2])
    torch.testing.assert_close(o3[:, 2:], out[:, 2:] + 1.0)
    # window 1: a query sees only its own key
    torch.testing.assert_close(P.attention(q, k, v, 0.5, window=1)[:, 0], v[:, 0])
    # window 3 at position 8 ignores keys 0..5
    k4 = k.clone()
    k4[:6] = 50.0
    torch.testing.assert_close(P.attention(q, k4, v, 0.5, window=3)[8], P.attention(q, k, v, 0.5, window=3)[8])


def test_gumbel_scalar_and_vector_forms_agree():
    for seed, pos in ((42, 0), (-3, 17), (123456789012, 4095)):
        vec = P.seeded_gumbel(seed, pos, 50)
        for col in (0, 1, 7, 49):
            assert abs(P.seeded_gumbel_scalar(seed, pos, col) - float(vec[col])) < 1e-6
    a = K.seeded_gumbel(torch.tensor([42, -3]), torch.tensor([5, 6]), 33)
    torch.testing.assert_close(a[0], P.seeded_gumbel(42, 5, 33))
    torch.testing.assert_close(a[1], P.seeded_gumbel(-3, 6, 33))


def test_sampling_rules():
    logits = torch.zeros(100)
    logits[[3, 42]] = 2.0
    assert P.sample_token(logits, 0.0, 1, 0) == 3                       # first index wins ties
    row = torch.tensor([10.0, 9.0, 8.0, -20.0, -20.0])
    assert all(P.sample_token(row, 2.0, 5, p, top_k=3) in (0, 1, 2) for p in range(100))
    assert all(P.sample_token(torch.tensor([10.0, 0, 0, 0, 0]), 1.0, 5, p, top_p=0.5) == 0 for p in range(50))
    draws = {P.sample_token(torch.zeros(50), 1.0, 9, p) for p in range(40)}
    assert len(draws) > 10                                               # the position seeds the draw


def test_bf16_storage_emulation_only_rounds(tiny_model_dirs):
    cfg, w = P.read_model_dir(tiny_model_dirs["a"])
    toks = list(range(20))
    a, b = P.forward(cfg, w, toks), P.forward(cfg, w, toks, store_bf16=True)
    assert 0 < float((a - b).abs().max()) < 0.5
    _, w64 = P.read_model_dir(tiny_model_dirs["a"], torch.float64)
    c = P.forward(cfg, w64, toks)
    assert c.dtype == torch.float64 and float((a.double() - c).abs().max()) < 1e-4
