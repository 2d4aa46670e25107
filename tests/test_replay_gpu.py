"""Trace replay on the GPU against the plain implementation: the same requests
whole, with the last 32 tokens one by one, in portions of changing size down to
two tokens, and mixed (up to four live requests, portions beside single tokens,
a pool so small that pages are used again); in float32 and in bfloat16; on tiny
configurations that differ in every size and option.

Attention in the tiny models is made sharp (q/k norm weights scaled up) so that
a wrong or missing key changes the logits by far more than rounding."""

import pytest
import torch

from tests import plain_qwen3, replay_util as ru
from tests.conftest import TINY

pytestmark = pytest.mark.gpu

# Tolerances.  A logit's error comes from the hidden state's error, not from the
# logit's own size, so bounds are absolute per row, scaled by the row's largest
# logit.
#   float32: two float32 implementations of the same formulas differ by their
#   reduction orders.  The yardstick is the plain implementation itself: run in
#   float64 it gives the reference value, and the engine's distance from that
#   value may be at most 4 times the distance of the plain float32 run (per
#   request), with a floor of 1e-6 of the scale.
#   bfloat16: against the plain implementation with bfloat16 STORAGE emulated
#   (float32 arithmetic; every tensor the reference keeps in bfloat16, and the
#   probabilities before P.V, rounded there).  What remains is accumulation order
#   and roundings that flip; 2e-2 of the scale is the reference's tolerance for
#   its bfloat16 kernels (tests/conftest.py:35-37 there).  Against pure float32
#   these sharpened tiny models differ by 0.1-0.6 from storage rounding alone,
#   which would hide faults; the emulated comparison does not.  The engine cannot
#   round at exactly the emulation's values (the tensor-core kernel rounds the
#   probabilities relative to a running maximum, tile by tile), so a part of the
#   roundings is independent of the emulation's.  The yardstick for that part is
#   again the model itself: R = what storage rounding does to the request's logits
#   (emulated minus float32 plain); the engine may differ from the emulation by at
#   most half of R, or 2e-2 of the scale where that is larger.
BF16_FRAC, BF16_ROUNDING_SHARE = 2e-2, 0.5
F32_FACTOR, F32_FLOOR = 4.0, 1e-6


def row_error(got, want):
    return float((got.double() - want.double()).abs().max())


def _requests(vocab, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


CASES = {
    "a": ([5, 17, 33, 70, 121], 1),
    "b": ([1, 9, 31, 64, 100], 4),
    "bw": ([3, 40, 77, 130, 24], 6),
    "c": ([2, 16, 48, 95], 8),
}


@pytest.fixture(scope="module")
def plain_logits(tiny_model_dirs):
    out = {}
    for name, (lens, seed) in CASES.items():
        cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs[name])
        _, w64 = plain_qwen3.read_model_dir(tiny_model_dirs[name], torch.float64)
        reqs = _requests(cfg["vocab_size"], lens, seed)
        out[name] = (cfg, reqs, {
            "float64": [plain_qwen3.forward(cfg, w64, r) for r in reqs],
            "float32": [plain_qwen3.forward(cfg, w, r) for r in reqs],
            "bfloat16": [plain_qwen3.forward(cfg, w, r, store_bf16=True) for r in reqs]})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings(name, dtype, tiny_model_dirs, plain_logits, tmp_path):
    cfg, reqs, refs = plain_logits[name]
    page = TINY[name]["page_size"]
    trace = ru.Trace()
    # the mixed cutting first sizes the pool; the others reuse it one request at a time
    ru.mixed(trace, reqs)
    ru.whole(trace, reqs)
    ru.last_one_by_one(trace, reqs)
    ru.portions(trace, reqs)
    out = ru.run_trace(tiny_model_dirs[name], dtype, trace, tmp_path / "out", page_size=page)
    got = ru.read_rows(out, trace, cfg["vocab_size"])
    assert got, "the trace wrote nothing"
    if dtype == "float32":
        want = refs["float64"]
        yard = [max(row_error(a, b) for a, b in zip(p32, p64))
                for p32, p64 in zip(refs["float32"], refs["float64"])]
    else:
        want = refs["bfloat16"]
        yard = [max(row_error(a, b) for a, b in zip(emu, p32))
                for emu, p32 in zip(refs["bfloat16"], refs["float32"])]
    worst = 0.0
    for (key, pos), row in got.items():
        i = int(key[1:])
        err = row_error(row, want[i][pos])
        scale = max(1.0, float(want[i][pos].abs().max()))
        bound = (max(F32_FACTOR * yard[i], F32_FLOOR * scale) if dtype == "float32"
                 else max(BF16_FRAC * scale, BF16_ROUNDING_SHARE * yard[i]))
        assert err <= bound, (f"{name}/{dtype}: request {key} position {pos}: "
                              f"abs diff {err:.4g} exceeds {bound:.4g}")
        worst = max(worst, err / scale)
    # every cutting covered every position of every request
    for kind in "mwtp":
        for i, r in enumerate(reqs):
            assert all((f"{kind}{i}", p) in got for p in range(len(r))), (kind, i)
    print(f"{name}/{dtype}: worst diff {worst:.3e} of the row's scale")


def test_cuttings_agree_bitwise_in_float32(tiny_model_dirs, plain_logits, tmp_path):
    """In the 32-bit path every kernel reduces in an order that depends on the
    token's position alone, so all cuttings give the same bits."""
    cfg, reqs, _ = plain_logits["b"]
    trace = ru.Trace()
    ru.mixed(trace, reqs)
    ru.whole(trace, reqs)
    ru.portions(trace, reqs)
    out = ru.run_trace(tiny_model_dirs["b"], "float32", trace, tmp_path / "o", page_size=32)
    got = ru.read_rows(out, trace, cfg["vocab_size"])
    for i, r in enumerate(reqs):
        for p in range(len(r)):
            assert torch.equal(got[(f"w{i}", p)], got[(f"m{i}", p)]), (i, p)
            assert torch.equal(got[(f"w{i}", p)], got[(f"p{i}", p)]), (i, p)
