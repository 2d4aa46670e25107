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

# tolerance against the float32 plain implementation
#   float32: reduction-order noise only
#   bfloat16: the reference's class of tolerance for bfloat16 kernels
#             (tests/conftest.py:35-37 there), on logits of unit scale
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=4e-2, rtol=4e-2)}


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
        reqs = _requests(cfg["vocab_size"], lens, seed)
        out[name] = (cfg, reqs, [plain_qwen3.forward(cfg, w, r) for r in reqs])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings(name, dtype, tiny_model_dirs, plain_logits, tmp_path):
    cfg, reqs, ref = plain_logits[name]
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
    worst = 0.0
    for (key, pos), row in got.items():
        i = int(key[1:])
        want = ref[i][pos]
        worst = max(worst, float((row - want).abs().max()))
        try:
            torch.testing.assert_close(row, want, **TOL[dtype])
        except AssertionError as e:
            raise AssertionError(f"{name}/{dtype}: request {key} position {pos} "
                                 f"(first wrong token of this cutting): {e}") from None
    # every cutting covered every position of every request
    for kind in "mwtp":
        for i, r in enumerate(reqs):
            assert all((f"{kind}{i}", p) in got for p in range(len(r))), (kind, i)
    print(f"{name}/{dtype}: worst abs diff {worst:.3e}")


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
