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
    # heads of 128: lengths around the tiles of 128 keys and rows, up to several tiles
    "d": ([5, 129, 300, 517, 700], 12),
    "e": ([64, 128, 257, 390, 655], 14),
    # benchmark layer sizes: prompts of many key tiles and decode over many splits
    "f": ([1300, 150, 2100, 700], 16),
}
# portion sizes of the "portions" and "mixed" cuttings: the long requests of the head-128
# models also get portions above 128 rows (the library's matrix product, several query
# tiles per sequence) beside the small ones
SIZES = {
    "d": dict(portions=(13, 130, 2, 257, 5, 2, 64, 200, 3), mixed=(11, 150, 2, 17, 129, 5, 2, 300, 3)),
    "e": dict(portions=(200, 7, 2, 131, 2, 31, 256, 3), mixed=(140, 2, 17, 260, 5, 2, 29, 3)),
    "f": dict(portions=(512, 100, 2, 700, 129, 31), mixed=(400, 2, 130, 512, 17, 257, 3)),
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


def check_rows(name, dtype, got, refs):
    """Every written row against the plain implementation, within the bounds of this file's
    header; returns the worst difference as a share of its row's scale."""
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
        WORST_SHARE[(name, dtype)] = max(WORST_SHARE.get((name, dtype), 0.0), err / max(yard[i], 1e-30))
    return worst


WORST_SHARE: dict = {}     # (case, dtype) -> largest difference seen, in units of the request's yardstick


def covered(got, reqs, kinds):
    """Every cutting wrote every position of every request."""
    for kind in kinds:
        for i, r in enumerate(reqs):
            assert all((f"{kind}{i}", p) in got for p in range(len(r))), (kind, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings(name, dtype, tiny_model_dirs, plain_logits, tmp_path):
    cfg, reqs, refs = plain_logits[name]
    page = TINY[name]["page_size"]
    sizes = SIZES.get(name, {})
    trace = ru.Trace()
    # the mixed cutting first sizes the pool; the others reuse it one request at a time
    ru.mixed(trace, reqs, **({"sizes": sizes["mixed"]} if sizes else {}))
    ru.whole(trace, reqs)
    ru.last_one_by_one(trace, reqs)
    ru.portions(trace, reqs, **({"sizes": sizes["portions"]} if sizes else {}))
    out = ru.run_trace(tiny_model_dirs[name], dtype, trace, tmp_path / "out", page_size=page)
    got = ru.read_rows(out, trace, cfg["vocab_size"])
    assert got, "the trace wrote nothing"
    worst = check_rows(name, dtype, got, refs)
    covered(got, reqs, "mwtp")
    print(f"{name}/{dtype}: worst diff {worst:.3e} of the row's scale, "
          f"{WORST_SHARE[(name, dtype)]:.3f} of the request's yardstick")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["d", "e", "b"])
def test_replay_with_captured_graphs(name, dtype, tiny_model_dirs, tmp_path):
    """The step function as generation runs it: pure-decode steps and steps whose shape
    has come twice before are replayed as captured CUDA graphs.  Four requests of one
    length, cut alike, so that every shape repeats (portions of 96 and of 200 tokens, then
    single tokens), and the mixed cutting on top; every row against the plain
    implementation, and the replayed run against a launched run of the same trace: equal
    bits (a captured step sizes its grids for the longest sequence its block-table width
    allows, which must not change what a row adds up).  A replayed step runs with its bucket's
    row count and the launched run of this test with the step's own, so both runs keep every
    matrix product on the few-rows kernel, whose sums do not depend on the row count (which
    product kernel a row count selects is the one thing a bucket may change; the many-rows
    kernels under graphs are compared in test_generate_gpu.py with lengths on bucket lines)."""
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs[name])
    _, w64 = plain_qwen3.read_model_dir(tiny_model_dirs[name], torch.float64)
    n = 200 if name == "b" else 520
    same = _requests(cfg["vocab_size"], [n] * 4, 41)
    other = _requests(cfg["vocab_size"], [33, 150, 77], 42)
    reqs = same + other
    refs = {"float64": [plain_qwen3.forward(cfg, w64, r) for r in reqs],
            "float32": [plain_qwen3.forward(cfg, w, r) for r in reqs],
            "bfloat16": [plain_qwen3.forward(cfg, w, r, store_bf16=True) for r in reqs]}
    trace = ru.Trace()
    passes = {"": 96, "x": 96, "y": 200, "z": 200}     # every shape of a pass comes again in the next
    for prefix, portion in passes.items():
        ru.lockstep(trace, same, portion=portion, prefix=prefix)
    ru.mixed(trace, reqs)
    page = TINY[name]["page_size"]
    outs = {}
    for graphs in (True, False):
        out = ru.run_trace(tiny_model_dirs[name], dtype, trace, tmp_path / f"out{int(graphs)}",
                           page_size=page, cuda_graphs=graphs,
                           extra_env={"DIB200_GEMM_MAX_ROWS": "1000000"})
        outs[graphs] = ru.read_rows(out, trace, cfg["vocab_size"])
    for key_pos, row in outs[True].items():
        assert torch.equal(row, outs[False][key_pos]), key_pos
    worst = 0.0
    for prefix in passes:                              # "xl0" is request 0 again
        got = {(k[len(prefix):], pos): row for (k, pos), row in outs[True].items()
               if k.startswith(prefix + "l")}
        worst = max(worst, check_rows(name, dtype, got, refs))
        covered(got, same, "l")
    got = {kp: row for kp, row in outs[True].items() if kp[0].startswith("m")}
    worst = max(worst, check_rows(name, dtype, got, refs))
    covered(got, reqs, "m")
    print(f"{name}/{dtype} with graphs: worst diff {worst:.3e} of the row's scale, "
          f"{WORST_SHARE[(name, dtype)]:.3f} of the request's yardstick")


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
