"""Generation through the Python entry point and the command line on the GPU:
greedy and temperature tokens against the plain implementation, under small token
budgets and a pool so small that requests are preempted; long decoding through
the CUDA-graph path; the first tokens of a sequence."""

import json
import subprocess
import sys

import pytest
import torch

from tests import plain_qwen3
from tests.rounding import divergence_is_a_rounding_flip
from tests.conftest import ROOT, TINY

pytestmark = pytest.mark.gpu


def _engine(model_dir, dtype, **kw):
    from deterministic_inference_b200 import Engine, EngineConfig
    base = dict(kv_pool_tokens=2048, page_size=16, max_reqs=16, max_seq_len=512)
    base.update(kw)
    return Engine(EngineConfig(model_path=str(model_dir), dtype=dtype, device="cuda:0", **base))


def _prompts(vocab, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab - 1, (n,), generator=g).tolist() for n in lens]


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_float32_equals_plain(name, tiny_model_dirs):
    from deterministic_inference_b200 import SamplingParams
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs[name])
    lens, n_new = ((5, 17, 33), 8) if name == "a" else ((1, 9, 31, 64, 100), 12)
    prompts = _prompts(cfg["vocab_size"], lens, 1 if name == "a" else 4)
    want = [plain_qwen3.generate(cfg, w, p, n_new) for p in prompts]
    page = TINY[name]["page_size"]
    tight = 64 if name == "a" else 160        # fewer tokens than the requests hold together
    for kw in (dict(), dict(max_prefill_tokens=13), dict(kv_pool_tokens=tight, max_prefill_tokens=32),
               dict(cuda_graphs=False)):
        eng = _engine(tiny_model_dirs[name], "float32", page_size=page, **kw)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=n_new, ignore_eos=True))
        assert [o.token_ids for o in outs] == want, kw
        eng.cache.check_invariants()
        assert eng.cache.num_free_pages() == eng.cache.usable_pages()
        if kw.get("kv_pool_tokens") == 160:
            assert sum(o.num_preemptions for o in outs) > 0      # the pool did run out


def test_temperature_float32_equals_plain(tiny_model_dirs):
    from deterministic_inference_b200 import SamplingParams
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs["a"])
    prompts = _prompts(cfg["vocab_size"], (5, 17, 33), 1)
    for kw in (dict(), dict(top_k=20, top_p=0.9)):
        want = [plain_qwen3.generate(cfg, w, p, 8, 0.8, 7, **kw) for p in prompts]
        for ekw in (dict(), dict(max_prefill_tokens=8)):
            eng = _engine(tiny_model_dirs["a"], "float32", **ekw)
            outs = eng.generate(prompts, SamplingParams(temperature=0.8, seed=7, max_new_tokens=8,
                                                        ignore_eos=True, **kw))
            assert [o.token_ids for o in outs] == want, (kw, ekw)


@pytest.mark.parametrize("name", ["a", "b", "bw", "c"])
def test_greedy_bfloat16_follows_plain(name, tiny_model_dirs):
    from deterministic_inference_b200 import SamplingParams
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs[name])
    prompts = _prompts(cfg["vocab_size"], (3, 20, 47), 5)
    want = [plain_qwen3.generate(cfg, w, p, 10) for p in prompts]
    eng = _engine(tiny_model_dirs[name], "bfloat16", page_size=TINY[name]["page_size"],
                  max_prefill_tokens=24)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    for p, o, wnt in zip(prompts, outs, want):
        ok, why = divergence_is_a_rounding_flip(cfg, w, p, o.token_ids, wnt)
        assert ok, (why, o.token_ids, wnt)
        assert len(o.token_ids) == len(wnt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs(dtype, tiny_model_dirs):
    """200 decoded tokens cross page, split and width-bucket edges; with and
    without CUDA graphs the tokens are the same, and in float32 they equal the plain
    implementation's."""
    from deterministic_inference_b200 import SamplingParams
    name = "bw"
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs[name])
    prompts = _prompts(cfg["vocab_size"], (7, 30), 6)
    sp = SamplingParams(max_new_tokens=200, ignore_eos=True)
    a = _engine(tiny_model_dirs[name], dtype, page_size=16).generate(prompts, sp)
    eng = _engine(tiny_model_dirs[name], dtype, page_size=16, cuda_graphs=False)
    b = eng.generate(prompts, sp)
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    if dtype == "float32":
        want = [plain_qwen3.generate(cfg, w, p, 200) for p in prompts]
        assert [o.token_ids for o in a] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype, tiny_model_dirs):
    """Prompts of one and two tokens (positions 0 and 1), decoded from there."""
    from deterministic_inference_b200 import SamplingParams
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs["c"])
    prompts = [[5], [7, 250], [1, 2, 3]]
    want = [plain_qwen3.generate(cfg, w, p, 5) for p in prompts]
    outs = _engine(tiny_model_dirs["c"], dtype).generate(
        prompts, SamplingParams(max_new_tokens=5, ignore_eos=True))
    if dtype == "float32":
        assert [o.token_ids for o in outs] == want
    else:
        for p, o, wnt in zip(prompts, outs, want):
            ok, why = divergence_is_a_rounding_flip(cfg, w, p, o.token_ids, wnt)
            assert ok, (why, o.token_ids, wnt)


def test_command_line(tiny_model_dirs):
    cfg, w = plain_qwen3.read_model_dir(tiny_model_dirs["a"])
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    want = plain_qwen3.generate(cfg, w, prompt, 6)
    out = subprocess.run(
        [sys.executable, "-m", "deterministic_inference_b200", "generate", "--model",
         str(tiny_model_dirs["a"]), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
         "--max-new-tokens", "6", "--ignore-eos", "--kv-pool-tokens", "512", "--max-seq-len", "256"],
        cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["token_ids"] == want and rec["finish_reason"] == "length"


def test_preset_with_random_weights_on_the_device():
    """``model_config`` + ``random_seed``: no folder; the same seed gives the same tokens."""
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams, preset
    outs = []
    for _ in range(2):
        eng = Engine(EngineConfig(model_config=preset("tiny_b"), random_seed=3, dtype="bfloat16",
                                  kv_pool_tokens=512, page_size=32, max_reqs=4, max_seq_len=256,
                                  device="cuda:0"))
        outs.append(eng.generate([[1, 2, 3, 4, 5]], SamplingParams(max_new_tokens=8, ignore_eos=True))[0].token_ids)
    assert outs[0] == outs[1] and len(outs[0]) == 8


@pytest.mark.parametrize("name,layers", [("qwen3_0_6b", 2), ("qwen3_8b", 2), ("qwen3_32b", 1)])
def test_published_shapes_run(name, layers):
    """The layer sizes of the three benchmark shapes (16/8, 32/8 and 64/8 heads of 128,
    widths 1024/4096/5120, intermediate 3072/12288/25600, vocabulary 151936) with a few
    layers and random weights drawn on the device: a prompt in two portions, a second
    request, then decoding through the graph path; every kernel takes its fast path
    without complaint and the float32 engine agrees on the first tokens."""
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams, preset
    from deterministic_inference_b200.kernels import attention_bf16, gemm_bf16, ops
    cfg = preset(name, num_hidden_layers=layers, max_window_layers=layers)
    prompts = _prompts(cfg.vocab_size, (300, 37), 9)
    outs = {}
    for dtype in ("bfloat16", "float32"):
        eng = Engine(EngineConfig(model_config=cfg, random_seed=1, dtype=dtype, kv_pool_tokens=2048,
                                  max_reqs=8, max_seq_len=1024, max_prefill_tokens=256,
                                  device="cuda:0"))
        n = 24 if dtype == "bfloat16" else 3
        outs[dtype] = [o.token_ids for o in eng.generate(
            prompts, SamplingParams(max_new_tokens=n, ignore_eos=True))]
        del eng
        torch.cuda.empty_cache()
    assert all(len(t) == 24 for t in outs["bfloat16"])
    assert gemm_bf16.status() == 0
    assert ops._lib("attention_bf16").dib_attention_bf16_status() == 0
    # the first token of each request agrees with the 32-bit path (later ones may flip on
    # near ties of a random model's flat logits)
    assert [t[0] for t in outs["bfloat16"]] == [t[0] for t in outs["float32"]]


@pytest.mark.parametrize("name,layers", [("qwen3_0_6b", 2), ("qwen3_8b", 2), ("qwen3_32b", 1)])
def test_published_shapes_logits_agree_across_dtypes(name, layers):
    """At the benchmark layer sizes the bfloat16 and the float32 step give the same
    logits up to bfloat16 storage (about 1% of the largest logit after a few layers):
    a kernel that mishandles a width, a head count or an intermediate size in one of the
    two paths shows here as a difference of the logits' own size."""
    from deterministic_inference_b200 import EngineConfig, preset
    from deterministic_inference_b200.engine.batch import SequenceInput
    from deterministic_inference_b200.engine.runner import ModelRunner
    cfg = preset(name, num_hidden_layers=layers, max_window_layers=layers)
    toks = _prompts(cfg.vocab_size, (300,), 9)[0]
    res = {}
    for dtype in ("bfloat16", "float32"):
        r = ModelRunner(EngineConfig(model_config=cfg, random_seed=1, dtype=dtype, kv_pool_tokens=1024,
                                     max_reqs=4, max_seq_len=512, device="cuda:0"))
        slot = r.cache.allocate_slot()
        r.step([SequenceInput(slot, toks[:200], 0, [])])
        logits, _ = r.step([SequenceInput(slot, toks[200:], 200, [0, 50, 99])])
        res[dtype] = logits.float().cpu()
        del r
        torch.cuda.empty_cache()
    a, b = res["bfloat16"], res["float32"]
    assert (a - b).abs().max().item() <= 0.03 * b.abs().max().item()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_replayed_as_graphs_give_the_bits_of_launched_steps(dtype, tiny_model_dirs):
    """Steps whose bucket of shapes comes again are captured and replayed as CUDA graphs
    (from the third time on): prompts of six lengths of one bucket (33 to 48 tokens) one after
    the other, a two-sequence mixed step with portions of 3 to 7 tokens, decode steps, steps of
    three or four decoded tokens beside a portion (one bucket: padding entries fill it).  Every
    step's logits equal, bit for bit, those of a runner that launches every step kernel by
    kernel with no row of padding; and the graphs were in fact used, one for each bucket."""
    from deterministic_inference_b200 import EngineConfig
    from deterministic_inference_b200.engine.batch import SequenceInput
    from deterministic_inference_b200.engine.runner import ModelRunner
    model_dir = tiny_model_dirs["b"]
    vocab = plain_qwen3.read_model_dir(model_dir)[0]["vocab_size"]
    runners = [ModelRunner(EngineConfig(model_path=str(model_dir), dtype=dtype, device="cuda:0",
                                        kv_pool_tokens=4096, page_size=TINY["b"]["page_size"],
                                        max_reqs=16, max_seq_len=512, cuda_graphs=g)) for g in (True, False)]
    assert runners[0].step_graphs is not None and runners[1].step_graphs is None
    lens = (40, 37, 48, 33, 45, 41)
    portions = (5, 3, 7, 4, 6)
    prompts = _prompts(vocab, lens + (25,) * 10, 21)
    outs = [[], []]
    for k, r in enumerate(runners):
        slots = [r.cache.allocate_slot() for _ in prompts]
        pos = list(lens)                                            # tokens of the first six requests in the cache

        def done(logits):
            torch.cuda.synchronize()        # the step graphs decide by a finished step's times
            return logits.clone()

        for s, p in zip(slots[:6], prompts[:6]):                    # one bucket, six lengths
            outs[k].append(done(r.step([SequenceInput(s, p, 0, [0, len(p) - 1])])[0]))

        def decodes(which, token):
            es = [SequenceInput(slots[i], [token], pos[i], [0]) for i in which]
            for i in which:
                pos[i] += 1
            return es

        for rep in range(5):                                        # a decode beside a portion
            n = portions[rep]
            outs[k].append(done(r.step([SequenceInput(slots[6 + rep], prompts[6 + rep][:n], 0, [n - 1])]
                                       + decodes((0,), rep + 1))[0]))
        for step in range(6):                                       # pure decode of three requests
            outs[k].append(done(r.step(decodes((1, 2, 3), step + 7))[0]))
        for rep in range(5):                                        # three or four decodes beside a portion:
            n = portions[rep]                                       # one bucket of four one-token sequences
            which = (1, 2, 3, 4) if rep % 2 else (5, 2, 4)
            logits, batch = r.step(decodes(which, rep + 20)
                                   + [SequenceInput(slots[11 + rep], prompts[11 + rep][:n], 0, [n - 1])])
            assert len(batch.logit_rows) == len(which) + 1 and all(len(x) == 1 for x in batch.logit_rows)
            outs[k].append(done(logits[[x[0] for x in batch.logit_rows]]))
    assert len(outs[0]) == len(outs[1]) == 22
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    g = runners[0].step_graphs
    assert g.captures == 3 and g.replays == 4 + 3 + 3       # the three buckets, from their third step on
    assert runners[0].decode_graphs.replays == 6            # the pure-decode steps


def test_long_prompts_and_a_wide_decode_batch_against_plain(tiny_model_dirs):
    """At the benchmark's layer sizes (model "f": width 1,024, 16 + 8 heads of 128, a window
    on the second layer, sharpened weights): 24 requests with prompts of 1,200 to 1,400
    tokens, three of them fed in portions of 512, the others whole seven at a time, then
    all decoded together for a few steps through the replayed graph.  The bfloat16 steps
    take the tcgen05 prompt kernel behind cached prefixes over many key tiles and the
    decode attention that walks many splits per CTA; the logits of six of the requests are
    compared with the plain implementation (bfloat16 storage emulated) under the bound of
    the replay tests."""
    from deterministic_inference_b200 import EngineConfig
    from deterministic_inference_b200.engine.batch import SequenceInput
    from deterministic_inference_b200.engine.runner import ModelRunner
    from tests.test_replay_gpu import BF16_FRAC, BF16_ROUNDING_SHARE
    model_dir = tiny_model_dirs["f"]
    cfg, w = plain_qwen3.read_model_dir(model_dir)
    n_req, steps = 24, 4
    g = torch.Generator().manual_seed(31)
    lens = torch.randint(1200, 1401, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n + steps,), generator=g).tolist() for n in lens]
    r = ModelRunner(EngineConfig(model_path=str(model_dir), dtype="bfloat16", kv_pool_tokens=40960,
                                 max_reqs=32, max_seq_len=2048, device="cuda:0"))
    slots = [r.cache.allocate_slot() for _ in range(n_req)]
    got = {}                                               # (request, position) -> logits row
    for i in (0, 7, 23):                                   # three prompts portion by portion
        for a in range(0, lens[i], 512):
            b = min(lens[i], a + 512)
            lg, _ = r.step([SequenceInput(slots[i], prompts[i][a:b], a, [b - a - 1] if b == lens[i] else [])])
        got[(i, lens[i] - 1)] = lg[0].float().cpu()
    rest = [i for i in range(n_req) if i not in (0, 7, 23)]
    for k in range(0, len(rest), 7):                        # the others whole, seven at a time
        group = rest[k:k + 7]
        lg, batch = r.step([SequenceInput(slots[i], prompts[i][:lens[i]], 0, [lens[i] - 1]) for i in group])
        for i, rows in zip(group, batch.logit_rows):
            got[(i, lens[i] - 1)] = lg[rows[0]].float().cpu()
    for s in range(steps):                                  # all decode together, given tokens
        lg, batch = r.step([SequenceInput(slots[i], [prompts[i][lens[i] + s]], lens[i] + s, [0])
                            for i in range(n_req)])
        for i, rows in enumerate(batch.logit_rows):
            got[(i, lens[i] + s)] = lg[rows[0]].float().cpu()
    assert r.decode_graphs.replays == steps
    from deterministic_inference_b200.kernels import ops
    ops.check_kernel_status()
    for i in (0, 7, 23, 3, 12, 18):
        emu = plain_qwen3.forward(cfg, w, prompts[i], store_bf16=True)
        p32 = plain_qwen3.forward(cfg, w, prompts[i])
        yard = float((emu - p32).abs().max())
        for pos in range(lens[i] - 1, lens[i] + steps):
            want = emu[pos]
            scale = max(1.0, float(want.abs().max()))
            err = float((got[(i, pos)].double() - want.double()).abs().max())
            assert err <= max(BF16_FRAC * scale, BF16_ROUNDING_SHARE * yard), (i, pos, err, scale, yard)


@pytest.mark.parametrize("name", ["d", "e"])
def test_bfloat16_bits_of_a_token_do_not_depend_on_its_step(name, tiny_model_dirs):
    """With ``library_products=False`` every bfloat16 kernel adds up in an order that
    depends on the token's own position and the weights' shapes alone.  So the logits of
    a request are the same bits (a) alone and beside three other requests of other
    lengths, (b) launched kernel by kernel and replayed from a captured graph, also one
    captured for a bucket of longer portions, (c) with its prompt cut into portions of 512,
    of 500 and of 100 tokens.  Heads of 128: the tcgen05
    prompt kernel in its paired, neighbour and single-tile forms, the TMA decode kernels,
    the package's matrix product at 1 to 1,700 rows."""
    from deterministic_inference_b200 import EngineConfig
    from deterministic_inference_b200.engine.batch import SequenceInput
    from deterministic_inference_b200.engine.runner import ModelRunner
    model_dir = tiny_model_dirs[name]
    vocab = plain_qwen3.read_model_dir(model_dir)[0]["vocab_size"]
    g = torch.Generator().manual_seed(77)
    main = torch.randint(0, vocab, (1000,), generator=g).tolist()
    others = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (700, 40, 333)]
    want_places = [0, 99, 100, 511, 512, 998, 999]

    def runner(graphs):
        return ModelRunner(EngineConfig(model_path=str(model_dir), dtype="bfloat16", device="cuda:0",
                                        kv_pool_tokens=8192, page_size=TINY[name]["page_size"], max_reqs=16,
                                        max_seq_len=1024, cuda_graphs=graphs, library_products=False))

    def feed(r, portion, beside=(), decode_tail=8):
        """The main request in portions of ``portion`` tokens (its last tokens one by one),
        each step together with the next portions of the ``beside`` requests; returns its
        logits at ``want_places`` and at the single tokens."""
        slot = r.cache.allocate_slot()
        oslots = [r.cache.allocate_slot() for _ in beside]
        odone = [0] * len(beside)
        rows, c = {}, 0
        while c < len(main):
            left = len(main) - c
            n = 1 if left <= decode_tail else min(portion, left - decode_tail)
            want = [p - c for p in want_places if c <= p < c + n] if n > 1 else [0]
            entries = [SequenceInput(slot, main[c:c + n], c, want)]
            for i, o in enumerate(beside):
                if odone[i] < len(o):
                    m = min(1 if odone[i] > len(o) - 5 else 150, len(o) - odone[i])
                    entries.append(SequenceInput(oslots[i], o[odone[i]:odone[i] + m], odone[i], []))
                    odone[i] += m
            logits, batch = r.step(entries)
            for w, row in zip(want, batch.logit_rows[0]):
                rows[c + w] = logits[row].clone()
            c += n
        for s in [slot] + oslots:
            r.cache.release_slot(s)
        return rows

    base = feed(runner(False), 512)
    assert sorted(base) == sorted(set(want_places) | set(range(992, 1000)))
    variants = {
        "beside three others": feed(runner(False), 512, beside=others),
        "portions of 100": feed(runner(False), 100),
        "portions of 100 beside others": feed(runner(False), 100, beside=others),
    }
    r = runner(True)
    for _ in range(3):                      # the third time every repeated shape is replayed
        variants["replayed"] = feed(r, 512)
    assert r.step_graphs.replays >= 2 and r.decode_graphs.replays >= 8
    # portions of 500 and 492 tokens: the third time they run through graphs captured for 512
    # and 496 token rows, the rest of which is padding
    before = r.step_graphs.replays
    for _ in range(3):
        variants["replayed with padding rows"] = feed(r, 500)
    assert r.step_graphs.replays == before + 2
    assert {k[0][0] for k in r.step_graphs.graphs} >= {512, 496}
    for what, rows in variants.items():
        for p, row in base.items():
            assert torch.equal(rows[p], row), (what, p)
    from deterministic_inference_b200.kernels import gemm_bf16
    gemm_bf16.set_library_products(True)


def test_generation_with_debug_checks_on(tiny_model_dirs):
    """``debug_checks=True``: every step's metadata (launched steps, replayed graphs and their
    padding sequences) passes the host-side checks and the tokens are those of an engine
    without them."""
    from deterministic_inference_b200 import SamplingParams
    cfg = plain_qwen3.read_model_dir(tiny_model_dirs["bw"])[0]
    prompts = _prompts(cfg["vocab_size"], (3, 20, 47, 20, 20), 5)
    sp = SamplingParams(max_new_tokens=40, ignore_eos=True)
    outs = []
    for debug in (True, False):
        eng = _engine(tiny_model_dirs["bw"], "bfloat16", page_size=16, max_prefill_tokens=24,
                      kv_pool_tokens=512, debug_checks=debug)
        outs.append([o.token_ids for o in eng.generate(prompts, sp)])
        if debug:
            assert eng.runner.decode_graphs.replays > 0 and eng.runner._check is not None
    assert outs[0] == outs[1]
