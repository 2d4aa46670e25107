"""The engine's host logic (cache manager, batch packing, step function, scheduler,
entry point) on a machine without a GPU: the kernel wrappers are replaced by their
plain PyTorch restatements (fixture ``torch_ops``), everything else is the product
code.  Logits and tokens are compared with the plain implementation under every
cutting.  The GPU tests repeat this with the real kernels."""

import pytest
import torch

from deterministic_inference_b200.config import EngineConfig, SamplingParams
from deterministic_inference_b200.engine import Engine, ModelRunner, SequenceInput
from tests import plain_qwen3
from tests.conftest import TINY


def runner_for(model_dir, page, pool=512, **kw):
    return ModelRunner(EngineConfig(model_path=str(model_dir), dtype="float32", device="cpu",
                                    kv_pool_tokens=pool, page_size=page, max_reqs=8,
                                    max_seq_len=512, **kw))


@pytest.mark.parametrize("name", ["a", "bw", "c"])
def test_cuttings_on_cpu(name, tiny_model_dirs, torch_ops):
    d = tiny_model_dirs[name]
    cfg, w = plain_qwen3.read_model_dir(d)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg["vocab_size"], (75,), generator=g).tolist()
    other = torch.randint(0, cfg["vocab_size"], (40,), generator=g).tolist()
    ref, ref_other = plain_qwen3.forward(cfg, w, toks), plain_qwen3.forward(cfg, w, other)
    r = runner_for(d, TINY[name]["page_size"], pool=192)
    tol = dict(atol=2e-5, rtol=1e-4)

    # whole, wanting a subset of places
    s = r.cache.allocate_slot()
    logits, _ = r.step([SequenceInput(s, toks, 0, [0, 5, 74])])
    torch.testing.assert_close(logits, ref[[0, 5, 74]], **tol)
    r.cache.release_slot(s)

    # portions of changing size beside another request that decodes token by token
    s, o = r.cache.allocate_slot(), r.cache.allocate_slot()
    r.step([SequenceInput(o, other[:20], 0, [])])
    c, oc = 0, 20
    for n in (13, 2, 7, 2, 30, 5, 16):
        entries = [SequenceInput(s, toks[c:c + n], c, list(range(n)))]
        if oc < len(other):
            entries.insert(0, SequenceInput(o, other[oc:oc + 1], oc, [0]))
        logits, batch = r.step(entries)
        rows = batch.logit_rows
        torch.testing.assert_close(logits[rows[-1]], ref[c:c + n], **tol)
        if len(entries) == 2:
            torch.testing.assert_close(logits[rows[0]], ref_other[oc:oc + 1], **tol)
            oc += 1
        c += n
    assert c == 75
    r.cache.release_slot(s)
    r.cache.release_slot(o)
    r.cache.check_invariants()


def test_entry_point_matches_plain_generation(tiny_model_dirs, torch_ops):
    d = tiny_model_dirs["a"]
    cfg, w = plain_qwen3.read_model_dir(d)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 255, (n,), generator=g).tolist() for n in (5, 17, 33)]
    for temp, kw in ((0.0, {}), (0.8, dict(top_k=20, top_p=0.9))):
        sp = SamplingParams(temperature=temp, seed=7, max_new_tokens=8, ignore_eos=True, **kw)
        want = [plain_qwen3.generate(cfg, w, p, 8, temp, 7, **kw) for p in prompts]
        for ekw in (dict(kv_pool_tokens=1024), dict(kv_pool_tokens=1024, max_prefill_tokens=8),
                    dict(kv_pool_tokens=64, max_prefill_tokens=16),
                    dict(kv_pool_tokens=1024, async_scheduling=False),
                    dict(kv_pool_tokens=64, max_prefill_tokens=16, async_scheduling=False)):
            eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", page_size=16,
                                      max_reqs=8, max_seq_len=256, **ekw))
            outs = eng.generate(prompts, sp)
            assert [o.token_ids for o in outs] == want, (temp, ekw)
            assert [o.finish_reason for o in outs] == ["length"] * 3
            eng.cache.check_invariants()
            assert eng.cache.num_free_pages() == eng.cache.usable_pages()


@pytest.mark.parametrize("async_scheduling", [True, False])
def test_eos_ends_a_request(tiny_model_dirs, torch_ops, async_scheduling):
    """With tokens read one step late a request that stops on a token has been fed one
    token too many; nothing of that shows in its output or in the cache's books."""
    d = tiny_model_dirs["a"]
    cfg, w = plain_qwen3.read_model_dir(d)
    prompts = [[3, 1, 4, 1, 5], [9, 2, 6, 5, 3, 5, 8]]
    free = [plain_qwen3.generate(cfg, w, p, 6) for p in prompts]
    eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=256,
                              max_reqs=4, max_seq_len=256, async_scheduling=async_scheduling))
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=6, stop_token_ids=[free[0][2]]),
                                  SamplingParams(max_new_tokens=6, ignore_eos=True)])
    cut = free[0].index(free[0][2]) + 1
    assert outs[0].token_ids == free[0][:cut] and outs[0].finish_reason == "stop"
    assert outs[1].token_ids == free[1] and outs[1].finish_reason == "length"
    eng.cache.check_invariants()
    assert eng.cache.num_free_pages() == eng.cache.usable_pages() and not eng.has_work()


def test_add_request_refuses_what_can_never_run(tiny_model_dirs, torch_ops):
    eng = Engine(EngineConfig(model_path=str(tiny_model_dirs["a"]), dtype="float32", device="cpu",
                              kv_pool_tokens=64, max_reqs=4, max_seq_len=128))
    with pytest.raises(ValueError, match="cache pool"):
        eng.add_request(prompt_ids=[1] * 60, params=SamplingParams(max_new_tokens=10))
    with pytest.raises(ValueError, match="position limit"):
        eng.add_request(prompt_ids=[1] * 10, params=SamplingParams(max_new_tokens=200))
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request(prompt_ids=[1, 999])
    with pytest.raises(ValueError, match="empty"):
        eng.add_request(prompt_ids=[])


def test_no_cpu_path_in_the_product():
    """Without the test's stand-ins the engine refuses CPU tensors loudly."""
    from deterministic_inference_b200.kernels import ops
    from deterministic_inference_b200.kernels.ops import KernelError
    with pytest.raises(KernelError, match="no CPU path"):
        ops.rms_norm(torch.randn(2, 8), torch.ones(8), 1e-6)
    with pytest.raises(KernelError, match="no CPU path"):
        ops.linear(torch.randn(2, 8), torch.randn(4, 8))


def test_prompt_tile_lists_name_every_tile_once():
    """The lists of query tiles that the prompt attention kernels take (a CTA per pair of
    tiles from both ends of a prompt, per pair of neighbours, per tile, per chunk of a
    pair's key range) name every tile of every prompt sequence exactly once per chunk it
    needs, never a tile of a decoding sequence, and pair only tiles of one sequence."""
    import random
    from deterministic_inference_b200.kernels.attention_bf16 import (extend_chunk_units, extend_tile_pairs,
                                                                     extend_tiles)
    rng = random.Random(5)
    for _ in range(200):
        nd = rng.randint(0, 3)
        q_lens = [1] * nd + [rng.choice([1, 2, 63, 64, 65, 128, 129, rng.randint(1, 1500)])
                             for _ in range(rng.randint(1, 5))]
        kv_lens = [q + rng.choice([0, 0, 1, 700, 5000]) for q in q_lens]
        tpt = rng.choice([8, 64, 128])
        want = sorted((s, t0) for s in range(nd, len(q_lens)) for t0 in range(0, q_lens[s], tpt))
        seqs, starts = extend_tiles(q_lens, nd, tpt)
        assert sorted(zip(seqs, starts)) == want
        for window, alone, neighbours in ((0, False, False), (0, True, False), (0, False, True), (300, False, False)):
            seqs, a, b = extend_tile_pairs(q_lens, kv_lens, nd, tpt, window, alone, neighbours)
            got = sorted([(s, x) for s, x in zip(seqs, a)] + [(s, y) for s, y in zip(seqs, b) if y >= 0])
            assert got == want, (q_lens, tpt, window, alone, neighbours)
            assert all(x >= 0 and (y < 0 or y != x) for x, y in zip(a, b))
            if alone:
                assert all(y < 0 for y in b)
        chunk_tiles = rng.choice([1, 8, 11])
        seqs, a, b, chunks = extend_chunk_units(q_lens, kv_lens, nd, tpt, chunk_tiles)
        span = chunk_tiles * 128
        need = []
        for s in range(nd, len(q_lens)):
            prefix = kv_lens[s] - q_lens[s]
            for t0 in range(0, q_lens[s], 2 * tpt):
                last = prefix + min(t0 + 2 * tpt, q_lens[s]) - 1
                need += [(s, t0, c) for c in range(last // span + 1)]
        assert sorted(zip(seqs, a, chunks)) == sorted(need)
        assert all(y < 0 or y == x + tpt for x, y in zip(a, b))


@pytest.mark.parametrize("seed", [2553, 2734, 2789])
def test_a_request_preempted_with_its_last_token_in_flight_retires(seed, tiny_model_dirs, torch_ops):
    """Tokens are read one step late.  A request can be preempted in the very step whose
    in-flight token is its last: it is then finished while it waits, holds nothing, and has
    to be retired from the waiting queue.  Re-admitted it would run a first portion without
    a logits row (its prompt plus outputs exceed the token budget), never be scheduled
    again and keep ``has_work()`` true for ever.  These draws (pool of 48 tokens, budget 8)
    reach that state."""
    import random
    d = tiny_model_dirs["a"]
    cfg, w = plain_qwen3.read_model_dir(d)
    rnd = random.Random(seed)
    pool, budget = rnd.choice([48, 64]), rnd.choice([8, 12, 16])
    eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", page_size=16,
                              kv_pool_tokens=pool, max_reqs=8, max_seq_len=256,
                              max_prefill_tokens=budget))
    prompts, news, rids = [], [], []
    for _ in range(rnd.randint(2, 4)):
        pl, mn = rnd.randint(10, 40), rnd.randint(1, 6)
        pl = min(pl, pool - mn)
        prompts.append([rnd.randrange(255) for _ in range(pl)])
        news.append(mn)
        rids.append(eng.add_request(prompt_ids=prompts[-1],
                                    params=SamplingParams(max_new_tokens=mn, ignore_eos=True)))
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
        assert steps < 400, (eng.scheduler.running, list(eng.scheduler.waiting))
    outs = [eng.get_output(r) for r in rids]
    assert sum(o.num_preemptions for o in outs) > 0
    assert [o.token_ids for o in outs] == [plain_qwen3.generate(cfg, w, p, n) for p, n in zip(prompts, news)]
    eng.cache.check_invariants()
    assert eng.cache.num_free_pages() == eng.cache.usable_pages()


def test_debug_checks_catch_bad_step_metadata(tiny_model_dirs, torch_ops):
    """``debug_checks``: every step's packed metadata is validated on the host before it
    reaches the device, and the cache's books after it.  A step that is in order passes;
    a token id outside the vocabulary, a block table that names a page outside the pool,
    keys on a page the sequence does not hold, and a logits row beyond the step's tokens are
    each refused by name."""
    import numpy as np
    from deterministic_inference_b200.engine.batch import (PackedLayout, StepCheckError, check_packed,
                                                           describe_step, fill_packed)
    d = tiny_model_dirs["bw"]          # two cache groups: all keys, and a window
    r = ModelRunner(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=256,
                                 page_size=16, max_reqs=8, max_seq_len=256, debug_checks=True))
    assert r._check is not None
    s = r.cache.allocate_slot()
    r.step([SequenceInput(s, list(range(40)), 0, [39])])        # in order: passes, books checked
    r.step([SequenceInput(s, [1], 40, [0])])
    with pytest.raises(StepCheckError, match="token id"):
        r.step([SequenceInput(s, [100000], 41, [0])])
    # the packed array itself, with one field spoilt at a time
    groups = list(r.cache.page_groups.values())
    entries = [SequenceInput(s, [5, 6, 7], 41, [2])]
    r.cache.allocate(s, 44)
    shape = describe_step(entries, r.cache)
    lay = PackedLayout(shape.t, 1, 1, shape.width, len(groups))
    host = np.zeros(lay.size, dtype=np.int32)
    fill_packed(host, lay, shape, r.cache, groups)
    vocab, maxpos = 512, 512
    check_packed(host, lay, r.cache, groups, vocab, maxpos)
    for field, value, message in ((("bt", 0), 10 ** 6, "block-table entry"), (("bt", 0), 0, "does not hold"),
                                  ("logit_indices", 3, "logits row"), ("positions", 600, "position"),
                                  (("sm", 1), 10 ** 7, "cache slot"), ("state_slots", 99, "state slot")):
        bad = host.copy()
        seg = lay.seg(bad, field)
        seg[-1 if field == ("bt", 0) and value == 0 else 0] = value
        if field == ("bt", 0) and value == 0:
            seg[2] = 0          # the page that holds keys 32..47
        with pytest.raises(StepCheckError, match=message):
            check_packed(bad, lay, r.cache, groups, vocab, maxpos)


def test_a_step_padded_to_a_bucket_keeps_its_rows_and_parks_the_rest_on_page_zero(tiny_model_dirs, torch_ops):
    """``fill_packed`` into a layout with more token rows and one more sequence than the step
    has (a captured graph's bucket, or a launched step that runs with its bucket's rows): the
    step's own rows, boundaries, lengths and block tables are those of the unpadded layout;
    the rows after them belong to one padding sequence on state slot 0 whose block table is
    all page 0, with positions inside one page and cache slots on page 0; the padded array
    passes the debug check.  A layout with several padding sequences gives each one token
    and the last the rest; layouts that do not fit are refused.  ``token_bucket`` rounds up
    by a sixteenth of an octave and names a lower bound of its bucket."""
    import numpy as np
    from deterministic_inference_b200.engine.batch import (PackedLayout, build_step_batch, check_packed,
                                                           describe_step, fill_packed)
    from deterministic_inference_b200.engine.graphs import StepGraphs, token_bucket
    d = tiny_model_dirs["bw"]
    r = ModelRunner(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=512,
                                 page_size=16, max_reqs=8, max_seq_len=256))
    s1, s2 = r.cache.allocate_slot(), r.cache.allocate_slot()
    r.step([SequenceInput(s1, list(range(30)), 0, [])])
    entries = [SequenceInput(s2, list(range(100, 137)), 0, [36]), SequenceInput(s1, [7], 30, [0])]
    for e in entries:
        r.cache.allocate(e.slot, e.num_computed + len(e.tokens))
    groups = list(r.cache.page_groups.values())
    shape = describe_step(entries, r.cache)
    assert shape.q_lens == [1, 37] and StepGraphs.padded_tokens(shape) == 1 + 48
    exact = PackedLayout(shape.t, 2, 2, shape.width, len(groups))
    padded = PackedLayout(49, 3, 2, shape.width + 3, len(groups))
    a, b = np.zeros(exact.size, dtype=np.int32), np.full(padded.size, 77, dtype=np.int32)
    fill_packed(a, exact, shape, r.cache, groups)
    fill_packed(b, padded, shape, r.cache, groups)
    for name in ("input_ids", "positions", "token_seq"):
        assert (padded.seg(b, name)[:38] == exact.seg(a, name)).all()
    assert padded.seg(b, "cu_q_lens").tolist() == [0, 1, 38, 49]
    assert padded.seg(b, "seq_lens").tolist() == [31, 37, 11] and padded.seg(b, "state_slots").tolist()[2] == 0
    assert (padded.seg(b, "token_seq")[38:] == 2).all() and (padded.seg(b, "input_ids")[38:] == 0).all()
    assert padded.seg(b, "positions")[38:].max() < 16
    assert padded.seg(b, "logit_indices").tolist() == exact.seg(a, "logit_indices").tolist()
    for gi in range(len(groups)):
        bt = padded.seg(b, ("bt", gi)).reshape(3, padded.width)
        assert (bt[2] == 0).all() and (bt[:2, :exact.width] == exact.seg(a, ("bt", gi)).reshape(2, exact.width)).all()
        assert (padded.seg(b, ("sm", gi))[:38] == exact.seg(a, ("sm", gi))).all()
        assert (padded.seg(b, ("sm", gi))[38:] < 16).all()
    check_packed(b, padded, r.cache, groups, 512, 512)
    # a padding sequence may be left without a token; a request's sequence may not
    tight = PackedLayout(38, 3, 2, shape.width, len(groups))
    c = np.zeros(tight.size, dtype=np.int32)
    fill_packed(c, tight, shape, r.cache, groups)
    assert tight.seg(c, "cu_q_lens").tolist() == [0, 1, 38, 38]
    check_packed(c, tight, r.cache, groups, 512, 512)
    # several padding sequences: one token each, the last takes the rest
    many = PackedLayout(38 + 6, 2 + 3, 2 + 3, shape.width, len(groups))
    m = np.zeros(many.size, dtype=np.int32)
    fill_packed(m, many, shape, r.cache, groups)
    assert many.seg(m, "cu_q_lens").tolist() == [0, 1, 38, 39, 40, 44]
    assert many.seg(m, "logit_indices").tolist()[2:] == [38, 39, 40]
    check_packed(m, many, r.cache, groups, 512, 512)
    for t, nb in ((37, 2), (40, 2), (39, 5)):        # fewer rows than tokens; rows without a sequence; too few rows
        lay = PackedLayout(t, nb, 2, shape.width, len(groups))
        with pytest.raises(ValueError, match="does not fit"):
            fill_packed(np.zeros(lay.size, dtype=np.int32), lay, shape, r.cache, groups)
    # padding sequences given as entries (state slot 0): one-token sequences come first, so they
    # follow the step's own one-token sequence; block table rows of zeros, cache slot 0
    with_dummies = entries + [SequenceInput(0, [0], 0, [0])] * 3
    shape4 = describe_step(with_dummies, r.cache)
    assert shape4.q_lens == [1, 1, 1, 1, 37] and shape4.order == [1, 2, 3, 4, 0] and shape4.slots[1:4] == [0, 0, 0]
    assert StepGraphs.padded_tokens(shape4) == 4 + 48 == StepGraphs.padded_tokens(shape) + 3
    lay4 = PackedLayout(4 + 48, 6, 5, shape.width, len(groups))
    d = np.zeros(lay4.size, dtype=np.int32)
    fill_packed(d, lay4, shape4, r.cache, groups)
    assert lay4.seg(d, "cu_q_lens").tolist() == [0, 1, 2, 3, 4, 41, 52]
    assert lay4.seg(d, "seq_lens").tolist() == [31, 1, 1, 1, 37, 11]
    assert lay4.seg(d, "logit_indices").tolist() == [0, 1, 2, 3, 40]
    for gi in range(len(groups)):
        bt = lay4.seg(d, ("bt", gi)).reshape(6, lay4.width)
        assert (bt[1:4] == 0).all() and (bt[5] == 0).all() and (lay4.seg(d, ("sm", gi))[1:4] == 0).all()
    check_packed(d, lay4, r.cache, groups, 512, 512)
    # the launched step that runs with its bucket's rows
    batch = build_step_batch(entries, r.cache, "cpu", pad_to=StepGraphs.padded_tokens)
    assert batch.num_tokens == 49 and batch.num_seqs == 3 and batch.q_lens == [1, 37, 11]
    assert batch.input_ids.shape[0] == 49 and batch.cu_q_lens.tolist() == [0, 1, 38, 49]
    for q in (2, 16, 17, 100, 128, 129, 1000, 2047, 2048, 2049, 5000):
        bucket, lowest = token_bucket(q)
        assert lowest <= q <= bucket and bucket - q <= max(15, q // 16)
        assert token_bucket(bucket)[0] == bucket and token_bucket(lowest)[0] <= bucket


def test_step_graphs_capture_only_where_the_host_is_the_bound(tiny_model_dirs, torch_ops):
    """The step graphs' decision from a bucket's timed launched step: the host's time to issue
    the launches against the device's time between two events.  A bucket whose host time is
    half of the device's or more is host-bound (worth a graph at once); one below that is
    remembered as device-bound, not timed again, and left to the patient rule."""
    from deterministic_inference_b200.engine.graphs import StepGraphs

    class Event:
        def __init__(self, ms):
            self.ms, self.done = ms, True

        def query(self):
            return self.done

        def elapsed_time(self, other):
            return other.ms - self.ms

    r = ModelRunner(EngineConfig(model_path=str(tiny_model_dirs["bw"]), dtype="float32", device="cpu",
                                 kv_pool_tokens=256, page_size=16, max_reqs=8, max_seq_len=256))
    sg = StepGraphs(r.model, r.cache, r.device)
    assert sg.host_bound_share == 0.5 and sg.patient_repeats > sg.min_repeats
    assert not sg._host_bound("never launched")
    sg._launching = "a"
    end = Event(4.0)
    sg.launched(0.0039, Event(0.0), end)             # 3.9 ms of host time for 4.0 ms on the device
    end.done = False                                 # the step has not finished: not known yet, asked again
    assert sg._launching is None and not sg._host_bound("a") and "a" in sg.timings
    end.done = True
    assert sg._host_bound("a") and "a" not in sg.device_bound
    sg._launching = "b"
    sg.launched(0.0019, Event(0.0), Event(8.2))      # 1.9 ms of host time for 8.2 ms on the device
    assert not sg._host_bound("b") and "b" in sg.device_bound and "b" not in sg.timings
    sg.launched(1.0, Event(0.0), Event(1.0))         # no step was declined: nothing is recorded
    assert set(sg.timings) == {"a"}
