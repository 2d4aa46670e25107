"""The scheduler's decisions, on the host with a real cache manager (CPU tensors
off) and no model: admission, token budget, portions, decode beside prefill,
finishing, and what happens when pages run out.  The reference tests its host
logic the same way, with fakes for the GPU objects (tests/test_08_dvr_logic.py:20-52)."""

import torch

from deterministic_inference_b200.cache import CacheManager
from deterministic_inference_b200.config import SamplingParams
from deterministic_inference_b200.engine.request import Request, RequestState
from deterministic_inference_b200.engine.scheduler import Scheduler
from deterministic_inference_b200.parts import PagedKVSpec


def make(pages=64, page=4, budget=16, max_running=8, reqs=16):
    cache = CacheManager({0: PagedKVSpec(1, 8, None)}, num_pages=pages + 1, page_size=page,
                         max_reqs=reqs + 1, max_seq_len=4096, dtype=torch.float32, device="cpu",
                         allocate_device=False)
    return Scheduler(cache, budget, max_running), cache


def req(rid, plen, max_new=4):
    return Request(rid, list(range(plen)), SamplingParams(max_new_tokens=max_new, ignore_eos=True))


def run_step(sched, token=7):
    """What Engine.step does with the scheduler's decision, without a model."""
    out = sched.schedule()
    for s in out:
        r = s.request
        r.num_computed += s.num_tokens
        if r.num_computed == r.total_len:
            r.output_ids.append(token)
            r.check_finished()
    done = sched.release_finished()
    sched.cache.check_invariants()
    return out, done


def test_portions_under_the_token_budget():
    sched, _ = make(budget=16)
    sched.add(req(0, 40))
    sizes = []
    while not sched.running or sched.running[0].num_output == 0:
        out, _ = run_step(sched)
        sizes.append([(s.request.rid, s.num_tokens) for s in out])
    assert sizes == [[(0, 16)], [(0, 16)], [(0, 8)]]


def test_decode_tokens_come_first_and_prompts_share_what_is_left():
    sched, _ = make(budget=16)
    sched.add(req(0, 5, max_new=10))
    run_step(sched)                               # request 0 prefilled, now decoding
    sched.add(req(1, 30))
    sched.add(req(2, 3))
    out, _ = run_step(sched)
    assert [(s.request.rid, s.num_tokens) for s in out] == [(0, 1), (1, 15)]      # budget 16
    out, _ = run_step(sched)
    # request 1 is running now: it gets its next portion before request 2 is admitted
    assert [(s.request.rid, s.num_tokens) for s in out] == [(0, 1), (1, 15)]
    assert [r.rid for r in sched.waiting] == [2]
    out, _ = run_step(sched)
    assert [(s.request.rid, s.num_tokens) for s in out] == [(0, 1), (1, 1), (2, 3)]


def test_fcfs_head_blocks_the_queue():
    sched, cache = make(pages=6, page=4, budget=64)       # 24 tokens
    sched.add(req(0, 20))
    sched.add(req(1, 12))          # does not fit beside request 0
    sched.add(req(2, 2))           # would fit, but waits behind request 1
    out, _ = run_step(sched)
    assert [s.request.rid for s in out] == [0]
    assert [r.rid for r in sched.waiting] == [1, 2]


def test_limits_on_running_requests_and_slots():
    sched, _ = make(max_running=2, budget=64)
    for i in range(4):
        sched.add(req(i, 3, max_new=2))
    out, _ = run_step(sched)
    assert [s.request.rid for s in out] == [0, 1]
    out, done = run_step(sched)                          # both finish (max_new 2)
    assert [r.rid for r in done] == [0, 1] and all(r.state == RequestState.DONE for r in done)
    out, _ = run_step(sched)
    assert [s.request.rid for s in out] == [2, 3]


def test_finish_frees_pages_and_slot():
    sched, cache = make()
    sched.add(req(0, 9, max_new=1))
    free0, slots0 = cache.num_free_pages(), cache.num_free_slots
    _, done = run_step(sched)
    assert [r.finished_reason for r in done] == ["length"]
    assert cache.num_free_pages() == free0 and cache.num_free_slots == slots0
    assert not sched.has_work()


def test_eos_stops_unless_ignored():
    sched, _ = make()
    r = Request(0, [1, 2, 3], SamplingParams(max_new_tokens=5), eos_token_ids=(7,))
    sched.add(r)
    _, done = run_step(sched, token=7)
    assert done and done[0].finished_reason == "stop"
    r2 = Request(1, [1, 2, 3], SamplingParams(max_new_tokens=2, stop_token_ids=[9]), eos_token_ids=(7,))
    sched.add(r2)
    _, done = run_step(sched, token=9)
    assert done and done[0].finished_reason == "stop"


def test_out_of_pages_preempts_the_newest_and_everyone_finishes():
    # 6 pages of 4 tokens; two requests of 8 prompt tokens that want 12 more each: 40 tokens > 24
    sched, cache = make(pages=6, page=4, budget=64)
    a, b = req(0, 8, max_new=12), req(1, 8, max_new=12)
    sched.add(a)
    sched.add(b)
    steps = 0
    seen_preempt = False
    while sched.has_work():
        out, _ = run_step(sched)
        steps += 1
        if b.state == RequestState.WAITING and b.num_preemptions:
            seen_preempt = True
            assert b.num_computed == 0 and b.slot == -1 and sched.waiting[0] is b    # front of the queue
            assert a.state != RequestState.WAITING                                   # never the oldest
        assert steps < 200
    assert seen_preempt and a.num_preemptions == 0 and b.num_preemptions >= 1
    assert len(a.output_ids) == 12 and len(b.output_ids) == 12         # outputs kept across preemption
    assert cache.num_free_pages() == 6


def test_a_preempted_request_recomputes_prompt_and_outputs():
    sched, cache = make(pages=4, page=4, budget=64)
    a, b = req(0, 7, max_new=8), req(1, 4, max_new=8)
    sched.add(a)
    sched.add(b)
    while b.num_preemptions == 0:
        run_step(sched)
    n_out = b.num_output
    assert b.remaining == b.prompt_len + n_out        # everything has to go through the model again
    assert b.next_tokens(b.remaining) == b.prompt_ids + b.output_ids
    while sched.has_work():
        run_step(sched)
    assert len(b.output_ids) == 8


def test_lone_request_that_outgrows_the_pool_preempts_itself_and_is_not_readmitted_blindly():
    sched, cache = make(pages=2, page=4, budget=64)       # 8 tokens
    r = req(0, 6, max_new=10)                              # the engine refuses this at add_request
    sched.add(r)
    run_step(sched)
    for _ in range(5):
        run_step(sched)
    assert r.num_preemptions >= 1
    cache.check_invariants()


import pytest


@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_under_a_small_pool(seed):
    """Requests of random lengths arrive at random steps into a pool that holds only a few
    of them: every step keeps the token budget and the limit on running requests, a
    request never gets more tokens than it has left, decode tokens are single, no page
    is lost, a preempted request was admitted after every request that keeps running,
    and in the end every request has all its outputs and every page is free."""
    import random
    rng = random.Random(seed)
    pages, page, budget, max_running = rng.choice([8, 12, 20]), rng.choice([2, 4]), rng.choice([5, 16, 64]), rng.choice([2, 4, 8])
    sched, cache = make(pages=pages, page=page, budget=budget, max_running=max_running, reqs=12)
    cap = pages * page
    todo = []
    for rid in range(12):
        plen = rng.randint(1, max(1, cap // 2))
        max_new = rng.randint(1, max(1, cap - plen))          # fits the pool alone
        todo.append((rng.randint(0, 30), req(rid, plen, max_new=max_new)))
    todo.sort(key=lambda x: x[0])
    all_reqs = [r for _, r in todo]
    step = 0
    while todo or sched.has_work():
        while todo and todo[0][0] <= step:
            sched.add(todo.pop(0)[1])
        running_before = [r for r in all_reqs if r.state == RequestState.RUNNING]
        admitted_before = {r.rid: r.admit_order for r in running_before}
        preempts_before = {r.rid: r.num_preemptions for r in all_reqs}
        out, _ = run_step(sched)
        assert sum(s.num_tokens for s in out) <= budget
        assert len({s.request.rid for s in out}) == len(out) <= max_running
        for s in out:
            assert 1 <= s.num_tokens
        victims = [r for r in all_reqs if r.num_preemptions > preempts_before[r.rid]]
        if victims and len(running_before) > 1:
            # a victim was admitted after every request that kept running
            survivors = [r for r in running_before if r not in victims and r.finished_reason is None]
            for v in victims:
                if v.rid in admitted_before:
                    assert all(admitted_before[v.rid] > admitted_before[k.rid] for k in survivors)
        step += 1
        assert step < 5000
    for r in all_reqs:
        assert len(r.output_ids) == r.params.max_new_tokens, (r.rid, len(r.output_ids))
    assert cache.num_free_pages() == pages
    cache.check_invariants()
