"""``Engine``: the step loop over scheduler, step function and sampler, and the
offline ``generate`` call.  API as the reference's (sid/engine/engine.py:43-204):
``Engine(EngineConfig(...)).generate(prompts, SamplingParams(...))``,
``add_request``, ``step``, ``get_output``; prompts are token-id lists, or strings
when the model folder holds a tokenizer.

One step = schedule (running requests' tokens, admissions, preemptions), run the
mixed batch, sample where a request's tokens were all consumed, retire finished
requests.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from ..config.engine_config import EngineConfig, SamplingParams
from ..sampling.sampler import sample
from .batch import SequenceInput
from .request import Request
from .runner import ModelRunner
from .scheduler import Scheduler


# DIB200_NVTX=1: every engine step is an NVTX range (for a timeline profiler)
_NVTX = os.environ.get("DIB200_NVTX", "0") == "1"


@dataclass
class RequestOutput:
    rid: int
    prompt_ids: list
    token_ids: list
    text: str
    finish_reason: str
    num_preemptions: int = 0


class _InFlight:
    """The tokens a step sampled, on their way to the host."""

    def __init__(self, tokens_dev: torch.Tensor, row_req: list):
        self.tokens_dev, self.row_req = tokens_dev, row_req
        self.row_of = {r.rid: i for i, r in enumerate(row_req)}
        self.host = None
        self.event = None
        if tokens_dev.is_cuda:
            self.host = torch.empty(tokens_dev.shape, dtype=tokens_dev.dtype, pin_memory=True)
            self.host.copy_(tokens_dev, non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record()

    def read(self) -> list:
        if self.host is None:
            return self.tokens_dev.tolist()
        self.event.synchronize()
        return self.host.tolist()


class Engine:
    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg
        self.runner = ModelRunner(cfg)
        self.cache = self.runner.cache
        self.scheduler = Scheduler(self.cache, cfg.max_prefill_tokens, cfg.max_decode_batch)
        self.vocab_size = self.runner.model.plan.vocab_size
        self.eos_token_ids = tuple(self.runner.model.plan.eos_token_ids)
        self.tokenizer = None
        self._next_rid = 0
        self._done: dict[int, Request] = {}
        self._pool_capacity = self.cache.usable_pages() * cfg.page_size
        self._inflight = None
        self.async_scheduling = cfg.async_scheduling
        self.decode_graphs = self.runner.decode_graphs

    # ---- public API -----------------------------------------------------------

    def _tokenizer(self):
        if self.tokenizer is None:
            if self.cfg.model_path is None:
                raise ValueError("string prompts need a model folder with a tokenizer")
            from transformers import AutoTokenizer  # tokenizer only; no model code
            self.tokenizer = AutoTokenizer.from_pretrained(str(self.cfg.model_path))
        return self.tokenizer

    def add_request(self, prompt: Optional[str] = None, prompt_ids: Optional[list] = None,
                    params: Optional[SamplingParams] = None, chat: bool = False) -> int:
        params = params or SamplingParams()
        if prompt_ids is None:
            if prompt is None:
                raise ValueError("add_request needs prompt or prompt_ids")
            tok = self._tokenizer()
            if chat:
                prompt_ids = tok.apply_chat_template(
                    [{"role": "user", "content": prompt}], tokenize=True,
                    add_generation_prompt=True, return_dict=False)
            else:
                prompt_ids = tok.encode(prompt)
        prompt_ids = [int(t) for t in prompt_ids]
        if not prompt_ids:
            raise ValueError("empty prompt")
        bad = [t for t in prompt_ids if not 0 <= t < self.vocab_size]
        if bad:
            raise ValueError(f"token ids outside the vocabulary of {self.vocab_size}: {bad[:5]}")
        if len(prompt_ids) > self.cfg.max_prompt_len:
            raise ValueError(f"prompt too long: {len(prompt_ids)} > {self.cfg.max_prompt_len}")
        pos_limit = min(self.cfg.max_seq_len, self.runner.max_positions)
        total = len(prompt_ids) + params.max_new_tokens
        if total > pos_limit:
            raise ValueError(f"prompt ({len(prompt_ids)}) + max_new_tokens ({params.max_new_tokens}) "
                             f"exceeds the position limit {pos_limit}")
        if total > self._pool_capacity:
            raise ValueError(f"prompt ({len(prompt_ids)}) + max_new_tokens ({params.max_new_tokens}) "
                             f"exceeds the cache pool of {self._pool_capacity} tokens: the request "
                             "could never run; raise kv_pool_tokens or lower max_new_tokens")
        rid = self._next_rid
        self._next_rid += 1
        self.scheduler.add(Request(rid, prompt_ids, params, self.eos_token_ids))
        return rid

    def generate(self, prompts: list, params=None, chat: bool = False) -> list[RequestOutput]:
        """Run all prompts to completion; outputs in input order."""
        if params is None:
            params = [SamplingParams() for _ in prompts]
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(params)} SamplingParams")
        rids = []
        for p, sp in zip(prompts, params):
            if isinstance(p, str):
                rids.append(self.add_request(prompt=p, params=sp, chat=chat))
            else:
                rids.append(self.add_request(prompt_ids=p, params=sp))
        while self.has_work():
            self.step()
        self.check_kernels()
        return [self._output(self._done.pop(rid)) for rid in rids]

    def check_kernels(self) -> None:
        """Raise if a bounded wait inside a kernel ran out since the last check (the kernels
        then set an error word and end instead of spinning; their results are not valid).
        The words are read after the first launched step, after the warm-up of every graph
        capture, every 32 steps and at the end of ``generate``; reading synchronises.  A
        failure is reported once: the words are cleared when it is raised."""
        if self.runner.device.type == "cuda":
            from ..kernels import ops
            ops.check_kernel_status()

    def get_output(self, rid: int) -> Optional[RequestOutput]:
        req = self._done.pop(rid, None)
        return self._output(req) if req else None

    # ---- one step ----------------------------------------------------------------

    def step(self) -> None:
        """Schedule, run the batch, sample; read the tokens of the step BEFORE this
        one.  With ``async_scheduling`` the tokens a step samples stay on the device:
        the next step takes them as inputs there (``pending_row``), and the host reads
        them one step late, while the GPU already runs that next step.  A request
        that turns out to have stopped on an end-of-sequence token has then been fed
        one token too many; that result is dropped."""
        self._steps_since_check = getattr(self, "_steps_since_check", 0) + 1
        if self._steps_since_check >= 32:
            self._steps_since_check = 0
            self.check_kernels()
        nvtx = _NVTX and self.runner.device.type == "cuda"
        if nvtx:
            torch.cuda.nvtx.range_push("engine.step")
        try:
            self._step()
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()

    def _step(self) -> None:
        sched = self.scheduler.schedule()
        if not sched:
            if self._inflight is not None:
                self._collect()
                return
            for req in self.scheduler.release_finished():
                self._done[req.rid] = req
            if self.scheduler.waiting and not self.scheduler.running:
                head = self.scheduler.waiting[0]
                raise RuntimeError(
                    f"request {head.rid} cannot be admitted: it needs pages for "
                    f"{min(head.remaining, self.scheduler.token_budget)} tokens and the pool has "
                    f"{self.cache.num_free_pages()} free pages of {self.cfg.page_size}")
            return
        prev = self._inflight
        entries = []
        for s in sched:
            r, n = s.request, s.num_tokens
            last = r.num_computed + n == r.total_len
            pending_row = prev.row_of[r.rid] if (last and r.num_pending and prev is not None) else -1
            entries.append(SequenceInput(r.slot, r.next_tokens(n), r.num_computed,
                                         [n - 1] if last else [], pending_row))
        prev_tokens = prev.tokens_dev if prev is not None else None
        logits, batch = self.runner.step(entries, prev_tokens)
        rows = batch.logit_rows
        row_req: list = [None] * logits.shape[0]
        for i, s in enumerate(sched):
            s.request.num_computed += s.num_tokens
            for row in rows[i]:
                row_req[row] = s.request
        flight = None
        if row_req:
            # the generated token's position is the sequence's length so far
            tokens_dev = sample(logits, [r.params for r in row_req], [r.total_len for r in row_req])
            for r in row_req:
                r.num_pending += 1
            flight = _InFlight(tokens_dev, row_req)
        if prev is not None:
            self._collect()                  # the step before this one
        self._inflight = flight
        if flight is not None and not self.async_scheduling:
            self._collect()

    def _collect(self) -> None:
        """Read the in-flight step's tokens, give them to their requests, retire."""
        flight, self._inflight = self._inflight, None
        for r, tok in zip(flight.row_req, flight.read()):
            r.num_pending -= 1
            if r.finished_reason is not None:
                continue                     # it had stopped already: this token is dropped
            r.output_ids.append(int(tok))
            r.check_finished()
        for req in self.scheduler.release_finished():
            self._done[req.rid] = req

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def _output(self, req: Request) -> RequestOutput:
        text = ""
        if self.tokenizer is not None:
            text = self.tokenizer.decode(req.output_ids, skip_special_tokens=True)
        return RequestOutput(rid=req.rid, prompt_ids=req.prompt_ids, token_ids=list(req.output_ids),
                             text=text, finish_reason=req.finished_reason or "abort",
                             num_preemptions=req.num_preemptions)
