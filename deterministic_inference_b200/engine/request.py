"""A request and its life: WAITING -> RUNNING -> DONE, and back to WAITING when
it is preempted.

The reference's invariant (sid/engine/request.py:8-15,66-71) is kept in another
form: ``num_computed`` counts the tokens of ``prompt + outputs`` whose keys are
in the cache; the newest sampled token is not among them until it is fed back.
A step feeds ``all_ids[num_computed : num_computed + n]``; when that reaches the
end of ``all_ids`` the logits of the last token give the next token, whose
position is ``len(all_ids)`` (sid/engine/batch.py:3-10).  A preempted request
drops to ``num_computed = 0`` and recomputes prompt and outputs alike.
"""

from __future__ import annotations

import enum
from typing import Optional

from ..config.engine_config import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    DONE = "done"


class Request:
    def __init__(self, rid: int, prompt_ids: list, params: SamplingParams, eos_token_ids=()):
        self.rid = rid
        self.prompt_ids = list(prompt_ids)
        self.params = params
        self.eos_token_ids = set(eos_token_ids)
        if params.stop_token_ids:
            self.eos_token_ids.update(params.stop_token_ids)
        self.output_ids: list[int] = []
        self.state = RequestState.WAITING
        self.finished_reason: Optional[str] = None
        self.slot: int = -1
        self.num_computed = 0
        self.num_pending = 0          # tokens sampled on the device, not yet read by the host
        self.num_preemptions = 0
        self.admit_order = -1

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_ids)

    @property
    def num_output(self) -> int:
        return len(self.output_ids)

    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids) + self.num_pending

    @property
    def done_generating(self) -> bool:
        """All the tokens it may generate are sampled (some perhaps not yet read)."""
        return self.finished_reason is not None or \
            len(self.output_ids) + self.num_pending >= self.params.max_new_tokens

    @property
    def remaining(self) -> int:
        """Tokens that still have to go through the model before the next token
        can be sampled."""
        return self.total_len - self.num_computed

    def next_tokens(self, n: int) -> list:
        """The next n token ids; a token not yet read from the device is given as 0
        (the step patches it in on the device)."""
        c = self.num_computed
        p = self.prompt_len
        if c + n <= p:
            return self.prompt_ids[c:c + n]
        return (self.prompt_ids + self.output_ids + [0] * self.num_pending)[c:c + n]

    def check_finished(self) -> None:
        """sid/engine/request.py:84-95: EOS (unless ignore_eos) -> "stop";
        max_new_tokens reached -> "length"."""
        if self.num_output == 0:
            self.finished_reason = None
        elif not self.params.ignore_eos and self.output_ids[-1] in self.eos_token_ids:
            self.finished_reason = "stop"
        elif self.num_output >= self.params.max_new_tokens:
            self.finished_reason = "length"
        else:
            self.finished_reason = None

    def __repr__(self) -> str:
        return (f"Request(rid={self.rid}, state={self.state.value}, P={self.prompt_len}, "
                f"N={self.num_output}, computed={self.num_computed}, finished={self.finished_reason})")
