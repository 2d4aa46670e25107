"""Plain data that describes a model as parts.

A model is a ``ModelPlan``: a tuple of ``LayerSpec`` (which mixer, feed-forward,
norms and block arrangement a layer is made of, each with its sizes and
constants as parameters) and a ``schedule``, the order in which layers run.  The
schedule is data too: an entry may name a layer a second time, and it names the
cache its mixer uses, so a layer may read the cache another entry wrote.

Nothing in this module knows an architecture; the architecture's configuration
class produces a plan, and the generic decoder builds and runs it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and its parameters (sizes, constants,
    checkpoint names)."""

    kind: str
    params: dict = field(default_factory=dict)

    def __hash__(self):  # params is a dict; identity is enough for frozen use
        return id(self)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec               # arrangement of the parts below and the residual
    mixer: PartSpec               # token mixer (attention here)
    feed_forward: PartSpec        # dense or experts
    mixer_norm: PartSpec          # norm in front of the mixer
    feed_forward_norm: PartSpec   # norm in front of the feed-forward


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  ``cache`` is the id of the cache (or state) its
    mixer works on; exactly one entry writes a given cache, and it runs before
    the entries that only read it."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec               # token ids -> hidden states
    head: PartSpec                    # hidden states of the wanted rows -> float32 logits
    final_norm: PartSpec
    layers: tuple
    schedule: tuple
    max_positions: int
    eos_token_ids: tuple = ()
    ignored_names: tuple = ()         # checkpoint tensors that may be present and are not used
    ignored_substrings: tuple = ()

    def validate(self) -> None:
        writers: dict[int, int] = {}
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {pos} names layer {e.layer}, "
                                 f"the plan has {len(self.layers)}")
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"cache {e.cache} is written by schedule entries "
                                     f"{writers[e.cache]} and {pos}")
                writers[e.cache] = pos
        for pos, e in enumerate(self.schedule):
            if not e.writes_cache:
                if e.cache not in writers:
                    raise ValueError(f"schedule entry {pos} reads cache {e.cache} that no entry writes")
                if writers[e.cache] > pos:
                    raise ValueError(f"schedule entry {pos} reads cache {e.cache} before "
                                     f"entry {writers[e.cache]} writes it")


@dataclass(frozen=True)
class TensorSpec:
    """A checkpoint tensor a part needs: name, shape, and what it is.

    role "matrix": a linear weight [out, in], cast to the engine dtype.
    role "table":  the embedding [vocab, hidden], cast to the engine dtype.
    role "vector": a norm weight; kept in float32 whatever it is stored as
                   (norm math is float32).
    ``init`` names the law the random-weights mode draws it from.
    """

    name: str
    shape: tuple
    role: str = "matrix"
    init: str = "normal"          # "normal": N(0, std); "one_plus_normal": 1 + N(0, norm_std)


@dataclass(frozen=True)
class PagedKVSpec:
    """Cache need of an attention-like mixer: keys and values per token.
    ``window`` None: all keys are kept; an int: only the last ``window`` keys are
    ever read, so older pages can be given back."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> tuple:
        return ("paged_kv", self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Cache need of a mixer with per-request state of fixed size."""

    shape: tuple
    dtype: str = "float32"

    def group_key(self) -> tuple:
        return ("state", tuple(self.shape), self.dtype)
