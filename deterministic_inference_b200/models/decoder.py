"""The generic decoder: embedding part, a schedule of blocks, final norm, head part.

It is built from a ``ModelPlan`` alone and runs one step: the tokens of the
batch through every schedule entry, each entry's mixer working on the cache the
entry names, then the head on the requested rows only
(sid/model/qwen3.py:88-115).  Which architecture the plan came from is not
known here.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..parts import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, BuildContext, ModelPlan,
                     TensorSpec)


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device):
        plan.validate()
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        self.ctx = BuildContext(dtype=dtype, device=self.device)
        self.blocks = []
        self.mixers = []
        for spec in plan.layers:
            mixer = MIXERS.build(spec.mixer, self.ctx)
            ff = FEED_FORWARDS.build(spec.feed_forward, self.ctx)
            n1 = NORMS.build(spec.mixer_norm, self.ctx)
            n2 = NORMS.build(spec.feed_forward_norm, self.ctx)
            self.blocks.append(BLOCKS.create(spec.block, self.ctx, mixer=mixer, feed_forward=ff,
                                             mixer_norm=n1, feed_forward_norm=n2))
            self.mixers.append(mixer)
        self.final_norm = NORMS.build(plan.final_norm, self.ctx)
        self.embedding = EMBEDDINGS.build(plan.embedding, self.ctx)
        self.head = HEADS.build(plan.head, self.ctx)

    # ---- weights ------------------------------------------------------------

    def parts(self):
        yield self.embedding
        for b in self.blocks:
            yield b.mixer
            yield b.feed_forward
            yield b.mixer_norm
            yield b.feed_forward_norm
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> list[TensorSpec]:
        """Every checkpoint tensor the model needs, in a fixed order (the order
        the random-weights mode draws them in): embedding, layers, final norm, head."""
        specs = []
        for part in self.parts():
            specs.extend(part.tensor_specs())
        seen = set()
        for s in specs:
            if s.name in seen:
                raise ValueError(f"tensor {s.name!r} is claimed by two parts")
            seen.add(s.name)
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            if part is self.head and self.head.tied:
                # a tied head shares the embedding's table, handed to it under the key None
                part.load({**tensors, None: self.embedding.table()})
            else:
                part.load(tensors)

    # ---- caches ---------------------------------------------------------------

    def cache_specs(self) -> dict[int, object]:
        """cache id -> the need of the mixer that writes it."""
        out = {}
        for e in self.plan.schedule:
            spec = self.mixers[e.layer].cache_spec()
            if spec is None:
                continue
            if e.writes_cache:
                out[e.cache] = spec
        for e in self.plan.schedule:
            spec = self.mixers[e.layer].cache_spec()
            if spec is not None and not e.writes_cache:
                if out[e.cache].group_key() != spec.group_key():
                    raise ValueError(f"layer {e.layer} reads cache {e.cache} of another kind: "
                                     f"{spec} vs {out[e.cache]}")
        return out

    # ---- one step ---------------------------------------------------------------

    def forward(self, step, cache_manager) -> torch.Tensor:
        """float32 logits [R, V] at ``step.logit_indices``."""
        hidden = self.embedding.forward(step.input_ids)
        residual = None
        for e in self.plan.schedule:
            cache = cache_manager.view(e.cache, step, writes=e.writes_cache)
            hidden, residual = self.blocks[e.layer].forward(hidden, residual, step, cache)
        # the head is applied to the requested rows only: gather first, then the
        # last residual add and the final norm on those rows
        if step.num_logits == 0:
            return torch.empty(0, self.plan.vocab_size, dtype=torch.float32, device=hidden.device)
        if step.logits_of_all_rows:
            # (a decode step: nothing to gather, and the last block's output may stay the
            # split sums it came as)
            rows, res_rows = hidden, residual
        else:
            rows = ops.gather_rows(hidden, step.logit_indices)
            res_rows = None if residual is None else ops.gather_rows(residual, step.logit_indices)
        if res_rows is None:
            rows = self.final_norm.forward(rows)
        else:
            rows, _ = self.final_norm.add_forward(rows, res_rows)
        return self.head.forward(rows)
