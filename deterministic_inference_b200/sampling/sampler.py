"""Sampling from float32 logits rows.

Greedy (temperature 0): argmax, lowest index on ties.  Otherwise softmax of
logits / temperature, optional top-k / top-p filtering, and a Gumbel-max draw
whose noise is a pure function of (seed, position of the generated token,
vocabulary id), so a request's draw does not depend on the batch
(sid/engine/sampler.py:22-69).  The position convention is the reference's:
the token generated after n tokens of the sequence has position n
(sid/engine/batch.py:3-10).

argmax and the Gumbel draw are this package's kernels.  top-k / top-p: the kernels find,
without a sort, the probability threshold that the reference's sort-and-cumulate rule
amounts to (tokens that tie with the threshold all stay; masses are added in fixed
point), and draw among the ids at or above it.  Only when some row asks for it.
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops


def sample(logits: torch.Tensor, params: list, sample_positions: list) -> torch.Tensor:
    """int32 [R] token ids.  ``params[i]`` is the ``SamplingParams`` of row i and
    ``sample_positions[i]`` the absolute position of the token it generates."""
    r = logits.shape[0]
    if r == 0:
        return torch.empty(0, dtype=torch.int32, device=logits.device)
    if all(p.temperature <= 0 for p in params):
        return ops.argmax(logits)
    dev = logits.device
    filtered = any(p.temperature > 0 and (p.top_k > 0 or p.top_p < 1.0) for p in params)
    # the rows' parameters go to the device in ONE copy from pinned memory that does not
    # make the host wait: int64 [seeds | positions | top_k], float32 [temperatures | top_p]
    n64, n32 = (3 if filtered else 2) * r, (2 if filtered else 1) * r
    host = torch.empty(n64 * 8 + n32 * 4, dtype=torch.uint8, pin_memory=dev.type == "cuda")
    view = host.numpy()
    h64, h32 = view[:n64 * 8].view(np.int64), view[n64 * 8:].view(np.float32)
    h64[:r] = [p.seed for p in params]
    h64[r:2 * r] = sample_positions
    h32[:r] = [p.temperature for p in params]
    if filtered:
        h64[2 * r:] = [p.top_k if p.top_k > 0 else -1 for p in params]
        h32[r:] = [p.top_p for p in params]
    device = host.to(dev, non_blocking=True)
    d64, d32 = device[:n64 * 8].view(torch.int64), device[n64 * 8:].view(torch.float32)
    seeds, pos, temps = d64[:r], d64[r:2 * r], d32[:r]
    if filtered:
        # the kernels drop what top-k / top-p drop, by a threshold found without a sort
        return ops.gumbel_sample(logits, temps, seeds, pos, top_ks=d64[2 * r:], top_ps=d32[r:])
    return ops.gumbel_sample(logits, temps, seeds, pos)
