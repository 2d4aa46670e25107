"""CUDA-graph replay of pure-decode steps (every sequence brings one token).

A decode step of a small model is bound by launch latency, not by the GPU; the
step function's kernels for a batch-size bucket are captured once and replayed
with the step's metadata copied into the captured buffers.
"""

from __future__ import annotations


class DecodeGraphs:
    def __init__(self, runner):
        self.runner = runner

    def usable(self, entries) -> bool:
        return False

    def run(self, entries):
        raise NotImplementedError
