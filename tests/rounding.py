"""Telling a rounding flip from a fault in bfloat16 greedy generation."""

from tests import plain_qwen3


def divergence_is_a_rounding_flip(cfg, w, prompt, got, want):
    """bfloat16 greedy tokens may leave the float32 plain implementation's only where
    rounding can flip the argmax.  At the first differing token: R = what bfloat16
    storage rounding does to this position's logits (plain implementation with
    storage emulated minus plain float32).  The engine's logits lie within 1.5 R of
    the float32 ones (tests/test_replay_gpu.py), so the token it picked must be within
    3 R of the best one in the float32 logits."""
    for i, (a, b) in enumerate(zip(got, want)):
        if a != b:
            ctx = prompt + want[:i]
            l32 = plain_qwen3.forward(cfg, w, ctx)[-1]
            lemu = plain_qwen3.forward(cfg, w, ctx, store_bf16=True)[-1]
            r = float((l32 - lemu).abs().max())
            gap = float(l32[b] - l32[a])
            return gap <= 3 * r + 1e-3, f"token {i}: gap {gap:.3f}, rounding effect {r:.3f}"
    return True, ""
