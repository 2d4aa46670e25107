"""Plain, slow Qwen3-dense forward: whole sequences, no cache, float32, CPU or GPU.

This file is the oracle of the test suite.  It shares no code with the package:
it reads ``config.json`` and ``model.safetensors`` by itself and restates each
formula of the reference engine (paths are relative to the reference project,
Aayaan-Sahu/deterministic-inference) one function per part.  Every function
cites the lines it restates.  The one formula that has no counterpart in the
reference is the sliding window of ``attention`` (the reference reads none of
the window keys of config.json); it follows the meaning of the config.json keys
``use_sliding_window`` / ``sliding_window`` / ``max_window_layers``: layers with
index >= max_window_layers let a query at position p see keys p-W+1 .. p.

The comparison of this file with the reference's own model code, run once on
the CPU, is ``tests/golden/make_golden.py``; its small outputs are committed
under ``tests/golden/`` and checked by ``tests/test_plain_vs_golden.py``.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import torch


# --------------------------------------------------------------------------
# reading a model folder (no package code)
# --------------------------------------------------------------------------

_ST_DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "I32": torch.int32,
    "I64": torch.int64,
}


def read_safetensors(path: Path) -> dict[str, torch.Tensor]:
    """Minimal safetensors reader: 8-byte little-endian header length, JSON
    header {name: {dtype, shape, data_offsets}}, then raw little-endian data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        buf = bytearray(raw[base + a:base + b])
        t = torch.frombuffer(buf, dtype=dt) if b > a else torch.empty(0, dtype=dt)
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def read_model_dir(model_dir, dtype=torch.float32) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and all tensors upcast to ``dtype`` (float32; float64
    gives the reference value that float32 implementations are measured against)
    (sid/model/loader.py:30-55 for the keys, :64-68 for the files)."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    tensors: dict[str, torch.Tensor] = {}
    for f in sorted(model_dir.glob("*.safetensors")):
        tensors.update(read_safetensors(f))
    return cfg, {k: v.to(dtype) for k, v in tensors.items()}


# --------------------------------------------------------------------------
# parts, one function each
# --------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * 1/sqrt(mean(x^2) + eps) * w over the last dim, eps inside the
    root, weight multiplies directly (sid/kernels/rmsnorm.py:14-24)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(var + eps)) * w


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """f[p, i] = p * theta^(-i/(D/2)), i < D/2, formed in float32
    (sid/kernels/rope.py:41-48)."""
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) / half))
    return torch.outer(positions.to(torch.float32), inv_freq)


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """NeoX rotate-half over the full head dim: x1 = x[..., :D/2], x2 = x[..., D/2:];
    out = [x1 cos - x2 sin, x2 cos + x1 sin] (sid/kernels/rope.py:15-37).
    x: [T, heads, D]; angles: [T, D/2]."""
    half = x.shape[-1] // 2
    angles = angles.to(x.dtype)          # the angle itself is always formed in float32
    cos = angles.cos()[:, None, :]
    sin = angles.sin()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int | None = None, rnd=None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.
    q: [T, Hq, D], k/v: [T, Hkv, D]; q head h reads kv head h // (Hq/Hkv);
    s = (q.k) * scale with the scale applied after the dot product; a query at
    position p sees keys 0..p; softmax and P.V in float32
    (sid/kernels/extend_attention.py:55,80-109; tests/conftest.py:11-32).
    ``window`` (not in the reference): keys older than p-window+1 are masked.
    ``rnd`` (bfloat16 storage emulation): the reference's prefill kernel rounds
    the unnormalised probabilities exp(s - max) to bfloat16 before P.V and divides
    by the float32 sum (sid/kernels/extend_attention.py:100-109)."""
    t, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    pos = torch.arange(t)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > (pos[:, None] - window)
    out = torch.empty_like(q)
    for h in range(hq):
        kh = h // group
        s = (q[:, h] @ k[:, kh].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        if rnd is None:
            out[:, h] = torch.softmax(s, dim=-1) @ v[:, kh]
        else:
            e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            out[:, h] = (rnd(e) @ v[:, kh]) / e.sum(dim=-1, keepdim=True)
    return out


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
           w_down: torch.Tensor, rnd=None) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), silu(z) = z * sigmoid(z), no biases
    (sid/model/qwen3.py:82-86)."""
    rnd = rnd or (lambda z: z)
    g = rnd(x @ w_gate.T)
    u = rnd(x @ w_up.T)
    return rnd(rnd((g * torch.sigmoid(g)) * u) @ w_down.T)


def layer_window(cfg: dict, layer: int) -> int | None:
    """Window of a layer from config.json (no counterpart in the reference)."""
    if not cfg.get("use_sliding_window", False):
        return None
    if cfg.get("sliding_window") is None:
        return None
    if layer < cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return None
    return int(cfg["sliding_window"])


def _identity(x):
    return x


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    """What storing a float32 value as bfloat16 and reading it back gives."""
    return x.to(torch.bfloat16).to(x.dtype)


def attention_block(h: torch.Tensor, cfg: dict, w: dict, layer: int, rnd=_identity) -> torch.Tensor:
    """q/k/v projections without bias, per-head RMSNorm of q and k with one
    weight [D] shared by the heads and the layer norms' eps, then RoPE, then
    attention with scale D^-0.5, then the output projection
    (sid/model/qwen3.py:43-80; head_dim explicit, sid/config.py:42)."""
    p = f"model.layers.{layer}.self_attn."
    t = h.shape[0]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = rnd(h @ w[p + "q_proj.weight"].T).view(t, hq, d)
    k = rnd(h @ w[p + "k_proj.weight"].T).view(t, hkv, d)
    v = rnd(h @ w[p + "v_proj.weight"].T).view(t, hkv, d)
    q = rms_norm(q, w[p + "q_norm.weight"], eps)
    k = rms_norm(k, w[p + "k_norm.weight"], eps)
    ang = rope_angles(torch.arange(t), d, cfg["rope_theta"])
    q, k = rnd(apply_rope(q, ang)), rnd(apply_rope(k, ang))
    o = rnd(attention(q, k, v, d ** -0.5, layer_window(cfg, layer),
                      None if rnd is _identity else rnd))
    return rnd(o.reshape(t, hq * d) @ w[p + "o_proj.weight"].T)


def forward(cfg: dict, w: dict, token_ids, store_bf16: bool = False) -> torch.Tensor:
    """Logits [T, V] of one whole sequence.  Pre-norm residual stream: at each
    norm site the residual takes the block's output first and the norm reads
    the sum (sid/model/qwen3.py:88-115, sid/kernels/rmsnorm.py:27-42); final
    norm, then the head, which is the embedding when tie_word_embeddings
    (sid/model/loader.py:74-82).

    ``store_bf16``: all arithmetic stays float32, but every tensor the reference
    stores in bfloat16 between two kernels (projection outputs, q and k after
    norm and rotation, attention output, the gated product, norm outputs, the
    residual: sid/model/qwen3.py:49-115, sid/kernels/rmsnorm.py:34-42) is rounded
    to bfloat16 there.  The difference between the two modes is what rounding
    alone does to this model; tests use it to tell rounding from faults."""
    rnd = round_bf16 if store_bf16 else _identity
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    eps = cfg["rms_norm_eps"]
    res = w["model.embed_tokens.weight"][ids]
    h = rnd(rms_norm(res, w["model.layers.0.input_layernorm.weight"], eps))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        s = res + attention_block(h, cfg, w, i, rnd)
        h = rnd(rms_norm(s, w[p + "post_attention_layernorm.weight"], eps))   # reads the unrounded sum
        res = rnd(s)                                                           # stored rounded
        s = res + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                         w[p + "mlp.down_proj.weight"], rnd)
        nxt = (f"model.layers.{i + 1}.input_layernorm.weight"
               if i + 1 < cfg["num_hidden_layers"] else "model.norm.weight")
        h = rnd(rms_norm(s, w[nxt], eps))
        res = rnd(s)
    head = (w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False)
            else w["lm_head.weight"])
    return h @ head.T


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


def _wrap(x: int) -> int:
    """Two's-complement wrap-around to a signed 64-bit value."""
    x &= _MASK64
    return x - (1 << 64) if x >= (1 << 63) else x


def seeded_gumbel_scalar(seed: int, pos: int, col: int) -> float:
    """Gumbel noise as a pure function of (seed, position, vocabulary id),
    restated with Python integers (sid/engine/sampler.py:22-29): wrap-around
    int64 products and xors, the low 24 bits as a uniform in [0,1)."""
    import math
    step = _wrap(_wrap(seed * 19349663) ^ _wrap(pos * 73856093))
    hashed = _wrap(_wrap(step * 8589934591) ^ _wrap(col * 479001599))
    u = torch.tensor(float(hashed % (1 << 24)), dtype=torch.float32) / (1 << 24)
    eps = torch.tensor(1e-10, dtype=torch.float32)
    return float(-torch.log(-torch.log(u + eps) + eps))


def seeded_gumbel(seed: int, pos: int, num_cols: int) -> torch.Tensor:
    """Vector form of ``seeded_gumbel_scalar`` with int64 tensors
    (sid/engine/sampler.py:22-29)."""
    step = torch.tensor(seed, dtype=torch.int64) * 19349663 ^ torch.tensor(pos, dtype=torch.int64) * 73856093
    cols = torch.arange(num_cols, dtype=torch.int64)
    hashed = step * 8589934591 ^ cols * 479001599
    u = (hashed % (2 ** 24)).float() / (2 ** 24)
    return -torch.log(-torch.log(u + 1e-10) + 1e-10)


def sample_token(logits: torch.Tensor, temperature: float, seed: int, pos: int,
                 top_k: int = -1, top_p: float = 1.0) -> int:
    """One row.  temperature 0: argmax, lowest index on ties.  Otherwise
    p = softmax(logits / temperature); sort descending; drop a token when the
    mass before it exceeds top_p or its rank >= top_k; never drop rank 0;
    token = argmax(log(p + 1e-10) + gumbel(seed, pos, vocab id)) over the kept
    ids (sid/engine/sampler.py:32-69).  ``pos`` is the absolute position of the
    token being generated (sid/engine/batch.py:3-10)."""
    logits = logits.float()
    if temperature <= 0:
        return int(torch.argmax(logits))
    probs = torch.softmax(logits / temperature, dim=-1)
    ps, idx = probs.sort(descending=True)
    cum = torch.cumsum(ps, dim=-1)
    dropped = (cum - ps) > top_p
    if top_k > 0:
        dropped |= torch.arange(len(ps)) >= top_k
    dropped[0] = False
    keep = torch.zeros_like(dropped)
    keep[idx] = ~dropped
    logp = torch.where(keep, torch.log(probs + 1e-10), torch.full_like(probs, float("-inf")))
    return int(torch.argmax(logp + seeded_gumbel(seed, pos, len(probs))))


def generate(cfg: dict, w: dict, prompt, max_new_tokens: int, temperature: float = 0.0,
             seed: int = 42, top_k: int = -1, top_p: float = 1.0,
             eos_ids=()) -> list[int]:
    """Token-by-token generation that recomputes the whole sequence each time.
    The token generated after n tokens has position n
    (sid/engine/batch.py:3-10, sid/engine/request.py:84-95)."""
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        logits = forward(cfg, w, seq)[-1]
        tok = sample_token(logits, temperature, seed, len(seq), top_k, top_p)
        out.append(tok)
        seq.append(tok)
        if tok in eos_ids:
            break
    return out
