"""Plain PyTorch restatement of every kernel, with the signatures of
``deterministic_inference_b200.kernels.ops``.

Two uses, both in tests only: (1) the float32 reference each CUDA kernel is
compared with; (2) patched over ``ops`` (fixture ``torch_ops`` in conftest.py) so
that the engine's host logic (cache, batch building, step function, scheduler)
can be exercised on a machine without a GPU.  The package never imports this
file.

Formulas: the reference project's kernels, cited per function (paths relative to
Aayaan-Sahu/deterministic-inference).
"""

from __future__ import annotations

import torch


def embedding(ids, table):
    """sid/model/qwen3.py:93"""
    return table[ids.long()]


def patch_token_ids(input_ids, patch_dst, patch_src, prev_tokens):
    ok = patch_dst >= 0
    input_ids[patch_dst[ok].long()] = prev_tokens[patch_src[ok].long()]


def _rms(x32, w, eps):
    """sid/kernels/rmsnorm.py:14-24"""
    var = (x32 * x32).mean(dim=-1, keepdim=True)
    return x32 * (1.0 / torch.sqrt(var + eps)) * w.float()


def rms_norm(x, weight, eps):
    return _rms(x.float(), weight, eps).to(x.dtype)


def add_rms_norm(x, residual, weight, eps):
    """In place like the kernel (sid/kernels/rmsnorm.py:27-42): the residual is
    stored rounded, the norm reads the unrounded sum."""
    s = x.float() + residual.float()
    residual.copy_(s.to(residual.dtype))
    x.copy_(_rms(s, weight, eps).to(x.dtype))
    return x, residual


def qk_norm_rope_cache(qkv, num_heads, num_kv_heads, head_dim, q_norm_weight, k_norm_weight, eps,
                       cos_sin, positions, kv_cache, slot_mapping, page_size):
    """sid/model/qwen3.py:49-61, sid/kernels/rmsnorm.py:72-75, sid/kernels/rope.py:15-37,
    sid/csrc/flash_decode.cu:275-296 (cache layout [pages, 2, Hkv, page, D] is this
    package's own)."""
    t = qkv.shape[0]
    d = head_dim
    x = qkv.float()
    q = x[:, :num_heads * d].reshape(t, num_heads, d)
    k = x[:, num_heads * d:(num_heads + num_kv_heads) * d].reshape(t, num_kv_heads, d)
    v = x[:, (num_heads + num_kv_heads) * d:].reshape(t, num_kv_heads, d)
    if q_norm_weight is not None:
        q = _rms(q, q_norm_weight, eps)
    if k_norm_weight is not None:
        k = _rms(k, k_norm_weight, eps)
    if cos_sin is not None:
        r = cos_sin.shape[1]
        half = r // 2
        tab = cos_sin[positions.long()]
        cos, sin = tab[:, None, :half], tab[:, None, half:]

        def rot(y):
            y1, y2, rest = y[..., :half], y[..., half:r], y[..., r:]
            return torch.cat([y1 * cos - y2 * sin, y2 * cos + y1 * sin, rest], dim=-1)
        q, k = rot(q), rot(k)
    if kv_cache is not None:
        sm = slot_mapping.long()
        ok = sm >= 0
        page, off = sm[ok] // page_size, sm[ok] % page_size
        kv_cache[page, 0, :, off, :] = k[ok].to(kv_cache.dtype)
        kv_cache[page, 1, :, off, :] = v[ok].to(kv_cache.dtype)
    return q.to(qkv.dtype).contiguous()


def reshape_and_cache(k, v, kv_cache, slot_mapping):
    """sid/csrc/flash_decode.cu:275-296"""
    page_size = kv_cache.shape[3]
    sm = slot_mapping.long()
    ok = sm >= 0
    page, off = sm[ok] // page_size, sm[ok] % page_size
    kv_cache[page, 0, :, off, :] = k[ok]
    kv_cache[page, 1, :, off, :] = v[ok]


def paged_attention(q, kv_cache, meta, scale, window=None, defer=False):
    """Every token against the cached keys of its sequence, causal by absolute
    position, float32 softmax (sid/kernels/extend_attention.py:80-109,
    tests/conftest.py:11-32)."""
    t, hq, d = q.shape
    _, _, hkv, page_size, _ = kv_cache.shape
    group = hq // hkv
    out = torch.empty(t, hq, d, dtype=torch.float32, device=q.device)
    token_seq = meta.token_seq.tolist()
    positions = meta.positions.tolist()
    bt = meta.block_table
    for i in range(t):
        s, p = token_seq[i], positions[i]
        first = max(0, p - window + 1) if window else 0
        keys = torch.arange(first, p + 1, device=q.device)
        pages = bt[s, (keys // page_size)].long()
        offs = keys % page_size
        k = kv_cache[pages, 0, :, offs, :].float()      # [n, Hkv, D]
        v = kv_cache[pages, 1, :, offs, :].float()
        for h in range(hq):
            kh = h // group
            sc = (k[:, kh] @ q[i, h].float()) * scale
            out[i, h] = torch.softmax(sc, dim=-1) @ v[:, kh]
    return out.to(q.dtype)


def silu_mul(gate_up):
    """sid/model/qwen3.py:85-86"""
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def gated_linear(x, w_gate_up):
    """sid/model/qwen3.py:84-86"""
    return silu_mul(linear(x, w_gate_up))


def gather_rows(x, index):
    """sid/model/qwen3.py:113"""
    return x[index.long()].contiguous()


def linear(x, weight, out_dtype=None):
    """sid/model/qwen3.py:38 (float32 accumulation)."""
    y = x.float() @ weight.float().T
    return y.to(out_dtype or x.dtype)


def argmax(logits):
    """sid/engine/sampler.py:36-38"""
    return torch.argmax(logits, dim=-1).to(torch.int32)


def seeded_gumbel(seeds, sample_pos, num_cols):
    """sid/engine/sampler.py:22-29"""
    step = seeds * 19349663 ^ sample_pos * 73856093
    cols = torch.arange(num_cols, dtype=torch.int64, device=seeds.device)
    hashed = step.unsqueeze(-1) * 8589934591 ^ cols * 479001599
    u = (hashed % (2 ** 24)).float() / (2 ** 24)
    return -torch.log(-torch.log(u + 1e-10) + 1e-10)


def gumbel_scores(logits, temperatures, seeds, sample_positions, keep=None):
    """log(p + 1e-10) + gumbel for kept ids, -inf elsewhere (sid/engine/sampler.py:44-66)."""
    temps = torch.where(temperatures > 0, temperatures, torch.ones_like(temperatures))
    probs = torch.softmax(logits / temps.unsqueeze(-1), dim=-1)
    logp = torch.log(probs + 1e-10)
    if keep is not None:
        logp = torch.where(keep.bool(), logp, torch.full_like(logp, float("-inf")))
    return logp + seeded_gumbel(seeds, sample_positions, logits.shape[1])


def keep_mask(logits, temperatures, top_ks, top_ps):
    """uint8 [R, V]: 1 for ids that survive top-k / top-p by the reference's rule
    (sid/engine/sampler.py:44-62): probabilities sorted descending; a token is dropped when
    the mass before it exceeds top_p or its rank reaches top_k; the first stays."""
    temps = torch.where(temperatures > 0, temperatures, torch.ones_like(temperatures))
    p = torch.softmax(logits / temps.unsqueeze(-1), dim=-1)
    order = torch.argsort(p, dim=-1, descending=True, stable=True)
    sorted_p = torch.gather(p, -1, order)
    before = torch.cumsum(sorted_p, dim=-1) - sorted_p
    rank = torch.arange(p.shape[-1], device=p.device).unsqueeze(0)
    limit = torch.where(top_ks > 0, top_ks, torch.full_like(top_ks, p.shape[-1])).unsqueeze(-1)
    stays = (before <= top_ps.unsqueeze(-1)) & (rank < limit)
    stays[:, 0] = True
    mask = torch.zeros_like(stays)
    mask.scatter_(-1, order, stays)
    return mask.to(torch.uint8).contiguous()


def gumbel_sample(logits, temperatures, seeds, sample_positions, keep=None, top_ks=None, top_ps=None):
    """sid/engine/sampler.py:32-69"""
    if top_ks is not None:
        keep = keep_mask(logits, temperatures, top_ks, top_ps)
    greedy = torch.argmax(logits, dim=-1)
    sampled = torch.argmax(gumbel_scores(logits, temperatures, seeds, sample_positions, keep), dim=-1)
    return torch.where(temperatures > 0, sampled, greedy).to(torch.int32)


ALL = ("patch_token_ids", "embedding", "rms_norm", "add_rms_norm", "qk_norm_rope_cache", "reshape_and_cache",
       "paged_attention", "silu_mul", "gated_linear", "gather_rows", "linear", "argmax", "gumbel_sample")
