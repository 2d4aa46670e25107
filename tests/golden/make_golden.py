"""Runs the REFERENCE's own model code once, on the CPU, on tiny random models,
and stores its logits and sampled tokens under tests/golden/ for
tests/test_plain_vs_golden.py.

    python tests/golden/make_golden.py /path/to/deterministic-inference

The reference (Aayaan-Sahu/deterministic-inference) imports on a CPU, but its
norm / rope / prefill-attention kernels are Triton and its cache write is CUDA,
so ``Qwen3Model.forward`` (sid/model/qwen3.py:88-115) cannot run as shipped.  Its
forward resolves those kernels as module globals (sid/model/qwen3.py:23-26) and
takes the cache as an argument, so this script substitutes them, for this run
only, by the float32 PyTorch references that the reference's OWN tests use
(``torch_rmsnorm`` tests/test_01_triton_ops.py:13-15, ``ref_attention``
tests/conftest.py:11-32, the rotate-half formula tests/test_01_triton_ops.py:72-83)
and a dict-backed cache.  Everything else is the reference's code: its loader
(fused qkv / gate_up, tied head), its forward orchestration, residual flow, row
selection and head, and its sampler (sid/engine/sampler.py runs on the CPU as is).

The models are written by this package's random-weights mode; their tensors are
drawn from a seeded CPU generator, and a checksum is stored so the test can tell
if the generator changed.  Nothing of the reference is copied into this
repository; only the numbers it produced.
"""

import importlib.util
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent

CASES = [("tiny_a", 0, 1, 33), ("tiny_b", 3, 4, 31)]       # preset, weight seed, token seed, tokens


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str) -> None:
    ref_root = Path(ref_root)
    sys.path.insert(0, str(ref_root))
    import sid.model.qwen3 as rq
    from sid.engine.batch import ForwardBatch, ForwardMode
    from sid.engine.sampler import sample as ref_sample
    from sid.model.loader import load_model_config, load_weights
    ref_conftest = load_by_path("ref_conftest", ref_root / "tests" / "conftest.py")
    ref_attention = ref_conftest.ref_attention

    def torch_rmsnorm(x, w, eps):                        # tests/test_01_triton_ops.py:13-15
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)) * w.float()

    def rmsnorm(x, w, eps):
        return torch_rmsnorm(x, w, eps).to(x.dtype)

    def fused_add_rmsnorm(x, residual, w, eps):           # in place, as sid/kernels/rmsnorm.py:60-70
        residual += x
        x.copy_(torch_rmsnorm(residual, w, eps).to(x.dtype))
        return x, residual

    def qk_head_rmsnorm(x, w, eps):
        return rmsnorm(x, w, eps)

    class Rope(rq.RotaryEmbedding):                       # the table is the reference's own
        def apply(self, q, k, positions):
            half = self.head_dim // 2
            tab = self.cos_sin[positions]
            cos, sin = tab[:, None, :half], tab[:, None, half:]
            for x in (q, k):                              # tests/test_01_triton_ops.py:78-81
                xf = x.float()
                x1, x2 = xf[..., :half], xf[..., half:]
                x.copy_(torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype))

    def extend_attention_fwd(q, k_buf, v_buf, qo_indptr, kv_indptr, kv_indices, max_extend_len, scale):
        out = torch.empty_like(q)
        for b in range(qo_indptr.numel() - 1):
            qs, qe = int(qo_indptr[b]), int(qo_indptr[b + 1])
            idx = kv_indices[int(kv_indptr[b]):int(kv_indptr[b + 1])].long()
            prefix = idx.numel() - (qe - qs)
            out[qs:qe] = ref_attention(q[qs:qe], k_buf[idx], v_buf[idx], scale,
                                       causal_offset=prefix).to(q.dtype)
        return out

    class Ext:
        @staticmethod
        def reshape_and_cache(k, v, k_pool, v_pool, slots):
            k_pool[slots] = k
            v_pool[slots] = v

    class Cache:
        ext = Ext()

        def __init__(self, layers, slots, hkv, d):
            self.k = [torch.zeros(slots, hkv, d) for _ in range(layers)]
            self.v = [torch.zeros(slots, hkv, d) for _ in range(layers)]

        def layer(self, i):
            return self.k[i], self.v[i]

    rq.rmsnorm, rq.fused_add_rmsnorm, rq.qk_head_rmsnorm = rmsnorm, fused_add_rmsnorm, qk_head_rmsnorm
    rq.RotaryEmbedding, rq.extend_attention_fwd = Rope, extend_attention_fwd

    sys.path.insert(0, str(REPO))
    from deterministic_inference_b200.config import preset
    from deterministic_inference_b200.weights import write_random_model
    plain = load_by_path("plain_qwen3", REPO / "tests" / "plain_qwen3.py")

    meta = {}
    for name, wseed, tseed, n in CASES:
        with tempfile.TemporaryDirectory() as d:
            write_random_model(preset(name), wseed, d)
            mcfg = load_model_config(Path(d), d)
            weights = load_weights(Path(d), mcfg, "cpu", dtype=torch.float32)
            model = rq.Qwen3Model(mcfg, weights, "cpu")
            g = torch.Generator().manual_seed(tseed)
            toks = torch.randint(0, mcfg.vocab_size, (n,), generator=g)
            slots = torch.arange(1, n + 1)
            ptr = torch.tensor([0, n], dtype=torch.int32)
            fb = ForwardBatch(mode=ForwardMode.PREFILL, input_ids=toks, positions=torch.arange(n),
                              out_slots=slots, qo_indptr=ptr, kv_indptr=ptr,
                              kv_indices=slots.to(torch.int32), max_extend_len=n,
                              sample_indices=torch.arange(n))
            cache = Cache(mcfg.num_layers, n + 1, mcfg.num_kv_heads, mcfg.head_dim)
            logits = model.forward(fb, cache, None, decode_backend="triton")
            pc, pw = plain.read_model_dir(d)
            ours = plain.forward(pc, pw, toks.tolist())
            diff = float((ours - logits).abs().max())
            print(f"{name}: reference logits {tuple(logits.shape)}, plain implementation differs by {diff:.3e}")
            np.save(HERE / f"{name}_logits.npy", logits.numpy().astype(np.float32))
            checksum = float(sum(v.double().abs().sum() for v in pw.values()))
            meta[name] = dict(weight_seed=wseed, token_seed=tseed, tokens=toks.tolist(),
                              weights_abs_sum=checksum, plain_vs_reference_max_abs_diff=diff)

    # the reference's sampler on fixed logits
    g = torch.Generator().manual_seed(11)
    logits = 3 * torch.randn(12, 997, generator=g)
    temps = torch.tensor([0.0, 0.7, 1.3] * 4)
    top_ks = torch.tensor([-1, -1, -1, 20, 20, 20, -1, -1, -1, 5, 5, 5])
    top_ps = torch.tensor([1.0] * 6 + [0.9] * 6)
    seeds = torch.tensor([42, 7, -3, 123456789012] * 3)
    pos = torch.arange(100, 112)
    toks = ref_sample(logits, temps, top_ks, top_ps, seeds, pos)
    np.save(HERE / "sampler_logits.npy", logits.numpy())
    meta["sampler"] = dict(temperatures=temps.tolist(), top_ks=top_ks.tolist(), top_ps=top_ps.tolist(),
                           seeds=seeds.tolist(), positions=pos.tolist(), tokens=toks.tolist())
    (HERE / "golden.json").write_text(json.dumps(meta, indent=1))
    print("sampler tokens:", toks.tolist())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of a checkout of Aayaan-Sahu/deterministic-inference>")
    main(sys.argv[1])
