"""Each part alone against its plain counterpart, and the generality of the
assembly: a toy mixer with state of its own, a toy feed-forward with routing, a toy
position encoding, a toy embedding (scaled) and a toy head (capped logits), all defined
here, are registered, built into a model by a plan, loaded and stepped through the
engine's step function without a change to the package; a plan may name a layer twice and
let a layer read another layer's cache; and a toy architecture registered here generates
through ``Engine.generate`` from a model folder."""

import pytest
import torch

from deterministic_inference_b200.cache import CacheManager
from deterministic_inference_b200.engine.batch import SequenceInput, build_step_batch
from deterministic_inference_b200.kernels import ops
from deterministic_inference_b200.models.decoder import DecoderModel
from deterministic_inference_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS,
                                                BuildContext, LayerSpec, ModelPlan, PagedKVSpec,
                                                PartSpec, ScheduleEntry, StateSpec, TensorSpec,
                                                register_embedding, register_feed_forward,
                                                register_head, register_mixer,
                                                register_position_encoding)
from deterministic_inference_b200.parts.base import (FeedForward, Head, Mixer, PositionEncoding,
                                                     TokenEmbedding)
from tests import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ctx(dtype):
    return BuildContext(dtype=dtype, device=torch.device(DEV))


def tol(dtype):
    return dict(atol=2e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    n = NORMS.build(PartSpec("rms_norm", dict(name="n.weight", size=96, eps=1e-5)), ctx(dtype))
    assert [(s.name, s.shape, s.role) for s in n.tensor_specs()] == [("n.weight", (96,), "vector")]
    w = torch.randn(96, device=DEV)
    n.load({"n.weight": w})
    x = torch.randn(7, 96, device=DEV).to(dtype)
    r = torch.randn(7, 96, device=DEV).to(dtype)
    torch.testing.assert_close(n.forward(x).float(), P.rms_norm(x.float(), w, 1e-5), **tol(dtype))
    s = x.float() + r.float()
    y, r2 = n.add_forward(x.clone(), r.clone())
    torch.testing.assert_close(y.float(), P.rms_norm(s, w, 1e-5), **tol(dtype))
    torch.testing.assert_close(r2.float(), s.to(dtype).float(), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    ff = FEED_FORWARDS.build(PartSpec("gated_mlp", dict(prefix="m.", hidden_size=80,
                                                        intermediate_size=112)), ctx(dtype))
    t = {s.name: (0.2 * torch.randn(s.shape, device=DEV)).to(dtype) for s in ff.tensor_specs()}
    ff.load(t)
    x = torch.randn(9, 80, device=DEV).to(dtype)
    # bfloat16: the plain formula with the stored tensors rounded where the engine stores them
    want = P.swiglu(x.float(), t["m.gate_proj.weight"].float(), t["m.up_proj.weight"].float(),
                    t["m.down_proj.weight"].float(), P.round_bf16 if dtype == torch.bfloat16 else None)
    torch.testing.assert_close(ops.as_tensor(ff.forward(x)).float(), want, **tol(dtype))
    with pytest.raises(ValueError, match="activation"):
        FEED_FORWARDS.build(PartSpec("gated_mlp", dict(prefix="m.", hidden_size=8, intermediate_size=8,
                                                       activation="gelu")), ctx(dtype))


def test_position_encoding_part():
    pe = POSITION_ENCODINGS.build(PartSpec("rope", dict(head_dim=48, rotary_dim=48, theta=5e4,
                                                        max_positions=300)), ctx(torch.float32))
    tab = pe.rotary_table()
    ang = P.rope_angles(torch.arange(300), 48, 5e4)
    # float32 pow differs by an ulp between devices; times a position of 300 that is ~3e-5
    torch.testing.assert_close(tab.cpu(), torch.cat([ang.cos(), ang.sin()], -1), atol=1e-4, rtol=0)
    assert POSITION_ENCODINGS.build(PartSpec("none", {}), ctx(torch.float32)).rotary_table() is None


def _attention_setup(dtype, hq, hkv, d, window=None, page=16):
    spec = PartSpec("gqa_attention", dict(
        prefix="a.", hidden_size=72, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=d ** -0.5,
        qk_norm_eps=1e-6, window=window,
        position_encoding=PartSpec("rope", dict(head_dim=d, rotary_dim=d, theta=1e4, max_positions=256))))
    mixer = MIXERS.build(spec, ctx(dtype))
    g = torch.Generator().manual_seed(3)
    t = {}
    for s in mixer.tensor_specs():
        if s.role == "vector":
            t[s.name] = (1 + 0.1 * torch.randn(s.shape, generator=g)).to(DEV)
        else:
            t[s.name] = (0.15 * torch.randn(s.shape, generator=g)).to(device=DEV, dtype=dtype)
    mixer.load(t)
    cache = CacheManager({0: mixer.cache_spec()}, num_pages=12, page_size=page, max_reqs=4,
                         max_seq_len=128, dtype=dtype, device=DEV)
    return mixer, t, cache


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,window", [(6, 2, 32, None), (4, 4, 16, 9), (8, 1, 64, None)])
def test_attention_part_whole_and_in_portions(dtype, hq, hkv, d, window):
    mixer, t, cache = _attention_setup(dtype, hq, hkv, d, window)
    assert mixer.cache_spec() == PagedKVSpec(hkv, d, window)
    n = 50
    x = torch.randn(n, 72, generator=torch.Generator().manual_seed(4)).to(device=DEV, dtype=dtype)
    # plain: the reference's attention block on the whole sequence
    cfg = dict(num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, rms_norm_eps=1e-6,
               rope_theta=1e4, num_hidden_layers=1,
               **(dict(use_sliding_window=True, sliding_window=window, max_window_layers=0) if window else {}))
    w = {("model.layers.0.self_attn." + k[2:]): v.float().cpu() for k, v in t.items()}
    want = P.attention_block(x.float().cpu(), cfg, w, 0,
                             P.round_bf16 if dtype == torch.bfloat16 else P._identity)
    slot = cache.allocate_slot()
    outs, c = [], 0
    for m in (20, 1, 1, 11, 2, 15):
        cache.allocate(slot, c + m)
        step = build_step_batch([SequenceInput(slot, [0] * m, c, [])], cache, DEV)
        # (a projection with split k hands its partial products on: ops.as_tensor adds them)
        outs.append(ops.as_tensor(mixer.forward(x[c:c + m].contiguous(), step, cache.view(0, step))))
        cache.release_passed(slot, c + m)
        c += m
    torch.testing.assert_close(torch.cat(outs).float().cpu(), want, **tol(dtype))


# ----------------------------------------------------------------- toy parts

@register_mixer("toy_running_mean")
class RunningMean(Mixer):
    """A mixer with per-request state of fixed size: y_t = W * mean(x_0..x_t).  The
    state (sum and count) lives in the request's state slot and is carried across
    portions."""

    def __init__(self, ctx, prefix, hidden_size):
        self.prefix, self.h = prefix, hidden_size

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "w", (self.h, self.h))]

    def load(self, tensors):
        self.w = tensors[self.prefix + "w"]

    def cache_spec(self):
        return StateSpec((self.h + 1,), "float32")

    def forward(self, x, step, cache):
        out = torch.empty_like(x)
        slots = step.state_slots.tolist()
        cu = step.cu_q_lens.tolist()
        for b, slot in enumerate(slots):
            xs = x[cu[b]:cu[b + 1]].float()
            st = cache.state[slot]
            sums = st[:self.h] + torch.cumsum(xs, 0)
            counts = st[self.h] + torch.arange(1, xs.shape[0] + 1, device=x.device)
            out[cu[b]:cu[b + 1]] = ((sums / counts[:, None]) @ self.w.float().T).to(x.dtype)
            st[:self.h] = sums[-1]
            st[self.h] = counts[-1]
        return out


@register_feed_forward("toy_routed")
class ToyRouted(FeedForward):
    """A feed-forward with routing: each token goes to the expert whose router
    logit (float32) is largest; expert e scales by its vector."""

    def __init__(self, ctx, prefix, hidden_size, num_experts):
        self.prefix, self.h, self.e = prefix, hidden_size, num_experts

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "router", (self.e, self.h)),
                TensorSpec(self.prefix + "scale", (self.e, self.h))]

    def load(self, tensors):
        self.router, self.scale = tensors[self.prefix + "router"], tensors[self.prefix + "scale"]

    def forward(self, x):
        choice = (x.float() @ self.router.float().T).argmax(-1)
        return (x.float() * self.scale.float()[choice]).to(x.dtype)


@register_position_encoding("toy_scaled_rope")
class ScaledRope(PositionEncoding):
    """Another position encoding: rotation over half of the head, positions divided by
    a factor; the attention mixer's fused kernel takes it as a table."""

    def __init__(self, ctx, head_dim, factor, max_positions):
        self.ctx, self.d, self.factor, self.n = ctx, head_dim, factor, max_positions

    def rotary_table(self):
        half = self.d // 4
        inv = 1.0 / (100.0 ** (torch.arange(half, dtype=torch.float32, device=self.ctx.device) / half))
        f = torch.outer(torch.arange(self.n, dtype=torch.float32, device=self.ctx.device) / self.factor, inv)
        return torch.cat([f.cos(), f.sin()], -1).contiguous()


@register_embedding("toy_scaled_embedding")
class ScaledEmbedding(TokenEmbedding):
    """Another embedding: the gathered rows are multiplied by a constant."""

    def __init__(self, ctx, name, vocab_size, hidden_size, factor):
        self.name, self.v, self.h, self.factor = name, vocab_size, hidden_size, factor

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.v, self.h), role="table")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def table(self):
        return self.weight

    def forward(self, ids):
        return (ops.embedding(ids, self.weight).float() * self.factor).to(self.weight.dtype)


@register_head("toy_capped_head")
class CappedHead(Head):
    """Another head: tied to the embedding's table, logits squashed to (-cap, cap)."""

    tied = True

    def __init__(self, ctx, cap):
        self.cap = cap

    def load(self, tensors):
        self.weight = tensors[None]

    def forward(self, rows):
        logits = ops.as_tensor(ops.linear(rows, self.weight, out_dtype=torch.float32))
        return self.cap * torch.tanh(logits / self.cap)


def _toy_plan(h=48, vocab=64):
    attn = lambda i: PartSpec("gqa_attention", dict(
        prefix=f"l{i}.attn.", hidden_size=h, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
        qk_norm_eps=None, window=None,
        position_encoding=PartSpec("toy_scaled_rope", dict(head_dim=16, factor=2.0, max_positions=128))))
    norm = lambda n: PartSpec("rms_norm", dict(name=n, size=h, eps=1e-5))
    layers = (
        LayerSpec(PartSpec("pre_norm", {}), PartSpec("toy_running_mean", dict(prefix="l0.mix.", hidden_size=h)),
                  PartSpec("toy_routed", dict(prefix="l0.ff.", hidden_size=h, num_experts=3)),
                  norm("l0.n1"), norm("l0.n2")),
        LayerSpec(PartSpec("pre_norm", {}), attn(1),
                  PartSpec("gated_mlp", dict(prefix="l1.ff.", hidden_size=h, intermediate_size=80)),
                  norm("l1.n1"), norm("l1.n2")),
    )
    # layer 1 runs twice (the second time on a cache of its own), then once more reading
    # the cache its first run wrote; layer 0's state is cache 0
    schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 2),
                ScheduleEntry(1, 1, writes_cache=False))
    return ModelPlan(hidden_size=h, vocab_size=vocab,
                     embedding=PartSpec("toy_scaled_embedding", dict(name="emb", vocab_size=vocab,
                                                                      hidden_size=h, factor=3.0)),
                     head=PartSpec("toy_capped_head", dict(cap=5.0)),
                     final_norm=norm("final"), layers=layers, schedule=schedule, max_positions=128)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_parts_are_registered_built_and_stepped(dtype):
    plan = _toy_plan()
    model = DecoderModel(plan, dtype, DEV)
    g = torch.Generator().manual_seed(8)
    tensors = {}
    for s in model.tensor_specs():
        x = torch.randn(s.shape, generator=g)
        tensors[s.name] = ((1 + 0.1 * x).to(DEV) if s.role == "vector"
                           else (0.2 * x).to(device=DEV, dtype=dtype))
    model.load(tensors)
    specs = model.cache_specs()
    assert isinstance(specs[0], StateSpec) and isinstance(specs[1], PagedKVSpec) and set(specs) == {0, 1, 2}
    cache = CacheManager(specs, num_pages=16, page_size=16, max_reqs=4, max_seq_len=128,
                         dtype=dtype, device=DEV)
    assert len(cache.page_groups) == 1 and len(cache.state_groups) == 1

    def run(cuts, toks, slot):
        outs, c = [], 0
        for n in cuts:
            cache.allocate(slot, c + n)
            cache.reset_fresh_state()
            step = build_step_batch([SequenceInput(slot, toks[c:c + n], c, list(range(n)))], cache, DEV)
            outs.append(model.forward(step, cache))
            c += n
        return torch.cat(outs)

    toks = torch.randint(0, 64, (40,), generator=g).tolist()
    a = cache.allocate_slot()
    whole = run([40], toks, a)
    cache.release_slot(a)
    b = cache.allocate_slot()          # the same slot again: its state must start from zero
    parts = run([7, 1, 1, 13, 2, 16], toks, b)
    assert whole.shape == (40, 64) and torch.isfinite(whole).all()
    assert float(whole.abs().max()) < 5.0 and float(whole.abs().max()) > 0.5      # the head's cap is at work
    assert [s.name for s in model.tensor_specs()].count("emb") == 1 and model.head.weight is model.embedding.table()
    torch.testing.assert_close(parts, whole, **(dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16
                                                else dict(atol=1e-4, rtol=1e-4)))
    # two requests in one batch keep their states apart
    c2 = cache.allocate_slot()
    cache.allocate(c2, 40)
    cache.reset_fresh_state()
    cache.release_slot(b)
    b = cache.allocate_slot()
    cache.allocate(b, 40)
    cache.reset_fresh_state()
    other = torch.randint(0, 64, (40,), generator=g).tolist()
    step = build_step_batch([SequenceInput(b, toks, 0, [39]), SequenceInput(c2, other, 0, [39])], cache, DEV)
    both = model.forward(step, cache)
    torch.testing.assert_close(both[0], whole[39], **(dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16
                                                      else dict(atol=1e-4, rtol=1e-4)))


def test_plan_validation():
    plan = _toy_plan()
    bad = ModelPlan(**{**plan.__dict__, "schedule": (ScheduleEntry(0, 0), ScheduleEntry(1, 0))})
    with pytest.raises(ValueError, match="written by"):
        bad.validate()
    bad = ModelPlan(**{**plan.__dict__, "schedule": (ScheduleEntry(1, 1, writes_cache=False),)})
    with pytest.raises(ValueError, match="no entry writes"):
        bad.validate()
    with pytest.raises(KeyError, match="unknown mixer kind"):
        MIXERS.build(PartSpec("nope", {}), ctx(torch.float32))


class ToyConfig:
    """A toy architecture's configuration class, registered from this file: config.json
    gives the width and the vocabulary, ``plan()`` the toy plan above (a mixer with state,
    a routed feed-forward, a scaled embedding, a capped head, a layer run twice)."""

    def __init__(self, h, vocab):
        self.h, self.vocab = h, vocab

    @classmethod
    def from_dict(cls, d, generation_config=None):
        return cls(int(d["toy_width"]), int(d["toy_vocab"]))

    @classmethod
    def from_json(cls, model_dir):
        import json
        from pathlib import Path
        return cls.from_dict(json.loads((Path(model_dir) / "config.json").read_text()))

    def to_dict(self):
        return {"architectures": ["ToyForCausalLM"], "toy_width": self.h, "toy_vocab": self.vocab}

    def plan(self):
        return _toy_plan(self.h, self.vocab)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_generates_through_the_engine(dtype, tmp_path):
    """The toy architecture is registered by name, its model folder is written with the
    package's random-weights writer and loaded by its loader, and ``Engine.generate`` runs
    it: prompts in portions under a small token budget, a pool so small that requests are
    preempted (their state is rebuilt from token 0), decoding with CUDA graphs switched on:
    the mixer keeps per-request state, so no step is captured, and the tokens are those of
    an engine without graphs."""
    import json
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams
    from deterministic_inference_b200.models.registry import register_architecture
    from deterministic_inference_b200.weights import write_random_model
    register_architecture("ToyForCausalLM", ToyConfig)
    cfg = ToyConfig(48, 64)
    write_random_model(cfg, 5, tmp_path)
    assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["ToyForCausalLM"]
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 64, (n,), generator=g).tolist() for n in (5, 23, 40, 9)]
    sp = SamplingParams(max_new_tokens=12, ignore_eos=True)
    outs = {}
    for name, kw in (("graphs", dict(cuda_graphs=True)), ("launched", dict(cuda_graphs=False)),
                     ("portions", dict(cuda_graphs=True, max_prefill_tokens=7)),
                     ("tight", dict(cuda_graphs=True, kv_pool_tokens=96, max_prefill_tokens=16))):
        eng = Engine(EngineConfig(model_path=str(tmp_path), dtype=dtype, device=DEV, page_size=16,
                                  max_reqs=8, max_seq_len=128, **{"kv_pool_tokens": 1024, **kw}))
        res = eng.generate(prompts, sp)
        outs[name] = [o.token_ids for o in res]
        assert all(len(t) == 12 for t in outs[name])
        if eng.runner.decode_graphs is not None:
            assert eng.runner.decode_graphs.replays == 0 and eng.runner.step_graphs.replays == 0
        if name == "tight":
            assert sum(o.num_preemptions for o in res) > 0
        eng.cache.check_invariants()
    assert outs["graphs"] == outs["launched"]
    if dtype == "float32":
        # other cuts add the mixer's running sums in another order: the first tokens agree
        # (later ones follow from them)
        assert [t[0] for t in outs["portions"]] == [t[0] for t in outs["graphs"]]
        assert [t[0] for t in outs["tight"]] == [t[0] for t in outs["graphs"]]
