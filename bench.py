"""Benchmark of the engine on one B200: decode tokens/s (batch 8 by default, also
batch 1 and 64), prefill tokens/s at 2,048 tokens, both with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Default model: the layer sizes of
Qwen3-0.6B (28 layers, hidden 1024, 16/8 heads of 128, intermediate 3072,
vocabulary 151936, tied head), random weights N(0, 0.02) from seed 0, bfloat16,
page size 16; each request holds 2,048 cached tokens when decoding starts.

``value``   decode tokens/s timed on the device (CUDA events): K decode steps through
            ``ModelRunner.step`` and the sampler (argmax), the sampled tokens handed to
            the next step on the device; nothing is read on the host in between.
``e2e``     the same through ``Engine.step()``: scheduler, packing, one
            host-to-device copy of the step's metadata from pinned memory, the
            graph, sampling, and the device-to-host read of the sampled tokens,
            every step.
``prefill`` a prompt of 2,048 tokens, whole, of a length not run before, through the
            captured graph of its bucket of prompt lengths (``value``, ``ms``); the same
            launched kernel by kernel (``launched_ms``, ``cold_ms``: a bucket's first two
            prompts) and replayed again (``replayed_ms``).
``points``  decode at batch 1 and 64; ``points_<preset>``: decode and prefill at a larger
            model's layer sizes with fewer layers (``config.second_model`` names both
            layer counts).
``--impl reference`` runs the unmodified reference engine on the same workload.
Every decode step reads all weights and the live cache (about 3 GB at batch 8),
far more than the 126 MB L2, so no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


REF_TREE = ROOT / "baseline" / "_ref"


def _stub_tokenizer(folder: Path) -> None:
    """The reference's ``Engine`` builds a tokenizer from the model folder whatever the
    prompts are; a three-word one satisfies it (requests come as token ids)."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    tok = Tokenizer(WordLevel({"<unk>": 0, "a": 1, "b": 2}, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>"}))


def reference_arm(a) -> int:
    """The unmodified reference (a copy of its tree under ``baseline/_ref``; it has no
    packaging metadata, so it is put on the module path instead of installed) through its
    own public API: ``sid.engine.engine.Engine(EngineConfig(mode=NONDET))``,
    ``add_request(prompt_ids=...)`` and ``step()``.  Same model shape, random weights,
    batch, context, steps and warm-up as this repository's arm.  Its ``step()`` ends with
    the device-to-host read of the sampled tokens, so one timing gives both ``value`` and
    ``e2e``.  Nothing of this package's kernels is loaded in this process: only the
    random-weights writer (plain torch on the CPU) makes the model folder."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
        return 0

    if a.gpus != 1:
        return unavailable("the reference is a single-GPU engine (no collective code); N>1 is not run")
    if not (REF_TREE / "sid" / "engine" / "engine.py").exists():
        return unavailable("no copy of the reference's tree under baseline/_ref")
    import tempfile
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        from deterministic_inference_b200.config import preset
        from deterministic_inference_b200.weights import write_random_model
        full = preset(a.preset)
        layers = a.layers or full.num_hidden_layers
        cfg = preset(a.preset, num_hidden_layers=layers, max_window_layers=layers)
        pk = peaks()
        sizes = sorted({a.batch, *[int(x) for x in a.points.split(",") if x.strip()]})
        max_b = max(sizes)
        new_tokens = max(a.steps, a.point_steps) + a.warmup + 32
        with tempfile.TemporaryDirectory(prefix="dib200_ref_model_") as folder:
            folder = Path(folder)
            write_random_model(cfg, 0, folder)
            _stub_tokenizer(folder)
            sys.path.insert(0, str(REF_TREE))
            from sid.config import EngineConfig as RefEngineConfig, Mode, SamplingParams as RefParams
            from sid.engine.engine import Engine as RefEngine
            pool = max_b * (a.context + new_tokens + 64) + a.prefill_tokens + 4096
            eng = RefEngine(RefEngineConfig(
                model_path=str(folder), mode=Mode.NONDET, kv_pool_tokens=pool,
                max_reqs=max(256, max_b + 8), max_seq_len=max(8192, a.context + new_tokens + 64),
                max_prompt_len=max(a.context, a.prefill_tokens), max_prefill_tokens=8192,
                max_decode_batch=max(256, max_b), device="cuda"))
            gen = torch.Generator().manual_seed(1)

            def random_prompt(n):
                return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

            def timed(fn):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                s.record()
                fn()
                e.record()
                torch.cuda.synchronize()
                return s.elapsed_time(e)

            def drain():
                while eng.scheduler.has_work():
                    eng.step()
                eng._done.clear()

            # prefill of one whole prompt: the step that admits it runs it and samples one token
            prompt = random_prompt(a.prefill_tokens)
            flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
            ms_list = []
            for it in range(0 if a.no_prefill else 6):
                eng.add_request(prompt_ids=prompt, params=RefParams(max_new_tokens=1, ignore_eos=True))
                flush.zero_()
                ms = timed(eng.step)
                drain()
                if it >= 3:
                    ms_list.append(ms)
            prefill = None
            if ms_list:
                pms = sorted(ms_list)[len(ms_list) // 2]
                _, flops = model_bytes_and_flops(cfg, layers, 1, 0, a.prefill_tokens)
                prefill = {"value": a.prefill_tokens / (pms / 1e3), "tokens": a.prefill_tokens, "ms": pms,
                           "frac": flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12)}

            def decode(batch, steps, sample_clocks=False):
                sp = RefParams(max_new_tokens=steps + a.warmup + 32, ignore_eos=True)
                for _ in range(batch):
                    eng.add_request(prompt_ids=random_prompt(a.context), params=sp)
                eng.step()                          # admits all and prefills them, untimed
                assert len(eng.scheduler.active) == batch and not eng.scheduler.waiting
                for _ in range(a.warmup):
                    eng.step()
                sampler = ClockSampler()
                if sample_clocks:
                    sampler.start()
                ms = timed(lambda: [eng.step() for _ in range(steps)])
                clocks = sampler.stop() if sample_clocks else None
                assert all(len(r.output_ids) >= steps + a.warmup for r in eng.scheduler.active)
                for r in eng.scheduler.active:      # stop them: the next step retires them
                    r.params.max_new_tokens = len(r.output_ids)
                    r.check_finished()
                drain()
                return ms, clocks

            ms, clocks = decode(a.batch, a.steps, sample_clocks=True)
            points = {}
            for b in sizes:
                if b != a.batch:
                    pms, _ = decode(b, a.point_steps)
                    points[f"decode_b{b}"] = b * a.point_steps / (pms / 1e3)
    except Exception as exc:  # the reference's kernels or its build failed here: say so, run nothing again
        return unavailable(f"{type(exc).__name__}: {exc}")
    value = a.batch * a.steps / (ms / 1e3)
    mean_ctx = a.context + a.warmup + a.steps / 2
    decode_bytes, _ = model_bytes_and_flops(cfg, layers, a.batch, mean_ctx, 0)
    achieved = decode_bytes / (ms / a.steps / 1e3) / 1e9
    print(json.dumps({
        "metric": "decode tok/s (bf16, 1 B200)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": dict(bench_config(a, cfg, full, layers), page_size=1),
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None,
                "d2h_bytes_per_step": a.batch * 8,
                "note": "the reference's step() reads the sampled tokens on the host every step; "
                        "value and e2e are the same timing"},
        "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]},
        "points": points}))
    return 0


def bench_config(a, cfg, full, layers: int) -> dict:
    return {"model": a.preset, "layers": layers, "layers_full": full.num_hidden_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied_head": cfg.tie_word_embeddings, "global_batch": a.batch,
            "seq_len": a.context, "context": 4096, "page_size": 16,
            "weights": "random N(0,0.02) seed 0", "parallelism": "1 GPU",
            "l2": "inputs larger than L2 (weights+cache per step)"}


def model_bytes_and_flops(cfg, layers: int, batch: int, ctx: float, prefill_tokens: int):
    h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    hq, hkv, v = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    layer_params = (hq + 2 * hkv) * d * h + h * hq * d + 3 * h * i
    weight_bytes = 2 * (layers * layer_params + v * h)            # every matrix once, head once
    kv_bytes_per_token = 2 * hkv * d * 2 * layers
    decode_bytes = weight_bytes + batch * ctx * kv_bytes_per_token
    t = prefill_tokens
    prefill_flops = 2 * t * layers * layer_params + layers * 2 * t * t * d * hq + 2 * v * h
    return decode_bytes, prefill_flops


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="qwen3_0_6b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="cached tokens per request")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset has")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64", help="extra decode batch sizes")
    ap.add_argument("--point-steps", type=int, default=64)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="mixed: the continuous-batching run of the benchmark configurations "
                         "(64 requests, prompts uniform in [128, 2048], 256 outputs each, "
                         "temperature 0.7) through Engine.generate; prints its own line")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--second-preset", default="qwen3_8b",
                    help="layer sizes measured after the main model (decode batch 8 and 64, prefill), "
                         "with --second-layers layers; 'none' to skip")
    ap.add_argument("--second-layers", type=int, default=12)
    ap.add_argument("--profile", default=None, choices=["decode", "prefill"],
                    help="bracket this region with cudaProfilerStart/Stop (for ncu "
                         "--profile-from-start off); the numbers of such a run are not a result")
    a = ap.parse_args()

    if a.warmup < 3:
        a.warmup = 3
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU only (this engine is single-GPU); --gpus {a.gpus} is not run")
        return 2

    import torch

    from deterministic_inference_b200 import EngineConfig, SamplingParams, preset
    from deterministic_inference_b200.engine.batch import SequenceInput
    from deterministic_inference_b200.engine.engine import Engine
    from deterministic_inference_b200.kernels import ops
    from deterministic_inference_b200.sampling.sampler import sample

    full = preset(a.preset)
    layers = a.layers or full.num_hidden_layers
    cfg = preset(a.preset, num_hidden_layers=layers, max_window_layers=layers)
    pk = peaks()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator().manual_seed(1)
    greedy = SamplingParams(max_new_tokens=1 << 20, ignore_eos=True)

    def random_prompt(vocab, n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def timed(fn):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e)

    def make_engine(mcfg, sizes, steps_most):
        max_b = max(sizes)
        per_req = a.context + steps_most + a.warmup + 96
        pool = max_b * (-(-per_req // 16) * 16) + a.prefill_tokens + 1024
        longest_prompt = a.prefill_tokens + 64        # the prefill run also feeds a few tokens more
        return Engine(EngineConfig(
            model_config=mcfg, random_seed=0, dtype="bfloat16", kv_pool_tokens=pool, page_size=16,
            max_reqs=max(256, max_b + 8),
            max_seq_len=max(8192, -(-per_req // 1024) * 1024, longest_prompt),
            max_prefill_tokens=max(8192, longest_prompt), max_decode_batch=max(256, max_b),
            device="cuda:0"))

    def launches_now(runner):
        """Kernels launched so far: the wrappers' own count plus what replayed graphs hold."""
        n = ops.launch_count
        for g in (runner.decode_graphs, runner.step_graphs):
            if g is not None:
                n += g.kernels_replayed
        return n

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > L2

    def measure_prefill(engine, mcfg, n_layers, profile=False):
        """One prompt of ``--prefill-tokens`` tokens, whole, to its first logits.  The engine
        launches a step kernel by kernel the first two times its bucket of shapes is seen
        (prompt lengths rounded up by a sixteenth of an octave) and replays the bucket's
        captured graph from the third time on, whatever the length inside the bucket.  Timed:
        ``launched_ms``: the prompt launched, bucket and libraries new (first) and known
        (second); ``value``/``ms``: a prompt of a length NOT run before, its bucket's graph
        captured (what a prompt costs in a running engine); ``replayed_ms``: the same length
        again.  Every timed prompt goes through ``ModelRunner.step`` from host tokens."""
        runner, cache = engine.runner, engine.cache
        n = a.prefill_tokens
        prompt = random_prompt(mcfg.vocab_size, n + 1)

        def once(tokens, profiled=False):
            slot = cache.allocate_slot()
            flush.zero_()
            if profiled:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
            ms = timed(lambda: runner.step([SequenceInput(slot, tokens, 0, [len(tokens) - 1])]))
            if profiled:
                torch.cuda.profiler.stop()
            cache.release_slot(slot)
            return ms

        once(prompt[:n + 40])                    # another bucket: load the libraries, warm the clocks
        launched = [once(prompt[:n - 2]), once(prompt[:n - 1])]      # the bucket's first and second time
        once(prompt[:n - 3])                     # the third: captured, then replayed
        sg = runner.step_graphs
        replays0 = sg.replays if sg is not None else 0
        fresh = once(prompt[:n], profiled=profile)                   # a length not run before
        replayed = [once(prompt[:n]) for _ in range(3)]
        in_graph = sg is not None and sg.replays - replays0 == 4
        ms = fresh if in_graph else min(launched + [fresh] + replayed)   # never captured: all were launched
        replayed_ms = sorted(replayed)[1] if in_graph else None
        _, flops = model_bytes_and_flops(mcfg, n_layers, 1, 0, n)
        frac = lambda t: flops / (t / 1e3) / (pk["bf16_tflops"] * 1e12)
        return {"value": n / (ms / 1e3), "tokens": n, "ms": ms, "cold_ms": min(launched),
                "launched_ms": [round(x, 3) for x in launched], "replayed_ms": replayed_ms,
                "frac": frac(ms), "frac_launched": frac(min(launched)),
                "note": ("value, ms and frac: a prompt length not run before, replayed through the "
                         "captured graph of its bucket of lengths; launched_ms: kernel by kernel, "
                         "the bucket's first and second time" if in_graph else
                         "value, ms and frac: launched kernel by kernel (the device bounds this step, so "
                         "its bucket is not captured before it has come many times)")}

    def fill_requests(engine, mcfg, batch):
        slots = [engine.cache.allocate_slot() for _ in range(batch)]
        group = max(1, 8192 // a.context)
        for i in range(0, batch, group):
            engine.runner.step([SequenceInput(s, random_prompt(mcfg.vocab_size, a.context), 0, [])
                                for s in slots[i:i + group]])
        return slots

    def device_decode(engine, mcfg, batch, steps, warmup, sample_clocks=False, profile=False):
        """``steps`` decode steps of ``batch`` requests through ``ModelRunner.step`` and the
        sampler, the sampled tokens handed to the next step on the device; nothing is read
        on the host inside the timed region."""
        runner = engine.runner
        slots = fill_requests(engine, mcfg, batch)
        params = [greedy] * batch
        state = {"tokens": None}

        def one(k):
            pend = state["tokens"] is not None
            entries = [SequenceInput(s, [0], a.context + k, [0], i if pend else -1)
                       for i, s in enumerate(slots)]
            logits, _ = runner.step(entries, state["tokens"])
            state["tokens"] = sample(logits, params, [a.context + k + 1] * batch)

        for k in range(warmup):
            one(k)
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        n0 = launches_now(runner)
        if profile:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        ms = timed(lambda: [one(k) for k in range(warmup, warmup + steps)])
        if profile:
            torch.cuda.profiler.stop()
        launches = launches_now(runner) - n0
        clocks = sampler.stop() if sample_clocks else None
        for s in slots:
            engine.cache.release_slot(s)
        return ms, launches, clocks

    def decode_roofline(mcfg, n_layers, batch, steps, warmup, ms):
        mean_ctx = a.context + warmup + steps / 2
        nbytes, _ = model_bytes_and_flops(mcfg, n_layers, batch, mean_ctx, 0)
        achieved = nbytes / (ms / steps / 1e3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}

    sizes = sorted({a.batch, *[int(x) for x in a.points.split(",") if x.strip()]})
    engine = make_engine(cfg, sizes, max(a.steps, a.point_steps))
    graphs = engine.runner.decode_graphs

    if a.workload == "mixed":
        n_req, n_out = 64, 256
        lens = torch.randint(128, 2049, (n_req,), generator=gen).tolist()
        prompts = [random_prompt(cfg.vocab_size, n) for n in lens]
        sp = SamplingParams(max_new_tokens=n_out, temperature=0.7, seed=7, ignore_eos=True)
        # the first pass captures the CUDA graphs this workload needs (one per bucket of batch
        # size and context length, tens of milliseconds each); the second is the steady state
        runs = []
        for _ in range(2):
            steps0, replays0 = engine.runner.steps_run, (graphs.replays if graphs else 0)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = engine.generate(prompts, sp)
            torch.cuda.synchronize()
            runs.append(time.perf_counter() - t0)
            assert all(len(o.token_ids) == n_out for o in outs)
        dt = runs[1]
        print(json.dumps({
            "metric": "continuous batching output tok/s (bf16, 1 B200)", "value": n_req * n_out / dt,
            "first_pass_value": n_req * n_out / runs[0],
            "graph_captures": {"decode": graphs.captures if graphs else 0,
                               "decode_seconds": graphs.capture_seconds if graphs else 0.0,
                               "steps": engine.runner.step_graphs.captures if engine.runner.step_graphs else 0,
                               "steps_seconds": engine.runner.step_graphs.capture_seconds
                               if engine.runner.step_graphs else 0.0},
            "unit": "tokens/s", "n_gpus": 1, "seconds": dt, "requests": n_req,
            "prompt_tokens": sum(lens), "output_tokens": n_req * n_out, "temperature": 0.7,
            "steps": engine.runner.steps_run - steps0, "preemptions": engine.scheduler.num_preemptions,
            "graph_replays": (graphs.replays if graphs else 0) - replays0, "dtype": "bf16", "data": "synthetic",
            "config": {"model": a.preset, "layers": layers, "layers_full": full.num_hidden_layers,
                       "max_prefill_tokens": engine.cfg.max_prefill_tokens}}))
        return 0

    prefill = None if a.no_prefill else measure_prefill(engine, cfg, layers, a.profile == "prefill")

    # ---------------- decode, timed on the device ----------------
    ms, launches, clocks = device_decode(engine, cfg, a.batch, a.steps, a.warmup, sample_clocks=True,
                                         profile=a.profile == "decode")
    value = a.batch * a.steps / (ms / 1e3)
    roofline = decode_roofline(cfg, layers, a.batch, a.steps, a.warmup, ms)
    points = {}
    for b in sizes:
        if b != a.batch:
            pms, _, _ = device_decode(engine, cfg, b, a.point_steps, a.warmup)
            points[f"decode_b{b}"] = b * a.point_steps / (pms / 1e3)
            points[f"decode_b{b}_frac"] = decode_roofline(cfg, layers, b, a.point_steps, a.warmup, pms)["frac"]

    # ---------------- decode end to end through Engine.step() ----------------
    e2e = None
    if not a.no_e2e:
        sp = SamplingParams(max_new_tokens=a.steps + a.warmup + 32, ignore_eos=True)   # nobody finishes inside the timed steps
        for _ in range(a.batch):
            engine.add_request(prompt_ids=random_prompt(cfg.vocab_size, a.context), params=sp)
        while any(r.num_output == 0 for r in list(engine.scheduler.running) + list(engine.scheduler.waiting)):
            engine.step()                       # prefill, untimed
        for _ in range(a.warmup):
            engine.step()
        e2e_ms = timed(lambda: [engine.step() for _ in range(a.steps)])
        assert all(r.num_output + r.num_pending >= a.steps for r in engine.scheduler.running)
        meta_bytes = max(c.layout.size for c in graphs.graphs.values()) * 4 if graphs and graphs.graphs else 0
        e2e = {"value": a.batch * a.steps / (e2e_ms / 1e3), "unit": "tokens/s",
               "ms_per_step": e2e_ms / a.steps,
               "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": a.batch * 4}
        while engine.has_work():
            engine.step()

    # ---------------- the same at a larger model's layer sizes, fewer layers ----------------
    second = None
    if a.second_preset and a.second_preset != "none" and a.profile is None:
        del engine, graphs
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        full2 = preset(a.second_preset)
        l2 = min(a.second_layers, full2.num_hidden_layers)
        cfg2 = preset(a.second_preset, num_hidden_layers=l2, max_window_layers=l2)
        eng2 = make_engine(cfg2, [8, 64], a.point_steps)
        second = {"model": a.second_preset, "layers": l2, "layers_full": full2.num_hidden_layers,
                  "hidden": cfg2.hidden_size, "heads": cfg2.num_attention_heads,
                  "kv_heads": cfg2.num_key_value_heads, "intermediate": cfg2.intermediate_size}
        if not a.no_prefill:
            pf = measure_prefill(eng2, cfg2, l2)
            second.update(prefill_tok_s=pf["value"], prefill_ms=pf["ms"], prefill_frac=pf["frac"],
                          prefill_launched_ms=pf["cold_ms"])
        for b in (8, 64):
            pms, _, _ = device_decode(eng2, cfg2, b, a.point_steps, a.warmup)
            second[f"decode_b{b}"] = b * a.point_steps / (pms / 1e3)
            second[f"decode_b{b}_frac"] = decode_roofline(cfg2, l2, b, a.point_steps, a.warmup, pms)["frac"]
        del eng2

    config = bench_config(a, cfg, full, layers)
    if second is not None:
        config["second_model"] = f"{second['model']} layer sizes, {second['layers']} of {second['layers_full']} layers"
    line = {
        "metric": "decode tok/s (bf16, 1 B200)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours", "config": config,
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": roofline, "points": points, "points_" + (a.second_preset or "none"): second,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
